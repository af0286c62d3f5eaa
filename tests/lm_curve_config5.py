#!/usr/bin/env python
"""Loss curve of benchmark configuration 5 at its real size, product against torch (not a pytest
file: it takes minutes of GPU time; run it by hand, the tables under profiles/ come from it).

The 24-layer sky-1-style LM (hidden 2048, 16 x 128 heads, ffn 5632, vocabulary 32768), AdamW
lr 3e-4 betas (0.9, 0.95) wd 0.1, global batch 64 x 2048 uniform-random tokens per step, seed 4.
The global batch is the same whatever the number of ranks: rank r of N takes sequences
[r * 64 / N, (r + 1) * 64 / N) as microbatches of 8 sequences, so the N-rank curve must equal the
one-rank curve up to the order of the f32 gradient sums -- that is the check of the product's
data-parallel reduction (Sky1LM._reduce) at full size.

    python tests/lm_curve_config5.py --steps 50 --torch-bf16-steps 50 --torch-f32-steps 3 --out lm_curve_n1.json
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        --master-port 29511 tests/lm_curve_config5.py --steps 50 --out lm_curve_n8.json

The torch arms are the checker (oracle/lm_ref.py): `f32` = full f32 products on bf16-rounded
weights; `bf16` = the same graph under torch.autocast(bfloat16), i.e. bf16 matrix products with f32
accumulation and f32 softmax / norms / loss -- the arithmetic of the reference's cuBLASLt bf16
path, which cannot run here.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

SEQS, VOCAB = 64, 32768


def main() -> None:
    import torch
    import torch.distributed as dist

    import cleanlm_b200 as cdl

    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--torch-bf16-steps", type=int, default=0)
    ap.add_argument("--torch-f32-steps", type=int, default=0)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    blk = cdl.sky1.Sky1Config()
    cfg = cdl.sky1.Sky1LMConfig(block=blk, layers=24, vocab=VOCAB)
    gen = torch.Generator().manual_seed(4)
    data = torch.randint(0, VOCAB, (args.steps, SEQS, blk.seqlen + 1), generator=gen, dtype=torch.int32)
    per_rank = SEQS // world
    mb = per_rank // blk.batch
    assert mb * blk.batch * world == SEQS, "the number of ranks must divide 8 microbatches"
    mine = data[:, rank * per_rank:(rank + 1) * per_rank]
    tok = mine[..., :-1].reshape(args.steps, mb, -1).contiguous().pin_memory()
    tgt = mine[..., 1:].reshape(args.steps, mb, -1).contiguous().pin_memory()
    global_tokens = SEQS * blk.seqlen

    # Initial weights from the device generator: the same values on every rank, drawn in seconds.
    model = cdl.sky1.Sky1LM(cfg, seed=4, device=dev, init_on_device=True)
    init = None
    if rank == 0 and (args.torch_bf16_steps or args.torch_f32_steps):
        init = {name: model.view("master", name).detach().cpu().clone() for name, _, _ in model.layout}
    d_tok = torch.empty(mb, blk.tokens, dtype=torch.int32, device=dev)
    d_tgt = torch.empty_like(d_tok)
    losses = []
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(args.steps):
        d_tok.copy_(tok[i], non_blocking=True)
        d_tgt.copy_(tgt[i], non_blocking=True)
        loss = model.train_step(d_tok, d_tgt, global_tokens=global_tokens)
        if world > 1:
            dist.all_reduce(loss)
        losses.append(loss.item())
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    assert cdl._lib.device_status() == 0
    del model
    torch.cuda.empty_cache()
    result = {"world": world, "steps": args.steps, "microbatches_per_rank": mb,
              "product": losses, "product_seconds": seconds}

    if init is not None:
        from oracle import block_ref, lm_ref

        c = dict(heads=blk.heads, kv_heads=blk.kv_heads, head_dim=blk.head_dim, eps=blk.eps)
        table = block_ref.rope_table(blk.seqlen, blk.head_dim)
        kw = dict(lr=cfg.lr, beta1=cfg.beta1, beta2=cfg.beta2, eps=cfg.adam_eps, wd=cfg.weight_decay,
                  device="cuda", checkpoint_blocks=True, microbatches=SEQS // blk.batch)
        batches = [(data[i, :, :-1].long(), data[i, :, 1:].long()) for i in range(args.steps)]
        if args.torch_bf16_steps:
            with torch.autocast(device_type="cuda", dtype=torch.bfloat16):
                result["torch_bf16_autocast"], _ = lm_ref.train(init, batches[:args.torch_bf16_steps], c, table,
                                                                cfg.layers, **kw)
            torch.cuda.empty_cache()
        if args.torch_f32_steps:
            result["torch_f32"], _ = lm_ref.train(init, batches[:args.torch_f32_steps], c, table, cfg.layers, **kw)
    if rank == 0:
        text = json.dumps(result)
        print(text)
        if args.out:
            Path(args.out).parent.mkdir(parents=True, exist_ok=True)
            Path(args.out).write_text(text)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

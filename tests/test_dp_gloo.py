"""The data-parallel RECIPE on CPU with gloo, world size 2: every rank scales its loss by
1 / GLOBAL token count, gradients are summed with all_reduce, and the result equals the gradient
of the mean loss over the whole batch on one rank.  This checks the recipe the N > 1 path follows,
with the torch restatement's arithmetic (oracle/lm_ref.py), so it needs no GPU; the product's own
data-parallel code (Sky1LM._reduce, the communication stream, the split backward) is checked on
GPUs by tests/test_dp_nccl.py and tests/test_block.py."""
import os
import socket
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make(seed=0):
    gen = torch.Generator().manual_seed(seed)
    cfg = dict(heads=1, kv_heads=1, head_dim=128, eps=1e-6)
    hidden, ffn, vocab = 128, 136, 64
    p = {"embedding": torch.randn(vocab, hidden, generator=gen) * 0.05,
         "lm_head": torch.randn(hidden, vocab, generator=gen) * 0.05,
         "final_norm": torch.ones(hidden),
         "blocks.0.norm1": torch.ones(hidden), "blocks.0.norm2": torch.ones(hidden),
         "blocks.0.wqkv": torch.randn(hidden, 384, generator=gen) * 0.05,
         "blocks.0.wo": torch.randn(128, hidden, generator=gen) * 0.05,
         "blocks.0.wup": torch.randn(hidden, ffn, generator=gen) * 0.05,
         "blocks.0.wgate": torch.randn(hidden, ffn, generator=gen) * 0.05,
         "blocks.0.wdown": torch.randn(ffn, hidden, generator=gen) * 0.05}
    data = torch.randint(0, vocab, (4, 33), generator=gen)
    return cfg, p, data


def _grads(p, tokens, targets, cfg, scale):
    sys.path.insert(0, str(ROOT))
    from oracle import block_ref, lm_ref

    w = {n: t.clone().double().requires_grad_(True) for n, t in p.items()}
    loss = lm_ref.lm_loss(w, tokens, targets, cfg, block_ref.rope_table(32, 128), 1, torch.float64,
                          reduction="sum") * scale
    loss.backward()
    return {n: t.grad for n, t in w.items()}, loss.detach()


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg, p, data = _make()
    shard = data[rank * 2:(rank + 1) * 2]
    global_tokens = data.shape[0] * 32
    g, loss = _grads(p, shard[:, :-1], shard[:, 1:], cfg, 1.0 / global_tokens)
    names = sorted(g)
    flat = torch.cat([g[n].flatten() for n in names])  # one bucket, reduced in place
    dist.all_reduce(flat)
    dist.all_reduce(loss)
    if rank == 0:
        torch.save({"flat": flat, "loss": loss}, out)
    dist.destroy_process_group()


def test_recipe_two_rank_gradient_sum_equals_global_mean_gradient(tmp_path):
    out = str(tmp_path / "dp.pt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    got = torch.load(out)
    cfg, p, data = _make()
    g, loss = _grads(p, data[:, :-1], data[:, 1:], cfg, 1.0 / (data.shape[0] * 32))
    flat = torch.cat([g[n].flatten() for n in sorted(g)])
    assert torch.allclose(got["flat"], flat, rtol=1e-9, atol=1e-12)
    assert torch.allclose(got["loss"], loss, rtol=1e-12)

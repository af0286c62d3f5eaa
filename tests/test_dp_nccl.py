"""The product's data-parallel code on two GPUs with NCCL: `Sky1LM.forward_backward` with its
per-layer all-reduces on the communication stream (`Sky1LM._reduce`), `optimizer_step` waiting for
that stream, and gradient clipping by the global norm taken AFTER the reduction.  Two ranks with
one microbatch each must reproduce one rank that accumulates both microbatches: the same reduced
gradient (f32 summation order aside), the same losses and the same weights after three steps.
Skipped on a box with fewer than two GPUs."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
STEPS = 3


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _config(cdl):
    sky1 = cdl.sky1
    blk = sky1.Sky1Config(batch=2, seqlen=256, hidden=256, heads=2, kv_heads=2, head_dim=128, ffn=512,
                          deterministic=True)
    return sky1.Sky1LMConfig(block=blk, layers=2, vocab=2048, lr=1e-3, max_grad_norm=0.5)


def _data(cfg):
    gen = torch.Generator().manual_seed(21)
    b = cfg.block
    d = torch.randint(0, cfg.vocab, (STEPS, 2, b.batch, b.seqlen + 1), generator=gen, dtype=torch.int32)
    return d[..., :-1].reshape(STEPS, 2, -1).contiguous(), d[..., 1:].reshape(STEPS, 2, -1).contiguous()


def _run(model, tok, tgt, global_tokens):
    """First step by hand (to look at the reduced gradient), then STEPS - 1 train_steps."""
    out = {"loss": []}
    mb = tok.shape[1]
    model.loss.zero_()
    for i in range(mb):
        model.forward_backward(tok[0, i], tgt[0, i], 1.0 / global_tokens, reduce_grads=(i == mb - 1))
    if model.comm is not None:
        torch.cuda.current_stream().wait_stream(model.comm)
    out["grads"] = model.grads.clone()
    model.optimizer_step()
    out["loss"].append(model.loss.clone())
    for s in range(1, STEPS):
        out["loss"].append(model.train_step(tok[s], tgt[s], global_tokens=global_tokens).clone())
    torch.cuda.synchronize()
    out["master"] = model.master.clone()
    return out


def _worker(rank, world, port, path):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    import cleanlm_b200 as cdl

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    cfg = _config(cdl)
    model = cdl.sky1.Sky1LM(cfg, seed=4, device=f"cuda:{rank}")
    tok, tgt = _data(cfg)
    global_tokens = tok.shape[1] * tok.shape[2]
    out = _run(model, tok[:, rank:rank + 1].cuda(), tgt[:, rank:rank + 1].cuda(), global_tokens)
    loss = torch.stack(out["loss"]).flatten()
    dist.all_reduce(loss)  # a rank's loss is its share of the global mean
    assert cdl._lib.device_status() == 0
    if rank == 0:
        torch.save({"grads": out["grads"].cpu(), "master": out["master"].cpu(), "loss": loss.cpu()}, path)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_equal_one_rank_with_two_microbatches(cdl, gpu_ok, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    path = str(tmp_path / "dp2.pt")
    mp.spawn(_worker, args=(2, _free_port(), path), nprocs=2, join=True)
    got = torch.load(path)

    cfg = _config(cdl)
    model = cdl.sky1.Sky1LM(cfg, seed=4)
    assert model.world == 1
    tok, tgt = _data(cfg)
    ref = _run(model, tok.cuda(), tgt.cuda(), tok.shape[1] * tok.shape[2])
    g_ref, g_got = ref["grads"].cpu(), got["grads"]
    scale = g_ref.abs().max().item()
    assert (g_got - g_ref).abs().max().item() <= 2e-5 * scale, "reduced gradient differs"
    loss_ref = torch.stack(ref["loss"]).flatten().cpu()
    assert torch.allclose(got["loss"], loss_ref, rtol=2e-4), (got["loss"], loss_ref)
    # Three clipped AdamW steps later the weights agree to a small fraction of one step (lr = 1e-3).
    diff = (got["master"] - ref["master"].cpu()).abs()
    assert diff.max().item() <= 1e-3 and diff.mean().item() <= 2e-5, (diff.max().item(), diff.mean().item())

"""TEST INFRASTRUCTURE — torch restatement of the sky-1 LM training step (stand-in for the
reference's Sky1Executor, crates/sky-1/src/training/model/mod.rs:209-420, which is dead code in the
reference and cannot run).  PARITY UNPINNED for the same reason as oracle/block_ref.py.

Embedding -> blocks -> final RMSNorm -> LM head -> mean cross-entropy; AdamW with decoupled weight
decay (none on norm gains, decoder.rs:724-731).  Used by tests only.
"""
from __future__ import annotations

import torch

from . import block_ref

BLOCK_PARAMS = ("norm1", "wqkv", "wo", "norm2", "wup", "wgate", "wdown")


def lm_loss(params: dict, tokens: torch.Tensor, targets: torch.Tensor, cfg: dict, table, layers: int,
            dtype=torch.float32, reduction="mean") -> torch.Tensor:
    """tokens, targets: int64 [B, S].  params: names as in Sky1LM ('embedding', 'blocks.i.name',
    'final_norm', 'lm_head')."""
    x = params["embedding"].to(dtype)[tokens]
    for i in range(layers):
        w = {n: params[f"blocks.{i}.{n}"] for n in BLOCK_PARAMS}
        x = block_ref.block_forward(x, w, cfg, table, dtype)
    h = block_ref.rmsnorm(x, params["final_norm"].to(dtype), cfg["eps"])
    logits = h @ params["lm_head"].to(dtype)
    return torch.nn.functional.cross_entropy(logits.reshape(-1, logits.shape[-1]), targets.reshape(-1),
                                             reduction=reduction)


def adamw_step(params: dict, grads: dict, m: dict, v: dict, step: int, lr, beta1, beta2, eps, wd):
    """In-place AdamW on f32 tensors; no weight decay for names containing 'norm'."""
    b1c, b2c = 1 - beta1 ** step, 1 - beta2 ** step
    for n, p in params.items():
        g = grads[n]
        m[n].mul_(beta1).add_(g, alpha=1 - beta1)
        v[n].mul_(beta2).addcmul_(g, g, value=1 - beta2)
        decay = 0.0 if "norm" in n else wd
        p.sub_(lr * ((m[n] / b1c) / ((v[n] / b2c).sqrt() + eps) + decay * p))


def train(params: dict, batches, cfg: dict, table, layers: int, lr=3e-4, beta1=0.9, beta2=0.95,
          eps=1e-8, wd=0.1, dtype=torch.float32, round_weights_to_bf16=True):
    """Runs one optimizer step per (tokens, targets) batch; returns the list of losses.
    With round_weights_to_bf16 the forward uses bf16-rounded copies of the f32 master weights,
    like the device's bf16 replicas."""
    master = {n: p.detach().clone().float() for n, p in params.items()}
    m = {n: torch.zeros_like(p) for n, p in master.items()}
    v = {n: torch.zeros_like(p) for n, p in master.items()}
    losses = []
    for step, (tokens, targets) in enumerate(batches, start=1):
        work = {n: (p.to(torch.bfloat16).float() if round_weights_to_bf16 else p.clone()).requires_grad_(True)
                for n, p in master.items()}
        loss = lm_loss(work, tokens, targets, cfg, table, layers, dtype)
        loss.backward()
        losses.append(float(loss.detach()))
        adamw_step(master, {n: w.grad for n, w in work.items()}, m, v, step, lr, beta1, beta2, eps, wd)
    return losses, master

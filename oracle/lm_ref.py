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
            dtype=torch.float32, reduction="mean", checkpoint_blocks=False) -> torch.Tensor:
    """tokens, targets: int64 [B, S].  params: names as in Sky1LM ('embedding', 'blocks.i.name',
    'final_norm', 'lm_head').  With checkpoint_blocks every block is recomputed in the backward
    (same arithmetic, less memory: needed for the 24-layer model at 8 x 2048 tokens)."""
    x = params["embedding"].to(dtype)[tokens]
    for i in range(layers):
        w = {n: params[f"blocks.{i}.{n}"] for n in BLOCK_PARAMS}
        if checkpoint_blocks:
            from torch.utils.checkpoint import checkpoint

            names = list(w)
            x = checkpoint(lambda xx, *ws: block_ref.block_forward(xx, dict(zip(names, ws)), cfg, table, dtype),
                           x, *[w[n] for n in names], use_reentrant=False)
        else:
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
          eps=1e-8, wd=0.1, dtype=torch.float32, round_weights_to_bf16=True, device="cpu",
          checkpoint_blocks=False, microbatches=1):
    """Runs one optimizer step per (tokens, targets) batch; returns the list of losses.
    With round_weights_to_bf16 the forward uses bf16-rounded copies of the f32 master weights,
    like the device's bf16 replicas.  `device` moves the whole computation (the checker may run on
    the GPU for the full-size model: plain torch f32 arithmetic, none of the product's kernels).
    With microbatches > 1 a batch is split along its first dimension and the gradients of the
    per-token mean over the WHOLE batch are accumulated (crates/sky-1/src/skyred/training.rs:263-317)."""
    if str(device) != "cpu":
        torch.backends.cuda.matmul.allow_tf32 = False  # full f32 products in the checker
    master = {n: p.detach().to(device).float().clone() for n, p in params.items()}
    table = table.to(device)
    m = {n: torch.zeros_like(p) for n, p in master.items()}
    v = {n: torch.zeros_like(p) for n, p in master.items()}
    losses = []
    for step, (tokens, targets) in enumerate(batches, start=1):
        tokens, targets = tokens.to(device), targets.to(device)
        work = {n: (p.to(torch.bfloat16).float() if round_weights_to_bf16 else p.clone()).requires_grad_(True)
                for n, p in master.items()}
        total = 0.0
        for tk, tg in zip(tokens.chunk(microbatches), targets.chunk(microbatches)):
            loss = lm_loss(work, tk, tg, cfg, table, layers, dtype, reduction="sum",
                           checkpoint_blocks=checkpoint_blocks) / targets.numel()
            loss.backward()
            total += float(loss.detach())
        losses.append(total)
        adamw_step(master, {n: w.grad for n, w in work.items()}, m, v, step, lr, beta1, beta2, eps, wd)
        del work
    return losses, master

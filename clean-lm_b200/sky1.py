"""sky-1 decoder block on the C ABI (host side of `cdl_b200_sky1_block_fwd/_bwd`).

Mirrors the reference's DecoderExecutor (crates/sky-1/src/training/model/decoder.rs:332-752):
parameters are bf16 replicas stored [in, out] with f32 gradients (parameter.rs:11-17), the forward
saves qkv / attn / lse / o / up / gate / act, and the backward accumulates weight gradients.
torch only owns the memory; every kernel is in libcleandl_b200.so.
"""
from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass

import torch

from . import _lib
from ._lib import check, lib

PARAM_NAMES = _lib._BLOCK_PARAMS


@dataclass
class Sky1Config:
    batch: int = 8
    seqlen: int = 2048
    hidden: int = 2048
    heads: int = 16
    kv_heads: int = 16
    head_dim: int = 128
    ffn: int = 5632
    eps: float = 1e-6
    rope_base: float = 10000.0
    deterministic: bool = False  # weight-gradient GEMMs with a fixed summation order

    @property
    def tokens(self) -> int:
        return self.batch * self.seqlen

    @property
    def qkv_dim(self) -> int:
        return (self.heads + 2 * self.kv_heads) * self.head_dim

    def param_shapes(self) -> dict:
        hd = self.heads * self.head_dim
        return {"norm1": (self.hidden,), "wqkv": (self.hidden, self.qkv_dim), "wo": (hd, self.hidden),
                "norm2": (self.hidden,), "wup": (self.hidden, self.ffn),
                "wgate": (self.hidden, self.ffn), "wdown": (self.ffn, self.hidden)}

    def param_count(self) -> int:
        return sum(math.prod(s) for s in self.param_shapes().values())

    def c_struct(self) -> _lib.CdlSky1Config:
        return _lib.CdlSky1Config(self.batch, self.seqlen, self.hidden, self.heads, self.kv_heads,
                                  self.head_dim, self.ffn, self.eps,
                                  _lib.CDL_SKY1_DETERMINISTIC if self.deterministic else 0)

    def flops_fwd_bwd(self) -> float:
        """Algorithmic FLOP of one block forward + backward: 3 x the five GEMMs' 2MNK plus causal
        attention forward (4 B H S^2 D / 2) and backward (2.5 x forward)."""
        t, hd = self.tokens, self.heads * self.head_dim
        gemm = 2.0 * t * (self.hidden * self.qkv_dim + hd * self.hidden + 3 * self.hidden * self.ffn)
        attn = 4.0 * self.batch * self.heads * self.seqlen ** 2 * self.head_dim / 2
        return 3 * gemm + 3.5 * attn


def rope_table(seqlen: int, head_dim: int, base: float = 10000.0, device="cuda") -> torch.Tensor:
    """f32 [seqlen, head_dim] = cos | sin of pos * base^(-2i/D) (rotate-half convention)."""
    half = head_dim // 2
    inv_freq = base ** (-torch.arange(half, dtype=torch.float64) * 2.0 / head_dim)
    ang = torch.arange(seqlen, dtype=torch.float64)[:, None] * inv_freq[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=1).to(torch.float32).to(device)


def init_params(cfg: Sky1Config, seed: int, std: float = 0.02) -> dict:
    """bf16 weights ~ N(0, std) and norm gains = 1, generated on the CPU from `seed`."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in cfg.param_shapes().items():
        if name.startswith("norm"):
            out[name] = torch.ones(shape, dtype=torch.bfloat16)
        else:
            out[name] = (torch.randn(shape, generator=gen) * std).to(torch.bfloat16)
    return out


class Sky1Block:
    """One decoder block: device weights, f32 gradient buffers, saved activations."""

    def __init__(self, cfg: Sky1Config, params: dict, device="cuda", grads: dict | None = None,
                 workspace: torch.Tensor | None = None, table: torch.Tensor | None = None,
                 cu_seqlens: torch.Tensor | None = None, max_seqlen: int | None = None):
        """`cu_seqlens` (i32 [num_seqs + 1], device) makes the cfg.tokens rows a ragged batch: sequence
        b is rows cu_seqlens[b] .. cu_seqlens[b + 1] (the layout of the reference's
        `decoder_ragged_seqlen`, decoder.rs:372-378); `max_seqlen` bounds every length.  Rows after
        the last sequence are padding: x there must be finite and dy zero."""
        self.cfg = cfg
        self.device = device
        self.cu_seqlens = cu_seqlens
        self._rg_c = None
        if cu_seqlens is not None:
            if cu_seqlens.dtype != torch.int32 or not cu_seqlens.is_cuda or cu_seqlens.dim() != 1:
                raise _lib.CdlError(-1, "cu_seqlens must be an i32 vector on the device")
            max_seqlen = int(max_seqlen if max_seqlen else cfg.tokens)
            self._rg_c = _lib.CdlSky1Ragged(cu_seqlens.data_ptr(), cu_seqlens.numel() - 1, max_seqlen)
        def on_device(p):  # views of a caller-owned flat buffer are used in place, not copied
            if p.is_cuda and p.dtype == torch.bfloat16 and p.is_contiguous():
                return p
            return p.to(device=device, dtype=torch.bfloat16).contiguous()

        self.params = {n: on_device(params[n]) for n in PARAM_NAMES}
        for n, shape in cfg.param_shapes().items():
            if tuple(self.params[n].shape) != tuple(shape):
                raise _lib.CdlError(-1, f"parameter {n} must have shape {shape}")
        # Gradients may be views into a caller-owned flat bucket (see the data-parallel step).
        self.grads = grads if grads is not None else {
            n: torch.zeros(s, dtype=torch.float32, device=device) for n, s in cfg.param_shapes().items()}
        t = cfg.tokens
        bf = dict(dtype=torch.bfloat16, device=device)
        self.saved = {
            "qkv": torch.empty(t, cfg.qkv_dim, **bf),
            "attn": torch.empty(t, cfg.heads * cfg.head_dim, **bf),
            # dense: [batch, heads, seqlen]; ragged: [heads, tokens] -- the same number of elements
            "lse": torch.empty(cfg.batch, cfg.heads, cfg.seqlen, dtype=torch.float32, device=device),
            "o": torch.empty(t, cfg.hidden, **bf),
            "up": torch.empty(t, cfg.ffn, **bf),
            "gate": torch.empty(t, cfg.ffn, **bf),
            "act": torch.empty(t, cfg.ffn, **bf),
        }
        rows = self._rg_c.max_seqlen if self._rg_c is not None else cfg.seqlen
        self.table = table if table is not None else rope_table(rows, cfg.head_dim, cfg.rope_base, device)
        self._cfg_c = cfg.c_struct()
        fwd, bwd = ctypes.c_size_t(0), ctypes.c_size_t(0)
        if self._rg_c is not None:
            check(lib.cdl_b200_sky1_block_workspace_bytes_ragged(
                ctypes.byref(self._cfg_c), ctypes.byref(self._rg_c), ctypes.byref(fwd), ctypes.byref(bwd)))
        else:
            check(lib.cdl_b200_sky1_block_workspace_bytes(ctypes.byref(self._cfg_c), ctypes.byref(fwd),
                                                          ctypes.byref(bwd)))
        self.workspace_bytes = max(fwd.value, bwd.value)
        self.workspace = workspace if workspace is not None else torch.empty(
            self.workspace_bytes, dtype=torch.uint8, device=device)
        if self.workspace.numel() < self.workspace_bytes:
            raise _lib.CdlError(-1, f"workspace must hold {self.workspace_bytes} bytes")
        self._w_c = _lib.CdlSky1Weights(*(self.params[n].data_ptr() for n in PARAM_NAMES))
        self._g_c = _lib.CdlSky1Grads(*(self.grads[n].data_ptr() for n in PARAM_NAMES))
        self._s_c = _lib.CdlSky1Saved(*(self.saved[n].data_ptr()
                                        for n in ("qkv", "attn", "lse", "o", "up", "gate", "act")))
        self._x = None

    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def forward(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """x: bf16 [tokens, hidden] (or [batch, seqlen, hidden]); keeps a reference for backward."""
        cfg = self.cfg
        if x.dtype != torch.bfloat16 or x.numel() != cfg.tokens * cfg.hidden or not x.is_contiguous():
            raise _lib.CdlError(-1, "x must be a contiguous bf16 tensor of [tokens, hidden]")
        out = torch.empty_like(x) if out is None else out
        if self._rg_c is not None:
            check(lib.cdl_b200_sky1_block_fwd_ragged(
                ctypes.byref(self._cfg_c), ctypes.byref(self._w_c), x.data_ptr(), self.table.data_ptr(),
                ctypes.byref(self._rg_c), ctypes.byref(self._s_c), out.data_ptr(),
                self.workspace.data_ptr(), self.workspace.numel(), self._stream()))
            self._x = x
            return out
        check(lib.cdl_b200_sky1_block_fwd(
            ctypes.byref(self._cfg_c), ctypes.byref(self._w_c), x.data_ptr(), self.table.data_ptr(),
            ctypes.byref(self._s_c), out.data_ptr(), self.workspace.data_ptr(),
            self.workspace.numel(), self._stream()))
        self._x = x
        return out

    #: gradient groups in the order the backward completes them (cdl_sky1_grad_events)
    GRAD_GROUPS = (("wdown",), ("wup",), ("wgate", "norm2"), ("wo",), ("wqkv", "norm1"))

    def backward(self, dy: torch.Tensor, dx: torch.Tensor | None = None, phase: int = 0,
                 events=None) -> torch.Tensor:
        """dy: gradient of the forward's output. Accumulates into self.grads; returns dx.
        phase 1 / 2 run the FFN half / the attention half (see cdl_b200_sky1_block_bwd).
        `events`: five torch.cuda.Event, one per entry of GRAD_GROUPS, each recorded on the
        current stream as soon as that group's gradients are complete (whole backward only)."""
        if self._x is None:
            raise _lib.CdlError(-1, "backward called before forward")
        if dy.dtype != torch.bfloat16 or dy.numel() != self._x.numel() or not dy.is_contiguous():
            raise _lib.CdlError(-1, "dy must be a contiguous bf16 tensor shaped like x")
        dx = torch.empty_like(dy) if dx is None else dx
        if events is not None:
            if phase != 0 or len(events) != len(self.GRAD_GROUPS):
                raise _lib.CdlError(-1, "events: five events and the whole backward (phase 0)")
            handles = []
            for e in events:
                if not e.cuda_event:  # torch creates the CUDA event at its first record
                    e.record()
                handles.append(e.cuda_event)
            ev_c = _lib.CdlSky1GradEvents(*handles)
            check(lib.cdl_b200_sky1_block_bwd_events(
                ctypes.byref(self._cfg_c), ctypes.byref(self._w_c), self._x.data_ptr(),
                self.table.data_ptr(), ctypes.byref(self._rg_c) if self._rg_c is not None else None,
                ctypes.byref(self._s_c), dy.data_ptr(), ctypes.byref(self._g_c), dx.data_ptr(),
                self.workspace.data_ptr(), self.workspace.numel(), ctypes.byref(ev_c), self._stream()))
            return dx
        if self._rg_c is not None:
            check(lib.cdl_b200_sky1_block_bwd_ragged(
                ctypes.byref(self._cfg_c), ctypes.byref(self._w_c), self._x.data_ptr(),
                self.table.data_ptr(), ctypes.byref(self._rg_c), ctypes.byref(self._s_c), dy.data_ptr(),
                ctypes.byref(self._g_c), dx.data_ptr(), self.workspace.data_ptr(),
                self.workspace.numel(), phase, self._stream()))
            return dx
        check(lib.cdl_b200_sky1_block_bwd(
            ctypes.byref(self._cfg_c), ctypes.byref(self._w_c), self._x.data_ptr(),
            self.table.data_ptr(), ctypes.byref(self._s_c), dy.data_ptr(), ctypes.byref(self._g_c),
            dx.data_ptr(), self.workspace.data_ptr(), self.workspace.numel(), phase, self._stream()))
        return dx

    def zero_grads(self):
        for g in self.grads.values():
            g.zero_()


# ======================================================================= full LM training step
@dataclass
class Sky1LMConfig:
    """24-layer sky-1-style LM of benchmark configuration 5 by default."""

    block: Sky1Config
    layers: int = 24
    vocab: int = 32768
    lr: float = 3e-4
    beta1: float = 0.9
    beta2: float = 0.95
    adam_eps: float = 1e-8
    weight_decay: float = 0.1
    max_grad_norm: float = 0.0  # 0 = no clipping

    def param_count(self) -> int:
        return self.layers * self.block.param_count() + 2 * self.vocab * self.block.hidden + self.block.hidden


_BLOCK_ORDER = ("wdown", "wup", "wgate", "wo", "wqkv", "norm2", "norm1")  # decayed first, gains last


class Sky1LM:
    """Embedding -> blocks -> final RMSNorm -> LM head -> cross-entropy, with the optimizer state.

    Follows the reference's Sky1Executor (crates/sky-1/src/training/model/mod.rs:209-420): f32
    master weights with bf16 replicas, f32 gradients accumulated over microbatches
    (crates/sky-1/src/skyred/training.rs:263-317), AdamW without weight decay on norm gains.
    All parameters live in flat buffers laid out in BACKWARD order (LM head first, embedding
    last) so a data-parallel run can all-reduce a layer's gradient slice as soon as that layer's
    backward has been enqueued.
    """

    def __init__(self, cfg: Sky1LMConfig, seed: int = 4, device="cuda", std: float = 0.02,
                 process_group=None, init_on_device: bool = False):
        """`init_on_device` draws the initial weights with the device's generator (seconds for the
        24-layer model) instead of the host's; both are N(0, std) from `seed`, but not the same
        values."""
        import torch.distributed as dist

        self.cfg, self.device = cfg, torch.device(device)
        b = cfg.block
        self.world = dist.get_world_size(process_group) if (dist.is_available() and dist.is_initialized()) else 1
        self.group = process_group
        layout = [("lm_head", (b.hidden, cfg.vocab), True), ("final_norm", (b.hidden,), False)]
        for layer in reversed(range(cfg.layers)):
            for n in _BLOCK_ORDER:
                layout.append((f"blocks.{layer}.{n}", b.param_shapes()[n], not n.startswith("norm")))
        layout.append(("embedding", (cfg.vocab, b.hidden), True))
        self.layout, self.offsets, off = layout, {}, 0
        for name, shape, _ in layout:
            self.offsets[name] = (off, math.prod(shape))
            off += math.prod(shape)
        self.numel = off
        f32 = dict(dtype=torch.float32, device=self.device)
        self.master = torch.empty(off, **f32)
        self.m = torch.zeros(off, **f32)
        self.v = torch.zeros(off, **f32)
        self.grads = torch.zeros(off, **f32)
        self.replica = torch.empty(off, dtype=torch.bfloat16, device=self.device)
        init_dev = self.device if init_on_device else torch.device("cpu")
        gen = torch.Generator(device=init_dev).manual_seed(seed)
        # drawn in name order, so the values do not depend on the flat layout
        for name, shape, _ in sorted(layout, key=lambda t: t[0]):
            o, n = self.offsets[name]
            if "norm" in name:
                self.master[o:o + n].fill_(1.0)
            else:
                self.master[o:o + n].copy_(
                    (torch.randn(shape, generator=gen, device=init_dev) * std).reshape(-1))
        self.replica.copy_(self.master)
        # contiguous runs with one weight-decay setting -> one AdamW launch each
        self.segments = []
        for name, shape, decay in layout:
            o, n = self.offsets[name]
            if self.segments and self.segments[-1][2] == decay and self.segments[-1][0] + self.segments[-1][1] == o:
                self.segments[-1][1] += n
            else:
                self.segments.append([o, n, decay])
        t = b.tokens
        self.table = rope_table(b.seqlen, b.head_dim, b.rope_base, self.device)
        self.blocks = []
        workspace = None
        for layer in range(cfg.layers):
            params = {n: self.view("replica", f"blocks.{layer}.{n}") for n in PARAM_NAMES}
            grads = {n: self.view("grads", f"blocks.{layer}.{n}") for n in PARAM_NAMES}
            blk = Sky1Block(b, params, device=self.device, grads=grads, workspace=workspace, table=self.table)
            workspace = blk.workspace
            self.blocks.append(blk)
        bf = dict(dtype=torch.bfloat16, device=self.device)
        self.acts = [torch.empty(t, b.hidden, **bf) for _ in range(cfg.layers + 1)]
        self.hf = torch.empty(t, b.hidden, **bf)
        self.r_inv = torch.empty(t, **f32)
        self.logits = torch.empty(t, cfg.vocab, **bf)
        self.loss_tok = torch.empty(t, **f32)
        self.loss = torch.zeros(1, **f32)
        self.sumsq = torch.zeros(1, **f32)
        self.dx = [torch.empty(t, b.hidden, **bf) for _ in range(2)]
        self.red_scratch = torch.empty(4096, dtype=torch.uint8, device=self.device)
        self.norm_scratch = torch.empty(ops_norm_bwd_scratch(t, b.hidden), dtype=torch.uint8, device=self.device)
        self.step_count = 0
        self.comm = torch.cuda.Stream(device=self.device) if self.world > 1 else None
        self._tokens = None

    def view(self, which: str, name: str) -> torch.Tensor:
        o, n = self.offsets[name]
        shape = next(s for nm, s, _ in self.layout if nm == name)
        return getattr(self, which)[o:o + n].view(shape)

    # ---- one microbatch
    def forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor, loss_scale: float,
                         reduce_grads: bool = True) -> None:
        """tokens, targets: i32 [tokens] on the device.  Adds loss_scale * sum of token losses to
        self.loss and accumulates gradients of that quantity.  With reduce_grads (the last
        microbatch of a step) every layer's gradient slice is all-reduced as soon as its backward
        is enqueued."""
        from . import ops

        L, c = _lib, self.cfg
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        ta = L.tensor_arg
        tok, tgt = ta(tokens), ta(targets)
        emb = ta(self.view("replica", "embedding"))
        x0 = ta(self.acts[0])
        check(lib.cdl_b200_embedding_fwd(L.ref(tok), L.ref(emb), L.ref(x0), st))
        for i, blk in enumerate(self.blocks):
            blk.forward(self.acts[i], self.acts[i + 1])
        xl, hf, gam, rinv = ta(self.acts[-1]), ta(self.hf), ta(self.view("replica", "final_norm")), ta(self.r_inv)
        check(lib.cdl_b200_rmsnorm_fwd(L.ref(xl), L.ref(gam), None, c.block.eps, L.ref(hf), L.ref(rinv), st))
        ops.matmul(self.hf, self.view("replica", "lm_head"), out=self.logits)
        lg, lt = ta(self.logits), ta(self.loss_tok)
        check(lib.cdl_b200_cross_entropy(L.ref(lg), L.ref(tgt), L.ref(lt), loss_scale, st))
        check(lib.cdl_b200_sum(self.loss_tok.data_ptr(), self.loss_tok.numel(), self.loss.data_ptr(),
                               loss_scale, 0, 1, self.red_scratch.data_ptr(), 4096, st))
        # backward
        g_head = self.view("grads", "lm_head")
        ops.matmul(self.hf.T, self.logits, ops.MatmulOpts(out=torch.float32, c=g_head, beta=1.0), out=g_head)
        ops.matmul(self.logits, self.view("replica", "lm_head").T, out=self.hf)  # d_hf, in place of hf
        dgam, dxl = ta(self.view("grads", "final_norm")), ta(self.dx[0])
        check(lib.cdl_b200_rmsnorm_bwd(L.ref(xl), L.ref(hf), None, L.ref(gam), L.ref(rinv), L.ref(dxl),
                                       L.ref(dgam), self.norm_scratch.data_ptr(),
                                       self.norm_scratch.numel(), st))
        if reduce_grads:
            self._reduce("lm_head", "final_norm")
        cur = 0
        for i in reversed(range(c.layers)):
            self.blocks[i]._x = self.acts[i]
            self.blocks[i].backward(self.dx[cur], self.dx[cur ^ 1])
            cur ^= 1
            if reduce_grads:
                self._reduce(f"blocks.{i}.{_BLOCK_ORDER[0]}", f"blocks.{i}.{_BLOCK_ORDER[-1]}")
        d0, ge = ta(self.dx[cur]), ta(self.view("grads", "embedding"))
        check(lib.cdl_b200_embedding_bwd(L.ref(tok), L.ref(d0), L.ref(ge), st))
        if reduce_grads:
            self._reduce("embedding", "embedding")

    def _reduce(self, first: str, last: str) -> None:
        if self.world == 1:
            return
        import torch.distributed as dist

        lo = self.offsets[first][0]
        hi = self.offsets[last][0] + self.offsets[last][1]
        ev = torch.cuda.Event()
        ev.record()
        with torch.cuda.stream(self.comm):
            self.comm.wait_event(ev)
            dist.all_reduce(self.grads[lo:hi], group=self.group)

    # ---- optimizer
    def optimizer_step(self, lr: float | None = None) -> None:
        c = self.cfg
        if self.comm is not None:
            torch.cuda.current_stream().wait_stream(self.comm)
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        self.step_count += 1
        sumsq_ptr = None
        if c.max_grad_norm > 0:
            check(lib.cdl_b200_sum(self.grads.data_ptr(), self.numel, self.sumsq.data_ptr(), 1.0, 1, 0,
                                   self.red_scratch.data_ptr(), 4096, st))
            sumsq_ptr = self.sumsq.data_ptr()
        for o, n, decay in self.segments:
            hp = _lib.CdlAdamwParams(lr if lr is not None else c.lr, c.beta1, c.beta2, c.adam_eps,
                                     c.weight_decay if decay else 0.0, self.step_count, 1.0,
                                     c.max_grad_norm)
            check(lib.cdl_b200_adamw(self.master.data_ptr() + 4 * o, self.replica.data_ptr() + 2 * o,
                                     self.grads.data_ptr() + 4 * o, self.m.data_ptr() + 4 * o,
                                     self.v.data_ptr() + 4 * o, n, sumsq_ptr, ctypes.byref(hp), st))

    def train_step(self, tokens: torch.Tensor, targets: torch.Tensor, global_tokens: int | None = None,
                   lr: float | None = None) -> torch.Tensor:
        """tokens, targets: i32 [microbatches, tokens_per_microbatch].  One optimizer step over all
        microbatches (gradient accumulation); returns the device scalar with the mean loss of this
        rank's share (sum over ranks = global mean)."""
        mb = tokens.shape[0]
        total = global_tokens if global_tokens is not None else tokens.numel() * self.world
        self.loss.zero_()
        for i in range(mb):
            self.forward_backward(tokens[i], targets[i], 1.0 / total, reduce_grads=(i == mb - 1))
        self.optimizer_step(lr)
        return self.loss


def ops_norm_bwd_scratch(rows: int, cols: int) -> int:
    n = ctypes.c_size_t(0)
    check(lib.cdl_b200_rmsnorm_bwd_scratch_bytes(rows, cols, ctypes.byref(n)))
    return max(n.value, 16)

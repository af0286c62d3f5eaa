"""Checkpoint wire format (crates/sky-1/src/training/checkpoint.rs): container layout, tensor
names, round trips.  The container tests need no GPU; the LM round trip does."""
import json
import math
import struct

import numpy as np
import pytest
import torch


def _ckpt():
    # the module has no CUDA dependency of its own; load it without importing the package
    import importlib.util
    from pathlib import Path

    path = Path(__file__).resolve().parents[1] / "clean-lm_b200" / "checkpoint.py"
    spec = importlib.util.spec_from_file_location("cdl_checkpoint", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class FakeLM:
    """The attributes of Sky1LM the checkpoint code touches, on the CPU."""

    def __init__(self, layers=2, hidden=8, ffn=12, qkv=24, vocab=16, seed=0):
        shapes = {"wdown": (ffn, hidden), "wup": (hidden, ffn), "wgate": (hidden, ffn), "wo": (hidden, hidden),
                  "wqkv": (hidden, qkv), "norm2": (hidden,), "norm1": (hidden,)}
        self.layout = [("lm_head", (hidden, vocab), True), ("final_norm", (hidden,), False)]
        for layer in reversed(range(layers)):
            for n, s in shapes.items():
                self.layout.append((f"blocks.{layer}.{n}", s, not n.startswith("norm")))
        self.layout.append(("embedding", (vocab, hidden), True))
        self.offsets, off = {}, 0
        for name, shape, _ in self.layout:
            self.offsets[name] = (off, math.prod(shape))
            off += math.prod(shape)
        gen = torch.Generator().manual_seed(seed)
        self.master = torch.randn(off, generator=gen)
        self.m = torch.randn(off, generator=gen)
        self.v = torch.rand(off, generator=gen)
        self.replica = self.master.to(torch.bfloat16)
        self.step_count = 17

    def view(self, which, name):
        o, n = self.offsets[name]
        shape = next(s for nm, s, _ in self.layout if nm == name)
        return getattr(self, which)[o:o + n].view(shape)


def test_reference_names():
    ck = _ckpt()
    assert ck.reference_name("embedding") == "embeddings.weight"
    assert ck.reference_name("final_norm") == "final_norm.gamma"
    assert ck.reference_name("lm_head") == "lm_head.weight"
    assert ck.reference_name("blocks.3.wqkv") == "decoder_blocks[3]/qkv_proj.weight"
    assert ck.reference_name("blocks.0.norm1") == "decoder_blocks[0]/pre_qkv_norm.gamma"
    assert ck.reference_name("blocks.11.norm2") == "decoder_blocks[11]/pre_ffn_norm.gamma"
    assert ck.reference_name("blocks.2.wup") == "decoder_blocks[2]/ffn.up"
    assert ck.reference_name("blocks.2.wgate") == "decoder_blocks[2]/ffn.gate"
    assert ck.reference_name("blocks.2.wdown") == "decoder_blocks[2]/ffn.down"
    assert ck.reference_name("blocks.2.wo") == "decoder_blocks[2]/o_proj.weight"
    with pytest.raises(KeyError):
        ck.reference_name("blocks.2.bias")


def test_container_layout(tmp_path):
    ck = _ckpt()
    a = np.arange(6, dtype=np.float32).reshape(2, 3)
    b = np.array([1.5, -2.0], dtype=np.float32)
    path = tmp_path / "t.safetensors"
    ck.write_safetensors(path, [("x.weight", a), ("y:adam_m", b)], {"train_step": "5"})
    raw = path.read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    assert n % 8 == 0
    header = json.loads(raw[8:8 + n])
    assert header["__metadata__"] == {"train_step": "5"}
    assert header["x.weight"] == {"dtype": "F32", "shape": [2, 3], "data_offsets": [0, 24]}
    assert header["y:adam_m"] == {"dtype": "F32", "shape": [2], "data_offsets": [24, 32]}
    assert len(raw) == 8 + n + 32
    assert np.frombuffer(raw[8 + n:8 + n + 24], dtype="<f4").tolist() == a.reshape(-1).tolist()
    tensors, meta = ck.read_safetensors(path)
    assert meta == {"train_step": "5"}
    assert np.array_equal(tensors["x.weight"], a) and np.array_equal(tensors["y:adam_m"], b)


def test_container_rejects_bad_files(tmp_path):
    ck = _ckpt()
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"\x01\x02")
    with pytest.raises(ValueError, match="too short"):
        ck.read_safetensors(p)
    p.write_bytes(struct.pack("<Q", 1000) + b"{}")
    with pytest.raises(ValueError, match="exceeds"):
        ck.read_safetensors(p)
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(ValueError, match="inconsistent"):
        ck.read_safetensors(p)
    with pytest.raises(ValueError, match="duplicate"):
        ck.write_safetensors(tmp_path / "d.safetensors", [("a", np.zeros(1, np.float32)), ("a", np.zeros(1, np.float32))])


def test_lm_round_trip_on_cpu(tmp_path):
    ck = _ckpt()
    src = FakeLM(seed=1)
    ck.save_checkpoint(src, tmp_path)
    model, meta_m = ck.read_safetensors(tmp_path / "model.safetensors")
    optim, meta_o = ck.read_safetensors(tmp_path / "optimizer.safetensors")
    assert meta_m == {} and meta_o == {"train_step": "17"}
    assert len(model) == len(src.layout) and len(optim) == 2 * len(src.layout)
    assert model["decoder_blocks[1]/ffn.up"].shape == (8, 12)
    assert set(optim) == {k + s for k in model for s in (":adam_m", ":adam_v")}
    dst = FakeLM(seed=2)
    assert ck.load_checkpoint(dst, tmp_path) == 17
    assert torch.equal(dst.master, src.master) and torch.equal(dst.m, src.m) and torch.equal(dst.v, src.v)
    assert torch.equal(dst.replica, src.master.to(torch.bfloat16)) and dst.step_count == 17
    # a checkpoint of another configuration is refused
    with pytest.raises(ValueError, match="shape"):
        ck.load_checkpoint(FakeLM(hidden=16, qkv=48, seed=3), tmp_path)
    with pytest.raises(KeyError, match="no tensor"):
        ck.load_checkpoint(FakeLM(layers=3, seed=3), tmp_path)


@pytest.mark.gpu
def test_lm_resume_is_bit_exact(cdl, gpu_ok, tmp_path, monkeypatch):
    """Train two steps, save, load into a fresh model, and continue both: same loss, same weights.
    (K-sliced weight-gradient GEMMs add with atomics in no fixed order; the deterministic mode
    switches that off so that the two runs can be compared bit for bit.)"""
    monkeypatch.setenv("CDL_B200_DETERMINISTIC", "1")
    sky1 = cdl.sky1
    block = sky1.Sky1Config(batch=2, seqlen=128, hidden=256, heads=2, kv_heads=2, head_dim=128, ffn=384)
    cfg = sky1.Sky1LMConfig(block=block, layers=2, vocab=512, lr=1e-3)
    gen = torch.Generator().manual_seed(0)
    toks = torch.randint(0, cfg.vocab, (3, 1, block.tokens), generator=gen, dtype=torch.int32).cuda()
    tgts = torch.randint(0, cfg.vocab, (3, 1, block.tokens), generator=gen, dtype=torch.int32).cuda()
    a = sky1.Sky1LM(cfg, seed=4)
    for i in range(2):
        a.train_step(toks[i], tgts[i])
    cdl.checkpoint.save_checkpoint(a, tmp_path)
    b = sky1.Sky1LM(cfg, seed=9)
    assert cdl.checkpoint.load_checkpoint(b, tmp_path) == 2
    la = a.train_step(toks[2], tgts[2]).clone()
    lb = b.train_step(toks[2], tgts[2]).clone()
    torch.cuda.synchronize()
    assert torch.equal(la, lb)
    assert torch.equal(a.master, b.master) and torch.equal(a.m, b.m) and torch.equal(a.v, b.v)

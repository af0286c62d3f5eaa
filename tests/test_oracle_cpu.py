"""CPU checks of the oracle (oracle/cpu_ref.c, oracle/block_ref.py): against the committed golden
fixtures (float64 torch results, tests/golden/make_golden.py) and against the properties the
reference's own tests rely on (mask alignment, -inf LSE for rows without keys, error bound)."""
from pathlib import Path

import numpy as np
import torch

from oracle import block_ref
from oracle import cpu_oracle as oracle

GOLDEN = Path(__file__).resolve().parent / "golden"


def close(a, b, tol=2e-6):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.abs(a - b).max() <= tol * max(1.0, np.abs(b).max())


def test_matmul_matches_golden_and_bound():
    g = np.load(GOLDEN / "matmul.npz")
    out, bound = oracle.matmul(g["a"], g["b"], g["c"], float(g["alpha"]), float(g["beta"]))
    assert close(out, g["out"])
    ref_bound = 0.5 * np.abs(g["a"].astype(np.float64)) @ np.abs(g["b"].astype(np.float64)) \
        + np.abs(2.0 * g["c"].astype(np.float64))
    assert close(bound, ref_bound, 1e-6)
    tol = oracle.matmul_tolerance(out, bound, True)
    assert (tol > 0).all()


def test_matmul_batched_no_c():
    rng = np.random.default_rng(1)
    a = oracle.bf16_round(rng.standard_normal((3, 17, 40)).astype(np.float32))
    b = oracle.bf16_round(rng.standard_normal((3, 40, 24)).astype(np.float32))
    out, _ = oracle.matmul(a, b)
    assert close(out, np.einsum("bik,bkj->bij", a.astype(np.float64), b.astype(np.float64)))


def test_bf16_round_is_round_to_nearest_even():
    x = torch.randn(10000, generator=torch.Generator().manual_seed(0))
    assert np.array_equal(oracle.bf16_round(x.numpy()), x.to(torch.bfloat16).float().numpy())


def test_rmsnorm_matches_golden():
    g = np.load(GOLDEN / "rmsnorm.npz")
    y, r_inv = oracle.rmsnorm_fwd(g["x"], g["scale"], g["bias"], float(g["eps"]))
    assert close(y, g["y"]) and close(r_inv, g["r_inv"])
    dx, dscale = oracle.rmsnorm_bwd(g["x"], g["dy"], g["scale"], None, float(g["eps"]))
    assert close(dx, g["dx"]) and close(dscale, g["dscale"], 1e-9)
    res = np.ones_like(g["x"])
    dx2, dscale2 = oracle.rmsnorm_bwd(g["x"], g["dy"], g["scale"], res, float(g["eps"]),
                                      dscale_init=np.full(g["x"].shape[1], 3.0))
    assert close(dx2, g["dx"] + 1.0) and close(dscale2, g["dscale"] + 3.0, 1e-9)


def test_attention_matches_golden():
    g = np.load(GOLDEN / "attention.npz")
    r = oracle.attention(g["q"], g["k"], g["v"], g["d_out"], causal=True)
    for name in ("out", "lse", "dq", "dk", "dv"):
        assert close(r[name], g[name], 5e-6), name


def test_attention_rows_without_keys():
    """sq > sk with the bottom-right aligned mask: the first sq - sk rows see no key."""
    rng = np.random.default_rng(2)
    q = oracle.bf16_round(rng.standard_normal((1, 6, 1, 128)).astype(np.float32))
    kv = oracle.bf16_round(rng.standard_normal((1, 4, 1, 128)).astype(np.float32))
    r = oracle.attention(q, kv, kv, q, causal=True)
    assert np.isneginf(r["lse"][0, 0, :2]).all() and np.isfinite(r["lse"][0, 0, 2:]).all()
    assert (r["out"][0, :2] == 0).all() and (r["dq"][0, :2] == 0).all()


def test_attention_tolerance_formula():
    e = np.array([0.0, -2.0, 0.5, -np.inf], dtype=np.float32)
    t = oracle.attention_tolerance(e, 1e-2, 1e-2)
    assert np.allclose(t[:3], 1e-2 * 2.0 + 1e-2 * np.abs(e[:3]))


def test_block_oracle_float32_agrees_with_float64():
    cfg = dict(heads=2, kv_heads=1, head_dim=128, eps=1e-6)
    gen = torch.Generator().manual_seed(5)
    w = {"norm1": torch.ones(256), "norm2": torch.ones(256),
         "wqkv": torch.randn(256, 512, generator=gen) * 0.05, "wo": torch.randn(256, 256, generator=gen) * 0.05,
         "wup": torch.randn(256, 264, generator=gen) * 0.05, "wgate": torch.randn(256, 264, generator=gen) * 0.05,
         "wdown": torch.randn(264, 256, generator=gen) * 0.05}
    x = torch.randn(1, 64, 256, generator=gen)
    dy = torch.randn(1, 64, 256, generator=gen)
    t = block_ref.rope_table(64, 128)
    o64, dx64, g64 = block_ref.block_forward_backward(x, w, dy, cfg, t)
    o32, dx32, g32 = block_ref.block_forward_backward(x, w, dy, cfg, t, dtype=torch.float32)
    assert close(o32, o64, 1e-4) and close(dx32, dx64, 1e-4)
    assert all(close(g32[n], g64[n], 1e-4) for n in g64)


def test_rope_is_a_rotation_and_backward_is_its_inverse():
    t = block_ref.rope_table(32, 128).double()
    x = torch.randn(1, 32, 3, 128, dtype=torch.float64, generator=torch.Generator().manual_seed(6))
    y = block_ref.rope(x, t)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    inv = torch.cat([t[:, :64], -t[:, 64:]], dim=1)
    assert torch.allclose(block_ref.rope(y, inv), x)

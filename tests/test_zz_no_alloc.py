"""The allocation-free RMSNorm backward (cdl_b200_rmsnorm_bwd_static) must give exactly what the
scratch-taking entry point gives.

It exists for hosts that can neither allocate device memory nor lend a scratch slice at the point
where they run the backward (allocator callbacks, fixed-budget real-time loops, plugins whose host
owns all memory); it keeps its scratch in an 8 MiB array inside the library's device image.  Two
calls in a row are checked because the array is shared by all calls and keeps the previous call's
contents.  The file is named so that pytest collects it last.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(cdl, static, x, dy, res, w, r_inv, dscale):
    L = cdl._lib
    dx = torch.empty_like(x)
    args = [L.tensor_arg(t) for t in (x, dy, res, w, r_inv, dx, dscale)]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if static:
        L.check(L.lib.cdl_b200_rmsnorm_bwd_static(*(L.ref(a) for a in args), stream))
    else:
        n = cdl.ops.norm_bwd_scratch_bytes(*x.shape)
        scratch = torch.empty(n, dtype=torch.uint8, device=x.device)
        L.check(L.lib.cdl_b200_rmsnorm_bwd(*(L.ref(a) for a in args),
                                           ctypes.c_void_p(scratch.data_ptr()), n, stream))
    torch.cuda.synchronize()
    return dx


def test_static_scratch_matches_caller_scratch_twice(cdl, gpu_ok):
    gen = torch.Generator().manual_seed(42)
    # Two different problems back to back: the second call finds the first call's partial sums
    # in the shared array (and uses fewer partial rows than the first wrote).
    for rows, cols, with_res in ((3000, 2048, True), (70, 1024, False)):
        x = torch.randn(rows, cols, generator=gen).to(torch.bfloat16).cuda()
        dy = torch.randn(rows, cols, generator=gen).to(torch.bfloat16).cuda()
        res = torch.randn(rows, cols, generator=gen).to(torch.bfloat16).cuda() if with_res else None
        w = (1 + 0.02 * torch.randn(cols, generator=gen)).to(torch.bfloat16).cuda()
        r_inv = cdl.ops.norm_fwd(x, cdl.ops.NormFwdOpts(scale=w, save_stats=True)).r_inv
        ds0 = torch.randn(cols, generator=gen).cuda()
        ds_ref, ds_new = ds0.clone(), ds0.clone()
        dx_ref = _run(cdl, False, x, dy, res, w, r_inv, ds_ref)
        dx_new = _run(cdl, True, x, dy, res, w, r_inv, ds_new)
        # Same kernels, same launch shape, fixed summation order: bit-identical.
        assert torch.equal(dx_new, dx_ref)
        assert torch.equal(ds_new, ds_ref)


def test_static_scratch_rejects_wide_rows(cdl, gpu_ok):
    L = cdl._lib
    x = torch.zeros(4, 4096, dtype=torch.bfloat16, device="cuda")
    w = torch.ones(4096, dtype=torch.bfloat16, device="cuda")
    r = torch.ones(4, device="cuda")
    ds = torch.zeros(4096, device="cuda")
    args = [L.tensor_arg(t) for t in (x, x, None, w, r, torch.empty_like(x), ds)]
    st = L.lib.cdl_b200_rmsnorm_bwd_static(*(L.ref(a) for a in args), None)
    assert st == -2 and "at most 2048 columns" in L.last_error()

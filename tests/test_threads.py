"""The library from several host threads at once.  The reference's `Executor::execute(&self, ..)`
may be called from any thread, repeatedly, for different streams
(crates/cleandl/src/execgraph/op.rs:130-142; executors are `Send + Sync`), so every entry point must
be re-entrant: results computed concurrently on per-thread streams equal, bit for bit, what one
thread computes alone, and an error message raised in one thread never shows up in another
(the status message is thread-local)."""
import threading

import pytest
import torch

pytestmark = pytest.mark.gpu

THREADS = 4
ROUNDS = 25


def _inputs(seed):
    gen = torch.Generator().manual_seed(seed)
    a = torch.randn(384, 512, generator=gen).to(torch.bfloat16).cuda()
    b = torch.randn(512, 640, generator=gen).to(torch.bfloat16).cuda()
    x = torch.randn(300, 2048, generator=gen).to(torch.bfloat16).cuda()
    w = (1 + 0.1 * torch.randn(2048, generator=gen)).to(torch.bfloat16).cuda()
    q, k, v = (torch.randn(1, 256, 2, 128, generator=gen).to(torch.bfloat16).cuda() for _ in range(3))
    return a, b, x, w, q, k, v


def _compute(cdl, inp):
    a, b, x, w, q, k, v = inp
    d = cdl.ops.matmul(a, b)
    y = cdl.ops.norm_fwd(x, cdl.ops.NormFwdOpts(scale=w, save_stats=True))
    o = cdl.ops.attention_fwd(q, k, v)
    yq, _ = cdl.mx.quantize(x, rowwise=True)
    return d, y.y, y.r_inv, o.out, o.lse, yq.values, yq.scale_factors


def test_concurrent_calls_on_per_thread_streams_are_bit_equal(cdl, gpu_ok):
    inputs = [_inputs(100 + i) for i in range(THREADS)]
    expected = [_compute(cdl, inp) for inp in inputs]
    torch.cuda.synchronize()
    results, errors = [None] * THREADS, []
    start = threading.Barrier(THREADS)

    def worker(i):
        try:
            torch.cuda.set_device(0)
            stream = torch.cuda.Stream()
            start.wait()
            with torch.cuda.stream(stream):
                for _ in range(ROUNDS):
                    out = _compute(cdl, inputs[i])
                stream.synchronize()
            results[i] = out
        except Exception as e:  # reported in the main thread
            errors.append((i, repr(e)))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(THREADS)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for i in range(THREADS):
        for got, exp in zip(results[i], expected[i]):
            assert torch.equal(got, exp), f"thread {i}: a concurrent result differs"


def test_error_messages_stay_in_their_thread(cdl, gpu_ok):
    a, b, x, w, *_ = _inputs(7)
    bad_b = torch.randn(100, 64).to(torch.bfloat16).cuda()  # contraction dimensions differ
    seen, errors = [], []
    start = threading.Barrier(2)

    def failing():
        start.wait()
        for _ in range(200):
            try:
                cdl.ops.norm_fwd(x, cdl.ops.NormFwdOpts(scale=w[:64]))  # a scale of the wrong length
                errors.append("the invalid call was accepted")
            except cdl._lib.CdlError as e:
                seen.append(str(e))

    def working():
        start.wait()
        try:
            torch.cuda.set_device(0)
            with torch.cuda.stream(torch.cuda.Stream()):
                for _ in range(200):
                    cdl.ops.matmul(a, b)
                    cdl.ops.norm_fwd(x, cdl.ops.NormFwdOpts(scale=w))
                torch.cuda.current_stream().synchronize()
        except Exception as e:
            errors.append(repr(e))

    with pytest.raises(cdl._lib.CdlError):
        cdl.ops.matmul(a, bad_b)
    t1, t2 = threading.Thread(target=failing), threading.Thread(target=working)
    t1.start(); t2.start(); t1.join(); t2.join()
    assert not errors, errors
    # every failure carries the norm's own message, never one of the other thread's operators
    assert len(seen) == 200 and len(set(seen)) == 1 and "norm" in seen[0], seen[:2]

"""cleandl_b200: B200 (sm_100a) kernels behind clean-lm's exec-graph operators.

The product is `libcleandl_b200.so` (hand-written CUDA behind the C ABI of
`include/cleandl_b200.h`).  This Python package is the host-side harness: a ctypes binding
(`_lib`), operator front ends that mirror the reference's `Matmul`, `NormFwd`, `AttentionFwd`
and `AttentionBwd` graph nodes (`ops`), the sky-1 block / LM step built from them (`sky1`), checkpoints in the reference's
safetensors layout (`checkpoint`), and block-scaled MXFP8 tensors with the operators that produce
and consume them (`mx`).
PyTorch is used for device memory, streams and torch.distributed only.
"""
from . import _lib  # noqa: F401  (raises if the CUDA library has not been built)
from . import ops  # noqa: F401
from . import sky1  # noqa: F401
from . import checkpoint  # noqa: F401
from . import mx  # noqa: F401
from . import sky1_mx  # noqa: F401

__all__ = ["_lib", "ops", "sky1", "checkpoint", "mx", "sky1_mx"]

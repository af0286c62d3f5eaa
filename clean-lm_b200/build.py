"""Builds libcleandl_b200.so (sm_100a only) from csrc/ with nvcc, in-tree.

Mirrors the role of the reference's kernel-build-util (crates/kernel-build-util/src/lib.rs:81-125):
it emits code for exactly one architecture, and the library refuses other devices at run time.
There is no other backend and no CPU path.  Run as `python clean-lm_b200/build.py` or through
`__graft_entry__.build()`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libcleandl_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the library can only be built with the CUDA toolkit")
    return nvcc


def _stale(out: Path, deps: list[Path]) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(verbose: bool = False, force: bool = False, defines: list[str] | None = None,
          out: Path | None = None) -> Path:
    """Compiles every csrc/*.cu and links the shared library. Returns its path.

    `defines` (e.g. ["CDL_ATTN_POLY_MASK=0x1111u"]) and `out` build a variant with other values of
    the tunable macros into another file (with its own object directory), for side-by-side timing;
    the package loads the variant when CLEANDL_B200_LIB names it."""
    nvcc = _nvcc()
    global OBJ_DIR, LIB_PATH
    flags = list(NVCC_FLAGS)
    if defines or out:
        out = Path(out or PKG_DIR / "libcleandl_b200_variant.so").resolve()
        OBJ_DIR, LIB_PATH = out.parent / (out.stem + "_obj"), out
        flags += [f"-D{d}" for d in (defines or [])]
        force = True
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + [
        PKG_DIR.parent / "include" / "cleandl_b200.h"
    ]

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc, *flags, "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
            if verbose:
                sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(sources) or 1)) as ex:
        objs = list(ex.map(compile_one, sources))
    if force or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    args = sys.argv[1:]
    out = args[args.index("-o") + 1] if "-o" in args else None
    print(build(verbose="-v" in args, force="-f" in args, out=out,
                defines=[a[2:] for a in args if a.startswith("-D")]))

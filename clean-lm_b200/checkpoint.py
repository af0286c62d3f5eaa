"""Checkpoints in the reference's wire format, for interchange with clean-lm.

The reference writes two safetensors files per checkpoint directory
(crates/sky-1/src/training/checkpoint.rs:66-113):

  model.safetensors      f32 master weights, one tensor per parameter
  optimizer.safetensors  f32 `<name>:adam_m` and `<name>:adam_v` per parameter, and the metadata
                         entry `train_step` (a decimal string)

A parameter's name is the `/`-joined path of its owners followed by `.` and its own name
(checkpoint.rs:26, 64-66): `embeddings.weight`, `decoder_blocks[3]/qkv_proj.weight`,
`decoder_blocks[3]/ffn.up`, `final_norm.gamma`, `lm_head.weight` (crates/sky-1/src/training/model/
mod.rs:75-103, decoder.rs:224-253).  Shapes are the parameters' own: weights `[in, out]`.

The container is plain safetensors: an 8-byte little-endian header length, a JSON header mapping
each tensor name to `{"dtype", "shape", "data_offsets"}` (plus `__metadata__`), padded with spaces
to a multiple of 8 bytes, then the tensor bytes back to back.  It is written and parsed here
directly (the `safetensors` package is not a dependency of this library).
"""
from __future__ import annotations

import json
import os
import struct
from pathlib import Path
from typing import Dict, Iterable, Optional, Tuple

import numpy as np

_DTYPES = {"F32": np.dtype("<f4"), "F64": np.dtype("<f8"), "I32": np.dtype("<i4"), "I64": np.dtype("<i8"),
           "U8": np.dtype("u1")}
_NAMES = {v: k for k, v in _DTYPES.items()}

# this library's per-block parameter names -> the reference's `<owner>.<name>`
BLOCK_NAMES = {"norm1": "pre_qkv_norm.gamma", "wqkv": "qkv_proj.weight", "wo": "o_proj.weight",
               "norm2": "pre_ffn_norm.gamma", "wup": "ffn.up", "wgate": "ffn.gate", "wdown": "ffn.down"}


def reference_name(name: str) -> str:
    """Maps a `Sky1LM` parameter name (`embedding`, `blocks.<i>.<param>`, `final_norm`, `lm_head`)
    to the name the reference's CheckpointBuilder gives the same parameter."""
    if name == "embedding":
        return "embeddings.weight"
    if name == "final_norm":
        return "final_norm.gamma"
    if name == "lm_head":
        return "lm_head.weight"
    parts = name.split(".")
    if len(parts) == 3 and parts[0] == "blocks" and parts[2] in BLOCK_NAMES:
        return f"decoder_blocks[{int(parts[1])}]/{BLOCK_NAMES[parts[2]]}"
    raise KeyError(f"no reference name for parameter '{name}'")


def write_safetensors(path, tensors: Iterable[Tuple[str, np.ndarray]],
                      metadata: Optional[Dict[str, str]] = None) -> None:
    """Writes `tensors` (name, array) in the order given; arrays are stored little-endian, C order."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs, offset = [], 0
    for name, arr in tensors:
        arr = np.ascontiguousarray(arr)
        dt = arr.dtype.newbyteorder("<") if arr.dtype.byteorder == ">" else arr.dtype
        if np.dtype(dt) not in _NAMES:
            raise TypeError(f"tensor '{name}': dtype {arr.dtype} cannot be stored")
        if name in header:
            raise ValueError(f"duplicate tensor name '{name}'")
        blob = arr.astype(dt, copy=False).tobytes()
        header[name] = {"dtype": _NAMES[np.dtype(dt)], "shape": list(arr.shape),
                        "data_offsets": [offset, offset + len(blob)]}
        blobs.append(blob)
        offset += len(blob)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * (-len(text) % 8)
    tmp = Path(str(path) + ".tmp")
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for blob in blobs:
            f.write(blob)
    os.replace(tmp, path)


def read_safetensors(path) -> Tuple[Dict[str, np.ndarray], Dict[str, str]]:
    """Returns ({name: array}, metadata).  Arrays are copies, so the file can be closed."""
    with open(path, "rb") as f:
        raw = f.read()
    if len(raw) < 8:
        raise ValueError(f"{path}: too short for a safetensors file")
    (n,) = struct.unpack("<Q", raw[:8])
    if n > len(raw) - 8:
        raise ValueError(f"{path}: header length {n} exceeds the file")
    header = json.loads(raw[8:8 + n].decode("utf-8"))
    data = memoryview(raw)[8 + n:]
    meta = header.pop("__metadata__", None) or {}
    out = {}
    for name, info in header.items():
        dt = _DTYPES.get(info["dtype"])
        if dt is None:
            raise TypeError(f"{path}: tensor '{name}' has unsupported dtype {info['dtype']}")
        lo, hi = info["data_offsets"]
        shape = tuple(info["shape"])
        if hi - lo != int(np.prod(shape, dtype=np.int64)) * dt.itemsize or hi > len(data):
            raise ValueError(f"{path}: tensor '{name}' has inconsistent offsets")
        out[name] = np.frombuffer(data[lo:hi], dtype=dt).reshape(shape).copy()
    return out, dict(meta)


def save_checkpoint(lm, directory, train_step: Optional[int] = None) -> None:
    """Writes `model.safetensors` and `optimizer.safetensors` for a `Sky1LM` into `directory`."""
    directory = Path(directory)
    directory.mkdir(parents=True, exist_ok=True)
    step = lm.step_count if train_step is None else int(train_step)
    names = [name for name, _, _ in lm.layout]

    def host(which, name):
        return lm.view(which, name).detach().float().cpu().numpy()

    write_safetensors(directory / "model.safetensors",
                      ((reference_name(n), host("master", n)) for n in names))
    opt = []
    for n in names:
        opt.append((reference_name(n) + ":adam_m", host("m", n)))
        opt.append((reference_name(n) + ":adam_v", host("v", n)))
    write_safetensors(directory / "optimizer.safetensors", opt, {"train_step": str(step)})


def load_checkpoint(lm, directory) -> int:
    """Loads a checkpoint directory written by `save_checkpoint` or by the reference into a
    `Sky1LM` of the same configuration: master weights, bf16 replicas, Adam moments, step count.
    Returns the train step."""
    import torch

    directory = Path(directory)
    model, _ = read_safetensors(directory / "model.safetensors")
    optim, meta = read_safetensors(directory / "optimizer.safetensors")
    if "train_step" not in meta:
        raise ValueError("optimizer checkpoint is missing train_step metadata")
    step = int(meta["train_step"])
    for name, shape, _ in lm.layout:
        ref = reference_name(name)
        for which, table, key in (("master", model, ref), ("m", optim, ref + ":adam_m"),
                                  ("v", optim, ref + ":adam_v")):
            if key not in table:
                raise KeyError(f"checkpoint has no tensor '{key}'")
            arr = table[key]
            if tuple(arr.shape) != tuple(shape):
                raise ValueError(f"tensor '{key}' has shape {tuple(arr.shape)}, expected {tuple(shape)}")
            lm.view(which, name).copy_(torch.from_numpy(arr.astype(np.float32, copy=False)))
    lm.replica.copy_(lm.master)
    lm.step_count = step
    return step

"""Checkpoint reading (reference: src/compute/models/loader.py:27-76).

``SafetensorsSource`` indexes every ``*.safetensors`` file of a model directory from the
JSON headers alone and serves sub-block reads through the C++ mmap reader in
``csrc/host/hostops.cpp`` (rows and byte-columns a rank owns; nothing else is touched).
Without the native library it uses the ``safetensors`` wheel's lazy slices, which read the
same sub-blocks. Blocks are staged through pinned host memory when the destination is a GPU.
"""

from __future__ import annotations

import ctypes
import glob
import json
import os
import struct

import numpy as np
import torch

from ..ops import hostlib

__all__ = ["SafetensorsSource", "load_model", "write_safetensors"]

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "BOOL": (torch.bool, 1),
}
_DTYPE_NAMES = {v[0]: k for k, v in _DTYPES.items()}


def _read_header(path: str) -> tuple[dict, int]:
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) < 8:
            raise ValueError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", raw)
        size = os.path.getsize(path)
        if n > size - 8:
            raise ValueError(f"{path}: header length {n} exceeds file size {size}")
        try:
            header = json.loads(f.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise ValueError(f"{path}: corrupt safetensors header: {e}") from None
    return header, n


class SafetensorsSource:
    def __init__(self, model_dir: str, pin: bool = False) -> None:
        files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
        if not files:
            raise FileNotFoundError(f"no *.safetensors under {model_dir}")
        self._lib = hostlib.get()
        self._entries: dict[str, tuple[int, str, tuple[int, ...], int, int]] = {}
        self._files = files
        self._handles: list = [None] * len(files)
        self._lazy = [None] * len(files)
        self._pin = pin
        for fi, path in enumerate(files):
            header, _ = _read_header(path)
            for name, meta in header.items():
                if name == "__metadata__":
                    continue
                if meta["dtype"] not in _DTYPES:
                    raise ValueError(f"{path}: tensor {name} has unsupported dtype {meta['dtype']}")
                b, e = meta["data_offsets"]
                self._entries[name] = (fi, meta["dtype"], tuple(meta["shape"]), int(b), int(e))

    def names(self) -> list[str]:
        return list(self._entries)

    def has(self, name: str) -> bool:
        return name in self._entries

    def shape(self, name: str) -> tuple[int, ...]:
        return self._entries[name][2]

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self._entries[name][1]][0]

    def _handle(self, fi: int):
        if self._handles[fi] is None:
            h = self._lib.xv_st_open(self._files[fi].encode())
            if not h:
                raise OSError(f"cannot map {self._files[fi]}")
            self._handles[fi] = h
        return self._handles[fi]

    def read(self, name: str, row0: int = 0, nrows: int | None = None, col0: int = 0,
             ncols: int | None = None) -> torch.Tensor:
        fi, dt, shape, begin, end = self._entries[name]
        tdtype, esz = _DTYPES[dt]
        if len(shape) == 0:
            shape2 = (1, 1)
        elif len(shape) == 1:
            shape2 = (shape[0], 1)
        else:
            shape2 = (shape[0], int(np.prod(shape[1:])))
        nrows = shape2[0] - row0 if nrows is None else nrows
        ncols = shape2[1] - col0 if ncols is None else ncols
        if row0 < 0 or col0 < 0 or row0 + nrows > shape2[0] or col0 + ncols > shape2[1]:
            raise IndexError(f"{name}: block [{row0}:{row0+nrows}, {col0}:{col0+ncols}] outside {shape}")
        out_shape = (nrows,) if len(shape) <= 1 else (nrows, ncols)
        if self._lib is not None:
            out = torch.empty(out_shape, dtype=tdtype, pin_memory=self._pin and torch.cuda.is_available())
            rc = self._lib.xv_st_read_block(self._handle(fi), begin, shape2[1] * esz, row0, nrows,
                                            col0 * esz, ncols * esz, ctypes.c_void_p(out.data_ptr()))
            if rc != 0:
                raise ValueError(f"{self._files[fi]}: tensor {name} lies outside the file (truncated?)")
            return out
        from safetensors import safe_open

        if self._lazy[fi] is None:
            self._lazy[fi] = safe_open(self._files[fi], framework="pt")
        sl = self._lazy[fi].get_slice(name)
        if len(shape) <= 1:
            return sl[row0:row0 + nrows]
        t = sl[row0:row0 + nrows]
        return t.reshape(nrows, shape2[1])[:, col0:col0 + ncols].contiguous()

    def close(self) -> None:
        if self._lib is not None:
            for i, h in enumerate(self._handles):
                if h:
                    self._lib.xv_st_close(h)
                    self._handles[i] = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass


def load_model(model, model_dir: str) -> dict:
    """Fill ``model`` from the safetensors files of ``model_dir``."""
    src = SafetensorsSource(model_dir, pin=model.device.type == "cuda")
    try:
        return model.load_weights(src)
    finally:
        src.close()


def write_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Minimal writer (header + raw little-endian data), enough for synthetic checkpoints."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _DTYPE_NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * (-len(blob) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")

"""Chained 64-bit page hashes: ``h_i = XXH64(le64(h_{i-1}) | int32 tokens of page i)``, with
the parent omitted for the first page (reference: src/data/prefix/hash_util.py:16-30).

A request's whole chain is computed in one call into the C++ host library when it is
built (``csrc/host/hostops.cpp``); at 16-token pages a 2048-token prompt has 128 links, so
the per-link Python overhead of a hashing wheel matters. The pure-Python path produces the
same digests through the ``xxhash`` wheel, or blake2b if that is missing too.
"""

from __future__ import annotations

import ctypes
import struct

import numpy as np

from ...ops import hostlib

__all__ = ["compute_block_hash", "chain_hashes", "NO_PARENT"]

NO_PARENT = -1

try:  # optional wheel
    import xxhash as _xxhash
except ImportError:  # pragma: no cover
    _xxhash = None


def _digest_py(token_ids, parent: int) -> int:
    payload = np.asarray(token_ids, dtype=np.int32).tobytes()
    if parent != NO_PARENT:
        payload = struct.pack("<Q", parent) + payload
    if _xxhash is not None:
        return _xxhash.xxh64_intdigest(payload)
    import hashlib

    return int.from_bytes(hashlib.blake2b(payload, digest_size=8).digest(), "little")


def compute_block_hash(token_ids, prefix: int = NO_PARENT) -> int:
    """Hash of one page given its parent's hash (``-1`` for the first page)."""
    return chain_hashes(token_ids, len(token_ids), 1, prefix)[0]


def chain_hashes(token_ids, block_size: int, num_blocks: int, parent: int = NO_PARENT,
                 start_block: int = 0) -> list[int]:
    """Hashes of pages ``start_block .. start_block+num_blocks-1`` of ``token_ids``.

    ``parent`` is the hash of page ``start_block-1`` (``-1`` if ``start_block`` is 0).
    """
    if num_blocks <= 0:
        return []
    lo = start_block * block_size
    lib = hostlib.get()
    if lib is not None and (_xxhash is not None or lib is not None):
        toks = np.ascontiguousarray(token_ids[lo: lo + num_blocks * block_size], dtype=np.int32)
        if toks.size != num_blocks * block_size:
            raise ValueError("token_ids too short for the requested pages")
        out = np.empty(num_blocks, dtype=np.uint64)
        lib.xv_hash_chain(
            toks.ctypes.data_as(ctypes.c_void_p), num_blocks, block_size,
            ctypes.c_uint64(parent & 0xFFFFFFFFFFFFFFFF), int(parent != NO_PARENT),
            out.ctypes.data_as(ctypes.c_void_p),
        )
        return out.tolist()
    out_py: list[int] = []
    h = parent
    for i in range(num_blocks):
        h = _digest_py(token_ids[lo + i * block_size: lo + (i + 1) * block_size], h)
        out_py.append(h)
    return out_py

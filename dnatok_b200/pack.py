"""Host packing: DNA strings -> one contiguous ASCII buffer + int64 row offsets.

Counterpart of the reference's per-call packing (``"".join(seqs).encode("ascii")`` at
``src/dna_tokenizer.py:1795-1800``; pinned bytes + offsets at
``src/dnatok_bpe_kernel/dnatok_bpe.cu:872-887``).  Like the reference, input must be ASCII.
"""
from __future__ import annotations

from typing import Sequence, Tuple, Union

import numpy as np

Packed = Tuple[np.ndarray, np.ndarray]     # (uint8[total], int64[B+1])


def pack_strings(seqs: Sequence[Union[str, bytes]]) -> Packed:
    n = len(seqs)
    offsets = np.zeros(n + 1, dtype=np.int64)
    if n == 0:
        return np.zeros(0, dtype=np.uint8), offsets
    if isinstance(seqs[0], (bytes, bytearray)):
        lens = np.fromiter((len(s) for s in seqs), dtype=np.int64, count=n)
        buf = b"".join(seqs)
    else:
        lens = np.fromiter((len(s) for s in seqs), dtype=np.int64, count=n)
        try:
            buf = "".join(seqs).encode("ascii")
        except UnicodeEncodeError as e:
            raise ValueError("sequences must be ASCII: %s" % e) from None
    np.cumsum(lens, out=offsets[1:])
    flat = np.frombuffer(buf, dtype=np.uint8)
    if flat.shape[0] != offsets[-1]:
        raise ValueError("packed length mismatch")
    return flat, offsets


def pack_any(x) -> Packed:
    """Accept list[str] / list[bytes], a 2-D uint8 array of equal-length rows, or a
    ready (flat uint8, int64 offsets) pair."""
    if isinstance(x, tuple) and len(x) == 2:
        flat = np.ascontiguousarray(x[0], dtype=np.uint8).reshape(-1)
        offsets = np.ascontiguousarray(x[1], dtype=np.int64)
        if offsets.ndim != 1 or offsets.shape[0] < 1 or offsets[0] != 0 or offsets[-1] != flat.shape[0] \
                or np.any(np.diff(offsets) < 0):
            raise ValueError("offsets must start at 0, be non-decreasing and end at len(bytes)")
        return flat, offsets
    if isinstance(x, np.ndarray):
        if x.dtype != np.uint8 or x.ndim != 2:
            raise ValueError("array input must be uint8[B, L]")
        b, n = x.shape
        return np.ascontiguousarray(x).reshape(-1), np.arange(b + 1, dtype=np.int64) * n
    return pack_strings(x)


def pack_fasta(text: Union[bytes, bytearray, memoryview]) -> Packed:
    """FASTA text -> (flat uint8 bytes, int64 offsets), one row per record, through the native packer."""
    import ctypes
    from . import _cabi
    L = _cabi.lib()
    buf = np.frombuffer(bytes(text), dtype=np.uint8)
    n_rec, n_bytes = ctypes.c_int64(0), ctypes.c_int64(0)
    ptr = _cabi.np_ptr(buf) if buf.size else None
    _cabi.check(L.dnatok_pack_fasta(ptr, buf.size, None, 0, None, 0, ctypes.byref(n_rec), ctypes.byref(n_bytes)))
    flat = np.empty(n_bytes.value, dtype=np.uint8)
    offsets = np.zeros(n_rec.value + 1, dtype=np.int64)
    _cabi.check(L.dnatok_pack_fasta(ptr, buf.size, _cabi.np_ptr(flat), flat.size, _cabi.np_ptr(offsets), offsets.size,
                                    ctypes.byref(n_rec), ctypes.byref(n_bytes)))
    return flat, offsets

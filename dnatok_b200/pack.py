"""Host packing: DNA strings -> one contiguous ASCII buffer + int64 row offsets.

Counterpart of the reference's per-call packing (``"".join(seqs).encode("ascii")`` at
``src/dna_tokenizer.py:1795-1800``; pinned bytes + offsets at
``src/dnatok_bpe_kernel/dnatok_bpe.cu:872-887``).  Like the reference, input must be ASCII.
"""
from __future__ import annotations

from typing import Sequence, Tuple, Union

import numpy as np

Packed = Tuple[np.ndarray, np.ndarray]     # (uint8[total], int64[B+1])


def _native():
    try:
        from . import _pack
    except ImportError as e:
        raise RuntimeError("the host packer dnatok_b200/_pack.so is not built; run `python -m dnatok_b200.build` (%s)" % e)
    return _pack


def pack_sizes(seqs, pad_to: int = 0, trunc_to: int = 0) -> int:
    """Bytes the rows of a list take once packed (every row at least ``pad_to`` bytes, at most ``trunc_to``)."""
    if not isinstance(seqs, (list, tuple)):
        seqs = list(seqs)
    if not seqs:
        return 0
    return int(_native().sizes(seqs, np.zeros(len(seqs) + 1, dtype=np.int64), int(pad_to), int(trunc_to)))


def pack_strings(seqs: Sequence[Union[str, bytes]], *, table: bytes = None, pad_to: int = 0, pad_byte: int = ord("N"),
                 pad_left: bool = False, trunc_to: int = 0, out: np.ndarray = None) -> Packed:
    """Rows of a list into one buffer through the native packer (one pass over the list, threaded copy, no
    intermediate string).  ``table`` translates every byte on the way (256 entries); ``pad_to`` pads every
    shorter row to that many bytes with ``pad_byte`` on the chosen side; ``trunc_to`` keeps only the first
    so many bytes of a row; ``out`` is a uint8 buffer to fill
    (for instance pinned memory), which must be large enough."""
    if not isinstance(seqs, (list, tuple)):
        seqs = list(seqs)
    n = len(seqs)
    offsets = np.zeros(n + 1, dtype=np.int64)
    if n == 0:
        return np.zeros(0, dtype=np.uint8), offsets
    P = _native()
    total = P.sizes(seqs, offsets, int(pad_to), int(trunc_to))
    if out is None:
        out = np.empty(max(total, 1), dtype=np.uint8)
    elif out.size < total:
        raise ValueError("output buffer holds %d bytes, %d needed" % (out.size, total))
    P.copy(seqs, offsets, out, table, int(pad_to), int(pad_byte), 1 if pad_left else 0, 0, int(trunc_to))
    return out[:total], offsets


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

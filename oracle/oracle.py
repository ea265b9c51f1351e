"""TEST INFRASTRUCTURE ONLY - ctypes front end of the CPU checker plus HF-style batch assembly.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py`` import
this module.  ``libdnatok_oracle.so`` is built from ``dnatok_oracle.c`` by ``oracle/Makefile``.

``assemble`` restates what Hugging Face does around the model for one sequence per row
(`tokenizers` truncation, ``TemplateProcessing("[CLS] $A [SEP]")`` and padding): truncation
keeps the first ``max_length - n_special`` content tokens, then the specials are attached,
then rows are padded to the longest row or to ``max_length`` with ``pad_id`` and mask 0.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build() -> str:
    path = os.path.join(_HERE, "libdnatok_oracle.so")
    src = os.path.join(_HERE, "dnatok_oracle.c")
    if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libdnatok_oracle.so"])
    return path


def lib():
    global _LIB
    if _LIB is None:
        L = ctypes.CDLL(build())
        p = ctypes.c_void_p
        L.oracle_bpe_table_new.restype = p
        L.oracle_bpe_table_new.argtypes = [p, p, p, ctypes.c_int32]
        L.oracle_bpe_table_free.argtypes = [p]
        L.oracle_encode_batch.argtypes = [ctypes.c_int, p, p, ctypes.c_int64, p, ctypes.c_int, p, p, p, p,
                                          ctypes.c_int]
        for f in (L.oracle_bpe_word, L.oracle_bpe_word_naive):
            f.restype = ctypes.c_int64
            f.argtypes = [p, p, ctypes.c_int64, p, p]
        _LIB = L
    return _LIB


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p) if a is not None else None


class BpeTable:
    def __init__(self, merge_a, merge_b, merge_out):
        self.a = np.ascontiguousarray(merge_a, dtype=np.int32)
        self.b = np.ascontiguousarray(merge_b, dtype=np.int32)
        self.o = np.ascontiguousarray(merge_out, dtype=np.int32)
        self.h = lib().oracle_bpe_table_new(_ptr(self.a), _ptr(self.b), _ptr(self.o), len(self.a))

    def __del__(self):
        if getattr(self, "h", None):
            lib().oracle_bpe_table_free(self.h)
            self.h = None


def encode_ragged(kind: str, flat: np.ndarray, offsets: np.ndarray, *, lut256: np.ndarray,
                  k: int = 0, kmer_ids: np.ndarray | None = None, table: BpeTable | None = None,
                  threads: int = 1):
    """Content tokens of every row: returns (ids int32[sum len] laid out at the input offsets,
    counts int64[B])."""
    flat = np.ascontiguousarray(flat, dtype=np.uint8)
    offsets = np.ascontiguousarray(offsets, dtype=np.int64)
    lut256 = np.ascontiguousarray(lut256, dtype=np.int32)
    B = len(offsets) - 1
    out = np.empty(max(1, int(offsets[-1])), dtype=np.int32)
    counts = np.zeros(B, dtype=np.int64)
    kid = {"char": 0, "kmer": 1, "bpe": 2}[kind]
    km = np.ascontiguousarray(kmer_ids, dtype=np.int32) if kmer_ids is not None else None
    lib().oracle_encode_batch(kid, _ptr(flat), _ptr(offsets), B, _ptr(lut256), int(k), _ptr(km),
                              table.h if table is not None else None, _ptr(out), _ptr(counts),
                              int(threads))
    return out, counts


def bpe_word(table: BpeTable, s: bytes, byte_ids: np.ndarray, naive: bool = False) -> list[int]:
    buf = np.frombuffer(s, dtype=np.uint8)
    out = np.empty(max(1, len(buf)), dtype=np.int32)
    ids = np.ascontiguousarray(byte_ids, dtype=np.int32)
    f = lib().oracle_bpe_word_naive if naive else lib().oracle_bpe_word
    n = f(table.h, _ptr(buf), len(buf), _ptr(ids), _ptr(out))
    return out[:n].tolist()


def rows(ids: np.ndarray, offsets: np.ndarray, counts: np.ndarray) -> list[np.ndarray]:
    return [ids[offsets[i]:offsets[i] + counts[i]] for i in range(len(counts))]


def assemble(content_rows, *, pad_id: int, cls_id: int = -1, sep_id: int = -1,
             add_special: bool = True, max_length: int = 0, truncation: bool = False,
             padding="longest", pad_left: bool = False, id_dtype=np.int64, mask_dtype=np.int64):
    """HF batch assembly.  ``padding``: False -> list of arrays, 'longest' or 'max_length'."""
    pre = [cls_id] if (add_special and cls_id >= 0) else []
    post = [sep_id] if (add_special and sep_id >= 0) else []
    ns = len(pre) + len(post)
    out = []
    for r in content_rows:
        r = np.asarray(r)
        if truncation and max_length:
            r = r[:max(0, max_length - ns)]
        out.append(np.concatenate([np.array(pre, dtype=np.int64), r.astype(np.int64),
                                   np.array(post, dtype=np.int64)]))
    if not padding:
        return out
    width = max_length if padding == "max_length" else max((len(r) for r in out), default=0)
    ids = np.full((len(out), width), pad_id, dtype=id_dtype)
    mask = np.zeros((len(out), width), dtype=mask_dtype)
    for i, r in enumerate(out):
        if len(r) > width:
            raise ValueError("row %d has %d tokens > width %d (truncation off)" % (i, len(r), width))
        if pad_left:
            ids[i, width - len(r):] = r
            mask[i, width - len(r):] = 1
        else:
            ids[i, :len(r)] = r
            mask[i, :len(r)] = 1
    return ids, mask

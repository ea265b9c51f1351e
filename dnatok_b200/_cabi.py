"""ctypes binding of ``libdnatok_b200.so`` (declared in ``include/dnatok_b200.h``).

The library is built in-tree by ``dnatok_b200/build.py`` (nvcc, sm_100a).  There is no CPU
fallback: a missing library raises ``RuntimeError`` at load time.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_int, c_int32, c_int64, c_size_t, c_void_p

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "csrc", "libdnatok_b200.so")

OK = 0
ROW_TOO_LONG, ROW_NOT_CONVERGED, ROW_CLIPPED, ROW_OUTSIDE_HINT, ROW_STALLED = 1, 2, 4, 8, 16
KIND_CHAR, KIND_KMER, KIND_BPE = 0, 1, 2
BPE_MAX_WORD = 1 << 30

EXPORTS = (
    "dnatok_version", "dnatok_last_error", "dnatok_create_char", "dnatok_create_kmer",
    "dnatok_create_bpe", "dnatok_destroy", "dnatok_kind", "dnatok_scratch_bytes",
    "dnatok_max_tokens", "dnatok_prepare", "dnatok_write", "dnatok_encode",
    "dnatok_scan_lengths", "dnatok_encode_host", "dnatok_launch_count", "dnatok_host_copy_bytes",
    "dnatok_encode_bpe_builtin_scratch", "dnatok_set_option", "dnatok_set_row_bytes_hint",
    "dnatok_pack_fasta", "dnatok_embed", "dnatok_create_kmer_table", "dnatok_set_start_lut",
)
BUILTIN_SCRATCH_BYTES = 8 << 20


class Specials(Structure):
    _fields_ = [("pad_id", c_int32), ("unk_id", c_int32), ("cls_id", c_int32), ("sep_id", c_int32)]


class Format(Structure):
    _fields_ = [("id_bits", c_int32), ("mask_bits", c_int32), ("add_special", c_int32),
                ("pad_left", c_int32), ("max_tokens", c_int64), ("out_stride", c_int64)]


class DnatokError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__("dnatok_b200 error %d: %s" % (code, msg))
        self.code = code


_LIB = None


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "libdnatok_b200.so is not built (%s); run `python -m dnatok_b200.build`. "
            "There is no CPU fallback." % LIB_PATH)
    L = ctypes.CDLL(LIB_PATH)
    p = c_void_p
    L.dnatok_version.restype = c_int
    L.dnatok_last_error.restype = c_char_p
    L.dnatok_launch_count.restype = c_int64
    L.dnatok_host_copy_bytes.restype = None
    L.dnatok_host_copy_bytes.argtypes = [ctypes.POINTER(c_int64), ctypes.POINTER(c_int64)]
    L.dnatok_create_char.argtypes = [p, POINTER(Specials), POINTER(p)]
    L.dnatok_create_kmer.argtypes = [c_int, p, p, POINTER(Specials), POINTER(p)]
    L.dnatok_create_bpe.argtypes = [p, p, p, c_int32, p, POINTER(Specials), POINTER(p)]
    L.dnatok_create_kmer_table.argtypes = [c_int, p, p, c_int32, p, p, c_int, POINTER(Specials), POINTER(p)]
    L.dnatok_set_start_lut.argtypes = [p, p]
    L.dnatok_destroy.argtypes = [p]
    L.dnatok_destroy.restype = None
    L.dnatok_kind.argtypes = [p]
    L.dnatok_scratch_bytes.argtypes = [p, c_int64, c_int64]
    L.dnatok_scratch_bytes.restype = c_size_t
    L.dnatok_max_tokens.argtypes = [p, c_int64, c_int64, POINTER(Format)]
    L.dnatok_max_tokens.restype = c_int64
    L.dnatok_prepare.argtypes = [p, p, p, c_int64, c_int64, POINTER(Format), p, p, p, c_size_t, p]
    L.dnatok_write.argtypes = [p, p, p, c_int64, c_int64, POINTER(Format), p, p, p, p, p, p, c_size_t, p]
    L.dnatok_encode.argtypes = [p, p, p, c_int64, c_int64, POINTER(Format), p, p, p, p, p, p, c_size_t, p]
    L.dnatok_encode_bpe_builtin_scratch.argtypes = [p, p, p, c_int64, c_int64, POINTER(Format), p, p, p, p, p, p]
    L.dnatok_pack_fasta.argtypes = [p, c_int64, p, c_int64, p, c_int64, POINTER(c_int64), POINTER(c_int64)]
    L.dnatok_embed.argtypes = [p, p, p, c_int64, c_int64, POINTER(Format), p, c_int64, c_int64, p, p, p, p]
    L.dnatok_set_option.argtypes = [c_char_p, c_int64]
    L.dnatok_set_row_bytes_hint.argtypes = [p, c_int64, c_int64]
    L.dnatok_scan_lengths.argtypes = [p, c_int64, p, p]
    L.dnatok_encode_host.argtypes = [p, c_int, p, p, c_int64, POINTER(Format), p, c_int64, p, p, p, p,
                                     POINTER(c_int64)]
    if L.dnatok_version() != 1:
        raise RuntimeError("libdnatok_b200.so has ABI version %d, expected 1" % L.dnatok_version())
    _LIB = L
    return L


def check(rc: int) -> None:
    if rc != OK:
        raise DnatokError(rc, (lib().dnatok_last_error() or b"").decode())


def np_ptr(a) -> c_void_p:
    return a.ctypes.data_as(c_void_p)


class Handle:
    """Owns one ``dnatok_handle*``."""

    def __init__(self, spec):
        import numpy as np
        L = lib()
        sp = Specials(spec.specials.pad_id, spec.specials.unk_id, spec.specials.cls_id, spec.specials.sep_id)
        h = c_void_p()
        lut = np.ascontiguousarray(spec.lut256, dtype=np.int32)
        if spec.kind == "char":
            check(L.dnatok_create_char(np_ptr(lut), ctypes.byref(sp), ctypes.byref(h)))
            if getattr(spec, "start_lut256", None) is not None:
                start = np.ascontiguousarray(spec.start_lut256, dtype=np.int32)
                check(L.dnatok_set_start_lut(h, np_ptr(start)))
        elif spec.kind == "kmer" and getattr(spec, "kmer_table5", None) is not None:
            t5 = np.ascontiguousarray(spec.kmer_table5, dtype=np.int32)
            if t5.shape[0] != 5 ** spec.k:
                raise ValueError("kmer_table5 must have 5**k entries")
            ro = np.ascontiguousarray(spec.kmer_run_offsets, dtype=np.int32)
            ri = np.ascontiguousarray(spec.kmer_run_ids, dtype=np.int32)
            check(L.dnatok_create_kmer_table(int(spec.k), np_ptr(t5), np_ptr(ro), int(len(ro) - 1), np_ptr(ri) if len(ri) else None,
                                             np_ptr(lut), 1 if spec.kmer_tail_singles else 0, ctypes.byref(sp), ctypes.byref(h)))
        elif spec.kind == "kmer":
            km = np.ascontiguousarray(spec.kmer_ids, dtype=np.int32)
            if km.shape[0] != 4 ** spec.k:
                raise ValueError("kmer_ids must have 4**k entries")
            check(L.dnatok_create_kmer(int(spec.k), np_ptr(km), np_ptr(lut), ctypes.byref(sp), ctypes.byref(h)))
        elif spec.kind == "bpe":
            a = np.ascontiguousarray(spec.merge_a, dtype=np.int32)
            b = np.ascontiguousarray(spec.merge_b, dtype=np.int32)
            o = np.ascontiguousarray(spec.merge_out, dtype=np.int32)
            check(L.dnatok_create_bpe(np_ptr(a), np_ptr(b), np_ptr(o), len(a), np_ptr(lut), ctypes.byref(sp),
                                      ctypes.byref(h)))
        else:
            raise ValueError("unknown kind %r" % (spec.kind,))
        self.ptr = h
        self.kind = spec.kind

    def close(self) -> None:
        if getattr(self, "ptr", None):
            lib().dnatok_destroy(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

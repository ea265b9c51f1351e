"""The shared library loads, exports every symbol include/dnatok_b200.h declares, and its host-only
entry points (handle creation, table validation, sizing) behave.  No kernel is launched here."""
import ctypes
import os
import re

import numpy as np
import pytest

from dnatok_b200 import _cabi
from dnatok_b200.tables import Specials, TokenizerSpec

import helpers as H

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "dnatok_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(dnatok_[a-z_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = _cabi.lib()
    names = declared_symbols()
    assert len(names) >= 14
    for n in names:
        assert hasattr(L, n), n
    assert sorted(_cabi.EXPORTS) == names
    assert L.dnatok_version() == 1


def test_every_documented_option_is_accepted():
    """The tuning knobs listed in the header are the ones dnatok_set_option knows (set to their defaults here), and
    an unknown name is an error."""
    text = open(os.path.join(ROOT, "include", "dnatok_b200.h")).read()
    block = text[text.index("Process-wide tuning knobs"):text.index("int dnatok_set_option")]
    names = re.findall(r'^ \*   "([a-z_]+)"', block, flags=re.M)
    defaults = {"host_chunk_bytes": 64 << 20, "host_chunk_threshold": 128 << 20, "host_mask_threads": -1, "host_mask_early": 1,
                "host_mask_min_bytes": 16 << 20, "kmer_force_segments": 0, "kmer_poll_limit": 1 << 20,
                "kmer_test_withhold_ticket": -1, "kmer_overlap_launch": 1, "emit_overlap_launch": 1, "bpe_team_warps": 0,
                "bpe_team_max": 8, "bpe_overlap_launch": 1, "bpe_smem_table": 1, "bpe_fused_output": 1, "bpe_mixed_launch": 1,
                "bpe_block_team_rows": -1}
    assert sorted(names) == sorted(defaults)
    L = _cabi.lib()
    for n in names:
        assert L.dnatok_set_option(n.encode(), defaults[n]) == 0, n
    assert L.dnatok_set_option(b"no_such_knob", 1) != 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_cabi, "_LIB", None)
    monkeypatch.setattr(_cabi, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _cabi.lib()


@pytest.mark.parametrize("name", H.TOKENIZERS)
def test_handles_for_all_five_tokenizers(name):
    h = _cabi.Handle(H.spec(name))
    L = _cabi.lib()
    kind = {"char": 0, "kmer": 1, "bpe": 2}[H.spec(name).kind]
    assert L.dnatok_kind(h.ptr) == kind
    sb = L.dnatok_scratch_bytes(h.ptr, 1000, 1 << 20)
    if kind == 2:
        assert sb > 2 * (1 << 20)
    elif kind == 1:
        # one flag per segment of 256 windows and row (1,048 bp rows of 6-mers: one segment each)
        assert sb == 256 + 4 * 1000
        assert L.dnatok_scratch_bytes(h.ptr, 10, 1 << 20) == 256 + 4 * 10 * 69
    else:
        assert sb == 0
    fmt = _cabi.Format(64, 64, 1, 0, 0, 0)
    ns = (H.spec(name).specials.cls_id >= 0) + (H.spec(name).specials.sep_id >= 0)
    assert L.dnatok_max_tokens(h.ptr, 10, 500, ctypes.byref(fmt)) == 500 + 10 * ns
    h.close()
    h.close()


def _bpe_spec(a, b, o, lut=None):
    if lut is None:
        lut = np.full(256, 1, np.int32)
        for i, c in enumerate("ACGT"):
            lut[ord(c)] = 5 + i
    return TokenizerSpec("bpe", Specials(0, 1, 2, 3), 64, lut, merge_a=np.array(a, np.int32),
                         merge_b=np.array(b, np.int32), merge_out=np.array(o, np.int32))


def test_bpe_table_validation_errors():
    _cabi.Handle(_bpe_spec([5, 9], [6, 7], [9, 10])).close()
    with pytest.raises(_cabi.DnatokError, match="same token"):
        _cabi.Handle(_bpe_spec([5, 6], [6, 7], [9, 9]))
    with pytest.raises(_cabi.DnatokError, match="same token"):
        _cabi.Handle(_bpe_spec([5], [6], [7]))            # creates an initial symbol
    with pytest.raises(_cabi.DnatokError, match="twice"):
        _cabi.Handle(_bpe_spec([5, 5], [6, 6], [9, 10]))
    with pytest.raises(_cabi.DnatokError, match="16 bits"):
        _cabi.Handle(_bpe_spec([5], [6], [70000]))
    with pytest.raises(_cabi.DnatokError):
        _cabi.Handle(_bpe_spec([], [], []))
    # operands created by a later rank: accepted (the kernel then merges one pair per pass)
    _cabi.Handle(_bpe_spec([9, 5], [7, 6], [10, 9])).close()


def test_bad_arguments_return_codes_not_crashes():
    L = _cabi.lib()
    h = ctypes.c_void_p()
    sp = _cabi.Specials(0, 1, -1, -1)
    assert L.dnatok_create_char(None, ctypes.byref(sp), ctypes.byref(h)) == -1
    assert b"NULL" in L.dnatok_last_error()
    lut = np.zeros(256, np.int32)
    assert L.dnatok_create_kmer(9, _cabi.np_ptr(lut), _cabi.np_ptr(lut), ctypes.byref(sp), ctypes.byref(h)) == -3
    bad = _cabi.Specials(-5, 1, -1, -1)
    assert L.dnatok_create_char(_cabi.np_ptr(lut), ctypes.byref(bad), ctypes.byref(h)) == -1
    assert L.dnatok_kind(None) == -1
    L.dnatok_destroy(None)


def test_pack_fasta_native_packer():
    """Records, multi-line sequences, CRLF, blank lines, sequence before the first header."""
    from dnatok_b200.pack import pack_fasta

    def ref(text):
        rows, cur = [], None
        for line in text.decode().split("\n"):
            line = line.rstrip("\r \t")
            if not line:
                continue
            if line[0] in ">;":
                cur = []
                rows.append(cur)
            else:
                if cur is None:
                    cur = []
                    rows.append(cur)
                cur.append(line)
        return ["".join(r) for r in rows]

    cases = [b">a\nACGT\nACG\n>b desc\nTT\n", b"ACGT\nAC\n>x\nGG", b">only header\n", b"", b"\n\n>r1\r\nAC\r\nGT\r\n\r\n>r2\r\nNN",
             b">a\n>b\nA\n;c\nCC\n  \n"]
    rng = np.random.default_rng(0)
    big = []
    for i in range(300):
        n = int(rng.integers(0, 400))
        seq = bytes(np.frombuffer(b"ACGTN", np.uint8)[rng.integers(0, 5, n)])
        big.append(b">read%d\n" % i + b"\n".join(seq[j:j + 60] for j in range(0, n, 60)) + b"\n")
    cases.append(b"".join(big))
    for text in cases:
        flat, offs = pack_fasta(text)
        want = ref(text)
        assert len(offs) == len(want) + 1 and offs[0] == 0
        got = [bytes(flat[offs[i]:offs[i + 1]]).decode() for i in range(len(want))]
        assert got == want
    L = _cabi.lib()
    n1, n2 = ctypes.c_int64(), ctypes.c_int64()
    small = np.zeros(2, np.uint8)
    offs = np.zeros(8, np.int64)
    text = np.frombuffer(b">a\nACGT\n", np.uint8)
    assert L.dnatok_pack_fasta(_cabi.np_ptr(text), text.size, _cabi.np_ptr(small), 2, _cabi.np_ptr(offs), 8,
                               ctypes.byref(n1), ctypes.byref(n2)) == -5

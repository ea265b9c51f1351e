"""Tokenizers the fast k-mer form cannot express, through the complete window table (rows the reference
covers with its 5**k table and multi-token expansion, src/dna_tokenizer.py:743-822 and :1896-1953), and
per-character tokenizers whose first-position ids differ (:527-631, :1779-1820).  The tokenizers below are
re-creations of the shapes the reference's own tests use (tests/test_kmer_bytes_fallback.py:8-59: two
tokens for every window holding N, tail dropped; tests/test_ids_path_equivalence.py:310-345: k = 4, every
window one token, tail per character); the live tokenizer object is the oracle."""
import numpy as np
import pytest

from dnatok_b200 import tables

torch = pytest.importorskip("torch")


class TwoTokensForN:
    """k-mer tokenizer: clean windows get ids in order of first use, a window holding N gives the pair
    (97, 98), characters left over after the last whole window give nothing."""

    def __init__(self, k=3):
        self.k, self.pad_token_id, self.padding_side, self.seen = k, 0, "right", {}

    def _one(self, text):
        out = []
        for i in range(0, len(text) - self.k + 1, self.k):
            w = text[i:i + self.k]
            if "N" in w:
                out += [97, 98]
            else:
                out.append(self.seen.setdefault(w, len(self.seen) + 1))
        return out

    def __call__(self, texts, add_special_tokens=False, **kw):
        return {"input_ids": [self._one(t) for t in ([texts] if isinstance(texts, str) else texts)]}


class SumOfLetters:
    """k-mer tokenizer: a whole window is one token whose id is 100 + the sum of its letters' values
    (many windows share an id, windows with N included); the tail goes letter by letter."""

    def __init__(self, k=4):
        self.k, self.pad_token_id, self.value = k, 0, {"A": 1, "C": 2, "G": 3, "T": 4, "N": 5}

    def _one(self, text):
        out, i = [], 0
        while i < len(text):
            w = text[i:i + self.k]
            out += [100 + sum(self.value.get(c, 0) for c in w)] if len(w) == self.k else [self.value.get(c, 0) for c in w]
            i += len(w)
        return out

    def __call__(self, texts, add_special_tokens=False, **kw):
        return {"input_ids": [self._one(t) for t in ([texts] if isinstance(texts, str) else texts)]}


class FirstLetterDiffers:
    """One token per character; a character's id at the start of a sequence is 50 higher than later on."""

    def __init__(self):
        self.pad_token_id, self.unk_token_id = 0, 1
        self.later = {c: 10 + i for i, c in enumerate("ACGTNacgtn")}

    def _one(self, text):
        return [self.later.get(c, 1) + (50 if i == 0 else 0) for i, c in enumerate(text)]

    def __call__(self, texts, add_special_tokens=False, **kw):
        return {"input_ids": [self._one(t) for t in ([texts] if isinstance(texts, str) else texts)]}


def _strings(rng, n, lo, hi, alphabet="ACGTN", p=(0.23, 0.23, 0.23, 0.23, 0.08)):
    return ["".join(rng.choice(list(alphabet), size=int(k), p=p)) for k in rng.integers(lo, hi, size=n)]


@pytest.mark.parametrize("make", [TwoTokensForN, SumOfLetters])
def test_window_table_discovery_cpu(make):
    tok = make()
    spec = tables.spec_from_tokenizer(tok)
    assert spec.kind == "kmer" and spec.k == tok.k and spec.kmer_table5 is not None and len(spec.kmer_table5) == 5 ** tok.k
    assert spec.kmer_tail_singles == isinstance(tok, SumOfLetters)
    rng = np.random.default_rng(1)
    for s in _strings(rng, 200, 0, 90):
        assert tables.expected_kmer_table_ids(s, spec) == tok(s)["input_ids"][0]


def test_start_table_discovery_cpu():
    spec = tables.spec_from_tokenizer(FirstLetterDiffers())
    assert spec.kind == "char" and spec.start_lut256 is not None
    assert spec.start_lut256[ord("A")] == 60 and spec.lut256[ord("A")] == 10 and spec.lut256[ord("x")] == 1


@pytest.mark.gpu
@pytest.mark.parametrize("make", [TwoTokensForN, SumOfLetters])
@pytest.mark.parametrize("ids_dtype", ["int64", "int32"])
def test_window_table_tokenizers_on_gpu(make, ids_dtype):
    from dnatok_b200.tokenizer import B200Tokenizer
    live = make()
    tok = B200Tokenizer.from_hf(live)
    rng = np.random.default_rng(7)
    strs = _strings(rng, 300, 0, 400) + ["", "N" * 50, "ACG" * 200 + "NN", "A" * live.k, "A" * (live.k - 1), "ACGTN" * 333]
    want = [live(s)["input_ids"][0] for s in strs]
    from dnatok_b200.pack import pack_strings
    flat, offs = pack_strings(strs)
    d_b = torch.from_numpy(flat.copy()).cuda() if flat.size else torch.empty(0, dtype=torch.uint8, device="cuda")
    d_o = torch.from_numpy(offs).cuda()
    dt = getattr(torch, ids_dtype)
    # ragged
    enc = tok.encode_device(d_b, d_o, host_offsets=offs, padding=False, add_special_tokens=False, ids_dtype=dt)
    ids, oo = enc["input_ids"].cpu().numpy(), enc["offsets"].cpu().numpy()
    for i, w in enumerate(want):
        assert ids[oo[i]:oo[i + 1]].tolist() == w, "row %d %r" % (i, strs[i][:40])
    # padded to the longest, both sides, with mask
    for side in ("right", "left"):
        tok.padding_side = side
        enc = tok.encode_device(d_b, d_o, host_offsets=offs, padding="longest", add_special_tokens=False, ids_dtype=dt)
        ids, mask = enc["input_ids"].cpu().numpy(), enc["attention_mask"].cpu().numpy()
        width = max(len(w) for w in want)
        assert ids.shape == (len(strs), width)
        for i, w in enumerate(want):
            row = ([0] * (width - len(w)) + w) if side == "left" else (w + [0] * (width - len(w)))
            m = ([0] * (width - len(w)) + [1] * len(w)) if side == "left" else ([1] * len(w) + [0] * (width - len(w)))
            assert ids[i].tolist() == row and mask[i].tolist() == m, (side, i)
    # truncation to 20 tokens
    tok.padding_side = "right"
    enc = tok.encode_device(d_b, d_o, host_offsets=offs, padding="max_length", max_length=20, truncation=True,
                            add_special_tokens=False, ids_dtype=dt)
    ids = enc["input_ids"].cpu().numpy()
    for i, w in enumerate(want):
        assert ids[i].tolist() == (w[:20] + [0] * max(0, 20 - len(w)))
    # the HF call surface
    got = tok(strs[:50], add_special_tokens=False)["input_ids"]
    assert [list(g) for g in got] == want[:50]


@pytest.mark.gpu
def test_start_table_tokenizer_on_gpu():
    from dnatok_b200.tokenizer import B200Tokenizer
    live = FirstLetterDiffers()
    tok = B200Tokenizer.from_hf(live)
    rng = np.random.default_rng(9)
    strs = _strings(rng, 200, 0, 700, alphabet="ACGTNacx", p=(0.2, 0.2, 0.2, 0.2, 0.05, 0.05, 0.05, 0.05)) + ["", "A", "xA", "N" * 4097]
    want = [live(s)["input_ids"][0] for s in strs]
    got = tok(strs, add_special_tokens=False)["input_ids"]
    assert [list(g) for g in got] == want
    for side in ("right", "left"):
        tok.padding_side = side
        enc = tok(strs, padding=True, add_special_tokens=False, return_tensors="np")
        width = max(len(w) for w in want)
        for i, w in enumerate(want):
            row = ([0] * (width - len(w)) + w) if side == "left" else (w + [0] * (width - len(w)))
            assert enc["input_ids"][i].tolist() == row, (side, i)
    tok.padding_side = "right"
    enc = tok(strs, padding="max_length", max_length=33, truncation=True, add_special_tokens=False, return_tensors="np")
    for i, w in enumerate(want):
        assert enc["input_ids"][i].tolist() == w[:33] + [0] * max(0, 33 - len(w))

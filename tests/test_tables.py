"""Table extraction from Hugging Face tokenizers: the discovery step that feeds the kernels."""
import numpy as np
import pytest

from dnatok_b200 import tables
from dnatok_b200 import gputok_bpe_backend as backend
from oracle import hf_oracle

import helpers as H


def test_char_discovery():
    s = H.spec("char")
    assert s.kind == "char" and s.vocab_size == 10
    assert (s.specials.pad_id, s.specials.unk_id, s.specials.cls_id, s.specials.sep_id) == (0, 1, 2, 3)
    assert [int(s.lut256[ord(c)]) for c in "ACGTN"] == [5, 6, 7, 8, 9]
    assert int(s.lut256[ord("a")]) == 1 and int(s.lut256[200]) == 1


def test_byte_discovery_matches_reference_evo2_definition():
    s = H.spec("byte")
    assert s.kind == "char" and s.specials.pad_id == 1 and s.specials.unk_id == 0 and s.specials.cls_id == -1
    for c in range(33, 127):
        assert int(s.lut256[c]) == c


def test_kmer_discovery():
    s = H.spec("kmer6")
    assert s.kind == "kmer" and s.k == 6 and s.kmer_ids.shape == (4096,)
    assert np.array_equal(s.kmer_ids, np.arange(5, 4101))
    assert [int(s.lut256[ord(c)]) for c in "ACGTN"] == [4101, 4102, 4103, 4104, 4105]
    assert s.specials.cls_id == -1 and s.specials.sep_id == -1


def test_kmer_discovery_other_k():
    s = tables.spec_from_tokenizer(hf_oracle.kmer_tokenizer(3))
    assert s.kind == "kmer" and s.k == 3 and s.kmer_ids.shape == (64,)


def test_kmer_that_is_not_window_aligned_is_refused():
    """A tokenizer that emits one [UNK] for a whole window holding N (no per-character fallback)."""
    from tokenizers import Tokenizer, Regex
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Split
    from transformers import PreTrainedTokenizerFast
    tok = Tokenizer(WordLevel(hf_oracle.kmer_vocab(3), unk_token="[UNK]"))
    tok.pre_tokenizer = Split(Regex(".{1,3}"), "isolated")
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, pad_token="[PAD]", unk_token="[UNK]")
    with pytest.raises(tables.UnsupportedTokenizer):
        tables.spec_from_tokenizer(fast)


@pytest.mark.parametrize("name,n", [("bpe4096", 4087), ("bpe32000", 31991)])
def test_bpe_tables_in_hf_id_space(name, n):
    s = H.spec(name)
    assert s.kind == "bpe" and len(s.merge_a) == n
    # BpeTrainer layout: 5 specials, 4 bases, then one new token per rank
    assert np.array_equal(s.merge_out, 9 + np.arange(n))
    assert sorted(int(s.lut256[ord(c)]) for c in "ACGT") == [5, 6, 7, 8]
    assert int(s.lut256[ord("N")]) == 1 and (s.specials.cls_id, s.specials.sep_id) == (2, 3)
    inv = {v: k for k, v in s.vocab.items()}
    for r in (0, 17, n - 1):
        assert inv[int(s.merge_a[r])] + inv[int(s.merge_b[r])] == inv[int(s.merge_out[r])]


def test_normalizer_known_answers(golden):
    """Outputs recorded from the reference's _compile_normalizer_step."""
    for case in golden["normalizer"]["accepted"]:
        fn = tables.compile_normalizer_step(case["step"])
        assert fn is not None, case["step"]
        assert [fn(x) for x in case["inputs"]] == case["outputs"], case["step"]
    for step in golden["normalizer"]["rejected"]:
        assert tables.compile_normalizer_step(step) is None
    assert backend._compile_normalizer_step({"type": "Prepend", "prepend": "_"})("") == "_"


def test_supported_tokenizer_rules():
    ok, why = backend._supported_tokenizer({"model": {"type": "BPE", "merges": ["A A"]},
                                            "pre_tokenizer": {"type": "Whitespace"},
                                            "normalizer": {"type": "BertNormalizer"}})
    assert not ok and "normalizer" in why.lower()
    assert not backend._supported_tokenizer(None)[0]
    assert not backend._supported_tokenizer({"model": {"type": "WordLevel"}})[0]
    assert not backend._supported_tokenizer({"model": {"type": "BPE"}, "pre_tokenizer": {"type": "ByteLevel"}})[0]
    assert not backend._supported_tokenizer({"model": {"type": "BPE", "dropout": 0.1}})[0]
    assert backend._supported_tokenizer({"model": {"type": "BPE"}, "pre_tokenizer": None})[0]
    assert backend.GPUTokBPEBackend.is_supported(H.hf("bpe4096"))
    assert not backend.GPUTokBPEBackend.is_supported(H.hf("char"))
    assert backend._extract_merges({"model": {"merges": [["A", "C"], "G T"]}}) == ["A C", "G T"]
    with pytest.raises(ValueError):
        backend._extract_merges({"model": {"merges": [["A"]]}})


def test_discovery_of_a_tokenizer_that_rejects_ragged_batches():
    """A dict tokenizer that upper-cases, returns a rectangular tensor and so fails on a ragged
    batch (like the reference's CharTokenizer, src/dnatok_compat.py:220-238) is probed one text at a time."""
    import torch

    class Plain:
        pad_token_id, unk_token_id = 0, 9

        def __call__(self, text, **kw):
            texts = [text] if isinstance(text, str) else list(text)
            table = {"A": 3, "C": 4, "G": 5, "T": 6}
            return {"input_ids": torch.tensor([[table.get(c, 9) for c in t.upper()] for t in texts])}

    s = tables.spec_from_tokenizer(Plain())
    assert s.kind == "char" and (s.specials.pad_id, s.specials.unk_id, s.specials.cls_id) == (0, 9, -1)
    assert [int(s.lut256[ord(c)]) for c in "ACGTacgtNx"] == [3, 4, 5, 6, 3, 4, 5, 6, 9, 9]

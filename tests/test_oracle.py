"""The CPU checker against the golden vectors (Hugging Face output and the reference's own CPU
paths, recorded by tests/golden/make_golden.py) and against live Hugging Face."""
import numpy as np
import pytest

from dnatok_b200 import synth
from oracle import oracle

import helpers as H


@pytest.mark.parametrize("cfg", H.ALL_CONFIGS)
def test_oracle_matches_golden_hf_hashes(golden, cfg):
    g = golden["configs"][cfg]
    name, flat, offs = H.config_inputs(cfg)
    assert H.sha(flat) == g["input_sha256"], "synthetic generator drifted"
    ids, mask = H.oracle_batch(name, flat, offs, **H.call_to_kwargs(g["call"]))
    assert list(ids.shape) == g["shape"]
    assert H.sha(ids) == g["ids_sha256"]
    assert H.sha(mask) == g["mask_sha256"]
    assert ids[:2, :64].tolist() == g["first_rows"]
    assert int(mask.sum()) == g["n_tokens"]


def test_oracle_matches_golden_ragged(golden):
    g = golden["configs"]["cfg5_bpe32000_512reads"]
    name, flat, offs = H.config_inputs("cfg5_bpe32000_512reads")
    rows = H.oracle_batch(name, flat, offs, padding=False)
    assert H.sha(np.concatenate(rows)) == g["ragged_ids_sha256"]
    assert H.sha(np.concatenate([[0], np.cumsum([len(r) for r in rows])]).astype(np.int64)) == g["ragged_offsets_sha256"]


@pytest.mark.parametrize("cfg", ["cfg1_char", "cfg2_kmer6", "cfg4_byte_2x131072"])
def test_oracle_matches_reference_cpu_path(golden, cfg):
    """ids the reference's DNATok.encode_batch_to_ids produced (no specials, right padded)."""
    g = golden["reference_paths"][cfg]
    assert g["equals_hf_plain"]
    name, flat, offs = H.config_inputs(cfg)
    ids, _ = H.oracle_batch(name, flat, offs, add_special=False)
    assert list(ids.shape) == g["shape"]
    assert H.sha(ids) == g["ids_sha256"]


def test_oracle_matches_reference_evo2_tokenizer(golden):
    g = golden["reference_paths"]["evo2_byte_first4096"]
    name, flat, offs = H.config_inputs("cfg4_byte_2x131072")
    rows = H.oracle_rows(name, flat[:4096], np.array([0, 4096], dtype=np.int64))
    assert H.sha(rows[0].astype(np.int64)) == g["ids_sha256"]
    s = H.spec("byte")
    assert (s.specials.pad_id, s.specials.unk_id) == (g["pad_token_id"], g["unk_token_id"])


@pytest.mark.parametrize("cls", H.COMPAT_TOKENIZERS)
def test_oracle_matches_reference_tokenizer_classes(golden, cls):
    """ids the reference's own tokenizer classes (src/dnatok_compat.py:135-238) gave for the non-empty
    adversarial strings, against the oracle run on the table discovered from each class."""
    g = golden["compat_tokenizers"]["tokenizers"][cls]
    s = H.compat_spec(g)
    assert s.kind == "char"
    flat, offs = H.pack_strs(golden["compat_tokenizers"]["inputs"])
    ids, counts = oracle.encode_ragged("char", flat, offs, lut256=s.lut256)
    assert [r.tolist() for r in oracle.rows(ids, offs, counts)] == g["ids"]


@pytest.mark.parametrize("name", H.TOKENIZERS)
def test_oracle_matches_golden_adversarial(golden, name):
    strs = golden["adversarial_inputs"]
    flat, offs = H.pack_strs(strs)
    plain = H.oracle_batch(name, flat, offs, padding=False, add_special=False)
    special = H.oracle_batch(name, flat, offs, padding=False, add_special=True)
    assert [r.tolist() for r in plain] == golden["adversarial"][name]["plain"]
    assert [r.tolist() for r in special] == golden["adversarial"][name]["special"]


@pytest.mark.parametrize("name", ["bpe4096", "bpe32000"])
def test_bpe_queue_equals_definition(name):
    """The queue-driven merge loop against rescanning for the lowest-rank leftmost pair."""
    s, t = H.spec(name), H.bpe_table(name)
    rng = np.random.default_rng(7)
    words = [bytes(synth.config3(batch=1, length=int(n), seed=int(k))[0]) for k, n in enumerate(rng.integers(1, 400, 25))]
    words += [b"A" * n for n in (1, 2, 3, 4, 5, 8, 9, 31, 64, 257)] + [b"AC" * 100, b"ACGNNACG" * 9, b"acgt" * 5]
    for w in words:
        assert oracle.bpe_word(t, w, s.lut256) == oracle.bpe_word(t, w, s.lut256, naive=True)


@pytest.mark.parametrize("name", H.TOKENIZERS)
def test_oracle_matches_live_hf(name):
    """Fresh seeds (not the golden inputs), ragged lengths, live Hugging Face."""
    tok = H.hf(name)
    rng = np.random.default_rng(11)
    lens = rng.integers(0, 700, size=48)
    a = synth.config1(batch=48, length=700, seed=5)
    if name == "byte":
        a = synth.config4(batch=48, length=700, seed=5)
    strs = [bytes(a[i, :lens[i]]).decode() for i in range(48)]
    flat, offs = H.pack_strs(strs)
    enc = tok(strs, padding=True, return_tensors="np")
    ids, mask = H.oracle_batch(name, flat, offs)
    assert np.array_equal(ids, enc["input_ids"]) and np.array_equal(mask, enc["attention_mask"])
    enc = tok(strs, padding="max_length", max_length=64, truncation=True, return_tensors="np")
    ids, mask = H.oracle_batch(name, flat, offs, padding="max_length", max_length=64, truncation=True)
    assert np.array_equal(ids, enc["input_ids"]) and np.array_equal(mask, enc["attention_mask"])

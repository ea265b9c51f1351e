"""Property tests of the CPU checker and of the table semantics (hypothesis), no GPU."""
import numpy as np
from hypothesis import given, settings, strategies as st

from dnatok_b200 import tables
from oracle import oracle

import helpers as H

DNA = st.text(alphabet="ACGTNacgtnRY-", min_size=0, max_size=300)


@settings(max_examples=150, deadline=None)
@given(DNA)
def test_bpe_queue_equals_definition_on_any_string(s):
    spec, table = H.spec("bpe4096"), H.bpe_table("bpe4096")
    w = s.encode()
    a = oracle.bpe_word(table, w, spec.lut256)
    assert a == oracle.bpe_word(table, w, spec.lut256, naive=True)
    inv = {v: k for k, v in spec.vocab.items()}
    # decoding covers the string exactly; characters outside the alphabet are one [UNK] each
    assert sum(1 if t == spec.specials.unk_id else len(inv[t]) for t in a) == len(w)


@settings(max_examples=150, deadline=None)
@given(DNA, st.integers(min_value=1, max_value=8))
def test_kmer_checker_equals_table_semantics(s, k):
    rng = np.random.default_rng(k)
    kmer_ids = (5 + rng.permutation(4 ** k)).astype(np.int32)
    singles = np.full(256, 1, np.int32)
    for i, c in enumerate("ACGTN"):
        singles[ord(c)] = 5 + 4 ** k + i
    flat, offs = H.pack_strs([s])
    ids, counts = oracle.encode_ragged("kmer", flat, offs, lut256=singles, k=k, kmer_ids=kmer_ids)
    assert ids[:counts[0]].tolist() == tables.expected_kmer_ids(s, k, kmer_ids, singles)
    assert counts[0] <= len(s)


@settings(max_examples=60, deadline=None)
@given(st.lists(DNA, min_size=1, max_size=8), st.integers(min_value=2, max_value=40), st.booleans(), st.booleans())
def test_assembly_rules_match_live_hf(strs, max_length, special, left):
    """Truncation keeps max_length tokens including the specials; padding side; mask."""
    tok = H.hf("char")
    tok.padding_side = "left" if left else "right"
    try:
        want = tok(strs, padding="max_length", max_length=max_length, truncation=True, add_special_tokens=special,
                   return_tensors="np")
    finally:
        tok.padding_side = "right"
    flat, offs = H.pack_strs(strs)
    ids, mask = H.oracle_batch("char", flat, offs, padding="max_length", max_length=max_length, truncation=True,
                               add_special=special, pad_left=left)
    assert np.array_equal(ids, want["input_ids"]) and np.array_equal(mask, want["attention_mask"])

"""BPE plug-in slots against the live Hugging Face tokenizer: tokenizers that carry a normalizer
(the cases the reference pins at tests/test_gputok_bpe_backend.py:137-182: runs of N through a
GENA-LM style ``N{10,} -> -`` rule, a METAGENE style ``Prepend("_")``, mixed case) and the native
slot built from a merges file (reference src/dnatok_bpe_kernel/__init__.py:81-136)."""
import json

import numpy as np
import pytest

from dnatok_b200 import synth

import helpers as H

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

NORMALIZERS = {
    "gena_n_runs": {"type": "Sequence", "normalizers": [
        {"type": "Strip", "strip_left": True, "strip_right": True},
        {"type": "Replace", "pattern": {"Regex": "N{10,}"}, "content": "-"}]},
    "metagene_prepend": {"type": "Prepend", "prepend": "_"},
    "lowercase_then_upper_vocab": {"type": "Sequence", "normalizers": [
        {"type": "NFC"}, {"type": "Replace", "pattern": {"String": "n"}, "content": "N"}]},
}


def _hf_with_normalizer(kind):
    from tokenizers import Tokenizer
    from oracle import hf_oracle
    cfg = hf_oracle.load_tokenizer_json("bpe4096")
    cfg["normalizer"] = NORMALIZERS[kind]
    return hf_oracle._wrap(Tokenizer.from_str(json.dumps(cfg)))


def _cases():
    rng = np.random.default_rng(17)
    body = lambda n: "".join(rng.choice(list("ACGT"), size=n))
    out = []
    for run in (1, 5, 9, 10, 11, 20, 64):                     # N runs on both sides of the 10-N rule
        out.append(body(120) + "N" * run + body(77))
    out += ["N" * 30, body(40) + "N" * 12, "N" * 15 + body(40), body(300), "acgtnACGTN" * 12,
            body(64).lower() + body(64), "A", body(2047) + "N" * 10 + body(2049)]
    return out


@pytest.mark.parametrize("kind", list(NORMALIZERS))
def test_bpe_with_normalizer_matches_live_hf(kind):
    from dnatok_b200.gputok_bpe_backend import GPUTokBPEBackend
    from dnatok_b200.tokenizer import B200Tokenizer
    hf = _hf_with_normalizer(kind)
    strs = _cases()
    want = hf(strs, padding=True, add_special_tokens=False, return_tensors="np")
    assert GPUTokBPEBackend.is_supported(hf)
    be = GPUTokBPEBackend(hf, engine="dnatok")
    ids, mask = be.encode_batch(strs, device="cuda")
    assert np.array_equal(ids.cpu().numpy(), want["input_ids"])
    assert np.array_equal(mask.cpu().numpy(), want["attention_mask"].astype(np.uint8))
    # the HF call surface, special tokens included, one row at a time and as a batch
    mine = B200Tokenizer.from_hf(hf)
    full = hf(strs, padding=True, return_tensors="np")
    got = mine(strs, padding=True, return_tensors="np")
    assert np.array_equal(got["input_ids"], full["input_ids"])
    assert np.array_equal(got["attention_mask"], full["attention_mask"])
    for s in strs[:6]:
        assert mine.encode(s) == hf.encode(s)


def test_native_slot_from_merges_file(tmp_path):
    """DnatokBpeKernel(merges_path): ids in the reference's internal vocabulary, checked token by
    token against Hugging Face through id_to_token."""
    from dnatok_b200.gputok_bpe_backend import DnatokBpeKernel, _extract_merges
    from oracle import hf_oracle
    cfg = hf_oracle.load_tokenizer_json("bpe4096")
    merges = _extract_merges(cfg)
    path = tmp_path / "merges.txt"
    path.write_text("#version: 0.2\n" + "\n".join(merges) + "\n")
    k = DnatokBpeKernel(str(path), max_iters=1024)
    assert k.vocab_size() >= 256 + len(merges)
    assert k.id_to_token(ord("A")) == "A"
    first = merges[0].split(" ")
    assert k.id_to_token(256) == first[0] + first[1]          # single-byte operands exist already: the result takes id 256
    hf = H.hf("bpe4096")
    strs = synth.rows_to_strings(*synth.pack_rows(synth.config3(batch=20, length=900, seed=8))) + ["A" * 33, "ACGT"]
    ids, lens = k.tokenize_batch(strs, clone=True)
    assert ids.dtype == torch.int32 and lens.dtype == torch.int32 and ids.is_cuda
    ids, lens = ids.cpu().numpy(), lens.cpu().numpy()
    for i, s in enumerate(strs):
        want = hf.convert_ids_to_tokens(hf(s, add_special_tokens=False)["input_ids"])
        got = [k.id_to_token(t) for t in ids[i, :lens[i]]]
        assert got == want, "row %d" % i
        assert not ids[i, lens[i]:].any()
    with pytest.raises(RuntimeError):
        DnatokBpeKernel(str(tmp_path / "missing.txt"))
    with pytest.raises(IndexError):
        k.id_to_token(10 ** 6)

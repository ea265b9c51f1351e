"""Generate the committed golden vectors.  Needs a checkout of eniktab/DNAtok and Hugging Face
``tokenizers``:

    DNATOK_REFERENCE_SRC=<checkout>/src python tests/golden/make_golden.py

Writes ``tests/golden/golden.json`` (hashes + small literal cases) from three sources:
  * live Hugging Face tokenizers built by ``oracle/hf_oracle.py`` - the parity target;
  * the reference's own CPU paths imported from that checkout: ``DNATok`` (numpy LUT and
    k-mer paths) wrapped around those tokenizers, and the tokenizer classes of ``dnatok_compat``
    (``NTv3Tokenizer``, ``Evo2ByteTokenizer``, ``CharTokenizer``);
  * the reference's normaliser known answers (``tests/test_gputok_bpe_backend.py:319-425``),
    re-derived by calling its ``_compile_normalizer_step``.
The reference is needed only here; the tests read the vectors.
"""
import hashlib
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import transformers  # noqa: E402,F401  (must be imported before the reference's dnatok_compat)
import torch  # noqa: E402

from dnatok_b200 import synth  # noqa: E402
from oracle import hf_oracle  # noqa: E402

REF_SRC = os.environ.get("DNATOK_REFERENCE_SRC", "")


def sha(a) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


ADVERSARIAL = [
    "", "A", "N", "AC", "ACGTA", "ACGTAC", "ACGTACG", "NNNNNN", "ACGTNACGTACGT", "ACGTACNACGTAC",
    "acgtACGTacgt", "ACGTRYKMACGT", "A" * 7, "A" * 64, "A" * 255, "C" * 1024, "AC" * 300, "ACG" * 333,
    "N" * 50, "ACGT" * 3 + "N" * 7 + "ACGT" * 5 + "n", "TTTTTTTTTTTTTTA" * 20, "GATTACA" * 100 + "N",
    "ACGTAC" * 10 + "ACGTA", "NACGTA" * 5, "ACGTAN" * 5, "AAAAACAAAAAGAAAAAAT" * 30,
]


def hf_batch(tok, strs, **kw):
    enc = tok(strs, return_tensors="np", **kw)
    return enc["input_ids"], enc["attention_mask"]


class _Embedder(torch.nn.Module):
    def __init__(self, tokenizer):
        super().__init__()
        self.tokenizer = tokenizer
        self.pad_id = tokenizer.pad_token_id
        self.max_position_embeddings = None
        self._embed = torch.nn.Embedding(8, 2)

    def embed_tokens(self, input_ids, rc_invariant=False):
        return self._embed(input_ids.clamp(max=7))


def main():
    if not os.path.isdir(REF_SRC):
        raise SystemExit("set DNATOK_REFERENCE_SRC to the src/ directory of an eniktab/DNAtok checkout")
    sys.path.insert(0, REF_SRC)
    from dna_tokenizer import DNATok                      # reference, CPU numpy paths
    import gputok_bpe_backend as ref_backend              # reference normaliser compiler
    from dnatok_compat import Evo2ByteTokenizer           # reference byte-level tokenizer

    G = {"tokenizers_version": __import__("tokenizers").__version__, "configs": {}, "adversarial": {}}

    toks = {
        "char": hf_oracle.char_tokenizer(),
        "kmer6": hf_oracle.kmer_tokenizer(),
        "bpe4096": hf_oracle.bpe_tokenizer("bpe4096"),
        "byte": hf_oracle.byte_tokenizer(),
        "bpe32000": hf_oracle.bpe_tokenizer("bpe32000"),
    }

    def record(name, flat, offs, tok, call, keep_rows=2):
        strs = synth.rows_to_strings(flat, offs)
        ids, mask = hf_batch(tok, strs, **call)
        G["configs"][name] = {
            "input_sha256": sha(flat), "n_rows": len(strs), "call": {k: v for k, v in call.items()},
            "shape": list(ids.shape), "ids_sha256": sha(ids.astype(np.int64)),
            "mask_sha256": sha(mask.astype(np.int64)),
            "first_rows": ids[:keep_rows, :64].tolist(),
            "n_tokens": int(mask.sum()),
        }
        return strs, ids, mask

    f, o = synth.pack_rows(synth.config1())
    s1, ids1, _ = record("cfg1_char", f, o, toks["char"], dict(padding=True))
    f, o = synth.pack_rows(synth.config2())
    s2, ids2, _ = record("cfg2_kmer6", f, o, toks["kmer6"], dict(padding="max_length", max_length=1000, truncation=True))
    f, o = synth.pack_rows(synth.config3())
    record("cfg3_bpe4096", f, o, toks["bpe4096"], dict(padding=True))
    f, o = synth.pack_rows(synth.config4(batch=2, length=131072))
    s4, ids4, _ = record("cfg4_byte_2x131072", f, o, toks["byte"], dict(padding=True))
    f, o = synth.config5(n_reads=512)
    record("cfg5_bpe32000_512reads", f, o, toks["bpe32000"], dict(padding=True))

    # ragged (no padding) outputs of config 5: hash of the concatenated rows and the offsets
    strs = synth.rows_to_strings(f, o)
    rows = toks["bpe32000"](strs)["input_ids"]
    cat = np.concatenate([np.asarray(r, dtype=np.int64) for r in rows])
    G["configs"]["cfg5_bpe32000_512reads"]["ragged_ids_sha256"] = sha(cat)
    G["configs"]["cfg5_bpe32000_512reads"]["ragged_offsets_sha256"] = sha(
        np.concatenate([[0], np.cumsum([len(r) for r in rows])]).astype(np.int64))

    # adversarial strings, ids without and with specials, per tokenizer
    for name, tok in toks.items():
        G["adversarial"][name] = {
            "plain": [list(map(int, r)) for r in tok(ADVERSARIAL, add_special_tokens=False)["input_ids"]],
            "special": [list(map(int, r)) for r in tok(ADVERSARIAL, add_special_tokens=True)["input_ids"]],
        }
    G["adversarial_inputs"] = ADVERSARIAL

    # the reference's own CPU paths on the same inputs (no special tokens in the reference)
    ref = {}
    for name, tok, strs in (("cfg1_char", toks["char"], s1), ("cfg2_kmer6", toks["kmer6"], s2),
                            ("cfg4_byte_2x131072", toks["byte"], s4)):
        h = DNATok(_Embedder(tok), padding_side="right")
        h.discover()
        out = h.encode_batch_to_ids(strs)
        plain = np.asarray(tok(strs, add_special_tokens=False, padding=True, return_tensors="np")["input_ids"])
        ref[name] = {"path": "kmer" if getattr(h, "kmer_k", None) else "ascii_lut",
                     "shape": list(out.shape), "ids_sha256": sha(out.numpy().astype(np.int64)),
                     "equals_hf_plain": bool(np.array_equal(out.numpy(), plain))}
    evo = Evo2ByteTokenizer(vocab_size=512)
    seg = s4[0][:4096]
    e_ids = evo(seg)["input_ids"]
    ref["evo2_byte_first4096"] = {"ids_sha256": sha(np.asarray(e_ids, dtype=np.int64)),
                                  "pad_token_id": evo.pad_token_id, "unk_token_id": evo.unk_token_id}
    G["reference_paths"] = ref

    # the reference's DNATok API on a small ragged batch: encode_batch_to_ids and
    # encode_batch_with_padding, both padding sides (its default is left)
    rng = np.random.default_rng(99)
    api_seqs = []
    for n in [1, 5, 6, 7, 12, 13, 40, 64, 100, 37, 18, 90]:
        row = np.frombuffer(b"ACGT", np.uint8)[rng.integers(0, 4, n)].copy()
        if n in (40, 100, 13):
            row[n // 3:n // 3 + 3] = ord("N")
        api_seqs.append(bytes(row).decode())
    api = {"seqs": api_seqs, "cases": []}
    for tname in ("char", "kmer6"):
        for side in ("left", "right"):
            hlp = DNATok(_Embedder(toks[tname]), padding_side=side)
            hlp.discover()
            ids = hlp.encode_batch_to_ids(api_seqs)
            case = {"tokenizer": tname, "padding_side": side, "encode_batch_to_ids": ids.tolist(), "with_padding": []}
            for max_tokens, pad_to_max, pad_multiple in ((16, False, 16), (8, True, 4), (64, False, 1), (10, True, 16)):
                i2, m2 = hlp.encode_batch_with_padding(api_seqs, max_tokens, pad_to_max=pad_to_max, pad_multiple=pad_multiple)
                case["with_padding"].append({"max_tokens": max_tokens, "pad_to_max": pad_to_max, "pad_multiple": pad_multiple,
                                             "ids": i2.tolist(), "ids_dtype": str(i2.dtype), "mask": m2.tolist(),
                                             "mask_dtype": str(m2.dtype)})
            api["cases"].append(case)
    G["dnatok_api"] = api

    # the reference's constructor flags normalize_case / handle_invalid_chars and its token_len
    # attribute (its own tests: tests/test_benchmark_correctness.py:146-200), both padding sides
    flag_seqs = ["AcGt", "acgt", "ACGT", "ACXGT", "AC$GT", "acgtnNRYkm", "TTTTTTTTTTTTT", "a", "ACGTACGTACGTNACGTACxACGTAC",
                 "gattacaGATTACAgattacaN", "ACGTAC" * 3 + "acgtac" + "ACGTA"]
    flags = {"seqs": flag_seqs, "cases": []}
    for tname in ("char", "kmer6"):
        for side in ("left", "right"):
            for norm_case, handle in ((True, False), (False, True), (True, True)):
                for token_len in (None, 40):
                    hlp = DNATok(_Embedder(toks[tname]), padding_side=side, normalize_case=norm_case,
                                 handle_invalid_chars=handle)
                    hlp.discover()
                    hlp.token_len = token_len
                    ids = hlp.encode_batch_to_ids(flag_seqs)
                    flags["cases"].append({"tokenizer": tname, "padding_side": side, "normalize_case": norm_case,
                                           "handle_invalid_chars": handle, "token_len": token_len,
                                           "ids": ids.tolist()})
    G["dnatok_flags"] = flags

    # the reference's own tokenizer classes (src/dnatok_compat.py:135-238): the table this package
    # discovers from each by probing, and the class's own ids for every non-empty adversarial string
    from dnatok_compat import CharTokenizer, NTv3Tokenizer
    from dnatok_b200 import tables
    compat = {"inputs": [s for s in ADVERSARIAL if s], "tokenizers": {}}
    for cname, ctok in (("NTv3Tokenizer", NTv3Tokenizer()), ("Evo2ByteTokenizer", Evo2ByteTokenizer(vocab_size=512)),
                        ("CharTokenizer", CharTokenizer())):
        spec = tables.spec_from_tokenizer(ctok)
        rows = []
        for s_ in compat["inputs"]:
            r = ctok(s_, add_special_tokens=False)["input_ids"]
            r = r.tolist() if hasattr(r, "tolist") else r
            while len(r) == 1 and isinstance(r[0], list):
                r = r[0]
            rows.append([int(v) for v in r])
        compat["tokenizers"][cname] = {
            "kind": spec.kind, "vocab_size": int(spec.vocab_size), "lut256": [int(v) for v in spec.lut256],
            "pad_id": int(spec.specials.pad_id), "unk_id": int(spec.specials.unk_id),
            "cls_id": int(spec.specials.cls_id), "sep_id": int(spec.specials.sep_id), "ids": rows}
    G["compat_tokenizers"] = compat

    # normaliser known answers, produced by the reference's compiler
    cases = [
        ({"type": "Strip", "strip_left": True, "strip_right": True}, ["  ACGT  ", "ACGT"]),
        ({"type": "Strip", "strip_left": True, "strip_right": False}, ["  ACGT  "]),
        ({"type": "Replace", "pattern": {"String": "N"}, "content": "-"}, ["ACGTNNACGT"]),
        ({"type": "Replace", "pattern": {"Regex": "N{10,}"}, "content": "-"},
         ["ACGT" + "N" * 9 + "ACGT", "ACGT" + "N" * 10 + "ACGT"]),
        ({"type": "Prepend", "prepend": "_"}, ["ACGT", ""]),
        ({"type": "Lowercase"}, ["ACGTACGT"]),
        ({"type": "NFC"}, ["ACGT"]), ({"type": "NFKD"}, ["ACGT"]), ({"type": "StripAccents"}, ["ACGT"]),
        ({"type": "Sequence", "normalizers": [{"type": "Strip", "strip_left": True, "strip_right": True},
                                              {"type": "Replace", "pattern": {"Regex": "N{10,}"}, "content": "-"}]},
         ["   " + "N" * 12 + "ACGT  "]),
    ]
    norm = []
    for step, inputs in cases:
        fn = ref_backend._compile_normalizer_step(step)
        norm.append({"step": step, "inputs": inputs, "outputs": [fn(x) for x in inputs]})
    rejected = [{"type": "BertNormalizer"}, {"type": "Nmt"}, {"type": "Precompiled"}, {"type": "SomeNewThingHFAdds"},
                {"type": "Sequence", "normalizers": [{"type": "Strip"}, {"type": "BertNormalizer"}]}]
    for step in rejected:
        assert ref_backend._compile_normalizer_step(step) is None
    G["normalizer"] = {"accepted": norm, "rejected": rejected}

    with open(os.path.join(HERE, "golden.json"), "w") as fh:
        json.dump(G, fh, sort_keys=True, separators=(",", ":"))
    print("wrote golden.json;", {k: v["shape"] for k, v in G["configs"].items()})
    print("reference paths:", json.dumps(ref, indent=1))


if __name__ == "__main__":
    main()

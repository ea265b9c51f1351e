"""Command line front end: ``python -m dnatok_b200.cli info | encode | validate | bench``.

Same four commands, payload keys and exit codes as the reference's ``dnatok`` CLI
(``src/dnatok_cli.py:162-307``): ``info`` reports the selected path, ``encode`` prints the ids of one
sequence with padding stripped, ``validate`` compares n random ACGT windows with the Hugging Face
tokenizer (``add_special_tokens=False``) and exits 1 on any mismatch, ``bench`` measures
Mbp/s = sum(bp) / wall time for both.  The reference resolves a model name on the Hugging Face hub;
here ``--tokenizer`` is a ``tokenizer.json`` file, a local directory ``AutoTokenizer`` can load, or
one of the built-in synthetic tokenizers ``char``, ``byte``, ``kmer<k>``.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import sys
import time
from typing import Any, List


def _builtin(name: str):
    """Synthetic tokenizers with the vocabularies of the benchmark shapes, built with `tokenizers`."""
    import itertools
    from tokenizers import Regex, Tokenizer
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Sequence, Split
    from transformers import PreTrainedTokenizerFast
    specials = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"]
    if name == "byte":
        tok = Tokenizer(WordLevel({chr(i): i for i in range(512)}, unk_token=chr(0)))
        tok.pre_tokenizer = Split(Regex("[\\s\\S]"), "isolated")
        return PreTrainedTokenizerFast(tokenizer_object=tok, pad_token=chr(1), unk_token=chr(0))
    vocab = {s: i for i, s in enumerate(specials)}
    if name == "char":
        for c in "ACGTN":
            vocab[c] = len(vocab)
        tok = Tokenizer(WordLevel(vocab, unk_token="[UNK]"))
        tok.pre_tokenizer = Split(Regex("."), "isolated")
    elif name.startswith("kmer") and name[4:].isdigit():
        k = int(name[4:])
        for t in itertools.product("ACGT", repeat=k):
            vocab["".join(t)] = len(vocab)
        for c in "ACGTN":
            vocab[c] = len(vocab)
        tok = Tokenizer(WordLevel(vocab, unk_token="[UNK]"))
        tok.pre_tokenizer = Sequence([Split(Regex(".{1,%d}" % k), "isolated"), Split(Regex("[ACGT]{%d}|." % k), "isolated")])
    else:
        return None
    return PreTrainedTokenizerFast(tokenizer_object=tok, pad_token="[PAD]", unk_token="[UNK]")


def load_hf(spec: str):
    tok = _builtin(spec)
    if tok is not None:
        return tok
    if os.path.isfile(spec):
        from transformers import PreTrainedTokenizerFast
        if spec.endswith(".gz"):
            import gzip
            from tokenizers import Tokenizer
            with gzip.open(spec, "rt") as f:
                obj = Tokenizer.from_str(f.read())
            tok = PreTrainedTokenizerFast(tokenizer_object=obj)
        else:
            tok = PreTrainedTokenizerFast(tokenizer_file=spec)
        vocab = tok.get_vocab()
        for attr, names in (("pad_token", ("[PAD]", "<pad>")), ("unk_token", ("[UNK]", "<unk>"))):
            for n in names:
                if getattr(tok, attr) is None and n in vocab:
                    setattr(tok, attr, n)
        return tok
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(spec, trust_remote_code=False)


class _Embedder:
    def __init__(self, tokenizer):
        self.tokenizer = tokenizer

    def embed_tokens(self, ids):
        return ids


def _build(spec: str, padding_side: str = "right"):
    from .dna_tokenizer import DNATok
    hf = load_hf(spec)
    dn = DNATok(_Embedder(hf), padding_side=padding_side)
    dn.discover()
    return hf, dn


def _path(dn) -> str:
    if dn.bpe_backend is not None:
        return "gpu_bpe"
    return "kmer_lut" if dn.kmer_k else "ascii_lut"


def _strip(row: List[int], pad: int, side: str) -> List[int]:
    if side == "left":
        j = 0
        while j < len(row) and row[j] == pad:
            j += 1
        return row[j:]
    j = len(row)
    while j > 0 and row[j - 1] == pad:
        j -= 1
    return row[:j]


def _emit(payload: Any, as_json: bool) -> None:
    if as_json:
        print(json.dumps(payload))
    else:
        for k, v in payload.items():
            print("%-24s %s" % (k, v))


def cmd_info(a) -> int:
    hf, dn = _build(a.tokenizer)
    _emit({"tokenizer": a.tokenizer, "tokenizer_class": type(hf).__name__,
           "vocab_size": int(getattr(hf, "vocab_size", 0)) or len(hf.get_vocab()), "selected_path": _path(dn),
           "device": "cuda", "kmer_k": dn.kmer_k, "has_ascii_lut": dn.use_ids_path and not dn.kmer_k,
           "has_gpu_bpe_backend": dn.bpe_backend is not None, "padding_side": dn.padding_side,
           "id_pad": int(dn.id_pad)}, a.json)
    return 0


def cmd_encode(a) -> int:
    hf, dn = _build(a.tokenizer)
    ids = _strip(dn.encode_batch_to_ids([a.seq])[0].tolist(), int(dn.id_pad), dn.padding_side)
    _emit({"tokenizer": a.tokenizer, "sequence": a.seq[:80] + ("..." if len(a.seq) > 80 else ""),
           "sequence_length_bp": len(a.seq), "n_tokens": len(ids),
           "token_ids": ids if a.json else ids[:32] + (["..."] if len(ids) > 32 else []),
           "selected_path": _path(dn)}, a.json)
    return 0


def cmd_validate(a) -> int:
    hf, dn = _build(a.tokenizer)
    rng = random.Random(a.seed)
    seqs = ["".join(rng.choices("ACGT", k=a.window)) for _ in range(a.n)]
    mine = dn.encode_batch_to_ids(seqs).tolist()
    want = hf(seqs, add_special_tokens=False, padding=False, truncation=False)["input_ids"]
    pad = int(dn.id_pad)
    n_match, first = 0, None
    for i, s in enumerate(seqs):
        got = _strip(mine[i], pad, dn.padding_side)
        if got == list(want[i]):
            n_match += 1
        elif first is None:
            first = {"i": i, "seq_head": s[:40], "dnatok_head": got[:8], "hf_head": list(want[i])[:8]}
    _emit({"tokenizer": a.tokenizer, "n_sequences": a.n, "n_match": n_match, "n_mismatch": a.n - n_match,
           "match_rate": n_match / a.n, "selected_path": _path(dn), "first_mismatch": first}, a.json)
    return 0 if n_match == a.n else 1


def cmd_bench(a) -> int:
    import torch
    os.environ["RAYON_NUM_THREADS"] = str(a.hf_threads)
    os.environ["TOKENIZERS_PARALLELISM"] = "true" if a.hf_threads > 1 else "false"
    hf, dn = _build(a.tokenizer)
    rng = random.Random(a.seed)
    seqs = ["".join(rng.choices("ACGT", k=a.window)) for _ in range(a.n)]
    bp = sum(map(len, seqs))
    hf(seqs[:min(a.chunk, a.n)], add_special_tokens=False)
    dn.encode_batch_to_ids(seqs[:min(a.chunk, a.n)])
    t0 = time.perf_counter()
    for i in range(0, a.n, a.chunk):
        hf(seqs[i:i + a.chunk], add_special_tokens=False)
    t_hf = time.perf_counter() - t0
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(0, a.n, a.chunk):
        dn.encode_batch_to_ids(seqs[i:i + a.chunk])
    torch.cuda.synchronize()
    t_dn = time.perf_counter() - t0
    _emit({"tokenizer": a.tokenizer, "n_sequences": a.n, "window_bp": a.window, "chunk": a.chunk, "total_bp": bp,
           "hf_threads": a.hf_threads, "hf_time_s": round(t_hf, 4), "hf_mbp_per_s": round(bp / t_hf / 1e6, 2),
           "dnatok_time_s": round(t_dn, 4), "dnatok_mbp_per_s": round(bp / t_dn / 1e6, 2),
           "speedup_dnatok_vs_hf": round(t_hf / t_dn, 2), "selected_path": _path(dn), "device": "cuda"}, a.json)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="dnatok_b200")
    sub = ap.add_subparsers(dest="cmd", required=True)
    for name, fn in (("info", cmd_info), ("encode", cmd_encode), ("validate", cmd_validate), ("bench", cmd_bench)):
        p = sub.add_parser(name)
        p.add_argument("--tokenizer", "--model", dest="tokenizer", required=True)
        p.add_argument("--json", action="store_true")
        if name == "encode":
            p.add_argument("--seq", required=True)
        if name in ("validate", "bench"):
            p.add_argument("--n", type=int, default=100 if name == "validate" else 1000)
            p.add_argument("--window", type=int, default=1024 if name == "validate" else 4096)
            p.add_argument("--seed", type=int, default=0)
        if name == "bench":
            p.add_argument("--chunk", type=int, default=32)
            p.add_argument("--hf-threads", type=int, default=os.cpu_count() or 1)
        p.set_defaults(fn=fn)
    a = ap.parse_args(argv)
    try:
        return a.fn(a)
    except Exception as e:                                   # same contract as the reference CLI: message + non-zero exit
        print("error: %s: %s" % (type(e).__name__, e), file=sys.stderr)
        return 2


if __name__ == "__main__":
    sys.exit(main())

"""``python -m dnatok_b200.cli <command> --tokenizer T [...]`` - a small front end over ``B200Tokenizer``.

Commands and the keys they print follow the reference's ``dnatok`` tool (``src/dnatok_cli.py:162-307``:
``info``, ``encode``, ``validate``, ``bench``; exit code 1 when ``validate`` finds a mismatch, 2 on an
error) so that scripts written against it keep working; ``scenarios`` runs the eight read-length
workloads of its realistic benchmark (``benchmarks/run_realistic_benchmark.py:184-272``).  ``--tokenizer``
is a ``tokenizer.json`` (optionally gzipped), a local directory ``AutoTokenizer`` can load, or one of the
built-in synthetic tokenizers ``char``, ``byte``, ``kmer<k>`` (the reference resolves model names on the
Hugging Face hub, which is not reachable offline).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np

PATH_NAME = {"char": "ascii_lut", "kmer": "kmer_lut", "bpe": "gpu_bpe"}


def builtin_tokenizer(name: str):
    """Hugging Face tokenizers with the vocabularies of the benchmark shapes (None for other names)."""
    import itertools
    from tokenizers import Regex, Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    if name == "byte":
        core = Tokenizer(models.WordLevel({chr(i): i for i in range(512)}, unk_token=chr(0)))
        core.pre_tokenizer = pre_tokenizers.Split(Regex("[\\s\\S]"), "isolated")
        return PreTrainedTokenizerFast(tokenizer_object=core, pad_token=chr(1), unk_token=chr(0))
    k = int(name[4:]) if name.startswith("kmer") and name[4:].isdigit() else 0
    if name != "char" and not k:
        return None
    words = ["[PAD]", "[UNK]", "[CLS]", "[SEP]", "[MASK]"]
    if k:
        words += ["".join(t) for t in itertools.product("ACGT", repeat=k)]
    words += list("ACGTN")
    core = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="[UNK]"))
    splits = [pre_tokenizers.Split(Regex("."), "isolated")] if not k else \
        [pre_tokenizers.Split(Regex(".{1,%d}" % k), "isolated"), pre_tokenizers.Split(Regex("[ACGT]{%d}|." % k), "isolated")]
    core.pre_tokenizer = pre_tokenizers.Sequence(splits)
    return PreTrainedTokenizerFast(tokenizer_object=core, pad_token="[PAD]", unk_token="[UNK]")


def load_hf(where: str):
    tok = builtin_tokenizer(where)
    if tok is not None:
        return tok
    if os.path.isfile(where):
        from tokenizers import Tokenizer
        from transformers import PreTrainedTokenizerFast
        if where.endswith(".gz"):
            import gzip
            with gzip.open(where, "rt") as f:
                core = Tokenizer.from_str(f.read())
        else:
            core = Tokenizer.from_file(where)
        tok = PreTrainedTokenizerFast(tokenizer_object=core)
        have = tok.get_vocab()
        for attr, names in {"pad_token": ("[PAD]", "<pad>"), "unk_token": ("[UNK]", "<unk>")}.items():
            if getattr(tok, attr) is None:
                hit = next((n for n in names if n in have), None)
                if hit:
                    setattr(tok, attr, hit)
        return tok
    from transformers import AutoTokenizer
    return AutoTokenizer.from_pretrained(where, trust_remote_code=False)


class Session:
    """One Hugging Face tokenizer and the GPU tokenizer built from it."""

    def __init__(self, where: str):
        from .tokenizer import B200Tokenizer
        self.where = where
        self.hf = load_hf(where)
        self.gpu = B200Tokenizer.from_hf(self.hf)
        self.path = PATH_NAME[self.gpu.spec.kind]

    def rows(self, seqs):
        """Content ids of every sequence (no special tokens, no padding) as lists."""
        enc = self.gpu(seqs, add_special_tokens=False, return_attention_mask=False)
        return enc["input_ids"]

    def encode_timed(self, seqs, chunk):
        import torch
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for i in range(0, len(seqs), chunk):
            self.gpu(seqs[i:i + chunk], padding=True, add_special_tokens=False, return_tensors="pt")
        torch.cuda.synchronize()
        return time.perf_counter() - t0

    def hf_timed(self, seqs, chunk):
        t0 = time.perf_counter()
        for i in range(0, len(seqs), chunk):
            self.hf(seqs[i:i + chunk], add_special_tokens=False)
        return time.perf_counter() - t0


def random_windows(n, width, seed):
    rng = np.random.default_rng(seed)
    letters = np.frombuffer(b"ACGT", dtype=np.uint8)[rng.integers(0, 4, size=(n, width))]
    return [row.tobytes().decode("ascii") for row in letters]


def run_info(s: Session, a):
    sp = s.gpu.spec
    return 0, {"tokenizer": s.where, "tokenizer_class": type(s.hf).__name__, "vocab_size": int(s.gpu.vocab_size),
               "selected_path": s.path, "device": str(s.gpu.device), "kmer_k": sp.k or None,
               "has_ascii_lut": sp.kind == "char", "has_gpu_bpe_backend": sp.kind == "bpe",
               "padding_side": s.gpu.padding_side, "id_pad": int(s.gpu.pad_token_id)}


def run_encode(s: Session, a):
    ids = s.rows([a.seq])[0]
    shown = ids if a.json or len(ids) <= 32 else ids[:32] + ["..."]
    return 0, {"tokenizer": s.where, "sequence": a.seq if len(a.seq) <= 80 else a.seq[:80] + "...",
               "sequence_length_bp": len(a.seq), "n_tokens": len(ids), "token_ids": shown, "selected_path": s.path}


def run_validate(s: Session, a):
    seqs = random_windows(a.n, a.window, a.seed)
    want = s.hf(seqs, add_special_tokens=False, padding=False, truncation=False)["input_ids"]
    got = s.rows(seqs)
    bad = [i for i in range(a.n) if list(got[i]) != list(want[i])]
    first = None
    if bad:
        i = bad[0]
        first = {"i": i, "seq_head": seqs[i][:40], "dnatok_head": list(got[i])[:8], "hf_head": list(want[i])[:8]}
    return (1 if bad else 0), {"tokenizer": s.where, "n_sequences": a.n, "n_match": a.n - len(bad), "n_mismatch": len(bad),
                               "match_rate": (a.n - len(bad)) / max(a.n, 1), "selected_path": s.path, "first_mismatch": first}


def run_bench(s: Session, a):
    seqs = random_windows(a.n, a.window, a.seed)
    bp = a.n * a.window
    head = seqs[:min(a.chunk, a.n)]
    s.hf(head, add_special_tokens=False)
    s.gpu(head, padding=True, add_special_tokens=False, return_tensors="pt")
    t_hf, t_gpu = s.hf_timed(seqs, a.chunk), s.encode_timed(seqs, a.chunk)
    return 0, {"tokenizer": s.where, "n_sequences": a.n, "window_bp": a.window, "chunk": a.chunk, "total_bp": bp,
               "hf_threads": a.hf_threads, "hf_time_s": round(t_hf, 4), "hf_mbp_per_s": round(bp / t_hf / 1e6, 2),
               "dnatok_time_s": round(t_gpu, 4), "dnatok_mbp_per_s": round(bp / t_gpu / 1e6, 2),
               "speedup_dnatok_vs_hf": round(t_hf / t_gpu, 2), "selected_path": s.path, "device": str(s.gpu.device)}


def run_scenarios(s: Session, a):
    """Every read-length scenario: ids checked against Hugging Face on a sample of the reads, then the whole
    workload timed in chunks through both."""
    from . import synth
    out, code = {}, 0
    names = a.only.split(",") if a.only else list(synth.SCENARIOS)
    for name in names:
        reads = None if a.reads <= 0 else a.reads
        flat, offsets = synth.scenario(name, reads, a.seed)
        seqs = synth.rows_to_strings(flat, offsets)
        sample = seqs[:: max(1, len(seqs) // max(a.check, 1))][:a.check]
        want = s.hf(sample, add_special_tokens=False)["input_ids"]
        got = s.rows(sample)
        n_bad = sum(list(g) != list(w) for g, w in zip(got, want))
        code = code or (1 if n_bad else 0)
        s.gpu(seqs[:min(a.chunk, len(seqs))], padding=True, add_special_tokens=False, return_tensors="pt")
        t_gpu = s.encode_timed(seqs, a.chunk)
        t_hf = s.hf_timed(seqs, a.chunk) if not a.no_hf else float("nan")
        bp = int(offsets[-1])
        lens = np.diff(offsets)
        out[name] = {"description": synth.SCENARIOS[name][1], "n_reads": len(seqs), "total_bp": bp,
                     "length_min": int(lens.min()), "length_p50": int(np.median(lens)), "length_max": int(lens.max()),
                     "checked": len(sample), "mismatches": int(n_bad), "dnatok_mbp_per_s": round(bp / t_gpu / 1e6, 2),
                     "hf_mbp_per_s": None if a.no_hf else round(bp / t_hf / 1e6, 2),
                     "speedup_dnatok_vs_hf": None if a.no_hf else round(t_hf / t_gpu, 2)}
    return code, {"tokenizer": s.where, "selected_path": s.path, "chunk": a.chunk, "hf_threads": a.hf_threads, "scenarios": out}


COMMANDS = {"info": run_info, "encode": run_encode, "validate": run_validate, "bench": run_bench, "scenarios": run_scenarios}


def parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="dnatok_b200")
    sub = ap.add_subparsers(dest="command", required=True)
    for name in COMMANDS:
        p = sub.add_parser(name)
        p.add_argument("--tokenizer", "--model", dest="tokenizer", required=True)
        p.add_argument("--json", action="store_true")
        if name == "encode":
            p.add_argument("--seq", required=True)
        if name in ("validate", "bench", "scenarios"):
            p.add_argument("--seed", type=int, default=0)
        if name in ("validate", "bench"):
            p.add_argument("--n", type=int, default={"validate": 100, "bench": 1000}[name])
            p.add_argument("--window", type=int, default={"validate": 1024, "bench": 4096}[name])
        if name in ("bench", "scenarios"):
            p.add_argument("--chunk", type=int, default=32)
            p.add_argument("--hf-threads", type=int, default=os.cpu_count() or 1)
        if name == "scenarios":
            p.add_argument("--only", default="", help="comma-separated scenario names (default: all eight)")
            p.add_argument("--reads", type=int, default=0, help="reads per scenario (0: the scenario's own count)")
            p.add_argument("--check", type=int, default=64, help="reads per scenario compared with Hugging Face")
            p.add_argument("--no-hf", action="store_true", help="skip timing the Hugging Face tokenizer")
    return ap


def show(payload, as_json: bool) -> None:
    if as_json:
        print(json.dumps(payload))
        return
    for key, value in payload.items():
        if isinstance(value, dict):
            print(key)
            for k2, v2 in value.items():
                print("  %-18s %s" % (k2, v2))
        else:
            print("%-24s %s" % (key, value))


def main(argv=None) -> int:
    a = parser().parse_args(argv)
    if getattr(a, "hf_threads", None):
        os.environ["RAYON_NUM_THREADS"] = str(a.hf_threads)
        os.environ["TOKENIZERS_PARALLELISM"] = "true" if a.hf_threads > 1 else "false"
    try:
        code, payload = COMMANDS[a.command](Session(a.tokenizer), a)
    except Exception as e:                                   # message and a non-zero exit, like the reference tool
        print("error: %s: %s" % (type(e).__name__, e), file=sys.stderr)
        return 2
    show(payload, a.json)
    return code


if __name__ == "__main__":
    sys.exit(main())

"""Train the two BPE tokenizers of benchmark shapes 3 and 5 and store them as gzip fixtures.

    python tests/golden/train_bpe_fixtures.py [bpe4096] [bpe32000]

Shape 3: vocab 4,096 from a 10,000,000-base order-3 Markov corpus in 1,024-bp lines.
Shape 5: vocab 32,000 from a 50,000,000-base corpus in 10,000-bp records, one GC draw each.
BpeTrainer is deterministic for a fixed corpus; the fixtures remove the need to retrain.
"""
import gzip
import hashlib
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from dnatok_b200 import synth  # noqa: E402
from oracle import hf_oracle  # noqa: E402


def lines_of(a, total):
    flat = a.reshape(-1)[:total].tobytes().decode("ascii")
    n = a.shape[1]
    return [flat[i:i + n] for i in range(0, total, n)]


def main(which):
    for name in which:
        t = time.time()
        if name == "bpe4096":
            lines = lines_of(synth.config3_corpus(), 10_000_000)
            vocab = 4096
        elif name == "bpe32000":
            lines = lines_of(synth.config5_corpus(), 50_000_000)
            vocab = 32000
        else:
            raise SystemExit("unknown fixture " + name)
        t1 = time.time()
        tok = hf_oracle.train_bpe(lines, vocab)
        s = json.dumps(json.loads(tok.to_str()), sort_keys=True, separators=(",", ":"))
        path = os.path.join(HERE, name + ".tokenizer.json.gz")
        with open(path, "wb") as raw, gzip.GzipFile(fileobj=raw, mode="wb", mtime=0) as f:
            f.write(s.encode())
        print(name, "corpus %.1fs train %.1fs" % (t1 - t, time.time() - t1),
              "merges", len(json.loads(s)["model"]["merges"]),
              "sha256", hashlib.sha256(s.encode()).hexdigest(), os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1:] or ["bpe4096", "bpe32000"])

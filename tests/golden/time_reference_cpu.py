"""Time the reference's own CPU path (``DNATok.encode_batch_to_ids``: numpy LUT for single-base and byte
tokenizers, numpy k-mer path for 6-mers) on the synthetic shapes 1, 2 and 4.  Needs a checkout of
eniktab/DNAtok, like ``make_golden.py``:

    DNATOK_REFERENCE_SRC=<checkout>/src python tests/golden/time_reference_cpu.py

Prints one JSON object per shape: rows, base pairs, median seconds of 5 repetitions after 2 warm-ups, Mbp/s,
and the CPU cores of the machine.  The reference runs these paths in one Python thread (numpy).
"""
import json
import os
import statistics
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

import transformers  # noqa: E402,F401  (before the reference's dnatok_compat)

from dnatok_b200 import synth  # noqa: E402
from oracle import hf_oracle  # noqa: E402
from make_golden import _Embedder  # noqa: E402

REF_SRC = os.environ.get("DNATOK_REFERENCE_SRC", "")


def main():
    if not REF_SRC:
        sys.exit("set DNATOK_REFERENCE_SRC to the reference's src/ directory")
    sys.path.insert(0, REF_SRC)
    from dna_tokenizer import DNATok
    toks = {"char": hf_oracle.char_tokenizer(), "kmer6": hf_oracle.kmer_tokenizer(), "byte": hf_oracle.byte_tokenizer()}
    shapes = [("cfg1_char", "char", synth.config1(batch=4096, length=1024)),
              ("cfg2_kmer6", "kmer6", synth.config2(batch=2048, length=6000)),
              ("cfg4_byte", "byte", synth.config4(batch=8, length=1 << 20))]
    for label, tname, rows in shapes:
        strs = [bytes(r).decode("ascii") for r in rows]
        h = DNATok(_Embedder(toks[tname]), padding_side="right")
        h.discover()
        times = []
        for i in range(7):
            t0 = time.perf_counter()
            out = h.encode_batch_to_ids(strs)
            dt = time.perf_counter() - t0
            if i >= 2:
                times.append(dt)
        bp = int(rows.size)
        med = statistics.median(times)
        print(json.dumps({"shape": label, "rows": len(strs), "bp": bp, "out_shape": list(out.shape),
                          "seconds_median": round(med, 4), "Mbp/s": round(bp / med / 1e6, 1),
                          "cpu_cores": os.cpu_count(), "threads": "reference default (numpy, one Python thread)"}))


if __name__ == "__main__":
    main()

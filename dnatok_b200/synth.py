"""Seeded synthetic DNA for the five benchmark shapes.

Real genomic reads and the DNABERT-2 / GENA-LM / NT-v2 / Evo2 tokenizer files are not
available offline, so these generators stand in for them: they take the shapes (read
lengths, N rate, soft-mask rate, GC range) and are fully determined by a seed
(numpy ``default_rng``, PCG64).  Every generator returns ``bytes``-level data
(``uint8`` arrays) so no Python string work sits between the generator and the packer.

Shapes:
  1. char      64 x 1,024 bp, uniform ACGT, each base -> N with p = 0.01
  2. kmer6     256 x 6,000 bp, uniform ACGT, N runs of 1..50 bp until 0.5 % of the batch is N
  3. bpe4k     1,024 x 1,024 bp from an order-3 Markov chain (random transition rows)
  4. byte      8 x 1,048,576 bp, uniform ACGT, 40 % lower-case runs, 0.1 % N
  5. bpe32k    16,384 reads, log-uniform 150..10,000 bp, Markov chain tilted by a per-read GC
"""
from __future__ import annotations

import numpy as np

BASE_SEED = 20260000
_ACGT = np.frombuffer(b"ACGT", dtype=np.uint8)


def seed_for(config: int, stream: int = 0) -> int:
    return BASE_SEED + config + 1000 * stream


def uniform_acgt(rng: np.random.Generator, shape) -> np.ndarray:
    return _ACGT[rng.integers(0, 4, size=shape, dtype=np.uint8)]


def config1(batch: int = 64, length: int = 1024, seed: int | None = None) -> np.ndarray:
    """uint8[batch, length]: uniform ACGT with each position independently N at p=0.01."""
    rng = np.random.default_rng(seed_for(1) if seed is None else seed)
    a = uniform_acgt(rng, (batch, length))
    a[rng.random((batch, length)) < 0.01] = ord("N")
    return a


def config2(batch: int = 256, length: int = 6000, seed: int | None = None) -> np.ndarray:
    """uint8[batch, length]: uniform ACGT plus N runs of 1..50 bp covering >= 0.5 % of the batch."""
    rng = np.random.default_rng(seed_for(2) if seed is None else seed)
    a = uniform_acgt(rng, (batch, length))
    target = int(0.005 * batch * length)
    # Runs are drawn in blocks and applied in order until the N count reaches the target.
    n_now = 0
    while n_now < target:
        k = max(16, (target - n_now) // 20)
        rows = rng.integers(0, batch, size=k)
        runs = rng.integers(1, 51, size=k)
        starts = np.floor(rng.random(k) * (length - runs + 1)).astype(np.int64)
        for b, r, s in zip(rows.tolist(), runs.tolist(), starts.tolist()):
            seg = a[b, s:s + r]
            n_now += int(r - np.count_nonzero(seg == ord("N")))
            seg[:] = ord("N")
            if n_now >= target:
                break
    return a


def markov_rows(rng: np.random.Generator) -> np.ndarray:
    """float64[64, 4]: one Dirichlet(1,1,1,1) transition row per 3-base context."""
    return rng.dirichlet(np.ones(4), size=64)


def _markov_emit(rng: np.random.Generator, cum: np.ndarray, n_seq: int, length: int) -> np.ndarray:
    """Run ``n_seq`` independent order-3 chains for ``length`` steps, vectorised over chains.

    ``cum`` is float64[n_seq or 1, 64, 4] of cumulative transition probabilities.
    """
    out = np.empty((n_seq, length), dtype=np.uint8)
    ctx = rng.integers(0, 64, size=n_seq)
    rows = np.arange(n_seq) if cum.shape[0] == n_seq else np.zeros(n_seq, dtype=np.int64)
    for t in range(length):
        c = cum[rows, ctx]                      # [n_seq, 4]
        u = rng.random(n_seq)
        nxt = (u[:, None] >= c[:, :3]).sum(axis=1)
        out[:, t] = nxt
        ctx = ((ctx << 2) | nxt) & 63
    return _ACGT[out]


def config3_chain(seed: int | None = None) -> np.ndarray:
    rng = np.random.default_rng(seed_for(3, stream=1) if seed is None else seed)
    return markov_rows(rng)


def config3(batch: int = 1024, length: int = 1024, seed: int | None = None,
            chain: np.ndarray | None = None) -> np.ndarray:
    """uint8[batch, length] drawn from the order-3 chain of config 3."""
    P = config3_chain() if chain is None else chain
    rng = np.random.default_rng(seed_for(3) if seed is None else seed)
    cum = np.cumsum(P, axis=1)[None]
    return _markov_emit(rng, cum, batch, length)


def config3_corpus(total: int = 10_000_000, line: int = 1024, seed: int | None = None) -> np.ndarray:
    """Training corpus for the vocab-4,096 BPE: ``total`` bases as lines of ``line`` bp.

    Returned as uint8[n_lines, line]; the last line is cut short by the caller if ``total``
    is not a multiple of ``line``.
    """
    rng = np.random.default_rng(seed_for(3, stream=2) if seed is None else seed)
    n_lines = -(-total // line)
    cum = np.cumsum(config3_chain(), axis=1)[None]
    return _markov_emit(rng, cum, n_lines, line)


def _tilted_cum(P: np.ndarray, gc: np.ndarray) -> np.ndarray:
    """Per-record transition tables: C,G weighted by gc/0.5 and A,T by (1-gc)/0.5, renormalised."""
    w = np.empty((gc.shape[0], 4))
    w[:, 0] = w[:, 3] = (1.0 - gc) / 0.5
    w[:, 1] = w[:, 2] = gc / 0.5
    T = P[None, :, :] * w[:, None, :]
    T /= T.sum(axis=2, keepdims=True)
    return np.cumsum(T, axis=2)


def config5_chain(seed: int | None = None) -> np.ndarray:
    rng = np.random.default_rng(seed_for(5, stream=1) if seed is None else seed)
    return markov_rows(rng)


def config5_lengths(n_reads: int = 16384, seed: int | None = None) -> np.ndarray:
    rng = np.random.default_rng(seed_for(5, stream=3) if seed is None else seed)
    return np.floor(np.exp(rng.uniform(np.log(150.0), np.log(10000.0), size=n_reads))).astype(np.int64)


def config5(n_reads: int = 16384, seed: int | None = None):
    """Ragged reads: returns (bytes uint8[total], offsets int64[n_reads+1])."""
    lens = config5_lengths(n_reads, seed=None if seed is None else seed + 3)
    rng = np.random.default_rng(seed_for(5) if seed is None else seed)
    gc = rng.uniform(0.3, 0.7, size=n_reads)
    cum = _tilted_cum(config5_chain(), gc)
    full = _markov_emit(rng, cum, n_reads, int(lens.max()))
    offsets = np.zeros(n_reads + 1, dtype=np.int64)
    np.cumsum(lens, out=offsets[1:])
    flat = np.empty(int(offsets[-1]), dtype=np.uint8)
    for i in range(n_reads):
        flat[offsets[i]:offsets[i + 1]] = full[i, :lens[i]]
    return flat, offsets


def config5_corpus(total: int = 50_000_000, record: int = 10_000, seed: int | None = None) -> np.ndarray:
    """Training corpus for the vocab-32,000 BPE: uint8[n_records, record], one GC draw per record."""
    rng = np.random.default_rng(seed_for(5, stream=2) if seed is None else seed)
    n_rec = -(-total // record)
    gc = rng.uniform(0.3, 0.7, size=n_rec)
    cum = _tilted_cum(config5_chain(), gc)
    return _markov_emit(rng, cum, n_rec, record)


def config4(batch: int = 8, length: int = 1_048_576, seed: int | None = None) -> np.ndarray:
    """uint8[batch, length]: upper-case ACGT, alternating unmasked / soft-masked (lower-case)
    runs with geometric lengths of mean 450 / 300 bp (40 % lower case), then N at p=0.001."""
    rng = np.random.default_rng(seed_for(4) if seed is None else seed)
    a = uniform_acgt(rng, (batch, length))
    for b in range(batch):
        n_runs = int(length / 750 * 1.3) + 64
        up = rng.geometric(1.0 / 450.0, size=n_runs)
        lo = rng.geometric(1.0 / 300.0, size=n_runs)
        edges = np.cumsum(np.stack([up, lo], axis=1).reshape(-1))
        while edges[-1] < length:  # extremely unlikely; extend deterministically
            more = rng.geometric(1.0 / 375.0, size=64)
            edges = np.concatenate([edges, edges[-1] + np.cumsum(more)])
        mask = np.zeros(length + 1, dtype=np.int8)
        starts = edges[0::2]
        ends = edges[1::2]
        starts = starts[starts < length]
        ends = np.minimum(ends[:starts.shape[0]], length)
        np.add.at(mask, starts, 1)
        np.add.at(mask, ends, -1)
        low = np.cumsum(mask[:length]) > 0
        a[b, low] |= 0x20
    a[rng.random((batch, length)) < 0.001] = ord("N")
    return a


def pack_rows(a: np.ndarray):
    """Equal-length rows -> (flat bytes, int64 offsets)."""
    b, n = a.shape
    return np.ascontiguousarray(a).reshape(-1), np.arange(b + 1, dtype=np.int64) * n


def rows_to_strings(flat: np.ndarray, offsets: np.ndarray) -> list[str]:
    buf = flat.tobytes()
    return [buf[offsets[i]:offsets[i + 1]].decode("ascii") for i in range(len(offsets) - 1)]


# ----------------------------------------------------------------------------- read-length scenarios
# The eight workloads of the reference's realistic benchmark (benchmarks/run_realistic_benchmark.py:184-272)
# as seeded generators: the same names, read counts, length distributions, N rates and base compositions,
# drawn here with numpy (the reference draws with ``random.Random``; the sequences differ, the shapes do not).

SCENARIOS = {
    # name: (reads, description)
    "illumina_short": (5000, "short reads: length ~ Normal(150, 30) clipped to [50, 300]"),
    "pacbio_hifi": (1000, "HiFi long reads: length ~ Normal(15000, 3000) clipped to [5000, 25000]"),
    "nanopore_long": (500, "nanopore reads: length ~ LogNormal(ln 10000, 0.7) clipped to [1000, 100000]"),
    "gene_models": (2000, "gene-length records: log-uniform in [500, 50000]"),
    "mixed_clinical": (2000, "60 % short, 30 % medium (500..5000), 10 % long (~15000) reads, 0.5 % N"),
    "gc_low_20": (2000, "AT-rich genome (20 % GC), 1 kbp reads"),
    "gc_high_65": (2000, "GC-rich genome (65 % GC), 1 kbp reads"),
    "repeats_polyA": (1000, "1 kbp reads each holding a 200-bp poly-A stretch"),
}


def scenario(name: str, n_reads: int | None = None, seed: int = 0):
    """(flat uint8, int64 offsets) of one read-length scenario."""
    if name not in SCENARIOS:
        raise KeyError("unknown scenario %r (one of %s)" % (name, ", ".join(SCENARIOS)))
    n = SCENARIOS[name][0] if n_reads is None else int(n_reads)
    rng = np.random.default_rng(BASE_SEED + 7000 + 17 * list(SCENARIOS).index(name) + seed)
    clip = lambda x, lo, hi: np.clip(np.floor(x), lo, hi).astype(np.int64)
    weights, n_rate = np.full(4, 0.25), 0.0
    if name == "illumina_short":
        lens, n_rate = clip(rng.normal(150, 30, n), 50, 300), 0.001
    elif name == "pacbio_hifi":
        lens = clip(rng.normal(15000, 3000, n), 5000, 25000)
    elif name == "nanopore_long":
        lens, n_rate = clip(rng.lognormal(np.log(10000), 0.7, n), 1000, 100000), 0.002
    elif name == "gene_models":
        lens = clip(np.exp(rng.uniform(np.log(500), np.log(50000), n)), 500, 50000)
    elif name == "mixed_clinical":
        u = rng.random(n)
        lens = np.where(u < 0.60, clip(rng.normal(150, 30, n), 50, 300),
                        np.where(u < 0.90, clip(rng.uniform(500, 5000, n), 500, 5000),
                                 clip(rng.normal(15000, 5000, n), 5000, 30000)))
        n_rate = 0.005
    elif name == "gc_low_20":
        lens, weights = np.full(n, 1000, np.int64), np.array([0.40, 0.10, 0.10, 0.40])
    elif name == "gc_high_65":
        lens, weights = np.full(n, 1000, np.int64), np.array([0.175, 0.325, 0.325, 0.175])
    else:
        lens = np.full(n, 1000, np.int64)
    offsets = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(lens, out=offsets[1:])
    total = int(offsets[-1])
    flat = _ACGT[rng.choice(4, size=total, p=weights).astype(np.uint8)]
    if n_rate > 0:
        flat[rng.random(total) < n_rate] = ord("N")
    if name == "repeats_polyA":
        starts = offsets[:-1] + rng.integers(0, 800, size=n)
        for s in starts.tolist():
            flat[s:s + 200] = ord("A")
    return flat, offsets

"""Sharding by sequence, and the optional gather, as two gloo ranks on CPU."""
import os
import socket

import numpy as np
import pytest

from dnatok_b200 import shard, synth

import helpers as H


def test_partition_contiguous_is_order_preserving_and_balanced():
    rng = np.random.default_rng(0)
    lens = np.floor(np.exp(rng.uniform(np.log(150), np.log(10000), 4096))).astype(np.int64)
    for world in (1, 2, 4, 8):
        parts = shard.partition(lens, world)
        assert np.array_equal(np.concatenate(parts), np.arange(4096))
        loads = np.array([lens[p].sum() for p in parts])
        assert loads.max() <= loads.mean() * 1.02 + 10000
    parts = shard.partition(np.array([5, 5, 5]), 8)
    assert sum(len(p) for p in parts) == 3


def test_partition_greedy_and_restore_order():
    rng = np.random.default_rng(1)
    lens = rng.integers(1, 5000, 1000)
    parts = shard.partition(lens, 4, mode="greedy")
    assert sorted(np.concatenate(parts).tolist()) == list(range(1000))
    loads = np.array([lens[p].sum() for p in parts])
    assert loads.max() - loads.min() <= lens.max()
    full = rng.integers(0, 9, (1000, 7))
    back = shard.restore_order([full[p] for p in parts], parts)
    assert np.array_equal(back, full)


def test_take_rows():
    flat, offs = synth.config5(n_reads=64)
    for rows in (np.arange(10, 20), np.array([3, 9, 50])):
        f, o = shard.take_rows(flat, offs, rows)
        for j, i in enumerate(rows):
            assert np.array_equal(f[o[j]:o[j + 1]], flat[offs[i]:offs[i + 1]])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # every rank encodes its own shard (with the CPU checker standing in for the GPU) and
        # rank 0 gathers; the union must equal the unsharded result
        name, flat, offs = H.config_inputs("cfg3_bpe4096")
        flat, offs = flat[:offs[64]], offs[:65]
        parts = shard.partition(np.diff(offs), world)
        f, o = shard.take_rows(flat, offs, parts[rank])
        ids, _ = H.oracle_batch(name, f, o)
        full_ids, _ = H.oracle_batch(name, flat, offs)
        width = full_ids.shape[1]
        got = shard.gather_padded(torch.from_numpy(ids), [len(p) for p in parts], width, H.spec(name).specials.pad_id)
        if rank == 0:
            q.put(bool(np.array_equal(got.numpy(), full_ids)))
        else:
            assert got is None
    finally:
        dist.destroy_process_group()


def test_two_rank_shard_and_gather_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q.get(timeout=5) is True


def test_split_long_rows_is_exact_for_every_kind():
    """Pieces cut by split_long_rows tokenise to the same ids as the whole rows (CPU checker)."""
    from oracle import oracle
    rng = np.random.default_rng(5)
    for name in ("char", "kmer6", "bpe4096"):
        spec = H.spec(name)
        rows = [synth.config2(batch=1, length=n, seed=n)[0] for n in (50, 7001, 3, 20000)]     # ACGT with N runs
        flat = np.concatenate(rows)
        offs = np.concatenate([[0], np.cumsum([len(r) for r in rows])]).astype(np.int64)
        whole = H.oracle_rows(name, flat, offs)
        for max_bytes in (999, 4096, 100000):
            po, prow = shard.split_long_rows(flat, offs, spec, max_bytes)
            assert po[0] == 0 and po[-1] == offs[-1] and np.all(np.diff(po) >= 0) and len(prow) == len(po) - 1
            assert set(offs.tolist()) <= set(po.tolist())
            if name != "bpe4096":
                assert np.diff(po).max() <= max(max_bytes, 6)
            pieces = H.oracle_rows(name, flat, po)
            out_off = np.concatenate([[0], np.cumsum([len(p) for p in pieces])])
            ids = np.concatenate(pieces) if pieces else np.zeros(0, np.int64)
            ro = shard.join_pieces(out_off, prow, len(rows))
            for r in range(len(rows)):
                assert ids[ro[r]:ro[r + 1]].tolist() == whole[r].tolist(), (name, max_bytes, r)
    # a BPE row with nothing but mergeable symbols has no exact cut and stays whole
    spec = H.spec("bpe4096")
    flat = synth.config3(batch=1, length=5000, seed=1)[0]
    po, prow = shard.split_long_rows(flat, np.array([0, 5000]), spec, 1000)
    assert po.tolist() == [0, 5000] and prow.tolist() == [0]


def _split_rank_main(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # one word of 1,048,576 bp (the byte-level shape's row: 0.1 % N, which the BPE vocabulary does not know)
        # is cut at those N, the pieces are dealt to the ranks, every rank tokenises its pieces (the CPU checker
        # standing in for its GPU) and rank 0 puts the ids together
        name = "bpe4096"
        spec = H.spec(name)
        flat = np.ascontiguousarray(np.char.upper(synth.config4(batch=1, length=1 << 20, seed=3).view("S1")).view(np.uint8)[0])
        offs = np.array([0, flat.size], dtype=np.int64)
        po, prow = shard.split_long_rows(flat, offs, spec, flat.size // (4 * world))
        parts = shard.partition(np.diff(po), world)
        mine = parts[rank]
        f, o = shard.take_rows(flat, po, mine)
        rows = H.oracle_rows(name, f, o)
        ids = np.concatenate(rows).astype(np.int64) if rows else np.zeros(0, np.int64)
        counts = [None] * world
        dist.all_gather_object(counts, int(ids.size))
        buf = torch.zeros(max(counts), dtype=torch.int64)
        buf[:ids.size] = torch.from_numpy(ids)
        bucket = [torch.zeros(max(counts), dtype=torch.int64) for _ in range(world)] if rank == 0 else None
        dist.gather(buf, bucket, dst=0)
        if rank == 0:
            got = np.concatenate([bucket[r][:counts[r]].numpy() for r in range(world)])
            want = H.oracle_rows(name, flat, offs)[0]
            q.put((bool(np.array_equal(got, want)), len(po) - 1, int(np.diff(po).max())))
    finally:
        dist.destroy_process_group()


def test_one_megabase_word_split_over_two_ranks_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_split_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    ok, n_pieces, longest = q.get(timeout=5)
    assert ok and n_pieces >= 8 and longest < (1 << 20) // 4


def test_bind_host_to_gpu_is_harmless_without_nvml():
    """On a machine without a GPU driver the binding helper reports None and leaves the affinity alone."""
    import os
    from dnatok_b200.shard import bind_host_to_gpu
    before = os.sched_getaffinity(0)
    got = bind_host_to_gpu(0)
    assert got is None or set(got) <= before
    if got is None:
        assert os.sched_getaffinity(0) == before
    os.sched_setaffinity(0, before)


def test_read_length_scenarios_have_the_stated_shapes():
    """The eight workloads of the reference's realistic benchmark (benchmarks/run_realistic_benchmark.py:184-272):
    read counts, length ranges, base composition, N rate and the poly-A stretch."""
    from dnatok_b200 import synth
    bounds = {"illumina_short": (50, 300), "pacbio_hifi": (5000, 25000), "nanopore_long": (1000, 100000),
              "gene_models": (500, 50000), "mixed_clinical": (50, 30000), "gc_low_20": (1000, 1000),
              "gc_high_65": (1000, 1000), "repeats_polyA": (1000, 1000)}
    assert list(synth.SCENARIOS) == list(bounds)
    for name, (lo, hi) in bounds.items():
        n = min(synth.SCENARIOS[name][0], 300)
        flat, off = synth.scenario(name, n)
        lens = np.diff(off)
        assert len(lens) == n and lens.min() >= lo and lens.max() <= hi and off[-1] == flat.size
        assert set(np.unique(flat).tolist()) <= set(b"ACGTN")
        f2, o2 = synth.scenario(name, n)
        assert np.array_equal(flat, f2) and np.array_equal(off, o2)          # seeded
    gc = lambda f: np.isin(f, np.frombuffer(b"CG", np.uint8)).mean()
    assert abs(gc(synth.scenario("gc_low_20", 200)[0]) - 0.20) < 0.02
    assert abs(gc(synth.scenario("gc_high_65", 200)[0]) - 0.65) < 0.02
    flat, off = synth.scenario("repeats_polyA", 50)
    for i in range(50):
        row = flat[off[i]:off[i + 1]].tobytes()
        assert b"A" * 200 in row
    assert synth.scenario("mixed_clinical", 400)[0].tolist().count(ord("N")) > 0
    with pytest.raises(KeyError):
        synth.scenario("nope")


def test_native_packer_matches_join_encode():
    """dnatok_b200._pack against the Python packing it replaces, with translation, padding and truncation."""
    from dnatok_b200.pack import pack_sizes, pack_strings
    rng = np.random.default_rng(3)
    seqs = ["".join(rng.choice(list("ACGTNacgtn"), size=int(n))) for n in rng.integers(0, 400, size=300)]
    flat, off = pack_strings(seqs)
    assert flat.tobytes() == "".join(seqs).encode() and off.tolist() == np.concatenate([[0], np.cumsum([len(s) for s in seqs])]).tolist()
    assert pack_sizes(seqs) == flat.size
    mixed = [s.encode() if i % 3 == 0 else s for i, s in enumerate(seqs)]
    assert pack_strings(mixed)[0].tobytes() == flat.tobytes()
    upper = bytes((c - 32 if 97 <= c <= 122 else c) for c in range(256))
    assert pack_strings(seqs, table=upper)[0].tobytes() == "".join(seqs).upper().encode()
    f2, o2 = pack_strings(seqs, pad_to=120, trunc_to=200, pad_left=True)
    want = [s[:200].rjust(120, "N") for s in seqs]
    assert f2.tobytes() == "".join(want).encode() and o2[-1] == sum(map(len, want))
    f3, _ = pack_strings(seqs, pad_to=64, pad_byte=ord("-"))
    assert f3.tobytes() == "".join(s.ljust(64, "-") for s in seqs).encode()
    big = ["ACGT" * 3000] * 1500                                              # 18 MB: the threaded copy
    assert pack_strings(big)[0].tobytes() == ("ACGT" * 3000 * 1500).encode()
    assert pack_strings([])[0].size == 0
    with pytest.raises(ValueError):
        pack_strings(["AC\u00e9"])
    with pytest.raises(TypeError):
        pack_strings([7])
    with pytest.raises(ValueError):
        pack_strings(seqs, out=np.empty(3, np.uint8))

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

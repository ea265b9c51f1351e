#!/usr/bin/env python
"""Benchmark of the tokenisation hot path: Mbp/s encoded, bit-exact vs Hugging Face.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload kmer6|char|byte|bpe4k|bpe32k] [--scale S] [--no-extra]

One "step" is one pass of the hot path over one batch of seeded synthetic DNA.  The headline
workload is benchmark shape 2 (non-overlapping 6-mers, rows of 6,000 bp, right-padded to 1,000
tokens, int64 ids + int64 mask) scaled to 32,768 rows so that a step moves ~0.7 GB, far more
than the 126 MB L2.  ``value`` is measured with inputs resident in HBM (CUDA events on the
launching stream); ``e2e`` goes through ``dnatok_encode_host`` with pinned HOST buffers, so both
PCIe copies are inside the timed region.  ``per_config`` carries the other four shapes, each at
its literal size (launch-latency bound) and at a scaled size.

Multi-GPU (launched with torch.distributed.run): rows are sharded by sequence, every rank encodes
its own shard on its own GPU with no collective in the timed region (weak scaling: the per-GPU
shard has the single-GPU size); rank 0 prints max-over-ranks timing.

``--impl reference`` times the CPU side of the same workload on a bounded sample: the C
restatement in ``oracle/`` on all host threads (the line's value) and the live Hugging Face
``tokenizers`` call next to it.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from dnatok_b200 import synth  # noqa: E402

L2_BYTES = 126 * 1024 * 1024


# ----------------------------------------------------------------------------- workloads

def fixture_json(name):
    import gzip
    with gzip.open(os.path.join(ROOT, "tests", "golden", name + ".tokenizer.json.gz"), "rt") as f:
        return json.load(f)


def spec_for(kind):
    """Tables for the five shapes without touching Hugging Face (the product path)."""
    import itertools
    from dnatok_b200.tables import Specials, TokenizerSpec, bpe_spec_from_json
    if kind == "char":
        lut = np.full(256, 1, np.int32)
        for i, c in enumerate("ACGTN"):
            lut[ord(c)] = 5 + i
        return TokenizerSpec("char", Specials(0, 1, 2, 3), 10, lut)
    if kind == "byte":
        return TokenizerSpec("char", Specials(1, 0, -1, -1), 512, np.arange(256, dtype=np.int32))
    if kind == "kmer6":
        lut = np.full(256, 1, np.int32)
        for i, c in enumerate("ACGTN"):
            lut[ord(c)] = 4101 + i
        return TokenizerSpec("kmer", Specials(0, 1, -1, -1), 4106, lut, k=6,
                             kmer_ids=np.arange(5, 5 + 4096, dtype=np.int32))
    if kind == "bpe4k":
        return bpe_spec_from_json(fixture_json("bpe4096"))
    if kind == "bpe32k":
        return bpe_spec_from_json(fixture_json("bpe32000"))
    raise KeyError(kind)


def make_workload(kind, scale, seed_shift=0):
    """(flat uint8, offsets int64, call kwargs, description)."""
    if kind == "kmer6":
        rows = 256 * scale
        a = synth.config2(batch=rows, seed=synth.seed_for(2) + seed_shift)
        f, o = synth.pack_rows(a)
        return f, o, dict(padding="max_length", max_length=1000, truncation=True, add_special_tokens=False), \
            "cfg2 6-mer, %d x 6000 bp, pad to 1000, int64 ids+mask" % rows
    if kind == "char":
        rows = 64 * scale
        f, o = synth.pack_rows(synth.config1(batch=rows, seed=synth.seed_for(1) + seed_shift))
        return f, o, dict(padding="longest"), "cfg1 char, %d x 1024 bp, [CLS]..[SEP], int64 ids+mask" % rows
    if kind == "byte":
        rows = 8 * scale
        f, o = synth.pack_rows(synth.config4(batch=rows, seed=synth.seed_for(4) + seed_shift))
        return f, o, dict(padding="longest", ids_dtype="int32", return_attention_mask=False), \
            "cfg4 byte-level, %d x 1048576 bp, int32 ids" % rows
    if kind == "bpe4k":
        rows = 1024 * scale
        f, o = synth.pack_rows(synth.config3(batch=rows, seed=synth.seed_for(3) + seed_shift))
        return f, o, dict(padding="longest"), "cfg3 BPE vocab 4096, %d x 1024 bp, [CLS]..[SEP], pad to longest" % rows
    if kind == "bpe32k":
        f, o = synth.config5(n_reads=16384, seed=None if seed_shift == 0 else synth.seed_for(5) + seed_shift)
        if scale > 1:
            lens = np.diff(o)
            f = np.tile(f, scale)
            o = np.concatenate([[0], np.cumsum(np.tile(lens, scale))]).astype(np.int64)
        return f, o, dict(padding=False), "cfg5 BPE vocab 32000, %d reads 150..10000 bp, ragged ids" % (16384 * scale)
    raise KeyError(kind)


def algorithmic_bytes(total_in, n_rows, enc, ragged):
    """Input ASCII + (ragged only) offsets + every element of the returned ids / mask tensors."""
    b = int(total_in)
    if ragged:
        b += 8 * (n_rows + 1)
    for k in ("input_ids", "attention_mask"):
        if k in enc:
            b += enc[k].numel() * enc[k].element_size()
    return b


# ----------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples SM clock and throttle reasons with NVML while the timed region runs (read only)."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz, self._stop = [], set(), None, threading.Event()
        self.ok = False
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            pass

    def _names(self, bits):
        nv = self.nv
        table = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        return [k for k, v in table.items() if bits & v]

    def _one(self):
        try:
            self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
            get = getattr(self.nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                self.nv.nvmlDeviceGetCurrentClocksThrottleReasons
            self.reasons.update(self._names(get(self.h)))
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self._one()
            time.sleep(0.02)

    def __enter__(self):
        if self.ok:
            self.t = threading.Thread(target=self._run, daemon=True)
            self.t.start()
        return self

    def __exit__(self, *a):
        if self.ok:
            self._one()
            self._stop.set()
            self.t.join()

    def summary(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------- GPU arm

def torch_dtype(name):
    import torch
    return getattr(torch, name)


def device_kwargs(call):
    kw = dict(call)
    if "ids_dtype" in kw:
        kw["ids_dtype"] = torch_dtype(kw["ids_dtype"])
    return kw


KMER_NO_SCRATCH = False     # --kmer-no-scratch: time the k-mer kernel that encodes one row per warp


def time_device(tok, d_bytes, d_off, offsets, call, steps, warmup, barrier=None):
    """CUDA-event timing of ``steps`` encodes with inputs resident on the device.  Outputs and scratch
    are allocated once (first warm-up) and reused, so the timed region launches kernels only."""
    import torch
    from dnatok_b200 import _cabi
    kw = device_kwargs(call)
    ragged = kw.get("padding") is False
    enc = tok.encode_device(d_bytes, d_off, host_offsets=offsets, **kw)          # sizes + correctness of the call
    out = {k: enc[k] for k in ("input_ids", "attention_mask") if k in enc}
    need = _cabi.lib().dnatok_scratch_bytes(tok.handle.ptr, len(offsets) - 1, int(d_bytes.shape[0]))
    scratch = torch.empty(max(need, 1), dtype=torch.uint8, device=d_bytes.device)
    if not ragged and kw.get("padding") == "longest":
        # the stride is known now; later steps use it directly so no host sync sits in the loop
        kw = dict(kw, padding="max_length", max_length=int(enc["input_ids"].shape[1]))
    if KMER_NO_SCRATCH and tok.spec.kind == "kmer":
        scratch = False
    run = lambda: tok.encode_device(d_bytes, d_off, host_offsets=offsets, out=out, scratch=scratch, check=False, **kw)
    if ragged:
        run = make_ragged_runner(tok, d_bytes, d_off, offsets, kw, scratch, enc)
    for _ in range(warmup):
        run()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    # one pair of events around the K steps, on the stream the kernels are launched on: events between
    # the steps would put a few microseconds of idle time after every launch of a 0.15 ms kernel
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    l0 = _cabi.lib().dnatok_launch_count()
    ev0.record()
    for _ in range(steps):
        run()
    ev1.record()
    torch.cuda.synchronize()
    launches = _cabi.lib().dnatok_launch_count() - l0
    if barrier:
        barrier()
    total_ms = ev0.elapsed_time(ev1)
    per = np.full(steps, total_ms / steps)           # mean duration of a step, launch gaps included
    time_device.last_run = run
    return enc, per, total_ms, launches


def time_graph(run, reps=20, replays=10):
    """Kernel-only time of a launch-latency-bound shape: `reps` encodes captured in one CUDA graph,
    replayed `replays` times; returns ms per encode, or None when capture is not possible."""
    import torch
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            run()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                run()
        g.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(replays):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (reps * replays)
    except Exception:
        torch.cuda.synchronize()
        return None


def make_ragged_runner(tok, d_bytes, d_off, offsets, kw, scratch, enc):
    """Ragged output with preallocated buffers through the C ABI directly (no host sync per step)."""
    import torch
    from dnatok_b200 import _cabi
    L = _cabi.lib()
    B = len(offsets) - 1
    total = int(d_bytes.shape[0])
    fmt = tok._format(id_bits=64, mask_bits=0, add_special=kw.get("add_special_tokens", True), max_tokens=0, out_stride=0)
    bound = L.dnatok_max_tokens(tok.handle.ptr, B, total, ctypes.byref(fmt))
    ids = torch.empty(bound, dtype=torch.int64, device=d_bytes.device)
    out_off = torch.empty(B + 1, dtype=torch.int64, device=d_bytes.device)
    lengths = torch.empty(B, dtype=torch.int32, device=d_bytes.device)
    status = torch.empty(B, dtype=torch.int32, device=d_bytes.device)
    p = lambda t: ctypes.c_void_p(t.data_ptr())

    def run():
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        _cabi.check(L.dnatok_encode(tok.handle.ptr, p(d_bytes), p(d_off), B, total, ctypes.byref(fmt), p(ids), None,
                                    p(lengths), p(out_off), p(status), p(scratch), int(scratch.numel()), stream))
    return run


def time_e2e(tok, flat, offsets, call, steps, warmup):
    """Host buffers in, host buffers out, through dnatok_encode_host; wall clock (the call returns
    when the results are in host memory)."""
    import torch
    kw = dict(call)
    ids_dt = np.dtype(kw.pop("ids_dtype", "int64"))
    pin = lambda a: torch.from_numpy(a).pin_memory().numpy()
    flat_p, off_p = pin(np.ascontiguousarray(flat)), pin(offsets)
    first = tok.encode_host((flat_p, off_p), ids_dtype=ids_dt, **kw)
    n_ids = first["input_ids"].size
    out_ids = torch.empty(max(n_ids, 1) if kw.get("padding") is not False else int(offsets[-1]) + 2 * len(offsets),
                          dtype=torch_dtype(ids_dt.name)).pin_memory().numpy()
    out_mask = torch.empty(max(n_ids, 1), dtype=torch.int64).pin_memory().numpy() if "attention_mask" in first else None
    for _ in range(max(warmup - 1, 0)):
        tok.encode_host((flat_p, off_p), ids_dtype=ids_dt, out_ids=out_ids, out_mask=out_mask, **kw)
    t0 = time.perf_counter()
    for _ in range(steps):
        r = tok.encode_host((flat_p, off_p), ids_dtype=ids_dt, out_ids=out_ids, out_mask=out_mask, **kw)
    dt = time.perf_counter() - t0
    # bytes the library itself counted for the last call (a large mask is written by host threads
    # from the row lengths and does not cross the link)
    import ctypes
    from dnatok_b200 import _cabi
    a, b = ctypes.c_int64(0), ctypes.c_int64(0)
    _cabi.lib().dnatok_host_copy_bytes(ctypes.byref(a), ctypes.byref(b))
    return dt / steps, int(a.value), int(b.value)


def pcie_probe(mb=256, reps=5):
    """Host link measurement with pinned buffers and plain asynchronous copies: host->device alone,
    device->host alone, and both at once on two streams.  Prints one JSON line."""
    import torch
    n = mb << 20
    h_in = torch.empty(n, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(n, dtype=torch.uint8).pin_memory()
    d_in = torch.empty(n, dtype=torch.uint8, device="cuda")
    d_out = torch.empty(n, dtype=torch.uint8, device="cuda")
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()

    def run(h2d, d2h):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            if h2d:
                with torch.cuda.stream(s1):
                    d_in.copy_(h_in, non_blocking=True)
            if d2h:
                with torch.cuda.stream(s2):
                    h_out.copy_(d_out, non_blocking=True)
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / reps

    run(True, True)
    t_in, t_out, t_both = run(True, False), run(False, True), run(True, True)

    # the host's own memory beside the link: T threads copying between ordinary arrays (numpy releases the
    # interpreter lock), alone and while both link copies run.  A copy of x bytes reads x and writes x.
    import threading
    T = min(16, len(os.sched_getaffinity(0)))
    src = np.ones(n, dtype=np.uint8)
    dst = np.empty(n, dtype=np.uint8)
    cuts = [n * i // T for i in range(T + 1)]

    def host_copy(stop_at):
        done = [0] * T

        def work(i):
            while time.perf_counter() < stop_at:
                np.copyto(dst[cuts[i]:cuts[i + 1]], src[cuts[i]:cuts[i + 1]])
                done[i] += cuts[i + 1] - cuts[i]
        th = [threading.Thread(target=work, args=(i,)) for i in range(T)]
        for t in th:
            t.start()
        return th, done

    window = 0.25
    t0 = time.perf_counter()
    th, done = host_copy(t0 + window)
    for t in th:
        t.join()
    copy_alone = sum(done) / (time.perf_counter() - t0)
    t0 = time.perf_counter()
    th, done = host_copy(t0 + window)
    link_bytes = 0
    while time.perf_counter() < t0 + window:
        run(True, True)
        link_bytes += 2 * n * reps
    t_link = time.perf_counter() - t0
    for t in th:
        t.join()
    t_all = time.perf_counter() - t0
    print(json.dumps({"probe": "pcie", "mb_each_way": mb, "h2d_GB/s": round(n / t_in / 1e9, 1),
                      "d2h_GB/s": round(n / t_out / 1e9, 1), "both_ms": round(t_both * 1e3, 2),
                      "serial_ms": round((t_in + t_out) * 1e3, 2),
                      "duplex_GB/s_total": round(2 * n / t_both / 1e9, 1),
                      "duplex_over_serial": round((t_in + t_out) / t_both, 2),
                      "host_copy_threads": T, "host_copy_alone_GB/s": round(copy_alone / 1e9, 1),
                      "with_both_link_copies": {"link_GB/s_total": round(link_bytes / t_link / 1e9, 1),
                                                "host_copy_GB/s": round(sum(done) / t_all / 1e9, 1)},
                      "note": "host_copy figures are bytes copied per second; the memory traffic is twice that "
                              "(three times with the write-allocate reads)"}))


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def run_ours(args):
    import torch
    from dnatok_b200.tokenizer import B200Tokenizer
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the encode path has no CPU fallback")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    cores, all_cores = None, os.sched_getaffinity(0)
    if not args.no_affinity:
        from dnatok_b200.shard import bind_host_to_gpu
        cores = bind_host_to_gpu(local)          # before any pinned buffer is allocated
    if world > 1:
        # the ranks of one host share its cores: the threads that write attention masks are divided among them
        from dnatok_b200 import _cabi
        local_world = int(os.environ.get("LOCAL_WORLD_SIZE", str(world)))
        # (the stores bypass the cache, so a few threads per rank keep up with the copy; the mask never crosses the link)
        per_rank = min(4, max(2, len(all_cores) // max(local_world, 1)))
        if os.environ.get("DNATOK_HOST_MASK_THREADS") is not None:
            per_rank = int(os.environ["DNATOK_HOST_MASK_THREADS"])
        _cabi.check(_cabi.lib().dnatok_set_option(b"host_mask_threads", per_rank))
    barrier = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        barrier = lambda: (dist.barrier(), torch.cuda.synchronize())

    peak, peak_src = peaks()
    kind = args.workload
    scale = args.scale or {"kmer6": 128, "char": 1024, "byte": 16, "bpe4k": 64, "bpe32k": 2}[kind]
    tok = B200Tokenizer(spec_for(kind), device=local)
    flat, offsets, call, desc = make_workload(kind, scale, seed_shift=7919 * rank)
    d_bytes = torch.from_numpy(flat).cuda()
    d_off = torch.from_numpy(offsets).cuda()
    total_bp = int(offsets[-1])

    with ClockSampler(local) as clk:
        enc, per, total_ms, launches = time_device(tok, d_bytes, d_off, offsets, call, args.steps, args.warmup, barrier)
    ragged = call.get("padding") is False
    abytes = algorithmic_bytes(total_bp, len(offsets) - 1, enc, ragged)

    # end to end through the host-buffer entry point (rank-local; max over ranks below)
    if args.kernel_only:
        e2e_s, h2d, d2h = float("nan"), 0, 0
    else:
        e2e_s, h2d, d2h = time_e2e(tok, flat, offsets, call, max(3, min(args.steps, 10)), 2)
    os.sched_setaffinity(0, all_cores)           # the CPU baseline below may use every core again

    t = torch.tensor([total_ms, e2e_s], dtype=torch.float64, device="cuda")
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_s = float(t[0]), float(t[1])
    ms_per_step = total_ms / args.steps
    value = world * total_bp / (ms_per_step * 1e-3) / 1e6
    kernel_ms = float(np.mean(per))
    achieved = abytes / (kernel_ms * 1e-3) / 1e9

    line = {
        "metric": "Mbp/s encoded (bit-exact vs HF)", "value": round(value, 1), "unit": "Mbp/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8",
        "data": "synthetic (seeded; stands in for genomic reads and the NT-v2 tokenizer)",
        "config": {"workload": desc, "rows_per_gpu": len(offsets) - 1, "bp_per_gpu": total_bp,
                   "l2": "inputs+outputs per step (%.0f MB) exceed the 126 MB L2; no flush" % (abytes / 1e6)
                   if abytes > 2 * L2_BYTES else "working set fits L2",
                   "sharding": "by sequence, no collective in the timed region"},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 4), "traffic": None, "peak_source": peak_src,
                     "kernel": {"kmer6": "kmer_warp_rows_kernel", "char": "emit_padded_kernel", "byte": "emit_padded_kernel",
                                "bpe4k": "bpe_lanes_st_kernel", "bpe32k": "bpe_mixed_kernel"}[kind],
                     "algorithmic_bytes_per_launch": abytes, "kernel_ms": round(kernel_ms, 5)},
        "e2e": {"value": round(world * total_bp / e2e_s / 1e6, 1), "unit": "Mbp/s",
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "path": "dnatok_encode_host, pinned host buffers; the mask of a large padded batch is written by host "
                        "threads from the GPU's row lengths instead of crossing the link (bytes as counted by the library)",
                "host_cores": "as given" if not cores or len(cores) == len(all_cores)
                else "%d of %d, those next to the GPU" % (len(cores), len(all_cores))},
        "gpu_launches": int(launches), "clocks": clk.summary(),
    }
    if args.kernel_only:
        line["e2e"] = None
    if rank == 0 and world == 1 and not args.kernel_only:
        line["roofline"]["traffic"] = TRAFFIC.get(kind)
        line["cpu_baseline"] = cpu_baseline(kind, 1)
        if not args.no_extra:
            line["per_config"] = per_config(local, peak, args)
    if world > 1 and args.gather and "input_ids" in enc and enc["input_ids"].dim() == 2:
        # optional step, not part of the metric: bring every rank's padded ids to rank 0 over NCCL
        import torch.distributed as dist
        from dnatok_b200 import shard
        ids = enc["input_ids"]
        rows = [int(ids.shape[0])] * world
        shard.gather_padded(ids, rows, int(ids.shape[1]), tok.pad_token_id)          # warm-up
        torch.cuda.synchronize(); dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        got = shard.gather_padded(ids, rows, int(ids.shape[1]), tok.pad_token_id)
        b.record(); torch.cuda.synchronize()
        gt = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device="cuda")
        dist.all_reduce(gt, op=dist.ReduceOp.MAX)
        if rank == 0:
            ok = bool(torch.equal(got[:ids.shape[0]], ids))
            line["gather"] = {"ms": round(float(gt[0]), 3), "bytes_to_rank0": int(ids.numel() * ids.element_size() * (world - 1)),
                              "rank0_rows_ok": ok, "backend": "nccl"}
    if world > 1 and not args.no_extra:
        strong = strong_scaling(local, rank, world, peak)
        if rank == 0:
            line["strong_scaling"] = strong
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def strong_scaling(local, rank, world, peak):
    """Fixed total work split over the ranks (the other lines are weak scaling): the byte-level shape x16
    (128 rows of 1 Mbp, contiguous blocks) and the read set x2 (32,768 reads, longest-first bins).  Every rank
    builds the same seeded batch, takes its rows with shard.partition / take_rows and encodes them; the time is
    the max over ranks.  Outside the timed region rank 0 encodes the whole batch alone and compares every row's
    token count and id sum with what the ranks report, put back in order."""
    import torch
    import torch.distributed as dist
    from dnatok_b200 import shard
    from dnatok_b200.tokenizer import B200Tokenizer
    out = {}
    for kind, scale, mode in (("byte", 16, "contiguous"), ("bpe32k", 2, "greedy")):
        tok = B200Tokenizer(spec_for(kind), device=local)
        flat, offsets, call, desc = make_workload(kind, scale)
        parts = shard.partition(np.diff(offsets), world, mode=mode)
        f, o = shard.take_rows(flat, offsets, parts[rank])
        d_bytes, d_off = torch.from_numpy(np.ascontiguousarray(f)).cuda(), torch.from_numpy(o).cuda()
        barrier = lambda: (dist.barrier(), torch.cuda.synchronize())
        steps = 10
        enc, per, total_ms, launches = time_device(tok, d_bytes, d_off, o, call, steps, 3, barrier)
        t = torch.tensor([total_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0]) / steps

        def row_sums(e, n_rows):
            ids = e["input_ids"]
            if "offsets" in e:
                oo = e["offsets"]
                csum = torch.cat([torch.zeros(1, dtype=torch.int64, device=ids.device), torch.cumsum(ids, 0)])
                return (oo[1:] - oo[:-1]).cpu().numpy(), (csum[oo[1:]] - csum[oo[:-1]]).cpu().numpy()
            return e["lengths"].cpu().numpy().astype(np.int64), ids.sum(dim=1).cpu().numpy()
        mine = row_sums(enc, len(o) - 1)
        everyone = [None] * world
        dist.all_gather_object(everyone, (parts[rank], mine[0], mine[1]))
        ok = None
        if rank == 0:
            full = tok.encode_device(torch.from_numpy(flat).cuda(), torch.from_numpy(offsets).cuda(), host_offsets=offsets,
                                     **device_kwargs(call))
            want = row_sums(full, len(offsets) - 1)
            counts = np.zeros(len(offsets) - 1, np.int64)
            sums = np.zeros(len(offsets) - 1, np.int64)
            for rows, c, sm in everyone:
                counts[rows], sums[rows] = c, sm
            ok = bool(np.array_equal(counts, want[0]) and np.array_equal(sums, want[1]))
            del full
        out["%s/x%d" % (kind, scale)] = {"workload": desc, "partition": mode, "ms_per_step": round(ms, 5),
                                       "Mbp/s": round(int(offsets[-1]) / ms / 1e3, 1), "rows_per_rank": [int(len(p)) for p in parts],
                                       "bp_per_rank_max": int(max(np.diff(offsets)[p].sum() for p in parts)),
                                       "rows_equal_single_gpu": ok, "scaling": "strong"}
        del d_bytes, d_off, enc
        torch.cuda.empty_cache()
    return out


# dram bytes per launch of the dominant kernel from the committed ncu summaries (profiles/), scaled to
# the default workload where the capture ran on a smaller case; None until a capture exists.
TRAFFIC = {"kmer6": 665.6e6, "char": 1085.3e6}


def per_config(local, peak, args):
    """The other shapes: literal size (latency bound, many launches timed) and a scaled size."""
    import torch
    from dnatok_b200.tokenizer import B200Tokenizer
    out = {}
    plan = [("char", 1, 1024), ("kmer6", 1, None), ("bpe4k", 1, 32), ("byte", 1, 16), ("bpe32k", 1, None)]
    for kind, lit, big in plan:
        tok = B200Tokenizer(spec_for(kind), device=local)
        for label, sc in (("literal", lit), ("scaled", big)):
            if sc is None or (kind == args.workload and label == "scaled"):
                continue
            flat, offsets, call, desc = make_workload(kind, sc)
            d_bytes, d_off = torch.from_numpy(flat).cuda(), torch.from_numpy(offsets).cuda()
            steps = 50 if label == "literal" else 10
            enc, per, total_ms, launches = time_device(tok, d_bytes, d_off, offsets, call, steps, 3)
            ragged = call.get("padding") is False
            if ragged:
                n_tok = int(enc["offsets"][-1].item())
                ab = int(offsets[-1]) + 8 * len(offsets) + 8 * n_tok
            else:
                ab = algorithmic_bytes(int(offsets[-1]), len(offsets) - 1, enc, False)
            ms = total_ms / steps
            gms = time_graph(time_device.last_run) if label == "literal" else None
            out["%s/%s" % (kind, label)] = {
                "graph_replay_ms_per_step": None if gms is None else round(gms, 5),
                "graph_replay_Mbp/s": None if gms is None else round(int(offsets[-1]) / gms / 1e3, 1),
                "workload": desc, "ms_per_step": round(ms, 5), "Mbp/s": round(int(offsets[-1]) / ms / 1e3, 1),
                "algorithmic_GB/s": round(ab / ms / 1e6, 1), "frac_of_hbm_peak": round(ab / ms / 1e6 / peak, 4),
                "launches_per_step": launches // steps}
            del d_bytes, d_off, enc
            torch.cuda.empty_cache()
    out["embed_char/scaled"] = embed_line(local, peak)
    out["kmer6/list_str"] = list_str_line(local)
    return out


def list_str_line(local):
    """From a Python list of str to ids + mask tensors on the device through the call a user makes
    (``tok(seqs, ...)``): native packing into pinned memory, one copy in, the kernel.  Wall clock."""
    import torch
    from dnatok_b200.tokenizer import B200Tokenizer
    tok = B200Tokenizer(spec_for("kmer6"), device=local)
    flat, offsets, call, desc = make_workload("kmer6", 32)
    strs = synth.rows_to_strings(flat, offsets)
    kw = dict(padding="max_length", max_length=1000, truncation=True, add_special_tokens=False, return_tensors="pt")
    for _ in range(3):
        tok(strs, **kw)
    torch.cuda.synchronize()
    steps = 10
    t0 = time.perf_counter()
    for _ in range(steps):
        enc = tok(strs, **kw)
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / steps
    t0 = time.perf_counter()
    "".join(strs).encode("ascii")
    t_join = time.perf_counter() - t0
    return {"workload": "list of %d str x 6000 bp -> int64 ids + mask on the device (tok(seqs, ...))" % len(strs),
            "ms_per_step": round(dt * 1e3, 3), "Mbp/s": round(int(offsets[-1]) / dt / 1e6, 1),
            "python_join_encode_ms": round(t_join * 1e3, 3),
            "note": "python_join_encode_ms is the packing step alone as the reference does it (\"\".join(seqs).encode)"}


def embed_line(local, peak):
    """Fused tokenise -> embedding gather (char shape, 4,096 x 1,024 bp, 256-wide bf16 rows): ids never stored."""
    import torch
    from dnatok_b200.tokenizer import B200Tokenizer
    tok = B200Tokenizer(spec_for("char"), device=local)
    flat, offsets, call, desc = make_workload("char", 64)
    d_bytes, d_off = torch.from_numpy(flat).cuda(), torch.from_numpy(offsets).cuda()
    weight = torch.randn((10, 256), device="cuda").to(torch.bfloat16).contiguous()
    first = tok.embed_device(d_bytes, d_off, weight, host_offsets=offsets, padding="longest")
    buf = first["embeddings"]
    stride = int(buf.shape[1])
    run = lambda: tok.embed_device(d_bytes, d_off, weight, host_offsets=offsets, padding="max_length", max_length=stride, out=buf)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    steps = 10
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in ev:
        a.record(); run(); b.record()
    torch.cuda.synchronize()
    ms = float(np.mean([a.elapsed_time(b) for a, b in ev]))
    ab = int(offsets[-1]) + buf.numel() * buf.element_size()
    return {"workload": "char tokenise + gather of 256-wide bf16 rows, %d x 1024 bp" % (len(offsets) - 1),
            "ms_per_step": round(ms, 5), "Mbp/s": round(int(offsets[-1]) / ms / 1e3, 1),
            "algorithmic_GB/s": round(ab / ms / 1e6, 1), "frac_of_hbm_peak": round(ab / ms / 1e6 / peak, 4),
            "launches_per_step": 1}


# ----------------------------------------------------------------------------- CPU arm

def cpu_sample(kind):
    """A bounded sample of the workload: ~10-30 s of CPU work in total."""
    scale = {"kmer6": 64, "char": 64, "byte": 1, "bpe4k": 16, "bpe32k": 1}[kind]
    flat, offsets, call, desc = make_workload(kind, scale)
    if kind == "bpe32k":
        n = 4096
        flat, offsets = flat[:offsets[n]], offsets[:n + 1].copy()
        desc = "first 4096 reads of cfg5"
    return flat, offsets, call, desc


def cpu_baseline(kind, reps=1):
    """The C restatement (oracle/, all host threads) and live Hugging Face tokenizers on a bounded
    sample of the same workload, on this box's host cores."""
    from oracle import oracle as orc
    from dnatok_b200.tables import TokenizerSpec
    flat, offsets, call, desc = cpu_sample(kind)
    spec = spec_for(kind)
    threads = os.cpu_count() or 1
    table = orc.BpeTable(spec.merge_a, spec.merge_b, spec.merge_out) if spec.kind == "bpe" else None
    pad = call.get("padding")
    best = None
    for _ in range(1 + reps):
        t0 = time.perf_counter()
        ids, counts = orc.encode_ragged(spec.kind, flat, offsets, lut256=spec.lut256, k=spec.k, kmer_ids=spec.kmer_ids,
                                        table=table, threads=threads)
        if pad is not False:     # the padded int64 ids + mask the GPU path also produces
            sp = spec.specials
            orc.assemble(orc.rows(ids, offsets, counts), pad_id=sp.pad_id, cls_id=sp.cls_id, sep_id=sp.sep_id,
                         add_special=call.get("add_special_tokens", True), max_length=call.get("max_length", 0) or 0,
                         truncation=call.get("truncation", False), padding=pad)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    res = {"value": round(int(offsets[-1]) / best / 1e6, 2), "unit": "Mbp/s", "cores": threads, "kind": "port",
           "sample": "%s: %d rows, %.1f Mbp" % (desc, len(offsets) - 1, offsets[-1] / 1e6),
           "what": "oracle/dnatok_oracle.c (pthreads) + numpy padding/mask assembly"}
    res["hf_tokenizers"] = hf_baseline(kind, flat, offsets, call)
    return res


def hf_baseline(kind, flat, offsets, call):
    """Live Hugging Face fast tokenizer on (a prefix of) the sample, default Rayon threading."""
    try:
        os.environ.setdefault("TOKENIZERS_PARALLELISM", "true")
        from oracle import hf_oracle
        import tokenizers
        tok = {"char": hf_oracle.char_tokenizer, "kmer6": hf_oracle.kmer_tokenizer, "byte": hf_oracle.byte_tokenizer,
               "bpe4k": lambda: hf_oracle.bpe_tokenizer("bpe4096"), "bpe32k": lambda: hf_oracle.bpe_tokenizer("bpe32000")}[kind]()
        n_rows = len(offsets) - 1
        budget_bp = {"char": 4e6, "byte": 4e6, "kmer6": 60e6, "bpe4k": 60e6, "bpe32k": 30e6}[kind]
        n = int(min(n_rows, max(1, np.searchsorted(offsets, budget_bp))))
        strs = synth.rows_to_strings(flat, offsets[:n + 1])
        kw = {k: v for k, v in call.items() if k in ("padding", "max_length", "truncation", "add_special_tokens")}
        if kw.get("padding") == "longest":
            kw["padding"] = True
        tok(strs[:8], **kw)
        t0 = time.perf_counter()
        tok(strs, return_tensors="np" if kw.get("padding") else None, **kw)
        dt = time.perf_counter() - t0
        return {"value": round(int(offsets[n]) / dt / 1e6, 2), "unit": "Mbp/s", "threads": os.cpu_count(),
                "tokenizers": tokenizers.__version__, "sample_rows": n}
    except Exception as e:                                   # the baseline is context, never fatal
        return {"unavailable": "%s: %s" % (type(e).__name__, e)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    kind = args.workload
    flat, offsets, call, desc = cpu_sample(kind)
    base = None
    times = []
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        b = cpu_baseline_once(kind, flat, offsets, call)
        if i >= args.warmup:
            times.append(time.perf_counter() - t0)
        base = b
    ms = 1e3 * float(np.mean(times))
    value = int(offsets[-1]) / (ms * 1e-3) / 1e6
    cpu = {"value": round(value, 2), "unit": "Mbp/s", "cores": os.cpu_count() or 1, "kind": "port",
           "sample": "%s: %d rows, %.1f Mbp per step" % (desc, len(offsets) - 1, offsets[-1] / 1e6),
           "what": "oracle/dnatok_oracle.c (pthreads) + numpy padding/mask assembly",
           "hf_tokenizers": hf_baseline(kind, flat, offsets, call)}
    print(json.dumps({
        "impl": "reference", "metric": "Mbp/s encoded (bit-exact vs HF)", "value": round(value, 2), "unit": "Mbp/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u8", "data": "synthetic (seeded)",
        "config": {"workload": desc, "note": "CPU arm runs a bounded sample of the GPU arm's workload per step"},
        "cpu_baseline": cpu,
        "e2e": {"value": round(value, 2), "unit": "Mbp/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def cpu_baseline_once(kind, flat, offsets, call):
    from oracle import oracle as orc
    spec = spec_for(kind)
    table = _TABLES.get(kind)
    if spec.kind == "bpe" and table is None:
        table = _TABLES[kind] = orc.BpeTable(spec.merge_a, spec.merge_b, spec.merge_out)
    ids, counts = orc.encode_ragged(spec.kind, flat, offsets, lut256=spec.lut256, k=spec.k, kmer_ids=spec.kmer_ids,
                                    table=table, threads=os.cpu_count() or 1)
    pad = call.get("padding")
    if pad is not False:
        sp = spec.specials
        return orc.assemble(orc.rows(ids, offsets, counts), pad_id=sp.pad_id, cls_id=sp.cls_id, sep_id=sp.sep_id,
                            add_special=call.get("add_special_tokens", True), max_length=call.get("max_length", 0) or 0,
                            truncation=call.get("truncation", False), padding=pad)
    return ids, counts


_TABLES = {}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="kmer6", choices=["kmer6", "char", "byte", "bpe4k", "bpe32k"])
    ap.add_argument("--scale", type=int, default=0, help="batch multiplier over the literal shape (0: default)")
    ap.add_argument("--no-extra", action="store_true", help="skip the per_config section")
    ap.add_argument("--no-affinity", action="store_true",
                    help="leave the process on whatever cores it has instead of those next to its GPU")
    ap.add_argument("--kmer-no-scratch", action="store_true",
                    help="k-mer without scratch memory: one warp per row instead of queued row segments")
    ap.add_argument("--kmer-force-segments", action="store_true",
                    help="k-mer: use the segment encoder whatever the batch shape (library option kmer_force_segments)")
    ap.add_argument("--gather", action="store_true",
                    help="multi-GPU: also time the optional NCCL gather of the padded ids to rank 0 (outside the timed region)")
    ap.add_argument("--pcie-probe", action="store_true",
                    help="measure the host link (h2d, d2h, both at once) with pinned buffers and exit")
    ap.add_argument("--host-chunk-mb", type=int, default=None,
                    help="library option host_chunk_bytes in MiB (0: never split a host batch into overlapping chunks)")
    ap.add_argument("--host-chunk-threshold-mb", type=int, default=None,
                    help="library option host_chunk_threshold in MiB: smaller host batches are not split")
    ap.add_argument("--kernel-only", action="store_true",
                    help="device-resident timing only (no e2e, no CPU baseline): the form used under ncu")
    args = ap.parse_args()
    global KMER_NO_SCRATCH
    KMER_NO_SCRATCH = args.kmer_no_scratch
    if args.kmer_force_segments:
        from dnatok_b200 import _cabi
        _cabi.check(_cabi.lib().dnatok_set_option(b"kmer_force_segments", 1))
    args.warmup = max(args.warmup, 3)
    if args.pcie_probe:
        pcie_probe()
        return
    if args.host_chunk_mb is not None or args.host_chunk_threshold_mb is not None:
        from dnatok_b200 import _cabi
        if args.host_chunk_mb is not None:
            _cabi.check(_cabi.lib().dnatok_set_option(b"host_chunk_bytes", args.host_chunk_mb << 20))
        if args.host_chunk_threshold_mb is not None:
            _cabi.check(_cabi.lib().dnatok_set_option(b"host_chunk_threshold", args.host_chunk_threshold_mb << 20))
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

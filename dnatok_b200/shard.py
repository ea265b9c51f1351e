"""Sharding a batch by sequence over the GPUs of one box.

Rows are independent, so the hot path has no collective: each rank encodes its own rows on its
own GPU.  ``partition`` picks the rows; ``gather_padded`` is the optional step that brings
fixed-width results to rank 0 over NCCL (or gloo on CPU tensors in tests).  The reference has
no multi-GPU code at all (one process, one device: ``src/dnatok_bpe_kernel/dnatok_bpe.cu:869-870``).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import numpy as np


def partition(lengths: np.ndarray, world: int, mode: str = "contiguous") -> List[np.ndarray]:
    """Row indices per rank.

    ``contiguous``: consecutive blocks with near-equal total bases (order preserving; a
    concatenation of the rank outputs is the batch output).  ``greedy``: longest-first bin
    packing by bases for ragged read sets; use ``restore_order`` on the gathered rows.
    """
    lengths = np.asarray(lengths, dtype=np.int64)
    n = lengths.shape[0]
    if world <= 1:
        return [np.arange(n, dtype=np.int64)]
    if mode == "contiguous":
        csum = np.concatenate([[0], np.cumsum(lengths)])
        total = csum[-1]
        cuts = [0]
        for r in range(1, world):
            target = total * r / world
            j = int(np.searchsorted(csum, target, side="left"))
            j = min(max(j, cuts[-1]), n)
            # choose the nearer of j-1 / j
            if j > cuts[-1] and abs(csum[j - 1] - target) <= abs(csum[j] - target):
                j -= 1
            cuts.append(j)
        cuts.append(n)
        return [np.arange(cuts[r], cuts[r + 1], dtype=np.int64) for r in range(world)]
    if mode == "greedy":
        order = np.argsort(-lengths, kind="stable")
        load = np.zeros(world, dtype=np.int64)
        bins: List[List[int]] = [[] for _ in range(world)]
        for i in order.tolist():
            r = int(np.argmin(load))
            bins[r].append(i)
            load[r] += lengths[i]
        return [np.sort(np.asarray(b, dtype=np.int64)) for b in bins]
    raise ValueError("mode must be 'contiguous' or 'greedy'")


def safe_cut_bytes(spec) -> np.ndarray:
    """bool[256]: bytes next to which a row may be cut without changing its tokens.

    Per-character tokenizers: every byte.  BPE: bytes whose initial symbol takes part in no merge (the
    unknown id that N or lower case map to in an upper-case ACGT vocabulary, for instance): no merge ever
    crosses such a symbol, so the pieces on either side tokenise exactly as they do inside the whole row.
    k-mer tokenizers are cut by position (multiples of k), see ``split_long_rows``."""
    if spec.kind in ("char", "kmer"):
        return np.ones(256, dtype=bool)
    operands = set(np.asarray(spec.merge_a).tolist()) | set(np.asarray(spec.merge_b).tolist())
    return np.array([int(t) not in operands for t in np.asarray(spec.lut256)], dtype=bool)


def split_long_rows(flat: np.ndarray, offsets: np.ndarray, spec, max_bytes: int):
    """Cut rows longer than ``max_bytes`` into pieces that tokenise independently, for spreading one long
    record (a chromosome) over several GPUs.  Returns ``(piece_offsets int64[P + 1], piece_row int64[P])``:
    the pieces tile the same ``flat`` buffer in order and ``piece_row[p]`` is the row a piece came from.

    Cuts are exact: per-character tokenizers are cut anywhere, k-mer tokenizers at multiples of k from the
    row start, BPE tokenizers directly before or after a byte whose symbol never merges (``safe_cut_bytes``).
    A BPE row without such a byte near the wanted cut stays longer than ``max_bytes`` (up to whole): there is
    no exact cut inside a run of mergeable symbols.  Encode the pieces as rows WITHOUT special tokens and
    pass the ragged result to ``join_pieces``."""
    offsets = np.asarray(offsets, dtype=np.int64)
    if max_bytes < 1:
        raise ValueError("max_bytes must be positive")
    safe = safe_cut_bytes(spec)
    k = int(spec.k) if spec.kind == "kmer" else 1
    step = max(k, (int(max_bytes) // k) * k)
    cuts, owner = [0], []
    for r in range(len(offsets) - 1):
        lo, hi = int(offsets[r]), int(offsets[r + 1])
        at = lo
        while hi - at > max_bytes:
            want = at + step
            if spec.kind == "bpe":
                # the last safe position in (at, want]: a cut at position c is safe when byte c-1 or byte c never merges
                seg = flat[at:want + 1]
                ok = safe[seg]
                pos = np.flatnonzero(ok[:-1] | ok[1:]) + 1          # cut before seg[i+1] for every i with ok[i] or ok[i+1]
                pos = pos[pos <= want - at]
                if pos.size == 0:
                    # none inside the window: the first safe position after it, if the row has one
                    rest = safe[flat[want:hi]]
                    nxt = np.flatnonzero(rest)
                    if nxt.size == 0:
                        break
                    want = want + int(nxt[0]) + 1
                    if want >= hi:
                        break
                else:
                    want = at + int(pos[-1])
            cuts.append(want)
            owner.append(r)
            at = want
        cuts.append(hi)
        owner.append(r)
    piece_offsets = np.asarray(cuts, dtype=np.int64)
    # empty rows keep their (empty) piece; duplicates from a cut landing on a row end cannot occur (want < hi)
    return piece_offsets, np.asarray(owner, dtype=np.int64)


def join_pieces(piece_out_offsets: np.ndarray, piece_row: np.ndarray, n_rows: int) -> np.ndarray:
    """Row offsets into the ragged ids of the pieces: the pieces of a row are consecutive, so a row's tokens
    are the concatenation of its pieces' tokens and only the offsets need regrouping."""
    piece_out_offsets = np.asarray(piece_out_offsets, dtype=np.int64)
    first = np.searchsorted(piece_row, np.arange(n_rows), side="left")
    return np.concatenate([piece_out_offsets[first], piece_out_offsets[-1:]])


def take_rows(flat: np.ndarray, offsets: np.ndarray, rows: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """The sub-batch (flat bytes, offsets) made of ``rows``."""
    lens = (offsets[1:] - offsets[:-1])[rows]
    out_off = np.zeros(rows.shape[0] + 1, dtype=np.int64)
    np.cumsum(lens, out=out_off[1:])
    if rows.shape[0] and np.all(np.diff(rows) == 1):
        return flat[offsets[rows[0]]:offsets[rows[-1] + 1]], out_off
    out = np.empty(int(out_off[-1]), dtype=np.uint8)
    for j, i in enumerate(rows.tolist()):
        out[out_off[j]:out_off[j + 1]] = flat[offsets[i]:offsets[i + 1]]
    return out, out_off


def restore_order(parts: List[np.ndarray], rows_per_rank: List[np.ndarray]) -> np.ndarray:
    """Inverse of a partition for fixed-width results: parts[r] is [len(rows_per_rank[r]), W]."""
    n = sum(p.shape[0] for p in parts)
    width = max((p.shape[1] for p in parts if p.ndim == 2), default=0)
    out = np.zeros((n, width), dtype=parts[0].dtype if parts else np.int64)
    for p, rows in zip(parts, rows_per_rank):
        out[rows, :p.shape[1]] = p
    return out


def gather_padded(ids, n_rows_per_rank: List[int], width: int, pad_id: int, dst: int = 0, group=None):
    """Optional gather of fixed-width rows to ``dst`` with torch.distributed (NCCL for CUDA tensors,
    gloo for CPU tensors).  Every rank passes its [rows_r, w_r] tensor; rows are right-padded to
    ``width`` with ``pad_id`` first.  Returns the [sum rows, width] tensor on ``dst``, else None.
    Not part of the timed hot path."""
    import torch
    import torch.distributed as dist
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    mine = torch.full((n_rows_per_rank[rank], width), pad_id, dtype=ids.dtype, device=ids.device)
    mine[:, :ids.shape[1]] = ids
    max_rows = max(n_rows_per_rank)
    buf = torch.full((max_rows, width), pad_id, dtype=ids.dtype, device=ids.device)
    buf[:mine.shape[0]] = mine
    if rank == dst:
        bucket = [torch.empty_like(buf) for _ in range(world)]
        dist.gather(buf, bucket, dst=dst, group=group)
        return torch.cat([bucket[r][:n_rows_per_rank[r]] for r in range(world)], dim=0)
    dist.gather(buf, None, dst=dst, group=group)
    return None


def bind_host_to_gpu(device_index: int):
    """Pin the calling process to the CPU cores next to GPU ``device_index`` (NVML's ideal CPU
    affinity), so that the pinned host buffers it allocates afterwards land on the NUMA node the
    GPU's PCIe link hangs off.  With one process per GPU this keeps each rank's host<->device copies
    off the inter-socket link.  Returns the list of cores the process is bound to, or None when
    NVML is missing, reports nothing, or none of its cores is allowed to this process (cgroup)."""
    import os
    try:
        import pynvml
        pynvml.nvmlInit()
        try:
            h = pynvml.nvmlDeviceGetHandleByIndex(int(device_index))
            n_words = (os.cpu_count() + 63) // 64
            words = pynvml.nvmlDeviceGetCpuAffinity(h, n_words)
        finally:
            pynvml.nvmlShutdown()
    except Exception:
        return None
    ideal = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
    allowed = os.sched_getaffinity(0)
    cores = sorted(ideal & allowed)
    if not cores or len(cores) == len(allowed):
        return cores or None
    os.sched_setaffinity(0, cores)
    return cores

// k-mer tokenizers whose windows do not follow "clean window -> one id, anything else -> one id per
// character": every window over {A, C, G, T, N} is looked up in a 5^k table that holds either its id
// or a run of ids (the table the reference builds by tokenising all 5^k strings,
// src/dna_tokenizer.py:759-806, and replays in _encode_kmer_fallback_from_lut, :1896-1953).  A
// character outside ACGT counts as N, the reference's replace_with_n policy (:1318-1332).  The
// len % k tail gives one id per character, or nothing for tokenizers that drop it.
//
// One warp per row, 32 windows per trip: every lane looks its window up, a warp scan places the
// runs, the ids are stored.  Rows of such tokenizers are rare and short-listed at discovery, so
// this kernel is written for clarity; the 4^k kernels in kmer_kernel.cuh carry the bandwidth.
#pragma once
#include "kmer_kernel.cuh"

namespace dnatok {

struct KmerTable {
    const int32_t* table5;     // [5^k] id >= 0, or -(e + 1): run e of exp_ids
    const int32_t* exp_off;    // [n_runs + 1]
    const int32_t* exp_ids;
    const int32_t* singles;    // [256] id of a character of the tail
    int k;
    int tail_singles;          // 0: the len % k tail gives no tokens
};

constexpr int KT_WARPS = 8;

template <typename IdT, bool COUNT_ONLY>
__global__ void __launch_bounds__(KT_WARPS * 32)
kmer_table_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets, int64_t n_rows, KmerTable t,
                  RowFormat f, IdT* __restrict__ ids, void* __restrict__ mask, const int32_t* __restrict__ lengths_in,
                  int32_t* __restrict__ lengths_out, const int64_t* __restrict__ out_offsets, int32_t* __restrict__ status) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * KT_WARPS + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int64_t off = offsets[row];
    const int64_t len64 = offsets[row + 1] - off;
    const int len = (int)(len64 < 0x7fffffff ? len64 : 0x7fffffff);
    if (!COUNT_ONLY) kmer_flag_long_row(len64, status, row, lane);
    const int k = t.k;
    const int n_full = len / k, tail = len - n_full * k;
    const int n_win = n_full + (tail ? 1 : 0);
    const int cap = (int)(f.cap_content < 0x7fffffff ? f.cap_content : 0x7fffffff);
    const uint8_t* src = bytes + off;
    const bool ragged = f.out_stride == 0;
    KmerRow<IdT> r;
    r.src = src; r.len = len; r.n_win = n_win; r.room_total = 0; r.shift = 0;
    r.orow = nullptr; r.dst = nullptr;
    if (!COUNT_ONLY) {
        r.orow = ragged ? ids + out_offsets[row] : ids + row * f.out_stride;
        if (!ragged && f.pad_left) r.shift = (int)f.out_stride - lengths_in[row];
        r.dst = r.orow + r.shift + (f.cls_id >= 0 ? 1 : 0);
    }
    int base = 0;
    for (int w0 = 0; w0 < n_win; w0 += 32) {              // to the end of the row even past the cap: the count decides "clipped"
        const int w = w0 + lane;
        int cnt = 0, entry = 0;
        if (w < n_full) {
            int idx = 0;
            for (int i = 0; i < k; ++i) idx = idx * 5 + kmer_code(__ldg(src + w * k + i));
            entry = __ldg(t.table5 + idx);
            cnt = entry >= 0 ? 1 : __ldg(t.exp_off - entry) - __ldg(t.exp_off - entry - 1);
        } else if (w == n_full && tail) {
            cnt = t.tail_singles ? tail : 0;
        }
        int x = cnt;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, x, d);
            if (lane >= d) x += y;
        }
        const int total = __shfl_sync(0xffffffffu, x, 31);
        if (!COUNT_ONLY) {
            int pos = base + x - cnt;
            if (w < n_full) {
                if (entry >= 0) { if (pos < cap) r.dst[pos] = (IdT)entry; }
                else {
                    const int32_t* run = t.exp_ids + __ldg(t.exp_off - entry - 1);
                    for (int i = 0; i < cnt; ++i, ++pos) if (pos < cap) r.dst[pos] = (IdT)__ldg(run + i);
                }
            } else {
                for (int i = 0; i < cnt; ++i, ++pos) if (pos < cap) r.dst[pos] = (IdT)__ldg(t.singles + __ldg(src + n_full * k + i));
            }
        }
        base += total;
    }
    const bool clipped = base > cap;
    if (COUNT_ONLY) {
        const int n = base < cap ? base : cap;
        if (lane == 0) {
            lengths_out[row] = n + (f.cls_id >= 0 ? 1 : 0) + (f.sep_id >= 0 ? 1 : 0);
            if (status && f.clip_is_error && clipped) atomicOr(status + row, 4);
        }
        return;
    }
    kmer_finish_row<IdT, false>(r, row, base, cap, clipped, f, ids, mask, lengths_out, out_offsets, status, lane);
}

}  // namespace dnatok

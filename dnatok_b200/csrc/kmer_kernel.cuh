// Non-overlapping k-mer tokenisation.  One block walks one row tile by tile: the tile's raw
// ASCII is staged in shared memory with 128-bit loads, every thread packs its windows into 2-bit
// codes in registers, a block scan places each window's tokens (1 for a clean window, one per
// character for a window holding anything but ACGT and for the len%k tail), the tokens are staged
// in shared memory and flushed with 128-bit stores together with specials, padding and mask.
#pragma once
#include "common.cuh"

namespace dnatok {

constexpr int KMER_THREADS = 128;
constexpr int KMER_WPT = 8;                                  // windows per thread per tile
constexpr int KMER_TILE_W = KMER_THREADS * KMER_WPT;         // windows per tile
constexpr int KMER_MAX_K = 8;

__device__ __forceinline__ int kmer_code(uint32_t c) {       // A C G T -> 0..3, anything else -> 4
    return c == 'A' ? 0 : c == 'C' ? 1 : c == 'G' ? 2 : c == 'T' ? 3 : 4;
}

struct KmerSmem {
    int32_t single[256];
    int32_t warp_sum[KMER_THREADS / 32];
    int32_t tile_total;
};

// Exclusive block scan of one int per thread; returns the thread's offset, total in *total.
__device__ __forceinline__ int kmer_block_scan(int v, KmerSmem& s, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int x = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, d);
        if (lane >= d) x += y;
    }
    if (lane == 31) s.warp_sum[warp] = x;
    __syncthreads();
    int before = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < KMER_THREADS / 32; ++w) {
        const int ws = s.warp_sum[w];
        if (w < warp) before += ws;
        tot += ws;
    }
    *total = tot;
    __syncthreads();
    return before + x - v;
}

// Stage bytes [g, g+nb) into s_in so that byte i sits at s_in[a + i], a = g & 15.
__device__ __forceinline__ int kmer_stage(const uint8_t* __restrict__ g, int nb, uint8_t* s_in) {
    const int a = (int)(reinterpret_cast<uintptr_t>(g) & 15);
    const uint8_t* ga = g - a;
    const int nvec = (a + nb + 15) >> 4;
    for (int v = threadIdx.x; v < nvec; v += KMER_THREADS) {
        const int lo = v * 16, hi = lo + 16;
        if (lo >= a && hi <= a + nb) {
            reinterpret_cast<uint4*>(s_in)[v] = __ldg(reinterpret_cast<const uint4*>(ga) + v);
        } else {
            for (int i = lo; i < hi; ++i) s_in[i] = (i >= a && i < a + nb) ? __ldg(ga + i) : (uint8_t)0;
        }
    }
    return a;
}

// COUNT_ONLY: only lengths[] is written (the sizing pass for 'longest' padding and ragged output).
template <typename IdT, bool COUNT_ONLY>
__global__ void __launch_bounds__(KMER_THREADS)
kmer_rows_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets, int64_t n_rows,
                 int k, const int32_t* __restrict__ kmer_ids, const int32_t* __restrict__ single_ids,
                 RowFormat f, IdT* __restrict__ ids, void* __restrict__ mask,
                 const int32_t* __restrict__ lengths_in, int32_t* __restrict__ lengths_out,
                 const int64_t* __restrict__ out_offsets, int32_t* __restrict__ status) {
    extern __shared__ uint4 kmer_dyn[];
    __shared__ KmerSmem s;
    uint8_t* s_in = reinterpret_cast<uint8_t*>(kmer_dyn);                       // KMER_TILE_W*k + 32 bytes
    int32_t* s_tok = reinterpret_cast<int32_t*>(s_in + ((KMER_TILE_W * k + 32 + 15) & ~15));  // KMER_TILE_W*k ints
    for (int i = threadIdx.x; i < 256; i += KMER_THREADS) s.single[i] = single_ids[i];
    __syncthreads();

    const bool has_cls = f.cls_id >= 0, has_sep = f.sep_id >= 0;
    const int n_special = (has_cls ? 1 : 0) + (has_sep ? 1 : 0);
    const bool ragged = f.out_stride == 0;

    for (int64_t row = blockIdx.x; row < n_rows; row += gridDim.x) {
        const int64_t off = offsets[row];
        const int64_t len = offsets[row + 1] - off;
        const int64_t n_win = (len + k - 1) / k;
        const int64_t cap = f.cap_content;

        // Where the row's first token goes.  Left padding and ragged output need the row's
        // token count up front: taken from lengths_in / out_offsets.
        int64_t T_known = -1;
        if (!COUNT_ONLY) {
            if (ragged) T_known = out_offsets[row + 1] - out_offsets[row];
            else if (lengths_in) T_known = lengths_in[row];
        }
        IdT* orow = nullptr;
        int64_t shift = 0;
        if (!COUNT_ONLY) {
            orow = ragged ? ids + out_offsets[row] : ids + row * f.out_stride;
            if (!ragged && f.pad_left) shift = f.out_stride - T_known;   // host guarantees lengths_in here
        }

        int64_t carry = 0;        // content tokens placed so far (uncapped)
        int64_t w0 = 0;
        for (; w0 < n_win && carry < cap; w0 += KMER_TILE_W) {
            const int64_t b0 = w0 * k;
            const int nb = (int)((len - b0) < (int64_t)KMER_TILE_W * k ? (len - b0) : (int64_t)KMER_TILE_W * k);
            const int a = kmer_stage(bytes + off + b0, nb, s_in);
            __syncthreads();

            // pack this thread's windows
            int cnt[KMER_WPT];
            uint32_t idx[KMER_WPT];
            int my = 0;
#pragma unroll
            for (int j = 0; j < KMER_WPT; ++j) {
                const int wb = (threadIdx.x * KMER_WPT + j) * k;
                int wl = nb - wb; wl = wl < 0 ? 0 : (wl > k ? k : wl);
                uint32_t x = 0; int bad = (wl != k);
                for (int i = 0; i < wl; ++i) {
                    const int c = kmer_code(s_in[a + wb + i]);
                    bad |= (c >> 2);
                    x = (x << 2) | (uint32_t)(c & 3);
                }
                cnt[j] = bad ? wl : 1;
                idx[j] = bad ? 0xffffffffu : x;
                my += cnt[j];
            }
            int tile_total;
            int pos = kmer_block_scan(my, s, &tile_total);
            if (!COUNT_ONLY) {
#pragma unroll
                for (int j = 0; j < KMER_WPT; ++j) {
                    if (idx[j] != 0xffffffffu) {
                        s_tok[pos++] = __ldg(kmer_ids + idx[j]);
                    } else {
                        const int wb = (threadIdx.x * KMER_WPT + j) * k;
                        for (int i = 0; i < cnt[j]; ++i) s_tok[pos++] = s.single[s_in[a + wb + i]];
                    }
                }
                __syncthreads();
                int64_t m = tile_total;
                if (carry + m > cap) m = cap - carry;
                IdT* dst = orow + shift + (has_cls ? 1 : 0) + carry;
                const int32_t* st = s_tok;
                block_write_run<IdT>(dst, m, [=](int64_t j) { return (IdT)st[j]; });
            }
            carry += tile_total;
            __syncthreads();
        }

        const int64_t n = carry < cap ? carry : cap;
        const int64_t T = n + n_special;
        if (threadIdx.x == 0) {
            if (lengths_out) lengths_out[row] = (int32_t)T;
            if (status && f.clip_is_error && (carry > cap || w0 < n_win)) atomicOr(status + row, 4);
        }
        if (!COUNT_ONLY) {
            if (threadIdx.x == 0) {
                if (has_cls) orow[shift] = (IdT)f.cls_id;
                if (has_sep) orow[shift + T - 1] = (IdT)f.sep_id;
            }
            if (!ragged) {
                const IdT pad = (IdT)f.pad_id;
                if (f.pad_left) block_write_run<IdT>(orow, shift, [=](int64_t) { return pad; });
                else block_write_run<IdT>(orow + T, f.out_stride - T, [=](int64_t) { return pad; });
                block_write_mask_any(mask, f.mask_bits, row, f.out_stride, shift, shift + T);
            } else if (mask && f.mask_bits) {
                const int64_t o = out_offsets[row];
                if (f.mask_bits == 64) block_write_run<int64_t>((int64_t*)mask + o, T, [](int64_t) { return (int64_t)1; });
                else if (f.mask_bits == 32) block_write_run<int32_t>((int32_t*)mask + o, T, [](int64_t) { return (int32_t)1; });
                else block_write_run<uint8_t>((uint8_t*)mask + o, T, [](int64_t) { return (uint8_t)1; });
            }
        }
    }
}

}  // namespace dnatok

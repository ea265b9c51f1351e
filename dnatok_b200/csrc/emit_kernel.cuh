// One token per source element: the single-base / byte path (uint8 source through a 256-entry
// shared-memory LUT) and the output stage of the BPE path (uint16 merged tokens, identity).
// Special tokens, truncation, padding and the attention mask are produced in the same pass.
#pragma once
#include "common.cuh"

namespace dnatok {

constexpr int EMIT_THREADS = 256;
constexpr int EMIT_TILE = 4096;          // output columns per tile

template <typename SrcT, bool USE_LUT>
__device__ __forceinline__ int32_t emit_load(const SrcT* __restrict__ p, const int32_t* s_lut) {
    if (USE_LUT) return s_lut[(uint8_t)__ldg(p)];
    return (int32_t)__ldg(p);
}

// Padded output [n_rows, out_stride].  counts == nullptr: a row's content is its byte span.
template <typename SrcT, typename IdT, bool USE_LUT>
__global__ void __launch_bounds__(EMIT_THREADS)
emit_padded_kernel(const SrcT* __restrict__ src, const int64_t* __restrict__ offsets,
                   const int32_t* __restrict__ counts, int64_t n_rows,
                   const int32_t* __restrict__ lut, RowFormat f, IdT* __restrict__ ids,
                   void* __restrict__ mask, int32_t* __restrict__ lengths_out,
                   int32_t* __restrict__ status, int64_t tiles_per_row, int64_t n_tiles) {
    __shared__ int32_t s_lut[256];
    if (USE_LUT) {
        for (int i = threadIdx.x; i < 256; i += EMIT_THREADS) s_lut[i] = lut[i];
        __syncthreads();
    }
    constexpr int N = Vec16<IdT>::N;
    const bool has_cls = f.cls_id >= 0, has_sep = f.sep_id >= 0;
    const int64_t stride = f.out_stride;
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int64_t row = tile / tiles_per_row;
        const int64_t c0 = (tile - row * tiles_per_row) * EMIT_TILE;
        const int64_t off = offsets[row];
        const int64_t n_in = counts ? (int64_t)counts[row] : offsets[row + 1] - off;
        const int64_t n = n_in < f.cap_content ? n_in : f.cap_content;
        const int64_t T = n + (has_cls ? 1 : 0) + (has_sep ? 1 : 0);
        const int64_t shift = f.pad_left ? stride - T : 0;
        if (c0 == 0 && threadIdx.x == 0) {
            if (lengths_out) lengths_out[row] = (int32_t)T;
            if (status && f.clip_is_error && n_in > n) atomicOr(status + row, 4);
        }
        const SrcT* srow = src + off - (has_cls ? 1 : 0);
        IdT* orow = ids + row * stride;
        const bool aligned = ((reinterpret_cast<uintptr_t>(orow) & 15) == 0);
        int64_t c_end = c0 + EMIT_TILE < stride ? c0 + EMIT_TILE : stride;
        for (int64_t c = c0 + (int64_t)threadIdx.x * N; c < c_end; c += (int64_t)EMIT_THREADS * N) {
            IdT vals[N];
#pragma unroll
            for (int e = 0; e < N; ++e) {
                const int64_t t = c + e - shift;
                int32_t v = f.pad_id;
                if (t >= 0 && t < T && c + e < stride) {
                    if (has_cls && t == 0) v = f.cls_id;
                    else if (has_sep && t == T - 1) v = f.sep_id;
                    else v = emit_load<SrcT, USE_LUT>(srow + t, s_lut);
                }
                vals[e] = (IdT)v;
            }
            if (aligned && c + N <= stride) store_vec<IdT>(orow + c, vals);
            else {
#pragma unroll
                for (int e = 0; e < N; ++e) if (c + e < stride) orow[c + e] = vals[e];
            }
        }
        if (f.mask_bits) {
            // this tile's slice of the mask row
            const int64_t lo = shift - c0, hi = shift + T - c0, m = c_end - c0;
            if (f.mask_bits == 64)
                block_write_run<int64_t>((int64_t*)mask + row * stride + c0, m,
                                         [=](int64_t j) { return (int64_t)((j >= lo && j < hi) ? 1 : 0); });
            else if (f.mask_bits == 32)
                block_write_run<int32_t>((int32_t*)mask + row * stride + c0, m,
                                         [=](int64_t j) { return (int32_t)((j >= lo && j < hi) ? 1 : 0); });
            else
                block_write_run<uint8_t>((uint8_t*)mask + row * stride + c0, m,
                                         [=](int64_t j) { return (uint8_t)((j >= lo && j < hi) ? 1 : 0); });
        }
    }
}

// Ragged output: ids is one flat array, row i occupies [out_offsets[i], out_offsets[i+1]).
// The grid covers an upper bound of the total; tiles past the real total do nothing.
template <typename SrcT, typename IdT, bool USE_LUT>
__global__ void __launch_bounds__(EMIT_THREADS)
emit_ragged_kernel(const SrcT* __restrict__ src, const int64_t* __restrict__ offsets,
                   const int64_t* __restrict__ out_offsets, int64_t n_rows,
                   const int32_t* __restrict__ lut, RowFormat f, IdT* __restrict__ ids,
                   void* __restrict__ mask, int64_t n_tiles) {
    __shared__ int32_t s_lut[256];
    __shared__ int64_t s_rows[2];
    if (USE_LUT) {
        for (int i = threadIdx.x; i < 256; i += EMIT_THREADS) s_lut[i] = lut[i];
    }
    constexpr int N = Vec16<IdT>::N;
    const bool has_cls = f.cls_id >= 0, has_sep = f.sep_id >= 0;
    const int64_t total = out_offsets[n_rows];
    for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const int64_t e0 = tile * EMIT_TILE;
        if (e0 >= total) break;
        const int64_t e1 = e0 + EMIT_TILE < total ? e0 + EMIT_TILE : total;
        __syncthreads();
        if (threadIdx.x < 2) {
            // last row whose start is <= the first / last element of the tile
            const int64_t e = threadIdx.x == 0 ? e0 : e1 - 1;
            int64_t lo = 0, hi = n_rows - 1;
            while (lo < hi) {
                const int64_t mid = (lo + hi + 1) >> 1;
                if (out_offsets[mid] <= e) lo = mid; else hi = mid - 1;
            }
            s_rows[threadIdx.x] = lo;
        }
        __syncthreads();
        const int64_t r_lo = s_rows[0], r_hi = s_rows[1];
        for (int64_t c = e0 + (int64_t)threadIdx.x * N; c < e1; c += (int64_t)EMIT_THREADS * N) {
            IdT vals[N];
            int64_t lo = r_lo;
#pragma unroll
            for (int e = 0; e < N; ++e) {
                const int64_t g = c + e;
                int32_t v = f.pad_id;
                if (g < e1) {
                    int64_t hi = r_hi;              // rows are ordered, so the search restarts at lo
                    while (lo < hi) {
                        const int64_t mid = (lo + hi + 1) >> 1;
                        if (out_offsets[mid] <= g) lo = mid; else hi = mid - 1;
                    }
                    const int64_t t = g - out_offsets[lo];
                    const int64_t T = out_offsets[lo + 1] - out_offsets[lo];
                    if (has_cls && t == 0) v = f.cls_id;
                    else if (has_sep && t == T - 1) v = f.sep_id;
                    else v = emit_load<SrcT, USE_LUT>(src + offsets[lo] + t - (has_cls ? 1 : 0), s_lut);
                }
                vals[e] = (IdT)v;
            }
            if (c + N <= e1 && ((reinterpret_cast<uintptr_t>(ids + c) & 15) == 0)) store_vec<IdT>(ids + c, vals);
            else {
#pragma unroll
                for (int e = 0; e < N; ++e) if (c + e < e1) ids[c + e] = vals[e];
            }
        }
        if (mask && f.mask_bits) {
            if (f.mask_bits == 64) block_write_run<int64_t>((int64_t*)mask + e0, e1 - e0, [](int64_t) { return (int64_t)1; });
            else if (f.mask_bits == 32) block_write_run<int32_t>((int32_t*)mask + e0, e1 - e0, [](int64_t) { return (int32_t)1; });
            else block_write_run<uint8_t>((uint8_t*)mask + e0, e1 - e0, [](int64_t) { return (uint8_t)1; });
        }
    }
}

// Row lengths of the one-token-per-element paths (no data is read): min(n, cap) + specials.
__global__ void span_lengths_kernel(const int64_t* __restrict__ offsets, const int32_t* __restrict__ counts,
                                    int64_t n_rows, RowFormat f, int32_t* __restrict__ lengths,
                                    int32_t* __restrict__ status) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows) return;
    const int64_t n_in = counts ? (int64_t)counts[i] : offsets[i + 1] - offsets[i];
    const int64_t n = n_in < f.cap_content ? n_in : f.cap_content;
    lengths[i] = (int32_t)(n + (f.cls_id >= 0 ? 1 : 0) + (f.sep_id >= 0 ? 1 : 0));
    if (status && f.clip_is_error && n_in > n) atomicOr(status + i, 4);
}

// Exclusive scan of int32 lengths into int64 offsets, one block, chunk by chunk.
__global__ void __launch_bounds__(1024)
scan_lengths_kernel(const int32_t* __restrict__ lengths, int64_t n_rows, int64_t* __restrict__ out_offsets) {
    __shared__ int64_t s_warp[32];
    __shared__ int64_t s_carry;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) { s_carry = 0; out_offsets[0] = 0; }
    __syncthreads();
    for (int64_t base = 0; base < n_rows; base += 1024) {
        const int64_t i = base + tid;
        int64_t v = i < n_rows ? (int64_t)lengths[i] : 0;
        int64_t x = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int64_t y = __shfl_up_sync(0xffffffffu, x, d);
            if (lane >= d) x += y;
        }
        if (lane == 31) s_warp[warp] = x;
        __syncthreads();
        if (warp == 0) {
            int64_t w = s_warp[lane];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int64_t y = __shfl_up_sync(0xffffffffu, w, d);
                if (lane >= d) w += y;
            }
            s_warp[lane] = w;
        }
        __syncthreads();
        const int64_t incl = x + (warp ? s_warp[warp - 1] : 0) + s_carry;
        if (i < n_rows) out_offsets[i + 1] = incl;
        __syncthreads();
        if (tid == 1023) s_carry = incl;
        __syncthreads();
    }
}

}  // namespace dnatok

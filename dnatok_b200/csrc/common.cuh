// Shared device helpers: output format, 16-byte vector stores, run writers.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace dnatok {

// Device-side view of dnatok_format + dnatok_specials, resolved by the host.
struct RowFormat {
    int64_t out_stride;     // columns per row (padded) or 0 (ragged)
    int64_t cap_content;    // most content tokens a row may keep (truncation and stride already applied)
    int32_t cls_id;         // -1: none
    int32_t sep_id;         // -1: none
    int32_t pad_id;
    int32_t pad_left;
    int32_t mask_bits;      // 0, 8, 32, 64
    int32_t clip_is_error;  // rows cut by the stride (not by requested truncation) get DNATOK_ROW_CLIPPED
    int32_t store_status;   // 1: the status words were not zeroed: the kernel writes a row's word instead of OR-ing into it
                            // (only kernels in which one thread finishes a row, and only when the host says so)
};

template <typename T> struct Vec16;
template <> struct Vec16<int64_t>  { static constexpr int N = 2;  };
template <> struct Vec16<int32_t>  { static constexpr int N = 4;  };
template <> struct Vec16<uint8_t>  { static constexpr int N = 16; };

// Store N = 16/sizeof(T) consecutive elements with one 128-bit store; dst must be 16-byte aligned.
template <typename T>
__device__ __forceinline__ void store_vec(T* dst, const T* vals) {
    constexpr int N = Vec16<T>::N;
    union { uint4 v; T t[N]; } u;
#pragma unroll
    for (int i = 0; i < N; ++i) u.t[i] = vals[i];
    *reinterpret_cast<uint4*>(dst) = u.v;
}

// The block writes dst[0..m) = f(j), thread-strided, 128-bit stores on the aligned body.
template <typename T, typename F>
__device__ __forceinline__ void block_write_run(T* dst, int64_t m, F f) {
    constexpr int N = Vec16<T>::N;
    if (m <= 0) return;
    const int tid = threadIdx.x, nt = blockDim.x;
    int64_t head = (N - (int64_t)((reinterpret_cast<uintptr_t>(dst) / sizeof(T)) % N)) % N;
    if (head > m) head = m;
    for (int64_t j = tid; j < head; j += nt) dst[j] = f(j);
    const int64_t nv = (m - head) / N;
    for (int64_t v = tid; v < nv; v += nt) {
        T vals[N];
        const int64_t j0 = head + v * N;
#pragma unroll
        for (int e = 0; e < N; ++e) vals[e] = f(j0 + e);
        store_vec<T>(dst + j0, vals);
    }
    for (int64_t j = head + nv * N + tid; j < m; j += nt) dst[j] = f(j);
}

// Mask row: 1 on [lo, hi), 0 elsewhere on [0, stride).
template <typename M>
__device__ __forceinline__ void block_write_mask_row(M* row, int64_t stride, int64_t lo, int64_t hi) {
    block_write_run<M>(row, stride, [=](int64_t j) { return (M)((j >= lo && j < hi) ? 1 : 0); });
}

// Warp-level variants: the 32 lanes of one warp write dst[0..m).
template <typename T, typename F>
__device__ __forceinline__ void warp_write_run(T* dst, int64_t m, int lane, F f) {
    constexpr int N = Vec16<T>::N;
    if (m <= 0) return;
    int64_t head = (N - (int64_t)((reinterpret_cast<uintptr_t>(dst) / sizeof(T)) % N)) % N;
    if (head > m) head = m;
    for (int64_t j = lane; j < head; j += 32) dst[j] = f(j);
    const int64_t nv = (m - head) / N;
    for (int64_t v = lane; v < nv; v += 32) {
        T vals[N];
        const int64_t j0 = head + v * N;
#pragma unroll
        for (int e = 0; e < N; ++e) vals[e] = f(j0 + e);
        store_vec<T>(dst + j0, vals);
    }
    for (int64_t j = head + nv * N + lane; j < m; j += 32) dst[j] = f(j);
}

template <typename M>
__device__ __forceinline__ void warp_mask_row(M* row, int64_t stride, int64_t lo, int64_t hi, int lane) {
    warp_write_run<M>(row, stride, lane, [=](int64_t j) { return (M)((j >= lo && j < hi) ? 1 : 0); });
}

__device__ __forceinline__ void block_write_mask_any(void* mask, int mask_bits, int64_t row,
                                                     int64_t stride, int64_t lo, int64_t hi) {
    if (mask_bits == 64) block_write_mask_row<int64_t>((int64_t*)mask + row * stride, stride, lo, hi);
    else if (mask_bits == 32) block_write_mask_row<int32_t>((int32_t*)mask + row * stride, stride, lo, hi);
    else if (mask_bits == 8) block_write_mask_row<uint8_t>((uint8_t*)mask + row * stride, stride, lo, hi);
}

}  // namespace dnatok

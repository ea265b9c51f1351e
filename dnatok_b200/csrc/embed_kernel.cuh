// Fused tokenise -> embedding-row gather for one-token-per-byte tables: out[row, col, :] = W[id(row, col), :]
// with the ids never written to memory.  The reference prototypes this as a Triton kernel, one program
// per token and 128-wide blocks of the embedding row (src/dna_tokenizer.py:3465-3532); here a group of
// lanes copies a token's row in 16-byte pieces, and special tokens, truncation and padding are resolved
// per column exactly as the id kernels do.
#pragma once
#include "common.cuh"

namespace dnatok {

constexpr int EMBED_THREADS = 256;

// pieces: 16-byte pieces per embedding row; lanes_per_token: power of two <= 32, <= pieces.
// One warp takes 32 consecutive columns of one row: lane l resolves the id of column cs + l (one
// coalesced byte load for the whole span), then the warp copies the 32 rows, 32 / lanes_per_token
// tokens at a time, each token's id broadcast by a shuffle.
__global__ void __launch_bounds__(EMBED_THREADS)
embed_padded_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets, int64_t n_rows,
                    const int32_t* __restrict__ lut, RowFormat f, const uint4* __restrict__ weight,
                    int64_t vocab_rows, int pieces, int lanes_per_token, uint4* __restrict__ out,
                    int32_t* __restrict__ lengths_out, int32_t* __restrict__ status) {
    __shared__ int32_t s_lut[256];
    for (int i = threadIdx.x; i < 256; i += EMBED_THREADS) s_lut[i] = lut[i];
    __syncthreads();
    const bool has_cls = f.cls_id >= 0, has_sep = f.sep_id >= 0;
    const int64_t stride = f.out_stride;
    const int64_t spans_per_row = (stride + 31) / 32;
    const int64_t n_spans = n_rows * spans_per_row;
    const bool small = n_spans <= 0x7fffffff;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int tokens_per_trip = 32 / lanes_per_token;
    const int sub = lane / lanes_per_token, gl = lane % lanes_per_token;
    for (int64_t span = (int64_t)blockIdx.x * (EMBED_THREADS / 32) + warp; span < n_spans;
         span += (int64_t)gridDim.x * (EMBED_THREADS / 32)) {
        int64_t row, cs;
        if (small) {
            const uint32_t r32 = (uint32_t)span / (uint32_t)spans_per_row;
            row = r32;
            cs = (int64_t)((uint32_t)span - r32 * (uint32_t)spans_per_row) * 32;
        } else {
            row = span / spans_per_row;
            cs = (span - row * spans_per_row) * 32;
        }
        const int64_t off = offsets[row];
        const int64_t n_in = offsets[row + 1] - off;
        const int64_t n = n_in < f.cap_content ? n_in : f.cap_content;
        const int64_t T = n + (has_cls ? 1 : 0) + (has_sep ? 1 : 0);
        const int64_t shift = f.pad_left ? stride - T : 0;
        if (cs == 0 && lane == 0) {
            if (lengths_out) lengths_out[row] = (int32_t)T;
            if (status && f.clip_is_error && n_in > n) atomicOr(status + row, 4);
        }
        const int ncol = (int)(stride - cs < 32 ? stride - cs : 32);
        const int64_t t = cs + lane - shift;                 // this lane's token index within the row
        int32_t id = f.pad_id;
        if (t >= 0 && t < T) {
            if (has_cls && t == 0) id = f.cls_id;
            else if (has_sep && t == T - 1) id = f.sep_id;
            else id = s_lut[__ldg(bytes + off + t - (has_cls ? 1 : 0))];
        }
        if (id < 0 || id >= vocab_rows) id = f.pad_id;       // ids outside the weight matrix read the pad row
        uint4* dst = out + (row * stride + cs) * pieces;
        for (int k0 = 0; k0 < ncol; k0 += tokens_per_trip) {
            const int k = k0 + sub;
            const int32_t kid = __shfl_sync(0xffffffffu, id, k & 31);
            if (k < ncol) {
                const uint4* src = weight + (int64_t)kid * pieces;
                uint4* d = dst + (int64_t)k * pieces;
                for (int p = gl; p < pieces; p += lanes_per_token) d[p] = __ldg(src + p);
            }
        }
    }
}

}  // namespace dnatok

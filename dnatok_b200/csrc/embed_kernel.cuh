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
    const int64_t n_tokens = n_rows * stride;
    const int groups_per_block = EMBED_THREADS / lanes_per_token;
    const int group = threadIdx.x / lanes_per_token, gl = threadIdx.x % lanes_per_token;
    for (int64_t tk = (int64_t)blockIdx.x * groups_per_block + group; tk < n_tokens;
         tk += (int64_t)gridDim.x * groups_per_block) {
        const int64_t row = tk / stride, col = tk - row * stride;
        const int64_t off = offsets[row];
        const int64_t n_in = offsets[row + 1] - off;
        const int64_t n = n_in < f.cap_content ? n_in : f.cap_content;
        const int64_t T = n + (has_cls ? 1 : 0) + (has_sep ? 1 : 0);
        const int64_t shift = f.pad_left ? stride - T : 0;
        const int64_t t = col - shift;                       // token index within the row
        int32_t id = f.pad_id;
        if (t >= 0 && t < T) {
            if (has_cls && t == 0) id = f.cls_id;
            else if (has_sep && t == T - 1) id = f.sep_id;
            else id = s_lut[__ldg(bytes + off + t - (has_cls ? 1 : 0))];
        }
        if (col == 0 && gl == 0) {
            if (lengths_out) lengths_out[row] = (int32_t)T;
            if (status && f.clip_is_error && n_in > n) atomicOr(status + row, 4);
        }
        if (id < 0 || id >= vocab_rows) id = f.pad_id;       // ids outside the weight matrix read the pad row
        const uint4* src = weight + (int64_t)id * pieces;
        uint4* dst = out + tk * pieces;
        for (int p = gl; p < pieces; p += lanes_per_token) dst[p] = __ldg(src + p);
    }
}

}  // namespace dnatok

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

constexpr int EMIT_WARPS = EMIT_THREADS / 32;
constexpr int EMIT_SPAN = 512;           // output columns one warp produces per trip ...
constexpr int EMIT_SPAN_WIDE = 1024;     // ... and for 32-bit ids on long rows, where a trip of 512 stores too little

// Padded output [n_rows, out_stride].  counts == nullptr: a row's content is its byte span.
//
// A warp takes SPAN consecutive columns of one row.  The source elements under those columns are
// fetched as aligned 16-byte chunks (one or two per lane) into a per-warp shared-memory window,
// whatever the row's byte alignment and the one-column shift a leading special token causes; each
// lane then reads the N = 16/sizeof(IdT) elements of its output vector back as aligned words plus a
// funnel shift, maps them (LUT or identity) and issues one 16-byte store, so both the global loads
// and the global stores of a warp are contiguous.  Vectors that touch a special token, the
// truncation point or the padding take a per-column route.
template <typename SrcT, typename IdT, bool USE_LUT, int SPAN>
__global__ void __launch_bounds__(EMIT_THREADS)
emit_padded_kernel(const SrcT* __restrict__ src, const uint8_t* __restrict__ src_begin,
                   const uint8_t* __restrict__ src_end, const int64_t* __restrict__ offsets,
                   const int32_t* __restrict__ counts, int64_t n_rows,
                   const int32_t* __restrict__ lut, RowFormat f, IdT* __restrict__ ids,
                   void* __restrict__ mask, int32_t* __restrict__ lengths_out,
                   int32_t* __restrict__ status, int64_t spans_per_row, int64_t n_spans) {
    constexpr int N = Vec16<IdT>::N;
    constexpr int SZ = (int)sizeof(SrcT);
    constexpr int CHUNKS = SPAN * SZ / 16 + 1;               // 16-byte chunks covering a span at any alignment
    constexpr int VB = N * SZ;                                // source bytes under one output vector: 2, 4 or 8
    // Launched with programmatic stream serialisation: the next launch of the stream may be set up while this grid
    // drains, and this grid starts its work only once everything before it in the stream is complete and visible.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ int32_t s_lut[256];
    __shared__ uint4 s_win[EMIT_WARPS][CHUNKS + 1];
    if (USE_LUT) {
        for (int i = threadIdx.x; i < 256; i += EMIT_THREADS) s_lut[i] = lut[i];
        __syncthreads();
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t* win = reinterpret_cast<const uint32_t*>(s_win[warp]);
    const bool has_cls = f.cls_id >= 0, has_sep = f.sep_id >= 0;
    const int64_t stride = f.out_stride;
    const bool small = n_spans <= 0x7fffffff;

    constexpr int R = (CHUNKS + 31) / 32;                     // window chunks per lane

    struct Span {
        int64_t row, cs, n, T, shift, t_lo;
        const uint8_t* wbase;
        int ncol, a, need;                                    // need: window chunks that hold content of this span
        bool any_content;
    };
    auto describe = [&](int64_t span) {
        Span p;
        if (small) {
            const uint32_t r32 = (uint32_t)span / (uint32_t)spans_per_row;
            p.row = r32;
            p.cs = (int64_t)((uint32_t)span - r32 * (uint32_t)spans_per_row) * SPAN;
        } else {
            p.row = span / spans_per_row;
            p.cs = (span - p.row * spans_per_row) * SPAN;
        }
        const int64_t off = offsets[p.row];
        const int64_t n_in = counts ? (int64_t)counts[p.row] : offsets[p.row + 1] - off;
        p.n = n_in < f.cap_content ? n_in : f.cap_content;
        p.T = p.n + (has_cls ? 1 : 0) + (has_sep ? 1 : 0);
        p.shift = f.pad_left ? stride - p.T : 0;
        if (p.cs == 0 && lane == 0) {
            if (lengths_out) lengths_out[p.row] = (int32_t)p.T;
            if (status) {
                const int32_t bits = (f.clip_is_error && n_in > p.n) ? 4 : 0;
                if (f.store_status) status[p.row] = bits;       // the caller left the words unset: written, not OR-ed
                else if (bits) atomicOr(status + p.row, bits);
            }
        }
        p.ncol = (int)(stride - p.cs < SPAN ? stride - p.cs : SPAN);
        p.t_lo = p.cs - (p.shift + (has_cls ? 1 : 0));        // content index under the span's first column
        const uint8_t* wptr = reinterpret_cast<const uint8_t*>(src + off) + p.t_lo * SZ;
        p.a = (int)(reinterpret_cast<uintptr_t>(wptr) & 15);
        p.wbase = wptr - p.a;
        p.any_content = p.t_lo + p.ncol > 0 && p.t_lo < p.n;  // else the span is specials and padding only
        {
            // content columns of the span end at min(t_lo + ncol, n); chunks past them are not fetched
            const int64_t t_hi = p.t_lo + p.ncol < p.n ? p.t_lo + p.ncol : p.n;
            p.need = p.any_content ? (int)((p.a + (t_hi - p.t_lo) * SZ + 15) >> 4) + 1 : 0;
        }
        return p;
    };
    // the span's source window as aligned 16-byte chunks, into registers
    auto fetch = [&](const Span& p, uint4* regs) {
#pragma unroll
        for (int q = 0; q < R; ++q) {
            const int k = lane + 32 * q;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (k < p.need && k < CHUNKS) {
                const uint8_t* g = p.wbase + 16 * k;
                if (g >= src_begin && g + 16 <= src_end) v = __ldg(reinterpret_cast<const uint4*>(g));
                else {
                    uint8_t tmp[16];
#pragma unroll
                    for (int b = 0; b < 16; ++b) tmp[b] = (g + b >= src_begin && g + b < src_end) ? __ldg(g + b) : (uint8_t)0;
                    v = *reinterpret_cast<uint4*>(tmp);
                }
            }
            regs[q] = v;
        }
    };

    const int64_t span_step = (int64_t)gridDim.x * EMIT_WARPS;
    int64_t span = (int64_t)blockIdx.x * EMIT_WARPS + warp;
    if (span >= n_spans) return;
    Span cur = describe(span);
    uint4 pre[R];
    fetch(cur, pre);
    for (;;) {
        // the window of this span goes to shared memory; the next span's window is requested right away
        __syncwarp();
#pragma unroll
        for (int q = 0; q < R; ++q) if (lane + 32 * q < CHUNKS) s_win[warp][lane + 32 * q] = pre[q];
        __syncwarp();
        const int64_t next = span + span_step;
        const bool more = next < n_spans;
        Span nxt = cur;
        if (more) { nxt = describe(next); fetch(nxt, pre); }

        const int64_t row = cur.row, cs = cur.cs, n = cur.n, T = cur.T, shift = cur.shift, t_lo = cur.t_lo;
        const int ncol = cur.ncol, a = cur.a;
        const bool any_content = cur.any_content;
        IdT* orow = ids + row * stride + cs;
        const bool aligned = (reinterpret_cast<uintptr_t>(orow) & 15) == 0;

        // content occupies columns [c_lo, c_hi) of the span: vectors inside need no per-column checks
        int c_lo = 0, c_hi = 0;
        {
            const int64_t lo64 = t_lo < 0 ? -t_lo : 0, hi64 = n - t_lo;
            c_lo = (int)(lo64 < ncol ? lo64 : ncol);
            c_hi = (int)(hi64 < 0 ? 0 : (hi64 < ncol ? hi64 : ncol));
        }
        // ---- ids
        for (int v = lane; v * N < ncol; v += 32) {
            const int c0 = v * N;                              // column within the span
            const int boff = a + c0 * SZ;                      // byte offset of the vector's source in the window
            const uint32_t sh = (uint32_t)(boff & 3) * 8u;
            const uint32_t* wp = win + (boff >> 2);
            uint32_t lo = 0, hi = 0;
            if (any_content) {
                const uint32_t w0 = wp[0], w1 = wp[1];
                lo = __funnelshift_r(w0, w1, sh);
                if (VB > 4) hi = __funnelshift_r(w1, wp[2], sh);
            }
            IdT vals[N];
            const int64_t t0 = t_lo + c0;
            const bool interior = c0 >= c_lo && c0 + N <= c_hi;
#pragma unroll
            for (int e = 0; e < N; ++e) {
                uint32_t word = (e * SZ < 4) ? lo : hi;
                uint32_t x = SZ == 1 ? (word >> (8 * (e & 3))) & 0xFFu : (word >> (16 * (e & 1))) & 0xFFFFu;
                int32_t val = USE_LUT ? s_lut[x & 0xFFu] : (int32_t)x;
                if (!interior) {
                    const int64_t t = t0 + e;                  // content index of this column
                    const int64_t col = cs + c0 + e - shift;   // token index within the row
                    if (t < 0 || t >= n) {
                        val = f.pad_id;
                        if (has_cls && col == 0) val = f.cls_id;
                        else if (has_sep && col == T - 1 && col >= 0) val = f.sep_id;
                    }
                }
                vals[e] = (IdT)val;
            }
            if (aligned && c0 + N <= ncol) store_vec<IdT>(orow + c0, vals);
            else {
#pragma unroll
                for (int e = 0; e < N; ++e) if (c0 + e < ncol) orow[c0 + e] = vals[e];
            }
        }

        // ---- mask: ones on [shift, shift + T)
        if (f.mask_bits) {
            const int64_t lo = shift - cs, hi = shift + T - cs;
            if (f.mask_bits == 64) warp_mask_row<int64_t>((int64_t*)mask + row * stride + cs, ncol, lo, hi, lane);
            else if (f.mask_bits == 32) warp_mask_row<int32_t>((int32_t*)mask + row * stride + cs, ncol, lo, hi, lane);
            else warp_mask_row<uint8_t>((uint8_t*)mask + row * stride + cs, ncol, lo, hi, lane);
        }
        if (!more) break;
        span = next;
        cur = nxt;
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
        // A thread's elements rise through the tile, so the row under them only moves forward: its bounds and the place of
        // its source stay in registers and are fetched again only when an element lies past the row's end.
        int64_t lo = r_lo, row_start = 0, row_end = -1, src_at = 0;
        for (int64_t c = e0 + (int64_t)threadIdx.x * N; c < e1; c += (int64_t)EMIT_THREADS * N) {
            IdT vals[N];
#pragma unroll
            for (int e = 0; e < N; ++e) {
                const int64_t g = c + e;
                int32_t v = f.pad_id;
                if (g < e1) {
                    if (g >= row_end) {
                        int64_t hi = r_hi;          // rows are ordered, so the search restarts at lo
                        while (lo < hi) {
                            const int64_t mid = (lo + hi + 1) >> 1;
                            if (out_offsets[mid] <= g) lo = mid; else hi = mid - 1;
                        }
                        row_start = out_offsets[lo];
                        row_end = out_offsets[lo + 1];
                        src_at = offsets[lo] - (has_cls ? 1 : 0);
                    }
                    const int64_t t = g - row_start;
                    if (has_cls && t == 0) v = f.cls_id;
                    else if (has_sep && g == row_end - 1) v = f.sep_id;
                    else v = emit_load<SrcT, USE_LUT>(src + src_at + t, s_lut);
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

// Tokenizers whose id of a row's first character differs from the id the same character gets later
// (the reference keeps a second "start" table for them and patches column 0,
// src/dna_tokenizer.py:1779-1820 with :527-631): after the rows are written, one thread per row puts
// the start id under the row's first content column.
template <typename IdT>
__global__ void start_fix_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets, int64_t n_rows,
                                 const int32_t* __restrict__ start_lut, RowFormat f, IdT* __restrict__ ids,
                                 const int64_t* __restrict__ out_offsets) {
    const int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= n_rows) return;
    const int64_t off = offsets[row], n_in = offsets[row + 1] - off;
    const int64_t n = n_in < f.cap_content ? n_in : f.cap_content;
    if (n <= 0) return;
    const int has_cls = f.cls_id >= 0 ? 1 : 0, has_sep = f.sep_id >= 0 ? 1 : 0;
    const IdT v = (IdT)__ldg(start_lut + __ldg(bytes + off));
    if (f.out_stride == 0) { ids[out_offsets[row] + has_cls] = v; return; }
    const int64_t T = n + has_cls + has_sep;
    const int64_t shift = f.pad_left ? f.out_stride - T : 0;
    ids[row * f.out_stride + shift + has_cls] = v;
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

// Exclusive scan of int32 lengths into int64 offsets, one block, 4,096 rows per trip: every thread takes four
// consecutive lengths (one 16-byte load), so a batch of a few thousand rows is one load, one block-wide scan and
// one round of stores instead of a chain of them.
__global__ void __launch_bounds__(1024)
scan_lengths_kernel(const int32_t* __restrict__ lengths, int64_t n_rows, int64_t* __restrict__ out_offsets) {
    __shared__ int64_t s_warp[32];
    __shared__ int64_t s_carry;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) { s_carry = 0; out_offsets[0] = 0; }
    __syncthreads();
    const bool vec_ok = (reinterpret_cast<uintptr_t>(lengths) & 15) == 0;
    for (int64_t base = 0; base < n_rows; base += 4096) {
        const int64_t i = base + 4 * (int64_t)tid;
        int32_t l[4] = {0, 0, 0, 0};
        if (vec_ok && i + 4 <= n_rows) {
            const int4 q = *reinterpret_cast<const int4*>(lengths + i);
            l[0] = q.x; l[1] = q.y; l[2] = q.z; l[3] = q.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) if (i + e < n_rows) l[e] = lengths[i + e];
        }
        const int64_t v = (int64_t)l[0] + l[1] + l[2] + l[3];
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
        const int64_t incl = x + (warp ? s_warp[warp - 1] : 0) + s_carry;     // through this thread's four rows
        int64_t run = incl - v;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            run += l[e];
            if (i + e < n_rows) out_offsets[i + e + 1] = run;
        }
        __syncthreads();
        if (tid == 1023) s_carry = incl;
        __syncthreads();
    }
}

}  // namespace dnatok

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

// ---------------------------------------------------------------------------------------------
// Warp-per-row variant for batches of short and medium rows (reads, 6,000-bp windows): no shared
// memory and no block-wide barrier.  Per iteration a warp covers 64 windows; each lane owns two
// consecutive windows (2K bytes), fetched as aligned 32-bit words and re-aligned with funnel
// shifts, turned into 2-bit codes four bytes at a time, and - when every window of the chunk is a
// clean k-mer, the common case - stored as one 16-byte pair of ids at position base + 2*lane.  A
// chunk holding any other window (N, lower case, the len%K tail) takes the general route: per-lane
// token counts, a warp scan, scalar stores.
namespace dnatok {

constexpr int KW_WARPS = 8;
// Row-per-warp encoder: two rows (warps) per block, because a block's slot is only refilled when its slowest
// row is done (rows with N runs take longer); 16 such blocks per SM (32 warps, up to 64 registers per thread):
// the long loop keeps the words of four chunks in flight per lane, which pays more than a third more warps
// with half the loads each.
constexpr int KW_ROW_WARPS = 2;
constexpr int KW_BLOCKS_PER_SM = 16;
constexpr int KW_TRIP_CHUNKS = 4;       // clean chunks of 64 windows per trip of the long loop

// 2-bit codes of four ASCII bytes at once (A C G T -> 0 1 2 3 in each byte's low bits), and a word
// that is zero exactly in the bytes that are one of A, C, G, T.
__device__ __forceinline__ void acgt_codes4(uint32_t w, uint32_t* code, uint32_t* diff) {
    uint32_t c = (w >> 1) & 0x03030303u;
    c ^= (c >> 1) & 0x01010101u;
    const uint32_t c0 = c & 0x01010101u, c1 = (c >> 1) & 0x01010101u, c01 = c0 & c1;
    // 'A' + {0, 2, 6, 19}[code] is the only byte value that maps to this code legitimately
    const uint32_t expect = 0x41414141u + 2u * c0 + 6u * c1 + 11u * c01;
    *code = c;
    *diff = w ^ expect;
}

// Gather the four 2-bit codes of a word into 8 bits, first byte most significant.
__device__ __forceinline__ uint32_t pack_codes4(uint32_t code) { return (code * 0x40100401u) >> 24; }

template <typename IdT> struct IdPair;
template <> struct IdPair<int64_t> { using type = longlong2; };
template <> struct IdPair<int32_t> { using type = int2; };

// Tokens of windows [w_begin, w_end) of one row, counted by one warp with the encoder's window
// decoding and no stores; counting stops once `stop_at` tokens are reached.  *done tells whether the
// whole range was looked at.
template <int K>
__device__ __forceinline__ int kmer_count_windows(const uint8_t* __restrict__ src, int len, int64_t room_total, int lane,
                                                  int w_begin, int w_end, int stop_at, bool* done) {
    constexpr int NW = (2 * K + 3 + 3) / 4;
    const int n_full = len / K;
    int total = 0, w0 = w_begin;
    for (; w0 < w_end && total < stop_at; w0 += 64) {
        const int wa = w0 + 2 * lane;
        const int lim = w0 + 64 < w_end ? w0 + 64 : w_end;
        const int p = wa * K;
        int cnt = 0;
        if (wa + 2 <= lim && wa + 2 <= n_full && (int64_t)p + 2 * K + 8 <= room_total) {
            const uint8_t* g = src + p;
            const uint32_t sh = (uint32_t)(reinterpret_cast<uintptr_t>(g) & 3u) * 8u;
            const uint32_t* gw = reinterpret_cast<const uint32_t*>(g - (sh >> 3));
            uint32_t w[NW];
#pragma unroll
            for (int i = 0; i < NW; ++i) w[i] = __ldg(gw + i);
            uint32_t dA = 0, dB = 0;
#pragma unroll
            for (int i = 0; i < NW - 1; ++i) {
                const uint32_t r = __funnelshift_r(w[i], w[i + 1], sh);
                uint32_t c, d;
                acgt_codes4(r, &c, &d);
                uint32_t mA = 0, mB = 0;
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const int pos = 4 * i + b;
                    if (pos < K) mA |= 0xFFu << (8 * b);
                    else if (pos < 2 * K) mB |= 0xFFu << (8 * b);
                }
                dA |= d & mA;
                dB |= d & mB;
            }
            cnt = (dA == 0 ? 1 : K) + (dB == 0 ? 1 : K);
        } else {
            int lenA = 0, lenB = 0;
            if (wa < lim) { const int h = len - p; lenA = h < K ? h : K; }
            if (wa + 1 < lim) { const int h = len - p - K; lenB = h < K ? h : K; }
            bool okA = lenA == K, okB = lenB == K;
            for (int i = 0; i < lenA; ++i) okA &= kmer_code(__ldg(src + p + i)) < 4;
            for (int i = 0; i < lenB; ++i) okB &= kmer_code(__ldg(src + p + K + i)) < 4;
            cnt = (lenA == 0 ? 0 : (okA ? 1 : lenA)) + (lenB == 0 ? 0 : (okB ? 1 : lenB));
        }
        total += __reduce_add_sync(0xffffffffu, cnt);
    }
    *done = w0 >= w_end;
    return total;
}

// Token counts only (the sizing pass for 'longest' padding and for ragged output): one warp per row.
template <int K>
__global__ void __launch_bounds__(KW_WARPS * 32)
kmer_warp_count_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets, int64_t n_rows,
                       int64_t total_bytes, RowFormat f, int32_t* __restrict__ lengths_out,
                       int32_t* __restrict__ status) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * KW_WARPS + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const int n_special = (f.cls_id >= 0 ? 1 : 0) + (f.sep_id >= 0 ? 1 : 0);
    const int64_t off = offsets[row];
    const int64_t len64 = offsets[row + 1] - off;
    const int len = (int)(len64 < 0x7fffffff ? len64 : 0x7fffffff);
    const int n_win = (len + K - 1) / K;
    const int cap = (int)(f.cap_content < 0x7fffffff ? f.cap_content : 0x7fffffff);
    bool done;
    const int base = kmer_count_windows<K>(bytes + off, len, total_bytes - off, lane, 0, n_win, cap, &done);
    if (lane == 0) {
        const int n = base < cap ? base : cap;
        lengths_out[row] = n + n_special;
        if (status && f.clip_is_error && (base > cap || !done)) atomicOr(status + row, 4);
    }
}

// The same count for batches of few or very long rows: every warp counts segments of KSEG_WINDOWS
// windows (ticket t = segment t / n_rows of row t % n_rows, the last segment index without upper
// bound) and adds them to counts[row], which the caller zeroed and turns into lengths afterwards.
template <int K>
__global__ void __launch_bounds__(KW_WARPS * 32)
kmer_seg_count_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets, int64_t n_rows,
                      int64_t total_bytes, int n_seg, int seg_windows, int32_t* __restrict__ counts) {
    const int lane = threadIdx.x & 31;
    const int64_t n_tickets = n_rows * (int64_t)n_seg;
    const int64_t n_warps = (int64_t)gridDim.x * KW_WARPS;
    for (int64_t t = (int64_t)blockIdx.x * KW_WARPS + (threadIdx.x >> 5); t < n_tickets; t += n_warps) {
        const int seg = (int)(t / n_rows);
        const int64_t row = t - (int64_t)seg * n_rows;
        const int64_t off = offsets[row];
        const int64_t len64 = offsets[row + 1] - off;
        const int len = (int)(len64 < 0x7fffffff ? len64 : 0x7fffffff);
        const int n_win = (len + K - 1) / K;
        const int64_t w0 = (int64_t)seg * seg_windows;
        if (w0 >= n_win) continue;
        const int w_end = (seg == n_seg - 1 || w0 + seg_windows >= n_win) ? n_win : (int)w0 + seg_windows;
        bool done;
        const int cnt = kmer_count_windows<K>(bytes + off, len, total_bytes - off, lane, (int)w0, w_end, 0x7fffffff, &done);
        if (lane == 0 && cnt) atomicAdd(counts + row, cnt);
    }
}

// Everything one row's windows need, resolved once per row (or per row segment).
template <typename IdT>
struct KmerRow {
    const uint8_t* src;        // first byte of the row
    int len;                   // bytes in the row
    int n_win;                 // windows, the short last one included
    int64_t room_total;        // bytes from the row start to the end of the input buffer
    IdT* orow;                 // first output column of the row
    IdT* dst;                  // first content column (after padding and [CLS])
    int shift;                 // left padding columns
};

// A row of 2 GiB or more is encoded up to its first 2^31 - 1 bytes and reported.
__device__ __forceinline__ void kmer_flag_long_row(int64_t len64, int32_t* status, int64_t row, int lane) {
    if (len64 > 0x7fffffff && status && lane == 0) atomicOr(status + row, 1);
}

// off, end: the row's bounds in the input buffer (offsets[row], offsets[row + 1])
template <typename IdT, int K>
__device__ __forceinline__ KmerRow<IdT> kmer_row_setup(const uint8_t* bytes, int64_t off, int64_t end, int64_t row,
                                                       int64_t total_bytes, const RowFormat& f, IdT* ids,
                                                       const int32_t* lengths_in, const int64_t* out_offsets) {
    KmerRow<IdT> r;
    const int64_t len64 = end - off;
    r.len = (int)(len64 < 0x7fffffff ? len64 : 0x7fffffff);              // a longer row is cut here and flagged (kmer_flag_long_row)
    r.n_win = (r.len + K - 1) / K;
    r.src = bytes + off;
    r.room_total = total_bytes - off;
    const bool ragged = f.out_stride == 0;
    r.orow = ragged ? ids + out_offsets[row] : ids + row * f.out_stride;
    r.shift = 0;
    if (!ragged && f.pad_left) r.shift = (int)f.out_stride - lengths_in[row];
    r.dst = r.orow + r.shift + (f.cls_id >= 0 ? 1 : 0);
    return r;
}

// One warp encodes windows [w, w_end) of a row whose earlier windows produced `base` content tokens;
// returns the token count after them (it stops early once the cap is reached) and reports clipping.
// AFFINE: the 4**K table is base + index (checked on the host), so no gather is needed.
// FUSE_MASK: the mask has the ids' element type and is stored next to each id (mdelta elements away).
template <typename IdT, int K, bool AFFINE, bool FUSE_MASK>
__device__ __forceinline__ int kmer_encode_windows(const KmerRow<IdT>& r, int cap, const int32_t* __restrict__ kmer_ids,
                                                   int32_t affine_base, const int32_t* __restrict__ single_ids,
                                                   int64_t mdelta, int lane, int w, int w_end, int base, bool* clipped) {
    constexpr int NW = (2 * K + 3 + 3) / 4;            // aligned words covering 2K bytes at any byte offset
    constexpr uint32_t IDX_MASK = (1u << (2 * K)) - 1u;
    using Pair = typename IdPair<IdT>::type;
    const uint8_t* src = r.src;
    const int len = r.len;
    const int64_t room_total = r.room_total;
    IdT* dst = r.dst;
    IdT* mdst = dst + mdelta;
    const int n_full = len / K;                          // complete windows

    // The two windows of this lane in the chunk of `nwin` windows starting at window w0:
    // lengths, table indices, cleanliness.
    struct Two { int lenA, lenB; uint32_t idxA, idxB; bool cleanA, cleanB; int p; };
    auto decode = [&](int w0, int nwin) {
        Two t;
        const int wa = w0 + 2 * lane;
        int lim = w0 + nwin;                              // one past the chunk's last window
        if (lim > w_end) lim = w_end;
        t.p = wa * K;
        t.idxA = 0; t.idxB = 0;
        // both windows complete, inside the chunk, and the aligned words inside the buffer: the wide route
        if (wa + 2 <= lim && wa + 2 <= n_full && (int64_t)t.p + 2 * K + 8 <= room_total) {
            t.lenA = K; t.lenB = K;
            const uint8_t* g = src + t.p;
            const uint32_t sh = (uint32_t)(reinterpret_cast<uintptr_t>(g) & 3u) * 8u;
            const uint32_t* gw = reinterpret_cast<const uint32_t*>(g - (sh >> 3));
            uint32_t wd[NW];
#pragma unroll
            for (int i = 0; i < NW; ++i) wd[i] = __ldg(gw + i);
            uint32_t P = 0, dA = 0, dB = 0;
#pragma unroll
            for (int i = 0; i < NW - 1; ++i) {
                const uint32_t rr = __funnelshift_r(wd[i], wd[i + 1], sh);    // bytes 4i .. 4i+3 of the pair
                uint32_t c, d;
                acgt_codes4(rr, &c, &d);
                P |= pack_codes4(c) << (24 - 8 * i);
                // byte b of this word belongs to window A when 4i+b < K, to window B when K <= 4i+b < 2K
                uint32_t mA = 0, mB = 0;
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const int pos = 4 * i + b;
                    if (pos < K) mA |= 0xFFu << (8 * b);
                    else if (pos < 2 * K) mB |= 0xFFu << (8 * b);
                }
                dA |= d & mA;
                dB |= d & mB;
            }
            t.cleanA = dA == 0;
            t.cleanB = dB == 0;
            t.idxA = (P >> (32 - 2 * K)) & IDX_MASK;
            t.idxB = (P >> (32 - 4 * K)) & IDX_MASK;
        } else {
            // edge of the chunk, of the row or of the buffer: byte loads
            t.lenA = 0; t.lenB = 0;
            if (wa < lim) { const int h = len - t.p; t.lenA = h < K ? h : K; }
            if (wa + 1 < lim) { const int h = len - t.p - K; t.lenB = h < K ? h : K; }
            bool okA = t.lenA == K, okB = t.lenB == K;
            for (int i = 0; i < t.lenA; ++i) { const int c = kmer_code(__ldg(src + t.p + i)); okA &= c < 4; t.idxA = (t.idxA << 2) | (uint32_t)(c & 3); }
            for (int i = 0; i < t.lenB; ++i) { const int c = kmer_code(__ldg(src + t.p + K + i)); okB &= c < 4; t.idxB = (t.idxB << 2) | (uint32_t)(c & 3); }
            t.cleanA = okA; t.cleanB = okB;
        }
        return t;
    };
    auto emit = [&](int w0, int nwin, const Two& t) {
        const bool simple = (t.lenA == 0 || t.cleanA) && (t.lenB == 0 || t.cleanB);
        if (__all_sync(0xffffffffu, simple)) {
            // every window of the chunk is one token: this lane's tokens sit at base + 2*lane (+1)
            const int pos = base + 2 * lane;
            const IdT a = t.lenA ? (IdT)(AFFINE ? affine_base + (int32_t)t.idxA : __ldg(kmer_ids + t.idxA)) : (IdT)0;
            const IdT b = t.lenB ? (IdT)(AFFINE ? affine_base + (int32_t)t.idxB : __ldg(kmer_ids + t.idxB)) : (IdT)0;
            if (t.lenB && pos + 1 < cap && (reinterpret_cast<uintptr_t>(dst + pos) % (2 * sizeof(IdT))) == 0) {
                Pair v; v.x = a; v.y = b;
                *reinterpret_cast<Pair*>(dst + pos) = v;
                if (FUSE_MASK) { Pair one; one.x = 1; one.y = 1; *reinterpret_cast<Pair*>(mdst + pos) = one; }
            } else {
                if (t.lenA && pos < cap) { dst[pos] = a; if (FUSE_MASK) mdst[pos] = 1; }
                if (t.lenB && pos + 1 < cap) { dst[pos + 1] = b; if (FUSE_MASK) mdst[pos + 1] = 1; }
            }
            const int left = w_end - w0;
            base += left < nwin ? left : nwin;
        } else {
            const int cntA = t.lenA == 0 ? 0 : (t.cleanA ? 1 : t.lenA);
            const int cntB = t.lenB == 0 ? 0 : (t.cleanB ? 1 : t.lenB);
            int my = cntA + cntB, x = my;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int y = __shfl_up_sync(0xffffffffu, x, d);
                if (lane >= d) x += y;
            }
            const int total = __shfl_sync(0xffffffffu, x, 31);
            int pos = base + x - my;
            if (t.lenA) {
                if (t.cleanA) { if (pos < cap) { dst[pos] = (IdT)__ldg(kmer_ids + t.idxA); if (FUSE_MASK) mdst[pos] = 1; } ++pos; }
                else for (int i = 0; i < t.lenA; ++i, ++pos) if (pos < cap) { dst[pos] = (IdT)__ldg(single_ids + __ldg(src + t.p + i)); if (FUSE_MASK) mdst[pos] = 1; }
            }
            if (t.lenB) {
                if (t.cleanB) { if (pos < cap) { dst[pos] = (IdT)__ldg(kmer_ids + t.idxB); if (FUSE_MASK) mdst[pos] = 1; } ++pos; }
                else for (int i = 0; i < t.lenB; ++i, ++pos) if (pos < cap) { dst[pos] = (IdT)__ldg(single_ids + __ldg(src + t.p + K + i)); if (FUSE_MASK) mdst[pos] = 1; }
            }
            base += total;
        }
    };

    // Wide-route decode of the two windows held in wd (no bounds checks): table indices and a word
    // that is non-zero when either window holds anything but ACGT.
    auto load_words = [&](const uint32_t* gw, uint32_t* wd) {
#pragma unroll
        for (int i = 0; i < NW; ++i) wd[i] = __ldg(gw + i);
    };
    auto decode_words = [&](const uint32_t* wd, uint32_t sh, uint32_t* idxA, uint32_t* idxB) -> uint32_t {
        uint32_t P = 0, bad = 0;
#pragma unroll
        for (int i = 0; i < NW - 1; ++i) {
            const uint32_t rr = __funnelshift_r(wd[i], wd[i + 1], sh);
            uint32_t c, d;
            acgt_codes4(rr, &c, &d);
            P |= pack_codes4(c) << (24 - 8 * i);
            uint32_t m = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) if (4 * i + b < 2 * K) m |= 0xFFu << (8 * b);
            bad |= d & m;
        }
        *idxA = (P >> (32 - 2 * K)) & IDX_MASK;
        *idxB = (P >> (32 - 4 * K)) & IDX_MASK;
        return bad;
    };
    // windows [0, n_tight) are complete, inside [.., w_end) and their aligned words stay in the buffer
    int n_tight = n_full < w_end ? n_full : w_end;
    {
        const int64_t fit = (room_total - 8) / K;
        if (fit < n_tight) n_tight = fit < 0 ? 0 : (int)fit;
    }
    Pair one; one.x = 1; one.y = 1;

    bool peel = true;          // an odd element offset is first answered by a chunk of one window
    while (w < w_end && base < cap) {
        // 16-byte stores need an even element offset.  After an odd number of tokens (the [CLS] slot,
        // a chunk with single-base fallbacks) one window on its own puts the row back in step when it
        // is a clean k-mer; if it was not, a chunk of 63 windows follows.
        const bool al = (reinterpret_cast<uintptr_t>(dst + base) % (2 * sizeof(IdT))) == 0;
        if (al) {
            peel = true;
            bool dirty = false;
            // tight stretch: clean full chunks, two per trip, no per-token checks
            const uint8_t* g = src + (w + 2 * lane) * K;
            const uint32_t sh = (uint32_t)(reinterpret_cast<uintptr_t>(g) & 3u) * 8u;   // constant while w moves by 64: 64K % 4 == 0
            const uint32_t* gw = reinterpret_cast<const uint32_t*>(g - (sh >> 3));
            IdT* d = dst + base + 2 * lane;
            // KW_TRIP_CHUNKS clean chunks per trip while they last: more loads in flight per wait
            {
                constexpr int NCH = KW_TRIP_CHUNKS;
                while (w + 64 * NCH <= n_tight && base + 64 * NCH <= cap) {
                    uint32_t q[NCH][NW];
#pragma unroll
                    for (int i = 0; i < NCH; ++i) load_words(gw + i * 16 * K, q[i]);
                    uint32_t ia[NCH], ib[NCH], bad = 0;
#pragma unroll
                    for (int i = 0; i < NCH; ++i) bad |= decode_words(q[i], sh, &ia[i], &ib[i]);
                    if (__any_sync(0xffffffffu, bad != 0)) { dirty = true; break; }   // the two-chunk loop below sorts it out
#pragma unroll
                    for (int i = 0; i < NCH; ++i) {
                        Pair v;
                        v.x = (IdT)(AFFINE ? affine_base + (int32_t)ia[i] : __ldg(kmer_ids + ia[i]));
                        v.y = (IdT)(AFFINE ? affine_base + (int32_t)ib[i] : __ldg(kmer_ids + ib[i]));
                        *reinterpret_cast<Pair*>(d + 64 * i) = v;
                        if (FUSE_MASK) *reinterpret_cast<Pair*>(d + mdelta + 64 * i) = one;
                    }
                    gw += NCH * 16 * K; d += 64 * NCH; base += 64 * NCH; w += 64 * NCH;
                }
                dirty = false;                                    // the loops below look again
            }
            while (w + 128 <= n_tight && base + 128 <= cap) {
                uint32_t c0[NW], c1[NW];
                load_words(gw, c0);
                load_words(gw + 16 * K, c1);
                uint32_t a0, b0, a1, b1;
                const uint32_t bad0 = decode_words(c0, sh, &a0, &b0);
                const uint32_t bad1 = decode_words(c1, sh, &a1, &b1);
                Pair v0, v1;
                v0.x = (IdT)(AFFINE ? affine_base + (int32_t)a0 : __ldg(kmer_ids + a0));
                v0.y = (IdT)(AFFINE ? affine_base + (int32_t)b0 : __ldg(kmer_ids + b0));
                if (__any_sync(0xffffffffu, (bad0 | bad1) != 0)) {
                    // the general route takes over; a clean first chunk is still placed from here
                    if (!__any_sync(0xffffffffu, bad0 != 0)) {
                        *reinterpret_cast<Pair*>(d) = v0;
                        if (FUSE_MASK) *reinterpret_cast<Pair*>(d + mdelta) = one;
                        base += 64; w += 64;
                    }
                    dirty = true;
                    break;
                }
                v1.x = (IdT)(AFFINE ? affine_base + (int32_t)a1 : __ldg(kmer_ids + a1));
                v1.y = (IdT)(AFFINE ? affine_base + (int32_t)b1 : __ldg(kmer_ids + b1));
                *reinterpret_cast<Pair*>(d) = v0;
                *reinterpret_cast<Pair*>(d + 64) = v1;
                if (FUSE_MASK) { *reinterpret_cast<Pair*>(d + mdelta) = one; *reinterpret_cast<Pair*>(d + mdelta + 64) = one; }
                gw += 32 * K; d += 128; base += 128; w += 128;
            }
            // one more clean full chunk where two no longer fit
            if (!dirty && w + 64 <= n_tight && base + 64 <= cap) {
                uint32_t a0, b0, c0[NW];
                load_words(gw, c0);
                const uint32_t bad0 = decode_words(c0, sh, &a0, &b0);
                if (!__any_sync(0xffffffffu, bad0 != 0)) {
                    Pair v0;
                    v0.x = (IdT)(AFFINE ? affine_base + (int32_t)a0 : __ldg(kmer_ids + a0));
                    v0.y = (IdT)(AFFINE ? affine_base + (int32_t)b0 : __ldg(kmer_ids + b0));
                    *reinterpret_cast<Pair*>(d) = v0;
                    if (FUSE_MASK) *reinterpret_cast<Pair*>(d + mdelta) = one;
                    base += 64; w += 64;
                }
            }
            if (w >= w_end) break;
            if (base >= cap) break;
        }
        // one chunk by the general route (dirty windows, row edges, the last tokens before the cap)
        const int nwin = al ? 64 : (peel ? 1 : 63);
        if (!al) peel = false;
        const Two t0 = decode(w, nwin);
        emit(w, nwin, t0);
        w += nwin;
    }
    if (w < w_end) *clipped = true;
    if (base > cap) *clipped = true;
    return base;
}

// What remains once the content tokens of a row are placed: lengths, [CLS]/[SEP], padding, mask.
template <typename IdT, bool FUSE_MASK>
__device__ __forceinline__ void kmer_finish_row(const KmerRow<IdT>& r, int64_t row, int base, int cap, bool clipped,
                                                const RowFormat& f, IdT* ids, void* mask, int32_t* lengths_out,
                                                const int64_t* out_offsets, int32_t* status, int lane, int32_t more_bits = 0) {
    const bool has_cls = f.cls_id >= 0, has_sep = f.sep_id >= 0;
    const bool ragged = f.out_stride == 0;
    const int n = base < cap ? base : cap;
    const int T = n + (has_cls ? 1 : 0) + (has_sep ? 1 : 0);
    IdT* orow = r.orow;
    const int shift = r.shift;
    if (lane == 0) {
        if (lengths_out) lengths_out[row] = (int32_t)T;
        if (status) {
            const int32_t bits = more_bits | ((f.clip_is_error && clipped) ? 4 : 0);
            if (f.store_status) status[row] = bits;
            else if (bits) atomicOr(status + row, bits);
        }
        if (has_cls) { orow[shift] = (IdT)f.cls_id; if (FUSE_MASK) (reinterpret_cast<IdT*>(mask) + (orow - ids))[shift] = 1; }
        if (has_sep) { orow[shift + T - 1] = (IdT)f.sep_id; if (FUSE_MASK) (reinterpret_cast<IdT*>(mask) + (orow - ids))[shift + T - 1] = 1; }
    }
    if (!ragged) {
        const int stride = (int)f.out_stride;
        const IdT pad = (IdT)f.pad_id;
        if (f.pad_left) warp_write_run<IdT>(orow, shift, lane, [=](int64_t) { return pad; });
        else warp_write_run<IdT>(orow + T, stride - T, lane, [=](int64_t) { return pad; });
        if (FUSE_MASK) {
            IdT* mrow = reinterpret_cast<IdT*>(mask) + row * f.out_stride;
            if (f.pad_left) warp_write_run<IdT>(mrow, shift, lane, [](int64_t) { return (IdT)0; });
            else warp_write_run<IdT>(mrow + T, stride - T, lane, [](int64_t) { return (IdT)0; });
        } else if (f.mask_bits == 64) warp_mask_row<int64_t>((int64_t*)mask + row * f.out_stride, stride, shift, shift + T, lane);
        else if (f.mask_bits == 32) warp_mask_row<int32_t>((int32_t*)mask + row * f.out_stride, stride, shift, shift + T, lane);
        else if (f.mask_bits == 8) warp_mask_row<uint8_t>((uint8_t*)mask + row * f.out_stride, stride, shift, shift + T, lane);
    } else if (mask && f.mask_bits && !FUSE_MASK) {
        const int64_t o = out_offsets[row];
        if (f.mask_bits == 64) warp_write_run<int64_t>((int64_t*)mask + o, T, lane, [](int64_t) { return (int64_t)1; });
        else if (f.mask_bits == 32) warp_write_run<int32_t>((int32_t*)mask + o, T, lane, [](int64_t) { return (int32_t)1; });
        else warp_write_run<uint8_t>((uint8_t*)mask + o, T, lane, [](int64_t) { return (uint8_t)1; });
    }
}

// One warp per row, no scratch memory: used when the caller passes no scratch buffer.
template <typename IdT, int K, bool AFFINE, bool FUSE_MASK>
__global__ void __launch_bounds__(KW_ROW_WARPS * 32, KW_BLOCKS_PER_SM)
kmer_warp_rows_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets, int64_t n_rows,
                      int64_t total_bytes, const int32_t* __restrict__ kmer_ids, int32_t affine_base,
                      const int32_t* __restrict__ single_ids, RowFormat f, IdT* __restrict__ ids,
                      void* __restrict__ mask, const int32_t* __restrict__ lengths_in,
                      int32_t* __restrict__ lengths_out, const int64_t* __restrict__ out_offsets,
                      int32_t* __restrict__ status) {
    // Launched with programmatic stream serialisation: the next launch of the stream may be set up while this grid
    // drains, and this grid starts its work only once everything before it in the stream is complete and visible.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * KW_ROW_WARPS + (threadIdx.x >> 5);
    if (row >= n_rows) return;
    const KmerRow<IdT> r = kmer_row_setup<IdT, K>(bytes, offsets[row], offsets[row + 1], row, total_bytes, f, ids, lengths_in,
                                                  out_offsets);
    const int cap = (int)(f.cap_content < 0x7fffffff ? f.cap_content : 0x7fffffff);
    const int64_t mdelta = FUSE_MASK ? (reinterpret_cast<IdT*>(mask) - ids) : 0;
    const int32_t long_bit = offsets[row + 1] - offsets[row] > 0x7fffffff ? 1 : 0;    // cut at 2^31 - 1 bytes and reported
    bool clipped = false;
    const int base = kmer_encode_windows<IdT, K, AFFINE, FUSE_MASK>(r, cap, kmer_ids, affine_base, single_ids, mdelta, lane,
                                                                    0, r.n_win, 0, &clipped);
    kmer_finish_row<IdT, FUSE_MASK>(r, row, base, cap, clipped, f, ids, mask, lengths_out, out_offsets, status, lane, long_bit);
}

// Rows cut into segments of KSEG_WINDOWS windows.  Ticket t stands for segment t / n_rows of row
// t % n_rows; the warps draw tickets in rising order from a counter in the scratch buffer.
// A segment's place in the output depends on the tokens all earlier segments of its row produce
// (a window with an N yields K tokens, not one), which is settled by a decoupled look-back:
//   1. the warp loads and decodes its 256 windows into registers and counts their tokens;
//   2. it publishes that count in flags[segment * n_rows + row] as an "own" value;
//   3. it sums the "own" values of the segments before it, 32 per step, back to the nearest one that
//      already published a "total" (its own count plus everything before it) or to the row start;
//   4. it publishes its "total" and stores its tokens.
// Nothing is awaited before step 2, so the segments of one row run in parallel, and step 3 only
// waits for flags of earlier tickets.  A ticket is drawn by a warp that is running, and the warp
// reaches step 2 of that ticket without waiting for anybody, so the holders of the flags a warp
// waits for always make progress, however much of the grid the GPU keeps resident.  The waits are
// bounded all the same (poll_limit polls): a row whose wait ran out is reported with
// DNATOK_ROW_STALLED instead of tokens.  `withhold` (tests only, -1 otherwise) names a ticket whose
// holder publishes nothing, which is how the tests make a wait run out.
// The last segment of a row (short windows, the len % K tail) and segments that hold anything but
// clean k-mers place their tokens through kmer_encode_windows; clean ones store straight from
// registers, as 16-byte pairs whatever the parity of their output offset.
constexpr int KSEG_WINDOWS = 256;        // four chunks of 64 windows
constexpr int KSEG_BLOCKS_PER_SM = 4;    // 64 registers per thread: the decoded segment stays in registers
constexpr int KSEG_POLL_LIMIT = 1 << 20;    // default bound on the polls of one wait
constexpr uint32_t KSEG_OWN = 1u << 30, KSEG_TOTAL = 2u << 30, KSEG_POISON = 3u << 30, KSEG_VALUE = (1u << 30) - 1u;

template <typename IdT, int K, bool AFFINE, bool FUSE_MASK>
__global__ void __launch_bounds__(KW_WARPS * 32, KSEG_BLOCKS_PER_SM)
kmer_seg_rows_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets, int64_t n_rows,
                     int64_t total_bytes, const int32_t* __restrict__ kmer_ids, int32_t affine_base,
                     const int32_t* __restrict__ single_ids, RowFormat f, IdT* __restrict__ ids,
                     void* __restrict__ mask, const int32_t* __restrict__ lengths_in,
                     int32_t* __restrict__ lengths_out, const int64_t* __restrict__ out_offsets,
                     int32_t* __restrict__ status, int n_seg, uint32_t* __restrict__ flags,
                     unsigned long long* __restrict__ ticket_counter, int poll_limit, long long withhold) {
    constexpr int NW = (2 * K + 3 + 3) / 4;
    constexpr uint32_t IDX_MASK = (1u << (2 * K)) - 1u;
    constexpr int NCH = KSEG_WINDOWS / 64;
    using Pair = typename IdPair<IdT>::type;
    const int lane = threadIdx.x & 31;
    const int cap = (int)(f.cap_content < 0x7fffffff ? f.cap_content : 0x7fffffff);
    const int64_t mdelta = FUSE_MASK ? (reinterpret_cast<IdT*>(mask) - ids) : 0;
    const int64_t n_tickets = n_rows * (int64_t)n_seg;
    for (;;) {
        unsigned long long drawn = 0;
        if (lane == 0) drawn = atomicAdd(ticket_counter, 1ull);
        const int64_t t = (int64_t)__shfl_sync(0xffffffffu, drawn, 0);
        if (t >= n_tickets) break;
        const int seg = (int)(t / n_rows);
        const int64_t row = t - (int64_t)seg * n_rows;
        const int64_t off = offsets[row], end = offsets[row + 1];
        const bool publish = t != (int64_t)withhold;

        const KmerRow<IdT> r = kmer_row_setup<IdT, K>(bytes, off, end, row, total_bytes, f, ids, lengths_in, out_offsets);
        const int64_t w0 = (int64_t)seg * KSEG_WINDOWS;
        if (seg > 0 && w0 >= r.n_win) continue;                                  // the row ended in an earlier segment
        if (seg == 0) kmer_flag_long_row(end - off, status, row, lane);
        const bool last = seg == n_seg - 1 || w0 + KSEG_WINDOWS >= r.n_win;
        const int w_end = last ? r.n_win : (int)w0 + KSEG_WINDOWS;
        uint32_t* my_flag = flags + (int64_t)seg * n_rows + row;

        // the flags of the 32 segments before this one: asked for now, looked at after the decode
        uint32_t look = KSEG_TOTAL;                                              // before the row start: a total of 0
        if (seg - 1 - lane >= 0) look = *(const volatile uint32_t*)(flags + (int64_t)(seg - 1 - lane) * n_rows + row);

        // ---- 1. decode and count (segments that are not the last of their row hold complete windows only)
        int count = 0;
        bool in_regs = false, clean = false;
        uint32_t packed[NCH];                                                    // idxA | idxB << 16 per chunk
        if (!last) {
            int64_t fit = (r.room_total - 8) / K;                                // windows whose aligned words stay in the buffer
            if (w0 + KSEG_WINDOWS <= fit) {
                in_regs = true;
                const uint8_t* g = r.src + ((int)w0 + 2 * lane) * K;
                const uint32_t sh = (uint32_t)(reinterpret_cast<uintptr_t>(g) & 3u) * 8u;
                const uint32_t* gw = reinterpret_cast<const uint32_t*>(g - (sh >> 3));
                uint32_t wd[NCH][NW];
#pragma unroll
                for (int c = 0; c < NCH; ++c)
#pragma unroll
                    for (int i = 0; i < NW; ++i) wd[c][i] = __ldg(gw + c * 16 * K + i);
                int n_dirty = 0;
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    uint32_t P = 0, dA = 0, dB = 0;
#pragma unroll
                    for (int i = 0; i < NW - 1; ++i) {
                        const uint32_t rr = __funnelshift_r(wd[c][i], wd[c][i + 1], sh);
                        uint32_t cc, d;
                        acgt_codes4(rr, &cc, &d);
                        P |= pack_codes4(cc) << (24 - 8 * i);
                        uint32_t mA = 0, mB = 0;
#pragma unroll
                        for (int b = 0; b < 4; ++b) {
                            const int pos = 4 * i + b;
                            if (pos < K) mA |= 0xFFu << (8 * b);
                            else if (pos < 2 * K) mB |= 0xFFu << (8 * b);
                        }
                        dA |= d & mA;
                        dB |= d & mB;
                    }
                    packed[c] = ((P >> (32 - 2 * K)) & IDX_MASK) | (((P >> (32 - 4 * K)) & IDX_MASK) << 16);
                    n_dirty += __popc(__ballot_sync(0xffffffffu, dA != 0)) + __popc(__ballot_sync(0xffffffffu, dB != 0));
                }
                clean = n_dirty == 0;
                count = KSEG_WINDOWS + (K - 1) * n_dirty;
            } else {
                // the end of the input buffer is too close for aligned word loads: count byte by byte
                int cnt = 0;
                for (int w = (int)w0 + lane; w < w_end; w += 32) {
                    bool ok = true;
                    for (int i = 0; i < K; ++i) ok &= kmer_code(__ldg(r.src + w * K + i)) < 4;
                    cnt += ok ? 1 : K;
                }
                count = __reduce_add_sync(0xffffffffu, cnt);
            }
            // ---- 2. publish the own count (segment 0 knows its total already)
            if (lane == 0 && publish) *(volatile uint32_t*)my_flag = (seg == 0 ? KSEG_TOTAL : KSEG_OWN) | (uint32_t)count;
        }

        // ---- 3. tokens before this segment
        int base = 0;
        bool stalled = false;
        if (seg > 0) {
            int behind = seg - 1;                                                // segment lane 0 looks at
            int polls = 0;
            uint32_t sum = 0;
            for (;;) {
                const uint32_t st = look >> 30;
                const unsigned totals = __ballot_sync(0xffffffffu, st == 2u);
                const unsigned empties = __ballot_sync(0xffffffffu, st == 0u);
                if (__any_sync(0xffffffffu, st == 3u)) { stalled = true; break; }
                const int first_total = totals ? __ffs(totals) - 1 : 32;
                const unsigned wanted = first_total >= 31 ? 0xffffffffu : ((2u << first_total) - 1u);
                if (empties & wanted) {
                    if (++polls > poll_limit) { stalled = true; break; }
                    __nanosleep(64);
                } else {
                    sum += __reduce_add_sync(0xffffffffu, lane <= first_total ? (look & KSEG_VALUE) : 0u);
                    if (first_total < 32) break;
                    behind -= 32;
                }
                look = KSEG_TOTAL;
                if (behind - lane >= 0) look = *(const volatile uint32_t*)(flags + (int64_t)(behind - lane) * n_rows + row);
            }
            base = (int)sum;
        }
        if (stalled) {
            if (lane == 0) {
                if (status) atomicOr(status + row, 16);
                if (!last) *(volatile uint32_t*)my_flag = KSEG_POISON;
                else if (lengths_out) lengths_out[row] = 0;
            }
            continue;
        }
        // ---- 4. publish the total, place the tokens
        if (!last && seg > 0 && lane == 0 && publish) *(volatile uint32_t*)my_flag = KSEG_TOTAL | (uint32_t)(base + count);

        if (in_regs && clean && base + KSEG_WINDOWS <= cap) {
            IdT* d = r.dst + base;
            Pair one; one.x = 1; one.y = 1;
            if ((reinterpret_cast<uintptr_t>(d) % (2 * sizeof(IdT))) == 0) {
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    const uint32_t a = packed[c] & 0xFFFFu, b = packed[c] >> 16;
                    Pair v;
                    v.x = (IdT)(AFFINE ? affine_base + (int32_t)a : __ldg(kmer_ids + a));
                    v.y = (IdT)(AFFINE ? affine_base + (int32_t)b : __ldg(kmer_ids + b));
                    *reinterpret_cast<Pair*>(d + 64 * c + 2 * lane) = v;
                    if (FUSE_MASK) *reinterpret_cast<Pair*>(d + mdelta + 64 * c + 2 * lane) = one;
                }
            } else {
                // odd offset: the aligned pairs are (second window of this lane, first window of the next
                // lane); the segment's first and last token go out alone
#pragma unroll
                for (int c = 0; c < NCH; ++c) {
                    const uint32_t a = packed[c] & 0xFFFFu, b = packed[c] >> 16;
                    uint32_t a_next = __shfl_down_sync(0xffffffffu, a, 1);
                    const uint32_t a_chunk = c + 1 < NCH ? __shfl_sync(0xffffffffu, packed[c + 1 < NCH ? c + 1 : c] & 0xFFFFu, 0) : 0u;
                    if (lane == 31) a_next = a_chunk;
                    const IdT vb = (IdT)(AFFINE ? affine_base + (int32_t)b : __ldg(kmer_ids + b));
                    IdT* q = d + 64 * c + 2 * lane + 1;
                    if (c + 1 < NCH || lane < 31) {
                        Pair v;
                        v.x = vb;
                        v.y = (IdT)(AFFINE ? affine_base + (int32_t)a_next : __ldg(kmer_ids + a_next));
                        *reinterpret_cast<Pair*>(q) = v;
                        if (FUSE_MASK) *reinterpret_cast<Pair*>(q + mdelta) = one;
                    } else {
                        *q = vb;
                        if (FUSE_MASK) q[mdelta] = 1;
                    }
                    if (c == 0 && lane == 0) {
                        d[0] = (IdT)(AFFINE ? affine_base + (int32_t)a : __ldg(kmer_ids + a));
                        if (FUSE_MASK) d[mdelta] = 1;
                    }
                }
            }
            base += KSEG_WINDOWS;
        } else {
            bool clipped = false;
            base = kmer_encode_windows<IdT, K, AFFINE, FUSE_MASK>(r, cap, kmer_ids, affine_base, single_ids, mdelta, lane,
                                                                  (int)w0, w_end, base, &clipped);
            if (last) kmer_finish_row<IdT, FUSE_MASK>(r, row, base, cap, clipped, f, ids, mask, lengths_out, out_offsets, status, lane);
            else if (lane == 0 && status && f.clip_is_error && clipped) atomicOr(status + row, 4);
        }
    }
}

}  // namespace dnatok

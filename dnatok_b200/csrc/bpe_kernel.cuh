// BPE merge engine.  One warp owns one pre-tokenised word, held entirely in shared memory as
// four 16-bit arrays over the word's original positions: the token at each live position, the
// rank of the pair that starts there, and next / previous live position.  Every pass
//   1. finds the lowest rank among all live pairs (128-bit shared-memory loads, packed 16-bit
//      minima, one warp reduction),
//   2. marks the positions holding that rank as merge sites; for a pair of equal tokens (x, x)
//      only the first position of a run of such pairs is marked and its owner walks the run
//      left to right taking every other pair, which is Hugging Face's leftmost-first rule,
//   3. applies all sites (token replaced, right neighbour unlinked) and marks the positions
//      whose pair changed,
//   4. looks the changed pairs up again in the merge table,
// until no pair has a rank.  Merging every occurrence of the lowest rank in one pass gives the
// same result as Hugging Face's queue (one merge at a time, lowest rank then leftmost) when new
// pairs always rank above the merge that created them; the host checks that property of the
// table and otherwise selects one merge per pass (single_step).
//
// Words are binned by length into capacity classes so that short words do not pay for the
// shared memory of long ones; each class is one persistent launch whose warps pull words from a
// shared counter.  Merged tokens (uint16, Hugging Face ids) and per-row counts go to the
// caller's scratch; the emit kernels turn them into the final ids / mask layout.
//
// Same rule as the reference kernel states (src/dnatok_bpe_kernel/dnatok_bpe.cu:3-5,172-176),
// different machinery: that kernel keeps per-rank bucket lists and the word itself in global
// memory with one 256-thread block per sequence (:237-740).
#pragma once
#include "common.cuh"

namespace dnatok {

constexpr uint32_t BPE_NONE = 0xFFFFu;      // no rank / no position / dead token
constexpr int BPE_N_CLASSES = 7;            // capacities 256 << c, c = 0..6
constexpr int BPE_MIN_CAP = 256;

struct BpeDeviceTable {
    const uint32_t* disp;
    const uint32_t* slots;
    const uint16_t* merge_out;
    const uint16_t* byte_tok;
    int32_t single_step;
};

__device__ __forceinline__ uint32_t bpe_rank(const BpeDeviceTable& t, uint32_t a, uint32_t b) {
    const uint32_t s = __ldg(t.slots + __ldg(t.disp + a) + b);
    return (s >> 16) == a ? (s & 0xFFFFu) : BPE_NONE;
}

// Bytes of shared memory one word slot of capacity C takes.
__host__ __device__ constexpr int bpe_slot_bytes(int C) { return 8 * C + C / 8 + C / 8; }

// Bin rows by length.  class_count[c] rows land in class_list[c * n_rows ...].
__global__ void bpe_classify_kernel(const int64_t* __restrict__ offsets, int64_t n_rows,
                                    int32_t* __restrict__ class_count, int32_t* __restrict__ class_list,
                                    int32_t* __restrict__ counts, int32_t* __restrict__ status) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_rows) return;
    const int64_t n = offsets[i + 1] - offsets[i];
    counts[i] = 0;
    if (n <= 0) return;
    int c = 0;
    while (c < BPE_N_CLASSES && (int64_t)(BPE_MIN_CAP << c) < n) ++c;
    if (c >= BPE_N_CLASSES) { if (status) atomicOr(status + i, 1); return; }
    const int slot = atomicAdd(class_count + c, 1);
    class_list[(int64_t)c * n_rows + slot] = (int32_t)i;
}

template <int C>
__global__ void bpe_merge_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets,
                                 const int32_t* __restrict__ list, const int32_t* __restrict__ list_count,
                                 int32_t* __restrict__ work_counter, BpeDeviceTable t,
                                 uint16_t* __restrict__ out_tok, int32_t* __restrict__ counts,
                                 int32_t* __restrict__ status) {
    extern __shared__ uint4 bpe_dyn[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint8_t* slot = reinterpret_cast<uint8_t*>(bpe_dyn) + (size_t)warp * bpe_slot_bytes(C);
    uint16_t* rk = reinterpret_cast<uint16_t*>(slot);            // 16-byte aligned: slot size is a multiple of 16
    uint16_t* tok = rk + C;
    uint16_t* nxt = tok + C;
    uint16_t* prv = nxt + C;
    uint8_t* siteb = reinterpret_cast<uint8_t*>(prv + C);        // C/8 bytes: one flag byte per 8 positions
    uint32_t* dirty = reinterpret_cast<uint32_t*>(siteb + C / 8);// C/32 words
    const uint4* rk4 = reinterpret_cast<const uint4*>(rk);
    const int n_words = *list_count;

    for (;;) {
        int wi = 0;
        if (lane == 0) wi = atomicAdd(work_counter, 1);
        wi = __shfl_sync(0xffffffffu, wi, 0);
        if (wi >= n_words) break;
        const int row = list[wi];
        const int64_t off = offsets[row];
        const int n = (int)(offsets[row + 1] - off);          // 1 <= n <= C by classification
        const int nvec = (n + 7) >> 3;

        for (int i = lane; i < nvec * 8; i += 32) {
            if (i < n) {
                tok[i] = t.byte_tok[__ldg(bytes + off + i)];
                nxt[i] = (uint16_t)(i + 1 < n ? i + 1 : BPE_NONE);
                prv[i] = (uint16_t)(i ? i - 1 : BPE_NONE);
            }
            rk[i] = (uint16_t)BPE_NONE;
        }
        for (int i = lane; i < (nvec + 3) / 4; i += 32) dirty[i] = 0;
        __syncwarp();
        for (int i = lane; i + 1 < n; i += 32) rk[i] = (uint16_t)bpe_rank(t, tok[i], tok[i + 1]);
        __syncwarp();

        int pass = 0;
        for (; pass <= n; ++pass) {
            // 1. lowest rank
            uint32_t m = 0xFFFFFFFFu;
            for (int j = lane; j < nvec; j += 32) {
                const uint4 v = rk4[j];
                m = __vminu2(m, __vminu2(__vminu2(v.x, v.y), __vminu2(v.z, v.w)));
            }
            const uint32_t g = __reduce_min_sync(0xffffffffu, min(m & 0xFFFFu, m >> 16));
            if (g == BPE_NONE) break;
            const uint16_t newtok = __ldg(t.merge_out + g);
            const uint32_t gg = g | (g << 16);

            // 2. sites (reads only)
            uint32_t first_site = BPE_NONE;
            for (int j = lane; j < nvec; j += 32) {
                const uint4 v = rk4[j];
                const uint32_t w[4] = { v.x, v.y, v.z, v.w };
                uint32_t flags = 0;
                if ((__vcmpeq2(w[0], gg) | __vcmpeq2(w[1], gg) | __vcmpeq2(w[2], gg) | __vcmpeq2(w[3], gg)) != 0) {
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const uint32_t r = (w[e >> 1] >> ((e & 1) * 16)) & 0xFFFFu;
                        if (r == g) {
                            const int p = j * 8 + e;
                            bool site = true;
                            if (tok[nxt[p]] == tok[p]) {              // pair (x, x): only a run start is a site
                                const uint32_t l = prv[p];
                                if (l != BPE_NONE && rk[l] == g) site = false;
                            }
                            if (site) { flags |= 1u << e; if (first_site == BPE_NONE) first_site = p; }
                        }
                    }
                }
                siteb[j] = (uint8_t)flags;
            }
            uint32_t only = BPE_NONE;
            if (t.single_step) only = __reduce_min_sync(0xffffffffu, first_site);
            __syncwarp();

            // 3. apply
            for (int j = lane; j < nvec; j += 32) {
                uint32_t flags = siteb[j];
                while (flags) {
                    const int e = __ffs(flags) - 1;
                    flags &= flags - 1;
                    int p = j * 8 + e;
                    if (t.single_step && (uint32_t)p != only) continue;
                    const bool homo = tok[nxt[p]] == tok[p];
                    for (int guard = 0; guard < C; ++guard) {
                        const uint32_t q = nxt[p];
                        const uint32_t r = nxt[q];
                        tok[p] = newtok;
                        tok[q] = (uint16_t)BPE_NONE;
                        rk[q] = (uint16_t)BPE_NONE;
                        nxt[p] = (uint16_t)r;
                        if (r != BPE_NONE) prv[r] = (uint16_t)p;
                        atomicOr(dirty + (p >> 5), 1u << (p & 31));
                        const uint32_t l = prv[p];
                        if (l != BPE_NONE) atomicOr(dirty + (l >> 5), 1u << (l & 31));
                        if (!homo || t.single_step || r == BPE_NONE || rk[r] != g) break;
                        p = (int)r;       // next pair of the run (x, x)(x, x)...
                    }
                }
            }
            __syncwarp();

            // 4. re-rank the pairs that changed
            for (int i = lane; i < (nvec + 3) / 4; i += 32) {
                uint32_t d = dirty[i];
                if (d) {
                    dirty[i] = 0;
                    while (d) {
                        const int p = i * 32 + __ffs(d) - 1;
                        d &= d - 1;
                        const uint32_t a = tok[p];
                        if (a != BPE_NONE) {
                            const uint32_t r = nxt[p];
                            rk[p] = (uint16_t)(r == BPE_NONE ? BPE_NONE : bpe_rank(t, a, tok[r]));
                        }
                    }
                }
            }
            __syncwarp();
        }

        // compact the live tokens, in order, to out_tok[off ...]
        int base = 0;
        for (int i0 = 0; i0 < n; i0 += 32) {
            const int i = i0 + lane;
            const bool live = i < n && tok[i] != BPE_NONE;
            const uint32_t bal = __ballot_sync(0xffffffffu, live);
            if (live) out_tok[off + base + __popc(bal & ((1u << lane) - 1))] = tok[i];
            base += __popc(bal);
        }
        if (lane == 0) {
            counts[row] = base;
            if (pass > n && status) atomicOr(status + row, 2);
        }
        __syncwarp();
    }
}

}  // namespace dnatok

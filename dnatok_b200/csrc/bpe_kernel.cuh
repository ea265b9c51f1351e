// BPE merge engine: exact Hugging Face merge order in a handful of data-parallel rounds.
//
// A word (one pre-tokenised row) is kept as a COMPACT array of 16-bit tokens in shared memory (no
// links, no tombstones) and is owned by a team of W warps (W = 1 for short words, up to 8 for long
// ones).  A round:
//   1. every adjacent pair is looked up in the merge table (perfect hash, two dependent loads); its
//      rank is stored and B = min over the present ranks r of F[r] is reduced, where F[r] is the
//      lowest rank of any pair that contains the token rank r creates;
//   2. pairs with rank < B are candidates: one ballot mask per 32 positions, and one more for
//      "rank(i-1) <= rank(i)".  Hugging Face would take the candidates in (rank, position) order,
//      skipping a pair when an earlier one consumed one of its tokens.  On a path that greedy choice has a closed form: follow the strictly improving
//      priorities to the left and to the right of a candidate down to the local optimum; the
//      candidate is taken iff both walks have even length;
//   3. the two parities are prefix-XORs along runs of set bits in the masks.  They are computed on
//      the masks themselves, one lane per 32 positions: carry-propagating bit tricks inside a mask,
//      and a warp scan over the four possible carry functions (constant 0, constant 1, identity,
//      negation) across masks.  The same step gives the selected pairs, the surviving positions
//      and, by a warp prefix sum, where each group of 32 positions lands after compaction;
//   4. selected merges are applied and the array is compacted in place, tile by tile.
// Everything created in a round contains a new token, so it ranks >= B, above every pair merged in
// that round: the round equals the sequential queue run over the same ranks.  Rounds repeat until no
// pair has a rank: 5-7 rounds for DNA words of any length, ~3.3 position visits per input byte in
// total.  Equal ranks on neighbouring pairs (runs of one token) fall out of the same rule, because
// priority is (rank, position): every other pair from the left.
//
// A table whose merge operands may be created by later ranks has no usable F; for it the host
// selects single_step: one merge per round, the leftmost pair of the lowest rank.
//
// Words are binned by length into capacity classes (shared memory per word = 4.375 bytes per
// position); each class is one launch of resident teams that pull words from a shared counter.
// Merged tokens (uint16, Hugging Face ids) and per-row counts go to the caller's scratch; the emit
// kernels produce the final ids / mask layout.
//
// Same result as the rule the reference kernel states (src/dnatok_bpe_kernel/dnatok_bpe.cu:3-5,
// 172-176); that kernel walks the ranks one by one with per-rank bucket lists in global memory
// and one 256-thread block per sequence (:237-740).
#pragma once
#include "common.cuh"

namespace dnatok {

constexpr uint32_t BPE_NONE = 0xFFFFu;          // no rank
constexpr int BPE_N_CLASSES = 9;
constexpr int BPE_BLOCK_WARPS = 8;              // largest team: a whole block of 8 warps on one word
// Warps per block for teams of W warps.  One-warp teams sit 16 to a block: the block's fixed shared
// memory (pair table, reduction slots) is then paid three times per SM instead of five and 48 warps
// fit where 40 did.
__host__ __device__ constexpr int bpe_block_warps(int W) { return W == 1 ? 16 : BPE_BLOCK_WARPS; }

__host__ __device__ constexpr int bpe_class_capacity(int c) {
    return c < 8 ? (256 << c) : 49152;          // 256 ... 32768, 49152
}
// warps that share one word of a class
__host__ __device__ constexpr int bpe_class_team(int c) {
    return c <= 2 ? 1 : c == 3 ? 2 : c == 4 ? 4 : 8;
}
// tokens + ranks (2 bytes each) + three 32-bit words per 32 positions
__host__ __device__ constexpr int bpe_slot_bytes(int C) { return 4 * C + 3 * (C / 32) * 4; }

struct BpeDeviceTable {
    const uint32_t* disp;        // [n_tokens] row displacement of the left token
    const uint32_t* slots;       // (left << 16) | rank, 0xFFFFFFFF when empty
    const uint16_t* merge_out;   // [n_merges] token created by a rank
    const uint16_t* future;      // [n_merges] F: lowest rank of a pair containing that token
    const uint32_t* hot;         // [32 * 32] pairs of ids < 32: rank | F << 16 (0xFFFFFFFF: no merge)
    const uint16_t* byte_tok;    // [256]
    int32_t single_step;
};

__device__ __forceinline__ uint32_t bpe_rank(const BpeDeviceTable& t, uint32_t a, uint32_t b) {
    const uint32_t s = __ldg(t.slots + __ldg(t.disp + a) + b);
    return (s >> 16) == a ? (s & 0xFFFFu) : BPE_NONE;
}

// odd(i) = c(i) & ~odd(i-1), odd(-1) = prev_odd: parity of the length of the run of set bits
// ending at each bit, continued from the previous 32 positions.
__device__ __forceinline__ uint32_t run_parity(uint32_t c, bool prev_odd) {
    uint32_t se = c & ~(c << 1) & 0x55555555u;      // runs that start on an even bit
    if (prev_odd) se &= ~1u;                        // a run continuing an odd position behaves as odd-started
    const uint32_t fe = c & ~(c + se);              // all bits of those runs
    const uint32_t fo = c & ~fe;
    return (fe & 0x55555555u) | (fo & 0xAAAAAAAAu);
}

// Carry functions {0,1} -> {0,1} as two bits: bit 0 = f(0), bit 1 = f(1).
__device__ __forceinline__ uint32_t carry_fn(uint32_t c) {
    return (run_parity(c, false) >> 31) | ((run_parity(c, true) >> 31) << 1);
}
__device__ __forceinline__ uint32_t carry_apply(uint32_t f, bool x) { return (f >> (x ? 1 : 0)) & 1u; }
// first a, then b
__device__ __forceinline__ uint32_t carry_then(uint32_t a, uint32_t b) {
    return carry_apply(b, a & 1u) | (carry_apply(b, (a >> 1) & 1u) << 1);
}

// Bin rows by length: class_count[c] rows land in class_list[c * n_rows ...].  One atomic per
// warp and class (rows of a batch mostly share a class).  Classes outside class_mask are not
// launched by the host; a row that belongs to one is flagged instead of being dropped silently.
__global__ void bpe_classify_kernel(const int64_t* __restrict__ offsets, int64_t n_rows,
                                    int32_t* __restrict__ class_count, int32_t* __restrict__ class_list,
                                    int32_t* __restrict__ counts, int32_t* __restrict__ status,
                                    uint32_t class_mask) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int lane = threadIdx.x & 31;
    int c = -1;
    if (i < n_rows) {
        const int64_t n = offsets[i + 1] - offsets[i];
        counts[i] = 0;
        if (n > 0) {
            c = 0;
            while (c < BPE_N_CLASSES && (int64_t)bpe_class_capacity(c) < n) ++c;
            if (c >= BPE_N_CLASSES) { if (status) atomicOr(status + i, 1); c = -1; }
            else if (!((class_mask >> c) & 1u)) { if (status) atomicOr(status + i, 8); c = -1; }   // outside the caller's length hint
        }
    }
    for (int k = 0; k < BPE_N_CLASSES; ++k) {
        const uint32_t m = __ballot_sync(0xffffffffu, c == k);
        if (m == 0) continue;
        const int leader = __ffs(m) - 1;
        int base = 0;
        if (lane == leader) base = atomicAdd(class_count + k, __popc(m));
        base = __shfl_sync(0xffffffffu, base, leader);
        if (c == k) class_list[(int64_t)k * n_rows + base + __popc(m & ((1u << lane) - 1u))] = (int32_t)i;
    }
}

// Barrier over the W warps of one team (team index `team` within the block).
template <int W>
__device__ __forceinline__ void team_sync(int team) {
    if (W == 1) __syncwarp();
    else if (W == BPE_BLOCK_WARPS) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(W * 32) : "memory");
}

// C: capacity in positions; W: warps per word.
template <int C, int W>
__global__ void __launch_bounds__(bpe_block_warps(W) * 32)
bpe_rounds_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets,
                  const int32_t* __restrict__ list, const int32_t* __restrict__ list_count,
                  int32_t* __restrict__ work_counter, BpeDeviceTable t,
                  uint16_t* __restrict__ out_tok, int32_t* __restrict__ counts,
                  int32_t* __restrict__ status) {
    constexpr int BW = bpe_block_warps(W);
    constexpr int TEAMS = BW / W;
    constexpr int G = C / 32;
    extern __shared__ uint4 bpe_dyn[];
    __shared__ uint32_t s_red[BW][2];            // per-warp partial minima
    __shared__ uint32_t s_hot[32 * 32];                       // direct table for pairs of small ids
    for (int i = threadIdx.x; i < 32 * 32; i += BW * 32) s_hot[i] = __ldg(t.hot + i);
    __syncthreads();
    __shared__ int32_t s_word[TEAMS][2];                      // claimed word index, new length
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int team = warp / W, tw = warp % W;                 // team, warp within team
    const int tt = tw * 32 + lane;                            // thread within team
    const uint32_t lt = (1u << lane) - 1u;
    uint8_t* slot = reinterpret_cast<uint8_t*>(bpe_dyn) + (size_t)team * bpe_slot_bytes(C);
    uint16_t* tok = reinterpret_cast<uint16_t*>(slot);          // [C] live tokens, compact
    uint16_t* rk = tok + C;                                     // [C] rank of the pair (i, i+1)
    uint32_t* m_leq = reinterpret_cast<uint32_t*>(rk + C);      // [G] bit i: rank(i-1) <= rank(i); after step 3: survivors
    uint32_t* m_cs = m_leq + G;                                 // [G] candidates, then selected pairs
    uint32_t* g_aux = m_cs + G;                                 // [G] right-walk parity, then output base
    const int n_words = *list_count;

    for (;;) {
        if (tt == 0) s_word[team][0] = atomicAdd(work_counter, 1);
        team_sync<W>(team);
        const int wi = s_word[team][0];
        if (wi >= n_words) break;
        const int row = list[wi];
        const int64_t off = offsets[row];
        int n = (int)(offsets[row + 1] - off);               // 1 <= n <= C by classification

        for (int i = tt; i < n; i += W * 32) tok[i] = __ldg(t.byte_tok + __ldg(bytes + off + i));
        team_sync<W>(team);

        int round = 0;
        const int max_rounds = n + 2;
        for (; round < max_rounds; ++round) {
            const int groups = (n + 31) >> 5;
            // ---- 1: ranks of all pairs, bound B, lowest rank
            uint32_t bmin = BPE_NONE, gmin = BPE_NONE;
            for (int g = tw; g < groups; g += W) {
                const int i = g * 32 + lane;
                uint32_t r = BPE_NONE, fut = BPE_NONE;
                if (i + 1 < n) {
                    const uint32_t a = tok[i], b = tok[i + 1];
                    if ((a | b) < 32u) {                        // early rounds: both tokens are among the first ids
                        const uint32_t e = s_hot[a * 32u + b];
                        r = e & 0xFFFFu; fut = e >> 16;
                    } else {
                        r = bpe_rank(t, a, b);
                        if (r != BPE_NONE) fut = __ldg(t.future + r);
                    }
                }
                if (i < n) rk[i] = (uint16_t)r;
                gmin = min(gmin, r);
                bmin = min(bmin, fut);
            }
            gmin = __reduce_min_sync(0xffffffffu, gmin);
            bmin = __reduce_min_sync(0xffffffffu, bmin);
            if (W > 1) {
                if (lane == 0) { s_red[warp][0] = gmin; s_red[warp][1] = bmin; }
                team_sync<W>(team);
#pragma unroll
                for (int k = 0; k < W; ++k) {
                    gmin = min(gmin, s_red[team * W + k][0]);
                    bmin = min(bmin, s_red[team * W + k][1]);
                }
            } else {
                __syncwarp();
            }
            if (gmin == BPE_NONE) break;                       // no pair can merge: done (uniform over the team)
            const uint32_t B = t.single_step ? gmin + 1 : bmin;

            // ---- 2: candidate masks and "not worse than my left neighbour" masks
            for (int g = tw; g < groups; g += W) {
                const int i = g * 32 + lane;
                const uint32_t r = i < n ? (uint32_t)rk[i] : BPE_NONE;
                uint32_t rp = __shfl_up_sync(0xffffffffu, r, 1);
                if (lane == 0) rp = i > 0 ? (uint32_t)rk[i - 1] : BPE_NONE;
                const uint32_t cand = __ballot_sync(0xffffffffu, r < B);
                const uint32_t leq = __ballot_sync(0xffffffffu, rp <= r);
                if (lane == 0) { m_cs[g] = cand; m_leq[g] = leq; }
            }
            team_sync<W>(team);

            // ---- 3: on the masks, one lane per 32 positions (first warp of the team)
            if (tw == 0) {
                const int blocks = (groups + 31) >> 5;
                // 3a. right-walk parity, last block first
                bool carry = false;                            // parity bit of the position after the block
                for (int b = blocks - 1; b >= 0; --b) {
                    const int g = b * 32 + lane;
                    const bool live = g < groups;
                    const uint32_t cand = live ? m_cs[g] : 0u;
                    const uint32_t leq = live ? m_leq[g] : 0xFFFFFFFFu;
                    const uint32_t leq_next = g + 1 < groups ? m_leq[g + 1] : 0xFFFFFFFFu;
                    // bit i: the right neighbour ranks strictly better: not (rank(i) <= rank(i+1))
                    const uint32_t link = cand & ~((leq >> 1) | (leq_next << 31));
                    const uint32_t c = __brev(link);           // walk from the high positions down
                    // carry functions compose from the highest group of the block to the lowest
                    uint32_t f = carry_fn(c);
#pragma unroll
                    for (int d = 1; d < 32; d <<= 1) {
                        const uint32_t other = __shfl_down_sync(0xffffffffu, f, d);   // groups above, applied first
                        if (lane + d < 32) f = carry_then(other, f);
                    }
                    // f now maps the block's incoming carry to the carry leaving this group downwards
                    const uint32_t above = __shfl_down_sync(0xffffffffu, f, 1);
                    const bool cin = lane == 31 ? carry : (carry_apply(above, carry) != 0);
                    const uint32_t odd = __brev(run_parity(c, cin));
                    if (live) g_aux[g] = odd;
                    carry = carry_apply(__shfl_sync(0xffffffffu, f, 0), carry) != 0;
                }
                __syncwarp();
                // 3b. left-walk parity, selection, survivors, output bases, first block first
                carry = false;                                 // left parity bit of the position before the block
                uint32_t sel_carry = 0;                        // was the position before the block selected
                int base = 0;
                bool took = false;
                for (int b = 0; b < blocks; ++b) {
                    const int g = b * 32 + lane;
                    const bool live = g < groups;
                    const uint32_t cand = live ? m_cs[g] : 0u;
                    const uint32_t leq = live ? m_leq[g] : 0u;
                    const uint32_t link = cand & leq;          // the left neighbour is a candidate that goes first
                    uint32_t f = carry_fn(link);
#pragma unroll
                    for (int d = 1; d < 32; d <<= 1) {
                        const uint32_t other = __shfl_up_sync(0xffffffffu, f, d);     // groups below, applied first
                        if (lane >= d) f = carry_then(other, f);
                    }
                    const uint32_t below = __shfl_up_sync(0xffffffffu, f, 1);
                    const bool cin = lane == 0 ? carry : (carry_apply(below, carry) != 0);
                    const uint32_t oddl = run_parity(link, cin);
                    uint32_t sel = live ? (cand & ~oddl & ~g_aux[g]) : 0u;
                    carry = carry_apply(__shfl_sync(0xffffffffu, f, 31), carry) != 0;
                    if (t.single_step) {                       // only the leftmost pair of the lowest rank
                        const uint32_t any = __ballot_sync(0xffffffffu, sel != 0);
                        const int first = __ffs(any) - 1;
                        sel = (!took && lane == first) ? (sel & (0u - sel)) : 0u;
                        took = took || any != 0;
                    }
                    uint32_t prev = __shfl_up_sync(0xffffffffu, sel, 1) >> 31;
                    if (lane == 0) prev = sel_carry;
                    sel_carry = __shfl_sync(0xffffffffu, sel, 31) >> 31;
                    const int cnt_pos = n - g * 32;            // positions of this group
                    const uint32_t valid = !live ? 0u : (cnt_pos >= 32 ? 0xFFFFFFFFu : ((1u << cnt_pos) - 1u));
                    const uint32_t kept = valid & ~((sel << 1) | prev);
                    int x = __popc(kept), incl = x;
#pragma unroll
                    for (int d = 1; d < 32; d <<= 1) {
                        const int y = __shfl_up_sync(0xffffffffu, incl, d);
                        if (lane >= d) incl += y;
                    }
                    if (live) { m_cs[g] = sel; m_leq[g] = kept; g_aux[g] = (uint32_t)(base + incl - x); }   // m_leq is free now: survivors
                    base += __shfl_sync(0xffffffffu, incl, 31);
                }
                if (lane == 0) s_word[team][1] = base;
            }
            team_sync<W>(team);

            // ---- 4: merge and compact in place, W groups at a time
            const int n_new = s_word[team][1];
            for (int g0 = 0; g0 < groups; g0 += W) {
                const int g = g0 + tw;
                const int i = g * 32 + lane;
                uint32_t v = 0, kept = 0;
                int base = 0;
                if (g < groups) {
                    const uint32_t sel = m_cs[g];
                    kept = m_leq[g];                           // survivors of this group, from step 3
                    base = (int)g_aux[g];
                    if (i < n) v = tok[i];
                    if ((sel >> lane) & 1u) v = __ldg(t.merge_out + rk[i]);
                }
                team_sync<W>(team);                            // every warp has read its tokens of this tile
                if ((kept >> lane) & 1u) tok[base + __popc(kept & lt)] = (uint16_t)v;
            }
            team_sync<W>(team);
            n = n_new;
        }

        for (int i = tt; i < n; i += W * 32) out_tok[off + i] = tok[i];
        if (tt == 0) {
            counts[row] = n;
            if (round >= max_rounds && status) atomicOr(status + row, 2);
        }
        team_sync<W>(team);
    }
}

}  // namespace dnatok

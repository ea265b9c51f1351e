// BPE merge engine: exact Hugging Face merge order in a handful of data-parallel rounds.
//
// Hugging Face pops queue entries in (rank, position) order and skips an entry whose tokens were
// consumed.  A round here takes every pair whose rank is below B = min over the present ranks r of
// F[r], where F[r] is the lowest rank of any pair containing the token rank r creates: nothing
// created during the round can rank below B, so the round's outcome is the greedy matching of the
// candidate pairs in priority order.  On a path that choice has a closed form: follow the strictly
// improving priorities to the left and to the right of a candidate down to the local optimum; the
// candidate is taken iff both walks have even length.  The two parities are prefix-XORs along runs
// of set bits in two bit masks (32 positions per mask word): carry-propagating bit tricks inside a
// word, a carry handed from word to word.  Equal ranks on neighbouring pairs (runs of one token)
// fall out of the same rule because priority is (rank, position): every other pair from the left.
// Rounds repeat until no pair has a rank: 5-7 rounds for DNA words of any length.
//
// A table whose merge operands may be created by later ranks has no usable F; for it the host
// selects single_step: one merge per round, the leftmost pair of the lowest rank.
//
// Two kernels share that rule.
//
// bpe_lanes_kernel<W> (words up to 1,024 * W positions, W warps per word): every lane owns a
//   contiguous chunk of the word, at most 32 positions = one mask word, held as a column of a
//   slot-major token array in shared memory (slot j of lane g at j * (T + 2) + g, so that both
//   "all lanes read slot j" and "one lane walks its slots" are free of bank conflicts).  A lane
//   walks its chunk in a fully unrolled loop: tokens come from shared memory at compile-time
//   offsets, the looked-up entries stay in registers, the masks are built bit by bit in registers,
//   and nothing but the chunk borders, the carries and the compaction offsets crosses lanes.  After
//   the selection every surviving token is written to its new global position in the other buffer,
//   re-dealt so that all lanes again own equally many positions.
//
// bpe_long_kernel (longer words, one block of 32 warps per word): the same round over arrays in
//   global memory (tokens in place in the output area, ranks and masks in caller scratch),
//   position-parallel: lane i of a warp handles position 32 g + i and masks come from ballots.
//
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
constexpr uint32_t BPE_FULL = 0xFFFFFFFFu;

// Length classes: class c < BPE_LONG_CLASS holds words of up to 1,024 << c positions and runs
// bpe_lanes_kernel<1 << c>; the last class holds everything longer and runs bpe_long_kernel.
constexpr int BPE_LANE_SLOTS = 32;              // positions one lane can own
constexpr int BPE_LONG_CLASS = 6;
constexpr int BPE_N_CLASSES = BPE_LONG_CLASS + 1;
constexpr int BPE_LONG_WARPS = 32;
constexpr int64_t BPE_MAX_POSITIONS = (int64_t)1 << 30;     // longest word of the long class

__host__ __device__ constexpr int bpe_class_capacity(int c) { return (32 * BPE_LANE_SLOTS) << c; }
// warps per block for teams of W warps
__host__ __device__ constexpr int bpe_block_warps(int W) { return W < 8 ? 8 : W; }
// shared memory of one team: two token buffers, and for teams of several warps the exchange arrays
__host__ __device__ constexpr int bpe_team_bytes(int W) {
    return 2 * BPE_LANE_SLOTS * (32 * W + 2) * 2 + (W > 1 ? 32 * W * 16 : 0);
}
// caller scratch of one word of the long class: ranks (2 bytes per position) and three mask words per 32 positions
__host__ __device__ constexpr int64_t bpe_long_bytes(int64_t n) { return ((2 * n + 15) / 16 + 3 * ((n + 127) / 128)) * 16; }

struct BpeDeviceTable {
    const uint32_t* disp;        // [n_tokens] row displacement of the left token
    const uint2* slots;          // x = (left << 16) | rank, y = (created << 16) | F; all ones when empty
    const uint16_t* merge_out;   // [n_merges] token created by a rank
    const uint2* hot;            // [32 * 32] pairs of ids < 32, slot format
    const uint16_t* byte_tok;    // [256]
    int32_t single_step;
};

// key = F << 16 | rank (its minimum over a word gives the bound B), val = created << 16 | rank;
// both all ones when the pair does not merge.
__device__ __forceinline__ void bpe_lookup(const BpeDeviceTable& t, const uint2* s_hot, uint32_t a, uint32_t b,
                                           uint32_t& key, uint32_t& val) {
    uint2 s;
    if ((a | b) < 32u) {
        s = s_hot[a * 32u + b];
    } else {
        s = __ldg(t.slots + __ldg(t.disp + a) + b);
        if ((s.x >> 16) != a) s = make_uint2(BPE_FULL, BPE_FULL);
    }
    key = __byte_perm(s.x, s.y, 0x5410);        // low half of x, low half of y above it
    val = __byte_perm(s.x, s.y, 0x7610);        // low half of x, high half of y above it
}

// odd(i) = c(i) & ~odd(i-1), odd(-1) = 0: parity of the length of the run of set bits ending at
// each bit.
__device__ __forceinline__ uint32_t run_parity(uint32_t c) {
    const uint32_t se = c & ~(c << 1) & 0x55555555u;   // runs that start on an even bit
    const uint32_t fe = c & ~(c + se);                 // all bits of those runs
    const uint32_t fo = c & ~fe;
    return (fe & 0x55555555u) | (fo & 0xAAAAAAAAu);
}
// The run that starts at bit 0: with odd(-1) = 1 exactly its parities flip.
__device__ __forceinline__ uint32_t first_run(uint32_t c) { return c & ~(c + 1u); }

// Carry functions {0,1} -> {0,1} as two bits: bit 0 = f(0), bit 1 = f(1).
__device__ __forceinline__ uint32_t carry_apply(uint32_t f, bool x) { return (f >> (x ? 1 : 0)) & 1u; }
// first a, then b
__device__ __forceinline__ uint32_t carry_then(uint32_t a, uint32_t b) {
    return carry_apply(b, a & 1u) | (carry_apply(b, (a >> 1) & 1u) << 1);
}

// Run parities of one mask word per lane, the runs continuing from lane to lane: upwards
// (DOWN = false: bit `top` of lane l-1 precedes bit 0 of lane l) or downwards (DOWN = true: bit
// `top` of lane l+1 precedes bit 0 of lane l).  Every word holds top + 1 bits; `full` is the word
// with all of them set.  `carry` enters the first lane of the chain and leaves as the parity after
// the last one, so blocks of 32 lanes chain through it.  A word passes its incoming parity on only
// when all its bits are set; unless some lane has such a word the neighbour's own top bit is the
// carry and one shuffle replaces the scan over carry functions.
template <bool DOWN>
__device__ __forceinline__ uint32_t chain_parity(uint32_t c, int top, uint32_t full, bool& carry, int lane) {
    const uint32_t odd0 = run_parity(c);
    const uint32_t fr = first_run(c);
    const uint32_t out0 = (odd0 >> top) & 1u;
    bool cin;
    if (__ballot_sync(BPE_FULL, c == full) == 0u) {
        const uint32_t nb = DOWN ? __shfl_down_sync(BPE_FULL, out0, 1) : __shfl_up_sync(BPE_FULL, out0, 1);
        cin = (DOWN ? lane == 31 : lane == 0) ? carry : nb != 0u;
        carry = __shfl_sync(BPE_FULL, out0, DOWN ? 0 : 31) != 0u;
    } else {
        uint32_t f = out0 | ((((odd0 ^ fr) >> top) & 1u) << 1);
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t other = DOWN ? __shfl_down_sync(BPE_FULL, f, d) : __shfl_up_sync(BPE_FULL, f, d);
            if (DOWN ? lane + d < 32 : lane >= d) f = carry_then(other, f);     // the lanes before this one apply first
        }
        const uint32_t before = DOWN ? __shfl_down_sync(BPE_FULL, f, 1) : __shfl_up_sync(BPE_FULL, f, 1);
        cin = (DOWN ? lane == 31 : lane == 0) ? carry : carry_apply(before, carry) != 0u;
        carry = carry_apply(__shfl_sync(BPE_FULL, f, DOWN ? 0 : 31), carry) != 0u;
    }
    return cin ? odd0 ^ fr : odd0;
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
            while (c < BPE_LONG_CLASS && (int64_t)bpe_class_capacity(c) < n) ++c;
            if (n > BPE_MAX_POSITIONS) { if (status) atomicOr(status + i, 1); c = -1; }
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

// Barrier over the W warps of one team (team index `team` within a block of BW warps).
template <int W, int BW>
__device__ __forceinline__ void team_sync(int team) {
    if (W == 1) __syncwarp();
    else if (W == BW) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(W * 32) : "memory");
}

// floor(x / d) for x * d < 2^32, d >= 1: inv = ceil(2^32 / d), or 0 for d = 1.
__device__ __forceinline__ uint32_t bpe_inv(uint32_t d) { return d > 1u ? 0xFFFFFFFFu / d + 1u : 0u; }
__device__ __forceinline__ uint32_t bpe_div(uint32_t x, uint32_t d, uint32_t inv) { return d > 1u ? __umulhi(x, inv) : x; }

// W: warps per word.
template <int W>
__global__ void __launch_bounds__(bpe_block_warps(W) * 32)
bpe_lanes_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets,
                 const int32_t* __restrict__ list, const int32_t* __restrict__ list_count,
                 int32_t* __restrict__ work_counter, BpeDeviceTable t,
                 uint16_t* __restrict__ out_tok, int32_t* __restrict__ counts,
                 int32_t* __restrict__ status) {
    constexpr int P = BPE_LANE_SLOTS;
    constexpr int T = 32 * W;                    // lanes of a team
    constexpr int STRIDE = T + 2;                // elements between the slots of one lane
    constexpr int BW = bpe_block_warps(W);
    constexpr int TEAMS = BW / W;
    extern __shared__ uint4 bpe_dyn[];
    __shared__ uint2 s_hot[32 * 32];             // direct table for pairs of small ids
    __shared__ uint16_t s_btok[256];
    __shared__ uint32_t s_red[BW];               // per-warp partial minima
    __shared__ int32_t s_word[TEAMS][2];         // claimed word index, new length
    for (int i = threadIdx.x; i < 32 * 32; i += BW * 32) s_hot[i] = __ldg(t.hot + i);
    for (int i = threadIdx.x; i < 256; i += BW * 32) s_btok[i] = __ldg(t.byte_tok + i);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int team = warp / W, tw = warp % W;    // team, warp within team
    const int g = tw * 32 + lane;                // lane within team
    uint8_t* area = reinterpret_cast<uint8_t*>(bpe_dyn) + (size_t)team * bpe_team_bytes(W);
    uint16_t* cur = reinterpret_cast<uint16_t*>(area);           // [P][STRIDE] live tokens
    uint16_t* nxt = cur + P * STRIDE;                            // [P][STRIDE] the next round's
    uint16_t* xf = nxt + P * STRIDE;                             // [T] rank of every lane's first pair   (W > 1)
    uint16_t* xl = xf + T;                                       // [T] rank of every lane's last pair    (W > 1)
    uint32_t* m_a = reinterpret_cast<uint32_t*>(xl + T);         // [T] right-walk links, then selected pairs
    uint32_t* m_b = m_a + T;                                     // [T] left-walk links, then survivors
    uint32_t* m_c = m_b + T;                                     // [T] candidates, then output base
    const int n_words = *list_count;

    for (;;) {
        int wi;
        if (W == 1) {
            wi = 0;
            if (lane == 0) wi = atomicAdd(work_counter, 1);
            wi = __shfl_sync(BPE_FULL, wi, 0);
        } else {
            if (g == 0) s_word[team][0] = atomicAdd(work_counter, 1);
            team_sync<W, BW>(team);
            wi = s_word[team][0];
        }
        if (wi >= n_words) break;
        const int row = list[wi];
        const int64_t off = offsets[row];
        int n = (int)(offsets[row + 1] - off);               // 1 <= n <= T * P by classification
        uint32_t Pp = (uint32_t)(n + T - 1) / T;             // positions per lane: lane g owns [g Pp, (g + 1) Pp)
        uint32_t inv = bpe_inv(Pp);

        for (int i = g; i < n; i += T) {
            const uint32_t l = bpe_div((uint32_t)i, Pp, inv);
            cur[((uint32_t)i - l * Pp) * STRIDE + l] = s_btok[__ldg(bytes + off + i)];
        }
        team_sync<W, BW>(team);

        int round = 0;
        const int max_rounds = n + 2;
        for (; round < max_rounds; ++round) {
            // ---- A: entries of the lane's pairs, the word's bound, "right neighbour ranks better" bits
            const uint16_t* col = cur + g;
            const int p0 = g * (int)Pp;
            uint32_t val[P];
            uint32_t emin = BPE_FULL, gt = 0, r_prev = BPE_NONE;
            uint32_t a = col[0];
            const uint32_t t_right = cur[g + 1];             // first token of the next lane (padding element after the last lane)
#pragma unroll
            for (int j = 0; j < P; ++j) {
                if (j < (int)Pp) {
                    uint32_t b = col[((j + 1) % P) * STRIDE];
                    if (j + 1 == (int)Pp) b = t_right;
                    uint32_t key = BPE_FULL, v = BPE_FULL;
                    if (p0 + j + 1 < n) bpe_lookup(t, s_hot, a, b, key, v);
                    const uint32_t r = v & 0xFFFFu;
                    if (t.single_step) key = r == BPE_NONE ? BPE_FULL : (((r + 1u) << 16) | r);
                    val[j] = v;
                    emin = min(emin, key);
                    if (j > 0) gt |= (r_prev > r ? 1u : 0u) << (j - 1);
                    r_prev = r;
                    a = b;
                }
            }
            const uint32_t r_first = val[0] & 0xFFFFu, r_last = r_prev;
            emin = __reduce_min_sync(BPE_FULL, emin);
            uint32_t r_nf, r_pl;                             // the next lane's first rank, the previous lane's last rank
            if (W == 1) {
                r_nf = __shfl_down_sync(BPE_FULL, r_first, 1);
                r_pl = __shfl_up_sync(BPE_FULL, r_last, 1);
                if (lane == 31) r_nf = BPE_NONE;
                if (lane == 0) r_pl = BPE_NONE;
            } else {
                xf[g] = (uint16_t)r_first;
                xl[g] = (uint16_t)r_last;
                if (lane == 0) s_red[warp] = emin;
                team_sync<W, BW>(team);
#pragma unroll
                for (int k = 0; k < W; ++k) emin = min(emin, s_red[team * W + k]);
                r_nf = g + 1 < T ? (uint32_t)xf[g + 1] : BPE_NONE;
                r_pl = g > 0 ? (uint32_t)xl[g - 1] : BPE_NONE;
            }
            if (emin == BPE_FULL) break;                     // no pair can merge: done (uniform over the team)
            const uint32_t B = emin >> 16;

            // ---- B: candidate and link masks of the lane's positions
            const int top = (int)Pp - 1, sh = 32 - (int)Pp;
            const uint32_t full = BPE_FULL >> sh;
            gt |= (r_last > r_nf ? 1u : 0u) << top;
            uint32_t cand = 0;
#pragma unroll
            for (int j = 0; j < P; ++j)
                if (j < (int)Pp) cand |= ((val[j] & 0xFFFFu) < B ? 1u : 0u) << j;
            const uint32_t leq = (~(gt << 1) & ~1u) | (r_pl <= r_first ? 1u : 0u);   // bit j: rank(j-1) <= rank(j)
            const uint32_t link_r = cand & gt;               // the right neighbour is a candidate that goes first
            const uint32_t link_l = cand & leq;              // the left neighbour is a candidate that goes first
            const int len = min(max(n - p0, 0), (int)Pp);
            const uint32_t valid = len >= 32 ? BPE_FULL : ((1u << len) - 1u);

            // ---- selection on the masks
            uint32_t sel, kept;
            int q0, n_new;
            if (W == 1) {
                bool carry = false;
                const uint32_t odd_r = __brev(chain_parity<true>(__brev(link_r) >> sh, top, full, carry, lane) << sh);
                carry = false;
                const uint32_t odd_l = chain_parity<false>(link_l, top, full, carry, lane);
                sel = cand & ~odd_l & ~odd_r;
                if (t.single_step) {                         // only the leftmost pair of the lowest rank
                    const uint32_t any = __ballot_sync(BPE_FULL, sel != 0u);
                    sel = lane == __ffs(any) - 1 ? (sel & (0u - sel)) : 0u;
                }
                uint32_t prev = __shfl_up_sync(BPE_FULL, (sel >> top) & 1u, 1);
                if (lane == 0) prev = 0u;
                kept = valid & ~((sel << 1) | prev);
                const int x = __popc(kept);
                int incl = x;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int y = __shfl_up_sync(BPE_FULL, incl, d);
                    if (lane >= d) incl += y;
                }
                q0 = incl - x;
                n_new = __shfl_sync(BPE_FULL, incl, 31);
            } else {
                m_a[g] = link_r; m_b[g] = link_l; m_c[g] = cand;
                team_sync<W, BW>(team);
                if (tw == 0) {
                    bool carry = false;
                    for (int b = W - 1; b >= 0; --b) {       // right walks, last lanes first
                        const int gg = b * 32 + lane;
                        m_a[gg] = __brev(chain_parity<true>(__brev(m_a[gg]) >> sh, top, full, carry, lane) << sh);
                    }
                    __syncwarp();
                    carry = false;
                    uint32_t sel_carry = 0;                  // was the last pair of the lane before the block selected
                    int base = 0;
                    bool took = false;
                    for (int b = 0; b < W; ++b) {
                        const int gg = b * 32 + lane;
                        const uint32_t odd_l = chain_parity<false>(m_b[gg], top, full, carry, lane);
                        uint32_t s = m_c[gg] & ~odd_l & ~m_a[gg];
                        if (t.single_step) {
                            const uint32_t any = __ballot_sync(BPE_FULL, s != 0u);
                            s = (!took && lane == __ffs(any) - 1) ? (s & (0u - s)) : 0u;
                            took = took || any != 0u;
                        }
                        uint32_t prev = __shfl_up_sync(BPE_FULL, (s >> top) & 1u, 1);
                        if (lane == 0) prev = sel_carry;
                        sel_carry = __shfl_sync(BPE_FULL, (s >> top) & 1u, 31);
                        const int ln = min(max(n - gg * (int)Pp, 0), (int)Pp);
                        const uint32_t vd = ln >= 32 ? BPE_FULL : ((1u << ln) - 1u);
                        const uint32_t kp = vd & ~((s << 1) | prev);
                        const int x = __popc(kp);
                        int incl = x;
#pragma unroll
                        for (int d = 1; d < 32; d <<= 1) {
                            const int y = __shfl_up_sync(BPE_FULL, incl, d);
                            if (lane >= d) incl += y;
                        }
                        m_a[gg] = s; m_b[gg] = kp; m_c[gg] = (uint32_t)(base + incl - x);
                        base += __shfl_sync(BPE_FULL, incl, 31);
                    }
                    if (lane == 0) s_word[team][1] = base;
                }
                team_sync<W, BW>(team);
                sel = m_a[g]; kept = m_b[g]; q0 = (int)m_c[g];
                n_new = s_word[team][1];
            }

            // ---- C: merge, and deal the survivors out again in the other buffer
            const uint32_t Pn = (uint32_t)(n_new + T - 1) / T, inv_n = bpe_inv(Pn);
            uint32_t q = (uint32_t)q0;
#pragma unroll
            for (int j = 0; j < P; ++j) {
                if (j < (int)Pp && ((kept >> j) & 1u)) {
                    uint32_t v = col[j * STRIDE];
                    if ((sel >> j) & 1u) v = val[j] >> 16;
                    const uint32_t l = bpe_div(q, Pn, inv_n);
                    nxt[(q - l * Pn) * STRIDE + l] = (uint16_t)v;
                    ++q;
                }
            }
            team_sync<W, BW>(team);
            uint16_t* sw = cur; cur = nxt; nxt = sw;
            n = n_new; Pp = Pn; inv = inv_n;
        }

        for (int q = g; q < n; q += T) {
            const uint32_t l = bpe_div((uint32_t)q, Pp, inv);
            out_tok[off + q] = cur[((uint32_t)q - l * Pp) * STRIDE + l];
        }
        if (g == 0) {
            counts[row] = n;
            if (round >= max_rounds && status) atomicOr(status + row, 2);
        }
        team_sync<W, BW>(team);
    }
}

// Words beyond the lanes kernel's capacity: one block per word, state in global memory.  The
// tokens live in place in the output area (uint16 at the input offsets); ranks and the three mask
// arrays sit in a per-word piece of `long_area`, claimed from `long_cursor` by the block.
__global__ void __launch_bounds__(BPE_LONG_WARPS * 32)
bpe_long_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets,
                const int32_t* __restrict__ list, const int32_t* __restrict__ list_count,
                int32_t* __restrict__ work_counter, BpeDeviceTable t, uint16_t* __restrict__ out_tok,
                int32_t* __restrict__ counts, int32_t* __restrict__ status,
                uint8_t* __restrict__ long_area, unsigned long long* __restrict__ long_cursor) {
    constexpr int W = BPE_LONG_WARPS;
    __shared__ uint32_t s_red[W][2];
    __shared__ uint2 s_hot[32 * 32];
    __shared__ long long s_word[2];                           // claimed word index / new length, scratch offset
    for (int i = threadIdx.x; i < 32 * 32; i += W * 32) s_hot[i] = __ldg(t.hot + i);
    __syncthreads();
    const int lane = threadIdx.x & 31, tw = threadIdx.x >> 5;
    const int tt = threadIdx.x;
    const uint32_t lt = (1u << lane) - 1u;
    const int n_words = *list_count;

    for (;;) {
        if (tt == 0) {
            const int w = atomicAdd(work_counter, 1);
            s_word[0] = w;
            if (w < n_words) {
                const int r = list[w];
                s_word[1] = (long long)atomicAdd(long_cursor, (unsigned long long)bpe_long_bytes(offsets[r + 1] - offsets[r]));
            }
        }
        __syncthreads();
        const int wi = (int)s_word[0];
        if (wi >= n_words) break;
        const int row = list[wi];
        const int64_t off = offsets[row];
        int n = (int)(offsets[row + 1] - off);
        const int G0 = (n + 31) >> 5;
        uint16_t* tok = out_tok + off;                                    // [n] live tokens, compact
        uint8_t* piece = long_area + s_word[1];
        uint16_t* rk = reinterpret_cast<uint16_t*>(piece);                // [n] rank of the pair (i, i+1)
        uint32_t* m_leq = reinterpret_cast<uint32_t*>(piece + ((2 * (int64_t)n + 15) / 16) * 16);   // bit i: rank(i-1) <= rank(i); later: survivors
        uint32_t* m_cs = m_leq + ((G0 + 3) / 4) * 4;                      // candidates, then selected pairs
        uint32_t* g_aux = m_cs + ((G0 + 3) / 4) * 4;                      // right-walk parity, then output base
        __syncthreads();                                                  // s_word is free again

        for (int i = tt; i < n; i += W * 32) tok[i] = __ldg(t.byte_tok + __ldg(bytes + off + i));
        __syncthreads();

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
                    uint32_t key, v;
                    bpe_lookup(t, s_hot, tok[i], tok[i + 1], key, v);
                    r = key & 0xFFFFu; fut = key >> 16;
                }
                if (i < n) rk[i] = (uint16_t)r;
                gmin = min(gmin, r);
                if (r != BPE_NONE) bmin = min(bmin, fut);
            }
            gmin = __reduce_min_sync(BPE_FULL, gmin);
            bmin = __reduce_min_sync(BPE_FULL, bmin);
            if (lane == 0) { s_red[tw][0] = gmin; s_red[tw][1] = bmin; }
            __syncthreads();
#pragma unroll
            for (int k = 0; k < W; ++k) { gmin = min(gmin, s_red[k][0]); bmin = min(bmin, s_red[k][1]); }
            if (gmin == BPE_NONE) break;                       // no pair can merge: done (uniform over the block)
            const uint32_t B = t.single_step ? gmin + 1 : bmin;

            // ---- 2: candidate masks and "not worse than my left neighbour" masks
            for (int g = tw; g < groups; g += W) {
                const int i = g * 32 + lane;
                const uint32_t r = i < n ? (uint32_t)rk[i] : BPE_NONE;
                uint32_t rp = __shfl_up_sync(BPE_FULL, r, 1);
                if (lane == 0) rp = i > 0 ? (uint32_t)rk[i - 1] : BPE_NONE;
                const uint32_t cand = __ballot_sync(BPE_FULL, r < B);
                const uint32_t leq = __ballot_sync(BPE_FULL, rp <= r);
                if (lane == 0) { m_cs[g] = cand; m_leq[g] = leq; }
            }
            __syncthreads();

            // ---- 3: on the masks, one lane per 32 positions (first warp)
            if (tw == 0) {
                const int blocks = (groups + 31) >> 5;
                bool carry = false;                            // right walks, last block first
                for (int b = blocks - 1; b >= 0; --b) {
                    const int g = b * 32 + lane;
                    const bool live = g < groups;
                    const uint32_t cand = live ? m_cs[g] : 0u;
                    const uint32_t leq = live ? m_leq[g] : BPE_FULL;
                    const uint32_t leq_next = g + 1 < groups ? m_leq[g + 1] : BPE_FULL;
                    // bit i: the right neighbour ranks strictly better: not (rank(i) <= rank(i+1))
                    const uint32_t link = cand & ~((leq >> 1) | (leq_next << 31));
                    const uint32_t odd = __brev(chain_parity<true>(__brev(link), 31, BPE_FULL, carry, lane));
                    if (live) g_aux[g] = odd;
                }
                __syncwarp();
                carry = false;                                 // left walks, selection, survivors, output bases
                uint32_t sel_carry = 0;                        // was the position before the block selected
                int base = 0;
                bool took = false;
                for (int b = 0; b < blocks; ++b) {
                    const int g = b * 32 + lane;
                    const bool live = g < groups;
                    const uint32_t cand = live ? m_cs[g] : 0u;
                    const uint32_t leq = live ? m_leq[g] : 0u;
                    const uint32_t oddl = chain_parity<false>(cand & leq, 31, BPE_FULL, carry, lane);
                    uint32_t sel = live ? (cand & ~oddl & ~g_aux[g]) : 0u;
                    if (t.single_step) {                       // only the leftmost pair of the lowest rank
                        const uint32_t any = __ballot_sync(BPE_FULL, sel != 0);
                        const int first = __ffs(any) - 1;
                        sel = (!took && lane == first) ? (sel & (0u - sel)) : 0u;
                        took = took || any != 0;
                    }
                    uint32_t prev = __shfl_up_sync(BPE_FULL, sel, 1) >> 31;
                    if (lane == 0) prev = sel_carry;
                    sel_carry = __shfl_sync(BPE_FULL, sel, 31) >> 31;
                    const int cnt_pos = n - g * 32;            // positions of this group
                    const uint32_t valid = !live ? 0u : (cnt_pos >= 32 ? BPE_FULL : ((1u << cnt_pos) - 1u));
                    const uint32_t kept = valid & ~((sel << 1) | prev);
                    int x = __popc(kept), incl = x;
#pragma unroll
                    for (int d = 1; d < 32; d <<= 1) {
                        const int y = __shfl_up_sync(BPE_FULL, incl, d);
                        if (lane >= d) incl += y;
                    }
                    if (live) { m_cs[g] = sel; m_leq[g] = kept; g_aux[g] = (uint32_t)(base + incl - x); }
                    base += __shfl_sync(BPE_FULL, incl, 31);
                }
                if (lane == 0) s_word[0] = base;
            }
            __syncthreads();

            // ---- 4: merge and compact in place, W groups at a time
            const int n_new = (int)s_word[0];
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
                __syncthreads();                               // every warp has read its tokens of this tile
                if ((kept >> lane) & 1u) tok[base + __popc(kept & lt)] = (uint16_t)v;
            }
            __syncthreads();
            n = n_new;
        }

        if (tt == 0) {
            counts[row] = n;
            if (round >= max_rounds && status) atomicOr(status + row, 2);
        }
        __syncthreads();
    }
}

}  // namespace dnatok

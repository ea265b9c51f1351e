// BPE merge engine: exact Hugging Face merge order in a handful of data-parallel rounds.
//
// One warp owns one pre-tokenised word, kept as a COMPACT array of 16-bit tokens in shared memory
// (no links, no tombstones).  A round:
//   A. every adjacent pair is looked up in the merge table (perfect hash, two dependent loads);
//      its rank is stored and B = min over the present ranks r of F[r] is reduced, where F[r] is
//      the lowest rank of any pair that contains the token rank r creates;
//   B. pairs with rank < B are candidates.  Hugging Face would take them in (rank, position)
//      order, skipping a pair when an earlier one consumed one of its tokens.  On a path that
//      greedy choice has a closed form: follow the strictly improving priorities to the left and to
//      the right of a candidate down to the local optimum; the candidate is taken iff both walks
//      have even length.  The two parities are segmented prefix-XORs, computed 32 positions at a
//      time with carry-propagating bit tricks on ballot masks (one backward sweep, one forward);
//   C. the forward sweep also applies the selected merges and compacts the array in place.
// Everything created in a round contains a new token, so it ranks >= B, above every pair merged
// in that round: the round equals the sequential queue run over the same ranks.  Rounds repeat
// until no pair has a rank: 5-7 rounds for DNA words of any length, ~3.3 position visits per
// input byte in total.  Equal ranks on neighbouring pairs (runs of one token) fall out of the same
// rule, because priority is (rank, position): every other pair from the left.
//
// A table whose merge operands may be created by later ranks has no usable F; for it the host
// selects single_step: one merge per round, the leftmost pair of the lowest rank.
//
// Words are binned by length into capacity classes (shared memory per word = 4.125 bytes per
// position); each class is one launch of resident warps that pull words from a shared counter.
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
constexpr int BPE_WARPS = 8;                    // warps (= words in flight) per block

__host__ __device__ constexpr int bpe_class_capacity(int c) {
    return c < 8 ? (256 << c) : 49152;          // 256 ... 32768, 49152
}
__host__ __device__ constexpr int bpe_slot_bytes(int C) { return 4 * C + C / 8; }

struct BpeDeviceTable {
    const uint32_t* disp;        // [n_tokens] row displacement of the left token
    const uint32_t* slots;       // (left << 16) | rank, 0xFFFFFFFF when empty
    const uint16_t* merge_out;   // [n_merges] token created by a rank
    const uint16_t* future;      // [n_merges] F: lowest rank of a pair containing that token
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

// Bin rows by length: class_count[c] rows land in class_list[c * n_rows ...].  One atomic per
// warp and class (rows of a batch mostly share a class).
__global__ void bpe_classify_kernel(const int64_t* __restrict__ offsets, int64_t n_rows,
                                    int32_t* __restrict__ class_count, int32_t* __restrict__ class_list,
                                    int32_t* __restrict__ counts, int32_t* __restrict__ status) {
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

template <int C>
__global__ void __launch_bounds__(BPE_WARPS * 32)
bpe_rounds_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets,
                  const int32_t* __restrict__ list, const int32_t* __restrict__ list_count,
                  int32_t* __restrict__ work_counter, BpeDeviceTable t,
                  uint16_t* __restrict__ out_tok, int32_t* __restrict__ counts,
                  int32_t* __restrict__ status) {
    extern __shared__ uint4 bpe_dyn[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t lt = (1u << lane) - 1u;
    uint8_t* slot = reinterpret_cast<uint8_t*>(bpe_dyn) + (size_t)warp * bpe_slot_bytes(C);
    uint16_t* tok = reinterpret_cast<uint16_t*>(slot);          // [C] live tokens, compact
    uint16_t* rk = tok + C;                                     // [C] rank of the pair (i, i+1)
    uint32_t* oddr = reinterpret_cast<uint32_t*>(rk + C);       // [C/32] right-walk parity bits per 32 positions
    const int n_words = *list_count;

    for (;;) {
        int wi = 0;
        if (lane == 0) wi = atomicAdd(work_counter, 1);
        wi = __shfl_sync(0xffffffffu, wi, 0);
        if (wi >= n_words) break;
        const int row = list[wi];
        const int64_t off = offsets[row];
        int n = (int)(offsets[row + 1] - off);               // 1 <= n <= C by classification

        for (int i = lane; i < n; i += 32) tok[i] = __ldg(t.byte_tok + __ldg(bytes + off + i));
        __syncwarp();

        int round = 0;
        const int max_rounds = n + 2;
        for (; round < max_rounds; ++round) {
            const int groups = (n + 31) >> 5;
            // ---- A: ranks of all pairs, bound B, lowest rank
            uint32_t bmin = BPE_NONE, gmin = BPE_NONE;
            for (int g = 0; g < groups; ++g) {
                const int i = g * 32 + lane;
                uint32_t r = BPE_NONE;
                if (i + 1 < n) r = bpe_rank(t, tok[i], tok[i + 1]);
                if (i < n) rk[i] = (uint16_t)r;
                if (r != BPE_NONE) {
                    gmin = min(gmin, r);
                    bmin = min(bmin, (uint32_t)__ldg(t.future + r));
                }
            }
            gmin = __reduce_min_sync(0xffffffffu, gmin);
            if (gmin == BPE_NONE) break;                       // no pair can merge: done
            uint32_t B = __reduce_min_sync(0xffffffffu, bmin);
            if (t.single_step) B = gmin + 1;
            __syncwarp();

            // ---- B: parity of the improving walk to the right, last group first
            bool carry = false;                                // parity bit of position 32(g+1)
            for (int g = groups - 1; g >= 0; --g) {
                const int i = g * 32 + lane;
                const uint32_t r = i < n ? (uint32_t)rk[i] : BPE_NONE;
                const uint32_t rn = i + 1 < n ? (uint32_t)rk[i + 1] : BPE_NONE;
                const bool link = r < B && rn < r;             // the right neighbour is a candidate with better priority
                const uint32_t c = __brev(__ballot_sync(0xffffffffu, link));
                const uint32_t odd = __brev(run_parity(c, carry));
                if (lane == 0) oddr[g] = odd;
                carry = odd & 1u;
            }
            __syncwarp();

            // ---- C: left-walk parity, selection, merge and in-place compaction, first group first
            carry = false;                                     // left parity bit of position 32g - 1
            uint32_t prev_sel = 0;                             // was position 32g - 1 selected (its partner is dropped)
            int out = 0;
            bool took_one = false;
            for (int g = 0; g < groups; ++g) {
                const int i = g * 32 + lane;
                const uint32_t r = i < n ? (uint32_t)rk[i] : BPE_NONE;
                const uint32_t rp = i > 0 && i < n ? (uint32_t)rk[i - 1] : BPE_NONE;
                const uint32_t tk = i < n ? (uint32_t)tok[i] : 0u;
                const bool cand = r < B;
                const bool link = cand && rp <= r;             // rp <= r < B: the left neighbour is a candidate and goes first
                const uint32_t candm = __ballot_sync(0xffffffffu, cand);
                const uint32_t oddl = run_parity(__ballot_sync(0xffffffffu, link), carry);
                carry = oddl >> 31;
                uint32_t sel = candm & ~oddl & ~oddr[g];
                if (t.single_step) {                           // only the leftmost pair of the lowest rank
                    sel = took_one ? 0u : (sel & (0u - sel));
                    took_one = took_one || sel != 0;
                }
                const uint32_t valid = (i < n ? 1u : 0u);
                const uint32_t validm = __ballot_sync(0xffffffffu, valid);
                const uint32_t dropped = (sel << 1) | prev_sel;          // positions consumed as the right half of a pair
                const uint32_t kept = validm & ~dropped;
                uint32_t v = tk;
                if ((sel >> lane) & 1u) v = __ldg(t.merge_out + r);
                __syncwarp();                                  // every lane has read this group's tokens
                if ((kept >> lane) & 1u) tok[out + __popc(kept & lt)] = (uint16_t)v;
                out += __popc(kept);
                prev_sel = sel >> 31;
            }
            n = out;
            __syncwarp();
        }

        for (int i = lane; i < n; i += 32) out_tok[off + i] = tok[i];
        if (lane == 0) {
            counts[row] = n;
            if (round >= max_rounds && status) atomicOr(status + row, 2);
        }
        __syncwarp();
    }
}

}  // namespace dnatok

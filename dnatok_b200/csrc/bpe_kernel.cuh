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
    return 2 * (BPE_LANE_SLOTS + 1) * (32 * W + 2) * 2 + (W > 1 ? 32 * W * 8 : 0);
}
// caller scratch of one word of the long class: ranks (2 bytes per position) and three mask words per 32 positions
__host__ __device__ constexpr int64_t bpe_long_bytes(int64_t n) { return ((2 * n + 15) / 16 + 3 * ((n + 127) / 128)) * 16; }

struct BpeDeviceTable {
    const uint32_t* disp;        // [n_tokens] row displacement of the left token
    const uint2* slots;          // x = (rank << 16) | created, y = (left << 16) | F; all ones when empty
    const uint16_t* merge_out;   // [n_merges] token created by a rank
    const uint2* hot;            // [32 * 32] pairs of ids < 32: x as in slots, y = (F << 16) | rank; all ones when no merge
    const uint16_t* byte_tok;    // [256]
    int32_t single_step;
    uint32_t hot_ranks;          // every rank below this creates an id < 32
    uint32_t bytes_hot;          // 1: every initial symbol is an id < 32
    uint32_t filler;             // one past the largest token id: a token whose pairs never merge (disp and slots have room for it)
    // the table packed for shared memory (NULL when it does not exist): 16-bit displacements, 32-bit slots
    // (left << 16) | rank, one word (F << 16) | created id per rank
    const uint4* compact;
    uint32_t compact_bytes, compact_slot, compact_info, compact_last;
};

// Shared-memory addresses of the three parts of the packed table.
struct BpeSmemTable { uint32_t disp, slot, info, last; };

// One table entry: x = (rank << 16) | created id, y = (left id << 16) | F.  Ranks compare like the x
// words themselves (equal ranks create equal ids), so x is what the kernels keep per pair.  What
// the kernels work with is the pair (x, key), key = (F << 16) | rank: the minimum of the keys over a
// word gives the bound B (upper half) and tells whether any pair merges.  The table in shared
// memory holds (x, key) directly; an entry from global memory is checked against its left id first.
__device__ __forceinline__ uint2 bpe_cold_entry(const BpeDeviceTable& t, uint32_t a, uint32_t b) {
    uint2 s = __ldg(t.slots + __ldg(t.disp + a) + b);
    s.y = (s.y >> 16) == a ? __byte_perm(s.x, s.y, 0x5432) : BPE_FULL;
    if (s.y == BPE_FULL) s.x = BPE_FULL;
    return s;
}

constexpr int BPE_HOT_STRIDE = 36;              // row stride of the shared-memory table: the 16 pairs of four consecutive ids fall into 16 different banks
constexpr int BPE_HOT_WORDS = 33 * BPE_HOT_STRIDE;   // row and column 32 stay empty: 32 is the filler token behind the end of a word
constexpr uint32_t BPE_FILLER = 32;

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
// with all of them set.  A word passes its incoming parity on only when all its bits are set;
// unless some lane has such a word the neighbour's own top bit is the carry and one shuffle
// replaces the scan over carry functions.
//
// chain_prepare does everything that does not depend on the parity entering the block of 32 lanes
// and returns the block's carry function (what leaves the block as a function of what enters);
// chain_finish takes the entering parity and gives the lane's parities.
struct ChainPrep {
    uint32_t odd0, fr;   // parities with nothing entering the word; the run they flip on when something does
    uint32_t f;          // fast: parity leaving the word; else: carry function from the block's entry to this word's exit
    bool fast;
};

template <bool DOWN>
__device__ __forceinline__ ChainPrep chain_prepare(uint32_t c, int top, uint32_t full, int lane, uint32_t& block_fn) {
    ChainPrep p;
    p.odd0 = run_parity(c);
    p.fr = first_run(c);
    const uint32_t out0 = (p.odd0 >> top) & 1u;
    p.fast = __ballot_sync(BPE_FULL, c == full) == 0u;
    if (p.fast) {
        p.f = out0;
        block_fn = __shfl_sync(BPE_FULL, out0, DOWN ? 0 : 31) * 3u;      // a constant function
    } else {
        uint32_t f = out0 | ((((p.odd0 ^ p.fr) >> top) & 1u) << 1);
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const uint32_t other = DOWN ? __shfl_down_sync(BPE_FULL, f, d) : __shfl_up_sync(BPE_FULL, f, d);
            if (DOWN ? lane + d < 32 : lane >= d) f = carry_then(other, f);     // the lanes before this one apply first
        }
        p.f = f;
        block_fn = __shfl_sync(BPE_FULL, f, DOWN ? 0 : 31);
    }
    return p;
}

template <bool DOWN>
__device__ __forceinline__ uint32_t chain_finish(const ChainPrep& p, bool carry, int lane) {
    const uint32_t before = DOWN ? __shfl_down_sync(BPE_FULL, p.f, 1) : __shfl_up_sync(BPE_FULL, p.f, 1);
    const bool cin = (DOWN ? lane == 31 : lane == 0) ? carry : (p.fast ? before != 0u : carry_apply(before, carry) != 0u);
    return cin ? p.odd0 ^ p.fr : p.odd0;
}

// Both steps for blocks visited one after the other: `carry` enters the block and leaves it updated.
template <bool DOWN>
__device__ __forceinline__ uint32_t chain_parity(uint32_t c, int top, uint32_t full, bool& carry, int lane) {
    uint32_t fn;
    const ChainPrep p = chain_prepare<DOWN>(c, top, full, lane, fn);
    const uint32_t odd = chain_finish<DOWN>(p, carry, lane);
    carry = carry_apply(fn, carry) != 0u;
    return odd;
}

// Where the merge kernels leave a row's final token count (the count after truncation plus the special
// tokens), so that no separate pass over the rows is needed: lengths may be NULL.
struct BpeLengths {
    int32_t* lengths;
    int64_t cap_content;     // most content tokens a row may keep
    int32_t n_special;
    int32_t clip_is_error;   // rows cut by the output width (not by requested truncation) get DNATOK_ROW_CLIPPED
    // When ids is set the merge kernels also write every finished row in its final padded layout ([CLS] tokens
    // [SEP] padding, or the padding first), so no output pass follows; otherwise the tokens go to the scratch buffer.
    void* ids;
    void* mask;              // may be NULL
    int64_t out_stride;
    int32_t cls_id, sep_id, pad_id, pad_left;
    int32_t id_bits, mask_bits;
    // 1: the caller did not zero the status words: the kernel that sees a row first (the binning pass, or the merge
    // kernel when rows are not binned) writes the row's word instead of OR-ing into it
    int32_t store_status;
};
// A row's status bits into its word.
__device__ __forceinline__ void bpe_put_status(int32_t* status, int64_t row, int32_t bits, bool store) {
    if (!status) return;
    if (store) status[row] = bits;
    else if (bits) atomicOr(status + row, bits);
}
__device__ __forceinline__ int32_t bpe_put_length(const BpeLengths& L, int64_t row, int64_t n) {
    const int64_t kept = n < L.cap_content ? n : L.cap_content;
    if (L.lengths) L.lengths[row] = (int32_t)kept + L.n_special;
    return (L.clip_is_error && n > kept) ? 4 : 0;            // DNATOK_ROW_CLIPPED
}

// One finished row of n tokens into the caller's padded layout, the columns dealt to the T threads that worked on
// the row (g: this thread's index among them); tok(i) returns token i.
template <typename TokFn>
__device__ __forceinline__ void bpe_write_row(const BpeLengths& L, int64_t row, int n, int g, int T, TokFn tok) {
    const int stride = (int)L.out_stride;
    const int kept = n < L.cap_content ? n : (int)L.cap_content;
    const bool has_cls = L.cls_id >= 0, has_sep = L.sep_id >= 0;
    const int total = kept + (has_cls ? 1 : 0) + (has_sep ? 1 : 0);
    const int c0 = (L.pad_left ? stride - total : 0) + (has_cls ? 1 : 0);     // column of the first content token
    const int64_t base = row * L.out_stride;
    for (int col = g; col < stride; col += T) {
        const int i = col - c0;
        int32_t v = L.pad_id;
        bool on = true;
        if (i >= 0 && i < kept) v = (int32_t)tok(i);
        else if (i == -1 && has_cls) v = L.cls_id;
        else if (i == kept && has_sep) v = L.sep_id;
        else on = false;
        if (L.id_bits == 64) reinterpret_cast<int64_t*>(L.ids)[base + col] = v;
        else reinterpret_cast<int32_t*>(L.ids)[base + col] = v;
        if (L.mask) {
            if (L.mask_bits == 64) reinterpret_cast<int64_t*>(L.mask)[base + col] = on;
            else if (L.mask_bits == 32) reinterpret_cast<int32_t*>(L.mask)[base + col] = on;
            else reinterpret_cast<uint8_t*>(L.mask)[base + col] = on;
        }
    }
}


// Bin rows by length: class_count[c] rows land in class_list[c * n_rows ...].  One atomic per
// warp and class (rows of a batch mostly share a class).  Classes outside class_mask are not
// launched by the host; a row that belongs to one is flagged instead of being dropped silently.
__global__ void bpe_classify_kernel(const int64_t* __restrict__ offsets, int64_t n_rows,
                                    int32_t* __restrict__ class_count, int32_t* __restrict__ class_list,
                                    int32_t* __restrict__ counts, int32_t* __restrict__ status,
                                    uint32_t class_mask, BpeLengths len_out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int lane = threadIdx.x & 31;
    int c = -1;
    if (i < n_rows) {
        const int64_t n = offsets[i + 1] - offsets[i];
        int32_t bits = 0;
        counts[i] = 0;
        if (n > 0) {
            c = 0;
            while (c < BPE_LONG_CLASS && (int64_t)bpe_class_capacity(c) < n) ++c;
            if (n > BPE_MAX_POSITIONS) { bits = 1; c = -1; }
            else if (!((class_mask >> c) & 1u)) { bits = 8; c = -1; }   // outside the caller's length hint
        }
        if (c < 0) {                                              // no kernel will visit this row
            bpe_put_length(len_out, i, 0);
            if (len_out.ids) bpe_write_row(len_out, i, 0, 0, 1, [](int) { return 0u; });
        }
        bpe_put_status(status, i, bits, len_out.store_status != 0);
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
// BAR0 is the hardware barrier of team 0; code that runs teams of several widths in one block gives every
// width its own range of barriers.
template <int W, int BW, int BAR0 = 1>
__device__ __forceinline__ void team_sync(int team) {
    if (W == 1) __syncwarp();
    else if (W == BW) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(team + BAR0), "r"(W * 32) : "memory");
}

// Shared-memory accesses by 32-bit address in the shared window: the lanes kernel keeps its buffer
// addresses in registers and reaches every slot with a compile-time offset.
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ void sts_u16(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((uint16_t)v) : "memory");
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint2 lds_u64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
    return v;
}

// The entry of the pair (a, b) from the packed table in shared memory: three dependent shared-memory
// loads where bpe_cold_entry makes two dependent loads from global memory.
__device__ __forceinline__ uint2 bpe_smem_entry(const BpeSmemTable& st, uint32_t a, uint32_t b) {
    const uint32_t idx = min(lds_u16(st.disp + 2u * a) + b, st.last);
    const uint32_t s = lds_u32(st.slot + 4u * idx);
    const bool hit = (s >> 16) == a;
    const uint32_t r = hit ? (s & 0xFFFFu) : 0u;
    const uint32_t inf = lds_u32(st.info + 4u * r);
    uint2 e;
    e.x = hit ? (r << 16) | (inf & 0xFFFFu) : BPE_FULL;
    e.y = hit ? (inf & 0xFFFF0000u) | r : BPE_FULL;
    return e;
}

// floor(x / d) for 1 <= d <= 32, x < 2^16: __umulhi(2 x + 1, ceil(2^31 / d)).
__device__ __forceinline__ uint32_t bpe_inv(uint32_t d) { return (0x80000000u + d - 1u) / d; }

// The per-slot bodies of the lanes kernel run from the lane's last slot down to slot 0 through a
// switch on the slot count with fall-through cases: one indirect jump instead of a guard per slot,
// every slot index a compile-time constant (shared-memory offsets, register names, mask bits), and
// no value handed from slot to slot except the accumulators.
#define BPE_SLOTS_DOWN(X) \
    X(31) X(30) X(29) X(28) X(27) X(26) X(25) X(24) X(23) X(22) X(21) X(20) X(19) X(18) X(17) X(16) \
    X(15) X(14) X(13) X(12) X(11) X(10) X(9) X(8) X(7) X(6) X(5) X(4) X(3) X(2) X(1) X(0)

#ifndef BPE_LANES_MIN_BLOCKS
#define BPE_LANES_MIN_BLOCKS 4
#endif
__host__ __device__ constexpr int bpe_min_blocks(int W) { return W <= 8 ? BPE_LANES_MIN_BLOCKS : W == 16 ? 2 : 1; }

// Block-wide tables of the lanes code, in static shared memory of the kernel that runs it.
struct BpeLanesShared {
    uint2* hot;          // [BPE_HOT_WORDS] direct table for pairs of small ids, row stride BPE_HOT_STRIDE
    uint16_t* btok;      // [256] initial symbol of every byte
    uint32_t* inv;       // [BPE_LANE_SLOTS + 1] bpe_inv(d)
    uint32_t* red;       // [BW] per-warp partial minima
    uint32_t* fn;        // [BW] per-warp carry functions of the two walks
    uint32_t* blk;       // [BW] per-warp survivor count and border bits
    int32_t* word;       // [BW] claimed word index, at the team's first warp
};
#define BPE_LANES_SHARED(BW_, sh)                                      \
    __shared__ uint2 sh##_hot[BPE_HOT_WORDS];                          \
    __shared__ uint16_t sh##_btok[256];                                \
    __shared__ uint32_t sh##_inv[BPE_LANE_SLOTS + 1];                  \
    __shared__ uint32_t sh##_red[BW_], sh##_fn[BW_], sh##_blk[BW_];    \
    __shared__ int32_t sh##_word[BW_];                                 \
    const BpeLanesShared sh{sh##_hot, sh##_btok, sh##_inv, sh##_red, sh##_fn, sh##_blk, sh##_word}

template <int BW>
__device__ __forceinline__ void bpe_lanes_setup(const BpeLanesShared& sh, const BpeDeviceTable& t) {
    for (int i = threadIdx.x; i < BPE_HOT_WORDS; i += BW * 32) sh.hot[i] = make_uint2(BPE_FULL, BPE_FULL);
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * 32; i += BW * 32) sh.hot[(i >> 5) * BPE_HOT_STRIDE + (i & 31)] = __ldg(t.hot + i);
    for (int i = threadIdx.x; i < 256; i += BW * 32) sh.btok[i] = __ldg(t.byte_tok + i);
    if (threadIdx.x >= 1 && threadIdx.x <= BPE_LANE_SLOTS) sh.inv[threadIdx.x] = bpe_inv(threadIdx.x);
    __syncthreads();
}

// The words of one list through teams of W warps, in a block of BW warps whose teams each own TEAM_BYTES of
// the dynamic shared memory.  list == NULL: no binning was done because the caller vouches that every row
// fits; the n_words rows are taken as they come, and a row longer than direct_limit is flagged and left empty.
template <int W, int BW, int BAR0, int TEAM_BYTES, bool ST = false>
__device__ __forceinline__ void bpe_lanes_body(const BpeLanesShared& sh, const BpeSmemTable& stab, uint16_t* const sm,
                 const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets,
                 const int32_t* __restrict__ list, const int n_words,
                 int32_t* __restrict__ work_counter, const BpeDeviceTable& t,
                 uint16_t* __restrict__ out_tok, int32_t* __restrict__ counts,
                 int32_t* __restrict__ status, const BpeLengths& len_out, int32_t direct_limit) {
    constexpr int P = BPE_LANE_SLOTS;
    constexpr int T = 32 * W;                    // lanes of a team
    constexpr int STRIDE = T + 2;                // elements between the slots of one lane
    constexpr int BUF = (P + 1) * STRIDE;        // one token buffer: P slots and the copy of the next lane's first token
    static_assert(TEAM_BYTES >= (int)bpe_team_bytes(W), "team area too small");
    uint16_t* const s_btok = sh.btok;
    uint32_t* const s_inv = sh.inv;
    uint32_t* const s_red = sh.red;
    uint32_t* const s_fn = sh.fn;
    uint32_t* const s_blk = sh.blk;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int team = warp / W, tw = warp % W;    // team, warp within team
    int32_t* const s_word = sh.word + team * W;
    const int g = tw * 32 + lane;                // lane within team
    // All token traffic goes through shared-memory byte addresses held in registers.
    constexpr uint32_t S2 = 2 * STRIDE;          // bytes between the slots of one lane
    const uint32_t team_base = (uint32_t)team * (TEAM_BYTES / 2);
    const uint32_t hot_base = smem_u32(sh.hot);
    uint32_t cur = smem_u32(sm + team_base + g); // this lane's column in the buffer of live tokens
    uint32_t nxt = cur + 2 * BUF;                // ... and in the buffer the round writes
    uint32_t* const xf = reinterpret_cast<uint32_t*>(sm + team_base + 2 * BUF);   // [T] entry of every lane's first pair (W > 1)
    uint32_t* const xl = xf + T;                                                  // [T] entry of every lane's last pair  (W > 1)

    // work_counter == NULL: the batch is a single wave (no more words than teams in the grid), and team k of block b
    // takes word b + k * blocks, with no counter to claim from (and none to zero before the launch)
    bool first = true;
    for (;;) {
        int wi;
        if (!work_counter) {
            wi = first ? (int)blockIdx.x + (int)gridDim.x * team : n_words;
            first = false;
        } else if (W == 1) {
            wi = 0;
            if (lane == 0) wi = atomicAdd(work_counter, 1);
            wi = __shfl_sync(BPE_FULL, wi, 0);
        } else {
            if (g == 0) s_word[0] = atomicAdd(work_counter, 1);
            team_sync<W, BW, BAR0>(team);
            wi = s_word[0];
        }
        if (wi >= n_words) {
            team_sync<W, BW, BAR0>(team);                    // the claim slot is reused by whatever this team runs next
            break;
        }
        const int row = list ? list[wi] : wi;
        const int64_t off = offsets[row];
        const int64_t n64 = offsets[row + 1] - off;
        int n = (int)n64;                                    // 1 <= n <= T * P by classification
        if (!list && (n64 < 1 || n64 > direct_limit)) {      // direct rows are not vetted: an empty row, or one the hint misstated
            if (g == 0) {
                counts[row] = 0;
                bpe_put_length(len_out, row, 0);
                bpe_put_status(status, row, n64 > 0 ? 8 : 0, len_out.store_status != 0);
            }
            if (len_out.ids) bpe_write_row(len_out, row, 0, g, T, [](int) { return 0u; });
            team_sync<W, BW, BAR0>(team);                          // everybody has read the claimed index
            continue;
        }
        uint32_t Pp = (uint32_t)(n + T - 1) / T;             // positions per lane: lane g owns [g Pp, (g + 1) Pp)
        uint32_t inv = s_inv[Pp];

        // While every token of the word is a small id (all_hot) the pairs come from the shared-memory
        // table and the filler behind the end of the word is that table's empty row 32; afterwards they
        // come from the table in global memory and the filler is the id one past the vocabulary.
        bool all_hot = t.bytes_hot != 0u;
        uint32_t filler = all_hot ? BPE_FILLER : t.filler;
        if (g == 0) sts_u16(cur + 2 * T, filler);            // what the last lane sees as "the next lane's first token"
        // Every lane fetches its own chunk of the word as aligned 32-bit words (all requested before the
        // first is used), maps the bytes to tokens and fills its column.
        {
            const uint32_t c0 = (uint32_t)g * Pp;            // first position of this lane
            const uintptr_t a0 = reinterpret_cast<uintptr_t>(bytes + off + c0);
            const uint32_t mis = (uint32_t)(a0 & 3u);
            const uint32_t* src = reinterpret_cast<const uint32_t*>(a0 - mis);
            const int first = (int)c0 - (int)mis;            // position of byte 0 of src[0]
            uint32_t w[P / 4 + 1];
#pragma unroll
            for (int k = 0; k <= P / 4; ++k)                 // a word is read when it holds a byte of the word
                w[k] = (4 * k < (int)(Pp + mis) && first + 4 * k < n && first + 4 * k + 3 >= 0) ? __ldg(src + k) : 0u;
#pragma unroll
            for (int k = 0; k < P / 4; ++k) {
                if (4 * k < (int)Pp) {
                    const uint32_t r = __funnelshift_r(w[k], w[k + 1], 8 * mis);
#pragma unroll
                    for (int bb = 0; bb < 4; ++bb) {
                        const uint32_t tk = s_btok[(r >> (8 * bb)) & 0xFFu];
                        sts_u16(cur + (4 * k + bb) * S2, (int)c0 + 4 * k + bb < n ? tk : filler);
                    }
                }
            }
        }
        team_sync<W, BW, BAR0>(team);

        int round = 0;
        const int max_rounds = n + 2;
        for (; round < max_rounds; ++round) {
            const int top = (int)Pp - 1, sh = 32 - (int)Pp;
            const int p0 = g * (int)Pp;
            // the next lane's first token becomes this lane's slot Pp, so that every slot finds its right neighbour one slot up
            uint32_t t_up = lds_u16(cur + 2);                // handed from slot to slot: the token one slot up
            sts_u16(cur + Pp * S2, t_up);
            team_sync<W, BW, BAR0>(team);

            // ---- A: entries of the lane's pairs, the word's bound, "right neighbour ranks better" bits.
            // While every token of the word is a small id all pairs come from the shared-memory table and
            // the slots are straight-line code; afterwards each lane takes the table its pair needs.
            uint32_t val[P + 1];                             // x word of every pair's entry: (rank << 16) | created id
            uint32_t gt = 0;                                 // bit j: the pair right of slot j's ranks better
            uint32_t emin = BPE_FULL;
#define BPE_A_TAIL(J)                                                                         \
                    val[J] = e.x;                                                             \
                    emin = min(emin, e.y);                                                    \
                    if (e.x > val[J + 1]) gt |= 1u << J;
            if (all_hot) {
                switch (Pp) {
#define BPE_A(J)                                                                              \
                    case J + 1: {                                                             \
                        const uint32_t a = lds_u16(cur + J * S2), b = t_up;                   \
                        const uint2 e = lds_u64(hot_base + (a * BPE_HOT_STRIDE + b) * 8u);   /* the filler's pairs are empty */ \
                        t_up = a;                                                             \
                        BPE_A_TAIL(J)                                                         \
                    }
                    BPE_SLOTS_DOWN(BPE_A)
#undef BPE_A
                    default: break;
                }
            } else {
                switch (Pp) {
#define BPE_A(J)                                                                              \
                    case J + 1: {                                                             \
                        const uint32_t a = lds_u16(cur + J * S2), b = t_up;                   \
                        const uint2 e = ST ? bpe_smem_entry(stab, a, b) : bpe_cold_entry(t, a, b);   /* the filler's pairs are empty */ \
                        t_up = a;                                                             \
                        BPE_A_TAIL(J)                                                         \
                    }
                    BPE_SLOTS_DOWN(BPE_A)
#undef BPE_A
                    default: break;
                }
            }
#undef BPE_A_TAIL
            uint32_t v_top = val[0];                         // the entry of the last slot, whichever register holds it
            switch (top) {
#define BPE_T(J) case J: v_top = val[J]; break;
                BPE_SLOTS_DOWN(BPE_T)
#undef BPE_T
                default: break;
            }
            gt &= (1u << top) - 1u;                          // the last slot was compared with nothing; set below
            const uint32_t v_first = val[0];
            emin = __reduce_min_sync(BPE_FULL, emin);
            uint32_t v_nf, v_pl;                             // the next lane's first entry, the previous lane's last entry
            if (W == 1) {
                v_nf = __shfl_down_sync(BPE_FULL, v_first, 1);
                v_pl = __shfl_up_sync(BPE_FULL, v_top, 1);
                if (lane == 31) v_nf = BPE_FULL;
                if (lane == 0) v_pl = BPE_FULL;
            } else {
                xf[g] = v_first;
                xl[g] = v_top;
                if (lane == 0) s_red[warp] = emin;
                team_sync<W, BW, BAR0>(team);
#pragma unroll
                for (int k = 0; k < W; ++k) emin = min(emin, s_red[team * W + k]);
                v_nf = g + 1 < T ? xf[g + 1] : BPE_FULL;
                v_pl = g > 0 ? xl[g - 1] : BPE_FULL;
            }
            if (emin == BPE_FULL) break;                     // no pair can merge: done (uniform over the team)
            const uint32_t Bs = emin & 0xFFFF0000u;          // rank < B  <=>  entry < B << 16

            // ---- B: candidate and link masks of the lane's positions
            if (v_top > v_nf) gt |= 1u << top;
            uint32_t cand = 0, vmax = 0;                     // vmax: the highest-ranking candidate's entry
            switch (Pp) {
#define BPE_B(J) case J + 1: if (val[J] < Bs) { cand |= 1u << J; vmax = max(vmax, val[J]); }
                BPE_SLOTS_DOWN(BPE_B)
#undef BPE_B
                default: break;
            }
            // the round creates small ids only if all its candidates rank below t.hot_ranks
            const bool big = (vmax >> 16) >= t.hot_ranks && cand != 0u;
            const uint32_t full = BPE_FULL >> sh;
            const uint32_t leq = (~(gt << 1) & ~1u) | (v_pl <= v_first ? 1u : 0u);   // bit j: rank(j-1) <= rank(j)
            const uint32_t link_r = cand & gt;               // the right neighbour is a candidate that goes first
            const uint32_t link_l = cand & leq;              // the left neighbour is a candidate that goes first
            const int len = min(max(n - p0, 0), (int)Pp);
            const uint32_t valid = len >= 32 ? BPE_FULL : ((1u << len) - 1u);

            // ---- selection on the masks
            uint32_t sel, kept;
            int q0, n_new;
            if (W == 1) {
                all_hot = all_hot && !__any_sync(BPE_FULL, big);
                bool carry = false;
                const uint32_t odd_r = __brev(chain_parity<true>(__brev(link_r) >> sh, top, full, carry, lane) << sh);
                carry = false;
                const uint32_t odd_l = chain_parity<false>(link_l, top, full, carry, lane);
                sel = cand & ~odd_l & ~odd_r;
                if (t.single_step) {                         // only the leftmost pair of the lowest rank
                    const uint32_t any = __ballot_sync(BPE_FULL, sel != 0u);
                    sel = lane == __ffs(any) - 1 ? (sel & (0u - sel)) : 0u;
                }
                uint32_t prev = __shfl_up_sync(BPE_FULL, sel >> top, 1);
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
                // every warp works on its own 32 lanes; what crosses warps are the blocks' carry functions
                // (first barrier) and their survivor counts with the border bits (second barrier)
                uint32_t fn_r, fn_l;
                const ChainPrep pr = chain_prepare<true>(__brev(link_r) >> sh, top, full, lane, fn_r);
                const ChainPrep pl = chain_prepare<false>(link_l, top, full, lane, fn_l);
                const uint32_t any_cand = t.single_step ? __ballot_sync(BPE_FULL, cand != 0u) : 0u;
                const bool any_big = __any_sync(BPE_FULL, big);
                if (lane == 0) s_fn[warp] = fn_r | (fn_l << 2) | (any_cand ? 16u : 0u) | (any_big ? 32u : 0u);
                team_sync<W, BW, BAR0>(team);
                bool carry_r = false, carry_l = false, earlier = false;
#pragma unroll
                for (int k = 0; k < W; ++k) all_hot = all_hot && !(s_fn[team * W + k] & 32u);
                for (int k = W - 1; k > tw; --k) carry_r = carry_apply(s_fn[team * W + k] & 3u, carry_r) != 0u;
                for (int k = 0; k < tw; ++k) {
                    const uint32_t f = s_fn[team * W + k];
                    carry_l = carry_apply((f >> 2) & 3u, carry_l) != 0u;
                    earlier = earlier || (f & 16u);
                }
                const uint32_t odd_r = __brev(chain_finish<true>(pr, carry_r, lane) << sh);
                const uint32_t odd_l = chain_finish<false>(pl, carry_l, lane);
                sel = cand & ~odd_l & ~odd_r;
                if (t.single_step)                           // only the leftmost pair of the lowest rank
                    sel = (!earlier && lane == __ffs(any_cand) - 1) ? (cand & (0u - cand)) : 0u;
                uint32_t prev = __shfl_up_sync(BPE_FULL, sel >> top, 1);
                if (lane == 0) prev = 0u;                    // corrected below from the block before
                kept = valid & ~((sel << 1) | prev);
                const int x = __popc(kept);
                int incl = x;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int y = __shfl_up_sync(BPE_FULL, incl, d);
                    if (lane >= d) incl += y;
                }
                const uint32_t first_valid = __shfl_sync(BPE_FULL, valid & 1u, 0);
                if (lane == 31) s_blk[warp] = (uint32_t)incl | ((sel >> top) << 16) | (first_valid << 17);
                team_sync<W, BW, BAR0>(team);
                // lane k looks at block k: its count drops by one when the block before it merged across the border
                const uint32_t w = lane < W ? s_blk[team * W + lane] : 0u;
                uint32_t lost = __shfl_up_sync(BPE_FULL, (w >> 16) & 1u, 1);
                if (lane == 0) lost = 0u;
                lost &= (w >> 17) & 1u;
                const int tot = (int)(w & 0xFFFFu) - (int)lost;
                int bincl = tot;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int y = __shfl_up_sync(BPE_FULL, bincl, d);
                    if (lane >= d) bincl += y;
                }
                const int base = __shfl_sync(BPE_FULL, bincl - tot, tw);
                n_new = __shfl_sync(BPE_FULL, bincl, 31);
                const bool mine_lost = __shfl_sync(BPE_FULL, lost, tw) != 0u;
                if (mine_lost && lane == 0) kept &= ~1u;
                q0 = base + incl - x - ((mine_lost && lane > 0) ? 1 : 0);
            }

            // ---- C: merge, and deal the survivors out again in the other buffer, last slot first.
            // Position q goes to lane l = q / Pn, slot q - l Pn: byte 2 (q STRIDE - l (Pn STRIDE - 1)) of the buffer.
            const uint32_t Pn = (uint32_t)(n_new + T - 1) / T, inv_n = s_inv[Pn];
            const uint32_t back = 2 * (Pn * STRIDE - 1);
            const uint32_t dst = nxt - 2 * g;                // start of the buffer the round writes
            uint32_t q = (uint32_t)q0 + (uint32_t)__popc(kept);
            switch (Pp) {
#define BPE_C(J)                                                                              \
                case J + 1: {                                                                 \
                    const bool keep_ = (kept & (1u << J)) != 0u;                              \
                    if (keep_) --q;                                                           \
                    const uint32_t l_ = __umulhi(2u * q + 1u, inv_n);                         \
                    const uint32_t tk_ = lds_u16(cur + J * S2);                               \
                    if (keep_) sts_u16(dst + q * S2 - l_ * back, (sel & (1u << J)) ? val[J] : tk_); \
                }
                BPE_SLOTS_DOWN(BPE_C)
#undef BPE_C
                default: break;
            }
            {                                                // filler behind the new end, up to the lanes' common slot count
                filler = all_hot ? BPE_FILLER : t.filler;
                const uint32_t pt = (uint32_t)n_new + (uint32_t)g;
                if (pt < Pn * T) {
                    const uint32_t l_ = __umulhi(2u * pt + 1u, inv_n);
                    sts_u16(dst + pt * S2 - l_ * back, filler);
                }
                if (g == 0) sts_u16(dst + 2 * T, filler);    // the column behind the last lane
            }
            team_sync<W, BW, BAR0>(team);
            const uint32_t sw = cur; cur = nxt; nxt = sw;
            n = n_new; Pp = Pn; inv = inv_n;
        }

        if (len_out.ids) {
            const uint32_t col0 = cur - 2 * g;               // the team's buffer
            bpe_write_row(len_out, row, n, g, T, [&](int q) {
                const uint32_t l = __umulhi(2u * (uint32_t)q + 1u, inv);
                return lds_u16(col0 + 2 * (((uint32_t)q - l * Pp) * STRIDE + l));
            });
        } else {
            for (int q = g; q < n; q += T) {
                const uint32_t l = __umulhi(2u * (uint32_t)q + 1u, inv);
                out_tok[off + q] = (uint16_t)lds_u16(cur - 2 * g + 2 * (((uint32_t)q - l * Pp) * STRIDE + l));
            }
        }
        if (g == 0) {
            counts[row] = n;
            const int32_t bits = bpe_put_length(len_out, row, n) | (round >= max_rounds ? 2 : 0);
            bpe_put_status(status, row, bits, len_out.store_status != 0 && !list);   // binned rows were written by the binning pass
        }
        team_sync<W, BW, BAR0>(team);
    }
}

// W: warps per word.
template <int W>
__global__ void __launch_bounds__(bpe_block_warps(W) * 32, bpe_min_blocks(W))
bpe_lanes_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets,
                 const int32_t* __restrict__ list, const int32_t* __restrict__ list_count,
                 int32_t* __restrict__ work_counter, BpeDeviceTable t,
                 uint16_t* __restrict__ out_tok, int32_t* __restrict__ counts,
                 int32_t* __restrict__ status, BpeLengths len_out, int32_t n_direct, int32_t direct_limit) {
    constexpr int BW = bpe_block_warps(W);
    extern __shared__ uint4 bpe_dyn[];
    BPE_LANES_SHARED(BW, sh);
    bpe_lanes_setup<BW>(sh, t);
    bpe_lanes_body<W, BW, 1, (int)bpe_team_bytes(W)>(sh, BpeSmemTable{}, reinterpret_cast<uint16_t*>(bpe_dyn), bytes, offsets, list,
                                                     list ? *list_count : n_direct, work_counter, t, out_tok, counts,
                                                     status, len_out, direct_limit);
}

// The same for a vocabulary whose packed table fits into shared memory beside the teams' buffers: one block of
// 32 warps per SM, the table copied in once per block, every lookup of the general mode answered from it.
constexpr int BPE_ST_WARPS = 32;
__host__ __device__ constexpr size_t bpe_st_team_area(int W) { return (size_t)(BPE_ST_WARPS / W) * bpe_team_bytes(W); }
template <int W>
__global__ void __launch_bounds__(BPE_ST_WARPS * 32, 1)
bpe_lanes_st_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets,
                    const int32_t* __restrict__ list, const int32_t* __restrict__ list_count,
                    int32_t* __restrict__ work_counter, BpeDeviceTable t,
                    uint16_t* __restrict__ out_tok, int32_t* __restrict__ counts,
                    int32_t* __restrict__ status, BpeLengths len_out, int32_t n_direct, int32_t direct_limit) {
    // Launched with programmatic stream serialisation when the launch before it in the stream may be a kernel: this
    // grid's blocks can be placed while that one drains, and wait here until it is complete and visible.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    extern __shared__ uint4 bpe_dyn[];
    BPE_LANES_SHARED(BPE_ST_WARPS, sh);
    uint4* const tab = bpe_dyn + bpe_st_team_area(W) / 16;
    for (uint32_t i = threadIdx.x; i < t.compact_bytes / 16; i += BPE_ST_WARPS * 32) tab[i] = __ldg(t.compact + i);
    bpe_lanes_setup<BPE_ST_WARPS>(sh, t);                     // ends with a block-wide barrier
    const uint32_t base = smem_u32(tab);
    const BpeSmemTable stab{base, base + t.compact_slot, base + t.compact_info, t.compact_last};
    {
        // A small batch is spread over all blocks: only as many teams of a block take part as the words per
        // block ask for (words are claimed from one counter, and the blocks that start first would otherwise
        // take them all while other SMs stay idle).
        const int n_words = list ? *list_count : n_direct;
        const int active = (n_words + (int)gridDim.x - 1) / (int)gridDim.x;
        if ((int)(threadIdx.x >> 5) / W >= active) return;
    }
    // sixteen teams of two warps need sixteen hardware barriers: barrier 0 is theirs as well once the set-up is over
    bpe_lanes_body<W, BPE_ST_WARPS, (W == 2 ? 0 : 1), (int)bpe_team_bytes(W), true>(sh, stab, reinterpret_cast<uint16_t*>(bpe_dyn), bytes,
                                                                     offsets, list, list ? *list_count : n_direct, work_counter,
                                                                     t, out_tok, counts, status, len_out, direct_limit);
}

// Rows of several length classes in one launch: a block of BPE_MIXED_WARPS warps works through the classes
// from the widest team to the narrowest, splitting into more and more teams on the way, so a batch of mixed
// lengths has one tail instead of one per class.  levels.classes[k] holds the classes (bit c: class c) that
// run with teams of 1 << k warps; a team's area at every width lies inside the area of the team it was part
// of one width up, and every width has its own hardware barriers, so teams move on without waiting for their
// block.
constexpr int BPE_MIXED_WARPS = 16;
constexpr int BPE_MIXED_LEVELS = 5;
__host__ __device__ constexpr size_t bpe_mixed_warp_bytes() {      // shared memory per warp so that every width fits
    size_t m = 0;
    for (int w = 1; w <= BPE_MIXED_WARPS; w *= 2) {
        const size_t per = (bpe_team_bytes(w) + (size_t)w - 1) / (size_t)w;
        if (per > m) m = per;
    }
    return (m + 15) / 16 * 16;
}
__host__ __device__ constexpr size_t bpe_mixed_bytes() { return bpe_mixed_warp_bytes() * BPE_MIXED_WARPS; }
struct BpeMixedLevels { uint32_t classes[BPE_MIXED_LEVELS]; };

template <int W, int BAR0>
__device__ __forceinline__ void bpe_mixed_level(const BpeLanesShared& sh, uint16_t* sm, uint32_t classes,
                 const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets,
                 const int32_t* __restrict__ class_list, int64_t n_rows, const int32_t* __restrict__ class_count,
                 int32_t* __restrict__ work, const BpeDeviceTable& t, uint16_t* __restrict__ out_tok,
                 int32_t* __restrict__ counts, int32_t* __restrict__ status, const BpeLengths& len_out) {
    for (; classes; classes &= classes - 1u) {
        const int c = __ffs(classes) - 1;
        bpe_lanes_body<W, BPE_MIXED_WARPS, BAR0, (int)(bpe_mixed_warp_bytes() * W)>(
            sh, BpeSmemTable{}, sm, bytes, offsets, class_list + (int64_t)c * n_rows, class_count[c], work + c, t, out_tok, counts, status,
            len_out, 0);
    }
}

__global__ void __launch_bounds__(BPE_MIXED_WARPS * 32, 2)
bpe_mixed_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets,
                 const int32_t* __restrict__ class_list, int64_t n_rows, const int32_t* __restrict__ class_count,
                 int32_t* __restrict__ work, BpeDeviceTable t, uint16_t* __restrict__ out_tok,
                 int32_t* __restrict__ counts, int32_t* __restrict__ status, BpeLengths len_out, BpeMixedLevels levels) {
    extern __shared__ uint4 bpe_dyn[];
    BPE_LANES_SHARED(BPE_MIXED_WARPS, sh);
    bpe_lanes_setup<BPE_MIXED_WARPS>(sh, t);
    uint16_t* const sm = reinterpret_cast<uint16_t*>(bpe_dyn);
#define BPE_LEVEL(K, BAR0) \
    bpe_mixed_level<(1 << K), BAR0>(sh, sm, levels.classes[K], bytes, offsets, class_list, n_rows, class_count, work, t, \
                                    out_tok, counts, status, len_out);
    BPE_LEVEL(4, 0) BPE_LEVEL(3, 1) BPE_LEVEL(2, 3) BPE_LEVEL(1, 7) BPE_LEVEL(0, 0)
#undef BPE_LEVEL
}
#undef BPE_SLOTS_DOWN

// Words beyond the lanes kernel's capacity: one block per word, state in global memory.  The
// tokens live in place in the output area (uint16 at the input offsets); ranks and the three mask
// arrays sit in a per-word piece of `long_area`, claimed from `long_cursor` by the block.
__global__ void __launch_bounds__(BPE_LONG_WARPS * 32)
bpe_long_kernel(const uint8_t* __restrict__ bytes, const int64_t* __restrict__ offsets,
                const int32_t* __restrict__ list, const int32_t* __restrict__ list_count,
                int32_t* __restrict__ work_counter, BpeDeviceTable t, uint16_t* __restrict__ out_tok,
                int32_t* __restrict__ counts, int32_t* __restrict__ status,
                uint8_t* __restrict__ long_area, unsigned long long* __restrict__ long_cursor, BpeLengths len_out) {
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
                    const uint32_t a = tok[i], b = tok[i + 1];
                    const uint2 e = (a | b) < 32u ? s_hot[a * 32u + b] : bpe_cold_entry(t, a, b);
                    r = e.x >> 16; fut = e.y >> 16;
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

        if (len_out.ids) bpe_write_row(len_out, row, n, tt, W * 32, [&](int q) { return (uint32_t)tok[q]; });
        if (tt == 0) {
            counts[row] = n;
            const int32_t bits = bpe_put_length(len_out, row, n) | (round >= max_rounds ? 2 : 0);
            bpe_put_status(status, row, bits, false);
        }
        __syncthreads();
    }
}

}  // namespace dnatok

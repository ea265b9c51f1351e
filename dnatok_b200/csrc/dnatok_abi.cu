// C ABI of the library (see include/dnatok_b200.h): handles, table upload, format resolution,
// kernel launches and the host-buffer pipeline.  No PyTorch, no allocation inside the device
// entry points other than the one-time table upload per device.
#include "../../include/dnatok_b200.h"

#include <atomic>
#include <climits>
#include <condition_variable>
#include <functional>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "bpe_kernel.cuh"
#include "bpe_table.h"
#include "embed_kernel.cuh"
#include "emit_kernel.cuh"
#include "kmer_kernel.cuh"
#include "kmer_table_kernel.cuh"

using namespace dnatok;

namespace {

thread_local std::string g_err;
std::atomic<int64_t> g_launches{0};
std::atomic<int64_t> g_host_mask_threads{-1};                 // -1: as many as the host has cores, at most 4; 0: mask copied from the device
std::atomic<int64_t> g_host_mask_min_bytes{16ll << 20};      // smaller masks are not worth the threads
thread_local int64_t g_last_h2d = 0, g_last_d2h = 0;          // bytes the last dnatok_encode_host of this thread copied
std::atomic<int64_t> g_kmer_force_segments{0};                // 1: segment encoder whenever scratch is given
std::atomic<int64_t> g_kmer_poll_limit{1 << 20};              // polls before a segment gives up waiting for the one before it
std::atomic<int64_t> g_kmer_test_withhold{-1};                // tests: the ticket whose segment publishes nothing
std::atomic<int64_t> g_host_chunk_bytes{64ll << 20};         // bytes over the host link (in + out) per chunk of the host pipeline
std::atomic<int64_t> g_host_chunk_threshold{128ll << 20};    // batches below this size are not chunked
std::atomic<int64_t> g_bpe_team_warps{0};                    // BPE: force this team width (warps per word); 0: choose by batch size
std::atomic<int64_t> g_bpe_team_max{8};                      // BPE: widest team the automatic choice takes
std::atomic<int64_t> g_kmer_overlap_launch{1};               // k-mer row kernel launched with programmatic stream serialisation
std::atomic<int64_t> g_emit_overlap_launch{1};               // padded output kernel launched with programmatic stream serialisation
std::atomic<int64_t> g_host_mask_early{1};                   // host path: masks whose row lengths follow from the byte counts are written at once
std::atomic<int64_t> g_bpe_overlap_launch{1};                // BPE shared-memory-table kernel launched with programmatic stream serialisation
std::atomic<int64_t> g_bpe_smem_table{1};                    // BPE: keep a small vocabulary's merge table in shared memory
std::atomic<int64_t> g_bpe_fused_output{1};                  // BPE, padded layout through dnatok_encode: merge kernels write the final rows
std::atomic<int64_t> g_bpe_mixed{1};                         // BPE: batches of several length classes in one launch
std::atomic<int64_t> g_bpe_block_team_rows{-1};              // BPE: batches up to this many rows use a block per word; -1: 8 per SM

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}

#define CUDA_TRY(expr)                                                                          \
    do {                                                                                        \
        cudaError_t e_ = (expr);                                                                \
        if (e_ != cudaSuccess) return fail(DNATOK_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e_)); \
    } while (0)

#define LAUNCH_CHECK(name)                                                                      \
    do {                                                                                        \
        ++g_launches;                                                                           \
        cudaError_t e_ = cudaGetLastError();                                                    \
        if (e_ != cudaSuccess) return fail(DNATOK_ERR_CUDA, "launch of %s: %s", name, cudaGetErrorString(e_)); \
    } while (0)

struct DeviceTables {
    int32_t* lut256 = nullptr;       // char LUT / k-mer single ids
    uint8_t* bpe_compact = nullptr;  // BPE: the merge table packed for shared memory (when it exists)
    int32_t* start_lut = nullptr;    // char: ids of a row's first character, when they differ
    int32_t* kmer_ids = nullptr;
    int32_t* table5 = nullptr;       // table-driven k-mer handles: 5^k windows, runs
    int32_t* exp_off = nullptr;
    int32_t* exp_ids = nullptr;
    uint32_t* disp = nullptr;
    uint64_t* slots = nullptr;
    uint16_t* merge_out = nullptr;
    uint64_t* hot = nullptr;
    uint16_t* byte_tok = nullptr;
    int sm_count = 0;
    // host-pipeline staging (grow only)
    uint8_t* st_bytes = nullptr;  size_t st_bytes_cap = 0;
    int64_t* st_offsets = nullptr; size_t st_offsets_cap = 0;
    void* st_ids = nullptr;       size_t st_ids_cap = 0;
    void* st_mask = nullptr;      size_t st_mask_cap = 0;
    int32_t* st_lengths = nullptr; size_t st_rows_cap = 0;
    int32_t* st_status = nullptr;
    int64_t* st_out_offsets = nullptr;
    void* st_scratch = nullptr;   size_t st_scratch_cap = 0;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev_lengths = nullptr;  // marks the arrival of the row lengths in host memory
    // chunked host pipeline: three streams, one event per chunk, per-row words, pinned chunk-local offsets
    cudaStream_t pipe_streams[3] = {nullptr, nullptr, nullptr};
    std::vector<cudaEvent_t> pipe_events;
    void* st_pipe_rows = nullptr; size_t st_pipe_rows_cap = 0;    // lengths then status, int32 each
    int64_t* h_offsets = nullptr; size_t h_offsets_cap = 0;
    int32_t* h_rows = nullptr; size_t h_rows_cap = 0;   // pinned: row lengths and status on their way back (2 x n_rows)
};

}  // namespace

struct dnatok_handle {
    int kind = 0;
    dnatok_specials sp{};
    std::vector<int32_t> lut256;
    int k = 0;
    std::vector<int32_t> kmer_ids;
    std::vector<int32_t> start_lut;    // char: 256 ids of a row's first character; empty: same as lut256
    std::vector<int32_t> table5, exp_off, exp_ids;   // table-driven k-mer handles (dnatok_create_kmer_table)
    bool kmer_table = false;
    int tail_singles = 1;
    int32_t kmer_affine_base = -1;     // >= 0 when kmer_ids[i] == base + i for every i
    bool lut_identity = false;         // char: id == byte value for every byte (byte-level tokenizers)
    int64_t hint_min_row = 0, hint_max_row = 0;   // caller's bounds on row length in bytes; 0, 0: unknown
    BpeHostTable bpe;
    std::mutex mu;
    std::map<int, DeviceTables> dev;
};

namespace {

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

template <typename T>
int upload(T** dst, const std::vector<T>& src) {
    CUDA_TRY(cudaMalloc((void**)dst, src.size() * sizeof(T)));
    CUDA_TRY(cudaMemcpy(*dst, src.data(), src.size() * sizeof(T), cudaMemcpyHostToDevice));
    return 0;
}

struct BpeLaunchInfo;
int bpe_launch_info(int dev, const BpeLaunchInfo** out);

// Tables of the handle on the current device (uploaded on first use).
int tables_for_current_device(dnatok_handle* h, DeviceTables** out) {
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(h->mu);
    auto it = h->dev.find(dev);
    if (it == h->dev.end()) {
        it = h->dev.emplace(dev, DeviceTables()).first;
        DeviceTables& d = it->second;
        struct Undo {                                    // a failed upload leaves no half-built entry behind
            dnatok_handle* h; int dev; bool keep;
            ~Undo() {
                if (keep) return;
                DeviceTables& x = h->dev[dev];
                void* ptrs[] = {x.lut256, x.start_lut, x.kmer_ids, x.table5, x.exp_off, x.exp_ids, x.disp, x.slots, x.merge_out, x.hot, x.byte_tok, x.bpe_compact};
                for (void* p : ptrs) if (p) cudaFree(p);
                h->dev.erase(dev);
            }
        } undo{h, dev, false};
        CUDA_TRY(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
        int rc = upload(&d.lut256, h->lut256);
        if (rc) return rc;
        if (h->kind == DNATOK_KIND_KMER && !h->kmer_table && (rc = upload(&d.kmer_ids, h->kmer_ids))) return rc;
        if (h->kmer_table) {
            if ((rc = upload(&d.table5, h->table5))) return rc;
            if ((rc = upload(&d.exp_off, h->exp_off))) return rc;
            if ((rc = upload(&d.exp_ids, h->exp_ids))) return rc;
        }
        if (!h->start_lut.empty() && (rc = upload(&d.start_lut, h->start_lut))) return rc;
        if (h->kind == DNATOK_KIND_BPE) {
            if ((rc = upload(&d.disp, h->bpe.disp))) return rc;
            if (!h->bpe.compact.empty() && (rc = upload(&d.bpe_compact, h->bpe.compact))) return rc;
            if ((rc = upload(&d.slots, h->bpe.slots))) return rc;
            if ((rc = upload(&d.merge_out, h->bpe.merge_out))) return rc;
            if ((rc = upload(&d.hot, h->bpe.hot))) return rc;
            if ((rc = upload(&d.byte_tok, h->bpe.byte_tok))) return rc;
            const BpeLaunchInfo* info;
            if ((rc = bpe_launch_info(dev, &info))) return rc;     // configures every merge kernel once per device
        }
        undo.keep = true;
    }
    *out = &it->second;
    return 0;
}

int check_format(const dnatok_format* f, bool host) {
    if (!f) return fail(DNATOK_ERR_INVALID, "format is NULL");
    if (f->id_bits != 32 && f->id_bits != 64) return fail(DNATOK_ERR_INVALID, "id_bits must be 32 or 64");
    if (f->mask_bits != 0 && f->mask_bits != 8 && f->mask_bits != 32 && f->mask_bits != 64)
        return fail(DNATOK_ERR_INVALID, "mask_bits must be 0, 8, 32 or 64");
    if (f->max_tokens < 0) return fail(DNATOK_ERR_INVALID, "max_tokens < 0");
    if (f->out_stride < (host ? -1 : 0)) return fail(DNATOK_ERR_INVALID, "out_stride < 0");
    return 0;
}

int n_special(const dnatok_handle* h, const dnatok_format* f) {
    return f->add_special ? (h->sp.cls_id >= 0) + (h->sp.sep_id >= 0) : 0;
}

// stride: the padded width in effect (0 = ragged / not yet known).
int resolve(const dnatok_handle* h, const dnatok_format* f, int64_t stride, RowFormat* r) {
    const int ns = n_special(h, f);
    r->out_stride = stride;
    r->cls_id = f->add_special ? h->sp.cls_id : -1;
    r->sep_id = f->add_special ? h->sp.sep_id : -1;
    r->pad_id = h->sp.pad_id;
    r->pad_left = f->pad_left ? 1 : 0;
    r->mask_bits = f->mask_bits;
    int64_t cap = INT64_MAX;
    r->clip_is_error = 0;
    r->store_status = 0;
    if (f->max_tokens > 0) {
        if (f->max_tokens < ns) return fail(DNATOK_ERR_INVALID, "max_tokens smaller than the special tokens");
        cap = f->max_tokens - ns;
    }
    if (stride > 0) {
        if (stride < ns) return fail(DNATOK_ERR_INVALID, "out_stride smaller than the special tokens");
        if (stride - ns < cap) { cap = stride - ns; r->clip_is_error = 1; }
    }
    r->cap_content = cap;
    return 0;
}

struct BpeScratch {
    uint16_t* tokens;       // [total_bytes] merged tokens at the input offsets
    int32_t* counts;        // [n_rows] content tokens per row
    int32_t* class_count;   // [16]
    int32_t* work;          // [16]
    unsigned long long* long_cursor;   // bytes of long_area handed out
    int32_t* class_list;    // [BPE_N_CLASSES * n_rows]
    uint8_t* long_area;     // ranks and masks of the words of the long class
    size_t long_bytes;
    size_t bytes;
};

// The long class (words beyond the lanes kernel's capacity) needs extra working memory; it is left
// out when no row of the batch can be that long (by the total size or by the caller's hint).
BpeScratch bpe_scratch_layout(const dnatok_handle* h, void* base, int64_t n_rows, int64_t total_bytes) {
    BpeScratch s;
    size_t o = 0;
    uint8_t* b = (uint8_t*)base;
    s.tokens = (uint16_t*)(b + o);      o += align_up((size_t)total_bytes * 2 + 16, 256);
    s.counts = (int32_t*)(b + o);       o += align_up((size_t)n_rows * 4 + 4, 256);
    s.class_count = (int32_t*)(b + o);  o += 64;
    s.work = (int32_t*)(b + o);         o += 64;
    s.long_cursor = (unsigned long long*)(b + o);   o += 64;
    o = align_up(o, 256);
    s.class_list = (int32_t*)(b + o);   o += align_up((size_t)n_rows * 4 * BPE_N_CLASSES + 4, 256);
    int64_t longest = total_bytes;
    if (h->hint_max_row > 0 && h->hint_max_row < longest) longest = h->hint_max_row;
    s.long_area = (uint8_t*)(b + o);
    s.long_bytes = 0;
    if (longest > bpe_class_capacity(BPE_LONG_CLASS - 1)) {
        const int64_t words = total_bytes / bpe_class_capacity(BPE_LONG_CLASS - 1) + 1;
        s.long_bytes = align_up((size_t)(2 * total_bytes + total_bytes / 2 + 64 * words), 256);
    }
    o += s.long_bytes;
    s.bytes = o;
    return s;
}

// Resident blocks per SM of every merge kernel on a device; filling it also sets the kernels'
// shared-memory attribute, so a later launch does nothing but launch.
struct BpeLaunchInfo { int lanes[BPE_LONG_CLASS]; int mixed; int st_room[BPE_LONG_CLASS]; };   // resident blocks per SM of every merge kernel; st_room: bytes a shared-memory table may take beside the teams of each width (0: kernel not usable)

template <int W>
int bpe_setup_st(int* room) {
    cudaFuncAttributes fa;
    CUDA_TRY(cudaFuncGetAttributes(&fa, bpe_lanes_st_kernel<W>));
    int dev = 0, most = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    CUDA_TRY(cudaDeviceGetAttribute(&most, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    const int64_t dyn = (int64_t)most - (int64_t)fa.sharedSizeBytes;
    *room = 0;
    if (dyn <= (int64_t)bpe_st_team_area(W)) return 0;
    CUDA_TRY(cudaFuncSetAttribute(bpe_lanes_st_kernel<W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn));
    *room = (int)(dyn - (int64_t)bpe_st_team_area(W));
    return 0;
}

template <int W>
int bpe_setup_lanes(int* bps) {
    constexpr int BW = bpe_block_warps(W);
    const size_t smem = (size_t)(BW / W) * bpe_team_bytes(W);
    CUDA_TRY(cudaFuncSetAttribute(bpe_lanes_kernel<W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(bps, bpe_lanes_kernel<W>, BW * 32, smem));
    if (*bps < 1) *bps = 1;
    return 0;
}

int bpe_launch_info(int dev, const BpeLaunchInfo** out) {
    static std::mutex mu;
    static std::map<int, BpeLaunchInfo> info;
    std::lock_guard<std::mutex> lock(mu);
    auto it = info.find(dev);
    if (it == info.end()) {
        BpeLaunchInfo li{};
        int rc;
        if ((rc = bpe_setup_lanes<1>(&li.lanes[0])) || (rc = bpe_setup_lanes<2>(&li.lanes[1])) ||
            (rc = bpe_setup_lanes<4>(&li.lanes[2])) || (rc = bpe_setup_lanes<8>(&li.lanes[3])) ||
            (rc = bpe_setup_lanes<16>(&li.lanes[4])) || (rc = bpe_setup_lanes<32>(&li.lanes[5])))
            return rc;
        if ((rc = bpe_setup_st<1>(&li.st_room[0])) || (rc = bpe_setup_st<2>(&li.st_room[1])) ||
            (rc = bpe_setup_st<4>(&li.st_room[2])) || (rc = bpe_setup_st<8>(&li.st_room[3])) ||
            (rc = bpe_setup_st<16>(&li.st_room[4])) || (rc = bpe_setup_st<32>(&li.st_room[5])))
            return rc;
        CUDA_TRY(cudaFuncSetAttribute(bpe_mixed_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bpe_mixed_bytes()));
        CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&li.mixed, bpe_mixed_kernel, BPE_MIXED_WARPS * 32, bpe_mixed_bytes()));
        if (li.mixed < 1) li.mixed = 1;
        cudaFuncAttributes fa;
        CUDA_TRY(cudaFuncGetAttributes(&fa, bpe_long_kernel));      // loads the kernel's code now, not at its first launch
        CUDA_TRY(cudaFuncGetAttributes(&fa, bpe_classify_kernel));
        // ... and the kernels of the output stage, for both id widths
        CUDA_TRY(cudaFuncGetAttributes(&fa, span_lengths_kernel));
        CUDA_TRY(cudaFuncGetAttributes(&fa, scan_lengths_kernel));
        CUDA_TRY(cudaFuncGetAttributes(&fa, emit_padded_kernel<uint16_t, int64_t, false, EMIT_SPAN>));
        CUDA_TRY(cudaFuncGetAttributes(&fa, emit_padded_kernel<uint16_t, int32_t, false, EMIT_SPAN>));
        CUDA_TRY(cudaFuncGetAttributes(&fa, emit_ragged_kernel<uint16_t, int64_t, false>));
        CUDA_TRY(cudaFuncGetAttributes(&fa, emit_ragged_kernel<uint16_t, int32_t, false>));
        it = info.emplace(dev, li).first;
    }
    *out = &it->second;
    return 0;
}

// Class CLS's rows through teams of W warps (W >= 1 << CLS).
template <int CLS, int W>
int launch_bpe_lanes(const DeviceTables& d, const BpeLaunchInfo& li, const BpeDeviceTable& t, const uint8_t* bytes,
                     const int64_t* offsets, int64_t n_rows, const BpeScratch& s, int32_t* status, const BpeLengths& lo,
                     bool direct, cudaStream_t st) {
    constexpr int WI = W == 1 ? 0 : W == 2 ? 1 : W == 4 ? 2 : W == 8 ? 3 : W == 16 ? 4 : 5;
    if (t.compact && g_bpe_smem_table.load() && t.compact_bytes <= (uint32_t)li.st_room[WI]) {
        // the whole merge table fits into shared memory beside the teams: one block of 32 warps per SM
        constexpr int ST_TEAMS = BPE_ST_WARPS / W;
        int64_t grid = d.sm_count;                          // every SM takes part, however few the words (the kernel
        if (grid > n_rows) grid = n_rows;                    // lets only as many of a block's teams work as are needed)
        if (grid < 1) grid = 1;
        // Rows that are not binned and fit the grid's teams in one go need no work counter: every team takes the word
        // its position names.  Then nothing is zeroed before the launch, the launch before this one in the stream is
        // a kernel as a rule, and programmatic stream serialisation lets this grid's blocks be placed while it drains.
        const bool one_wave = direct && n_rows <= grid * ST_TEAMS;
        if (direct && !one_wave) CUDA_TRY(cudaMemsetAsync(s.work + CLS, 0, 4, st));
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)grid);
        cfg.blockDim = dim3(BPE_ST_WARPS * 32);
        cfg.dynamicSmemBytes = bpe_st_team_area(W) + t.compact_bytes;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = g_bpe_overlap_launch.load() ? 1 : 0;
        const int32_t* list = direct ? nullptr : s.class_list + (int64_t)CLS * n_rows;
        const int32_t* list_count = s.class_count + CLS;
        int32_t* work = one_wave ? nullptr : s.work + CLS;
        cudaLaunchKernelEx(&cfg, bpe_lanes_st_kernel<W>, bytes, offsets, list, list_count, work, t, s.tokens, s.counts, status, lo,
                           (int32_t)n_rows, (int32_t)bpe_class_capacity(CLS));
        LAUNCH_CHECK("bpe_lanes_st_kernel");
        return 0;
    }
    constexpr int BW = bpe_block_warps(W);
    constexpr int TEAMS = BW / W;                              // words in flight per block
    const size_t smem = (size_t)TEAMS * bpe_team_bytes(W);
    // Resident-size grid: every team pulls words from the class's shared counter.
    int64_t grid = (int64_t)d.sm_count * li.lanes[WI];
    const int64_t need = (n_rows + TEAMS - 1) / TEAMS;
    if (grid > need) grid = need;
    if (grid < 1) grid = 1;
    const bool one_wave = direct && grid == need;             // as above: no counter to claim from, none to zero
    if (direct && !one_wave) CUDA_TRY(cudaMemsetAsync(s.work + CLS, 0, 4, st));
    bpe_lanes_kernel<W><<<(unsigned)grid, BW * 32, smem, st>>>(
        bytes, offsets, direct ? nullptr : s.class_list + (int64_t)CLS * n_rows, s.class_count + CLS,
        one_wave ? nullptr : s.work + CLS, t, s.tokens, s.counts, status, lo, (int32_t)n_rows, (int32_t)bpe_class_capacity(CLS));
    LAUNCH_CHECK("bpe_lanes_kernel");
    return 0;
}

// A small batch cannot fill the GPU with one warp per word: a word then gets a wider team, which shortens
// each of its rounds.  widen is the team width asked for (a power of two); a class never runs narrower
// than its own width.
template <int CLS>
int launch_bpe_class(const DeviceTables& d, const BpeLaunchInfo& li, const BpeDeviceTable& t, const uint8_t* bytes,
                     const int64_t* offsets, int64_t n_rows, const BpeScratch& s, int32_t* status, const BpeLengths& lo,
                     bool direct, int widen, cudaStream_t st) {
    constexpr int W = 1 << CLS;
#define BPE_WIDE(W2) \
    if (W < W2 && widen >= W2) return launch_bpe_lanes<CLS, (W < W2 ? W2 : W)>(d, li, t, bytes, offsets, n_rows, s, status, lo, direct, st);
    BPE_WIDE(32) BPE_WIDE(16) BPE_WIDE(8) BPE_WIDE(4) BPE_WIDE(2)
#undef BPE_WIDE
    return launch_bpe_lanes<CLS, W>(d, li, t, bytes, offsets, n_rows, s, status, lo, direct, st);
}

// Team width for a batch of n_rows words of at most max_row bytes.  Wider teams shorten a word's rounds but
// take more of the GPU per word, so the width is the largest power of two that (a) keeps all words of the
// batch resident at once on half of the GPU's warp slots (measured: beyond that a second wave costs more
// than the shorter rounds save) and (b) leaves every lane at least four positions.  A large batch stays at
// one warp per word.
int bpe_team_width(const DeviceTables& d, const BpeLaunchInfo& li, int64_t n_rows, int64_t max_row) {
    const int64_t forced = g_bpe_team_warps.load();
    if (forced > 0) return (int)(forced > 32 ? 32 : forced);
    const int64_t lim = g_bpe_block_team_rows.load();
    if (lim >= 0) return n_rows <= lim ? 8 : 1;
    const int64_t slots = (int64_t)d.sm_count * li.lanes[0] * 8 / 2;     // li.lanes[0]: blocks of 8 warps per SM
    const int64_t widest = g_bpe_team_max.load();
    int w = 1;
    while (2 * w <= widest && (int64_t)(2 * w) * n_rows <= slots && (int64_t)(2 * w) * 128 <= max_row) w *= 2;
    return w;
}

// lengths (may be NULL) receives every row's final token count for the format rf.
// ids (may be NULL): when given and the layout is padded, the merge kernels write the final ids and mask
// themselves and no output pass is needed afterwards.
int run_bpe_merge(dnatok_handle* h, const DeviceTables& d, const uint8_t* bytes, const int64_t* offsets,
                  int64_t n_rows, int64_t total_bytes, int32_t* status, void* scratch, size_t scratch_bytes,
                  const RowFormat& rf, int32_t* lengths, cudaStream_t st, void* ids = nullptr, void* mask = nullptr,
                  int id_bits = 0, bool status_unset = false) {
    if (!scratch) return fail(DNATOK_ERR_SCRATCH, "BPE needs a scratch buffer (dnatok_scratch_bytes)");
    if (reinterpret_cast<uintptr_t>(scratch) & 255) return fail(DNATOK_ERR_SCRATCH, "scratch must be 256-byte aligned");
    BpeScratch s = bpe_scratch_layout(h, scratch, n_rows, total_bytes);
    if (s.bytes > scratch_bytes) return fail(DNATOK_ERR_SCRATCH, "scratch too small: %zu < %zu", scratch_bytes, s.bytes);
    if (n_rows == 0) return 0;
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    const BpeLaunchInfo* li;
    if (int rc = bpe_launch_info(dev, &li)) return rc;
    // classes that can hold a row of this batch: bounded by the total size and by the caller's hint
    uint32_t class_mask = 0;
    int64_t max_row = total_bytes;                          // no row is longer than this
    {
        int64_t lo = 1, hi = total_bytes;
        if (h->hint_max_row > 0) { lo = h->hint_min_row > 1 ? h->hint_min_row : 1; if (h->hint_max_row < hi) hi = h->hint_max_row; }
        for (int c = 0; c < BPE_N_CLASSES; ++c) {
            const int64_t c_lo = c == 0 ? 1 : bpe_class_capacity(c - 1) + 1;
            const int64_t c_hi = c < BPE_LONG_CLASS ? bpe_class_capacity(c) : INT64_MAX;
            if (c_hi >= lo && c_lo <= hi) class_mask |= 1u << c;
        }
        max_row = hi;
    }
    if (((class_mask >> BPE_LONG_CLASS) & 1u) && !s.long_bytes) class_mask &= ~(1u << BPE_LONG_CLASS);
    const BpeLengths lo{lengths, rf.cap_content, (rf.cls_id >= 0 ? 1 : 0) + (rf.sep_id >= 0 ? 1 : 0), rf.clip_is_error,
                        ids, rf.mask_bits ? mask : nullptr, rf.out_stride, rf.cls_id, rf.sep_id, rf.pad_id, rf.pad_left,
                        id_bits, rf.mask_bits, status_unset ? 1 : 0};
    // One class only, by the caller's bounds on the row lengths: the rows need no binning, the class's kernel
    // takes them as they come (and flags a row the bounds misstated).
    const bool direct = h->hint_max_row > 0 && (class_mask & (class_mask - 1)) == 0 && !((class_mask >> BPE_LONG_CLASS) & 1u);
    // class_count, work and long_cursor are adjacent; rows that are not binned need at most their class's work counter,
    // which launch_bpe_lanes zeroes when it uses it
    if (!direct) CUDA_TRY(cudaMemsetAsync(s.class_count, 0, 192, st));
    if (!direct) {
        bpe_classify_kernel<<<(unsigned)((n_rows + 255) / 256), 256, 0, st>>>(offsets, n_rows, s.class_count,
                                                                           s.class_list, s.counts, status, class_mask, lo);
        LAUNCH_CHECK("bpe_classify_kernel");
    }
    BpeDeviceTable t{d.disp, reinterpret_cast<const uint2*>(d.slots), d.merge_out, reinterpret_cast<const uint2*>(d.hot),
                     d.byte_tok, h->bpe.batch_safe ? 0 : 1, h->bpe.hot_ranks, h->bpe.bytes_hot ? 1u : 0u, h->bpe.n_tokens,
                     reinterpret_cast<const uint4*>(d.bpe_compact), (uint32_t)h->bpe.compact.size(), h->bpe.compact_slot,
                     h->bpe.compact_info, h->bpe.compact_last};
    // Classes outside the mask are not launched; a row that falls into one is flagged by the classifier.
    // Longest class first: its few, slow words start while nothing else competes for the SMs.
    if ((class_mask >> BPE_LONG_CLASS) & 1u) {
        int64_t grid = total_bytes / bpe_class_capacity(BPE_LONG_CLASS - 1);     // no more words than this can be that long
        if (grid > n_rows) grid = n_rows;
        if (grid > d.sm_count) grid = d.sm_count;
        if (grid < 1) grid = 1;
        bpe_long_kernel<<<(unsigned)grid, BPE_LONG_WARPS * 32, 0, st>>>(
            bytes, offsets, s.class_list + (int64_t)BPE_LONG_CLASS * n_rows, s.class_count + BPE_LONG_CLASS,
            s.work + BPE_LONG_CLASS, t, s.tokens, s.counts, status, s.long_area, s.long_cursor, lo);
        LAUNCH_CHECK("bpe_long_kernel");
    }
    int rc;
    const int widen = bpe_team_width(d, *li, n_rows, max_row);
    if (!direct && g_bpe_mixed.load()) {
        // the classes below the widest in one launch, every class at the width of its own or the batch's, whichever is wider
        BpeMixedLevels lv{};
        int level_of_widen = 0;
        while ((2 << level_of_widen) <= widen && level_of_widen + 1 < BPE_MIXED_LEVELS) ++level_of_widen;
        uint32_t any = 0;
        for (int c = 0; c < BPE_MIXED_LEVELS; ++c)
            if ((class_mask >> c) & 1u) { lv.classes[c > level_of_widen ? c : level_of_widen] |= 1u << c; any = 1; }
        if ((class_mask >> 5) & 1u)
            if ((rc = launch_bpe_class<5>(d, *li, t, bytes, offsets, n_rows, s, status, lo, false, widen, st))) return rc;
        if (any) {
            int64_t grid = (int64_t)d.sm_count * li->mixed;
            if (grid > n_rows) grid = n_rows;
            bpe_mixed_kernel<<<(unsigned)grid, BPE_MIXED_WARPS * 32, bpe_mixed_bytes(), st>>>(
                bytes, offsets, s.class_list, n_rows, s.class_count, s.work, t, s.tokens, s.counts, status, lo, lv);
            LAUNCH_CHECK("bpe_mixed_kernel");
        }
        return 0;
    }
#define BPE_CLASS(CLS)                                                                                              \
    if (((class_mask >> CLS) & 1u) && (rc = launch_bpe_class<CLS>(d, *li, t, bytes, offsets, n_rows, s, status, lo, direct, widen, st))) \
        return rc;
    BPE_CLASS(5) BPE_CLASS(4) BPE_CLASS(3) BPE_CLASS(2) BPE_CLASS(1) BPE_CLASS(0)
#undef BPE_CLASS
    return 0;
}

template <typename SrcT, bool LUT>
int launch_emit(const DeviceTables& d, const SrcT* src, const int64_t* offsets, const int32_t* counts,
                int64_t n_rows, int64_t total_bytes, const RowFormat& rf, int id_bits, void* ids, void* mask,
                int32_t* lengths, const int64_t* out_offsets, int32_t* status, cudaStream_t st) {
    if (n_rows == 0) return 0;
    if (rf.out_stride > 0) {
        const uint8_t* sb = reinterpret_cast<const uint8_t*>(src);
        const uint8_t* se = sb + (size_t)total_bytes * sizeof(SrcT);
        // 32-bit ids on rows of several thousand columns: wider spans, so a trip stores 4 KiB as it does for 64-bit ids
        const bool wide = id_bits == 32 && sizeof(SrcT) == 1 && rf.out_stride >= 4 * EMIT_SPAN_WIDE;
        const int64_t span_cols = wide ? EMIT_SPAN_WIDE : EMIT_SPAN;
        const int64_t spr = (rf.out_stride + span_cols - 1) / span_cols;
        const int64_t n_spans = spr * n_rows;
        const int64_t blocks = (n_spans + EMIT_WARPS - 1) / EMIT_WARPS;
        const unsigned grid = (unsigned)(blocks < (int64_t)d.sm_count * 32 ? blocks : (int64_t)d.sm_count * 32);
        // programmatic stream serialisation, as for the k-mer row kernel
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(EMIT_THREADS);
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = g_emit_overlap_launch.load() ? 1 : 0;
        const int32_t* lut = d.lut256;
        if (id_bits == 64)
            cudaLaunchKernelEx(&cfg, emit_padded_kernel<SrcT, int64_t, LUT, EMIT_SPAN>, src, sb, se, offsets, counts, n_rows, lut, rf,
                               (int64_t*)ids, mask, lengths, status, spr, n_spans);
        else if (wide)
            cudaLaunchKernelEx(&cfg, emit_padded_kernel<uint8_t, int32_t, LUT, EMIT_SPAN_WIDE>, reinterpret_cast<const uint8_t*>(src),
                               sb, se, offsets, counts, n_rows, lut, rf, (int32_t*)ids, mask, lengths, status, spr, n_spans);
        else
            cudaLaunchKernelEx(&cfg, emit_padded_kernel<SrcT, int32_t, LUT, EMIT_SPAN>, src, sb, se, offsets, counts, n_rows, lut, rf,
                               (int32_t*)ids, mask, lengths, status, spr, n_spans);
        LAUNCH_CHECK("emit_padded_kernel");
    } else {
        const int64_t bound = total_bytes + 2 * n_rows;
        const int64_t n_tiles = (bound + EMIT_TILE - 1) / EMIT_TILE;
        if (n_tiles == 0) return 0;
        const unsigned grid = (unsigned)(n_tiles < (int64_t)d.sm_count * 64 ? n_tiles : (int64_t)d.sm_count * 64);
        if (id_bits == 64)
            emit_ragged_kernel<SrcT, int64_t, LUT><<<grid, EMIT_THREADS, 0, st>>>(src, offsets, out_offsets, n_rows, d.lut256, rf,
                                                                                  (int64_t*)ids, mask, n_tiles);
        else
            emit_ragged_kernel<SrcT, int32_t, LUT><<<grid, EMIT_THREADS, 0, st>>>(src, offsets, out_offsets, n_rows, d.lut256, rf,
                                                                                  (int32_t*)ids, mask, n_tiles);
        LAUNCH_CHECK("emit_ragged_kernel");
    }
    return 0;
}

// The one-token-per-character path: the emit kernel, then the start ids where the handle has them.
int launch_char(const dnatok_handle* h, const DeviceTables& d, const uint8_t* bytes, const int64_t* offsets, int64_t n_rows,
                int64_t total_bytes, const RowFormat& rf, int id_bits, void* ids, void* mask, int32_t* lengths,
                const int64_t* out_offsets, int32_t* status, cudaStream_t st) {
    int rc = h->lut_identity
        ? launch_emit<uint8_t, false>(d, bytes, offsets, nullptr, n_rows, total_bytes, rf, id_bits, ids, mask, lengths, out_offsets, status, st)
        : launch_emit<uint8_t, true>(d, bytes, offsets, nullptr, n_rows, total_bytes, rf, id_bits, ids, mask, lengths, out_offsets, status, st);
    if (rc || h->start_lut.empty() || n_rows == 0) return rc;
    const unsigned grid = (unsigned)((n_rows + 255) / 256);
    if (id_bits == 64) start_fix_kernel<int64_t><<<grid, 256, 0, st>>>(bytes, offsets, n_rows, d.start_lut, rf, (int64_t*)ids, out_offsets);
    else start_fix_kernel<int32_t><<<grid, 256, 0, st>>>(bytes, offsets, n_rows, d.start_lut, rf, (int32_t*)ids, out_offsets);
    LAUNCH_CHECK("start_fix_kernel");
    return 0;
}

template <typename IdT, int K>
void launch_kmer_warp_k(const DeviceTables& d, int32_t affine_base, const uint8_t* bytes, const int64_t* offsets,
                        int64_t n_rows, int64_t total_bytes, const RowFormat& rf, void* ids, void* mask,
                        const int32_t* lengths_in, int32_t* lengths_out, const int64_t* out_offsets, int32_t* status,
                        cudaStream_t st) {
    const unsigned grid = (unsigned)((n_rows + KW_ROW_WARPS - 1) / KW_ROW_WARPS);
    // the mask rides along with the ids when it has their element type and their 16-byte phase (the pair stores of
    // both use one alignment test)
    const bool fuse = mask && rf.mask_bits == (int)sizeof(IdT) * 8 &&
                      ((reinterpret_cast<uintptr_t>(mask) ^ reinterpret_cast<uintptr_t>(ids)) & 15) == 0;
    const bool affine = affine_base >= 0;
    // Programmatic stream serialisation: the kernel's blocks may be placed on the SMs while the launch before it
    // in the stream drains; they wait (griddepcontrol.wait) until that launch is complete before they touch memory.
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(KW_ROW_WARPS * 32);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_kmer_overlap_launch.load() ? 1 : 0;
    const int32_t* kmer_ids = d.kmer_ids;
    const int32_t* singles = d.lut256;
    IdT* ids_t = (IdT*)ids;
#define KLAUNCH(A, F) cudaLaunchKernelEx(&cfg, kmer_warp_rows_kernel<IdT, K, A, F>, bytes, offsets, n_rows, total_bytes, kmer_ids,    \
                                         affine_base, singles, rf, ids_t, mask, lengths_in, lengths_out, out_offsets, status)
    if (affine && fuse) KLAUNCH(true, true);
    else if (affine) KLAUNCH(true, false);
    else if (fuse) KLAUNCH(false, true);
    else KLAUNCH(false, false);
#undef KLAUNCH
}

// Scratch of the segmented k-mer kernel: one flag per (segment, row).  The number of segments follows
// the average row (or the caller's row-length hint, when that is larger); longer rows finish inside
// the last segment.
struct KmerScratch { unsigned long long* tickets; uint32_t* flags; int n_seg; size_t bytes; };

KmerScratch kmer_scratch_layout(const dnatok_handle* h, void* base, int64_t n_rows, int64_t total_bytes) {
    KmerScratch s{};
    if (n_rows <= 0) { s.n_seg = 1; s.bytes = 256; return s; }
    const int64_t k = h->k;
    int64_t row_bytes = (total_bytes + n_rows - 1) / n_rows;
    const int64_t segw = KSEG_WINDOWS;
    const int64_t total_seg = total_bytes / (k * segw) + 1;                    // segments the whole batch holds
    if (h->hint_max_row > row_bytes) row_bytes = h->hint_max_row;
    int64_t n_seg = ((row_bytes + k - 1) / k + segw - 1) / segw;
    // a hint far above the average must not blow the ticket space up
    const int64_t most = 4 * total_seg / n_rows + 1;
    if (n_seg > most) n_seg = most;
    if (n_seg < 1) n_seg = 1;
    if (n_seg > (1 << 20)) n_seg = 1 << 20;
    s.n_seg = (int)n_seg;
    s.tickets = (unsigned long long*)base;                       // the ticket counter has the first 256 bytes to itself
    s.flags = (uint32_t*)((uint8_t*)base + 256);
    s.bytes = 256 + (size_t)n_seg * (size_t)n_rows * 4;
    return s;
}

template <typename IdT, int K>
void launch_kmer_seg_k(const DeviceTables& d, int32_t affine_base, const uint8_t* bytes, const int64_t* offsets,
                       int64_t n_rows, int64_t total_bytes, const RowFormat& rf, void* ids, void* mask,
                       const int32_t* lengths_in, int32_t* lengths_out, const int64_t* out_offsets, int32_t* status,
                       const KmerScratch& ks, cudaStream_t st) {
    const int64_t tickets = n_rows * ks.n_seg;
    const bool fuse = mask && rf.mask_bits == (int)sizeof(IdT) * 8;
    const bool affine = affine_base >= 0;
    // as many blocks as the GPU keeps resident (the warps draw tickets from a counter, so a smaller or a
    // larger grid would also finish; this size keeps every SM busy without idle blocks queued behind)
    int bps = KSEG_BLOCKS_PER_SM;
    {
        int q = 0;
        cudaError_t e = affine && fuse ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&q, kmer_seg_rows_kernel<IdT, K, true, true>, KW_WARPS * 32, 0)
                        : affine       ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&q, kmer_seg_rows_kernel<IdT, K, true, false>, KW_WARPS * 32, 0)
                        : fuse         ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&q, kmer_seg_rows_kernel<IdT, K, false, true>, KW_WARPS * 32, 0)
                                       : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&q, kmer_seg_rows_kernel<IdT, K, false, false>, KW_WARPS * 32, 0);
        if (e == cudaSuccess && q >= 1) bps = q;
    }
    const int64_t want = (tickets + KW_WARPS - 1) / KW_WARPS, resident = (int64_t)d.sm_count * bps;
    const unsigned grid = (unsigned)(want < resident ? want : resident);
    const int poll_limit = (int)g_kmer_poll_limit.load();
    const long long withhold = (long long)g_kmer_test_withhold.load();
#define KLAUNCH(A, F) kmer_seg_rows_kernel<IdT, K, A, F><<<grid, KW_WARPS * 32, 0, st>>>(                           \
        bytes, offsets, n_rows, total_bytes, d.kmer_ids, affine_base, d.lut256, rf, (IdT*)ids, mask, lengths_in,    \
        lengths_out, out_offsets, status, ks.n_seg, ks.flags, ks.tickets, poll_limit, withhold)
    if (affine && fuse) KLAUNCH(true, true);
    else if (affine) KLAUNCH(true, false);
    else if (fuse) KLAUNCH(false, true);
    else KLAUNCH(false, false);
#undef KLAUNCH
}

template <typename IdT>
void launch_kmer_seg(int k, const DeviceTables& d, int32_t affine_base, const uint8_t* bytes, const int64_t* offsets,
                     int64_t n_rows, int64_t total_bytes, const RowFormat& rf, void* ids, void* mask,
                     const int32_t* lengths_in, int32_t* lengths_out, const int64_t* out_offsets, int32_t* status,
                     const KmerScratch& ks, cudaStream_t st) {
#define KCASE(KK) case KK: launch_kmer_seg_k<IdT, KK>(d, affine_base, bytes, offsets, n_rows, total_bytes, rf, ids, mask, \
                                                      lengths_in, lengths_out, out_offsets, status, ks, st); break;
    switch (k) { KCASE(1) KCASE(2) KCASE(3) KCASE(4) KCASE(5) KCASE(6) KCASE(7) KCASE(8) }
#undef KCASE
}

template <typename IdT>
void launch_kmer_warp(int k, const DeviceTables& d, int32_t affine_base, const uint8_t* bytes, const int64_t* offsets,
                      int64_t n_rows, int64_t total_bytes, const RowFormat& rf, void* ids, void* mask,
                      const int32_t* lengths_in, int32_t* lengths_out, const int64_t* out_offsets, int32_t* status,
                      cudaStream_t st) {
#define KCASE(KK) case KK: launch_kmer_warp_k<IdT, KK>(d, affine_base, bytes, offsets, n_rows, total_bytes, rf, ids, mask, \
                                                       lengths_in, lengths_out, out_offsets, status, st); break;
    switch (k) { KCASE(1) KCASE(2) KCASE(3) KCASE(4) KCASE(5) KCASE(6) KCASE(7) KCASE(8) }
#undef KCASE
}

// With a scratch buffer, batches of few or very long rows are encoded (and counted) as row segments.
// Otherwise rows of ordinary length go one per warp and batches of very long rows one per block.
constexpr int64_t KMER_WARP_MAX_AVG_LEN = 32768;

int launch_span_lengths(const int64_t* offsets, const int32_t* counts, int64_t n_rows, const RowFormat& rf,
                        int32_t* lengths, int32_t* status, cudaStream_t st);

template <bool COUNT_ONLY>
int launch_kmer(dnatok_handle* h, const DeviceTables& d, const uint8_t* bytes, const int64_t* offsets,
                int64_t n_rows, int64_t total_bytes, const RowFormat& rf, int id_bits, void* ids, void* mask,
                const int32_t* lengths_in, int32_t* lengths_out, const int64_t* out_offsets,
                int32_t* status, void* scratch, size_t scratch_bytes, cudaStream_t st, bool status_unset = false) {
    if (n_rows == 0) return 0;
    const int k = h->k;
    // status_unset: the caller left the status words as they were.  The row-per-warp encoder writes every row's word
    // itself (so nothing sits between two such launches in a stream); every other kernel ORs bits into zeroed words.
    bool need_zero = status_unset && status;
    auto zero_now = [&]() -> int {
        if (need_zero) CUDA_TRY(cudaMemsetAsync(status, 0, (size_t)n_rows * 4, st));
        need_zero = false;
        return 0;
    };
    if (h->kmer_table) {
        if (int rc = zero_now()) return rc;
        const KmerTable t{d.table5, d.exp_off, d.exp_ids, d.lut256, k, h->tail_singles};
        const unsigned grid = (unsigned)((n_rows + KT_WARPS - 1) / KT_WARPS);
        if (id_bits == 64)
            kmer_table_kernel<int64_t, COUNT_ONLY><<<grid, KT_WARPS * 32, 0, st>>>(bytes, offsets, n_rows, t, rf, (int64_t*)ids, mask,
                                                                                  lengths_in, lengths_out, out_offsets, status);
        else
            kmer_table_kernel<int32_t, COUNT_ONLY><<<grid, KT_WARPS * 32, 0, st>>>(bytes, offsets, n_rows, t, rf, (int32_t*)ids, mask,
                                                                                  lengths_in, lengths_out, out_offsets, status);
        LAUNCH_CHECK("kmer_table_kernel");
        return 0;
    }
    // The segment encoder spends about half as many instructions again per row (look-back, a second
    // pass over segments that hold an N), and its fixed deal of segments to warps cannot follow SMs
    // that run at different speeds the way block scheduling does: it is the choice where one warp
    // per row would leave the GPU short of work (few rows) or rows are very long; large batches of
    // ordinary rows run faster one row per warp.
    const bool few_rows = n_rows < (int64_t)d.sm_count * 8;
    const bool long_rows = total_bytes / n_rows > KMER_WARP_MAX_AVG_LEN;
    // the flags carry 30-bit token counts: a row that might hold 2^30 tokens stays with the other kernels
    const int64_t longest = h->hint_max_row > 0 && h->hint_max_row < total_bytes ? h->hint_max_row : total_bytes;
    // a row that gave up is reported through the status array only: without one the segment encoder is not used
    if (!COUNT_ONLY && status && scratch && !(reinterpret_cast<uintptr_t>(scratch) & 255) && longest < (1ll << 30) &&
        (few_rows || long_rows || g_kmer_force_segments)) {
        const KmerScratch ks = kmer_scratch_layout(h, scratch, n_rows, total_bytes);
        if (ks.bytes <= scratch_bytes && (ks.n_seg > 1 || g_kmer_force_segments)) {
            if (int rc = zero_now()) return rc;
            CUDA_TRY(cudaMemsetAsync(scratch, 0, ks.bytes, st));
            if (id_bits == 64) launch_kmer_seg<int64_t>(k, d, h->kmer_affine_base, bytes, offsets, n_rows, total_bytes, rf, ids, mask,
                                                        lengths_in, lengths_out, out_offsets, status, ks, st);
            else launch_kmer_seg<int32_t>(k, d, h->kmer_affine_base, bytes, offsets, n_rows, total_bytes, rf, ids, mask,
                                          lengths_in, lengths_out, out_offsets, status, ks, st);
            LAUNCH_CHECK("kmer_seg_rows_kernel");
            return 0;
        }
    }
    if (COUNT_ONLY) if (int rc = zero_now()) return rc;
    if (COUNT_ONLY && scratch && !(reinterpret_cast<uintptr_t>(scratch) & 255) && (few_rows || long_rows)) {
        const KmerScratch ks = kmer_scratch_layout(h, scratch, n_rows, total_bytes);
        if (ks.bytes <= scratch_bytes && ks.n_seg > 1) {
            int32_t* counts = reinterpret_cast<int32_t*>(ks.flags);
            CUDA_TRY(cudaMemsetAsync(counts, 0, (size_t)n_rows * 4, st));
            const int64_t want = (n_rows * ks.n_seg + KW_WARPS - 1) / KW_WARPS, most = (int64_t)d.sm_count * 8;
            const unsigned grid = (unsigned)(want < most ? want : most);
#define KCASE(KK) case KK: kmer_seg_count_kernel<KK><<<grid, KW_WARPS * 32, 0, st>>>(bytes, offsets, n_rows, total_bytes, ks.n_seg, \
                                                                                 KSEG_WINDOWS, counts); break;
            switch (k) { KCASE(1) KCASE(2) KCASE(3) KCASE(4) KCASE(5) KCASE(6) KCASE(7) KCASE(8) }
#undef KCASE
            LAUNCH_CHECK("kmer_seg_count_kernel");
            return launch_span_lengths(offsets, counts, n_rows, rf, lengths_out, status, st);
        }
    }
    if (COUNT_ONLY && total_bytes / n_rows <= KMER_WARP_MAX_AVG_LEN) {
        const unsigned grid = (unsigned)((n_rows + KW_WARPS - 1) / KW_WARPS);
#define KCASE(KK) case KK: kmer_warp_count_kernel<KK><<<grid, KW_WARPS * 32, 0, st>>>(bytes, offsets, n_rows, total_bytes, rf, \
                                                                                  lengths_out, status); break;
        switch (k) { KCASE(1) KCASE(2) KCASE(3) KCASE(4) KCASE(5) KCASE(6) KCASE(7) KCASE(8) }
#undef KCASE
        LAUNCH_CHECK("kmer_warp_count_kernel");
        return 0;
    }
    if (!COUNT_ONLY && total_bytes / n_rows <= KMER_WARP_MAX_AVG_LEN) {
        RowFormat rfw = rf;
        if (need_zero) { rfw.store_status = 1; need_zero = false; }
        if (id_bits == 64) launch_kmer_warp<int64_t>(k, d, h->kmer_affine_base, bytes, offsets, n_rows, total_bytes, rfw, ids, mask, lengths_in,
                                                     lengths_out, out_offsets, status, st);
        else launch_kmer_warp<int32_t>(k, d, h->kmer_affine_base, bytes, offsets, n_rows, total_bytes, rfw, ids, mask, lengths_in,
                                       lengths_out, out_offsets, status, st);
        LAUNCH_CHECK("kmer_warp_rows_kernel");
        return 0;
    }
    if (int rc = zero_now()) return rc;
    const size_t smem = (size_t)((KMER_TILE_W * k + 32 + 15) & ~15) + (size_t)KMER_TILE_W * k * 4;
    const unsigned grid = (unsigned)(n_rows < (int64_t)d.sm_count * 64 ? n_rows : (int64_t)d.sm_count * 64);
    if (id_bits == 64)
        kmer_rows_kernel<int64_t, COUNT_ONLY><<<grid, KMER_THREADS, smem, st>>>(bytes, offsets, n_rows, k, d.kmer_ids, d.lut256, rf,
                                                                                (int64_t*)ids, mask, lengths_in, lengths_out, out_offsets, status);
    else
        kmer_rows_kernel<int32_t, COUNT_ONLY><<<grid, KMER_THREADS, smem, st>>>(bytes, offsets, n_rows, k, d.kmer_ids, d.lut256, rf,
                                                                                (int32_t*)ids, mask, lengths_in, lengths_out, out_offsets, status);
    LAUNCH_CHECK("kmer_rows_kernel");
    return 0;
}

int launch_span_lengths(const int64_t* offsets, const int32_t* counts, int64_t n_rows, const RowFormat& rf,
                        int32_t* lengths, int32_t* status, cudaStream_t st) {
    if (n_rows == 0) return 0;
    span_lengths_kernel<<<(unsigned)((n_rows + 255) / 256), 256, 0, st>>>(offsets, counts, n_rows, rf, lengths, status);
    LAUNCH_CHECK("span_lengths_kernel");
    return 0;
}

// Attention mask of a padded batch written by host threads from the row lengths the GPU produced:
// ones on [shift, shift + T) of every row, zeros elsewhere.  The mask is a function of the lengths
// alone, so a large one is cheaper to make where it is wanted than to carry over the host link.
// The stores bypass the cache (the mask is written once and read by someone else later): an ordinary
// store first reads the line it is about to overwrite, which doubles the memory traffic of a buffer
// that the copies from the GPU are competing with.
#if defined(__x86_64__) || defined(_M_X64)
#include <emmintrin.h>
inline void put_once(int64_t* p, int64_t v) { _mm_stream_si64(reinterpret_cast<long long*>(p), v); }
inline void put_once(int32_t* p, int32_t v) { _mm_stream_si32(p, v); }
inline void put_once(uint8_t* p, uint8_t v) { *p = v; }
inline void put_once_done() { _mm_sfence(); }
#else
template <typename M> inline void put_once(M* p, M v) { *p = v; }
inline void put_once_done() {}
#endif

// Host workers that outlive a call: starting a thread and giving it the device's context costs far more than
// writing its share of a mask, so the threads are started once and handed jobs.  run(n, fn) calls fn(0) on the
// calling thread and fn(1) .. fn(n - 1) on workers, and returns when all are done.  One job at a time.
class HostPool {
public:
    static HostPool& get() {
        static HostPool* pool = new HostPool();      // never destroyed: the workers sleep until the process ends
        return *pool;
    }
    void run(int n, const std::function<void(int)>& fn) {
        if (n <= 1) { fn(0); return; }
        std::lock_guard<std::mutex> one_job(job_mu_);
        {
            std::unique_lock<std::mutex> lk(mu_);
            while ((int)threads_.size() < n - 1) {
                const int id = (int)threads_.size() + 1;
                threads_.emplace_back([this, id] { loop(id); });
            }
            fn_ = &fn; want_ = n; pending_ = n - 1; ++generation_;
        }
        cv_.notify_all();
        fn(0);
        std::unique_lock<std::mutex> lk(mu_);
        done_.wait(lk, [this] { return pending_ == 0; });
        fn_ = nullptr;
    }

private:
    void loop(int id) {
        uint64_t seen = 0;
        for (;;) {
            const std::function<void(int)>* fn;
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_.wait(lk, [&] { return generation_ != seen; });
                seen = generation_;
                if (id >= want_) continue;           // this job needs fewer workers
                fn = fn_;
            }
            (*fn)(id);
            {
                std::lock_guard<std::mutex> lk(mu_);
                if (--pending_ == 0) done_.notify_one();
            }
        }
    }
    std::mutex mu_, job_mu_;
    std::condition_variable cv_, done_;
    std::vector<std::thread> threads_;
    const std::function<void(int)>* fn_ = nullptr;
    int want_ = 0, pending_ = 0;
    uint64_t generation_ = 0;
};

template <typename M>
void fill_mask_rows(M* mask, const int32_t* lengths, int64_t r0, int64_t r1, int64_t stride, bool pad_left) {
    for (int64_t r = r0; r < r1; ++r) {
        M* row = mask + r * stride;
        int64_t T = lengths[r];
        if (T < 0) T = 0;
        if (T > stride) T = stride;
        const int64_t lo = pad_left ? stride - T : 0;
        for (int64_t j = 0; j < lo; ++j) put_once(row + j, (M)0);
        for (int64_t j = lo; j < lo + T; ++j) put_once(row + j, (M)1);
        for (int64_t j = lo + T; j < stride; ++j) put_once(row + j, (M)0);
    }
    put_once_done();
}

// Pinned landing place for row lengths and status words: a copy to the caller's arrays, which are ordinary memory
// as a rule, would block the calling thread until everything before it in the stream is done.
int pinned_rows(DeviceTables* d, int64_t n_rows) {
    const size_t need = (size_t)n_rows * 8 + 64;
    if (need <= d->h_rows_cap) return 0;
    if (d->h_rows) CUDA_TRY(cudaFreeHost(d->h_rows));
    d->h_rows = nullptr; d->h_rows_cap = 0;
    CUDA_TRY(cudaMallocHost((void**)&d->h_rows, need + 65536));
    d->h_rows_cap = need + 65536;
    return 0;
}

// The attention mask of a large padded batch, written by n_threads host workers once the row lengths
// have arrived, while the ids are still being copied back.
struct HostMask {
    int device = 0;
    void* mask = nullptr; int mask_bits = 0; const int32_t* lengths = nullptr; int64_t n_rows = 0, stride = 0;
    bool pad_left = false; cudaEvent_t ev_lengths = nullptr;
};

void host_mask_worker(const HostMask& hm, int t, int n_threads, int* err) {
    if (cudaSetDevice(hm.device) != cudaSuccess || cudaEventSynchronize(hm.ev_lengths) != cudaSuccess) { *err = 1; return; }
    const int64_t r0 = hm.n_rows * t / n_threads, r1 = hm.n_rows * (t + 1) / n_threads;
    if (hm.mask_bits == 64) fill_mask_rows<int64_t>((int64_t*)hm.mask, hm.lengths, r0, r1, hm.stride, hm.pad_left);
    else if (hm.mask_bits == 32) fill_mask_rows<int32_t>((int32_t*)hm.mask, hm.lengths, r0, r1, hm.stride, hm.pad_left);
    else fill_mask_rows<uint8_t>((uint8_t*)hm.mask, hm.lengths, r0, r1, hm.stride, hm.pad_left);
}

int host_mask_fill(const HostMask& hm, int n_threads) {
    if (n_threads > hm.n_rows) n_threads = (int)hm.n_rows;
    if (n_threads < 1) n_threads = 1;
    std::vector<int> errs((size_t)n_threads, 0);
    HostPool::get().run(n_threads, [&](int t) { host_mask_worker(hm, t, n_threads, &errs[(size_t)t]); });
    for (int e : errs) if (e) return fail(DNATOK_ERR_CUDA, "a host worker could not wait for the row lengths");
    return 0;
}

int check_batch(const dnatok_handle* h, const void* bytes, const void* offsets, int64_t n_rows, int64_t total) {
    if (!h) return fail(DNATOK_ERR_INVALID, "handle is NULL");
    if (n_rows < 0 || total < 0) return fail(DNATOK_ERR_INVALID, "negative size");
    if (n_rows > INT32_MAX) return fail(DNATOK_ERR_INVALID, "more than 2^31-1 rows");
    if (!offsets) return fail(DNATOK_ERR_INVALID, "offsets is NULL");
    if (total > 0 && !bytes) return fail(DNATOK_ERR_INVALID, "bytes is NULL");
    return 0;
}

}  // namespace

extern "C" {

int dnatok_version(void) { return DNATOK_ABI_VERSION; }
const char* dnatok_last_error(void) { return g_err.c_str(); }
int64_t dnatok_launch_count(void) { return g_launches.load(); }
void dnatok_host_copy_bytes(int64_t* h2d, int64_t* d2h) {
    if (h2d) *h2d = g_last_h2d;
    if (d2h) *d2h = g_last_d2h;
}

int dnatok_set_option(const char* name, int64_t value) {
    if (!name) return fail(DNATOK_ERR_INVALID, "bad option");
    if (!strcmp(name, "bpe_block_team_rows")) { g_bpe_block_team_rows = value; return DNATOK_OK; }
    if (!strcmp(name, "bpe_team_warps")) { g_bpe_team_warps = value; return DNATOK_OK; }
    if (!strcmp(name, "bpe_team_max")) { g_bpe_team_max = value; return DNATOK_OK; }
    if (!strcmp(name, "kmer_overlap_launch")) { g_kmer_overlap_launch = value; return DNATOK_OK; }
    if (!strcmp(name, "emit_overlap_launch")) { g_emit_overlap_launch = value; return DNATOK_OK; }
    if (!strcmp(name, "host_mask_early")) { g_host_mask_early = value; return DNATOK_OK; }
    if (!strcmp(name, "bpe_overlap_launch")) { g_bpe_overlap_launch = value; return DNATOK_OK; }
    if (!strcmp(name, "bpe_smem_table")) { g_bpe_smem_table = value; return DNATOK_OK; }
    if (!strcmp(name, "bpe_fused_output")) { g_bpe_fused_output = value; return DNATOK_OK; }
    if (!strcmp(name, "bpe_mixed_launch")) { g_bpe_mixed = value; return DNATOK_OK; }
    if (!strcmp(name, "host_mask_min_bytes")) { g_host_mask_min_bytes = value < 0 ? 0 : value; return DNATOK_OK; }
    if (!strcmp(name, "host_mask_threads")) { g_host_mask_threads = value < -1 ? -1 : value; return DNATOK_OK; }
    if (!strcmp(name, "kmer_test_withhold_ticket")) { g_kmer_test_withhold = value < 0 ? -1 : value; return DNATOK_OK; }
    if (value < 0) return fail(DNATOK_ERR_INVALID, "bad option value");
    if (!strcmp(name, "host_chunk_bytes")) { g_host_chunk_bytes = value; return DNATOK_OK; }
    if (!strcmp(name, "kmer_force_segments")) { g_kmer_force_segments = value ? 1 : 0; return DNATOK_OK; }
    if (!strcmp(name, "kmer_poll_limit")) { g_kmer_poll_limit = value < 1 ? 1 : (value > (1 << 30) ? (1 << 30) : value); return DNATOK_OK; }
    if (!strcmp(name, "host_chunk_threshold")) { g_host_chunk_threshold = value; return DNATOK_OK; }
    return fail(DNATOK_ERR_INVALID, "unknown option %s", name);
}

static int check_specials(const dnatok_specials* sp) {
    if (!sp) return fail(DNATOK_ERR_INVALID, "specials is NULL");
    if (sp->pad_id < 0) return fail(DNATOK_ERR_INVALID, "pad_id < 0");
    return 0;
}

int dnatok_create_char(const int32_t lut[256], const dnatok_specials* sp, dnatok_handle** out) {
    if (!lut || !out) return fail(DNATOK_ERR_INVALID, "NULL argument");
    if (int rc = check_specials(sp)) return rc;
    auto* h = new (std::nothrow) dnatok_handle();
    if (!h) return fail(DNATOK_ERR_INVALID, "out of memory");
    h->kind = DNATOK_KIND_CHAR; h->sp = *sp;
    h->lut256.assign(lut, lut + 256);
    h->lut_identity = true;
    for (int i = 0; i < 256; ++i) h->lut_identity = h->lut_identity && lut[i] == i;
    *out = h;
    return DNATOK_OK;
}

int dnatok_create_kmer(int k, const int32_t* kmer_ids, const int32_t single_ids[256],
                       const dnatok_specials* sp, dnatok_handle** out) {
    if (!kmer_ids || !single_ids || !out) return fail(DNATOK_ERR_INVALID, "NULL argument");
    if (k < 1 || k > KMER_MAX_K) return fail(DNATOK_ERR_UNSUPPORTED, "k must be in 1..%d", KMER_MAX_K);
    if (int rc = check_specials(sp)) return rc;
    auto* h = new (std::nothrow) dnatok_handle();
    if (!h) return fail(DNATOK_ERR_INVALID, "out of memory");
    h->kind = DNATOK_KIND_KMER; h->sp = *sp; h->k = k;
    h->lut256.assign(single_ids, single_ids + 256);
    h->kmer_ids.assign(kmer_ids, kmer_ids + ((size_t)1 << (2 * k)));
    bool affine = kmer_ids[0] >= 0;
    for (size_t i = 0; i < h->kmer_ids.size() && affine; ++i) affine = kmer_ids[i] == kmer_ids[0] + (int32_t)i;
    h->kmer_affine_base = affine ? kmer_ids[0] : -1;
    *out = h;
    return DNATOK_OK;
}

int dnatok_create_kmer_table(int k, const int32_t* table5, const int32_t* run_offsets, int32_t n_runs, const int32_t* run_ids,
                             const int32_t single_ids[256], int tail_singles, const dnatok_specials* sp,
                             dnatok_handle** out) {
    if (!table5 || !single_ids || !out || n_runs < 0 || (n_runs && (!run_offsets || !run_ids)))
        return fail(DNATOK_ERR_INVALID, "NULL argument");
    if (k < 1 || k > KMER_MAX_K) return fail(DNATOK_ERR_UNSUPPORTED, "k must be in 1..%d", KMER_MAX_K);
    if (int rc = check_specials(sp)) return rc;
    size_t n5 = 1;
    for (int i = 0; i < k; ++i) n5 *= 5;
    for (size_t i = 0; i < n5; ++i)
        if (table5[i] < 0 && -(int64_t)table5[i] - 1 >= n_runs) return fail(DNATOK_ERR_INVALID, "window %zu names run %lld of %d", i, -(long long)table5[i] - 1, n_runs);
    for (int32_t e = 0; e < n_runs; ++e)
        if (run_offsets[e + 1] < run_offsets[e]) return fail(DNATOK_ERR_INVALID, "run offsets must not decrease");
    auto* h = new (std::nothrow) dnatok_handle();
    if (!h) return fail(DNATOK_ERR_INVALID, "out of memory");
    h->kind = DNATOK_KIND_KMER; h->sp = *sp; h->k = k;
    h->kmer_table = true;
    h->tail_singles = tail_singles ? 1 : 0;
    h->lut256.assign(single_ids, single_ids + 256);
    h->table5.assign(table5, table5 + n5);
    if (n_runs) {
        h->exp_off.assign(run_offsets, run_offsets + n_runs + 1);
        h->exp_ids.assign(run_ids, run_ids + run_offsets[n_runs]);
    }
    if (h->exp_off.empty()) h->exp_off.assign(1, 0);
    if (h->exp_ids.empty()) h->exp_ids.assign(1, 0);
    *out = h;
    return DNATOK_OK;
}

int dnatok_set_start_lut(dnatok_handle* h, const int32_t start_lut[256]) {
    if (!h || !start_lut) return fail(DNATOK_ERR_INVALID, "NULL argument");
    if (h->kind != DNATOK_KIND_CHAR) return fail(DNATOK_ERR_INVALID, "only one-token-per-character handles take a start table");
    std::lock_guard<std::mutex> lock(h->mu);
    if (!h->dev.empty()) return fail(DNATOK_ERR_INVALID, "the start table must be set before the handle is first used");
    h->start_lut.assign(start_lut, start_lut + 256);
    h->lut_identity = false;
    return DNATOK_OK;
}

int dnatok_create_bpe(const int32_t* a, const int32_t* b, const int32_t* o, int32_t n,
                      const int32_t byte_ids[256], const dnatok_specials* sp, dnatok_handle** out) {
    if (!a || !b || !o || !byte_ids || !out) return fail(DNATOK_ERR_INVALID, "NULL argument");
    if (int rc = check_specials(sp)) return rc;
    auto* h = new (std::nothrow) dnatok_handle();
    if (!h) return fail(DNATOK_ERR_INVALID, "out of memory");
    h->kind = DNATOK_KIND_BPE; h->sp = *sp;
    h->lut256.assign(byte_ids, byte_ids + 256);
    std::string err;
    if (int rc = build_bpe_table(a, b, o, n, byte_ids, &h->bpe, &err)) {
        delete h;
        return fail(rc, "%s", err.c_str());
    }
    *out = h;
    return DNATOK_OK;
}

void dnatok_destroy(dnatok_handle* h) {
    if (!h) return;
    int cur = 0;
    cudaGetDevice(&cur);
    for (auto& kv : h->dev) {
        DeviceTables& d = kv.second;
        if (cudaSetDevice(kv.first) != cudaSuccess) continue;
        if (d.stream) cudaStreamSynchronize(d.stream);
        void* ptrs[] = {d.lut256, d.start_lut, d.table5, d.exp_off, d.exp_ids, d.kmer_ids, d.disp, d.slots, d.merge_out, d.hot, d.byte_tok, d.bpe_compact, d.st_bytes, d.st_offsets,
                        d.st_ids, d.st_mask, d.st_lengths, d.st_status, d.st_out_offsets, d.st_scratch};
        for (void* p : ptrs) if (p) cudaFree(p);
        if (d.stream) cudaStreamDestroy(d.stream);
        if (d.ev_lengths) cudaEventDestroy(d.ev_lengths);
        for (auto& st : d.pipe_streams) if (st) { cudaStreamSynchronize(st); cudaStreamDestroy(st); }
        for (auto ev : d.pipe_events) cudaEventDestroy(ev);
        if (d.st_pipe_rows) cudaFree(d.st_pipe_rows);
        if (d.h_offsets) cudaFreeHost(d.h_offsets);
        if (d.h_rows) cudaFreeHost(d.h_rows);
    }
    if (!h->dev.empty()) cudaSetDevice(cur);
    delete h;
}

int dnatok_kind(const dnatok_handle* h) { return h ? h->kind : DNATOK_ERR_INVALID; }

int dnatok_set_row_bytes_hint(dnatok_handle* h, int64_t min_bytes, int64_t max_bytes) {
    if (!h || min_bytes < 0 || max_bytes < 0 || (max_bytes > 0 && min_bytes > max_bytes))
        return fail(DNATOK_ERR_INVALID, "bad row length hint");
    h->hint_min_row = min_bytes;
    h->hint_max_row = max_bytes;
    return DNATOK_OK;
}

size_t dnatok_scratch_bytes(const dnatok_handle* h, int64_t n_rows, int64_t total_bytes) {
    if (!h || n_rows < 0 || total_bytes < 0) return 0;
    if (h->kind == DNATOK_KIND_KMER) return h->kmer_table ? 0 : kmer_scratch_layout(h, nullptr, n_rows, total_bytes).bytes;
    if (h->kind != DNATOK_KIND_BPE) return 0;
    return bpe_scratch_layout(h, nullptr, n_rows, total_bytes).bytes;
}

int64_t dnatok_max_tokens(const dnatok_handle* h, int64_t n_rows, int64_t total_bytes, const dnatok_format* f) {
    if (!h || !f) return 0;
    return total_bytes + (int64_t)n_special(h, f) * n_rows;
}

int dnatok_scan_lengths(const int32_t* d_lengths, int64_t n_rows, int64_t* d_out_offsets, dnatok_stream stream) {
    if (!d_lengths || !d_out_offsets || n_rows < 0) return fail(DNATOK_ERR_INVALID, "bad argument");
    scan_lengths_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(d_lengths, n_rows, d_out_offsets);
    LAUNCH_CHECK("scan_lengths_kernel");
    return DNATOK_OK;
}

int dnatok_prepare(dnatok_handle* h, const uint8_t* d_bytes, const int64_t* d_offsets, int64_t n_rows,
                   int64_t total_bytes, const dnatok_format* fmt, int32_t* d_lengths, int32_t* d_status,
                   void* d_scratch, size_t scratch_bytes, dnatok_stream stream) {
    if (int rc = check_batch(h, d_bytes, d_offsets, n_rows, total_bytes)) return rc;
    if (int rc = check_format(fmt, false)) return rc;
    if (!d_lengths) return fail(DNATOK_ERR_INVALID, "d_lengths is NULL");
    cudaStream_t st = (cudaStream_t)stream;
    DeviceTables* d;
    if (int rc = tables_for_current_device(h, &d)) return rc;
    RowFormat rf;
    if (int rc = resolve(h, fmt, fmt->out_stride, &rf)) return rc;
    if (d_status && n_rows) CUDA_TRY(cudaMemsetAsync(d_status, 0, (size_t)n_rows * 4, st));
    switch (h->kind) {
        case DNATOK_KIND_CHAR:
            return launch_span_lengths(d_offsets, nullptr, n_rows, rf, d_lengths, d_status, st);
        case DNATOK_KIND_KMER:
            return launch_kmer<true>(h, *d, d_bytes, d_offsets, n_rows, total_bytes, rf, 64, nullptr, nullptr, nullptr, d_lengths,
                                     nullptr, d_status, d_scratch, scratch_bytes, st);
        default: {
            return run_bpe_merge(h, *d, d_bytes, d_offsets, n_rows, total_bytes, d_status, d_scratch, scratch_bytes, rf, d_lengths, st);
        }
    }
}

int dnatok_write(dnatok_handle* h, const uint8_t* d_bytes, const int64_t* d_offsets, int64_t n_rows,
                 int64_t total_bytes, const dnatok_format* fmt, const int32_t* d_lengths,
                 const int64_t* d_out_offsets, void* d_ids, void* d_mask, int32_t* d_status, void* d_scratch,
                 size_t scratch_bytes, dnatok_stream stream) {
    if (int rc = check_batch(h, d_bytes, d_offsets, n_rows, total_bytes)) return rc;
    if (int rc = check_format(fmt, false)) return rc;
    if (!d_ids && n_rows) return fail(DNATOK_ERR_INVALID, "d_ids is NULL");
    if (fmt->mask_bits && !d_mask && fmt->out_stride > 0) return fail(DNATOK_ERR_INVALID, "mask requested but d_mask is NULL");
    if (fmt->out_stride == 0 && !d_out_offsets) return fail(DNATOK_ERR_INVALID, "ragged output needs d_out_offsets");
    cudaStream_t st = (cudaStream_t)stream;
    DeviceTables* d;
    if (int rc = tables_for_current_device(h, &d)) return rc;
    RowFormat rf;
    if (int rc = resolve(h, fmt, fmt->out_stride, &rf)) return rc;
    switch (h->kind) {
        case DNATOK_KIND_CHAR:
            return launch_char(h, *d, d_bytes, d_offsets, n_rows, total_bytes, rf, fmt->id_bits, d_ids, d_mask, nullptr,
                               d_out_offsets, d_status, st);
        case DNATOK_KIND_KMER:
            if (fmt->out_stride > 0 && fmt->pad_left && !d_lengths)
                return fail(DNATOK_ERR_INVALID, "left padding needs d_lengths from dnatok_prepare");
            return launch_kmer<false>(h, *d, d_bytes, d_offsets, n_rows, total_bytes, rf, fmt->id_bits, d_ids, d_mask, d_lengths,
                                      nullptr, d_out_offsets, d_status, d_scratch, scratch_bytes, st);
        default: {
            if (!d_scratch) return fail(DNATOK_ERR_SCRATCH, "BPE write needs the scratch filled by dnatok_prepare");
            BpeScratch s = bpe_scratch_layout(h, d_scratch, n_rows, total_bytes);
            if (s.bytes > scratch_bytes) return fail(DNATOK_ERR_SCRATCH, "scratch too small");
            return launch_emit<uint16_t, false>(*d, s.tokens, d_offsets, s.counts, n_rows, total_bytes, rf, fmt->id_bits,
                                                d_ids, d_mask, nullptr, d_out_offsets, d_status, st);
        }
    }
}

int dnatok_encode(dnatok_handle* h, const uint8_t* d_bytes, const int64_t* d_offsets, int64_t n_rows,
                  int64_t total_bytes, const dnatok_format* fmt, void* d_ids, void* d_mask, int32_t* d_lengths,
                  int64_t* d_out_offsets, int32_t* d_status, void* d_scratch, size_t scratch_bytes,
                  dnatok_stream stream) {
    if (int rc = check_batch(h, d_bytes, d_offsets, n_rows, total_bytes)) return rc;
    if (int rc = check_format(fmt, false)) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const bool ragged = fmt->out_stride == 0;
    if (ragged && (!d_lengths || !d_out_offsets))
        return fail(DNATOK_ERR_INVALID, "ragged output needs d_lengths and d_out_offsets");
    DeviceTables* d;
    if (int rc = tables_for_current_device(h, &d)) return rc;
    RowFormat rf;
    if (int rc = resolve(h, fmt, fmt->out_stride, &rf)) return rc;

    if (h->kind == DNATOK_KIND_BPE && !ragged && g_bpe_fused_output.load() && fmt->out_stride < 0x7fffffff) {
        // padded BPE output: the merge kernels write ids and mask in their final layout
        if (!d_ids && n_rows) return fail(DNATOK_ERR_INVALID, "d_ids is NULL");
        if (fmt->mask_bits && !d_mask) return fail(DNATOK_ERR_INVALID, "mask requested but d_mask is NULL");
        // the status words are written by the first kernel that sees each row: no separate pass zeroes them
        return run_bpe_merge(h, *d, d_bytes, d_offsets, n_rows, total_bytes, d_status, d_scratch, scratch_bytes, rf, d_lengths,
                             st, d_ids, d_mask, fmt->id_bits, true);
    }
    const bool need_prepare = ragged || h->kind == DNATOK_KIND_BPE ||
                              (h->kind == DNATOK_KIND_KMER && fmt->pad_left);
    if (need_prepare) {
        if (!d_lengths) return fail(DNATOK_ERR_INVALID, "this format needs d_lengths");
        if (int rc = dnatok_prepare(h, d_bytes, d_offsets, n_rows, total_bytes, fmt, d_lengths, d_status, d_scratch,
                                    scratch_bytes, stream))
            return rc;
        if (ragged) {
            if (int rc = dnatok_scan_lengths(d_lengths, n_rows, d_out_offsets, stream)) return rc;
        }
        return dnatok_write(h, d_bytes, d_offsets, n_rows, total_bytes, fmt, d_lengths, d_out_offsets, d_ids, d_mask,
                            d_status, d_scratch, scratch_bytes, stream);
    }
    // padded char / right-padded k-mer: one kernel, lengths written on the way
    if (!d_ids && n_rows) return fail(DNATOK_ERR_INVALID, "d_ids is NULL");
    if (fmt->mask_bits && !d_mask) return fail(DNATOK_ERR_INVALID, "mask requested but d_mask is NULL");
    if (h->kind == DNATOK_KIND_CHAR) {
        // one span of every row writes the row's status word: nothing is zeroed first
        RowFormat rfc = rf;
        rfc.store_status = 1;
        return launch_char(h, *d, d_bytes, d_offsets, n_rows, total_bytes, rfc, fmt->id_bits, d_ids, d_mask, d_lengths, nullptr,
                           d_status, st);
    }
    // k-mer: the status words are zeroed inside, unless the kernel that runs writes them itself
    return launch_kmer<false>(h, *d, d_bytes, d_offsets, n_rows, total_bytes, rf, fmt->id_bits, d_ids, d_mask, nullptr, d_lengths,
                              nullptr, d_status, d_scratch, scratch_bytes, st, true);
}

// ------------------------------------------------------------------ fused embedding gather

int dnatok_embed(dnatok_handle* h, const uint8_t* d_bytes, const int64_t* d_offsets, int64_t n_rows,
                 int64_t total_bytes, const dnatok_format* fmt, const void* d_weight, int64_t vocab_rows,
                 int64_t row_bytes, void* d_out, int32_t* d_lengths, int32_t* d_status, dnatok_stream stream) {
    if (int rc = check_batch(h, d_bytes, d_offsets, n_rows, total_bytes)) return rc;
    if (int rc = check_format(fmt, false)) return rc;
    if (h->kind != DNATOK_KIND_CHAR) return fail(DNATOK_ERR_UNSUPPORTED, "dnatok_embed needs a one-token-per-byte handle");
    if (!h->start_lut.empty()) return fail(DNATOK_ERR_UNSUPPORTED, "dnatok_embed does not take handles with a start table");
    if (fmt->out_stride <= 0) return fail(DNATOK_ERR_INVALID, "dnatok_embed needs a padded layout (out_stride > 0)");
    if (!d_weight || !d_out) return fail(DNATOK_ERR_INVALID, "NULL weight or output");
    if (row_bytes <= 0 || row_bytes % 16 || vocab_rows <= 0) return fail(DNATOK_ERR_INVALID, "row_bytes must be a positive multiple of 16");
    if ((reinterpret_cast<uintptr_t>(d_weight) | reinterpret_cast<uintptr_t>(d_out)) & 15)
        return fail(DNATOK_ERR_INVALID, "weight and output must be 16-byte aligned");
    if (h->sp.pad_id >= vocab_rows) return fail(DNATOK_ERR_INVALID, "pad id outside the weight matrix");
    {
        // every id this handle can produce must be a row of the weight matrix; nothing is remapped silently
        int32_t top = -1;
        for (int32_t v : h->lut256) if (v > top) top = v;
        if (fmt->add_special) { if (h->sp.cls_id > top) top = h->sp.cls_id; if (h->sp.sep_id > top) top = h->sp.sep_id; }
        if (top >= vocab_rows)
            return fail(DNATOK_ERR_INVALID, "the tokenizer produces ids up to %d but the weight matrix has %lld rows", top,
                        (long long)vocab_rows);
    }
    cudaStream_t st = (cudaStream_t)stream;
    DeviceTables* d;
    if (int rc = tables_for_current_device(h, &d)) return rc;
    RowFormat rf;
    if (int rc = resolve(h, fmt, fmt->out_stride, &rf)) return rc;
    if (n_rows == 0) return DNATOK_OK;
    if (d_status) CUDA_TRY(cudaMemsetAsync(d_status, 0, (size_t)n_rows * 4, st));
    const int pieces = (int)(row_bytes / 16);
    int lanes = 1;
    while (lanes < 32 && lanes * 2 <= pieces) lanes *= 2;
    const int64_t spans = n_rows * ((fmt->out_stride + 31) / 32);
    int64_t blocks = (spans + EMBED_THREADS / 32 - 1) / (EMBED_THREADS / 32);
    const int64_t cap = (int64_t)d->sm_count * 32;
    if (blocks > cap) blocks = cap;
    embed_padded_kernel<<<(unsigned)blocks, EMBED_THREADS, 0, st>>>(d_bytes, d_offsets, n_rows, d->lut256, rf,
                                                                    (const uint4*)d_weight, vocab_rows, pieces, lanes,
                                                                    (uint4*)d_out, d_lengths, d_status);
    LAUNCH_CHECK("embed_padded_kernel");
    return DNATOK_OK;
}

// ------------------------------------------------------------------ host packing

// FASTA text -> packed sequence bytes + row offsets.  Header lines start with '>' (or ';'), sequence
// lines are concatenated without their line ends (LF or CRLF); blank lines are skipped.  Call with
// out_bytes == NULL to size: *n_records and *n_bytes are always set.  Returns DNATOK_ERR_CAPACITY when
// a given buffer is too small.  Text before the first header counts as one unnamed record.
int dnatok_pack_fasta(const char* text, int64_t n_text, uint8_t* out_bytes, int64_t bytes_capacity,
                      int64_t* out_offsets, int64_t offsets_capacity, int64_t* n_records, int64_t* n_bytes) {
    if ((!text && n_text) || n_text < 0 || !n_records || !n_bytes) return fail(DNATOK_ERR_INVALID, "bad argument");
    int64_t rec = 0, nb = 0;
    bool open_record = false;
    const bool write = out_bytes != nullptr && out_offsets != nullptr;
    int64_t i = 0;
    while (i < n_text) {
        const char* nl = (const char*)memchr(text + i, '\n', (size_t)(n_text - i));
        int64_t end = nl ? (nl - text) : n_text;          // line is [i, end)
        int64_t stop = end;
        while (stop > i && (text[stop - 1] == '\r' || text[stop - 1] == ' ' || text[stop - 1] == '\t')) --stop;
        if (stop > i) {
            if (text[i] == '>' || text[i] == ';') {
                if (write) {
                    if (rec >= offsets_capacity - 1) return fail(DNATOK_ERR_CAPACITY, "offsets buffer too small");
                    out_offsets[rec] = nb;
                }
                ++rec;
                open_record = true;
            } else {
                if (!open_record) {                           // sequence before any header
                    if (write) {
                        if (rec >= offsets_capacity - 1) return fail(DNATOK_ERR_CAPACITY, "offsets buffer too small");
                        out_offsets[rec] = nb;
                    }
                    ++rec;
                    open_record = true;
                }
                const int64_t len = stop - i;
                if (write) {
                    if (nb + len > bytes_capacity) return fail(DNATOK_ERR_CAPACITY, "bytes buffer too small");
                    memcpy(out_bytes + nb, text + i, (size_t)len);
                }
                nb += len;
            }
        }
        i = end + 1;
    }
    if (write) out_offsets[rec] = nb;
    *n_records = rec;
    *n_bytes = nb;
    return DNATOK_OK;
}

// ------------------------------------------------------------------ BPE without caller scratch
//
// The merge kernels need working memory beyond their inputs and outputs (merged tokens, per-row
// counts, the length-class lists and their counters).  dnatok_encode takes it from the caller;
// this variant takes it from one array that is part of the loaded library image, so the call
// itself never asks the CUDA runtime for memory.

static __device__ __align__(256) unsigned char g_builtin_scratch[DNATOK_BUILTIN_SCRATCH_BYTES];

namespace {
std::mutex g_builtin_mu;
std::map<int, void*> g_builtin_addr;   // device -> device address of g_builtin_scratch on that device
}

int dnatok_encode_bpe_builtin_scratch(dnatok_handle* h, const uint8_t* d_bytes, const int64_t* d_offsets,
                                      int64_t n_rows, int64_t total_bytes, const dnatok_format* fmt, void* d_ids,
                                      void* d_mask, int32_t* d_lengths, int64_t* d_out_offsets, int32_t* d_status,
                                      dnatok_stream stream) {
    if (int rc = check_batch(h, d_bytes, d_offsets, n_rows, total_bytes)) return rc;
    if (h->kind != DNATOK_KIND_BPE) return fail(DNATOK_ERR_INVALID, "only BPE handles use scratch memory");
    const size_t need = bpe_scratch_layout(h, nullptr, n_rows, total_bytes).bytes;
    if (need > (size_t)DNATOK_BUILTIN_SCRATCH_BYTES)
        return fail(DNATOK_ERR_CAPACITY,
                    "batch of %lld rows / %lld bytes needs %zu bytes of scratch; the built-in array holds %zu "
                    "(split the batch or use dnatok_encode with your own scratch)",
                    (long long)n_rows, (long long)total_bytes, need, (size_t)DNATOK_BUILTIN_SCRATCH_BYTES);
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    {
        // The merge tables are uploaded (allocated) by the first ordinary call on a device; this
        // entry point refuses to do that itself.
        std::lock_guard<std::mutex> lock(h->mu);
        if (h->dev.find(dev) == h->dev.end())
            return fail(DNATOK_ERR_INVALID,
                        "the handle's tables are not on device %d yet: make one dnatok_prepare / dnatok_encode call "
                        "on this device first (that call allocates them)", dev);
    }
    void* scratch = nullptr;
    {
        // g_builtin_scratch names a host-side stand-in here; the kernels need its address on the
        // current device, which the runtime resolves once per device.
        std::lock_guard<std::mutex> lock(g_builtin_mu);
        auto it = g_builtin_addr.find(dev);
        if (it == g_builtin_addr.end()) {
            CUDA_TRY(cudaGetSymbolAddress(&scratch, g_builtin_scratch));
            g_builtin_addr[dev] = scratch;
        } else scratch = it->second;
    }
    return dnatok_encode(h, d_bytes, d_offsets, n_rows, total_bytes, fmt, d_ids, d_mask, d_lengths, d_out_offsets,
                         d_status, scratch, (size_t)DNATOK_BUILTIN_SCRATCH_BYTES, stream);
}

// ------------------------------------------------------------------ host-buffer pipeline

static int grow(void** p, size_t* cap, size_t need) {
    if (need <= *cap) return 0;
    if (*p) CUDA_TRY(cudaFree(*p));
    *p = nullptr; *cap = 0;
    const size_t sz = align_up(need + need / 8, 1 << 20);
    CUDA_TRY(cudaMalloc(p, sz));
    *cap = sz;
    return 0;
}

// Fixed-stride output in row chunks over three streams: while chunk c is being encoded, chunk c+1 is
// on its way in and chunk c-1 on its way out, so the two directions of the host link (which carry
// their copies at the same time) and the kernels overlap.  Every chunk is an independent sub-batch
// with chunk-local offsets and its own piece of the device staging buffers and of the scratch, so
// nothing is reused and the issuing thread never waits.  The row lengths of a chunk come back
// before its ids; with host-written masks the worker threads wait for each chunk's lengths in turn
// and fill its mask rows while later chunks are still moving.
// Row lengths (tokens kept + special tokens) that follow from the rows' byte counts alone: one token per byte for the
// per-character tables; for k-mer tables a row with at least as many complete windows as it may keep tokens is cut to
// exactly that many, whatever its windows hold (every window yields at least one token).  Returns false as soon as a row's
// length depends on its content.  With these the host can write a padded batch's attention mask without waiting for
// the GPU; the lengths the GPU reports are compared afterwards.
static bool lengths_from_sizes(const dnatok_handle* h, const dnatok_format* f, int64_t stride, const int64_t* h_offsets,
                               int64_t n_rows, std::vector<int32_t>* out) {
    if (h->kind != DNATOK_KIND_CHAR && !(h->kind == DNATOK_KIND_KMER && !h->kmer_table && h->k > 0)) return false;
    RowFormat rf;
    if (resolve(h, f, stride, &rf)) return false;
    const int ns = n_special(h, f);
    out->resize((size_t)n_rows);
    for (int64_t r = 0; r < n_rows; ++r) {
        const int64_t len = h_offsets[r + 1] - h_offsets[r];
        int64_t t;
        if (h->kind == DNATOK_KIND_CHAR) t = len < rf.cap_content ? len : rf.cap_content;
        else if (len / h->k >= rf.cap_content) t = rf.cap_content;
        else return false;
        (*out)[(size_t)r] = (int32_t)(t + ns);
    }
    return true;
}

static int encode_host_pipelined(dnatok_handle* h, DeviceTables* d, int device, const uint8_t* h_bytes,
                                 const int64_t* h_offsets, int64_t n_rows, const dnatok_format* f,
                                 int64_t rows_per_chunk, void* h_ids, void* h_mask, int32_t* h_lengths,
                                 int32_t* h_status, int mask_threads) {
    const size_t id_sz = f->id_bits / 8, mask_sz = (f->mask_bits && h_mask) ? f->mask_bits / 8 : 0;
    const int64_t stride = f->out_stride;
    const int64_t total = h_offsets[n_rows];
    const int64_t n_chunks = (n_rows + rows_per_chunk - 1) / rows_per_chunk;
    const bool host_mask = mask_sz && mask_threads > 0 &&
                           (int64_t)((size_t)(n_rows * stride) * mask_sz) >= g_host_mask_min_bytes.load();
    dnatok_format cf = *f;
    if (!mask_sz || host_mask) cf.mask_bits = 0;

    // staging for the whole batch (grow only), chunk-local offsets in pinned host memory
    if (int rc = grow((void**)&d->st_bytes, &d->st_bytes_cap, (size_t)total + 64)) return rc;
    if (int rc = grow((void**)&d->st_offsets, &d->st_offsets_cap, (size_t)(n_rows + n_chunks) * 8)) return rc;
    if (int rc = grow(&d->st_ids, &d->st_ids_cap, (size_t)(n_rows * stride) * id_sz + 64)) return rc;
    if (mask_sz && !host_mask)
        if (int rc = grow(&d->st_mask, &d->st_mask_cap, (size_t)(n_rows * stride) * mask_sz + 64)) return rc;
    if (int rc = grow(&d->st_pipe_rows, &d->st_pipe_rows_cap, (size_t)n_rows * 8 + 64)) return rc;
    if ((size_t)(n_rows + n_chunks) * 8 > d->h_offsets_cap) {
        if (d->h_offsets) CUDA_TRY(cudaFreeHost(d->h_offsets));
        d->h_offsets = nullptr; d->h_offsets_cap = 0;
        const size_t cap = (size_t)(n_rows + n_chunks) * 8 + 65536;
        CUDA_TRY(cudaMallocHost((void**)&d->h_offsets, cap));
        d->h_offsets_cap = cap;
    }
    // k-mer chunks run one warp per row: several chunks are on the GPU at once, and the segment encoder
    // counts on having its whole grid resident
    size_t scratch_total = 0;
    std::vector<size_t> scratch_at((size_t)n_chunks + 1, 0);
    for (int64_t c = 0; c < n_chunks; ++c) {
        const int64_t r0 = c * rows_per_chunk, r1 = r0 + rows_per_chunk < n_rows ? r0 + rows_per_chunk : n_rows;
        scratch_at[(size_t)c] = scratch_total;
        if (h->kind == DNATOK_KIND_BPE)
            scratch_total += align_up(dnatok_scratch_bytes(h, r1 - r0, h_offsets[r1] - h_offsets[r0]), 256);
    }
    scratch_at[(size_t)n_chunks] = scratch_total;
    if (scratch_total) if (int rc = grow(&d->st_scratch, &d->st_scratch_cap, scratch_total)) return rc;
    while ((int64_t)d->pipe_events.size() < n_chunks) {
        cudaEvent_t ev;
        CUDA_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
        d->pipe_events.push_back(ev);
    }
    for (auto& st : d->pipe_streams) if (!st) CUDA_TRY(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));

    int32_t* d_len_all = (int32_t*)d->st_pipe_rows;
    int32_t* d_st_all = d_len_all + n_rows;
    if (int rc = pinned_rows(d, n_rows)) return rc;
    int32_t* hl = d->h_rows;                                   // lengths land here, status words behind them
    int32_t* hs = d->h_rows + n_rows;
    std::vector<int32_t> known;                                // lengths the host can tell beforehand (else empty)
    const bool lengths_known = host_mask && g_host_mask_early.load() && lengths_from_sizes(h, f, stride, h_offsets, n_rows, &known);
    for (int64_t c = 0; c < n_chunks; ++c) {
        const int64_t r0 = c * rows_per_chunk, r1 = r0 + rows_per_chunk < n_rows ? r0 + rows_per_chunk : n_rows;
        const int64_t rows = r1 - r0, b0 = h_offsets[r0], nbytes = h_offsets[r1] - b0;
        cudaStream_t st = d->pipe_streams[c % 3];
        int64_t* ho = d->h_offsets + r0 + c;                   // rows + 1 entries of this chunk
        for (int64_t i = 0; i <= rows; ++i) ho[i] = h_offsets[r0 + i] - b0;
        uint8_t* db = d->st_bytes + b0;
        int64_t* dof = d->st_offsets + r0 + c;
        if (nbytes) CUDA_TRY(cudaMemcpyAsync(db, h_bytes + b0, (size_t)nbytes, cudaMemcpyHostToDevice, st));
        CUDA_TRY(cudaMemcpyAsync(dof, ho, (size_t)(rows + 1) * 8, cudaMemcpyHostToDevice, st));
        uint8_t* dids = (uint8_t*)d->st_ids + (size_t)(r0 * stride) * id_sz;
        uint8_t* dmask = (mask_sz && !host_mask) ? (uint8_t*)d->st_mask + (size_t)(r0 * stride) * mask_sz : nullptr;
        if (int rc = dnatok_encode(h, db, dof, rows, nbytes, &cf, dids, dmask, d_len_all + r0, nullptr, d_st_all + r0,
                                   scratch_total ? (uint8_t*)d->st_scratch + scratch_at[(size_t)c] : nullptr,
                                   scratch_at[(size_t)c + 1] - scratch_at[(size_t)c], st))
            return rc;
        CUDA_TRY(cudaMemcpyAsync(hl + r0, d_len_all + r0, (size_t)rows * 4, cudaMemcpyDeviceToHost, st));
        if (h_status) CUDA_TRY(cudaMemcpyAsync(hs + r0, d_st_all + r0, (size_t)rows * 4, cudaMemcpyDeviceToHost, st));
        CUDA_TRY(cudaEventRecord(d->pipe_events[(size_t)c], st));
        CUDA_TRY(cudaMemcpyAsync((uint8_t*)h_ids + (size_t)(r0 * stride) * id_sz, dids, (size_t)(rows * stride) * id_sz,
                                 cudaMemcpyDeviceToHost, st));
        if (dmask)
            CUDA_TRY(cudaMemcpyAsync((uint8_t*)h_mask + (size_t)(r0 * stride) * mask_sz, dmask,
                                     (size_t)(rows * stride) * mask_sz, cudaMemcpyDeviceToHost, st));
    }
    g_last_h2d = total + (n_rows + n_chunks) * 8;
    g_last_d2h = n_rows * stride * (int64_t)(id_sz + (host_mask ? 0 : mask_sz)) + n_rows * 4 + (h_status ? n_rows * 4 : 0);
    int rc_mask = 0;
    if (host_mask) {
        // every worker takes its stripe of each chunk once that chunk's lengths have arrived
        const int nt = mask_threads;
        std::vector<int> errs((size_t)nt, 0);
        auto fill = [&](const int32_t* len, int64_t a, int64_t b) {
            if (f->mask_bits == 64) fill_mask_rows<int64_t>((int64_t*)h_mask, len, a, b, stride, f->pad_left != 0);
            else if (f->mask_bits == 32) fill_mask_rows<int32_t>((int32_t*)h_mask, len, a, b, stride, f->pad_left != 0);
            else fill_mask_rows<uint8_t>((uint8_t*)h_mask, len, a, b, stride, f->pad_left != 0);
        };
        auto work = [&](int t) {
            if (cudaSetDevice(device) != cudaSuccess) { errs[(size_t)t] = 1; return; }
            if (lengths_known) {                                 // nothing to wait for: the whole stripe at once
                fill(known.data(), n_rows * t / nt, n_rows * (t + 1) / nt);
                return;
            }
            for (int64_t c = 0; c < n_chunks; ++c) {
                if (cudaEventSynchronize(d->pipe_events[(size_t)c]) != cudaSuccess) { errs[(size_t)t] = 1; return; }
                const int64_t r0 = c * rows_per_chunk, r1 = r0 + rows_per_chunk < n_rows ? r0 + rows_per_chunk : n_rows;
                fill(hl, r0 + (r1 - r0) * t / nt, r0 + (r1 - r0) * (t + 1) / nt);
            }
        };
        HostPool::get().run(nt, work);
        if (lengths_known) {
            // the GPU's lengths have the last word: a row that came out otherwise gets its mask again
            for (auto& st : d->pipe_streams) if (st) CUDA_TRY(cudaStreamSynchronize(st));
            for (int64_t r = 0; r < n_rows; ++r)
                if (hl[r] != known[(size_t)r]) fill(hl, r, r + 1);
        }
        for (int e : errs) if (e) rc_mask = fail(DNATOK_ERR_CUDA, "a host worker could not wait for the row lengths");
    }
    for (auto& st : d->pipe_streams) if (st) CUDA_TRY(cudaStreamSynchronize(st));
    if (h_lengths) memcpy(h_lengths, hl, (size_t)n_rows * 4);
    if (h_status) memcpy(h_status, hs, (size_t)n_rows * 4);
    return rc_mask;
}

int dnatok_encode_host(dnatok_handle* h, int device, const uint8_t* h_bytes, const int64_t* h_offsets,
                       int64_t n_rows, const dnatok_format* fmt, void* h_ids, int64_t ids_capacity, void* h_mask,
                       int32_t* h_lengths, int64_t* h_out_offsets, int32_t* h_status, int64_t* out_stride_used) {
    if (!h) return fail(DNATOK_ERR_INVALID, "handle is NULL");
    if (int rc = check_format(fmt, true)) return rc;
    if (n_rows < 0 || !h_offsets) return fail(DNATOK_ERR_INVALID, "bad batch");
    const int64_t total = h_offsets[n_rows] - h_offsets[0];
    if (h_offsets[0] != 0) return fail(DNATOK_ERR_INVALID, "offsets must start at 0");
    if (int rc = check_batch(h, h_bytes, h_offsets, n_rows, total)) return rc;
    CUDA_TRY(cudaSetDevice(device));
    struct HintGuard {          // row lengths are known here: bound the BPE classes for this call only
        dnatok_handle* h; int64_t lo, hi;
        ~HintGuard() { h->hint_min_row = lo; h->hint_max_row = hi; }
    } guard{h, h->hint_min_row, h->hint_max_row};
    if (n_rows > 0) {
        int64_t lo = INT64_MAX, hi = 0;
        for (int64_t i = 0; i < n_rows; ++i) {
            const int64_t n = h_offsets[i + 1] - h_offsets[i];
            if (n < lo) lo = n;
            if (n > hi) hi = n;
        }
        if (hi > 0x7fffffff && h->kind == DNATOK_KIND_KMER)
            return fail(DNATOK_ERR_UNSUPPORTED, "a k-mer row of %lld bytes: rows must be shorter than 2 GiB", (long long)hi);
        h->hint_min_row = lo; h->hint_max_row = hi > 0 ? hi : 1;
    }
    DeviceTables* d;
    if (int rc = tables_for_current_device(h, &d)) return rc;
    if (!d->stream) CUDA_TRY(cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking));
    cudaStream_t st = d->stream;
    const int ns = n_special(h, fmt);
    const size_t id_sz = fmt->id_bits / 8, mask_sz = fmt->mask_bits / 8;

    {
        // Fixed stride known up front (given, or char rows padded to the longest): chunked pipeline
        // when the batch is large enough to split.
        int64_t pstride = fmt->out_stride;
        if (pstride < 0 && h->kind == DNATOK_KIND_CHAR) {
            const int64_t cap = fmt->max_tokens > 0 ? fmt->max_tokens - ns : INT64_MAX;
            pstride = 0;
            for (int64_t i = 0; i < n_rows; ++i) {
                int64_t n = h_offsets[i + 1] - h_offsets[i];
                if (n > cap) n = cap;
                if (n + ns > pstride) pstride = n + ns;
            }
        }
        if (pstride > 0 && n_rows >= 2) {
            int mask_threads = (int)g_host_mask_threads.load();
            if (mask_threads < 0) {
                const unsigned hc = std::thread::hardware_concurrency();
                mask_threads = hc == 0 ? 1 : (hc > 4 ? 4 : (int)hc);   // non-temporal stores: two threads keep up with the link, more only add contention
            }
            const bool want_mask = mask_sz && h_mask;
            const bool host_mask = want_mask && mask_threads > 0 &&
                                   (int64_t)((size_t)(n_rows * pstride) * mask_sz) >= g_host_mask_min_bytes.load();
            // bytes that cross the link per row: the input, the ids, and the mask unless host threads write it
            const size_t row_link = (size_t)pstride * (id_sz + ((want_mask && !host_mask) ? mask_sz : 0)) + (size_t)(total / n_rows) + 1;
            const size_t link_total = row_link * (size_t)n_rows;
            // The two directions of the host link carry copies at the same time (measured: both at once take
            // 0.57 of one after the other), so batches from 128 MiB up are split into chunks of about 64 MiB.
            const size_t CHUNK_BYTES = (size_t)g_host_chunk_bytes.load();
            const size_t threshold = (size_t)g_host_chunk_threshold.load();
            if (CHUNK_BYTES && link_total >= threshold && link_total >= 2 * CHUNK_BYTES) {
                if (n_rows * pstride > ids_capacity)
                    return fail(DNATOK_ERR_CAPACITY, "ids buffer holds %lld elements, %lld needed", (long long)ids_capacity,
                                (long long)(n_rows * pstride));
                int64_t rpc = (int64_t)(CHUNK_BYTES / row_link);
                if (rpc < 1) rpc = 1;
                if ((n_rows + rpc - 1) / rpc > 256) rpc = (n_rows + 255) / 256;      // at most 256 chunks
                dnatok_format pf = *fmt;
                pf.out_stride = pstride;
                if (int rc = encode_host_pipelined(h, d, device, h_bytes, h_offsets, n_rows, &pf, rpc, h_ids, h_mask, h_lengths,
                                                   h_status, mask_threads))
                    return rc;
                if (out_stride_used) *out_stride_used = pstride;
                return DNATOK_OK;
            }
        }
    }
    if (int rc = grow((void**)&d->st_bytes, &d->st_bytes_cap, (size_t)total + 64)) return rc;
    if (int rc = grow((void**)&d->st_offsets, &d->st_offsets_cap, (size_t)(n_rows + 1) * 8)) return rc;
    if ((size_t)n_rows + 1 > d->st_rows_cap) {
        for (void** p : {(void**)&d->st_lengths, (void**)&d->st_status, (void**)&d->st_out_offsets})
            if (*p) { CUDA_TRY(cudaFree(*p)); *p = nullptr; }
        d->st_rows_cap = 0;
        const size_t cap = (size_t)n_rows + n_rows / 8 + 1024;
        cudaError_t e1 = cudaMalloc((void**)&d->st_lengths, cap * 4);
        cudaError_t e2 = e1 == cudaSuccess ? cudaMalloc((void**)&d->st_status, cap * 4) : e1;
        cudaError_t e3 = e2 == cudaSuccess ? cudaMalloc((void**)&d->st_out_offsets, cap * 8) : e2;
        if (e3 != cudaSuccess) {
            for (void** p : {(void**)&d->st_lengths, (void**)&d->st_status, (void**)&d->st_out_offsets})
                if (*p) { cudaFree(*p); *p = nullptr; }
            return fail(DNATOK_ERR_CUDA, "staging allocation: %s", cudaGetErrorString(e3));
        }
        d->st_rows_cap = cap;
    }
    const size_t scratch_need = dnatok_scratch_bytes(h, n_rows, total);
    if (scratch_need) if (int rc = grow(&d->st_scratch, &d->st_scratch_cap, scratch_need)) return rc;

    CUDA_TRY(cudaMemcpyAsync(d->st_bytes, h_bytes, (size_t)total, cudaMemcpyHostToDevice, st));
    CUDA_TRY(cudaMemcpyAsync(d->st_offsets, h_offsets, (size_t)(n_rows + 1) * 8, cudaMemcpyHostToDevice, st));

    dnatok_format f = *fmt;
    int64_t stride = fmt->out_stride;
    bool prepared = false;
    if (stride < 0) {
        // pad to the longest row: char rows are sized on the host, the other kinds by the sizing pass
        int64_t longest = 0;
        if (h->kind == DNATOK_KIND_CHAR) {
            const int64_t cap = fmt->max_tokens > 0 ? fmt->max_tokens - ns : INT64_MAX;
            for (int64_t i = 0; i < n_rows; ++i) {
                int64_t n = h_offsets[i + 1] - h_offsets[i];
                if (n > cap) n = cap;
                if (n + ns > longest) longest = n + ns;
            }
        } else {
            f.out_stride = 0;
            if (int rc = dnatok_prepare(h, d->st_bytes, d->st_offsets, n_rows, total, &f, d->st_lengths, d->st_status,
                                        d->st_scratch, d->st_scratch_cap, st))
                return rc;
            std::vector<int32_t> tmp;
            int32_t* hl = h_lengths;
            if (!hl) { tmp.resize((size_t)n_rows + 1); hl = tmp.data(); }
            CUDA_TRY(cudaMemcpyAsync(hl, d->st_lengths, (size_t)n_rows * 4, cudaMemcpyDeviceToHost, st));
            CUDA_TRY(cudaStreamSynchronize(st));
            for (int64_t i = 0; i < n_rows; ++i) if (hl[i] > longest) longest = hl[i];
            prepared = true;
        }
        stride = longest;
        if (stride == 0) {                               // every row is empty: nothing to write but the row words
            CUDA_TRY(cudaStreamSynchronize(st));
            if (h_lengths) for (int64_t i = 0; i < n_rows; ++i) h_lengths[i] = 0;
            if (h_status) for (int64_t i = 0; i < n_rows; ++i) h_status[i] = 0;
            g_last_h2d = total + (n_rows + 1) * 8;
            g_last_d2h = 0;
            if (out_stride_used) *out_stride_used = 0;
            return DNATOK_OK;
        }
    }
    f.out_stride = stride;
    const bool ragged = stride == 0;
    const int64_t out_elems = ragged ? dnatok_max_tokens(h, n_rows, total, fmt) : n_rows * stride;
    if (!ragged && out_elems > ids_capacity) return fail(DNATOK_ERR_CAPACITY, "ids buffer holds %lld elements, %lld needed",
                                                         (long long)ids_capacity, (long long)out_elems);
    // a large mask of a padded batch is written by host threads while the ids are on their way back
    int mask_threads = (int)g_host_mask_threads.load();
    if (mask_threads < 0) {
        const unsigned hc = std::thread::hardware_concurrency();
        mask_threads = hc == 0 ? 1 : (hc > 4 ? 4 : (int)hc);   // non-temporal stores: two threads keep up with the link, more only add contention
    }
    const bool host_mask = mask_sz && h_mask && !ragged && mask_threads > 0 &&
                           (int64_t)((size_t)out_elems * mask_sz) >= g_host_mask_min_bytes.load();
    if (int rc = grow(&d->st_ids, &d->st_ids_cap, (size_t)out_elems * id_sz + 64)) return rc;
    if (mask_sz && h_mask && !host_mask)
        if (int rc = grow(&d->st_mask, &d->st_mask_cap, (size_t)out_elems * mask_sz + 64)) return rc;
    void* dmask = (mask_sz && h_mask && !host_mask) ? d->st_mask : nullptr;
    if (!dmask) f.mask_bits = 0;

    int rc;
    if (prepared) {
        rc = dnatok_write(h, d->st_bytes, d->st_offsets, n_rows, total, &f, d->st_lengths, nullptr, d->st_ids, dmask,
                          d->st_status, d->st_scratch, d->st_scratch_cap, st);
    } else {
        rc = dnatok_encode(h, d->st_bytes, d->st_offsets, n_rows, total, &f, d->st_ids, dmask, d->st_lengths,
                           d->st_out_offsets, d->st_status, d->st_scratch, d->st_scratch_cap, st);
    }
    if (rc) return rc;

    int64_t n_out = out_elems;
    if (ragged) {
        int64_t tot = 0;
        CUDA_TRY(cudaMemcpyAsync(&tot, d->st_out_offsets + n_rows, 8, cudaMemcpyDeviceToHost, st));
        CUDA_TRY(cudaStreamSynchronize(st));
        n_out = tot;
        if (n_out > ids_capacity) return fail(DNATOK_ERR_CAPACITY, "ids buffer holds %lld elements, %lld needed",
                                              (long long)ids_capacity, (long long)n_out);
        if (h_out_offsets)
            CUDA_TRY(cudaMemcpyAsync(h_out_offsets, d->st_out_offsets, (size_t)(n_rows + 1) * 8, cudaMemcpyDeviceToHost, st));
    }
    g_last_h2d = total + (n_rows + 1) * 8;
    g_last_d2h = n_out * (int64_t)id_sz + (ragged && h_out_offsets ? (n_rows + 1) * 8 : 0);
    if (host_mask && n_rows) {
        // lengths first (small), then the ids; the mask is filled while the ids are still being copied
        if (int rc2 = pinned_rows(d, n_rows)) return rc2;
        int32_t* hl = d->h_rows;
        int32_t* hs = d->h_rows + n_rows;
        CUDA_TRY(cudaMemcpyAsync(hl, d->st_lengths, (size_t)n_rows * 4, cudaMemcpyDeviceToHost, st));
        if (h_status) CUDA_TRY(cudaMemcpyAsync(hs, d->st_status, (size_t)n_rows * 4, cudaMemcpyDeviceToHost, st));
        if (!d->ev_lengths) CUDA_TRY(cudaEventCreateWithFlags(&d->ev_lengths, cudaEventDisableTiming));
        CUDA_TRY(cudaEventRecord(d->ev_lengths, st));
        if (n_out) CUDA_TRY(cudaMemcpyAsync(h_ids, d->st_ids, (size_t)n_out * id_sz, cudaMemcpyDeviceToHost, st));
        HostMask hm;
        hm.device = device; hm.mask = h_mask; hm.mask_bits = fmt->mask_bits; hm.lengths = hl; hm.n_rows = n_rows;
        hm.stride = stride; hm.pad_left = fmt->pad_left != 0; hm.ev_lengths = d->ev_lengths;
        if (int rc2 = host_mask_fill(hm, mask_threads)) return rc2;
        g_last_d2h += n_rows * 4 * (h_status ? 2 : 1);
        CUDA_TRY(cudaStreamSynchronize(st));
        if (h_lengths) memcpy(h_lengths, hl, (size_t)n_rows * 4);
        if (h_status) memcpy(h_status, hs, (size_t)n_rows * 4);
        if (out_stride_used) *out_stride_used = stride;
        return DNATOK_OK;
    }
    if (n_out) CUDA_TRY(cudaMemcpyAsync(h_ids, d->st_ids, (size_t)n_out * id_sz, cudaMemcpyDeviceToHost, st));
    if (dmask && n_out) { CUDA_TRY(cudaMemcpyAsync(h_mask, dmask, (size_t)n_out * mask_sz, cudaMemcpyDeviceToHost, st)); g_last_d2h += n_out * (int64_t)mask_sz; }
    if (h_lengths && n_rows) { CUDA_TRY(cudaMemcpyAsync(h_lengths, d->st_lengths, (size_t)n_rows * 4, cudaMemcpyDeviceToHost, st)); g_last_d2h += n_rows * 4; }
    if (h_status && n_rows) { CUDA_TRY(cudaMemcpyAsync(h_status, d->st_status, (size_t)n_rows * 4, cudaMemcpyDeviceToHost, st)); g_last_d2h += n_rows * 4; }
    CUDA_TRY(cudaStreamSynchronize(st));
    if (out_stride_used) *out_stride_used = ragged ? n_out : stride;
    return DNATOK_OK;
}

}  // extern "C"

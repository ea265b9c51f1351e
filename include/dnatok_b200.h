/* dnatok_b200 - C ABI of the B200 (sm_100a) genomic tokenizer kernels.
 *
 * Plain pointers and sizes only; no torch, no C++ types.  Every function returns DNATOK_OK (0)
 * or a negative error code, never throws and never aborts; dnatok_last_error() gives the text
 * of the last failure on the calling thread.  Device buffers are owned by the caller; a handle
 * owns only its lookup tables (uploaded once per device on first use) and, for the *_host
 * entry point, its staging buffers.  Calls on distinct handles are thread safe; one call per
 * handle at a time.
 *
 * Which reference interface each entry point stands in for (paths inside eniktab/DNAtok):
 *   dnatok_create_char    the ASCII LUT built by DNATok.discover, src/dna_tokenizer.py:995-1030
 *                         (_build_ascii_lut_probe_all :633-653)
 *   dnatok_create_kmer    _build_kmer_lut, src/dna_tokenizer.py:743-822 (+ tail LUT :957-971)
 *   dnatok_create_kmer_table  the same with every window's token run tabulated (:759-806, :1896-1953)
 *   dnatok_set_start_lut  the start / continuation tables, src/dna_tokenizer.py:527-631
 *   dnatok_create_bpe     DNATokBPE(merges_path, byte_to_id_lut, max_iters) constructor,
 *                         src/dnatok_bpe_kernel/dnatok_bpe.cu:797-862 (build_vocab_from_merges :761-791)
 *   dnatok_encode         char: _encode_batch_ascii_lut_numpy :1779-1820 / _map_ascii_bytes_to_ids_cuda
 *                         :2653-2723; k-mer: _encode_batch_kmer_numpy_partial :1369-1474 with
 *                         _encode_kmer_fallback_from_lut :1896-1953 / _map_kmer_bytes_to_ids_cuda
 *                         :2826-2940; BPE: DNATokBPE::tokenize_batch, dnatok_bpe.cu:865-947, plus the
 *                         remap / trim / pad / mask tail of GPUTokBPEBackend.encode_batch,
 *                         src/gputok_bpe_backend.py:577-601; padding and masks of
 *                         encode_batch_with_padding, src/dna_tokenizer.py:2150-2236
 *   dnatok_prepare/write  the two halves of dnatok_encode for callers that size the output from
 *                         the longest row (the reference's lens.max().item(), gputok_bpe_backend.py:584-585)
 *   dnatok_encode_host    the same path fed from host memory: host packing + H2D of
 *                         dnatok_bpe.cu:872-887 and the D2H of src/dna_tokenizer.py:2067-2083
 */
#ifndef DNATOK_B200_H
#define DNATOK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DNATOK_ABI_VERSION 1

/* return codes */
#define DNATOK_OK               0
#define DNATOK_ERR_INVALID     (-1)   /* bad argument */
#define DNATOK_ERR_CUDA        (-2)   /* a CUDA runtime call failed */
#define DNATOK_ERR_UNSUPPORTED (-3)   /* tables outside what the kernels implement */
#define DNATOK_ERR_SCRATCH     (-4)   /* scratch buffer missing or too small */
#define DNATOK_ERR_CAPACITY    (-5)   /* output buffer too small */

/* per-row status bits written to d_status (0 = fine) */
#define DNATOK_ROW_TOO_LONG       1   /* BPE word longer than DNATOK_BPE_MAX_WORD: row left empty; k-mer row of 2 GiB
                                         or more: only its first 2^31 - 1 bytes are encoded */
#define DNATOK_ROW_NOT_CONVERGED  2   /* BPE pass limit reached (cannot happen for a consistent table) */
#define DNATOK_ROW_CLIPPED        4   /* row had more tokens than out_stride and was cut to fit */
#define DNATOK_ROW_OUTSIDE_HINT   8   /* BPE row length outside dnatok_set_row_bytes_hint; row left empty */
#define DNATOK_ROW_STALLED        16  /* k-mer row segment gave up waiting for the segment before it; row left unfinished */

#define DNATOK_KIND_CHAR 0
#define DNATOK_KIND_KMER 1
#define DNATOK_KIND_BPE  2

#define DNATOK_BPE_MAX_WORD (1 << 30) /* longest BPE word (bytes): words of up to 32,768 bytes are merged in shared
                                         memory, longer ones in scratch memory (about 4.5 bytes of scratch per byte) */

typedef struct dnatok_handle dnatok_handle;
typedef void* dnatok_stream;          /* a cudaStream_t */

typedef struct {
    int32_t pad_id;
    int32_t unk_id;
    int32_t cls_id;                   /* emitted before the row when add_special; -1: none */
    int32_t sep_id;                   /* emitted after the row when add_special; -1: none */
} dnatok_specials;

typedef struct {
    int32_t id_bits;                  /* 32 or 64: element type of the ids output */
    int32_t mask_bits;                /* 0: no mask output; 8, 32 or 64: element type of the mask */
    int32_t add_special;              /* attach cls/sep */
    int32_t pad_left;                 /* 0: right padding (HF default), 1: left (DNATok default) */
    int64_t max_tokens;               /* truncate rows to this many tokens, specials included; 0: off */
    int64_t out_stride;               /* > 0: ids/mask are [n_rows, out_stride]; 0: ragged (ids only,
                                         d_out_offsets gives row starts); -1 (host entry point only):
                                         pad to the longest row */
} dnatok_format;

int dnatok_version(void);
const char* dnatok_last_error(void);

int dnatok_create_char(const int32_t lut[256], const dnatok_specials* sp, dnatok_handle** out);
int dnatok_create_kmer(int k, const int32_t* kmer_ids /* 4^k, product("ACGT") order */,
                       const int32_t single_ids[256], const dnatok_specials* sp, dnatok_handle** out);
/* A k-mer tokenizer given as the table of all 5^k windows over A, C, G, T, N (index = base-5 number of the
 * window, A C G T N = 0 1 2 3 4, first character most significant): table5[i] >= 0 is the window's id,
 * table5[i] = -(e + 1) names run e, ids run_ids[run_offsets[e] .. run_offsets[e + 1]).  Any other character counts
 * as N.  tail_singles != 0: the len % k characters left over give single_ids[c] each; 0: they give nothing.
 * Stands in for the reference's complete k-mer table with multi-token expansion: _build_kmer_lut,
 * src/dna_tokenizer.py:743-822 (kmer_lut / kmer_lut_offsets / kmer_lut_lengths / kmer_lut_flat), replayed by
 * _encode_kmer_fallback_from_lut :1896-1953 and _expand_kmer_packed_cuda :2736-2824.  dnatok_create_kmer remains the
 * fast form for tokenizers whose non-ACGT windows expand character by character. */
int dnatok_create_kmer_table(int k, const int32_t* table5, const int32_t* run_offsets, int32_t n_runs, const int32_t* run_ids,
                             const int32_t single_ids[256], int tail_singles, const dnatok_specials* sp,
                             dnatok_handle** out);
/* Ids of a row's FIRST character for one-token-per-character handles whose tokenizer gives a character another id at
 * the start of a sequence than later on.  Call before the handle is first used.  Stands in for the reference's start /
 * continuation tables: _resolve_cont_ids / _rebuild_ascii_luts_from_tokenizer, src/dna_tokenizer.py:527-631, applied to
 * column 0 at :1779-1820 and :2716-2721. */
int dnatok_set_start_lut(dnatok_handle* h, const int32_t start_lut[256]);
int dnatok_create_bpe(const int32_t* merge_a, const int32_t* merge_b, const int32_t* merge_out,
                      int32_t n_merges, const int32_t byte_ids[256], const dnatok_specials* sp,
                      dnatok_handle** out);
void dnatok_destroy(dnatok_handle* h);
int dnatok_kind(const dnatok_handle* h);

/* Optional bounds on the row lengths (bytes) of the batches that follow on this handle; 0, 0 clears
 * them.  The BPE path launches one kernel per length class and, without bounds, has to launch every
 * class the batch size allows; with bounds only the classes in range are launched.  A row outside
 * the bounds gets DNATOK_ROW_OUTSIDE_HINT and no tokens.  dnatok_encode_host derives the bounds from
 * its host offsets by itself.  No reference counterpart (its kernel is one launch, one block per row). */
int dnatok_set_row_bytes_hint(dnatok_handle* h, int64_t min_bytes, int64_t max_bytes);

/* Bytes of caller-owned device scratch dnatok_prepare / dnatok_encode use for this batch
 * (0 for char).  The scratch must be 256-byte aligned.  BPE requires it.  For k-mer it is optional
 * (one flag per row segment and a ticket counter): with it and with a status array, batches that one
 * warp per row could not spread over the whole GPU (few rows, or very long rows) are cut into segments
 * of 256 windows that the warps draw from the counter; without it one warp (or one block, for very
 * long rows) encodes each row.
 * Results are identical.  The size depends on the handle's row-length hint: query it after
 * dnatok_set_row_bytes_hint. */
size_t dnatok_scratch_bytes(const dnatok_handle* h, int64_t n_rows, int64_t total_bytes);

/* Upper bound on the number of ids a ragged output can hold for this batch. */
int64_t dnatok_max_tokens(const dnatok_handle* h, int64_t n_rows, int64_t total_bytes,
                          const dnatok_format* fmt);

/* Row i is d_bytes[d_offsets[i] .. d_offsets[i+1]).  All pointers are device pointers on the
 * current device; work is enqueued on `stream` and nothing is synchronised.
 *
 * dnatok_prepare: d_lengths[i] (int32) = tokens of row i after truncation, specials included.
 *   For BPE the merged tokens stay in d_scratch for the dnatok_write that follows.
 * dnatok_write:   fills d_ids / d_mask.  Padded: out_stride columns per row.  Ragged:
 *   d_out_offsets (int64[n_rows+1], input) gives each row's start; d_mask may be NULL.
 *   d_lengths must come from dnatok_prepare on the same batch, format and scratch.
 * dnatok_encode:  both steps.  Ragged: d_out_offsets is an output (exclusive scan of lengths).
 *   d_lengths and d_status may be NULL for padded output (for BPE only in dnatok_encode, where the merge kernels write
 *   the final rows themselves).  d_status needs no zeroing by the caller: every row's word is defined on return. */
int dnatok_prepare(dnatok_handle* h, const uint8_t* d_bytes, const int64_t* d_offsets,
                   int64_t n_rows, int64_t total_bytes, const dnatok_format* fmt,
                   int32_t* d_lengths, int32_t* d_status, void* d_scratch, size_t scratch_bytes,
                   dnatok_stream stream);
int dnatok_write(dnatok_handle* h, const uint8_t* d_bytes, const int64_t* d_offsets,
                 int64_t n_rows, int64_t total_bytes, const dnatok_format* fmt,
                 const int32_t* d_lengths, const int64_t* d_out_offsets, void* d_ids, void* d_mask,
                 int32_t* d_status, void* d_scratch, size_t scratch_bytes, dnatok_stream stream);
int dnatok_encode(dnatok_handle* h, const uint8_t* d_bytes, const int64_t* d_offsets,
                  int64_t n_rows, int64_t total_bytes, const dnatok_format* fmt,
                  void* d_ids, void* d_mask, int32_t* d_lengths, int64_t* d_out_offsets,
                  int32_t* d_status, void* d_scratch, size_t scratch_bytes, dnatok_stream stream);

/* BPE encode for callers that must not allocate.  No counterpart in the reference (its kernel
 * wrapper grows torch workspace tensors on demand, dnatok_bpe.cu:956-1015).
 *
 * Who needs it: a host that has already handed all device memory to its own pool (a serving
 * process, an inference engine's plug-in slot), or a latency-critical loop that cannot afford
 * the device-wide synchronisation an allocation or free may imply.  Such callers can still own
 * input and output buffers, but cannot size a scratch buffer per batch.
 *
 * Same arguments and results as dnatok_encode on a BPE handle, minus the scratch pair: the
 * working memory is one array of DNATOK_BUILTIN_SCRATCH_BYTES inside the library image, which
 * every GPU that loads the library holds until the process exits.  The call makes no cudaMalloc /
 * cudaFree and calls no allocating library routine.
 *   - Limit: dnatok_scratch_bytes(h, n_rows, total_bytes) must not exceed
 *     DNATOK_BUILTIN_SCRATCH_BYTES (about 2 bytes per input byte plus 32 per row), otherwise
 *     DNATOK_ERR_CAPACITY with the sizes in dnatok_last_error(); nothing is launched.
 *   - The handle's merge tables must already be on the current device: one earlier
 *     dnatok_prepare / dnatok_encode call there uploads them; otherwise DNATOK_ERR_INVALID.
 *     That earlier call also loads and configures every kernel the BPE path can launch (all
 *     length classes, both id widths), so that this entry point does not meet a kernel for the
 *     first time: loading a kernel's code is a step the CUDA runtime may allocate for.
 *   - The first call on each device also resolves the array's device address (once per device,
 *     with that device current); make that first call outside any stream capture.
 *   - All calls, on any handle and stream, share the one array, and it keeps the previous call's
 *     contents (the counters that must start at zero are cleared on the stream at the start of
 *     every call).  Two calls whose GPU work overlaps race on it: keep them on one stream or
 *     order them with events. */
#define DNATOK_BUILTIN_SCRATCH_BYTES (8u << 20)
int dnatok_encode_bpe_builtin_scratch(dnatok_handle* h, const uint8_t* d_bytes, const int64_t* d_offsets,
                                      int64_t n_rows, int64_t total_bytes, const dnatok_format* fmt,
                                      void* d_ids, void* d_mask, int32_t* d_lengths, int64_t* d_out_offsets,
                                      int32_t* d_status, dnatok_stream stream);

/* Exclusive scan: d_out_offsets[0] = 0, d_out_offsets[i+1] = sum of d_lengths[0..i]. */
int dnatok_scan_lengths(const int32_t* d_lengths, int64_t n_rows, int64_t* d_out_offsets,
                        dnatok_stream stream);

/* Same path with HOST buffers on device `device`: copies bytes and offsets in, runs the kernels,
 * copies ids / mask / lengths / status back and returns when they are in host memory.  Pinned
 * host buffers make the copies asynchronous; pageable ones work.  ids_capacity counts elements
 * of h_ids (and of h_mask when given).  With fmt->out_stride == -1 rows are padded to the
 * longest row; *out_stride_used receives the stride (or the total id count when ragged). */
int dnatok_encode_host(dnatok_handle* h, int device, const uint8_t* h_bytes,
                       const int64_t* h_offsets, int64_t n_rows, const dnatok_format* fmt,
                       void* h_ids, int64_t ids_capacity, void* h_mask, int32_t* h_lengths,
                       int64_t* h_out_offsets, int32_t* h_status, int64_t* out_stride_used);

/* Fused tokenise -> embedding gather for char / byte-level handles: d_out[row, col, :] =
 * d_weight[id(row, col), :] for the padded layout fmt describes (out_stride > 0; id_bits / mask_bits are
 * not used), without writing the ids.  d_weight is [vocab_rows, row_bytes] bytes per row (any element
 * type; row_bytes a multiple of 16), d_out is [n_rows, out_stride, row_bytes]; both 16-byte aligned.
 * Padding columns read the pad row.  Stands in for the reference's opt-in Triton kernel
 * _fused_tokenize_gather, src/dna_tokenizer.py:3465-3532. */
int dnatok_embed(dnatok_handle* h, const uint8_t* d_bytes, const int64_t* d_offsets, int64_t n_rows,
                 int64_t total_bytes, const dnatok_format* fmt, const void* d_weight, int64_t vocab_rows,
                 int64_t row_bytes, void* d_out, int32_t* d_lengths, int32_t* d_status, dnatok_stream stream);

/* Host packing of FASTA text into the (bytes, offsets) layout the encode entry points take: header
 * lines ('>' or ';') start a record, sequence lines are joined without their line ends.  Call once
 * with out_bytes == NULL to get *n_records and *n_bytes, then with buffers of n_bytes bytes and
 * n_records + 1 offsets.  Stands in for the reference's per-string packing loops
 * (src/dna_tokenizer.py:2594-2651, src/dnatok_bpe_kernel/dnatok_bpe.cu:872-887), which start from
 * Python strings. */
int dnatok_pack_fasta(const char* text, int64_t n_text, uint8_t* out_bytes, int64_t bytes_capacity,
                      int64_t* out_offsets, int64_t offsets_capacity, int64_t* n_records, int64_t* n_bytes);

/* Process-wide tuning knobs (no reference counterpart):
 *   "host_chunk_bytes"      bytes over the host link (input + output) per chunk when dnatok_encode_host splits a
 *                           fixed-stride batch into chunks whose copies in the two directions and kernels overlap;
 *                           0 disables splitting (default 64 MiB)
 *   "host_chunk_threshold"  only batches at least this large are split (default 128 MiB)
 *   "host_mask_threads"     dnatok_encode_host, padded output with a mask of 16 MiB or more: the mask is written by
 *                           this many host threads (non-temporal stores) while the ids are copied back, instead of
 *                           being produced on the GPU and copied too (-1, default: one per core, at most 4: two keep up
 *                           with the link, more only compete with the copies for the host's memory; 0: always copy the
 *                           mask from the device)
 *   "host_mask_early"       1 (default): when every row's length follows from its byte count (per-character tables; k-mer
 *                           rows with at least as many complete windows as tokens are kept) the mask is written without
 *                           waiting for the GPU, whose lengths are compared afterwards; 0: always wait for them
 *   "host_mask_min_bytes"   the size from which a mask is written by host threads (default 16 MiB)
 *   "kmer_force_segments"   1: use the k-mer segment encoder whenever scratch and a status array are given, whatever
 *                           the batch shape
 *   "kmer_poll_limit"       polls after which a k-mer row segment stops waiting for the segment before it and the row
 *                           gets DNATOK_ROW_STALLED (default 2^20, about 70 ms)
 *   "kmer_test_withhold_ticket"  for tests of that path: the segment with this ticket number (segment * n_rows + row)
 *                           publishes nothing, so the segments after it in its row give up; -1 (default): none
 *   "kmer_overlap_launch"   1 (default): the k-mer row kernel is launched with programmatic stream serialisation, so
 *                           its blocks can be placed while the launch before it in the stream drains (they wait for
 *                           that launch to complete before touching memory); 0: plain launch
 *   "emit_overlap_launch"   the same for the padded output kernel of the per-character path (default 1)
 *   "bpe_team_warps"        BPE: warps that work on one word (power of two up to 32; a word never gets fewer
 *                           than its length needs); 0 (default): chosen from the batch - the widest team that
 *                           keeps all words resident on half of the GPU and leaves a lane four positions
 *   "bpe_team_max"          widest team the automatic choice takes (default 8)
 *   "bpe_overlap_launch"    1 (default): the BPE kernel with the merge table in shared memory is launched with programmatic
 *                           stream serialisation (as "kmer_overlap_launch"); a batch of one length class that fits the
 *                           grid in one go is launched without a work counter, so nothing is zeroed between two encodes
 *   "bpe_smem_table"        1 (default): a vocabulary whose packed merge table fits into shared memory beside the
 *                           words in flight (about 75 KB: vocabularies of a few thousand tokens) is looked up there;
 *                           0: always in global memory
 *   "bpe_fused_output"      1 (default): dnatok_encode with a padded layout lets the BPE merge kernels write ids and
 *                           mask in their final place (one launch for a batch of one length class); 0: merged tokens
 *                           go to the scratch buffer and an output pass follows, as dnatok_prepare + dnatok_write do
 *   "bpe_mixed_launch"      1 (default): the rows of all length classes up to 16,384 bytes go through one launch
 *                           whose blocks work from the longest class down; 0: one launch per class
 *   "bpe_block_team_rows"   older switch, kept for tests: batches of at most this many rows use teams of eight
 *                           warps, larger ones a warp per word; -1 (default): the automatic choice above */
int dnatok_set_option(const char* name, int64_t value);

/* Number of kernels this library has launched from the calling process (for accounting). */
int64_t dnatok_launch_count(void);

/* Bytes the calling thread's last dnatok_encode_host copied host -> device and device ->
 * host.  With "host_mask_threads" active the mask of a large padded batch is not among them: host
 * threads write it from the row lengths the GPU returned.  No reference counterpart. */
void dnatok_host_copy_bytes(int64_t* h2d, int64_t* d2h);

#ifdef __cplusplus
}
#endif
#endif /* DNATOK_B200_H */

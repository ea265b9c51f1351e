// Host-side construction of the BPE merge table the kernels read.
//
// The table is a perfect hash of the pair (left id, right id) by row displacement: every left
// token `a` owns a row offset disp[a]; the pair (a, b) lives in slots[disp[a] + b], a 64-bit
// entry: low word (rank << 16) | created id, high word (a << 16) | future rank.  A lookup is two
// dependent loads and an equality test, with no probing and no false positives, and brings
// everything a merge needs.  Ids are Hugging Face ids, so the kernels emit final ids with no remap.
// (The reference keeps a cuco::static_map keyed by a 64-bit pair and remaps kernel ids to HF
// ids afterwards: src/dnatok_bpe_kernel/dnatok_bpe.cu:123-132,761-791,822-837 and
// src/gputok_bpe_backend.py:447-466.)
#pragma once
#include <stdint.h>
#include <string>
#include <vector>

namespace dnatok {

struct BpeHostTable {
    std::vector<uint32_t> disp;        // [n_tokens + 1]; the last entry belongs to the filler id n_tokens, which no pair contains
    std::vector<uint64_t> slots;       // [max disp + n_tokens]; low 32 bits (rank << 16) | created id, high 32 bits
                                       // (a << 16) | future rank (rank + 1 when the table is not batch-safe); all ones when empty
    std::vector<uint16_t> merge_out;   // [n_merges] id created by each rank
    std::vector<uint16_t> future;      // [n_merges] lowest rank of any pair containing that id, 0xFFFF if none
    std::vector<uint64_t> hot;         // [32 * 32] pairs of ids < 32: low word as in slots, high word (future rank << 16) | rank; all ones if no merge
    uint32_t hot_ranks = 0;            // every rank below this creates an id < 32
    bool bytes_hot = false;            // every initial symbol is an id < 32
    std::vector<uint16_t> byte_tok;    // [256] initial symbol of each byte
    // The same table packed for a kernel that keeps it in shared memory (empty when an id or a displacement does
    // not fit 16 bits): 16-bit displacements [n_tokens + 1], then 32-bit slots (left id << 16) | rank up to the last
    // used one plus one empty slot (larger indices are clamped to it), then one word per rank,
    // (future rank << 16) | created id.  compact_slot / compact_info are the byte offsets of the second and
    // third part (multiples of 16).
    std::vector<uint8_t> compact;
    uint32_t compact_slot = 0, compact_info = 0, compact_last = 0;   // compact_last: index of the empty last slot
    uint32_t n_tokens = 0;
    uint32_t n_merges = 0;
    // True when every merge's operands are created by lower ranks (or are initial symbols).
    // Then a pair that contains a freshly created token always ranks above the merge that
    // created it, `future` bounds what a round may create, and many ranks can be merged in one
    // round.  Otherwise the kernel merges one pair per round.
    bool batch_safe = false;
};

// Returns 0, or a negative code with a message in *err.
int build_bpe_table(const int32_t* merge_a, const int32_t* merge_b, const int32_t* merge_out,
                    int32_t n_merges, const int32_t byte_ids[256], BpeHostTable* out, std::string* err);

}  // namespace dnatok

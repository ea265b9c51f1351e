#include "bpe_table.h"

#include <algorithm>
#include <unordered_set>

namespace dnatok {

int build_bpe_table(const int32_t* a, const int32_t* b, const int32_t* o, int32_t n,
                    const int32_t byte_ids[256], BpeHostTable* t, std::string* err) {
    if (n <= 0 || n > 65534) { *err = "number of merges must be in 1..65534"; return -3; }
    uint32_t max_id = 0;
    for (int i = 0; i < 256; ++i) {
        if (byte_ids[i] < 0 || byte_ids[i] > 65534) { *err = "byte id outside 0..65534"; return -3; }
        max_id = std::max<uint32_t>(max_id, (uint32_t)byte_ids[i]);
    }
    for (int32_t r = 0; r < n; ++r) {
        if (a[r] < 0 || b[r] < 0 || o[r] < 0 || a[r] > 65534 || b[r] > 65534 || o[r] > 65534) {
            *err = "token id outside 0..65534 (ids are held in 16 bits)"; return -3;
        }
        max_id = std::max<uint32_t>(max_id, (uint32_t)std::max(a[r], std::max(b[r], o[r])));
    }
    const uint32_t n_tokens = max_id + 1;

    // Each rank must create a token no other rank creates, and no pair may appear twice:
    // Hugging Face validates a queue entry by the id it creates, which only coincides with
    // "the pair is unchanged" under these two conditions.
    std::vector<int32_t> created(n_tokens, -2);          // -2 never, -1 initial symbol, else rank
    for (int i = 0; i < 256; ++i) created[byte_ids[i]] = -1;
    std::unordered_set<uint64_t> seen;
    seen.reserve((size_t)n * 2);
    for (int32_t r = 0; r < n; ++r) {
        if (created[o[r]] != -2) { *err = "two merges (or a merge and an initial symbol) create the same token"; return -3; }
        created[o[r]] = r;
        if (!seen.insert(((uint64_t)a[r] << 32) | (uint32_t)b[r]).second) { *err = "a pair appears twice in the merges"; return -3; }
    }
    bool safe = true;
    for (int32_t r = 0; r < n && safe; ++r) {
        const int32_t ca = created[a[r]], cb = created[b[r]];
        if (ca == -2 || cb == -2 || ca >= r || cb >= r) safe = false;
    }

    // Row displacement, largest rows first, first fit.
    std::vector<std::vector<std::pair<uint32_t, uint32_t>>> rows(n_tokens);   // a -> (b, rank)
    for (int32_t r = 0; r < n; ++r) rows[a[r]].push_back({(uint32_t)b[r], (uint32_t)r});
    std::vector<uint32_t> order;
    for (uint32_t i = 0; i < n_tokens; ++i) if (!rows[i].empty()) order.push_back(i);
    std::stable_sort(order.begin(), order.end(), [&](uint32_t x, uint32_t y) { return rows[x].size() > rows[y].size(); });

    std::vector<uint32_t> slots((size_t)n_tokens, 0xFFFFFFFFu);      // low words first; widened below
    std::vector<uint32_t> disp(n_tokens, 0);
    size_t first_free = 0;
    for (uint32_t ai : order) {
        auto& row = rows[ai];
        uint32_t min_b = row[0].first;
        for (auto& e : row) min_b = std::min(min_b, e.first);
        while (first_free < slots.size() && slots[first_free] != 0xFFFFFFFFu) ++first_free;
        size_t d = first_free > min_b ? first_free - min_b : 0;
        for (;; ++d) {
            bool ok = true;
            for (auto& e : row) {
                const size_t s = d + e.first;
                if (s < slots.size() && slots[s] != 0xFFFFFFFFu) { ok = false; break; }
            }
            if (ok) break;
        }
        size_t need = d + n_tokens + 1;       // any b <= n_tokens (the kernels' filler id) must index inside the array
        if (need > slots.size()) slots.resize(need, 0xFFFFFFFFu);
        for (auto& e : row) slots[d + e.first] = (ai << 16) | e.second;
        disp[ai] = (uint32_t)d;
    }

    disp.push_back(0);                        // the filler id: no slot carries it as left id
    if (slots.size() < (size_t)n_tokens + 1) slots.resize((size_t)n_tokens + 1, 0xFFFFFFFFu);
    t->disp.swap(disp);
    t->merge_out.resize(n);
    for (int32_t r = 0; r < n; ++r) t->merge_out[r] = (uint16_t)o[r];
    t->future.assign(n, 0xFFFFu);
    for (int32_t r = 0; r < n; ++r) {
        for (int32_t x : {a[r], b[r]}) {
            const int32_t c = created[x];
            if (c >= 0 && (uint32_t)r < t->future[c]) t->future[c] = (uint16_t)r;
        }
    }
    auto entry = [&](int32_t r) {
        // without usable future ranks (not batch-safe) the bound is "just above this rank": one rank per round
        const uint64_t f = safe ? (uint64_t)t->future[r] : (uint64_t)r + 1;
        const uint64_t lo = ((uint64_t)r << 16) | (uint64_t)o[r];
        const uint64_t hi = ((uint64_t)a[r] << 16) | f;
        return lo | (hi << 32);
    };
    {
        uint32_t max_disp = 0;
        for (uint32_t d : t->disp) max_disp = std::max(max_disp, d);
        t->compact.clear();
        if (n_tokens + 1 < 0xFFFFu && max_disp <= 0xFFFFu && n > 0) {
            size_t used = 0;
            for (size_t i = 0; i < slots.size(); ++i) if (slots[i] != 0xFFFFFFFFu) used = i + 1;
            auto pad16 = [](size_t x) { return (x + 15) / 16 * 16; };
            const size_t off_slot = pad16(2 * t->disp.size()), off_info = off_slot + pad16(4 * (used + 1));
            t->compact.assign(off_info + pad16(4 * (size_t)n), 0xFF);
            uint16_t* d16 = reinterpret_cast<uint16_t*>(t->compact.data());
            uint32_t* s32 = reinterpret_cast<uint32_t*>(t->compact.data() + off_slot);
            uint32_t* i32 = reinterpret_cast<uint32_t*>(t->compact.data() + off_info);
            for (size_t i = 0; i < t->disp.size(); ++i) d16[i] = (uint16_t)t->disp[i];
            for (size_t i = 0; i < used; ++i) s32[i] = slots[i];
            s32[used] = 0xFFFFFFFFu;
            for (int32_t r = 0; r < n; ++r)
                i32[r] = ((safe ? (uint32_t)t->future[r] : (uint32_t)r + 1u) << 16) | (uint32_t)o[r];
            t->compact_slot = (uint32_t)off_slot;
            t->compact_info = (uint32_t)off_info;
            t->compact_last = (uint32_t)used;
        }
    }
    t->slots.assign(slots.size(), ~0ull);
    for (size_t i = 0; i < slots.size(); ++i)
        if (slots[i] != 0xFFFFFFFFu) t->slots[i] = entry((int32_t)(slots[i] & 0xFFFFu));
    // direct table for pairs of small ids (the initial symbols and the first merges of a trained
    // vocabulary): one shared-memory load answers the whole entry
    t->hot.assign(32 * 32, ~0ull);
    for (int32_t r = 0; r < n; ++r)
        if (a[r] < 32 && b[r] < 32) {
            const uint64_t e = entry(r);
            const uint64_t key = ((e >> 32) & 0xFFFFull) << 16 | (uint64_t)r;      // (F << 16) | rank
            t->hot[a[r] * 32 + b[r]] = (e & 0xFFFFFFFFull) | (key << 32);
        }
    t->bytes_hot = true;
    for (int i = 0; i < 256; ++i) t->bytes_hot = t->bytes_hot && byte_ids[i] < 32;
    t->hot_ranks = (uint32_t)n;
    for (int32_t r = n - 1; r >= 0; --r)
        if (o[r] >= 32) t->hot_ranks = (uint32_t)r;
    t->byte_tok.resize(256);
    for (int i = 0; i < 256; ++i) t->byte_tok[i] = (uint16_t)byte_ids[i];
    t->n_tokens = n_tokens;
    t->n_merges = (uint32_t)n;
    t->batch_safe = safe;
    return 0;
}

}  // namespace dnatok

/* TEST INFRASTRUCTURE ONLY - CPU restatement of the three tokenisation paths.
 *
 * Nothing in the shipped library links or calls this file; tests, the smoke check and the
 * CPU-baseline leg of the benchmark use it as the checker.
 *
 * What each function follows:
 *   oracle_char_row   reference src/dna_tokenizer.py:1779-1820 (_encode_batch_ascii_lut_numpy):
 *                     ids[t] = lut[byte[t]].
 *   oracle_kmer_row   reference src/dna_tokenizer.py:1369-1474 (_encode_batch_kmer_numpy_partial)
 *                     and :1896-1953 (_encode_kmer_fallback_from_lut), restricted to the
 *                     window-aligned vocabulary: a full window of k ACGT characters is one id,
 *                     any other window and the len%k tail expand to single-character ids.
 *   oracle_bpe_word   the merge loop of Hugging Face `tokenizers` 0.22 (third-party, Rust,
 *                     not vendored in the reference; pinned tokenizers==0.22.1 in
 *                     docker/requirements.txt:13): models/bpe/word.rs `Word::merge_all` -
 *                     a priority queue of (rank, position) entries, lowest rank first and
 *                     leftmost first within a rank; an entry is stale when the pair now at its
 *                     position no longer produces the recorded new id.  The reference's own
 *                     kernel states the same rule at src/dnatok_bpe_kernel/dnatok_bpe.cu:3-5.
 *   oracle_bpe_word_naive  the definition itself (rescan for the lowest-rank leftmost pair
 *                     after every single merge); used to cross-check the queue version.
 *
 * Rows are emitted as ragged id lists (content tokens only); special tokens, truncation,
 * padding and masks are composed in oracle/oracle.py following HF's post-processor rules.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ char / byte */

int64_t oracle_char_row(const uint8_t* s, int64_t n, const int32_t* lut, int32_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = lut[s[i]];
    return n;
}

/* ------------------------------------------------------------------ k-mer */

static inline int base_code(uint8_t c) {
    switch (c) { case 'A': return 0; case 'C': return 1; case 'G': return 2; case 'T': return 3; }
    return -1;
}

int64_t oracle_kmer_row(const uint8_t* s, int64_t n, int k, const int32_t* kmer_ids,
                        const int32_t* single_ids, int32_t* out) {
    int64_t m = 0;
    for (int64_t w = 0; w < n; w += k) {
        int64_t len = n - w < k ? n - w : k;
        int clean = (len == k);
        int64_t idx = 0;
        for (int64_t j = 0; j < len && clean; ++j) {
            int c = base_code(s[w + j]);
            if (c < 0) clean = 0; else idx = idx * 4 + c;
        }
        if (clean) out[m++] = kmer_ids[idx];
        else for (int64_t j = 0; j < len; ++j) out[m++] = single_ids[s[w + j]];
    }
    return m;
}

/* ------------------------------------------------------------------ BPE */

typedef struct {
    int32_t n_merges;
    uint64_t cap;            /* power of two */
    uint64_t* keys;          /* (a << 32) | b, or UINT64_MAX when empty */
    int32_t* rank;
    int32_t* new_id;
} oracle_bpe_table;

static inline uint64_t mix64(uint64_t x) {
    x ^= x >> 33; x *= 0xff51afd7ed558ccdULL; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ULL; x ^= x >> 33;
    return x;
}

oracle_bpe_table* oracle_bpe_table_new(const int32_t* a, const int32_t* b, const int32_t* out,
                                       int32_t n) {
    oracle_bpe_table* t = (oracle_bpe_table*)calloc(1, sizeof(*t));
    uint64_t cap = 16;
    while (cap < (uint64_t)n * 2 + 2) cap <<= 1;
    t->n_merges = n; t->cap = cap;
    t->keys = (uint64_t*)malloc(cap * sizeof(uint64_t));
    t->rank = (int32_t*)malloc(cap * sizeof(int32_t));
    t->new_id = (int32_t*)malloc(cap * sizeof(int32_t));
    memset(t->keys, 0xff, cap * sizeof(uint64_t));
    for (int32_t r = 0; r < n; ++r) {
        uint64_t key = ((uint64_t)(uint32_t)a[r] << 32) | (uint32_t)b[r];
        uint64_t h = mix64(key) & (cap - 1);
        int dup = 0;
        while (t->keys[h] != UINT64_MAX) {
            if (t->keys[h] == key) { dup = 1; break; }
            h = (h + 1) & (cap - 1);
        }
        if (dup) { t->rank[h] = r; t->new_id[h] = out[r]; continue; }  /* a repeated pair: the later line wins, as a map insert overwrites */
        t->keys[h] = key; t->rank[h] = r; t->new_id[h] = out[r];
    }
    return t;
}

void oracle_bpe_table_free(oracle_bpe_table* t) {
    if (!t) return;
    free(t->keys); free(t->rank); free(t->new_id); free(t);
}

static inline int bpe_find(const oracle_bpe_table* t, int32_t a, int32_t b, int32_t* rank,
                           int32_t* new_id) {
    uint64_t key = ((uint64_t)(uint32_t)a << 32) | (uint32_t)b;
    uint64_t h = mix64(key) & (t->cap - 1);
    while (t->keys[h] != UINT64_MAX) {
        if (t->keys[h] == key) { *rank = t->rank[h]; *new_id = t->new_id[h]; return 1; }
        h = (h + 1) & (t->cap - 1);
    }
    return 0;
}

typedef struct { int32_t rank, pos, new_id; } qent;

static inline int q_less(const qent* x, const qent* y) {   /* x pops before y */
    return x->rank != y->rank ? x->rank < y->rank : x->pos < y->pos;
}

static void q_push(qent* h, int64_t* n, qent e) {
    int64_t i = (*n)++;
    while (i > 0) {
        int64_t p = (i - 1) >> 1;
        if (!q_less(&e, &h[p])) break;
        h[i] = h[p]; i = p;
    }
    h[i] = e;
}

static qent q_pop(qent* h, int64_t* n) {
    qent top = h[0];
    qent last = h[--(*n)];
    int64_t i = 0, m = *n;
    for (;;) {
        int64_t c = 2 * i + 1;
        if (c >= m) break;
        if (c + 1 < m && q_less(&h[c + 1], &h[c])) ++c;
        if (!q_less(&h[c], &last)) break;
        h[i] = h[c]; i = c;
    }
    if (m > 0) h[i] = last;
    return top;
}

/* One pre-tokenised word: bytes -> initial symbols through byte_ids (an id < 0 is never
 * produced; characters outside the alphabet carry unk_id, which no merge names, so they act
 * as barriers exactly as HF's per-character [UNK] symbols do). */
int64_t oracle_bpe_word(const oracle_bpe_table* t, const uint8_t* s, int64_t n,
                        const int32_t* byte_ids, int32_t* out) {
    if (n <= 0) return 0;
    int32_t* c = (int32_t*)malloc(n * sizeof(int32_t));
    int32_t* prev = (int32_t*)malloc(n * sizeof(int32_t));
    int32_t* next = (int32_t*)malloc(n * sizeof(int32_t));
    uint8_t* live = (uint8_t*)malloc(n);
    qent* heap = (qent*)malloc((size_t)(3 * n + 4) * sizeof(qent));
    int64_t hn = 0;
    for (int64_t i = 0; i < n; ++i) {
        c[i] = byte_ids[s[i]]; prev[i] = (int32_t)i - 1; next[i] = i + 1 < n ? (int32_t)i + 1 : -1; live[i] = 1;
    }
    for (int64_t i = 0; i + 1 < n; ++i) {
        int32_t r, id;
        if (bpe_find(t, c[i], c[i + 1], &r, &id)) { qent e = { r, (int32_t)i, id }; q_push(heap, &hn, e); }
    }
    while (hn > 0) {
        qent top = q_pop(heap, &hn);
        if (!live[top.pos]) continue;
        if (next[top.pos] < 0) continue;
        int32_t np = next[top.pos];
        int32_t r, id;
        if (!bpe_find(t, c[top.pos], c[np], &r, &id) || id != top.new_id) continue;
        c[top.pos] = top.new_id;
        live[np] = 0;
        next[top.pos] = next[np];
        if (next[np] >= 0) prev[next[np]] = top.pos;
        if (prev[top.pos] >= 0) {
            int32_t p = prev[top.pos];
            if (bpe_find(t, c[p], c[top.pos], &r, &id)) { qent e = { r, p, id }; q_push(heap, &hn, e); }
        }
        if (next[top.pos] >= 0) {
            int32_t q = next[top.pos];
            if (bpe_find(t, c[top.pos], c[q], &r, &id)) { qent e = { r, top.pos, id }; q_push(heap, &hn, e); }
        }
    }
    int64_t m = 0;
    for (int64_t i = 0; i < n; ++i) if (live[i]) out[m++] = c[i];
    free(c); free(prev); free(next); free(live); free(heap);
    return m;
}

int64_t oracle_bpe_word_naive(const oracle_bpe_table* t, const uint8_t* s, int64_t n,
                              const int32_t* byte_ids, int32_t* out) {
    int64_t m = n;
    for (int64_t i = 0; i < n; ++i) out[i] = byte_ids[s[i]];
    for (;;) {
        int32_t best = INT32_MAX, best_id = 0; int64_t at = -1;
        for (int64_t i = 0; i + 1 < m; ++i) {
            int32_t r, id;
            if (bpe_find(t, out[i], out[i + 1], &r, &id) && r < best) { best = r; best_id = id; at = i; }
        }
        if (at < 0) break;
        out[at] = best_id;
        memmove(out + at + 1, out + at + 2, (size_t)(m - at - 2) * sizeof(int32_t));
        --m;
    }
    return m;
}

/* ------------------------------------------------------------------ batch driver
 * kind: 0 char, 1 k-mer, 2 BPE.  out holds sum(len) ids in total; row i's tokens are
 * written at out + offsets[i] and its count at counts[i].  n_threads > 1 spreads rows over
 * POSIX threads in blocks of 16 rows taken from a shared counter. */
#include <pthread.h>

typedef struct {
    int kind; const uint8_t* bytes; const int64_t* offsets; int64_t B;
    const int32_t* lut256; int k; const int32_t* kmer_ids; const oracle_bpe_table* t;
    int32_t* out; int64_t* counts; int64_t next;
} batch_job;

static void* batch_worker(void* arg) {
    batch_job* j = (batch_job*)arg;
    for (;;) {
        int64_t lo = __atomic_fetch_add(&j->next, 16, __ATOMIC_RELAXED);
        if (lo >= j->B) break;
        int64_t hi = lo + 16 < j->B ? lo + 16 : j->B;
        for (int64_t i = lo; i < hi; ++i) {
            const uint8_t* s = j->bytes + j->offsets[i];
            int64_t n = j->offsets[i + 1] - j->offsets[i];
            int32_t* o = j->out + j->offsets[i];
            if (j->kind == 0) j->counts[i] = oracle_char_row(s, n, j->lut256, o);
            else if (j->kind == 1) j->counts[i] = oracle_kmer_row(s, n, j->k, j->kmer_ids, j->lut256, o);
            else j->counts[i] = oracle_bpe_word(j->t, s, n, j->lut256, o);
        }
    }
    return 0;
}

void oracle_encode_batch(int kind, const uint8_t* bytes, const int64_t* offsets, int64_t B,
                         const int32_t* lut256, int k, const int32_t* kmer_ids,
                         const oracle_bpe_table* t, int32_t* out, int64_t* counts, int n_threads) {
    batch_job j = { kind, bytes, offsets, B, lut256, k, kmer_ids, t, out, counts, 0 };
    if (n_threads <= 1) { batch_worker(&j); return; }
    if (n_threads > 256) n_threads = 256;
    pthread_t th[256];
    int started = 0;
    for (int i = 0; i < n_threads - 1; ++i)
        if (pthread_create(&th[started], 0, batch_worker, &j) == 0) ++started;
    batch_worker(&j);
    for (int i = 0; i < started; ++i) pthread_join(th[i], 0);
}

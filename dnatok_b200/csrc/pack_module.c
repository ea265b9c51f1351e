/* dnatok_b200._pack - native host packer: list[str] / list[bytes] -> one contiguous ASCII buffer + row offsets.
 *
 * Stands in for the per-call packing of the reference, which joins Python strings and encodes them
 * ("".join(seqs).encode("ascii"), src/dna_tokenizer.py:1795-1800; per-row np.frombuffer loops in
 * encode_batch_to_ascii_bytes, :2594-2651) or copies std::string by std::string into a pinned tensor
 * (src/dnatok_bpe_kernel/dnatok_bpe.cu:872-887).  Here the row pointers and lengths are collected in one
 * pass over the list with the interpreter lock held, and the bytes are then copied by a few threads
 * without it, straight from the string objects into the caller's (pinned) buffer.  The copy can translate
 * every byte through a 256-entry table (upper-casing, mapping characters outside an alphabet to N: the
 * reference's normalize_case / handle_invalid_chars, src/dna_tokenizer.py:1535-1558) and pad every row to
 * a common width with a fill byte on either side (the string padding of encode_batch_with_padding,
 * :2183-2195).
 *
 *   sizes(seqs, offsets, pad_to=0, trunc_to=0) -> total bytes        offsets: writable int64[len(seqs) + 1]
 *   copy(seqs, offsets, out, table=None, pad_to=0, pad_byte=78, pad_left=0, threads=0, trunc_to=0) -> None
 * trunc_to > 0 keeps only the first trunc_to bytes of every row (the s[:max_chars] of :2168-2170).
 */
#define PY_SSIZE_T_CLEAN
#include <Python.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    const unsigned char* src;
    int64_t len;
} row_t;

/* pointer and length of one item; -1 with an exception set when it is neither ASCII str nor bytes */
static int item_view(PyObject* it, row_t* r) {
    if (PyUnicode_Check(it)) {
        if (!PyUnicode_IS_COMPACT_ASCII(it)) {
            PyErr_SetString(PyExc_ValueError, "sequences must be ASCII");
            return -1;
        }
        r->src = (const unsigned char*)PyUnicode_DATA(it);
        r->len = (int64_t)PyUnicode_GET_LENGTH(it);
        return 0;
    }
    if (PyBytes_Check(it)) {
        r->src = (const unsigned char*)PyBytes_AS_STRING(it);
        r->len = (int64_t)PyBytes_GET_SIZE(it);
        return 0;
    }
    if (PyByteArray_Check(it)) {
        r->src = (const unsigned char*)PyByteArray_AS_STRING(it);
        r->len = (int64_t)PyByteArray_GET_SIZE(it);
        return 0;
    }
    PyErr_SetString(PyExc_TypeError, "sequences must be str, bytes or bytearray");
    return -1;
}

static PyObject* pack_sizes(PyObject* self, PyObject* args, PyObject* kw) {
    static char* names[] = {"seqs", "offsets", "pad_to", "trunc_to", NULL};
    PyObject* seqs;
    Py_buffer ob;
    long long pad_to = 0, trunc_to = 0;
    if (!PyArg_ParseTupleAndKeywords(args, kw, "Ow*|LL", names, &seqs, &ob, &pad_to, &trunc_to)) return NULL;
    PyObject* fast = PySequence_Fast(seqs, "seqs must be a sequence");
    if (!fast) { PyBuffer_Release(&ob); return NULL; }
    const Py_ssize_t n = PySequence_Fast_GET_SIZE(fast);
    if (ob.len < (Py_ssize_t)((n + 1) * 8)) {
        PyErr_SetString(PyExc_ValueError, "offsets buffer too small");
        Py_DECREF(fast); PyBuffer_Release(&ob);
        return NULL;
    }
    int64_t* off = (int64_t*)ob.buf;
    int64_t total = 0;
    PyObject** items = PySequence_Fast_ITEMS(fast);
    for (Py_ssize_t i = 0; i < n; ++i) {
        row_t r;
        if (item_view(items[i], &r)) { Py_DECREF(fast); PyBuffer_Release(&ob); return NULL; }
        if (trunc_to > 0 && r.len > trunc_to) r.len = trunc_to;
        off[i] = total;
        total += r.len < pad_to ? pad_to : r.len;
    }
    off[n] = total;
    Py_DECREF(fast);
    PyBuffer_Release(&ob);
    return PyLong_FromLongLong(total);
}

typedef struct {
    const row_t* rows;
    const int64_t* off;
    unsigned char* out;
    const unsigned char* table;
    int64_t pad_to;
    int pad_byte, pad_left;
    Py_ssize_t lo, hi;
} job_t;

static void* copy_rows(void* p);

/* Copy workers that outlive a call: a list is often packed piece by piece (each piece goes onto the link while the
 * next is packed), and starting threads for every piece would cost more than the copy.  run_jobs() hands out the
 * jobs of one call to the workers and the calling thread; one call at a time.  A forked child starts without workers. */
static pthread_mutex_t pool_mu = PTHREAD_MUTEX_INITIALIZER, pool_run_mu = PTHREAD_MUTEX_INITIALIZER;
static pthread_cond_t pool_start = PTHREAD_COND_INITIALIZER, pool_done = PTHREAD_COND_INITIALIZER;
static void* pool_jobs = NULL;
static size_t pool_job_size = 0;
static int pool_n_jobs = 0, pool_next = 0, pool_left = 0, pool_threads = 0, pool_atfork_set = 0;
static unsigned long pool_generation = 0;

static void pool_take_jobs(void) {                 /* called with pool_mu held; returns with it held */
    while (pool_next < pool_n_jobs) {
        void* job = (char*)pool_jobs + pool_job_size * (size_t)pool_next++;
        pthread_mutex_unlock(&pool_mu);
        copy_rows(job);
        pthread_mutex_lock(&pool_mu);
        if (--pool_left == 0) pthread_cond_broadcast(&pool_done);
    }
}

static void* pool_worker(void* unused) {
    unsigned long seen = 0;
    (void)unused;
    pthread_mutex_lock(&pool_mu);
    for (;;) {
        while (seen == pool_generation) pthread_cond_wait(&pool_start, &pool_mu);
        seen = pool_generation;
        pool_take_jobs();
    }
    return NULL;
}

static void pool_child(void) {                     /* after fork(): the child has none of the threads */
    pthread_mutex_init(&pool_mu, NULL);
    pthread_mutex_init(&pool_run_mu, NULL);
    pthread_cond_init(&pool_start, NULL);
    pthread_cond_init(&pool_done, NULL);
    pool_threads = 0; pool_n_jobs = 0; pool_next = 0; pool_left = 0;
}

static void run_jobs(void* jobs, size_t job_size, int n) {
    pthread_mutex_lock(&pool_run_mu);
    pthread_mutex_lock(&pool_mu);
    if (!pool_atfork_set) { pthread_atfork(NULL, NULL, pool_child); pool_atfork_set = 1; }
    while (pool_threads < n - 1) {
        pthread_t th;
        if (pthread_create(&th, NULL, pool_worker, NULL)) break;       /* fewer workers: the caller does more itself */
        pthread_detach(th);
        ++pool_threads;
    }
    pool_jobs = jobs; pool_job_size = job_size; pool_n_jobs = n; pool_next = 0; pool_left = n;
    ++pool_generation;
    pthread_cond_broadcast(&pool_start);
    pool_take_jobs();
    while (pool_left > 0) pthread_cond_wait(&pool_done, &pool_mu);
    pool_n_jobs = 0;
    pthread_mutex_unlock(&pool_mu);
    pthread_mutex_unlock(&pool_run_mu);
}

static void* copy_rows(void* p) {
    const job_t* j = (const job_t*)p;
    for (Py_ssize_t i = j->lo; i < j->hi; ++i) {
        const row_t r = j->rows[i];
        unsigned char* dst = j->out + j->off[i];
        const int64_t width = j->off[i + 1] - j->off[i];
        const int64_t fill = width - r.len;                 /* > 0 only with pad_to */
        unsigned char* body = dst + (j->pad_left ? fill : 0);
        if (fill > 0) memset(j->pad_left ? dst : dst + r.len, j->pad_byte, (size_t)fill);
        if (j->table) {
            for (int64_t k = 0; k < r.len; ++k) body[k] = j->table[r.src[k]];
        } else {
            memcpy(body, r.src, (size_t)r.len);
        }
    }
    return NULL;
}

static PyObject* pack_copy(PyObject* self, PyObject* args, PyObject* kw) {
    static char* names[] = {"seqs", "offsets", "out", "table", "pad_to", "pad_byte", "pad_left", "threads", "trunc_to", NULL};
    PyObject *seqs, *table_obj = Py_None;
    Py_buffer ob, outb, tb;
    long long pad_to = 0, trunc_to = 0;
    int pad_byte = 'N', pad_left = 0, threads = 0;
    if (!PyArg_ParseTupleAndKeywords(args, kw, "Oy*w*|OLiiiL", names, &seqs, &ob, &outb, &table_obj, &pad_to, &pad_byte,
                                     &pad_left, &threads, &trunc_to))
        return NULL;
    int have_table = 0;
    PyObject* fast = NULL;
    row_t* rows = NULL;
    PyObject* result = NULL;
    if (table_obj != Py_None) {
        if (PyObject_GetBuffer(table_obj, &tb, PyBUF_SIMPLE)) goto done;
        have_table = 1;
        if (tb.len != 256) { PyErr_SetString(PyExc_ValueError, "table must hold 256 bytes"); goto done; }
    }
    fast = PySequence_Fast(seqs, "seqs must be a sequence");
    if (!fast) goto done;
    {
        const Py_ssize_t n = PySequence_Fast_GET_SIZE(fast);
        if (ob.len < (Py_ssize_t)((n + 1) * 8)) { PyErr_SetString(PyExc_ValueError, "offsets buffer too small"); goto done; }
        const int64_t* off = (const int64_t*)ob.buf;
        rows = (row_t*)malloc(sizeof(row_t) * (size_t)(n > 0 ? n : 1));
        if (!rows) { PyErr_NoMemory(); goto done; }
        PyObject** items = PySequence_Fast_ITEMS(fast);
        for (Py_ssize_t i = 0; i < n; ++i) {
            if (item_view(items[i], &rows[i])) goto done;
            if (trunc_to > 0 && rows[i].len > trunc_to) rows[i].len = trunc_to;
            const int64_t want = rows[i].len < pad_to ? pad_to : rows[i].len;
            if (off[i + 1] - off[i] != want) { PyErr_SetString(PyExc_ValueError, "offsets do not match the sequences"); goto done; }
        }
        const int64_t total = n ? off[n] : 0;
        if (outb.len < (Py_ssize_t)total) { PyErr_SetString(PyExc_ValueError, "output buffer too small"); goto done; }
        if (threads <= 0) threads = total >= (8 << 20) ? 8 : 1;
        if (threads > 64) threads = 64;
        if ((Py_ssize_t)threads > n) threads = n > 0 ? (int)n : 1;
        job_t jobs[64];
        /* rows are dealt to the threads in contiguous ranges of about equal bytes */
        Py_ssize_t lo = 0;
        for (int t = 0; t < threads; ++t) {
            const int64_t upto = total * (t + 1) / threads;
            Py_ssize_t hi = lo;
            while (hi < n && (t == threads - 1 || off[hi + 1] <= upto)) ++hi;
            if (t == threads - 1) hi = n;
            jobs[t] = (job_t){rows, off, (unsigned char*)outb.buf, have_table ? (const unsigned char*)tb.buf : NULL,
                              pad_to, pad_byte, pad_left, lo, hi};
            lo = hi;
        }
        Py_BEGIN_ALLOW_THREADS
        if (threads <= 1) copy_rows(&jobs[0]);
        else run_jobs(jobs, sizeof(job_t), threads);
        Py_END_ALLOW_THREADS
        result = Py_None;
        Py_INCREF(result);
    }
done:
    free(rows);
    Py_XDECREF(fast);
    if (have_table) PyBuffer_Release(&tb);
    PyBuffer_Release(&ob);
    PyBuffer_Release(&outb);
    return result;
}

static PyMethodDef methods[] = {
    {"sizes", (PyCFunction)(void (*)(void))pack_sizes, METH_VARARGS | METH_KEYWORDS,
     "sizes(seqs, offsets, pad_to=0) -> total: fill int64 offsets[len(seqs) + 1] and return the packed size"},
    {"copy", (PyCFunction)(void (*)(void))pack_copy, METH_VARARGS | METH_KEYWORDS,
     "copy(seqs, offsets, out, table=None, pad_to=0, pad_byte=78, pad_left=0, threads=0): copy the rows into out"},
    {NULL, NULL, 0, NULL}};

static struct PyModuleDef moddef = {PyModuleDef_HEAD_INIT, "_pack", "native host packer of dnatok_b200", -1, methods};

PyMODINIT_FUNC PyInit__pack(void) { return PyModule_Create(&moddef); }

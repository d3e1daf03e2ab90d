// Layer 1 of the C ABI: entry points that take COMET's host memref descriptors.
// Each one stages its operands into device memory on the library stream, calls
// the device-pointer entry point, copies the results back into the caller's
// memrefs and synchronises, so the generated host code that follows (printing,
// ta.reduce, the next ta.mul) sees finished host arrays, as it does after the
// loops COMET generates today.
#include <string.h>

#include <mutex>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "comm.cuh"
#include "hostcopy.cuh"

extern "C" {
// device-pointer layer (declared in include/comet_b200.h)
}

namespace cb200 {

// Bytes per VALUE in the host memrefs of the running entry point: 8 for the _f64_ symbols, 4 for the _f32_
// ones (COMET instantiates both, lib/ExecutionEngine/SparseUtils.cpp:2354-2400).  float values are widened to
// double on the device after the upload and results narrowed before the download, so both widths run the
// same (double) kernels; a float result is the correctly rounded double result.
static thread_local int g_vsz = 8;
struct ValueWidth {
    int old;
    explicit ValueWidth(int v) : old(g_vsz) { g_vsz = v; }
    ~ValueWidth() { g_vsz = old; }
};

struct Arr {   // a 1-D host memref
    void *data;
    int64_t n;
};

static int get1d(const char *what, int64_t rank, void *desc, size_t elem, Arr *out)
{
    out->data = nullptr;
    out->n = 0;
    if (!desc) return 0;
    if (rank != 1) return fail("%s: expected a rank-1 memref, got rank %lld", what, (long long)rank);
    comet_b200_memref1d *m = (comet_b200_memref1d *)desc;
    if (m->sizes[0] < 0) return fail("%s: negative size", what);
    if (m->sizes[0] > 1 && m->strides[0] != 1) return fail("%s: stride must be 1", what);
    out->data = (char *)m->aligned + m->offset * (int64_t)elem;
    out->n = m->sizes[0];
    return 0;
}

struct Mat {   // a 2-D host memref
    double *data;
    int64_t rows, cols, s0, s1;
};

static int get2d(const char *what, int64_t rank, void *desc, Mat *out)
{
    if (!desc || rank != 2) return fail("%s: expected a rank-2 memref", what);
    comet_b200_memref2d *m = (comet_b200_memref2d *)desc;
    out->data = (double *)((char *)m->aligned + m->offset * (int64_t)g_vsz);
    out->rows = m->sizes[0];
    out->cols = m->sizes[1];
    out->s0 = m->strides[0];
    out->s1 = m->strides[1];
    if (out->rows < 0 || out->cols < 0) return fail("%s: negative size", what);
    return 0;
}

enum { F_CSR, F_DCSR, F_COO };

struct HostSparse {
    int fmt;
    int isz;                              // bytes per index: 8 (_i64 entry points) or 4 (_i32)
    int64_t nrows, ncols, nnz, nstored;   // nstored: rows held (DCSR), else nrows
    char *a1pos, *a1crd, *a2pos, *a2crd;  // index arrays of `isz`-byte integers
    double *val;
};

static inline int64_t idx_get(const char *p, int64_t i, int isz)
{
    return isz == 8 ? ((const int64_t *)p)[i] : (int64_t)((const int32_t *)p)[i];
}

static inline void idx_set(char *p, int64_t i, int isz, int64_t v)
{
    if (isz == 8) ((int64_t *)p)[i] = v; else ((int32_t *)p)[i] = (int32_t)v;
}

#define SPARSE_ARGS(P) P##1format, P##2format, P##1pos_rank, P##1pos_ptr, P##1crd_rank, P##1crd_ptr, \
    P##2pos_rank, P##2pos_ptr, P##2crd_rank, P##2crd_ptr, P##val_rank, P##val_ptr, P##dims_rank, P##dims_ptr

static int get_sparse(const char *what, int isz, int32_t f1, int32_t f2, int64_t r1p, void *p1p, int64_t r1c,
                      void *p1c, int64_t r2p, void *p2p, int64_t r2c, void *p2c, int64_t rv, void *pv,
                      int64_t rd, void *pd, HostSparse *s)
{
    Arr a1pos, a1crd, a2pos, a2crd, val, dims;
    s->isz = isz;
    CB_TRY(get1d(what, r1p, p1p, isz, &a1pos));
    CB_TRY(get1d(what, r1c, p1c, isz, &a1crd));
    CB_TRY(get1d(what, r2p, p2p, isz, &a2pos));
    CB_TRY(get1d(what, r2c, p2c, isz, &a2crd));
    CB_TRY(get1d(what, rv, pv, g_vsz, &val));
    CB_TRY(get1d(what, rd, pd, 8, &dims));
    if (dims.n < 2 || !dims.data) return fail("%s: dims memref must hold {rows, cols}", what);
    s->nrows = ((int64_t *)dims.data)[0];
    s->ncols = ((int64_t *)dims.data)[1];
    if (s->nrows < 0 || s->ncols < 0) return fail("%s: negative dimension", what);
    s->a1pos = (char *)a1pos.data; s->a1crd = (char *)a1crd.data;
    s->a2pos = (char *)a2pos.data; s->a2crd = (char *)a2crd.data;
    s->val = (double *)val.data;
    if (f1 == COMET_B200_FMT_DENSE && f2 == COMET_B200_FMT_CU) {
        s->fmt = F_CSR;
        if (a2pos.n < s->nrows + 1) return fail("%s: CSR pos array shorter than rows+1", what);
        s->nstored = s->nrows;
        s->nnz = s->nrows > 0 ? idx_get(s->a2pos, s->nrows, isz) : 0;
    } else if (f1 == COMET_B200_FMT_CU && f2 == COMET_B200_FMT_CU) {
        s->fmt = F_DCSR;
        if (a1pos.n < 2) return fail("%s: DCSR A1pos must hold {0, stored rows}", what);
        s->nstored = idx_get(s->a1pos, 1, isz) - idx_get(s->a1pos, 0, isz);
        if (idx_get(s->a1pos, 0, isz) != 0) return fail("%s: DCSR A1pos[0] must be 0", what);
        if (a1crd.n < s->nstored || a2pos.n < s->nstored + 1)
            return fail("%s: DCSR arrays shorter than the stored row count", what);
        s->nnz = s->nstored > 0 ? idx_get(s->a2pos, s->nstored, isz) : 0;
    } else if (f1 == COMET_B200_FMT_CN && f2 == COMET_B200_FMT_S) {
        s->fmt = F_COO;
        if (a1pos.n < 2) return fail("%s: COO A1pos must hold {0, nnz}", what);
        if (idx_get(s->a1pos, 0, isz) != 0) return fail("%s: COO A1pos[0] must be 0", what);
        s->nnz = idx_get(s->a1pos, 1, isz);
        s->nstored = s->nrows;
        if (a1crd.n < s->nnz) return fail("%s: COO row coordinates shorter than nnz", what);
    } else {
        return fail("%s: unsupported format (%d, %d); CSR, DCSR and COO are handled", what, f1, f2);
    }
    if (s->nnz < 0) return fail("%s: negative nnz", what);
    if (a2crd.n < s->nnz || val.n < s->nnz) return fail("%s: crd/val arrays shorter than nnz", what);
    // The kernels trust the row pointer: check on the host that it starts at 0 and never decreases
    // (one pass over rows+1 integers), so that a malformed descriptor -- e.g. 32-bit arrays handed to
    // the 64-bit entry point -- is refused here instead of sending a kernel out of bounds.
    if (s->fmt != F_COO && s->nstored > 0) {
        int64_t prev = idx_get(s->a2pos, 0, isz);
        if (prev != 0) return fail("%s: pos[0] must be 0 (got %lld)", what, (long long)prev);
        for (int64_t i = 1; i <= s->nstored; i++) {
            const int64_t cur = idx_get(s->a2pos, i, isz);
            if (cur < prev) return fail("%s: pos decreases at row %lld (wrong index width?)", what, (long long)(i - 1));
            prev = cur;
        }
    }
    return 0;
}

// Device allocations of one call; freed (stream-ordered) when the object dies
// unless released to a longer-lived owner.
struct DevBag {
    cudaStream_t st;
    std::vector<void *> ptrs;
    explicit DevBag(cudaStream_t s) : st(s) {}
    ~DevBag() { for (void *p : ptrs) cudaFreeAsync(p, st); }
    int alloc(void **p, size_t bytes)
    {
        if (bytes == 0) bytes = 8;
        cudaError_t e = cudaMallocAsync(p, bytes, st);
        if (e != cudaSuccess) {
            *p = nullptr;
            return fail("device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
        }
        ptrs.push_back(*p);
        return 0;
    }
    int upload(void **p, const void *host, size_t bytes)
    {
        CB_TRY(alloc(p, bytes));
        if (bytes) CB_TRY(h2d(*p, host, bytes, st));
        return 0;
    }
    // An array every rank needs whole (the replicated operand of a sharded call): without a
    // communicator it is uploaded as it is; with one, this rank uploads slice number `rank` of it and
    // the slices are exchanged between the GPUs, so each PCIe link carries one N-th of the bytes.
    // Every rank must pass the same host contents.
    int upload_rep(void **p, const void *host, size_t bytes, Comm *cm)
    {
        if (!cm || cm->nranks == 1) return upload(p, host, bytes);
        const size_t s = comm_slice_bytes(bytes, cm->nranks);
        CB_TRY(alloc(p, s * (size_t)cm->nranks));
        const size_t lo = s * (size_t)cm->rank;
        if (lo < bytes) {
            const size_t n = bytes - lo < s ? bytes - lo : s;
            CB_TRY(h2d((char *)*p + lo, (const char *)host + lo, n, st));
        }
        return comm_allgather_inplace(cm, *p, s, st);
    }
    // n VALUES of the entry point's width -> double on the device
    int upload_val(double **p, const void *host, size_t n, Comm *cm = nullptr)
    {
        if (g_vsz == 8) return upload_rep((void **)p, host, n * 8, cm);
        void *narrow = nullptr;
        CB_TRY(upload_rep(&narrow, host, n * 4, cm));
        CB_TRY(alloc((void **)p, n * 8));
        return widen_f32_to_f64((const float *)narrow, *p, (int64_t)n, st);
    }
    // n doubles on the device -> VALUES of the entry point's width in the host array
    int download_val(void *host, const double *dev, size_t n)
    {
        if (n == 0) return 0;
        if (g_vsz == 8) return d2h(host, dev, n * 8, st);
        float *narrow = nullptr;
        CB_TRY(alloc((void **)&narrow, n * 4));
        CB_TRY(narrow_f64_to_f32(dev, narrow, (int64_t)n, st));
        return d2h(host, narrow, n * 4, st);
    }
    // n indices of isz bytes -> int64 on the device (int32 input is widened there, not on the host)
    int upload_idx(int64_t **p, const void *host, int64_t n, int isz, Comm *cm = nullptr)
    {
        if (isz == 8) return upload_rep((void **)p, host, (size_t)n * 8, cm);
        void *narrow = nullptr;
        CB_TRY(upload_rep(&narrow, host, (size_t)n * 4, cm));
        CB_TRY(alloc((void **)p, (size_t)n * 8));
        return widen_i32_to_i64((const int32_t *)narrow, *p, n, st);
    }
};

struct DevSparse {
    int64_t nrows_k;          // rows the kernels iterate over (stored rows for DCSR)
    int64_t *row_ids;         // DCSR row coordinates or null
    int64_t *pos, *crd, *rows;
    double *val;
};

static int pool_keep()
{
    static bool done[64] = {false};
    int d = 0;
    CB_CUDA(cudaGetDevice(&d));
    if (d >= 0 && d < 64 && !done[d]) {
        cudaMemPool_t pool;
        CB_CUDA(cudaDeviceGetDefaultMemPool(&pool, d));
        uint64_t keep = ~(uint64_t)0;
        CB_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
        done[d] = true;
    }
    return 0;
}

// Uploads a sparse operand; for COO it also derives the row pointer on the device.  The column
// coordinates (and DCSR's row coordinates) are range-checked on the device and the stream is
// synchronised, so a coordinate outside the matrix is reported here, before any kernel that gathers
// through it has been launched.
static int upload_sparse(const char *what, const HostSparse &h, DevBag &bag, DevSparse *d,
                         bool need_val = true, Comm *rep = nullptr)
{
    memset(d, 0, sizeof(*d));
    cudaStream_t st = bag.st;
    CB_TRY(bag.upload_idx(&d->crd, h.a2crd, h.nnz, h.isz, rep));
    if (need_val) CB_TRY(bag.upload_val(&d->val, h.val, (size_t)h.nnz, rep));
    int *flags = nullptr;                     // [0] coordinates in range, [1] COO rows ascending and in range
    CB_TRY(bag.alloc((void **)&flags, 2 * sizeof(int)));
    int got[2] = {1, 1};
    CB_CUDA(cudaMemcpyAsync(flags, got, sizeof(got), cudaMemcpyHostToDevice, st));
    CB_TRY(check_index_range(d->crd, h.nnz, h.ncols, flags, st));
    if (h.fmt == F_CSR) {
        d->nrows_k = h.nrows;
        CB_TRY(bag.upload_idx(&d->pos, h.a2pos, h.nrows + 1, h.isz, rep));
    } else if (h.fmt == F_DCSR) {
        d->nrows_k = h.nstored;
        CB_TRY(bag.upload_idx(&d->pos, h.a2pos, h.nstored + 1, h.isz, rep));
        CB_TRY(bag.upload_idx(&d->row_ids, h.a1crd, h.nstored, h.isz, rep));
        CB_TRY(check_index_range(d->row_ids, h.nstored, h.nrows, flags, st));
    } else {
        d->nrows_k = h.nrows;
        CB_TRY(bag.upload_idx(&d->rows, h.a1crd, h.nnz, h.isz, rep));
        CB_TRY(bag.alloc((void **)&d->pos, (size_t)(h.nrows + 1) * 8));
        CB_TRY(coo_rows_to_pos(d->rows, h.nnz, h.nrows, d->pos, flags + 1, st));
    }
    CB_CUDA(cudaMemcpyAsync(got, flags, sizeof(got), cudaMemcpyDeviceToHost, st));
    CB_CUDA(cudaStreamSynchronize(st));
    if (!got[1])
        return fail("%s: COO row coordinates must be ascending and inside [0, rows) "
                    "(the order the reference reader produces)", what);
    if (!got[0])
        return fail("%s: a coordinate lies outside the matrix (crd must be in [0, %lld)%s)", what,
                    (long long)h.ncols, h.fmt == F_DCSR ? ", stored row coordinates in [0, rows)" : "");
    return 0;
}

// Range check (then a stream synchronisation) of coordinate arrays uploaded outside upload_sparse:
// cols in [0, ncols), rows (COO row coordinates or DCSR stored-row coordinates, may be null) in [0, nrows).
static int verify_coords(const char *what, DevBag &bag, const int64_t *cols, int64_t ncoords, int64_t ncols,
                         const int64_t *rows, int64_t nrowcoords, int64_t nrows)
{
    int *flag = nullptr;
    CB_TRY(bag.alloc((void **)&flag, sizeof(int)));
    int got = 1;
    CB_CUDA(cudaMemcpyAsync(flag, &got, sizeof(int), cudaMemcpyHostToDevice, bag.st));
    CB_TRY(check_index_range(cols, ncoords, ncols, flag, bag.st));
    if (rows) CB_TRY(check_index_range(rows, nrowcoords, nrows, flag, bag.st));
    CB_CUDA(cudaMemcpyAsync(&got, flag, sizeof(int), cudaMemcpyDeviceToHost, bag.st));
    CB_CUDA(cudaStreamSynchronize(bag.st));
    if (!got) return fail("%s: a coordinate lies outside the %lld x %lld matrix", what, (long long)nrows, (long long)ncols);
    return 0;
}

// End of a host entry point: the stream's work is done and every staged copy has reached the caller's arrays.
static int finish(cudaStream_t st)
{
    CB_CUDA(cudaStreamSynchronize(st));
    return copies_drain();
}

static int need_stream(cudaStream_t *st)
{
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0)
        return fail("no CUDA device is available; libcomet_b200 has no CPU path");
    *st = lib_stream();
    if (!*st) return fail("could not create the library stream");
    return pool_keep();
}

// Handles created through the host layer also own their staged operands.
struct HostPlan {
    int isz, vsz;
    int64_t dev_handle;
    std::vector<void *> owned;
    int64_t nnz;
};
static std::mutex g_hp_mu;
static std::unordered_map<int64_t, HostPlan *> g_hplans;

static void fill_sizes(void *sizes_ptr, int64_t sizes_rank, int64_t nrows, int64_t ncols, int64_t nnz)
{
    Arr s;
    if (get1d("sizes", sizes_rank, sizes_ptr, 8, &s) != 0 || !s.data) return;
    // layout of read_input_sizes_2D for CSR (lib/ExecutionEngine/SparseUtils.cpp:1672-1687)
    int64_t v[11] = {1, 1, 0, 0, nrows + 1, nnz, 0, 0, nnz, nrows, ncols};
    for (int i = 0; i < 11 && i < s.n; i++) ((int64_t *)s.data)[i] = v[i];
}

// Sharded calls are collective: every rank of the communicator makes the same call.  A rank that finds
// a fault in its own operands must not simply return, or the others would wait for it in the next
// exchange.  So after the local checks the ranks agree on a status (an all-reduce of one integer);
// a rank that leaves early takes part from the destructor with a failure, and everybody returns.
struct ShardGuard {
    Comm *cm;
    cudaStream_t st;
    bool agreed;
    ShardGuard(Comm *c, cudaStream_t s) : cm(c), st(s), agreed(c == nullptr || c->nranks == 1) {}
    ~ShardGuard() { if (!agreed) exchange(1); }
    int exchange(int mine)
    {
        agreed = true;
        int64_t *d = nullptr, h = mine ? 1 : 0;
        if (cudaMallocAsync((void **)&d, 8, st) != cudaSuccess) return 1;
        cudaMemcpyAsync(d, &h, 8, cudaMemcpyHostToDevice, st);
        comm_allreduce_sum_i64(cm, d, 1, st);
        cudaMemcpyAsync(&h, d, 8, cudaMemcpyDeviceToHost, st);
        cudaStreamSynchronize(st);
        cudaFreeAsync(d, st);
        return h != 0;
    }
    // rc: this rank's status so far.  Returns non-zero if any rank failed.
    int agree(int rc)
    {
        if (agreed) return rc;
        const int any = exchange(rc);
        if (any && !rc) return fail("sharded call: another rank reported an error in its operands");
        return rc;
    }
};

static int spmv_host(const HostSparse &A, Arr x, Arr y, int semiring, int accumulate)
{
    if (x.n < A.ncols) return fail("spmv: x shorter than the column count");
    if (y.n < A.nrows) return fail("spmv: y shorter than the row count");
    cudaStream_t st;
    CB_TRY(need_stream(&st));
    DevBag bag(st);
    DevSparse dA;
    CB_TRY(upload_sparse("spmv", A, bag, &dA));
    double *dx, *dy;
    CB_TRY(bag.upload_val(&dx, x.data, (size_t)A.ncols));
    bool keep_old = accumulate || A.fmt == F_DCSR;   // rows DCSR does not store keep their value
    if (keep_old) CB_TRY(bag.upload_val(&dy, y.data, (size_t)A.nrows));
    else CB_TRY(bag.alloc((void **)&dy, (size_t)A.nrows * 8));
    if (!accumulate && A.fmt == F_DCSR) CB_CUDA(cudaMemsetAsync(dy, 0, (size_t)A.nrows * 8, st));
    CB_TRY(comet_b200_dev_spmv_f64_i64(dA.nrows_k, A.nnz, dA.row_ids, dA.pos, dA.crd, dA.val, dx, dy,
                                       semiring, accumulate, st));
    CB_TRY(bag.download_val(y.data, dy, (size_t)A.nrows));
    return finish(st);
}

// Large SpMM through the host entry point is bound by PCIe: B goes up, C comes back.  The two
// directions can run at the same time if the work is cut into column panels: panel j of B is
// uploaded while panel j-1 is multiplied and panel j-2 of C is downloaded (strided 2-D copies
// between the row-major host matrices and packed panels on the device, two buffers each).
// With a communicator, a rank uploads only its N-th of the rows of each panel of B and the panel is
// completed by an all-gather on the compute stream before the kernel that reads it.
// The events and the drain of the panel pipeline: whatever way the pipeline function leaves, the copy
// streams are drained and the events destroyed before the panel buffers go back to the pool.
struct PanelSync {
    cudaStream_t up, down, st;
    cudaEvent_t ev[7];
    int n = 0;
    PanelSync(cudaStream_t u, cudaStream_t d, cudaStream_t s) : up(u), down(d), st(s) {}
    int create(cudaEvent_t **out)
    {
        CB_CUDA(cudaEventCreateWithFlags(&ev[n], cudaEventDisableTiming));
        *out = &ev[n++];
        return 0;
    }
    int drain()
    {
        cudaError_t e1 = cudaStreamSynchronize(up), e2 = cudaStreamSynchronize(down), e3 = cudaStreamSynchronize(st);
        int rc = copies_drain();
        if (!rc && (e1 != cudaSuccess || e2 != cudaSuccess || e3 != cudaSuccess)) rc = fail("spmm: panel pipeline failed");
        return rc;
    }
    ~PanelSync()
    {
        cudaStreamSynchronize(up);
        cudaStreamSynchronize(down);
        cudaStreamSynchronize(st);
        copies_drain();
        for (int i = 0; i < n; i++) cudaEventDestroy(ev[i]);
    }
};

static int spmm_host_panels(const HostSparse &A, const DevSparse &dA, DevBag &bag, const Mat &B, const Mat &C,
                            int semiring, int64_t panel, cudaStream_t st, Comm *cm)
{
    cudaStream_t up = aux_stream(0), down = aux_stream(1);
    if (!up || !down) return fail("spmm: could not create the copy streams");
    const int64_t k = B.cols;
    const int nranks = cm ? cm->nranks : 1, rank = cm ? cm->rank : 0;
    const int64_t slice_rows = ceil_div(A.ncols, nranks);           // rows of B this rank uploads
    const int64_t my_lo = slice_rows * rank < A.ncols ? slice_rows * rank : A.ncols;
    const int64_t my_rows = A.ncols - my_lo < slice_rows ? A.ncols - my_lo : slice_rows;
    double *dB[2], *dC[2];
    for (int i = 0; i < 2; i++) {
        CB_TRY(bag.alloc((void **)&dB[i], (size_t)slice_rows * nranks * panel * 8));
        CB_TRY(bag.alloc((void **)&dC[i], (size_t)A.nrows * panel * 8));
    }
    PanelSync sync(up, down, st);        // declared after the buffers: it drains before they are freed
    cudaEvent_t *in[2], *comp[2], *out[2], *ready;
    for (int i = 0; i < 2; i++) {
        CB_TRY(sync.create(&in[i]));
        CB_TRY(sync.create(&comp[i]));
        CB_TRY(sync.create(&out[i]));
    }
    CB_TRY(sync.create(&ready));
    CB_CUDA(cudaEventRecord(*ready, st));                 // A is uploaded, panel buffers exist
    CB_CUDA(cudaStreamWaitEvent(up, *ready, 0));
    CB_CUDA(cudaStreamWaitEvent(down, *ready, 0));
    // tracing: a timed event after every upload, kernel and download, reported against `t0` at the end
    const bool tracing = getenv("COMET_B200_TRACE") != nullptr;
    std::vector<cudaEvent_t> tev;
    auto mark = [&](cudaStream_t s) {
        if (!tracing) return;
        cudaEvent_t e;
        if (cudaEventCreate(&e) == cudaSuccess) { cudaEventRecord(e, s); tev.push_back(e); }
    };
    mark(st);
    int64_t j = 0;
    for (int64_t c0 = 0; c0 < k; c0 += panel, j++) {
        const int b = (int)(j & 1);
        const int64_t w = (k - c0) < panel ? (k - c0) : panel;
        if (j >= 2) CB_CUDA(cudaStreamWaitEvent(up, *comp[b], 0));       // panel j-2 no longer reads dB[b]
        if (my_rows > 0)
            CB_TRY(h2d_2d(dB[b] + my_lo * panel, (size_t)panel * 8, B.data + my_lo * B.s0 + c0, (size_t)B.s0 * 8,
                          (size_t)w * 8, (size_t)my_rows, up));
        CB_CUDA(cudaEventRecord(*in[b], up));
        mark(up);
        trace("spmm: panel %lld upload enqueued", (long long)j);
        CB_CUDA(cudaStreamWaitEvent(st, *in[b], 0));
        if (nranks > 1) CB_TRY(comm_allgather_inplace(cm, dB[b], (size_t)slice_rows * panel * 8, st));
        if (j >= 2) CB_CUDA(cudaStreamWaitEvent(st, *out[b], 0));        // panel j-2 has left dC[b]
        CB_TRY(comet_b200_dev_spmm_f64_i64(dA.nrows_k, A.ncols, A.nnz, w, dA.row_ids, dA.pos, dA.crd, dA.val, dB[b],
                                           panel, dC[b], panel, semiring, 0, 0, st));
        CB_CUDA(cudaEventRecord(*comp[b], st));
        mark(st);
        CB_CUDA(cudaStreamWaitEvent(down, *comp[b], 0));
        CB_TRY(d2h_2d(C.data + c0, (size_t)C.s0 * 8, dC[b], (size_t)panel * 8, (size_t)w * 8, (size_t)A.nrows, down));
        CB_CUDA(cudaEventRecord(*out[b], down));
        mark(down);
        trace("spmm: panel %lld download enqueued", (long long)j);
    }
    const int drc = sync.drain();
    trace("spmm: drained");
    for (size_t i = 1; i < tev.size(); i++) {
        float ms = 0;
        cudaEventElapsedTime(&ms, tev[0], tev[i]);
        trace("spmm: device time, panel %zu %s done at %.3f ms", (i - 1) / 3,
              (i - 1) % 3 == 0 ? "upload" : ((i - 1) % 3 == 1 ? "all-gather + kernel" : "download"), ms);
    }
    for (cudaEvent_t e : tev) cudaEventDestroy(e);
    return drc;
}

static int spmm_check(const HostSparse &A, const Mat &B, const Mat &C)
{
    if (B.rows < A.ncols) return fail("spmm: B has fewer rows than A has columns");
    if (C.rows < A.nrows || C.cols != B.cols) return fail("spmm: C has the wrong shape");
    if ((B.cols > 1 && B.s1 != 1) || (C.cols > 1 && C.s1 != 1) || B.s0 < B.cols || C.s0 < C.cols)
        return fail("spmm: B and C must be row-major");
    return 0;
}

// cm != null: A and C are this rank's row block, B is the whole (replicated) dense operand.
static int spmm_host(const HostSparse &A, const Mat &B, const Mat &C, int semiring, int accumulate, Comm *cm)
{
    cudaStream_t st;
    CB_TRY(need_stream(&st));
    ShardGuard guard(cm, st);
    DevBag bag(st);
    DevSparse dA;
    trace("spmm: begin (%lld rows, %lld entries, rank %d of %d)", (long long)A.nrows, (long long)A.nnz,
          cm ? cm->rank : 0, cm ? cm->nranks : 1);
    int rc = spmm_check(A, B, C);
    if (!rc) rc = upload_sparse("spmm", A, bag, &dA);
    trace("spmm: A uploaded and checked");
    CB_TRY(guard.agree(rc));
    trace("spmm: ranks agreed");
    const int64_t k = B.cols;
    {
        // panels of 32 columns (256-byte rows) once the dense operands are big enough to matter
        int64_t panel = 32;
        const char *env = getenv("COMET_B200_SPMM_PANEL");
        if (env) panel = atoll(env);
        double min_bytes = 256e6;
        const char *menv = getenv("COMET_B200_SPMM_PANEL_MIN_BYTES");
        if (menv) min_bytes = atof(menv);
        // (decided from B alone: under a communicator every rank must take the same branch, and the
        // blocks of A differ from rank to rank)
        const bool big = (double)A.ncols * (double)k * 8.0 * 2.0 >= min_bytes;
        // Pageable host matrices are moved by the staged copier, whose worker threads would have to copy
        // panel rows of a few hundred bytes each out of / into the wide rows: measured slower than one
        // contiguous upload and one contiguous download (46 against 93 ms on two GPUs), so the panels are
        // kept for page-locked operands.  (Every rank decides from its own pointers; ranks that mix pinned
        // and pageable operands must force one mode with COMET_B200_SPMM_PANEL, since the all-gather of the
        // two paths differs.)
        const bool pinned = env || (!host_is_pageable(B.data) && !host_is_pageable(C.data));
        if (!accumulate && A.fmt != F_DCSR && panel >= 2 && panel % 2 == 0 && k >= 2 * panel && big &&
            semiring == COMET_B200_PLUS_TIMES && g_vsz == 8 && pinned)
            return spmm_host_panels(A, dA, bag, B, C, semiring, panel, st, cm);
    }
    double *dB, *dC;
    CB_TRY(bag.upload_val(&dB, B.data, (size_t)((A.ncols - 1) * B.s0 + k) * (A.ncols > 0), cm));
    size_t cbytes = A.nrows > 0 ? (size_t)((A.nrows - 1) * C.s0 + k) * 8 : 0;
    bool keep_old = accumulate || A.fmt == F_DCSR || C.s0 != k;
    if (keep_old) CB_TRY(bag.upload_val(&dC, C.data, cbytes / 8));
    else CB_TRY(bag.alloc((void **)&dC, cbytes));
    if (!accumulate && A.fmt == F_DCSR) CB_CUDA(cudaMemsetAsync(dC, 0, cbytes, st));
    CB_TRY(comet_b200_dev_spmm_f64_i64(dA.nrows_k, A.ncols, A.nnz, k, dA.row_ids, dA.pos, dA.crd,
                                       dA.val, dB, B.s0, dC, C.s0, semiring, accumulate, 0, st));
    if (cbytes) CB_TRY(bag.download_val(C.data, dC, cbytes / 8));
    return finish(st);
}

static void copy_pattern(const HostSparse &src, const HostSparse &dst)
{
    // the output tensor shares the sparse operand's pos/crd
    // (lib/Conversion/IndexTreeToSCF/SymbolicDomainConversion.cpp:277-297)
    const int isz = src.isz;
    if (src.fmt == F_CSR) {
        if (dst.a1pos && dst.a1pos != src.a1pos) idx_set(dst.a1pos, 0, isz, src.nrows);
        if (dst.a2pos != src.a2pos) memcpy(dst.a2pos, src.a2pos, (size_t)(src.nrows + 1) * isz);
    } else if (src.fmt == F_COO) {
        if (dst.a1pos != src.a1pos) { idx_set(dst.a1pos, 0, isz, 0); idx_set(dst.a1pos, 1, isz, src.nnz); }
        if (dst.a1crd != src.a1crd) memcpy(dst.a1crd, src.a1crd, (size_t)src.nnz * isz);
    }
    if (dst.a2crd != src.a2crd) memcpy(dst.a2crd, src.a2crd, (size_t)src.nnz * isz);
}

}  // namespace cb200

using namespace cb200;

#define GET_SPARSE(name, P, hs) \
    get_sparse(name, isz, P##1format, P##2format, P##1pos_rank, P##1pos_ptr, P##1crd_rank, P##1crd_ptr, \
               P##2pos_rank, P##2pos_ptr, P##2crd_rank, P##2crd_ptr, P##val_rank, P##val_ptr,       \
               P##dims_rank, P##dims_ptr, hs)

// all 24 arguments of one sparse operand, for forwarding
#define FWD_SPARSE(P) P##1format, P##1tile_format, P##2format, P##2tile_format, P##1pos_rank, P##1pos_ptr, \
    P##1crd_rank, P##1crd_ptr, P##1tile_pos_rank, P##1tile_pos_ptr, P##1tile_crd_rank, P##1tile_crd_ptr,     \
    P##2pos_rank, P##2pos_ptr, P##2crd_rank, P##2crd_ptr, P##2tile_pos_rank, P##2tile_pos_ptr,               \
    P##2tile_crd_rank, P##2tile_crd_ptr, P##val_rank, P##val_ptr, P##dims_rank, P##dims_ptr

#define UNUSED_TILES(P) (void)P##1tile_format; (void)P##2tile_format; (void)P##1tile_pos_rank; \
    (void)P##1tile_pos_ptr; (void)P##1tile_crd_rank; (void)P##1tile_crd_ptr; (void)P##2tile_pos_rank; \
    (void)P##2tile_pos_ptr; (void)P##2tile_crd_rank; (void)P##2tile_crd_ptr

// First argument of the *_impl functions below: bytes per index (8 or 4), plus MODE_SHARDED for the
// entry points that run under the device's communicator.
enum { MODE_SHARDED = 16 };

static int mode_comm(int mode, Comm **cm)
{
    *cm = nullptr;
    if (!(mode & MODE_SHARDED)) return 0;
    *cm = comm_current();
    if (!*cm) return fail("sharded call: this device has no communicator (comet_b200_comm_init comes first)");
    return 0;
}

static void spmv_impl(int isz, COMET_B200_SPARSE2D(A), int64_t x_rank, void *x_ptr, int64_t y_rank,
                      void *y_ptr, int32_t semiring, int32_t accumulate)
{
    UNUSED_TILES(A);
    clear_error();
    HostSparse A;
    Arr x, y;
    if (GET_SPARSE("spmv: A", A, &A)) return;
    if (get1d("spmv: x", x_rank, x_ptr, g_vsz, &x) || get1d("spmv: y", y_rank, y_ptr, g_vsz, &y)) return;
    spmv_host(A, x, y, semiring, accumulate);
}

static void spmm_impl(int mode, COMET_B200_SPARSE2D(A), int64_t B_rank, void *B_ptr, int64_t C_rank,
                      void *C_ptr, int32_t semiring, int32_t accumulate)
{
    UNUSED_TILES(A);
    clear_error();
    const int isz = mode & 15;
    Comm *cm;
    if (mode_comm(mode, &cm)) return;
    HostSparse A;
    Mat B, C;
    int rc = GET_SPARSE("spmm: A", A, &A) || get2d("spmm: B", B_rank, B_ptr, &B) || get2d("spmm: C", C_rank, C_ptr, &C);
    if (rc) {
        if (cm) { cudaStream_t st; if (!need_stream(&st)) ShardGuard(cm, st).agree(1); }
        return;
    }
    spmm_host(A, B, C, semiring, accumulate, cm);
}

static int sddmm_check(const HostSparse &S, const HostSparse &O, const Mat &X, const Mat &D)
{
    if (S.fmt != F_CSR || O.fmt != F_CSR) return fail("sddmm: S and O must be CSR");
    const int64_t k = X.cols;
    if (X.rows < S.nrows || (k > 1 && X.s1 != 1) || X.s0 < k) return fail("sddmm: X must be row-major [rows, K]");
    if (D.rows != k || D.cols < S.ncols) return fail("sddmm: D must have sizes {K, cols}");
    if (!((D.s0 == 1 && D.s1 >= k) || (D.s1 == 1 && D.s0 >= D.cols)))
        return fail("sddmm: D must be contiguous along one of its dimensions");
    return 0;
}

// Sharded: S, X and O are this rank's row block; D (all of Y) is the replicated operand.
static void sddmm_impl(int mode, COMET_B200_SPARSE2D(S), int64_t X_rank, void *X_ptr, int64_t D_rank,
                       void *D_ptr, COMET_B200_SPARSE2D(O))
{
    UNUSED_TILES(S);
    UNUSED_TILES(O);
    clear_error();
    const int isz = mode & 15;
    Comm *cm;
    if (mode_comm(mode, &cm)) return;
    cudaStream_t st;
    if (need_stream(&st)) return;
    ShardGuard guard(cm, st);
    HostSparse S, O;
    Mat X, D;
    DevBag bag(st);
    DevSparse dS;
    double *dX = nullptr, *dY = nullptr, *dOut = nullptr;
    int rc = GET_SPARSE("sddmm: S", S, &S) || GET_SPARSE("sddmm: O", O, &O) ||
             get2d("sddmm: X", X_rank, X_ptr, &X) || get2d("sddmm: D", D_rank, D_ptr, &D);
    if (!rc) rc = sddmm_check(S, O, X, D);
    if (!rc) rc = upload_sparse("sddmm", S, bag, &dS);
    const int64_t k = rc ? 0 : X.cols;
    if (!rc) rc = bag.upload_val(&dX, X.data, S.nrows > 0 ? (size_t)((S.nrows - 1) * X.s0 + k) : 0);
    if (guard.agree(rc)) return;
    int64_t ldy;
    if (D.s0 == 1) {                          // a row-major [cols, K] matrix viewed transposed
        ldy = D.s1;
        if (bag.upload_val(&dY, D.data, S.ncols > 0 ? (size_t)((S.ncols - 1) * ldy + k) : 0, cm)) return;
    } else {                                  // D[k, j]: transpose on the device
        double *dD;
        if (bag.upload_val(&dD, D.data, k > 0 ? (size_t)((k - 1) * D.s0 + S.ncols) : 0, cm)) return;
        ldy = k + (k & 1);
        if (bag.alloc((void **)&dY, (size_t)S.ncols * ldy * 8)) return;
        if (comet_b200_dev_transpose_f64(k, S.ncols, dD, D.s0, dY, ldy, st)) return;
    }
    if (bag.alloc((void **)&dOut, (size_t)S.nnz * 8)) return;
    if (comet_b200_dev_sddmm_f64_i64(S.nrows, S.nnz, k, dS.pos, dS.crd, dS.val, dX, X.s0, dY, ldy, dOut, st))
        return;
    if (bag.download_val(O.val, dOut, (size_t)S.nnz)) return;
    copy_pattern(S, O);
    finish(st);
}

static void elews_sd_impl(int isz, COMET_B200_SPARSE2D(A), int64_t B_rank, void *B_ptr,
                          COMET_B200_SPARSE2D(C))
{
    UNUSED_TILES(A);
    UNUSED_TILES(C);
    clear_error();
    HostSparse A, C;
    Mat B;
    if (GET_SPARSE("elews_mul: A", A, &A) || GET_SPARSE("elews_mul: C", C, &C)) return;
    if (get2d("elews_mul: B", B_rank, B_ptr, &B)) return;
    if (A.fmt == F_DCSR || C.fmt != A.fmt) { fail("elews_mul: A and C must both be CSR or both COO"); return; }
    if (B.rows < A.nrows || B.cols < A.ncols || (B.cols > 1 && B.s1 != 1)) { fail("elews_mul: B must be row-major [rows, cols]"); return; }
    cudaStream_t st;
    if (need_stream(&st)) return;
    DevBag bag(st);
    DevSparse dA;
    memset(&dA, 0, sizeof(dA));
    if (bag.upload_idx(&dA.crd, A.a2crd, A.nnz, A.isz)) return;
    if (bag.upload((void **)&dA.val, A.val, (size_t)A.nnz * 8)) return;
    if (A.fmt == F_CSR) { if (bag.upload_idx(&dA.pos, A.a2pos, A.nrows + 1, A.isz)) return; }
    else { if (bag.upload_idx(&dA.rows, A.a1crd, A.nnz, A.isz)) return; }
    if (verify_coords("elews_mul: A", bag, dA.crd, A.nnz, A.ncols, dA.rows, A.nnz, A.nrows)) return;
    double *dB, *dOut;
    if (bag.upload((void **)&dB, B.data, A.nrows > 0 ? (size_t)((A.nrows - 1) * B.s0 + A.ncols) * 8 : 0)) return;
    if (bag.alloc((void **)&dOut, (size_t)A.nnz * 8)) return;
    if (comet_b200_dev_elews_mul_sparse_dense_f64_i64(A.nrows, A.nnz, dA.pos, dA.rows, dA.crd, dA.val, dB,
                                                      B.s0, dOut, st))
        return;
    if (A.nnz && d2h(C.val, dOut, (size_t)A.nnz * 8, st)) return;
    copy_pattern(A, C);
    finish(st);
}

// C (dense) = A (sparse) .* B (dense): products land at A's stored positions, the rest of C keeps its values.
static void elews_to_dense_impl(int isz, COMET_B200_SPARSE2D(A), int64_t B_rank, void *B_ptr, int64_t C_rank,
                                void *C_ptr)
{
    UNUSED_TILES(A);
    clear_error();
    HostSparse A;
    Mat B, C;
    if (GET_SPARSE("elews_mul: A", A, &A)) return;
    if (get2d("elews_mul: B", B_rank, B_ptr, &B) || get2d("elews_mul: C", C_rank, C_ptr, &C)) return;
    if (B.rows < A.nrows || B.cols < A.ncols || C.rows < A.nrows || C.cols < A.ncols || (B.cols > 1 && B.s1 != 1) ||
        (C.cols > 1 && C.s1 != 1)) {
        fail("elews_mul: B and C must be row-major [rows, cols]");
        return;
    }
    cudaStream_t st;
    if (need_stream(&st)) return;
    DevBag bag(st);
    DevSparse dA;
    memset(&dA, 0, sizeof(dA));
    if (bag.upload_idx(&dA.crd, A.a2crd, A.nnz, A.isz)) return;
    if (bag.upload((void **)&dA.val, A.val, (size_t)A.nnz * 8)) return;
    int64_t nstored = A.nrows;
    if (A.fmt == F_COO) { if (bag.upload_idx(&dA.rows, A.a1crd, A.nnz, A.isz)) return; }
    else {
        nstored = A.nstored;
        if (bag.upload_idx(&dA.pos, A.a2pos, nstored + 1, A.isz)) return;
        if (A.fmt == F_DCSR && bag.upload_idx(&dA.row_ids, A.a1crd, nstored, A.isz)) return;
    }
    if (verify_coords("elews_mul: A", bag, dA.crd, A.nnz, A.ncols, A.fmt == F_COO ? dA.rows : dA.row_ids,
                      A.fmt == F_COO ? A.nnz : nstored, A.nrows))
        return;
    double *dB, *dC;
    const size_t bbytes = A.nrows > 0 ? (size_t)((A.nrows - 1) * B.s0 + A.ncols) * 8 : 0;
    const size_t cbytes = A.nrows > 0 ? (size_t)((A.nrows - 1) * C.s0 + A.ncols) * 8 : 0;
    if (bag.upload((void **)&dB, B.data, bbytes) || bag.upload((void **)&dC, C.data, cbytes)) return;
    if (comet_b200_dev_elews_mul_sparse_dense_to_dense_f64_i64(nstored, A.nnz, dA.row_ids, dA.pos, dA.rows, dA.crd,
                                                               dA.val, dB, B.s0, dC, C.s0, st))
        return;
    if (cbytes && d2h(C.data, dC, cbytes, st)) return;
    finish(st);
}

// n int64 indices on the device -> the caller's array of isz-byte integers
static int download_idx(DevBag &bag, const int64_t *dev, char *host, int64_t n, int isz, cudaStream_t st)
{
    if (n <= 0) return 0;
    if (isz == 8) {
        CB_TRY(d2h(host, dev, (size_t)n * 8, st));
        return 0;
    }
    int32_t *d32 = nullptr;
    CB_TRY(bag.alloc((void **)&d32, (size_t)n * 4));
    CB_TRY(narrow_any_i64_to_i32(dev, d32, n, st));
    CB_TRY(d2h(host, d32, (size_t)n * 4, st));
    return 0;
}

// B = transpose(A) for CSR -> CSR and COO -> COO, the two pairs transpose_2D handles
// (lib/ExecutionEngine/TransposeUtils.cpp:625-812).  The caller allocated B's arrays; like the
// reference this fills them, writes the placeholders (B1pos = {rows of B}, B1crd = {-1} for CSR;
// B1pos = {0, nnz} for COO) and swaps the two dimension sizes in `sizes`.
static void transpose_impl(int isz, int32_t A1format, int32_t A2format, int64_t A1pos_rank, void *A1pos_ptr,
                           int64_t A1crd_rank, void *A1crd_ptr, int64_t A2pos_rank, void *A2pos_ptr,
                           int64_t A2crd_rank, void *A2crd_ptr, int64_t Aval_rank, void *Aval_ptr, int32_t B1format,
                           int32_t B2format, int64_t B1pos_rank, void *B1pos_ptr, int64_t B1crd_rank, void *B1crd_ptr,
                           int64_t B2pos_rank, void *B2pos_ptr, int64_t B2crd_rank, void *B2crd_ptr,
                           int64_t Bval_rank, void *Bval_ptr, int64_t sizes_rank, void *sizes_ptr)
{
    clear_error();
    Arr a1pos, a1crd, a2pos, a2crd, aval, b1pos, b1crd, b2pos, b2crd, bval, sizes;
    if (get1d("transpose: A1pos", A1pos_rank, A1pos_ptr, isz, &a1pos) || get1d("transpose: A1crd", A1crd_rank, A1crd_ptr, isz, &a1crd) ||
        get1d("transpose: A2pos", A2pos_rank, A2pos_ptr, isz, &a2pos) || get1d("transpose: A2crd", A2crd_rank, A2crd_ptr, isz, &a2crd) ||
        get1d("transpose: Aval", Aval_rank, Aval_ptr, 8, &aval) || get1d("transpose: B1pos", B1pos_rank, B1pos_ptr, isz, &b1pos) ||
        get1d("transpose: B1crd", B1crd_rank, B1crd_ptr, isz, &b1crd) || get1d("transpose: B2pos", B2pos_rank, B2pos_ptr, isz, &b2pos) ||
        get1d("transpose: B2crd", B2crd_rank, B2crd_ptr, isz, &b2crd) || get1d("transpose: Bval", Bval_rank, Bval_ptr, 8, &bval) ||
        get1d("transpose: sizes", sizes_rank, sizes_ptr, isz, &sizes))
        return;
    if (!sizes.data || sizes.n < 2) { fail("transpose: sizes must hold {rows, cols}"); return; }
    const int64_t nrows = idx_get((char *)sizes.data, 0, isz), ncols = idx_get((char *)sizes.data, 1, isz);
    if (nrows < 0 || ncols < 0) { fail("transpose: negative dimension"); return; }
    const bool a_csr = A1format == COMET_B200_FMT_DENSE && A2format == COMET_B200_FMT_CU;
    const bool a_coo = A1format == COMET_B200_FMT_CN && A2format == COMET_B200_FMT_S;
    const bool b_csr = B1format == COMET_B200_FMT_DENSE && B2format == COMET_B200_FMT_CU;
    const bool b_coo = B1format == COMET_B200_FMT_CN && B2format == COMET_B200_FMT_S;
    if (!((a_csr && b_csr) || (a_coo && b_coo))) {
        fail("transpose: only CSR -> CSR and COO -> COO are handled (as in the reference runtime)");
        return;
    }
    int64_t nnz = 0;
    if (a_csr) {
        if (a2pos.n < nrows + 1) { fail("transpose: A2pos shorter than rows+1"); return; }
        int64_t prev = 0;
        for (int64_t i = 0; i <= nrows; i++) {
            const int64_t cur = idx_get((char *)a2pos.data, i, isz);
            if ((i == 0 && cur != 0) || cur < prev) { fail("transpose: A2pos is not a row pointer"); return; }
            prev = cur;
        }
        nnz = prev;
        if (b2pos.n < ncols + 1) { fail("transpose: B2pos shorter than cols+1"); return; }
    } else {
        if (a1pos.n < 2) { fail("transpose: COO A1pos must hold {0, nnz}"); return; }
        nnz = idx_get((char *)a1pos.data, 1, isz);
        if (nnz < 0 || a1crd.n < nnz || b1crd.n < nnz || b1pos.n < 2) { fail("transpose: COO arrays shorter than nnz"); return; }
    }
    if (a2crd.n < nnz || aval.n < nnz || b2crd.n < nnz || bval.n < nnz) { fail("transpose: crd/val arrays shorter than nnz"); return; }
    cudaStream_t st;
    if (need_stream(&st)) return;
    DevBag bag(st);
    int64_t *dcrd = nullptr, *dmaj = nullptr, *omaj = nullptr, *ocrd = nullptr;
    double *dval = nullptr, *oval = nullptr;
    if (bag.upload_idx(&dcrd, a2crd.data, nnz, isz) || bag.upload((void **)&dval, aval.data, (size_t)nnz * 8) ||
        bag.alloc((void **)&ocrd, (size_t)nnz * 8) || bag.alloc((void **)&oval, (size_t)nnz * 8))
        return;
    if (a_csr) {
        int64_t *dpos = nullptr;
        if (bag.upload_idx(&dpos, a2pos.data, nrows + 1, isz) || bag.alloc((void **)&omaj, (size_t)(ncols + 1) * 8)) return;
        if (verify_coords("transpose: A", bag, dcrd, nnz, ncols, nullptr, 0, nrows)) return;
        if (comet_b200_dev_csr_transpose_f64_i64(nrows, ncols, nnz, dpos, dcrd, dval, omaj, ocrd, oval, st)) return;
        if (download_idx(bag, omaj, (char *)b2pos.data, ncols + 1, isz, st)) return;
        if (b1pos.data && b1pos.n >= 1) idx_set((char *)b1pos.data, 0, isz, ncols);
        if (b1crd.data && b1crd.n >= 1) idx_set((char *)b1crd.data, 0, isz, -1);
    } else {
        if (bag.upload_idx(&dmaj, a1crd.data, nnz, isz) || bag.alloc((void **)&omaj, (size_t)nnz * 8)) return;
        // sorted by (column, row) of the input: the transposed matrix in the reader's order
        if (comet_b200_dev_sort_coo_f64_i64(nnz, ncols, nrows, dcrd, dmaj, dval, omaj, ocrd, oval, st)) return;
        if (download_idx(bag, omaj, (char *)b1crd.data, nnz, isz, st)) return;
        idx_set((char *)b1pos.data, 0, isz, 0);
        idx_set((char *)b1pos.data, 1, isz, nnz);
    }
    if (download_idx(bag, ocrd, (char *)b2crd.data, nnz, isz, st)) return;
    if (nnz && d2h(bval.data, oval, (size_t)nnz * 8, st)) return;
    if (finish(st)) return;
    idx_set((char *)sizes.data, 0, isz, ncols);
    idx_set((char *)sizes.data, 1, isz, nrows);
}

// Dense x sparse: A is a rank-1 (vector) or rank-2 row-major memref, C has the same rank.
static void dense_sparse_impl(int isz, int64_t A_rank, void *A_ptr, COMET_B200_SPARSE2D(B), int64_t C_rank,
                              void *C_ptr, int32_t semiring, int32_t accumulate)
{
    UNUSED_TILES(B);
    clear_error();
    HostSparse B;
    if (GET_SPARSE("dense x sparse: B", B, &B)) return;
    if (A_rank != C_rank || (A_rank != 1 && A_rank != 2)) { fail("dense x sparse: A and C must both be vectors or both matrices"); return; }
    int64_t m, lda, ldc;
    double *ha, *hc;
    if (A_rank == 1) {
        Arr a, c;
        if (get1d("dense x sparse: A", A_rank, A_ptr, 8, &a) || get1d("dense x sparse: C", C_rank, C_ptr, 8, &c)) return;
        if (a.n < B.nrows || c.n < B.ncols) { fail("dense x sparse: vector shorter than the matrix dimension"); return; }
        m = 1; lda = B.nrows; ldc = B.ncols; ha = (double *)a.data; hc = (double *)c.data;
    } else {
        Mat a, c;
        if (get2d("dense x sparse: A", A_rank, A_ptr, &a) || get2d("dense x sparse: C", C_rank, C_ptr, &c)) return;
        if (a.cols < B.nrows || c.cols < B.ncols || c.rows < a.rows || (a.cols > 1 && a.s1 != 1) || (c.cols > 1 && c.s1 != 1)) {
            fail("dense x sparse: A must be row-major [m, rows(B)] and C row-major [m, cols(B)]");
            return;
        }
        m = a.rows; lda = a.s0; ldc = c.s0; ha = a.data; hc = c.data;
    }
    cudaStream_t st;
    if (need_stream(&st)) return;
    DevBag bag(st);
    DevSparse dB;
    if (upload_sparse("dense x sparse", B, bag, &dB)) return;
    double *dA, *dC;
    const size_t abytes = m > 0 ? (size_t)((m - 1) * lda + B.nrows) * 8 : 0;
    const size_t cbytes = m > 0 ? (size_t)((m - 1) * ldc + B.ncols) * 8 : 0;
    if (bag.upload((void **)&dA, ha, abytes)) return;
    if (accumulate || ldc != B.ncols) { if (bag.upload((void **)&dC, hc, cbytes)) return; }
    else if (bag.alloc((void **)&dC, cbytes)) return;
    if (comet_b200_dev_dense_times_sparse_f64_i64(m, B.ncols, dB.nrows_k, B.nnz, dB.row_ids, dB.pos, dB.crd, dB.val, dA,
                                                  lda, dC, ldc, semiring, accumulate, st))
        return;
    if (cbytes && d2h(hc, dC, cbytes, st)) return;
    finish(st);
}

// cm != null (sharded): A, M and the output are this rank's row block, B is the replicated operand.
static int64_t sparse_out_symbolic(int isz, int kind, const HostSparse &A, const HostSparse &B,
                                   const HostSparse *M, int semiring, Arr cpos, int64_t sizes_rank,
                                   void *sizes_ptr, Comm *cm = nullptr)
{
    cudaStream_t st;
    if (need_stream(&st)) return 0;
    ShardGuard guard(cm, st);
    DevBag bag(st);
    DevSparse dA, dB, dM;
    memset(&dM, 0, sizeof(dM));
    int rc0 = 0;
    if (A.fmt != F_CSR || B.fmt != F_CSR || (M && M->fmt != F_CSR))
        rc0 = fail("sparse output: operands must be CSR (COMET's workspace transformation handles CSR only)");
    else if (cpos.n < A.nrows + 1) rc0 = fail("sparse output: C2pos shorter than rows+1");
    else if (kind == 0 && B.nrows < A.ncols) rc0 = fail("spgemm: B has fewer rows than A has columns");
    else if (kind == 1 && (B.nrows != A.nrows)) rc0 = fail("elews_mul: row counts differ");
    else if (M && M->nrows < A.nrows) rc0 = fail("spgemm: the mask has fewer rows than A");
    const bool sharded = cm && cm->nranks > 1;
    const bool same = !sharded && B.a2pos == A.a2pos && B.a2crd == A.a2crd && B.val == A.val;
    if (!rc0) rc0 = upload_sparse("A", A, bag, &dA);
    if (!rc0 && M) {
        if (M->a2pos == A.a2pos && M->a2crd == A.a2crd) dM = dA;
        else if (!sharded && !same && M->a2pos == B.a2pos && M->a2crd == B.a2crd) dM.pos = nullptr;   // set below
        else rc0 = upload_sparse("M", *M, bag, &dM, false);
    }
    if (guard.agree(rc0)) return 0;
    if (same) dB = dA;
    else if (upload_sparse("B", B, bag, &dB, true, cm)) return 0;
    if (M && !dM.pos && M->a2pos == B.a2pos && M->a2crd == B.a2crd) dM = dB;
    int64_t *dcpos;
    if (bag.alloc((void **)&dcpos, (size_t)(A.nrows + 1) * 8)) return 0;
    int64_t nnz = 0, dev_handle = 0;
    int rc;
    if (kind == 0)
        rc = comet_b200_dev_spgemm_symbolic_f64_i64(A.nrows, B.ncols, B.nnz, dA.pos, dA.crd, dA.val,
                                                    dB.pos, dB.crd, dB.val, M ? dM.pos : nullptr,
                                                    M ? dM.crd : nullptr, semiring, dcpos, &nnz,
                                                    &dev_handle, st);
    else
        rc = comet_b200_dev_elews_mul_sparse_sparse_symbolic_f64_i64(
            A.nrows, dA.pos, dA.crd, dA.val, dB.pos, dB.crd, dB.val, dcpos, &nnz, &dev_handle, st);
    if (rc) return 0;
    if (isz == 4 && nnz >= 0x7fffffffLL) {
        comet_b200_handle_destroy(dev_handle);
        return fail("sparse output: %lld entries do not fit 32-bit indices; use the _i64 entry point", (long long)nnz), 0;
    }
    void *pos_src = dcpos;
    if (isz == 4) {     // narrow the row pointer on the device before it goes back
        int32_t *p32;
        if (bag.alloc((void **)&p32, (size_t)(A.nrows + 1) * 4) || narrow_any_i64_to_i32(dcpos, p32, A.nrows + 1, st)) {
            comet_b200_handle_destroy(dev_handle);
            return 0;
        }
        pos_src = p32;
    }
    if (d2h(cpos.data, pos_src, (size_t)(A.nrows + 1) * isz, st) || finish(st)) {
        comet_b200_handle_destroy(dev_handle);
        return fail("sparse output: copy of C2pos failed"), 0;
    }
    fill_sizes(sizes_ptr, sizes_rank, A.nrows, kind == 0 ? B.ncols : A.ncols, nnz);
    if (cm) {
        // position of this block in the whole result: entries [11] and [12] of the sizes memref (when it has
        // them) receive the number of entries the lower ranks' blocks hold and the total over all ranks
        int64_t *dnnz = nullptr, *dall = nullptr;
        std::vector<int64_t> all((size_t)cm->nranks, 0);
        if (bag.upload((void **)&dnnz, &nnz, 8) || bag.alloc((void **)&dall, (size_t)cm->nranks * 8) ||
            comm_allgather_i64(cm, dnnz, dall, st) ||
            cudaMemcpyAsync(all.data(), dall, (size_t)cm->nranks * 8, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
            cudaStreamSynchronize(st) != cudaSuccess) {
            comet_b200_handle_destroy(dev_handle);
            return fail("sparse output: exchange of the per-rank entry counts failed"), 0;
        }
        int64_t before = 0, total = 0;
        for (int r = 0; r < cm->nranks; r++) { if (r < cm->rank) before += all[r]; total += all[r]; }
        Arr sz;
        if (get1d("sizes", sizes_rank, sizes_ptr, 8, &sz) == 0 && sz.data && sz.n >= 13) {
            ((int64_t *)sz.data)[11] = before;
            ((int64_t *)sz.data)[12] = total;
        }
    }
    HostPlan *hp = new HostPlan();
    hp->dev_handle = dev_handle;
    hp->nnz = nnz;
    hp->isz = isz;
    hp->vsz = g_vsz;
    hp->owned.swap(bag.ptrs);   // staged operands live until the numeric call
    std::lock_guard<std::mutex> lk(g_hp_mu);
    g_hplans[dev_handle] = hp;
    return dev_handle;
}

static int64_t spgemm_symbolic_impl(int mode, COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B),
                                    COMET_B200_SPARSE2D(M), int32_t mask_type, int32_t semiring,
                                    int64_t C2pos_rank, void *C2pos_ptr, int64_t sizes_rank,
                                    void *sizes_ptr)
{
    UNUSED_TILES(A);
    UNUSED_TILES(B);
    UNUSED_TILES(M);
    clear_error();
    const int isz = mode & 15;
    Comm *cm;
    if (mode_comm(mode, &cm)) return 0;
    HostSparse A, B, M;
    Arr cpos;
    const bool masked = mask_type == COMET_B200_MASK_PUSH;
    int rc = GET_SPARSE("spgemm: A", A, &A) || GET_SPARSE("spgemm: B", B, &B);
    if (!rc && mask_type != COMET_B200_MASK_NONE && mask_type != COMET_B200_MASK_PUSH)
        rc = fail("spgemm: unsupported mask type %d (none and push are handled)", mask_type);
    if (!rc && masked) rc = GET_SPARSE("spgemm: M", M, &M);
    if (!rc) rc = get1d("spgemm: C2pos", C2pos_rank, C2pos_ptr, isz, &cpos);
    if (rc) {
        if (cm) { cudaStream_t st; if (!need_stream(&st)) ShardGuard(cm, st).agree(1); }
        return 0;
    }
    return sparse_out_symbolic(isz, 0, A, B, masked ? &M : nullptr, semiring, cpos, sizes_rank, sizes_ptr, cm);
}

static int64_t elews_ss_symbolic_impl(int isz, COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B),
                                      int64_t C2pos_rank, void *C2pos_ptr, int64_t sizes_rank,
                                      void *sizes_ptr)
{
    UNUSED_TILES(A);
    UNUSED_TILES(B);
    clear_error();
    HostSparse A, B;
    Arr cpos;
    if (GET_SPARSE("elews_mul: A", A, &A) || GET_SPARSE("elews_mul: B", B, &B)) return 0;
    if (get1d("elews_mul: C2pos", C2pos_rank, C2pos_ptr, isz, &cpos)) return 0;
    return sparse_out_symbolic(isz, 1, A, B, nullptr, COMET_B200_PLUS_TIMES, cpos, sizes_rank, sizes_ptr);
}

static void spgemm_numeric_impl(int isz, int64_t handle, int64_t C2crd_rank, void *C2crd_ptr,
                                int64_t Cval_rank, void *Cval_ptr)
{
    clear_error();
    HostPlan *hp = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_hp_mu);
        auto it = g_hplans.find(handle);
        if (it != g_hplans.end()) { hp = it->second; g_hplans.erase(it); }
    }
    if (!hp) { fail("numeric phase: unknown handle %lld", (long long)handle); return; }
    cudaStream_t st = lib_stream();
    Arr crd, val;
    int rc = get1d("C2crd", C2crd_rank, C2crd_ptr, isz, &crd) || get1d("Cval", Cval_rank, Cval_ptr, g_vsz, &val);
    if (!rc && (hp->isz != isz || hp->vsz != g_vsz))
        rc = fail("numeric phase: the handle was created by the entry point of another index or value width");
    if (!rc && (crd.n < hp->nnz || val.n < hp->nnz)) rc = fail("numeric phase: C2crd/Cval shorter than nnz");
    int64_t *dcrd = nullptr;
    double *dval = nullptr;
    if (!rc && cudaMallocAsync((void **)&dcrd, (size_t)(hp->nnz ? hp->nnz : 1) * 8, st) != cudaSuccess)
        rc = fail("numeric phase: device allocation failed");
    if (!rc && cudaMallocAsync((void **)&dval, (size_t)(hp->nnz ? hp->nnz : 1) * 8, st) != cudaSuccess)
        rc = fail("numeric phase: device allocation failed");
    if (!rc) rc = comet_b200_dev_spgemm_numeric_f64_i64(hp->dev_handle, dcrd, dval, 0, st);
    else comet_b200_handle_destroy(hp->dev_handle);
    int32_t *dcrd32 = nullptr;
    if (!rc && hp->nnz && isz == 4) {
        if (cudaMallocAsync((void **)&dcrd32, (size_t)hp->nnz * 4, st) != cudaSuccess)
            rc = fail("numeric phase: device allocation failed");
        if (!rc) rc = narrow_any_i64_to_i32(dcrd, dcrd32, hp->nnz, st);
    }
    float *dval32 = nullptr;
    if (!rc && hp->nnz && g_vsz == 4) {
        if (cudaMallocAsync((void **)&dval32, (size_t)hp->nnz * 4, st) != cudaSuccess)
            rc = fail("numeric phase: device allocation failed");
        if (!rc) rc = narrow_f64_to_f32(dval, dval32, hp->nnz, st);
    }
    if (!rc && hp->nnz) {
        if (d2h(crd.data, isz == 4 ? (void *)dcrd32 : (void *)dcrd, (size_t)hp->nnz * isz, st) ||
            d2h(val.data, g_vsz == 4 ? (void *)dval32 : (void *)dval, (size_t)hp->nnz * g_vsz, st))
            rc = 1;
    }
    if (finish(st) && !rc) fail("numeric phase: synchronize failed");
    if (dcrd) cudaFreeAsync(dcrd, st);
    if (dcrd32) cudaFreeAsync(dcrd32, st);
    if (dval32) cudaFreeAsync(dval32, st);
    if (dval) cudaFreeAsync(dval, st);
    for (void *p : hp->owned) cudaFreeAsync(p, st);
    delete hp;
}

// Sharded: A and M are this rank's row block, B the replicated operand; out[0] receives the count over
// ALL ranks' blocks (an all-reduce on the stream of the counting kernels).
static void masked_count_impl(int mode, COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B),
                              COMET_B200_SPARSE2D(M), int32_t mask_type, int32_t semiring, int64_t out_rank,
                              void *out_ptr)
{
    UNUSED_TILES(A);
    UNUSED_TILES(B);
    UNUSED_TILES(M);
    clear_error();
    const int isz = mode & 15;
    Comm *cm;
    if (mode_comm(mode, &cm)) return;
    cudaStream_t st;
    if (need_stream(&st)) return;
    ShardGuard guard(cm, st);
    HostSparse A, B, M;
    Arr out;
    DevBag bag(st);
    DevSparse dA, dB, dM;
    memset(&dM, 0, sizeof(dM));
    int rc = GET_SPARSE("masked count: A", A, &A) || GET_SPARSE("masked count: B", B, &B) ||
             GET_SPARSE("masked count: M", M, &M);
    if (!rc && (get1d("masked count: out", out_rank, out_ptr, 8, &out) || out.n < 1))
        rc = fail("masked count: out must hold one int64");
    if (!rc && (mask_type != COMET_B200_MASK_PUSH || semiring != COMET_B200_PLUS_PAIR))
        rc = fail("masked count: only the push mask with the plus-pair semiring is handled");
    if (!rc && (A.fmt != F_CSR || B.fmt != F_CSR || M.fmt != F_CSR)) rc = fail("masked count: operands must be CSR");
    if (!rc && (B.nrows < A.ncols || M.nrows < A.nrows)) rc = fail("masked count: shapes do not match");
    const bool sharded = cm && cm->nranks > 1;
    const bool b_is_a = !rc && !sharded && B.a2pos == A.a2pos && B.a2crd == A.a2crd;
    const bool m_is_a = !rc && M.a2pos == A.a2pos && M.a2crd == A.a2crd;
    const bool m_is_b = !rc && !m_is_a && !sharded && M.a2pos == B.a2pos && M.a2crd == B.a2crd;
    if (!rc) rc = upload_sparse("A", A, bag, &dA, false);
    if (!rc) {
        if (m_is_a) dM = dA;
        else if (!m_is_b) rc = upload_sparse("M", M, bag, &dM, false);
    }
    if (guard.agree(rc)) return;
    if (b_is_a) dB = dA;
    else if (upload_sparse("B", B, bag, &dB, false, cm)) return;
    if (m_is_b) dM = dB;
    int64_t *dcount;
    if (bag.alloc((void **)&dcount, 8)) return;
    if (comet_b200_dev_masked_spgemm_count_f64_i64(0, A.nrows, B.ncols, A.nnz, B.nnz, M.nnz, dA.pos, dA.crd,
                                                   dB.pos, dB.crd, dM.pos, dM.crd, dcount, st))
        return;
    if (comm_allreduce_sum_i64(cm, dcount, 1, st)) return;
    if (cudaMemcpyAsync(out.data, dcount, 8, cudaMemcpyDeviceToHost, st) != cudaSuccess) { fail("masked count: copy failed"); return; }
    finish(st);
}

// ---------------------------------------------------------------------------
// Exported symbols: one per index width.  COMET's CPU target uses i64 indices
// (frontends/comet_dsl/comet.cpp:817-823); cometpy keeps scipy's int32 index
// arrays and then instantiates the _i32 symbols
// (frontends/numpy-scipy/cometpy/comet.py:198-218).  Narrow indices are widened
// on the device, so both widths run the same kernels.
// ---------------------------------------------------------------------------
extern "C" {

#define BOTH_WIDTHS(RET, NAME, IMPL, PARAMS, ...)                           \
    RET comet_b200_##NAME##_f64_i64 PARAMS { return IMPL(8, __VA_ARGS__); } \
    RET comet_b200_##NAME##_f64_i32 PARAMS { return IMPL(4, __VA_ARGS__); }

BOTH_WIDTHS(void, spmv, spmv_impl,
            (COMET_B200_SPARSE2D(A), int64_t x_rank, void *x_ptr, int64_t y_rank, void *y_ptr, int32_t semiring,
             int32_t accumulate),
            FWD_SPARSE(A), x_rank, x_ptr, y_rank, y_ptr, semiring, accumulate)
BOTH_WIDTHS(void, spmm, spmm_impl,
            (COMET_B200_SPARSE2D(A), int64_t B_rank, void *B_ptr, int64_t C_rank, void *C_ptr, int32_t semiring,
             int32_t accumulate),
            FWD_SPARSE(A), B_rank, B_ptr, C_rank, C_ptr, semiring, accumulate)
BOTH_WIDTHS(void, dense_times_sparse, dense_sparse_impl,
            (int64_t A_rank, void *A_ptr, COMET_B200_SPARSE2D(B), int64_t C_rank, void *C_ptr, int32_t semiring,
             int32_t accumulate),
            A_rank, A_ptr, FWD_SPARSE(B), C_rank, C_ptr, semiring, accumulate)
BOTH_WIDTHS(void, sddmm, sddmm_impl,
            (COMET_B200_SPARSE2D(S), int64_t X_rank, void *X_ptr, int64_t D_rank, void *D_ptr, COMET_B200_SPARSE2D(O)),
            FWD_SPARSE(S), X_rank, X_ptr, D_rank, D_ptr, FWD_SPARSE(O))
BOTH_WIDTHS(void, elews_mul_sparse_dense, elews_sd_impl,
            (COMET_B200_SPARSE2D(A), int64_t B_rank, void *B_ptr, COMET_B200_SPARSE2D(C)),
            FWD_SPARSE(A), B_rank, B_ptr, FWD_SPARSE(C))
BOTH_WIDTHS(void, elews_mul_sparse_dense_to_dense, elews_to_dense_impl,
            (COMET_B200_SPARSE2D(A), int64_t B_rank, void *B_ptr, int64_t C_rank, void *C_ptr),
            FWD_SPARSE(A), B_rank, B_ptr, C_rank, C_ptr)
BOTH_WIDTHS(int64_t, spgemm_symbolic, spgemm_symbolic_impl,
            (COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), COMET_B200_SPARSE2D(M), int32_t mask_type, int32_t semiring,
             int64_t C2pos_rank, void *C2pos_ptr, int64_t sizes_rank, void *sizes_ptr),
            FWD_SPARSE(A), FWD_SPARSE(B), FWD_SPARSE(M), mask_type, semiring, C2pos_rank ,
                C2pos_ptr, sizes_rank, sizes_ptr)
BOTH_WIDTHS(int64_t, elews_mul_sparse_sparse_symbolic, elews_ss_symbolic_impl,
            (COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), int64_t C2pos_rank, void *C2pos_ptr, int64_t sizes_rank,
             void *sizes_ptr),
            FWD_SPARSE(A), FWD_SPARSE(B), C2pos_rank, C2pos_ptr, sizes_rank, sizes_ptr)
BOTH_WIDTHS(void, spgemm_numeric, spgemm_numeric_impl,
            (int64_t handle, int64_t C2crd_rank, void *C2crd_ptr, int64_t Cval_rank, void *Cval_ptr),
            handle, C2crd_rank, C2crd_ptr, Cval_rank, Cval_ptr)
BOTH_WIDTHS(void, masked_spgemm_count, masked_count_impl,
            (COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), COMET_B200_SPARSE2D(M), int32_t mask_type, int32_t semiring,
             int64_t out_rank, void *out_ptr),
            FWD_SPARSE(A), FWD_SPARSE(B), FWD_SPARSE(M), mask_type, semiring, out_rank, out_ptr)

// float values (COMET instantiates _f32_ runtime symbols next to the _f64_ ones,
// lib/ExecutionEngine/SparseUtils.cpp:2354-2400): same implementations with 4-byte values in the host memrefs.
#define F32_WIDTHS(RET, NAME, IMPL, PARAMS, ...)                                                    \
    RET comet_b200_##NAME##_f32_i64 PARAMS { ValueWidth w_(4); return IMPL(8, __VA_ARGS__); }       \
    RET comet_b200_##NAME##_f32_i32 PARAMS { ValueWidth w_(4); return IMPL(4, __VA_ARGS__); }

F32_WIDTHS(void, spmv, spmv_impl,
           (COMET_B200_SPARSE2D(A), int64_t x_rank, void *x_ptr, int64_t y_rank, void *y_ptr, int32_t semiring,
            int32_t accumulate),
           FWD_SPARSE(A), x_rank, x_ptr, y_rank, y_ptr, semiring, accumulate)
F32_WIDTHS(void, spmm, spmm_impl,
           (COMET_B200_SPARSE2D(A), int64_t B_rank, void *B_ptr, int64_t C_rank, void *C_ptr, int32_t semiring,
            int32_t accumulate),
           FWD_SPARSE(A), B_rank, B_ptr, C_rank, C_ptr, semiring, accumulate)
F32_WIDTHS(void, sddmm, sddmm_impl,
           (COMET_B200_SPARSE2D(S), int64_t X_rank, void *X_ptr, int64_t D_rank, void *D_ptr, COMET_B200_SPARSE2D(O)),
           FWD_SPARSE(S), X_rank, X_ptr, D_rank, D_ptr, FWD_SPARSE(O))
F32_WIDTHS(int64_t, spgemm_symbolic, spgemm_symbolic_impl,
           (COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), COMET_B200_SPARSE2D(M), int32_t mask_type, int32_t semiring,
            int64_t C2pos_rank, void *C2pos_ptr, int64_t sizes_rank, void *sizes_ptr),
           FWD_SPARSE(A), FWD_SPARSE(B), FWD_SPARSE(M), mask_type, semiring, C2pos_rank,
           C2pos_ptr, sizes_rank, sizes_ptr)
F32_WIDTHS(void, spgemm_numeric, spgemm_numeric_impl,
           (int64_t handle, int64_t C2crd_rank, void *C2crd_ptr, int64_t Cval_rank, void *Cval_ptr),
           handle, C2crd_rank, C2crd_ptr, Cval_rank, Cval_ptr)

// The same operations on one row block per rank, under the communicator of comet_b200_comm_init.
#define SHARDED_WIDTHS(RET, NAME, IMPL, PARAMS, ...)                                              \
    RET comet_b200_##NAME##_sharded_f64_i64 PARAMS { return IMPL(8 | MODE_SHARDED, __VA_ARGS__); } \
    RET comet_b200_##NAME##_sharded_f64_i32 PARAMS { return IMPL(4 | MODE_SHARDED, __VA_ARGS__); }

SHARDED_WIDTHS(void, spmm, spmm_impl,
               (COMET_B200_SPARSE2D(A), int64_t B_rank, void *B_ptr, int64_t C_rank, void *C_ptr, int32_t semiring,
                int32_t accumulate),
               FWD_SPARSE(A), B_rank, B_ptr, C_rank, C_ptr, semiring, accumulate)
SHARDED_WIDTHS(void, sddmm, sddmm_impl,
               (COMET_B200_SPARSE2D(S), int64_t X_rank, void *X_ptr, int64_t D_rank, void *D_ptr, COMET_B200_SPARSE2D(O)),
               FWD_SPARSE(S), X_rank, X_ptr, D_rank, D_ptr, FWD_SPARSE(O))
SHARDED_WIDTHS(int64_t, spgemm_symbolic, spgemm_symbolic_impl,
               (COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), COMET_B200_SPARSE2D(M), int32_t mask_type, int32_t semiring,
                int64_t C2pos_rank, void *C2pos_ptr, int64_t sizes_rank, void *sizes_ptr),
               FWD_SPARSE(A), FWD_SPARSE(B), FWD_SPARSE(M), mask_type, semiring, C2pos_rank,
               C2pos_ptr, sizes_rank, sizes_ptr)
SHARDED_WIDTHS(void, masked_spgemm_count, masked_count_impl,
               (COMET_B200_SPARSE2D(A), COMET_B200_SPARSE2D(B), COMET_B200_SPARSE2D(M), int32_t mask_type, int32_t semiring,
                int64_t out_rank, void *out_ptr),
               FWD_SPARSE(A), FWD_SPARSE(B), FWD_SPARSE(M), mask_type, semiring, out_rank, out_ptr)

}  // extern "C"

#define TRANSPOSE_ARGS                                                                                               \
    int32_t A1format, int32_t A1tile_format, int32_t A2format, int32_t A2tile_format, int64_t A1pos_rank,            \
        void *A1pos_ptr, int64_t A1crd_rank, void *A1crd_ptr, int64_t A1tile_pos_rank, void *A1tile_pos_ptr,         \
        int64_t A1tile_crd_rank, void *A1tile_crd_ptr, int64_t A2pos_rank, void *A2pos_ptr, int64_t A2crd_rank,      \
        void *A2crd_ptr, int64_t A2tile_pos_rank, void *A2tile_pos_ptr, int64_t A2tile_crd_rank,                     \
        void *A2tile_crd_ptr, int64_t Aval_rank, void *Aval_ptr, int32_t B1format, int32_t B1tile_format,            \
        int32_t B2format, int32_t B2tile_format, int64_t B1pos_rank, void *B1pos_ptr, int64_t B1crd_rank,            \
        void *B1crd_ptr, int64_t B1tile_pos_rank, void *B1tile_pos_ptr, int64_t B1tile_crd_rank,                     \
        void *B1tile_crd_ptr, int64_t B2pos_rank, void *B2pos_ptr, int64_t B2crd_rank, void *B2crd_ptr,              \
        int64_t B2tile_pos_rank, void *B2tile_pos_ptr, int64_t B2tile_crd_rank, void *B2tile_crd_ptr,                \
        int64_t Bval_rank, void *Bval_ptr, int64_t sizes_rank, void *sizes_ptr
#define TRANSPOSE_BODY(ISZ)                                                                                          \
    (void)A1tile_format; (void)A2tile_format; (void)A1tile_pos_rank; (void)A1tile_pos_ptr; (void)A1tile_crd_rank;    \
    (void)A1tile_crd_ptr; (void)A2tile_pos_rank; (void)A2tile_pos_ptr; (void)A2tile_crd_rank; (void)A2tile_crd_ptr;  \
    (void)B1tile_format; (void)B2tile_format; (void)B1tile_pos_rank; (void)B1tile_pos_ptr; (void)B1tile_crd_rank;    \
    (void)B1tile_crd_ptr; (void)B2tile_pos_rank; (void)B2tile_pos_ptr; (void)B2tile_crd_rank; (void)B2tile_crd_ptr;  \
    transpose_impl(ISZ, A1format, A2format, A1pos_rank, A1pos_ptr, A1crd_rank, A1crd_ptr, A2pos_rank, A2pos_ptr,     \
                   A2crd_rank, A2crd_ptr, Aval_rank, Aval_ptr, B1format, B2format, B1pos_rank, B1pos_ptr,            \
                   B1crd_rank, B1crd_ptr, B2pos_rank, B2pos_ptr, B2crd_rank, B2crd_ptr, Bval_rank, Bval_ptr,         \
                   sizes_rank, sizes_ptr)

extern "C" void comet_b200_transpose_2D_f64_i64(TRANSPOSE_ARGS) { TRANSPOSE_BODY(8); }
extern "C" void comet_b200_transpose_2D_f64_i32(TRANSPOSE_ARGS) { TRANSPOSE_BODY(4); }

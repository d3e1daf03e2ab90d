// MatrixMarket entry lines parsed on the device.
//
// The host reads the file, parses the banner and the size line (a few dozen bytes) and uploads the rest
// of the text.  Three kernels then do what the reference's single-thread parser does line by line
// (lib/ExecutionEngine/SparseUtils.cpp:145-356):
//   1. count : every CTA counts the entry lines that START in its slice of the text (a line starts after
//              a newline; comment lines, which begin with '%', and blank lines do not count);
//   2. (exclusive scan of the per-CTA counts)
//   3. index : the same walk again, now writing the byte offset of entry line number k to line_off[k];
//   4. parse : one thread per line runs the line parser of mtxparse.cuh and writes row, column, value
//              and a status; a line the device parser does not take exactly (see that file) is flagged
//              and re-parsed by the host with strtoll / strtod, so the values are the reference's bit for bit.
// A `symmetric` banner doubles every off-diagonal entry right behind the entry itself, as the reference
// does; the second scan over (1 or 2) per line places them.
#include <stdlib.h>

#include <string>
#include <vector>

#include "common.cuh"
#include "hostcopy.cuh"
#include "mtxparse.cuh"

namespace cb200 {

static const int PL_THREADS = 256;
static const int PL_BYTES = 32;                        // text bytes per thread
static const int PL_SLICE = PL_THREADS * PL_BYTES;     // text bytes per CTA

// Does an entry line start at byte i?  (first byte of the text or the byte after a newline; not a comment,
// not blank)
__device__ __forceinline__ bool entry_line_starts(const char *__restrict__ text, int64_t n, int64_t i)
{
    if (i > 0 && text[i - 1] != '\n') return false;
    if (text[i] == '%') return false;
    for (int64_t j = i; j < n; j++) {
        const char ch = text[j];
        if (ch == '\n') return false;
        if (ch != ' ' && ch != '\t' && ch != '\r') return true;
    }
    return false;
}

template <bool WRITE>
__global__ void __launch_bounds__(PL_THREADS)
mtx_lines_kernel(const char *__restrict__ text, int64_t n, int64_t *__restrict__ cta_count,
                 const int64_t *__restrict__ cta_base, int64_t *__restrict__ line_off)
{
    __shared__ int warp_sum[PL_THREADS / 32];
    const int64_t s0 = (int64_t)blockIdx.x * PL_SLICE + (int64_t)threadIdx.x * PL_BYTES;
    int mine = 0;
    unsigned mask = 0;
    for (int b = 0; b < PL_BYTES; b++) {
        const int64_t i = s0 + b;
        if (i < n && entry_line_starts(text, n, i)) { mine++; mask |= 1u << b; }
    }
    // block-wide exclusive prefix of `mine`
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) warp_sum[w] = incl;
    __syncthreads();
    int before = 0, total = 0;
    for (int i = 0; i < PL_THREADS / 32; i++) {
        if (i < w) before += warp_sum[i];
        total += warp_sum[i];
    }
    if (!WRITE) {
        if (threadIdx.x == 0) cta_count[blockIdx.x] = total;
        return;
    }
    int64_t at = cta_base[blockIdx.x] + before + incl - mine;
    for (int b = 0; b < PL_BYTES; b++)
        if (mask & (1u << b)) line_off[at++] = s0 + b;
}

// status per line: PARSE_OK, or PARSE_HOST / PARSE_BAD (both re-parsed by the host); copies[k] = entries the
// line yields (2 for an off-diagonal entry of a symmetric file)
__global__ void __launch_bounds__(256)
mtx_parse_kernel(const char *__restrict__ text, int64_t n, const int64_t *__restrict__ line_off, int64_t nlines,
                 int array, int symmetric, int64_t nrows, int64_t *__restrict__ row, int64_t *__restrict__ col,
                 double *__restrict__ val, int *__restrict__ status, int64_t *__restrict__ copies)
{
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < nlines; k += (int64_t)gridDim.x * blockDim.x) {
        const char *p = text + line_off[k];
        const char *e = p;
        const char *lim = text + n;
        while (e < lim && *e != '\n') e++;
        int64_t r = 0, c = 0;
        double v = 0.0;
        const int st = mtx_parse_entry(p, e, array != 0, &r, &c, &v);
        if (array) {                                   // dense listing, column by column
            c = nrows ? k / nrows : 0;
            r = k - nrows * c;
        } else {
            r -= 1;
            c -= 1;
        }
        row[k] = r; col[k] = c; val[k] = v;
        status[k] = st;
        copies[k] = (symmetric && r != c) ? 2 : 1;
    }
}

// entries in file order, the mirror of an off-diagonal entry of a symmetric file right behind it
__global__ void __launch_bounds__(256)
mtx_expand_kernel(int64_t nlines, const int64_t *__restrict__ at, const int64_t *__restrict__ row,
                  const int64_t *__restrict__ col, const double *__restrict__ val, int skew, int64_t *__restrict__ orow,
                  int64_t *__restrict__ ocol, double *__restrict__ oval)
{
    for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < nlines; k += (int64_t)gridDim.x * blockDim.x) {
        const int64_t o = at[k];
        orow[o] = row[k]; ocol[o] = col[k]; oval[o] = val[k];
        if (at[k + 1] - o == 2) { orow[o + 1] = col[k]; ocol[o + 1] = row[k]; oval[o + 1] = skew ? -val[k] : val[k]; }
    }
}

struct DevFree {
    cudaStream_t st;
    std::vector<void *> p;
    ~DevFree() { for (void *q : p) cudaFreeAsync(q, st); }
    template <class T> int get(T **out, size_t n)
    {
        if (cudaMallocAsync((void **)out, (n ? n : 1) * sizeof(T), st) != cudaSuccess) {
            *out = nullptr;
            return fail("reader: device allocation of %zu bytes failed", n * sizeof(T));
        }
        p.push_back(*out);
        return 0;
    }
};

// body: the text after the size line.  On success *drow / *dcol / *dval (stream-ordered allocations the
// caller frees) hold *count coordinate entries in file order.  `path` only labels error messages.
int parse_market_body_on_device(const char *path, const char *body, int64_t nbytes, bool array, bool symmetric,
                                bool skew, int64_t nrows, int64_t ncols, int64_t capacity, int64_t **drow,
                                int64_t **dcol, double **dval, int64_t *count, cudaStream_t st)
{
    *drow = *dcol = nullptr;
    *dval = nullptr;
    *count = 0;
    if (nbytes <= 0) return 0;
    DevFree tmp{st, {}};
    char *text = nullptr;
    CB_TRY(tmp.get(&text, (size_t)nbytes));
    CB_TRY(h2d(text, body, (size_t)nbytes, st));
    const int64_t nctas = ceil_div(nbytes, PL_SLICE);
    int64_t *cta_count = nullptr, *cta_base = nullptr;
    CB_TRY(tmp.get(&cta_count, (size_t)nctas));
    CB_TRY(tmp.get(&cta_base, (size_t)nctas + 1));
    mtx_lines_kernel<false><<<(unsigned)nctas, PL_THREADS, 0, st>>>(text, nbytes, cta_count, nullptr, nullptr);
    CB_LAUNCH_CHECK();
    CB_TRY(exclusive_scan_i64(cta_count, cta_base, nctas, st));
    int64_t nlines = 0;
    CB_CUDA(cudaMemcpyAsync(&nlines, cta_base + nctas, 8, cudaMemcpyDeviceToHost, st));
    CB_CUDA(cudaStreamSynchronize(st));
    if (nlines == 0) return 0;
    if (!symmetric && nlines > capacity) return fail("reader: %s: more entries than the size line announces", path);
    int64_t *line_off = nullptr, *row = nullptr, *col = nullptr, *copies = nullptr, *at = nullptr;
    double *val = nullptr;
    int *status = nullptr;
    CB_TRY(tmp.get(&line_off, (size_t)nlines));
    CB_TRY(tmp.get(&row, (size_t)nlines));
    CB_TRY(tmp.get(&col, (size_t)nlines));
    CB_TRY(tmp.get(&val, (size_t)nlines));
    CB_TRY(tmp.get(&status, (size_t)nlines));
    CB_TRY(tmp.get(&copies, (size_t)nlines));
    CB_TRY(tmp.get(&at, (size_t)nlines + 1));
    mtx_lines_kernel<true><<<(unsigned)nctas, PL_THREADS, 0, st>>>(text, nbytes, nullptr, cta_base, line_off);
    CB_LAUNCH_CHECK();
    int64_t grid = ceil_div(nlines, 256);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (grid > cap) grid = cap;
    mtx_parse_kernel<<<(unsigned)grid, 256, 0, st>>>(text, nbytes, line_off, nlines, array, symmetric, nrows, row, col, val,
                                                     status, copies);
    CB_LAUNCH_CHECK();

    // lines the device parser did not take: the host parses them the way the reference does
    std::vector<int> hstatus((size_t)nlines);
    CB_CUDA(cudaMemcpyAsync(hstatus.data(), status, (size_t)nlines * sizeof(int), cudaMemcpyDeviceToHost, st));
    CB_CUDA(cudaStreamSynchronize(st));
    std::vector<int64_t> fix_k;
    for (int64_t k = 0; k < nlines; k++)
        if (hstatus[(size_t)k] != PARSE_OK) fix_k.push_back(k);
    if (!fix_k.empty()) {
        std::vector<int64_t> offs((size_t)nlines);
        CB_CUDA(cudaMemcpyAsync(offs.data(), line_off, (size_t)nlines * 8, cudaMemcpyDeviceToHost, st));
        CB_CUDA(cudaStreamSynchronize(st));
        for (int64_t k : fix_k) {
            const char *p = body + offs[(size_t)k], *e = p;
            while (e < body + nbytes && *e != '\n') e++;
            std::string line(p, e);
            char *l = &line[0], *t = nullptr;
            int64_t r, c;
            double v;
            if (array) {
                v = strtod(l, nullptr);
                c = nrows ? k / nrows : 0;
                r = k - nrows * c;
            } else {
                r = strtoll(l, &t, 0);
                if (t == l) return fail("reader: %s: bad entry line", path);
                l = t;
                c = strtoll(l, &t, 0);
                if (t == l) return fail("reader: %s: bad entry line", path);
                l = t;
                v = strtod(l, &t);
                if (t == l) v = 1.0;
                r -= 1;
                c -= 1;
            }
            const int64_t two = (symmetric && r != c) ? 2 : 1;
            CB_CUDA(cudaMemcpyAsync(row + k, &r, 8, cudaMemcpyHostToDevice, st));
            CB_CUDA(cudaMemcpyAsync(col + k, &c, 8, cudaMemcpyHostToDevice, st));
            CB_CUDA(cudaMemcpyAsync(val + k, &v, 8, cudaMemcpyHostToDevice, st));
            CB_CUDA(cudaMemcpyAsync(copies + k, &two, 8, cudaMemcpyHostToDevice, st));
            CB_CUDA(cudaStreamSynchronize(st));          // the sources are locals of this iteration
        }
    }

    // every coordinate inside the matrix?  (reported with the offending entry, like the host parser)
    int *flag = nullptr;
    CB_TRY(tmp.get(&flag, 1));
    int ok = 1;
    CB_CUDA(cudaMemcpyAsync(flag, &ok, sizeof(int), cudaMemcpyHostToDevice, st));
    CB_TRY(check_index_range(row, nlines, nrows, flag, st));
    CB_TRY(check_index_range(col, nlines, ncols, flag, st));
    CB_CUDA(cudaMemcpyAsync(&ok, flag, sizeof(int), cudaMemcpyDeviceToHost, st));
    CB_CUDA(cudaStreamSynchronize(st));
    if (!ok) {
        std::vector<int64_t> hr((size_t)nlines), hc((size_t)nlines);
        CB_CUDA(cudaMemcpyAsync(hr.data(), row, (size_t)nlines * 8, cudaMemcpyDeviceToHost, st));
        CB_CUDA(cudaMemcpyAsync(hc.data(), col, (size_t)nlines * 8, cudaMemcpyDeviceToHost, st));
        CB_CUDA(cudaStreamSynchronize(st));
        for (int64_t k = 0; k < nlines; k++)
            if (hr[(size_t)k] < 0 || hr[(size_t)k] >= nrows || hc[(size_t)k] < 0 || hc[(size_t)k] >= ncols)
                return fail("reader: %s: entry (%lld, %lld) outside %lld x %lld", path, (long long)hr[(size_t)k] + 1,
                            (long long)hc[(size_t)k] + 1, (long long)nrows, (long long)ncols);
    }

    CB_TRY(exclusive_scan_i64(copies, at, nlines, st));
    int64_t total = 0;
    CB_CUDA(cudaMemcpyAsync(&total, at + nlines, 8, cudaMemcpyDeviceToHost, st));
    CB_CUDA(cudaStreamSynchronize(st));
    if (total > capacity) return fail("reader: %s: more entries than the size line announces", path);
    int rc = 0;
    if (cudaMallocAsync((void **)drow, (size_t)total * 8, st) != cudaSuccess ||
        cudaMallocAsync((void **)dcol, (size_t)total * 8, st) != cudaSuccess ||
        cudaMallocAsync((void **)dval, (size_t)total * 8, st) != cudaSuccess)
        rc = fail("reader: device allocation failed");
    if (!rc) {
        mtx_expand_kernel<<<(unsigned)grid, 256, 0, st>>>(nlines, at, row, col, val, skew, *drow, *dcol, *dval);
        if (cudaGetLastError() != cudaSuccess) rc = fail("reader: expand kernel failed");
    }
    if (rc) {
        if (*drow) cudaFreeAsync(*drow, st);
        if (*dcol) cudaFreeAsync(*dcol, st);
        if (*dval) cudaFreeAsync(*dval, st);
        *drow = *dcol = nullptr;
        *dval = nullptr;
        return rc;
    }
    *count = total;
    return 0;
}

}  // namespace cb200

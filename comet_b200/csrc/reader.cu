// MatrixMarket reader with the sort on the device: stands in for read_input_sizes_2D_f64 and
// read_input_2D_f64_{i64,i32} of the reference runtime (lib/ExecutionEngine/SparseUtils.cpp:1631-2078).
//
// The reference parses the file into coordinates (CooMatrix::InitMarket, :145-356: 1-based -> 0-based,
// a `symmetric` banner mirrors every off-diagonal entry right behind the entry itself, `skew` negates the
// mirror, a missing value reads as 1.0, `array` files list a dense matrix column by column), sorts them
// with std::stable_sort by (row, col) without merging duplicates (:360-367), and fills CSR / DCSR / COO
// arrays, for CSR and COO through the triangular filter of the read mode (:462-520, :1859-1893).
// Here the host reads the file and parses only the banner and the size line; the entry lines are parsed
// (parse.cu) and the coordinates sorted (convert.cu) on the device, and the linear fill of the caller's
// arrays runs on the host over the sorted entries.  A parsed and sorted file is kept per path,
// as the reference keeps its FileReaderWrapper per file id, so the sizes call and the fill call that
// follows share one parse and one sort.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"

namespace cb200 {

int sort_coo(int64_t n, int64_t nmajor, int64_t nminor, const int64_t *major, const int64_t *minor,
             const double *vals, int64_t *major_out, int64_t *minor_out, double *vals_out, cudaStream_t st);

struct SortedFile {
    int64_t nrows = 0, ncols = 0;
    std::vector<int64_t> row, col;      // sorted by (row, col), file order among equals
    std::vector<double> val;
};

static std::mutex g_files_mu;
static std::map<std::string, SortedFile *> g_files;

int parse_market_body_on_device(const char *path, const char *body, int64_t nbytes, bool array, bool symmetric,
                                bool skew, int64_t nrows, int64_t ncols, int64_t capacity, int64_t **drow,
                                int64_t **dcol, double **dval, int64_t *count, cudaStream_t st);

static bool blank(const char *s, const char *e)
{
    for (; s < e; s++)
        if (*s != ' ' && *s != '\t' && *s != '\r') return false;
    return true;
}

struct MarketHeader {
    bool symmetric = false, skew = false, array = false;
    int64_t nrows = 0, ncols = 0, capacity = 0;     // capacity: entries the size line allows (doubled for symmetric files)
    size_t body = 0;                                // offset of the first byte after the size line
};

// Banner, comments and the size line: the only part of the file the host parses.
static int parse_header(const std::string &path, const std::string &text, MarketHeader *h)
{
    const char *p = text.data(), *end = p + text.size();
    while (p < end) {
        const char *nl = (const char *)memchr(p, '\n', (size_t)(end - p));
        const char *le = nl ? nl : end;
        const char *next = nl ? nl + 1 : end;
        if (*p == '%') {
            if (p + 1 < le && p[1] == '%') {
                const std::string banner(p, le);
                h->symmetric = banner.find("symmetric") != std::string::npos;
                h->skew = banner.find("skew") != std::string::npos;
                h->array = banner.find("array") != std::string::npos;
            }
        } else if (!blank(p, le)) {
            std::string line(p, le);                    // NUL-terminated copy for strtoll
            char *l = &line[0], *t = nullptr;
            long long a = strtoll(l, &t, 10);
            if (t == l) return fail("reader: %s: bad size line", path.c_str());
            l = t;
            long long b = strtoll(l, &t, 10);
            if (t == l) return fail("reader: %s: bad size line", path.c_str());
            l = t;
            long long c = strtoll(l, &t, 10);
            if (h->array) {
                h->capacity = a * b;
            } else {
                if (t == l) return fail("reader: %s: the size line needs rows, columns and entries", path.c_str());
                h->capacity = h->symmetric ? 2 * c : c;
            }
            if (a < 0 || b < 0 || h->capacity < 0) return fail("reader: %s: negative size", path.c_str());
            h->nrows = a;
            h->ncols = b;
            h->body = (size_t)(next - text.data());
            return 0;
        }
        p = next;
    }
    return fail("reader: %s: no size line", path.c_str());
}

// read the file, parse its entry lines and sort the entries on the device, once per path
static SortedFile *open_sorted(int32_t file_id)
{
    char name[64];
    if (file_id >= 0 && file_id < 9999) snprintf(name, sizeof(name), "SPARSE_FILE_NAME%d", file_id);
    else if (file_id == 9999) snprintf(name, sizeof(name), "SPARSE_FILE_NAME");
    else { fail("reader: file id %d is out of range", file_id); return nullptr; }
    const char *path = getenv(name);
    if (!path || !*path) { fail("reader: environment variable %s is not set", name); return nullptr; }
    if (!strstr(path, ".mtx")) { fail("reader: %s is not a MatrixMarket (.mtx) file", path); return nullptr; }
    std::lock_guard<std::mutex> lk(g_files_mu);
    auto it = g_files.find(path);
    if (it != g_files.end()) return it->second;

    FILE *f = fopen(path, "rb");
    if (!f) { fail("reader: cannot open %s", path); return nullptr; }
    std::string text;
    {
        char buf[1 << 16];
        size_t got;
        while ((got = fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, got);
        fclose(f);
    }
    MarketHeader h;
    if (parse_header(path, text, &h)) return nullptr;
    SortedFile *m = new SortedFile();
    m->nrows = h.nrows;
    m->ncols = h.ncols;
    if (text.size() > h.body) {
        int ndev = 0;
        if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) {
            fail("no CUDA device is available; libcomet_b200 has no CPU path");
            delete m;
            return nullptr;
        }
        cudaStream_t st = lib_stream();
        int64_t *dr = nullptr, *dc = nullptr, n = 0;
        double *dv = nullptr, *dv2 = nullptr;
        bool ok = parse_market_body_on_device(path, text.data() + h.body, (int64_t)(text.size() - h.body), h.array,
                                              h.symmetric, h.skew, h.nrows, h.ncols, h.capacity, &dr, &dc, &dv, &n,
                                              st) == 0;
        if (ok && n > 0) {
            ok = cudaMallocAsync((void **)&dv2, (size_t)n * 8, st) == cudaSuccess;
            if (!ok) fail("reader: device allocation failed");
            // the coordinates are sorted in place (they are rebuilt from the keys); the values are gathered
            if (ok) ok = sort_coo(n, m->nrows, m->ncols, dr, dc, dv, dr, dc, dv2, st) == 0;
            if (ok) {
                m->row.resize((size_t)n); m->col.resize((size_t)n); m->val.resize((size_t)n);
                cudaMemcpyAsync(m->row.data(), dr, (size_t)n * 8, cudaMemcpyDeviceToHost, st);
                cudaMemcpyAsync(m->col.data(), dc, (size_t)n * 8, cudaMemcpyDeviceToHost, st);
                cudaMemcpyAsync(m->val.data(), dv2, (size_t)n * 8, cudaMemcpyDeviceToHost, st);
                if (cudaStreamSynchronize(st) != cudaSuccess) { fail("reader: copy of the sorted entries failed"); ok = false; }
            }
        }
        if (dr) cudaFreeAsync(dr, st);
        if (dc) cudaFreeAsync(dc, st);
        if (dv) cudaFreeAsync(dv, st);
        if (dv2) cudaFreeAsync(dv2, st);
        if (!ok) { delete m; return nullptr; }
    }
    g_files[path] = m;
    return m;
}

// triangular filters of the read modes (SparseUtils.cpp:462-520): 1 everything, 2 strictly lower,
// 3 lower incl. diagonal, 4 strictly upper, 5 upper incl. diagonal
static inline bool keep(int mode, int64_t r, int64_t c)
{
    switch (mode) {
    case 2: return r > c;
    case 3: return r >= c;
    case 4: return r < c;
    case 5: return r <= c;
    default: return true;
    }
}

static int64_t count_kept(const SortedFile *m, int mode)
{
    if (mode < 2 || mode > 5) return (int64_t)m->row.size();
    int64_t n = 0;
    for (size_t i = 0; i < m->row.size(); i++) n += keep(mode, m->row[i], m->col[i]);
    return n;
}

static int64_t stored_rows(const SortedFile *m)
{
    int64_t nr = 0, prev = -1;
    for (size_t i = 0; i < m->row.size(); i++)
        if (m->row[i] != prev) { nr++; prev = m->row[i]; }
    return nr;
}

struct IdxArr {
    char *data;
    int64_t n;
    int isz;
    void set(int64_t i, int64_t v) const
    {
        if (isz == 8) ((int64_t *)data)[i] = v; else ((int32_t *)data)[i] = (int32_t)v;
    }
};

static int get_idx(const char *what, int64_t rank, void *desc, int isz, IdxArr *out)
{
    out->data = nullptr; out->n = 0; out->isz = isz;
    if (!desc) return 0;
    if (rank != 1) return fail("%s: expected a rank-1 memref", what);
    comet_b200_memref1d *d = (comet_b200_memref1d *)desc;
    if (d->sizes[0] > 1 && d->strides[0] != 1) return fail("%s: stride must be 1", what);
    out->data = (char *)d->aligned + d->offset * isz;
    out->n = d->sizes[0];
    return 0;
}

static void read_sizes(int32_t file_id, int32_t f1, int32_t f2, int64_t sizes_rank, void *sizes_ptr, int32_t mode)
{
    clear_error();
    IdxArr s;
    if (get_idx("read_input_sizes: sizes", sizes_rank, sizes_ptr, 8, &s)) return;
    if (!s.data || s.n < 11) { fail("read_input_sizes: the sizes memref needs 11 entries"); return; }
    const SortedFile *m = open_sorted(file_id);
    if (!m) return;
    int64_t v[11] = {0, 0, 0, 0, 0, 0, 0, 0, 0, m->nrows, m->ncols};
    if (f1 == COMET_B200_FMT_CN && f2 == COMET_B200_FMT_S) {
        const int64_t nnz = count_kept(m, mode);
        v[0] = 2; v[1] = nnz; v[4] = 1; v[5] = nnz; v[8] = nnz;
    } else if (f1 == COMET_B200_FMT_DENSE && f2 == COMET_B200_FMT_CU) {
        const int64_t nnz = count_kept(m, mode);
        v[0] = 1; v[1] = 1; v[4] = m->nrows + 1; v[5] = nnz; v[8] = nnz;
    } else if (f1 == COMET_B200_FMT_CU && f2 == COMET_B200_FMT_CU) {   // DCSR holds every entry, whatever the read mode
        const int64_t nr = stored_rows(m), nnz = (int64_t)m->row.size();
        v[0] = 2; v[1] = nr; v[4] = nr + 1; v[5] = nnz; v[8] = nnz;
    } else {
        fail("read_input_sizes: unsupported format (%d, %d); CSR, DCSR and COO are handled", f1, f2);
        return;
    }
    for (int i = 0; i < 11; i++) s.set(i, v[i]);
}

static void read_fill(int isz, int32_t file_id, int32_t f1, int32_t f2, int64_t r1p, void *p1p, int64_t r1c, void *p1c,
                      int64_t r2p, void *p2p, int64_t r2c, void *p2c, int64_t rv, void *pv, int32_t mode)
{
    clear_error();
    IdxArr a1pos, a1crd, a2pos, a2crd, av;
    if (get_idx("read_input: A1pos", r1p, p1p, isz, &a1pos) || get_idx("read_input: A1crd", r1c, p1c, isz, &a1crd) ||
        get_idx("read_input: A2pos", r2p, p2p, isz, &a2pos) || get_idx("read_input: A2crd", r2c, p2c, isz, &a2crd) ||
        get_idx("read_input: Aval", rv, pv, 8, &av))
        return;
    const SortedFile *m = open_sorted(file_id);
    if (!m) return;
    double *val = (double *)av.data;
    const int64_t n = (int64_t)m->row.size();
    // placeholders of the arrays a format does not use (printed as -1 by the reference's tests)
    if (a1pos.data && a1pos.n > 0) a1pos.set(0, -1);
    if (a1crd.data && a1crd.n > 0) a1crd.set(0, -1);
    if (a2pos.data && a2pos.n > 0) a2pos.set(0, -1);
    if (f1 == COMET_B200_FMT_CN && f2 == COMET_B200_FMT_S) {
        const int64_t nnz = count_kept(m, mode);
        if (a1pos.n < 2 || a1crd.n < nnz || a2crd.n < nnz || av.n < nnz) { fail("read_input: COO arrays too short"); return; }
        int64_t at = 0;
        for (int64_t i = 0; i < n; i++) {
            if (!keep(mode, m->row[i], m->col[i])) continue;
            a1crd.set(at, m->row[i]); a2crd.set(at, m->col[i]); val[at] = m->val[i];
            at++;
        }
        a1pos.set(0, 0); a1pos.set(1, at);
    } else if (f1 == COMET_B200_FMT_DENSE && f2 == COMET_B200_FMT_CU) {
        const int64_t nnz = count_kept(m, mode);
        if (a1pos.n < 1 || a2pos.n < m->nrows + 1 || a2crd.n < nnz || av.n < nnz) { fail("read_input: CSR arrays too short"); return; }
        int64_t at = 0, next_row = 0;
        for (int64_t i = 0; i < n; i++) {
            if (!keep(mode, m->row[i], m->col[i])) continue;
            for (; next_row <= m->row[i]; next_row++) a2pos.set(next_row, at);
            a2crd.set(at, m->col[i]); val[at] = m->val[i];
            at++;
        }
        for (; next_row <= m->nrows; next_row++) a2pos.set(next_row, at);
        a1pos.set(0, m->nrows);
    } else if (f1 == COMET_B200_FMT_CU && f2 == COMET_B200_FMT_CU) {
        const int64_t nr = stored_rows(m);
        if (a1pos.n < 2 || a1crd.n < nr || a2pos.n < nr + 1 || a2crd.n < n || av.n < n) { fail("read_input: DCSR arrays too short"); return; }
        int64_t at = 0, prev = -1;
        for (int64_t i = 0; i < n; i++) {
            if (m->row[i] != prev) { a2pos.set(at, i); a1crd.set(at, m->row[i]); at++; prev = m->row[i]; }
            a2crd.set(i, m->col[i]); val[i] = m->val[i];
        }
        a2pos.set(at, n);
        a1pos.set(0, 0); a1pos.set(1, at);
    } else {
        fail("read_input: unsupported format (%d, %d); CSR, DCSR and COO are handled", f1, f2);
    }
}

}  // namespace cb200

extern "C" void comet_b200_read_input_sizes_2D_f64(int32_t fileID, int32_t A1format, int32_t A1tile_format,
                                                   int32_t A2format, int32_t A2tile_format, int64_t sizes_rank,
                                                   void *sizes_ptr, int32_t readMode)
{
    (void)A1tile_format; (void)A2tile_format;
    cb200::read_sizes(fileID, A1format, A2format, sizes_rank, sizes_ptr, readMode);
}

#define READ_INPUT_ARGS                                                                                             \
    int32_t fileID, int32_t A1format, int32_t A1tile_format, int32_t A2format, int32_t A2tile_format,               \
        int64_t A1pos_rank, void *A1pos_ptr, int64_t A1crd_rank, void *A1crd_ptr, int64_t A1tile_pos_rank,          \
        void *A1tile_pos_ptr, int64_t A1tile_crd_rank, void *A1tile_crd_ptr, int64_t A2pos_rank, void *A2pos_ptr,   \
        int64_t A2crd_rank, void *A2crd_ptr, int64_t A2tile_pos_rank, void *A2tile_pos_ptr,                         \
        int64_t A2tile_crd_rank, void *A2tile_crd_ptr, int64_t Aval_rank, void *Aval_ptr, int32_t readMode
#define READ_INPUT_BODY(ISZ)                                                                                        \
    (void)A1tile_format; (void)A2tile_format; (void)A1tile_pos_rank; (void)A1tile_pos_ptr; (void)A1tile_crd_rank;   \
    (void)A1tile_crd_ptr; (void)A2tile_pos_rank; (void)A2tile_pos_ptr; (void)A2tile_crd_rank; (void)A2tile_crd_ptr; \
    cb200::read_fill(ISZ, fileID, A1format, A2format, A1pos_rank, A1pos_ptr, A1crd_rank, A1crd_ptr, A2pos_rank,     \
                     A2pos_ptr, A2crd_rank, A2crd_ptr, Aval_rank, Aval_ptr, readMode)

extern "C" void comet_b200_read_input_2D_f64_i64(READ_INPUT_ARGS) { READ_INPUT_BODY(8); }
extern "C" void comet_b200_read_input_2D_f64_i32(READ_INPUT_ARGS) { READ_INPUT_BODY(4); }

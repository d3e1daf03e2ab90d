// Multi-GPU plumbing of the library: one NCCL communicator per device, created from a unique id the
// host program distributes (one process per GPU), and the three collectives the sharded entry points
// need -- all-gather of a replicated operand's slices, all-gather of per-shard counts, all-reduce of
// a count.  NCCL is opened with dlopen on first use, so programs that stay on one GPU neither link
// nor load it.
//
// The path shards by contiguous row blocks of the left operand; the right operand (B, Y, L) is
// needed whole on every GPU.  Instead of every rank pushing all of it through its own PCIe link,
// each rank uploads one N-th and the slices are exchanged over NVLink into each GPU's OWN memory;
// the kernels then read local memory only (no peer pointers are handed to any kernel).
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "comm.cuh"

namespace cb200 {

namespace {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t,
                              cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*GetVersion)(int *) = nullptr;
};

NcclApi g_nccl;
std::mutex g_comm_mu;
Comm g_comm[64];

int load_nccl()
{
    if (g_nccl.handle) return 0;
    // a process that already holds NCCL (for instance through torch) gets that same copy back by soname
    const char *names[] = {"libnccl.so.2", "libnccl.so", nullptr};
    void *h = nullptr;
    for (int i = 0; names[i] && !h; i++) h = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
    if (!h) return fail("multi-GPU: libnccl.so.2 could not be loaded (%s)", dlerror());
#define SYM(field, name)                                                     \
    do {                                                                     \
        *(void **)(&g_nccl.field) = dlsym(h, name);                          \
        if (!g_nccl.field) return fail("multi-GPU: %s missing from NCCL", name); \
    } while (0)
    SYM(GetUniqueId, "ncclGetUniqueId");
    SYM(CommInitRank, "ncclCommInitRank");
    SYM(CommDestroy, "ncclCommDestroy");
    SYM(AllGather, "ncclAllGather");
    SYM(AllReduce, "ncclAllReduce");
    SYM(GetErrorString, "ncclGetErrorString");
    SYM(GetVersion, "ncclGetVersion");
#undef SYM
    g_nccl.handle = h;
    return 0;
}

#define CB_NCCL(expr)                                                                           \
    do {                                                                                        \
        ncclResult_t r_ = (expr);                                                               \
        if (r_ != ncclSuccess)                                                                  \
            return cb200::fail("%s failed: %s", #expr, g_nccl.GetErrorString ? g_nccl.GetErrorString(r_) : "?"); \
    } while (0)

Comm *slot()
{
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) return nullptr;
    return &g_comm[d];
}

}  // namespace

Comm *comm_current()
{
    Comm *c = slot();
    return (c && c->comm) ? c : nullptr;
}

size_t comm_slice_bytes(size_t total, int nranks)
{
    if (nranks < 1) nranks = 1;
    size_t s = (total + (size_t)nranks - 1) / (size_t)nranks;
    return (s + 255) & ~(size_t)255;     // slices start on 256-byte boundaries of the replicated buffer
}

int comm_allgather_inplace(Comm *c, void *buf, size_t slice_bytes, cudaStream_t st)
{
    if (!c || c->nranks == 1 || slice_bytes == 0) return 0;
    CB_NCCL(g_nccl.AllGather((const char *)buf + (size_t)c->rank * slice_bytes, buf, slice_bytes, ncclChar,
                             (ncclComm_t)c->comm, st));
    return 0;
}

int comm_allgather_i64(Comm *c, const int64_t *one, int64_t *all, cudaStream_t st)
{
    if (!c || c->nranks == 1) {
        CB_CUDA(cudaMemcpyAsync(all, one, sizeof(int64_t), cudaMemcpyDeviceToDevice, st));
        return 0;
    }
    CB_NCCL(g_nccl.AllGather(one, all, 1, ncclInt64, (ncclComm_t)c->comm, st));
    return 0;
}

int comm_allreduce_sum_i64(Comm *c, int64_t *buf, int64_t n, cudaStream_t st)
{
    if (!c || c->nranks == 1 || n <= 0) return 0;
    CB_NCCL(g_nccl.AllReduce(buf, buf, (size_t)n, ncclInt64, ncclSum, (ncclComm_t)c->comm, st));
    return 0;
}

}  // namespace cb200

using namespace cb200;

extern "C" {

int32_t comet_b200_comm_unique_id(void *id_out, int64_t id_bytes)
{
    clear_error();
    if (!id_out || id_bytes < (int64_t)sizeof(ncclUniqueId))
        return fail("comm_unique_id: the buffer must hold %d bytes", (int)sizeof(ncclUniqueId));
    CB_TRY(load_nccl());
    ncclUniqueId id;
    CB_NCCL(g_nccl.GetUniqueId(&id));
    memcpy(id_out, &id, sizeof(id));
    return 0;
}

int32_t comet_b200_comm_init(int32_t nranks, int32_t rank, const void *id_in)
{
    clear_error();
    if (nranks < 1 || rank < 0 || rank >= nranks) return fail("comm_init: rank %d of %d is not valid", rank, nranks);
    std::lock_guard<std::mutex> lk(g_comm_mu);
    Comm *c = slot();
    if (!c) return fail("comm_init: no usable CUDA device (the current device is the one the communicator binds to)");
    if (c->comm) return fail("comm_init: this device already holds a communicator; call comet_b200_comm_destroy first");
    if (nranks == 1) {              // nothing to exchange: the sharded entry points then behave like the plain ones
        c->nranks = 1;
        c->rank = 0;
        c->comm = (void *)c;
        return 0;
    }
    if (!id_in) return fail("comm_init: the unique id is missing");
    CB_TRY(load_nccl());
    ncclUniqueId id;
    memcpy(&id, id_in, sizeof(id));
    ncclComm_t comm = nullptr;
    CB_NCCL(g_nccl.CommInitRank(&comm, nranks, id, rank));
    c->comm = (void *)comm;
    c->nranks = nranks;
    c->rank = rank;
    return 0;
}

int32_t comet_b200_comm_nranks(void)
{
    Comm *c = comm_current();
    return c ? c->nranks : 0;
}

int32_t comet_b200_comm_rank(void)
{
    Comm *c = comm_current();
    return c ? c->rank : -1;
}

int32_t comet_b200_comm_destroy(void)
{
    clear_error();
    std::lock_guard<std::mutex> lk(g_comm_mu);
    Comm *c = slot();
    if (!c || !c->comm) return 0;
    if (c->nranks > 1) {
        cudaDeviceSynchronize();     // no collective of this communicator may still be in flight
        CB_NCCL(g_nccl.CommDestroy((ncclComm_t)c->comm));
    }
    c->comm = nullptr;
    c->nranks = 0;
    c->rank = 0;
    return 0;
}

int64_t comet_b200_comm_slice_bytes(int64_t total_bytes, int32_t nranks)
{
    return total_bytes < 0 ? 0 : (int64_t)comm_slice_bytes((size_t)total_bytes, nranks);
}

int32_t comet_b200_dev_allreduce_sum_i64(int64_t *buf, int64_t n, void *stream)
{
    clear_error();
    Comm *c = comm_current();
    if (!c) return fail("allreduce: no communicator on this device (comet_b200_comm_init comes first)");
    return comm_allreduce_sum_i64(c, buf, n, (cudaStream_t)stream);
}

int32_t comet_b200_dev_allgather_i64(const int64_t *one, int64_t *all, void *stream)
{
    clear_error();
    Comm *c = comm_current();
    if (!c) return fail("allgather: no communicator on this device (comet_b200_comm_init comes first)");
    return comm_allgather_i64(c, one, all, (cudaStream_t)stream);
}

int32_t comet_b200_dev_allgather_slices(void *buf, int64_t slice_bytes, void *stream)
{
    clear_error();
    Comm *c = comm_current();
    if (!c) return fail("allgather: no communicator on this device (comet_b200_comm_init comes first)");
    if (slice_bytes < 0) return fail("allgather: negative slice size");
    return comm_allgather_inplace(c, buf, (size_t)slice_bytes, (cudaStream_t)stream);
}

}

// Copies between HOST memrefs and the device for the host-memref entry points.
//
// COMET's generated code gets its memrefs from memref.alloc, i.e. malloc: pageable memory.  A
// cudaMemcpyAsync on pageable memory is staged by the driver through one internal buffer on the
// calling thread and reaches a fraction of the PCIe rate, and it is not asynchronous.  Here large
// copies on pageable memory go through a ring of page-locked chunks owned by the library instead:
// a few worker threads move the bytes between the caller's array and the chunks (several chunks in
// flight, so the memcpy bandwidth of several cores adds up) while the DMA engine moves chunks that are
// already filled, in stream order.  Page-locked (or registered) host memory and small copies take the
// plain cudaMemcpyAsync path.
//
//   h2d / h2d_2d : return when every byte of the host array has been read (like cudaMemcpyAsync on
//                  pageable memory); the device side is complete in stream order.
//   d2h / d2h_2d : return when every chunk's DMA has been enqueued; the bytes reach the host array
//                  on the worker threads.  copies_drain() waits for them and must be called (after
//                  the stream has been synchronised or not -- it waits on each chunk's own event)
//                  before the entry point returns to its caller.
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <mutex>
#include <string.h>
#include <thread>
#include <vector>

#include "common.cuh"
#include "hostcopy.cuh"

namespace cb200 {

namespace {

const size_t CHUNK = (size_t)4 << 20;     // bytes per page-locked chunk
const int SLOTS = 12;                     // chunks per device (48 MiB of page-locked memory)
const size_t STAGE_MIN_DEFAULT = (size_t)16 << 20;  // smaller copies are left to the driver (waking the workers costs more)

struct Slot {
    char *buf = nullptr;
    cudaEvent_t ev = nullptr;
    bool dma_pending = false;             // an H2D copy out of this chunk may still be running
};

struct Batch {                            // the chunks of one upload call
    int left = 0;
};

class Pool {
  public:
    explicit Pool(int device) : device_(device)
    {
        // half of the cores this process can count on: launchers that start one process per GPU export
        // LOCAL_WORLD_SIZE, and the processes of one node share its cores
        int share = 1;
        const char *lws = getenv("LOCAL_WORLD_SIZE");
        if (lws && atoi(lws) > 1) share = atoi(lws);
        int n = (int)std::thread::hardware_concurrency() / (2 * share);
        const char *env = getenv("COMET_B200_COPY_THREADS");
        if (env) n = atoi(env);
        if (n < 2) n = 2;
        if (n > 12) n = 12;
        for (int i = 0; i < SLOTS; i++) {
            Slot s;
            if (cudaHostAlloc((void **)&s.buf, CHUNK, cudaHostAllocDefault) != cudaSuccess) break;
            if (cudaEventCreateWithFlags(&s.ev, cudaEventDisableTiming) != cudaSuccess) { cudaFreeHost(s.buf); break; }
            slots_.push_back(s);
            free_.push_back((int)slots_.size() - 1);
        }
        for (int i = 0; i < n; i++) workers_.emplace_back([this] { work(); });
    }
    bool usable() const { return slots_.size() >= 2; }

    int acquire()
    {
        std::unique_lock<std::mutex> lk(mu_);
        cv_free_.wait(lk, [this] { return !free_.empty(); });
        const int i = free_.front();
        free_.pop_front();
        lk.unlock();
        if (slots_[i].dma_pending) {
            if (cudaEventSynchronize(slots_[i].ev) != cudaSuccess) failed_ = true;
            slots_[i].dma_pending = false;
        }
        return i;
    }
    void release(int i)
    {
        {
            std::lock_guard<std::mutex> lk(mu_);
            free_.push_back(i);
        }
        cv_free_.notify_one();
    }
    Slot &slot(int i) { return slots_[i]; }

    void submit(std::function<void()> fn, Batch *batch = nullptr)
    {
        {
            std::lock_guard<std::mutex> lk(mu_);
            tasks_.push_back(Task{std::move(fn), batch});
            pending_++;
            if (batch) batch->left++;
        }
        cv_task_.notify_one();
    }
    // waits until the tasks of one batch have run
    void wait(Batch *batch)
    {
        std::unique_lock<std::mutex> lk(mu_);
        cv_done_.wait(lk, [batch] { return batch->left == 0; });
    }
    bool take_failure() { return failed_.exchange(false); }
    // waits until every submitted task has run; returns non-zero if one of them failed
    int drain()
    {
        std::unique_lock<std::mutex> lk(mu_);
        cv_done_.wait(lk, [this] { return pending_ == 0; });
        const bool f = failed_.exchange(false);
        return f ? 1 : 0;
    }
    void fail_flag() { failed_ = true; }

  private:
    void work()
    {
        cudaSetDevice(device_);
        while (true) {
            Task t;
            {
                std::unique_lock<std::mutex> lk(mu_);
                cv_task_.wait(lk, [this] { return !tasks_.empty(); });
                t = std::move(tasks_.front());
                tasks_.pop_front();
            }
            t.fn();
            {
                std::lock_guard<std::mutex> lk(mu_);
                pending_--;
                if (t.batch) t.batch->left--;
                if (pending_ == 0 || (t.batch && t.batch->left == 0)) cv_done_.notify_all();
            }
        }
    }
    struct Task {
        std::function<void()> fn;
        Batch *batch = nullptr;
    };
    int device_;
    std::vector<Slot> slots_;
    std::deque<int> free_;
    std::deque<Task> tasks_;
    std::vector<std::thread> workers_;     // live until the process exits
    std::mutex mu_;
    std::condition_variable cv_free_, cv_task_, cv_done_;
    int pending_ = 0;
    std::atomic<bool> failed_{false};
};

std::mutex g_pool_mu;
Pool *g_pool[64] = {nullptr};

Pool *pool()
{
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(g_pool_mu);
    if (!g_pool[d]) g_pool[d] = new Pool(d);
    return g_pool[d]->usable() ? g_pool[d] : nullptr;
}

// COMET_B200_STAGED_COPIES=0 leaves every copy to the driver; COMET_B200_STAGE_MIN_BYTES moves the size from
// which pageable copies are staged (both read at every call: they are test and tuning knobs)
bool staging_enabled()
{
    const char *e = getenv("COMET_B200_STAGED_COPIES");
    return !(e && e[0] == '0');
}

size_t stage_min()
{
    const char *e = getenv("COMET_B200_STAGE_MIN_BYTES");
    if (e) {
        const long long v = atoll(e);
        if (v >= 0) return (size_t)v;
    }
    return STAGE_MIN_DEFAULT;
}

// rows x row_bytes, host rows `host_pitch` apart, device rows `dev_pitch` apart (a 1-D copy is one row cut
// into chunk-sized pieces by the callers below)
struct Piece {
    char *host;
    char *dev;
    size_t rows, row_bytes, host_pitch, dev_pitch;
};

void copy_rows(char *dst, size_t dpitch, const char *src, size_t spitch, size_t row_bytes, size_t rows)
{
    if (dpitch == row_bytes && spitch == row_bytes) {
        memcpy(dst, src, row_bytes * rows);
        return;
    }
    for (size_t r = 0; r < rows; r++) memcpy(dst + r * dpitch, src + r * spitch, row_bytes);
}

int staged(Pool *p, bool to_device, const Piece &pc, cudaStream_t st)
{
    Batch batch;
    // a chunk carries whole rows (packed), or a part of one row when a row is longer than a chunk
    const size_t rows_per_chunk = pc.row_bytes >= CHUNK ? 1 : CHUNK / pc.row_bytes;
    for (size_t r0 = 0; r0 < pc.rows; r0 += rows_per_chunk) {
        const size_t nr = pc.rows - r0 < rows_per_chunk ? pc.rows - r0 : rows_per_chunk;
        for (size_t b0 = 0; b0 < pc.row_bytes; b0 += CHUNK) {
            const size_t nb = pc.row_bytes - b0 < CHUNK ? pc.row_bytes - b0 : CHUNK;
            const int si = p->acquire();
            Slot &s = p->slot(si);
            char *host = pc.host + r0 * pc.host_pitch + b0;
            char *dev = pc.dev + r0 * pc.dev_pitch + b0;
            const size_t host_pitch = pc.host_pitch, dev_pitch = pc.dev_pitch;
            if (to_device) {
                p->submit([p, si, host, dev, nr, nb, host_pitch, dev_pitch, st] {
                    Slot &sl = p->slot(si);
                    copy_rows(sl.buf, nb, host, host_pitch, nb, nr);
                    cudaError_t e = cudaMemcpy2DAsync(dev, dev_pitch, sl.buf, nb, nb, nr, cudaMemcpyHostToDevice, st);
                    if (e == cudaSuccess) e = cudaEventRecord(sl.ev, st);
                    if (e != cudaSuccess) p->fail_flag();
                    sl.dma_pending = true;
                    p->release(si);
                }, &batch);
            } else {
                cudaError_t e = cudaMemcpy2DAsync(s.buf, nb, dev, dev_pitch, nb, nr, cudaMemcpyDeviceToHost, st);
                if (e == cudaSuccess) e = cudaEventRecord(s.ev, st);
                if (e != cudaSuccess) {
                    p->release(si);
                    return fail("staged copy to the host failed: %s", cudaGetErrorString(e));
                }
                p->submit([p, si, host, nr, nb, host_pitch] {
                    Slot &sl = p->slot(si);
                    if (cudaEventSynchronize(sl.ev) != cudaSuccess) p->fail_flag();
                    else copy_rows(host, host_pitch, sl.buf, nb, nb, nr);
                    p->release(si);
                });
            }
        }
    }
    // uploads: the host array must have been read, and every chunk's DMA enqueued, before the caller goes on
    if (to_device) {
        p->wait(&batch);
        if (p->take_failure()) return fail("staged copy to the device failed");
    }
    return 0;
}

}  // namespace

bool host_is_pageable(const void *p)
{
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return true;
    }
    return a.type == cudaMemoryTypeUnregistered;
}

int h2d_2d(void *dev, size_t dev_pitch, const void *host, size_t host_pitch, size_t row_bytes, size_t rows,
           cudaStream_t st)
{
    if (rows == 0 || row_bytes == 0) return 0;
    Pool *p = nullptr;
    if (staging_enabled() && row_bytes * rows >= stage_min() && host_is_pageable(host)) p = pool();
    if (!p) {
        CB_CUDA(cudaMemcpy2DAsync(dev, dev_pitch, host, host_pitch, row_bytes, rows, cudaMemcpyHostToDevice, st));
        return 0;
    }
    Piece pc = {(char *)host, (char *)dev, rows, row_bytes, host_pitch, dev_pitch};
    return staged(p, true, pc, st);
}

int d2h_2d(void *host, size_t host_pitch, const void *dev, size_t dev_pitch, size_t row_bytes, size_t rows,
           cudaStream_t st)
{
    if (rows == 0 || row_bytes == 0) return 0;
    Pool *p = nullptr;
    if (staging_enabled() && row_bytes * rows >= stage_min() && host_is_pageable(host)) p = pool();
    if (!p) {
        CB_CUDA(cudaMemcpy2DAsync(host, host_pitch, dev, dev_pitch, row_bytes, rows, cudaMemcpyDeviceToHost, st));
        return 0;
    }
    Piece pc = {(char *)host, (char *)dev, rows, row_bytes, host_pitch, dev_pitch};
    return staged(p, false, pc, st);
}

int h2d(void *dev, const void *host, size_t bytes, cudaStream_t st)
{
    if (bytes == 0) return 0;
    if (bytes < stage_min() || !staging_enabled() || !host_is_pageable(host)) {
        CB_CUDA(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, st));
        return 0;
    }
    return h2d_2d(dev, bytes, host, bytes, bytes, 1, st);
}

int d2h(void *host, const void *dev, size_t bytes, cudaStream_t st)
{
    if (bytes == 0) return 0;
    if (bytes < stage_min() || !staging_enabled() || !host_is_pageable(host)) {
        CB_CUDA(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, st));
        return 0;
    }
    return d2h_2d(host, bytes, dev, bytes, bytes, 1, st);
}

int copies_drain()
{
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= 64) return 0;
    Pool *p;
    {
        std::lock_guard<std::mutex> lk(g_pool_mu);
        p = g_pool[d];
    }
    if (p && p->drain()) return fail("a staged copy between host and device failed");
    return 0;
}

}  // namespace cb200

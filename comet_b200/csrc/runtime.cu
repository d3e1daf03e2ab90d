// Library state: error reporting, per-device scratch slots, the library stream.
#include <stdarg.h>
#include <string.h>
#include <time.h>

#include <mutex>

#include "common.cuh"

namespace cb200 {

static thread_local char g_err[1024] = "";
static int g_error_mode = -1;   // -1 = read COMET_B200_ON_ERROR on first use

static int error_mode()
{
    if (g_error_mode < 0) {
        const char *e = getenv("COMET_B200_ON_ERROR");
        g_error_mode = (e && strcmp(e, "return") == 0) ? 1 : 0;
    }
    return g_error_mode;
}

int fail(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    if (error_mode() == 0) {
        fprintf(stderr, "libcomet_b200: ERROR: %s\n", g_err);
        exit(1);
    }
    return 1;
}

void clear_error() { g_err[0] = 0; }

void trace(const char *fmt, ...)
{
    static int on = -1;
    static struct timespec t0;
    if (on < 0) {
        on = getenv("COMET_B200_TRACE") ? 1 : 0;
        clock_gettime(CLOCK_MONOTONIC, &t0);
    }
    if (!on) return;
    struct timespec t;
    clock_gettime(CLOCK_MONOTONIC, &t);
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    fprintf(stderr, "[comet_b200 %10.3f ms] %s\n", (t.tv_sec - t0.tv_sec) * 1e3 + (t.tv_nsec - t0.tv_nsec) * 1e-6, buf);
}

static const int kMaxDevices = 64;
struct DeviceState {
    void *ptr[SLOT_COUNT];
    size_t cap[SLOT_COUNT];
    cudaStream_t stream;
    cudaStream_t aux[2];
    int sms;
};
static DeviceState g_dev[kMaxDevices];
static std::mutex g_mu;

static DeviceState *state()
{
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= kMaxDevices) return nullptr;
    return &g_dev[d];
}

int scratch(Slot slot, size_t bytes, void **ptr)
{
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState *s = state();
    if (!s) return fail("no usable CUDA device (cudaGetDevice failed); libcomet_b200 has no CPU path");
    if (bytes < 256) bytes = 256;
    if (s->cap[slot] < bytes) {
        if (s->ptr[slot]) {
            // a kernel of an earlier call may still read the old buffer
            CB_CUDA(cudaDeviceSynchronize());
            CB_CUDA(cudaFree(s->ptr[slot]));
            s->ptr[slot] = nullptr;
            s->cap[slot] = 0;
        }
        size_t want = bytes + bytes / 8;   // head-room so slowly growing inputs do not reallocate
        want = (want + 255) & ~(size_t)255;
        cudaError_t e = cudaMalloc(&s->ptr[slot], want);
        if (e != cudaSuccess)
            return fail("cudaMalloc of %zu bytes of scratch failed: %s", want, cudaGetErrorString(e));
        s->cap[slot] = want;
    }
    *ptr = s->ptr[slot];
    return 0;
}

void scratch_release_all()
{
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState *s = state();
    if (!s) return;
    cudaDeviceSynchronize();
    for (int i = 0; i < SLOT_COUNT; i++) {
        if (s->ptr[i]) cudaFree(s->ptr[i]);
        s->ptr[i] = nullptr;
        s->cap[i] = 0;
    }
}

int sm_count()
{
    DeviceState *s = state();
    if (!s) return 148;
    if (s->sms == 0) {
        int d = 0, n = 0;
        cudaGetDevice(&d);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || n <= 0)
            n = 148;
        s->sms = n;
    }
    return s->sms;
}

cudaStream_t lib_stream()
{
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState *s = state();
    if (!s) return nullptr;
    if (!s->stream) {
        if (cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking) != cudaSuccess)
            s->stream = nullptr;
    }
    return s->stream;
}

cudaStream_t aux_stream(int i)
{
    std::lock_guard<std::mutex> lk(g_mu);
    DeviceState *s = state();
    if (!s || i < 0 || i > 1) return nullptr;
    if (!s->aux[i]) {
        if (cudaStreamCreateWithFlags(&s->aux[i], cudaStreamNonBlocking) != cudaSuccess) s->aux[i] = nullptr;
    }
    return s->aux[i];
}

}  // namespace cb200

extern "C" {

const char *comet_b200_last_error(void) { return cb200::g_err; }

void comet_b200_set_error_mode(int32_t return_instead_of_exit)
{
    cb200::g_error_mode = return_instead_of_exit ? 1 : 0;
}

int32_t comet_b200_version(void) { return 100; }

void comet_b200_release_scratch(void) { cb200::scratch_release_all(); }

}

// Host-side runtime of libmamba_b200: thread-local error text, device entry, version.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <vector>

#include "common.cuh"

namespace mb200 {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

// Immutable per-device attributes, filled on first use (idempotent, so a race only repeats the query).
static int g_sm_count[64] = {0};
static int g_checked[64] = {0};

int enter_device(int device)
{
    if (device < 0 || device >= 64) return fail(MB200_ERR_NO_DEVICE, "device index %d out of range", device);
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return fail(MB200_ERR_NO_DEVICE, "cudaSetDevice(%d): %s", device, cudaGetErrorString(e));
    if (!g_checked[device]) {
        int major = 0, sms = 0;
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
        if (major != 10)
            return fail(MB200_ERR_NO_DEVICE, "device %d has compute capability %d.x; this library holds sm_100a code only",
                        device, major);
        g_sm_count[device] = sms;
        g_checked[device] = 1;
    }
    return MB200_OK;
}

int sm_count(int device) { return g_sm_count[device]; }

cudaError_t ensure_dynamic_smem(const void *kernel, int bytes, int device)
{
    struct Entry { const void *kernel; int device, bytes; };
    static std::mutex mu;
    static std::vector<Entry> table;
    std::lock_guard<std::mutex> lock(mu);
    for (Entry &e : table)
        if (e.kernel == kernel && e.device == device) {
            if (e.bytes >= bytes) return cudaSuccess;
            const cudaError_t rc = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
            if (rc == cudaSuccess) e.bytes = bytes;
            return rc;
        }
    const cudaError_t rc = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (rc == cudaSuccess) table.push_back({kernel, device, bytes});
    return rc;
}

bool debug_sync()
{
    static int on = -1;
    if (on < 0) {
        const char *e = getenv("MB200_DEBUG_SYNC");
        on = (e && e[0] == '1') ? 1 : 0;
    }
    return on == 1;
}

void debug_after_launch(const char *what)
{
    fprintf(stderr, "[mb200] launched %s ...", what);
    fflush(stderr);
    const cudaError_t e = cudaDeviceSynchronize();
    fprintf(stderr, " %s\n", e == cudaSuccess ? "done" : cudaGetErrorString(e));
    fflush(stderr);
}

}  // namespace mb200

extern "C" int mb200_version(void) { return 100; }
extern "C" const char *mb200_last_error(void) { return mb200::g_error; }

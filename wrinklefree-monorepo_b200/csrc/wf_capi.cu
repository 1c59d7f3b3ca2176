// Error reporting, version and device check of the wf_b200 C ABI.
#include <atomic>
#include <cstring>

#include "wf_common.cuh"

namespace wf {

static thread_local char g_err[512] = "";

char* err_buf() { return g_err; }

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int cuda_fail(cudaError_t e, const char* what) {
    snprintf(g_err, sizeof(g_err), "CUDA error %d (%s) in %s", static_cast<int>(e), cudaGetErrorString(e), what);
    return WF_E_DEVICE;
}

static std::atomic<int> g_major[WF_MAX_DEVICES];  // compute capability major per device (0 = not queried yet)
static std::atomic<int> g_sms[WF_MAX_DEVICES];    // multiprocessor count per device (0 = not queried yet)

int current_device() {
    int dev = -1;
    return cudaGetDevice(&dev) == cudaSuccess ? dev : -1;
}

int require_device() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    int major = (dev >= 0 && dev < WF_MAX_DEVICES) ? g_major[dev].load(std::memory_order_relaxed) : 0;
    if (major == 0) {
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
        if (dev >= 0 && dev < WF_MAX_DEVICES) g_major[dev].store(major, std::memory_order_relaxed);
    }
    if (major != 10)
        return fail(WF_E_DEVICE, "device %d has compute capability %d.x; this library is built for sm_100a only", dev,
                    major);
    return WF_OK;
}

int num_sms() {
    const int dev = current_device();
    int n = (dev >= 0 && dev < WF_MAX_DEVICES) ? g_sms[dev].load(std::memory_order_relaxed) : 0;
    if (n <= 0) {
        if (dev < 0 || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        if (dev >= 0 && dev < WF_MAX_DEVICES) g_sms[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

}  // namespace wf

extern "C" {

int wf_version(void) { return 100; }

const char* wf_last_error(void) { return wf::err_buf(); }

int wf_device_check(void) { return wf::require_device(); }
}

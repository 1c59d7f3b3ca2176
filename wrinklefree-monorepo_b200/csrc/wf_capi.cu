// Error reporting, version and device check of the wf_b200 C ABI.
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

int require_device() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
    static thread_local int checked_dev = -1;
    if (checked_dev == dev) return WF_OK;
    int major = 0;
    e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
    if (major != 10)
        return fail(WF_E_DEVICE, "device %d has compute capability %d.x; this library is built for sm_100a only", dev,
                    major);
    checked_dev = dev;
    return WF_OK;
}

}  // namespace wf

extern "C" {

int wf_version(void) { return 100; }

const char* wf_last_error(void) { return wf::err_buf(); }

int wf_device_check(void) { return wf::require_device(); }
}

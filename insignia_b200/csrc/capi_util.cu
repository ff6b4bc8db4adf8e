// Error reporting and device queries shared by the C-ABI entry points.
#include "host_util.h"

#include <mutex>

namespace insg {

namespace {
thread_local std::string g_error;
}

void set_error(const std::string &msg) { g_error = msg; }

int fail(int code, const std::string &msg)
{
    g_error = msg;
    return code;
}

int cuda_fail(cudaError_t e, const char *what)
{
    g_error = std::string(what) + ": " + cudaGetErrorString(e);
    return INSG_E_CUDA;
}

int sm_count()
{
    // per device, cached; the decode path runs on one device per process
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return kSMsDefault;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = kSMsDefault;
        cached[dev] = n;
    }
    return cached[dev];
}

} // namespace insg

extern "C" {

const char *insg_last_error(void) { return insg::g_error.c_str(); }
int insg_version(void) { return 100; }
int insg_tune_set(const char *key, int value)
{
    (void)value;
    if (!key) return insg::fail(INSG_E_ARG, "tune: null key");
    return insg::fail(INSG_E_ARG, "unknown tuning key"); // this build has none: launch shapes are fixed per kernel
}

} // extern "C"

// Host-side plumbing of the C ABI: error strings, device checks.
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "common.cuh"

namespace ls {
namespace {
thread_local char g_err[512] = "";
struct DevInfo { int major = -1, sms = 0; };
DevInfo g_dev[64];
std::mutex g_mu;

int query(DevInfo &out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(LS_EARCH, "no CUDA device: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) return fail(LS_EINVAL, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_dev[dev].major < 0) {
        int major = 0, sms = 0;
        LS_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        LS_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        g_dev[dev].major = major;
        g_dev[dev].sms = sms;
    }
    out = g_dev[dev];
    return LS_OK;
}
}  // namespace

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof g_err, fmt, ap);
    va_end(ap);
    return code;
}

int check_device()
{
    DevInfo d;
    if (int rc = query(d)) return rc;
    if (d.major != 10) return fail(LS_EARCH, "this library runs on sm_100 (B200) only; device is sm_%d0", d.major);
    return LS_OK;
}

int current_device(int *dev)
{
    cudaError_t e = cudaGetDevice(dev);
    if (e != cudaSuccess) return fail(LS_ECUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    if (*dev < 0 || *dev >= 64) return fail(LS_EINVAL, "device index %d out of range", *dev);
    return LS_OK;
}

std::mutex &state_mutex()
{
    static std::mutex mu;
    return mu;
}

int sm_count()
{
    DevInfo d;
    return query(d) == LS_OK && d.sms > 0 ? d.sms : 148;
}
}  // namespace ls

extern "C" int ls_version(void) { return 100; }
extern "C" const char *ls_last_error(void) { return ls::g_err; }

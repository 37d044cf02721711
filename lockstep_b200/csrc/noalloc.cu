// ls_mxfp4_linear_noalloc: the MXFP4 linear forward (quantize the activations,
// then the tensor-core GEMM) for callers that must not allocate device memory.
//
// Who that is: code running where cudaMalloc is off limits -- a plugin called
// inside someone else's memory plan (an inference server or training loop
// that hands out every byte up front and treats a late allocation as a bug), a
// latency-critical loop where an allocation's implicit device synchronisation
// would stall every stream, or a host that forbids allocator calls on the
// thread that makes the call.  The regular path needs two temporaries between
// its two kernels (the packed activations and their scale bytes) plus an
// error word; the Python layer gets them from torch's allocator.  Here all
// three live in one array that is part of the library image, so the call
// touches no allocator at all.
//
// The price is a fixed capacity (kMaxElems activations per call) and shared
// state: every call on a device uses the same array.
#include <mutex>

#include "common.cuh"

namespace ls {
namespace {

constexpr int64_t kMaxElems = int64_t(1) << 24;        // M * K of the activations
constexpr int64_t kMaxSfBytes = int64_t(1) << 20;      // scale bytes (rows rounded up to 128)
constexpr int64_t kErrBytes = 256;
constexpr int64_t kScratchBytes = kErrBytes + kMaxElems / 2 + kMaxSfBytes;

// Resident in every GPU that loads the library, until the process exits.
static __device__ __align__(256) uint8_t g_scratch[kScratchBytes];

std::mutex g_mu;
uint8_t *g_scratch_addr[64] = {};                       // device address of g_scratch, per device

// `g_scratch` named in host code is only a handle for the runtime, not an
// address a kernel can use: the device address has to be asked for, once per
// device, with that device current.
int scratch_address(uint8_t **out)
{
    int dev = 0;
    LS_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(LS_EINVAL, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_scratch_addr[dev]) {
        uint8_t *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_scratch);
        if (e != cudaSuccess || !p)
            return fail(LS_ECUDA, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return LS_OK;
}

}  // namespace
}  // namespace ls

using namespace ls;

extern "C" int ls_mxfp4_linear_noalloc(const void *x, int x_dtype, const uint8_t *w_pk, const uint8_t *w_sf,
                                       void *c, int out_dtype, int64_t M, int64_t N, int64_t K,
                                       int32_t *status, void *stream)
{
    if (int rc = check_device()) return rc;
    if (M < 0 || N < 0) return fail(LS_EINVAL, "M=%lld and N=%lld must not be negative", (long long)M, (long long)N);
    if (K <= 0 || K % 128 != 0) return fail(LS_EINVAL, "K=%lld must be a positive multiple of 128", (long long)K);
    if (M == 0 || N == 0) return LS_OK;
    if (M > kMaxElems / K)                              // M * K > kMaxElems without the overflow
        return fail(LS_EINVAL, "no-alloc path holds at most %lld activation elements per call, got %lld x %lld",
                    (long long)kMaxElems, (long long)M, (long long)K);
    const int64_t sf_bytes = ls_sf_bytes(M, K);
    if (sf_bytes > kMaxSfBytes)
        return fail(LS_EINVAL, "no-alloc path holds at most %lld scale bytes per call, this shape needs %lld",
                    (long long)kMaxSfBytes, (long long)sf_bytes);
    uint8_t *scratch = nullptr;
    if (int rc = scratch_address(&scratch)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int *err = reinterpret_cast<int *>(scratch);
    uint8_t *packed = scratch + kErrBytes;
    uint8_t *sf = packed + kMaxElems / 2;
    // the error word must start at zero; packed bytes and scale bytes are fully
    // rewritten for the rows that are read back
    LS_CUDA(cudaMemsetAsync(err, 0, sizeof(int), st));
    if (int rc = ls_quantize_mxfp4(x, x_dtype, M, K, 32, LS_ROUND_REF, nullptr, packed, nullptr, nullptr, sf, stream))
        return rc;
    if (int rc = gemm_common(1, packed, nullptr, w_pk, sf, nullptr, w_sf, c, nullptr, out_dtype, M, N, K, stream, err))
        return rc;
    if (status) LS_CUDA(cudaMemcpyAsync(status, err, sizeof(int), cudaMemcpyDeviceToDevice, st));
    return LS_OK;
}

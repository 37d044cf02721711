// Operands given as E4M3 bytes that hold E2M1 values (the form lockstep's mxfp4_gemm_fp8
// takes, mxfp4_gemm.py:74-87: on Hopper the FP4 values are expanded to FP8 because the
// tensor cores there have no FP4 type).  The B200 tensor cores take E2M1 directly at twice
// the FP8 rate, so these kernels re-encode the bytes to packed E2M1 -- exactly, each byte
// is one of 16 values -- and the product runs on the MXFP4 kernel:
//   a  [M, K] K-contiguous            -> packed [M, K/2]
//   b  [K, N] N-contiguous            -> packed [N, K/2]  (transposed on the way)
//   b_scale [K/32, N] fp32 powers of 2 -> scale-factor bytes of a [N, K] operand
// A byte that is not an E2M1 value sets bit 1 of the device error word that ls_gemm_status
// reads (no synchronisation in the call itself).
#include "common.cuh"

namespace ls {
int *error_word();
namespace {

constexpr int kThreads = 256;

// E4M3 byte -> E2M1 code; ok = false if the byte is not one of the 16 images
// 00 30 38 3C 40 44 48 4C (and the same with the sign bit).
__device__ __forceinline__ uint32_t code_of(uint32_t b, bool &ok)
{
    const uint32_t m = b & 0x7Fu;
    const uint32_t mag = m == 0u ? 0u : (m == 0x30u ? 1u : ((m - 0x30u) >> 2));
    ok = ok && mag <= 7u && uint32_t((0x4C4844403C383000ull >> (8 * (mag & 7u))) & 0xFFu) == m;
    return (mag & 7u) | ((b >> 4) & 8u);
}

// 4 bytes (k, k+1, k+2, k+3 in ascending byte order) -> 2 packed bytes
__device__ __forceinline__ uint32_t pack4(uint32_t w, bool &ok)
{
    return code_of(w & 0xFFu, ok) | (code_of((w >> 8) & 0xFFu, ok) << 4) | (code_of((w >> 16) & 0xFFu, ok) << 8) |
           (code_of(w >> 24, ok) << 12);
}

__global__ void __launch_bounds__(kThreads)
e4m3_to_packed_kernel(const uint4 *__restrict__ src, uint2 *__restrict__ dst, int64_t n16, int *err)
{
    const int64_t stride = int64_t(gridDim.x) * kThreads;
    bool ok = true;
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < n16; i += stride) {
        const uint4 v = ld_stream(src + i);
        dst[i] = make_uint2(pack4(v.x, ok) | (pack4(v.y, ok) << 16), pack4(v.z, ok) | (pack4(v.w, ok) << 16));
    }
    if (!ok) atomicOr(err, 2);
}

// Tile of 128 (k) x 64 (n) bytes through shared memory: rows of b are read in 16-byte pieces,
// each thread then gathers 32 consecutive k of one n into 16 packed bytes.
constexpr int kTK = 128, kTN = 64, kPitch = kTN + 4;

__global__ void __launch_bounds__(kThreads)
e4m3_to_packed_t_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, int K, int N, int *err)
{
    __shared__ uint8_t tile[kTK * kPitch];
    const int k0 = blockIdx.y * kTK, n0 = blockIdx.x * kTN;
    const bool vec = (N & 15) == 0;
    for (int i = threadIdx.x; i < kTK * (kTN / 16); i += kThreads) {
        const int k = i / (kTN / 16), c = i % (kTN / 16), n = n0 + 16 * c;
        uint32_t w[4] = {0, 0, 0, 0};
        if (k0 + k < K) {
            if (vec && n + 16 <= N) {
                const uint4 v = *reinterpret_cast<const uint4 *>(src + int64_t(k0 + k) * N + n);
                w[0] = v.x, w[1] = v.y, w[2] = v.z, w[3] = v.w;
            } else {
                for (int j = 0; j < 16; j++)
                    if (n + j < N) w[j >> 2] |= uint32_t(src[int64_t(k0 + k) * N + n + j]) << (8 * (j & 3));
            }
        }
#pragma unroll
        for (int j = 0; j < 4; j++) *reinterpret_cast<uint32_t *>(&tile[k * kPitch + 16 * c + 4 * j]) = w[j];
    }
    __syncthreads();
    bool ok = true;
    const int n = threadIdx.x / 4, q = threadIdx.x % 4;          // 64 rows of the output, four 32-k pieces each
    if (n0 + n < N && k0 + 32 * q < K) {
        uint32_t out[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t o = 0;
#pragma unroll
            for (int t = 0; t < 8; t++) o |= code_of(tile[(32 * q + 8 * j + t) * kPitch + n], ok) << (4 * t);
            out[j] = o;
        }
        *reinterpret_cast<uint4 *>(dst + int64_t(n0 + n) * (K / 2) + (k0 + 32 * q) / 2) = make_uint4(out[0], out[1], out[2], out[3]);
    }
    if (!ok) atomicOr(err, 2);
}

// scale [K/32, rows] (rows contiguous) -> scale-factor bytes of a [rows, K] operand
__global__ void __launch_bounds__(kThreads)
scales_to_sf_t_kernel(const float *__restrict__ scale, int64_t rows, uint32_t kblocks, uint8_t *__restrict__ sf, int32_t *bad)
{
    const int64_t total = rows * kblocks, stride = int64_t(gridDim.x) * kThreads;
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < total; i += stride) {
        const uint32_t kb = uint32_t(i / rows), row = uint32_t(i - int64_t(kb) * rows);
        const uint32_t u = __float_as_uint(scale[i]);
        uint32_t e = (u >> 23) & 0xFFu;
        bool ok = (u & 0x807FFFFFu) == 0u && e >= 1u && e <= 254u;
        if (u == 0x00400000u) { ok = true; e = 0u; }          // 2^-127
        if (!ok) {
            if (bad) atomicAdd(bad, 1);
            e = 255u;
        }
        sf[sf_offset(row, kb, kblocks / 4)] = uint8_t(e);
    }
}

int grid_of(int64_t items)
{
    int64_t want = (items + kThreads - 1) / kThreads, cap = int64_t(sm_count()) * 8;
    return int(want < 1 ? 1 : (want < cap ? want : cap));
}

}  // namespace
}  // namespace ls

using namespace ls;

extern "C" int ls_e4m3_to_packed(const uint8_t *src, int64_t rows, int64_t K, uint8_t *packed, void *stream)
{
    if (int rc = check_device()) return rc;
    if (rows < 0 || K < 0 || K % 16 != 0) return fail(LS_EINVAL, "K=%lld must be a multiple of 16", (long long)K);
    if (rows == 0 || K == 0) return LS_OK;
    if (!src || !packed) return fail(LS_EINVAL, "null pointer");
    if (!aligned16(src) || (reinterpret_cast<uintptr_t>(packed) & 7)) return fail(LS_EALIGN, "src must be 16-byte aligned, packed 8-byte");
    int *err = error_word();
    if (!err) return fail(LS_ECUDA, "could not allocate the device error word");
    const int64_t n16 = rows * K / 16;
    e4m3_to_packed_kernel<<<grid_of(n16), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint4 *>(src), reinterpret_cast<uint2 *>(packed), n16, err);
    LS_LAUNCH_CHECK("e4m3_to_packed");
    return LS_OK;
}

extern "C" int ls_e4m3_to_packed_t(const uint8_t *src, int64_t K, int64_t N, uint8_t *packed, void *stream)
{
    if (int rc = check_device()) return rc;
    if (K < 0 || N < 0 || K % 32 != 0) return fail(LS_EINVAL, "K=%lld must be a multiple of 32", (long long)K);
    if (K == 0 || N == 0) return LS_OK;
    if (K >= (int64_t(1) << 31) || N >= (int64_t(1) << 31) || (K + kTK - 1) / kTK > 65535)
        return fail(LS_EINVAL, "shape too large");
    if (!src || !packed) return fail(LS_EINVAL, "null pointer");
    if (!aligned16(src) || !aligned16(packed)) return fail(LS_EALIGN, "src and packed must be 16-byte aligned");
    int *err = error_word();
    if (!err) return fail(LS_ECUDA, "could not allocate the device error word");
    dim3 grid(unsigned((N + kTN - 1) / kTN), unsigned((K + kTK - 1) / kTK));
    e4m3_to_packed_t_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(src, packed, int(K), int(N), err);
    LS_LAUNCH_CHECK("e4m3_to_packed_t");
    return LS_OK;
}

extern "C" int ls_scales_to_sf_t(const float *scale, int64_t rows, int64_t K, uint8_t *sf, int32_t *bad, void *stream)
{
    if (int rc = check_device()) return rc;
    if (rows < 0 || K < 0 || K % 128 != 0) return fail(LS_EINVAL, "K must be a multiple of 128");
    if (rows * (K / 32) == 0) return LS_OK;
    if (!scale || !sf) return fail(LS_EINVAL, "null pointer");
    scales_to_sf_t_kernel<<<grid_of(rows * (K / 32)), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        scale, rows, uint32_t(K / 32), sf, bad);
    LS_LAUNCH_CHECK("scales_to_sf_t");
    return LS_OK;
}

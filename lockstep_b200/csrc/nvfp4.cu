// NVFP4: blocks of 16 E2M1 values under one E4M3 scale (4.5 bits per element).
//
// The rule is the one lockstep's format study states (rig_sm75/quant_sim.cuh:90-97 with
// :20-33 and :57-69, applied per block as rig_q.cu:348-363 does):
//   amax  = max |v| over the block, NaNs skipped
//   scale = E4M3(amax / 6), round-half-even, saturating at 448; 2^-9 where that gives 0;
//           1.0 for a block without a positive maximum
//   code  = E2M1 value nearest to v / scale (IEEE division), ties to the smaller
//           magnitude; NaN and +-Inf quotients give magnitude 0
// A thread owns one block: 32 or 64 bytes in, 8 bytes of codes and one scale byte out.
// Four neighbouring lanes hold the four scales of one word of the tensor-core scale-factor
// layout, so the scale bytes leave as words.

#include "common.cuh"

namespace ls {
namespace {

constexpr int kThreads = 256;

struct Nvfp4Out {
    uint8_t *packed;       // [rows, K/2]
    uint8_t *scale_u8;     // [rows, K/16] E4M3 bytes, or NULL
    float *scale_f32;      // [rows, K/16] the same scales as fp32, or NULL
    uint8_t *sf;           // scale-factor layout, or NULL
    uint32_t kblocks;      // K / 16
    uint32_t nblocks;      // rows * kblocks
};

__device__ __forceinline__ uint32_t e4m3_byte_sat(float a)      // a >= 0, not NaN
{
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(a));
    return r & 0xFFu;
}

__device__ __forceinline__ float e4m3_value(uint32_t b)         // b in 0x01 .. 0x7E
{
    const uint32_t e = b >> 3, m = b & 7u;
    // normal: (8 + m) * 2^(e - 10); subnormal: m * 2^-9
    return e ? __uint_as_float((e + 120u) << 23 | m << 20) : float(m) * 0.001953125f;
}

__device__ __forceinline__ uint32_t nearest_e2m1(float x)
{
    const float a = fabsf(x);
    uint32_t c = uint32_t(a > 0.25f) + uint32_t(a > 0.75f) + uint32_t(a > 1.25f) + uint32_t(a > 1.75f) +
                 uint32_t(a > 2.5f) + uint32_t(a > 3.5f) + uint32_t(a > 5.0f);
    if (a == __uint_as_float(kBitsInf)) c = 0;                 // every distance is infinite: the first candidate stays
    return c | (x < 0.0f ? 8u : 0u);
}

template <typename T>
__device__ __forceinline__ void load16(const T *x, float (&v)[16]);

template <>
__device__ __forceinline__ void load16<float>(const float *x, float (&v)[16])
{
#pragma unroll
    for (int h = 0; h < 4; h++) {
        const uint4 w = ld_stream(reinterpret_cast<const uint4 *>(x) + h);
        v[4 * h] = __uint_as_float(w.x), v[4 * h + 1] = __uint_as_float(w.y);
        v[4 * h + 2] = __uint_as_float(w.z), v[4 * h + 3] = __uint_as_float(w.w);
    }
}

template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16 *x, float (&v)[16])
{
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const uint4 w = ld_stream(reinterpret_cast<const uint4 *>(x) + h);
        const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            v[8 * h + 2 * i] = __uint_as_float(u[i] << 16);
            v[8 * h + 2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
nvfp4_quantize_kernel(const T *__restrict__ x, Nvfp4Out o)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const uint32_t blk = blockIdx.x * kThreads + threadIdx.x;
    const bool in_range = blk < o.nblocks;
    float v[16];
    if (in_range) load16<T>(x + size_t(blk) * 16, v);
    else
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = 0.0f;
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(v[i]));        // fmaxf drops a NaN operand
    uint32_t sb = 0x38u;                                                 // 1.0
    if (amax > 0.0f) {
        sb = e4m3_byte_sat(__fdiv_rn(amax, 6.0f));
        if (sb == 0u) sb = 1u;                                           // the smallest subnormal, 2^-9
    }
    const float s = e4m3_value(sb);
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        lo |= nearest_e2m1(__fdiv_rn(v[i], s)) << (4 * i);
        hi |= nearest_e2m1(__fdiv_rn(v[8 + i], s)) << (4 * i);
    }
    if (in_range) reinterpret_cast<uint2 *>(o.packed)[blk] = make_uint2(lo, hi);
    // scale bytes of 4 consecutive blocks (same row: K / 16 is a multiple of 8) as one word
    uint32_t w = sb;
    w |= __shfl_down_sync(0xFFFFFFFFu, sb, 1) << 8;
    w |= __shfl_down_sync(0xFFFFFFFFu, sb, 2) << 16;
    w |= __shfl_down_sync(0xFFFFFFFFu, sb, 3) << 24;
    if (in_range && (threadIdx.x & 3) == 0) {
        if (o.scale_u8) *reinterpret_cast<uint32_t *>(o.scale_u8 + blk) = w;
        if (o.sf) {
            const uint32_t row = blk / o.kblocks, kb = blk - row * o.kblocks;
            *reinterpret_cast<uint32_t *>(o.sf + sf_offset(row, kb, o.kblocks / 4)) = w;
        }
    }
    if (in_range && o.scale_f32) o.scale_f32[blk] = s;
}

// packed codes x E4M3 block scales -> values; one thread per block of 16
template <bool BF16>
__global__ void __launch_bounds__(kThreads)
nvfp4_dequantize_kernel(const uint8_t *__restrict__ packed, const uint8_t *__restrict__ scale_u8, uint32_t nblocks,
                        void *__restrict__ out)
{
    const uint32_t blk = blockIdx.x * kThreads + threadIdx.x;
    if (blk >= nblocks) return;
    const uint2 pk = reinterpret_cast<const uint2 *>(packed)[blk];
    const uint32_t b = scale_u8[blk] & 0x7Fu;
    const float s = e4m3_value(b);
    float v[16];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        v[i] = e2m1_value((pk.x >> (4 * i)) & 0xFu) * s;
        v[8 + i] = e2m1_value((pk.y >> (4 * i)) & 0xFu) * s;
    }
    if (BF16) {
        uint32_t w[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
        uint4 *dst = reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(out) + size_t(blk) * 16);
        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
    } else {
        float4 *dst = reinterpret_cast<float4 *>(static_cast<float *>(out) + size_t(blk) * 16);
#pragma unroll
        for (int h = 0; h < 4; h++) dst[h] = make_float4(v[4 * h], v[4 * h + 1], v[4 * h + 2], v[4 * h + 3]);
    }
}

}  // namespace
}  // namespace ls

using namespace ls;

extern "C" int ls_quantize_nvfp4(const void *x, int x_dtype, int64_t rows, int64_t K, uint8_t *packed,
                                 uint8_t *scale_u8, float *scale_f32, uint8_t *sf, void *stream)
{
    if (int rc = check_device()) return rc;
    if (rows < 0 || K < 0 || K % 128 != 0) return fail(LS_EINVAL, "K=%lld must be a multiple of 128", (long long)K);
    if (x_dtype != LS_F32 && x_dtype != LS_BF16) return fail(LS_EINVAL, "unsupported dtype %d", x_dtype);
    const int64_t n = rows * K;
    if (n == 0) return LS_OK;
    if (!x || !packed) return fail(LS_EINVAL, "null pointer");
    if (n / 16 >= (int64_t(1) << 31)) return fail(LS_EINVAL, "more than 2^35 elements in one call");
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(packed) & 7) || (reinterpret_cast<uintptr_t>(scale_u8) & 3) ||
        (reinterpret_cast<uintptr_t>(scale_f32) & 3) || (reinterpret_cast<uintptr_t>(sf) & 3))
        return fail(LS_EALIGN, "x must be 16-byte, packed 8-byte, scale buffers 4-byte aligned");
    Nvfp4Out o{packed, scale_u8, scale_f32, sf, uint32_t(K / 16), uint32_t(n / 16)};
    const int grid = int((o.nblocks + kThreads - 1) / kThreads);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (x_dtype == LS_BF16) nvfp4_quantize_kernel<<<grid, kThreads, 0, st>>>(static_cast<const __nv_bfloat16 *>(x), o);
    else nvfp4_quantize_kernel<<<grid, kThreads, 0, st>>>(static_cast<const float *>(x), o);
    LS_LAUNCH_CHECK("quantize_nvfp4");
    return LS_OK;
}

extern "C" int ls_dequantize_nvfp4(const uint8_t *packed, const uint8_t *scale_u8, int64_t rows, int64_t K,
                                   void *out, int out_dtype, void *stream)
{
    if (int rc = check_device()) return rc;
    if (rows < 0 || K < 0 || K % 16 != 0) return fail(LS_EINVAL, "K=%lld must be a multiple of 16", (long long)K);
    if (out_dtype != LS_F32 && out_dtype != LS_BF16) return fail(LS_EINVAL, "unsupported dtype %d", out_dtype);
    const int64_t n = rows * K;
    if (n == 0) return LS_OK;
    if (!packed || !scale_u8 || !out) return fail(LS_EINVAL, "null pointer");
    if (n / 16 >= (int64_t(1) << 31)) return fail(LS_EINVAL, "more than 2^35 elements in one call");
    if ((reinterpret_cast<uintptr_t>(packed) & 7) || !aligned16(out))
        return fail(LS_EALIGN, "packed must be 8-byte, out 16-byte aligned");
    const uint32_t nblocks = uint32_t(n / 16);
    const int grid = int((nblocks + kThreads - 1) / kThreads);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (out_dtype == LS_BF16) nvfp4_dequantize_kernel<true><<<grid, kThreads, 0, st>>>(packed, scale_u8, nblocks, out);
    else nvfp4_dequantize_kernel<false><<<grid, kThreads, 0, st>>>(packed, scale_u8, nblocks, out);
    LS_LAUNCH_CHECK("dequantize_nvfp4");
    return LS_OK;
}

// LayerNorm fused with the MXFP4 quantization of its output: the input of the qkv and fc
// projections of lockstep's block (train.py:50,53: linear(ln(x))) goes from the residual
// stream to packed E2M1 + scale bytes in one pass, together with the bf16 copy of the
// normalized row that the backward pass needs.  The values quantized are exactly that bf16
// copy: LayerNorm in fp32 (as torch runs it under autocast), rounded to bf16, then
// quantize_mxfp4's arithmetic (fp4.py:57-72).
//
// One CTA of D / 8 threads per row (a thread owns 8 consecutive features: one 32-byte or
// 16-byte load), two reductions over the row (mean, then the centred sum of squares), four
// adjacent lanes share a block of 32.  HBM-bound: 4 or 2 bytes in, 2 + 0.53 bytes out per
// element.
#include "common.cuh"

namespace ls {
namespace {

__device__ __forceinline__ float cta_sum(float v, float *scratch)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    __syncthreads();                                   // scratch may still be read from the previous use
    if ((threadIdx.x & 31) == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.0f;
    for (int w = 0; w < nwarps; w++) t += scratch[w];  // the same order in every thread
    return t;
}

template <typename T>
__global__ void __launch_bounds__(1024)
layernorm_quantize_kernel(const T *__restrict__ x, const float *__restrict__ gamma, const float *__restrict__ beta,
                          float eps, int64_t rows, int D, __nv_bfloat16 *__restrict__ y, uint8_t *__restrict__ packed,
                          uint8_t *__restrict__ sf, float *__restrict__ mean_out, float *__restrict__ rstd_out)
{
    __shared__ float scratch[32];
    // lets a GEMM launched with programmatic stream serialization start its set-up under this
    // kernel; that GEMM waits for this grid to finish before it loads anything (no-op otherwise)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int c0 = threadIdx.x * 8;
    float g[8], b[8];
#pragma unroll
    for (int i = 0; i < 8; i++) g[i] = gamma ? gamma[c0 + i] : 1.0f, b[i] = beta ? beta[c0 + i] : 0.0f;
    const float inv_d = 1.0f / float(D);
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        float v[8];
        if constexpr (sizeof(T) == 4) {
            const float4 a = *reinterpret_cast<const float4 *>(x + r * D + c0), c = *reinterpret_cast<const float4 *>(x + r * D + c0 + 4);
            v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = c.x, v[5] = c.y, v[6] = c.z, v[7] = c.w;
        } else {
            const uint4 a = *reinterpret_cast<const uint4 *>(x + r * D + c0);
            const uint32_t u[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int i = 0; i < 4; i++) v[2 * i] = __uint_as_float(u[i] << 16), v[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
        }
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) s += v[i];
        const float mean = cta_sum(s, scratch) * inv_d;
        float q = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] -= mean, q += v[i] * v[i];
        const float rstd = rsqrtf(cta_sum(q, scratch) * inv_d + eps);
        if (threadIdx.x == 0) {
            if (mean_out) mean_out[r] = mean;
            if (rstd_out) rstd_out[r] = rstd;
        }
        uint32_t yw[4];
        uint32_t amax = 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i] * rstd * g[2 * i] + b[2 * i],
                                                           v[2 * i + 1] * rstd * g[2 * i + 1] + b[2 * i + 1]);
            yw[i] = *reinterpret_cast<const uint32_t *>(&h);
            v[2 * i] = __uint_as_float(yw[i] << 16), v[2 * i + 1] = __uint_as_float(yw[i] & 0xFFFF0000u);
            amax = max(amax, max(__float_as_uint(v[2 * i]) & 0x7FFFFFFFu, __float_as_uint(v[2 * i + 1]) & 0x7FFFFFFFu));
        }
        if (y) *reinterpret_cast<uint4 *>(y + r * D + c0) = make_uint4(yw[0], yw[1], yw[2], yw[3]);
        amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
        amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
        const uint32_t e8 = block_e8m0(amax);
        const float inv = __uint_as_float(e8 == 255u ? 0x7FC00000u : inv_scale_bits(e8));
        float t[8];
#pragma unroll
        for (int i = 0; i < 8; i++) t[i] = v[i] * inv;
        uint32_t pk;
        if (amax < kBitsInf) {
            pk = cvt_ref_e2m1x8(t);
        } else {
            pk = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) pk |= e2m1_code<false>(t[i]) << (4 * i);
        }
        reinterpret_cast<uint32_t *>(packed + r * (D / 2))[threadIdx.x] = pk;
        if ((threadIdx.x & 3) == 0) sf[sf_offset(uint32_t(r), uint32_t(threadIdx.x >> 2), uint32_t(D / 128))] = uint8_t(e8);
    }
}

}  // namespace
}  // namespace ls

using namespace ls;

extern "C" int ls_layernorm_quantize(const void *x, int x_dtype, const float *gamma, const float *beta, float eps,
                                     int64_t rows, int64_t D, void *y_bf16, uint8_t *packed, uint8_t *sf, float *mean,
                                     float *rstd, void *stream)
{
    if (int rc = check_device()) return rc;
    if (x_dtype != LS_F32 && x_dtype != LS_BF16) return fail(LS_EINVAL, "unsupported dtype %d", x_dtype);
    if (rows < 0 || D <= 0 || D % 256 != 0 || D > 8192) return fail(LS_EINVAL, "D=%lld must be a multiple of 256, at most 8192", (long long)D);
    if (rows == 0) return LS_OK;
    if (rows >= (int64_t(1) << 31)) return fail(LS_EINVAL, "too many rows");
    if (!x || !packed || !sf) return fail(LS_EINVAL, "null pointer");
    if (!aligned16(x) || !aligned16(y_bf16) || !aligned16(packed)) return fail(LS_EALIGN, "x, y and packed must be 16-byte aligned");
    const int threads = int(D / 8);
    const int64_t cap = int64_t(sm_count()) * (2048 / threads);
    const unsigned grid = unsigned(rows < cap ? rows : cap);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (x_dtype == LS_F32)
        layernorm_quantize_kernel<float><<<grid, threads, 0, st>>>(static_cast<const float *>(x), gamma, beta, eps, rows, int(D),
                                                                   static_cast<__nv_bfloat16 *>(y_bf16), packed, sf, mean, rstd);
    else
        layernorm_quantize_kernel<__nv_bfloat16><<<grid, threads, 0, st>>>(static_cast<const __nv_bfloat16 *>(x), gamma, beta, eps, rows,
                                                                           int(D), static_cast<__nv_bfloat16 *>(y_bf16), packed, sf,
                                                                           mean, rstd);
    LS_LAUNCH_CHECK("layernorm_quantize");
    return LS_OK;
}

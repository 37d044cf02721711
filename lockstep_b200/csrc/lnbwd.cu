// Backward of the LayerNorm that ls_layernorm_quantize fused into the projection's input
// (train.py:50,53: linear(ln(x))), from the statistics the forward pass kept:
//   xhat = (x - mean) rstd,  g = gy gamma
//   gx     = rstd (g - mean_D(g) - xhat mean_D(g xhat))
//   ggamma = sum_rows gy xhat,   gbeta = sum_rows gy
// One CTA of D / 8 threads per row, as the forward kernel: a thread owns 8 consecutive
// features and keeps their 16 column sums in registers over all rows of its CTA; the CTAs'
// partial sums go to a scratch array that two small kernels add in a fixed order (no atomics:
// the result does not depend on scheduling).  HBM-bound: x and gy in, gx out, once each.
#include "common.cuh"

namespace ls {
namespace {

__device__ __forceinline__ float2 cta_sum2(float a, float b, float2 *scratch)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a += __shfl_xor_sync(0xFFFFFFFFu, a, o);
        b += __shfl_xor_sync(0xFFFFFFFFu, b, o);
    }
    const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    __syncthreads();                                   // scratch may still be read from the previous row
    if ((threadIdx.x & 31) == 0) scratch[warp] = make_float2(a, b);
    __syncthreads();
    float2 t = make_float2(0.0f, 0.0f);
    for (int w = 0; w < nwarps; w++) t.x += scratch[w].x, t.y += scratch[w].y;      // the same order in every thread
    return t;
}

template <typename T>
__device__ __forceinline__ void load8(const T *p, float (&v)[8])
{
    if constexpr (sizeof(T) == 4) {
        const float4 a = *reinterpret_cast<const float4 *>(p), c = *reinterpret_cast<const float4 *>(p + 4);
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = c.x, v[5] = c.y, v[6] = c.z, v[7] = c.w;
    } else {
        const uint4 a = *reinterpret_cast<const uint4 *>(p);
        const uint32_t u[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; i++) v[2 * i] = __uint_as_float(u[i] << 16), v[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u);
    }
}

template <typename T>
__device__ __forceinline__ void store8(T *p, const float (&v)[8])
{
    if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    } else {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t *>(&h);
        }
        *reinterpret_cast<uint4 *>(p) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

template <typename TX, typename TG>
__global__ void __launch_bounds__(1024)
layernorm_backward_kernel(const TX *__restrict__ x, const TG *__restrict__ gy, const float *__restrict__ mean,
                          const float *__restrict__ rstd, const float *__restrict__ gamma, int64_t rows, int D,
                          TX *__restrict__ gx, float *__restrict__ part)
{
    __shared__ float2 scratch[32];
    const int c0 = threadIdx.x * 8;
    float g[8], acc_g[8], acc_b[8];
#pragma unroll
    for (int i = 0; i < 8; i++) g[i] = gamma ? gamma[c0 + i] : 1.0f, acc_g[i] = 0.0f, acc_b[i] = 0.0f;
    const float inv_d = 1.0f / float(D);
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        float xv[8], gv[8];
        load8(x + r * D + c0, xv);
        load8(gy + r * D + c0, gv);
        const float m = mean[r], rs = rstd[r];
        float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            xv[i] = (xv[i] - m) * rs;                  // xhat
            const float gg = gv[i] * g[i];
            s1 += gg, s2 += gg * xv[i];
            acc_g[i] += gv[i] * xv[i], acc_b[i] += gv[i];
        }
        const float2 tot = cta_sum2(s1, s2, scratch);
        const float a = tot.x * inv_d, b = tot.y * inv_d;
        float dx[8];
#pragma unroll
        for (int i = 0; i < 8; i++) dx[i] = rs * (gv[i] * g[i] - a - xv[i] * b);
        store8(gx + r * D + c0, dx);
    }
    float *pg = part + int64_t(blockIdx.x) * D + c0, *pb = part + (int64_t(gridDim.x) + blockIdx.x) * D + c0;
    *reinterpret_cast<float4 *>(pg) = make_float4(acc_g[0], acc_g[1], acc_g[2], acc_g[3]);
    *reinterpret_cast<float4 *>(pg + 4) = make_float4(acc_g[4], acc_g[5], acc_g[6], acc_g[7]);
    *reinterpret_cast<float4 *>(pb) = make_float4(acc_b[0], acc_b[1], acc_b[2], acc_b[3]);
    *reinterpret_cast<float4 *>(pb + 4) = make_float4(acc_b[4], acc_b[5], acc_b[6], acc_b[7]);
}

// part [2][nparts][D] -> ggamma [D], gbeta [D] in two steps, each adding in a fixed order.
// Step 1: CTA (x, y) owns 32 columns and the partial rows p with p % kSplits == y; its 8 warps
// take every 8th of those in ascending order and their eight sums are added in warp order.
// Step 2: one thread per column adds the kSplits results in ascending order.
constexpr int kSplits = 16;

__global__ void __launch_bounds__(256)
layernorm_backward_sum1_kernel(const float *__restrict__ part, int nparts, int D, float *__restrict__ part2)
{
    __shared__ float sm[2][8][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, c = blockIdx.x * 32 + lane;
    float sg = 0.0f, sb = 0.0f;
    for (int p = blockIdx.y + kSplits * warp; p < nparts; p += kSplits * 8) {
        sg += part[int64_t(p) * D + c];
        sb += part[(int64_t(nparts) + p) * D + c];
    }
    sm[0][warp][lane] = sg, sm[1][warp][lane] = sb;
    __syncthreads();
    if (warp == 0) {
        float tg = 0.0f, tb = 0.0f;
        for (int w = 0; w < 8; w++) tg += sm[0][w][lane], tb += sm[1][w][lane];
        part2[int64_t(blockIdx.y) * D + c] = tg;
        part2[int64_t(kSplits + blockIdx.y) * D + c] = tb;
    }
}

__global__ void __launch_bounds__(256)
layernorm_backward_sum2_kernel(const float *__restrict__ part2, int D, float *__restrict__ ggamma, float *__restrict__ gbeta)
{
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= D) return;
    float tg = 0.0f, tb = 0.0f;
    for (int s = 0; s < kSplits; s++) tg += part2[int64_t(s) * D + c], tb += part2[int64_t(kSplits + s) * D + c];
    if (ggamma) ggamma[c] = tg;
    if (gbeta) gbeta[c] = tb;
}

int parts_for(int64_t rows, int64_t D)
{
    const int threads = int(D / 8);
    const int64_t cap = int64_t(sm_count()) * (threads >= 512 ? 2 : threads >= 256 ? 4 : 8);
    return int(rows < cap ? rows : cap);
}

}  // namespace
}  // namespace ls

using namespace ls;

extern "C" int64_t ls_layernorm_backward_scratch(int64_t rows, int64_t D)
{
    if (rows < 0 || D <= 0 || D % 256 != 0 || D > 8192) return -1;
    return int64_t(2) * (parts_for(rows, D) + kSplits) * D;
}

extern "C" int ls_layernorm_backward(const void *gy, int gy_dtype, const void *x, int x_dtype, const float *mean,
                                     const float *rstd, const float *gamma, int64_t rows, int64_t D, void *gx,
                                     float *ggamma, float *gbeta, float *scratch, void *stream)
{
    if (int rc = check_device()) return rc;
    if ((x_dtype != LS_F32 && x_dtype != LS_BF16) || (gy_dtype != LS_F32 && gy_dtype != LS_BF16))
        return fail(LS_EINVAL, "unsupported dtype %d / %d", x_dtype, gy_dtype);
    if (rows < 0 || D <= 0 || D % 256 != 0 || D > 8192) return fail(LS_EINVAL, "D=%lld must be a multiple of 256, at most 8192", (long long)D);
    if (rows == 0) return LS_OK;
    if (rows >= (int64_t(1) << 31)) return fail(LS_EINVAL, "too many rows");
    if (!gy || !x || !mean || !rstd || !gx || !scratch) return fail(LS_EINVAL, "null pointer");
    if (!aligned16(gy) || !aligned16(x) || !aligned16(gx) || !aligned16(scratch)) return fail(LS_EALIGN, "gy, x, gx and scratch must be 16-byte aligned");
    const int threads = int(D / 8), parts = parts_for(rows, D);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define LS_LNB(TX, TG) layernorm_backward_kernel<TX, TG><<<parts, threads, 0, st>>>(static_cast<const TX *>(x), static_cast<const TG *>(gy), mean, rstd, gamma, rows, int(D), static_cast<TX *>(gx), scratch)
    if (x_dtype == LS_F32 && gy_dtype == LS_F32) LS_LNB(float, float);
    else if (x_dtype == LS_F32) LS_LNB(float, __nv_bfloat16);
    else if (gy_dtype == LS_F32) LS_LNB(__nv_bfloat16, float);
    else LS_LNB(__nv_bfloat16, __nv_bfloat16);
#undef LS_LNB
    LS_LAUNCH_CHECK("layernorm_backward");
    if (ggamma || gbeta) {
        float *part2 = scratch + int64_t(2) * parts * D;
        layernorm_backward_sum1_kernel<<<dim3(unsigned(D / 32), kSplits), 256, 0, st>>>(scratch, parts, int(D), part2);
        layernorm_backward_sum2_kernel<<<int((D + 255) / 256), 256, 0, st>>>(part2, int(D), ggamma, gbeta);
        LS_LAUNCH_CHECK("layernorm_backward_sum");
    }
    return LS_OK;
}

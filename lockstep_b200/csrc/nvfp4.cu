// NVFP4: blocks of 16 E2M1 values under one E4M3 scale (4.5 bits per element).
//
// The rule is the one lockstep's format study states (rig_sm75/quant_sim.cuh:90-97 with
// :20-33 and :57-69, applied per block as rig_q.cu:348-363 does):
//   amax  = max |v| over the block, NaNs skipped
//   scale = E4M3(amax / 6), round-half-even, saturating at 448; 2^-9 where that gives 0;
//           1.0 for a block without a positive maximum
//   code  = E2M1 value nearest to v / scale (IEEE division), ties to the smaller
//           magnitude; NaN and +-Inf quotients give magnitude 0
// The literal evaluation executes no division per element.  The code's magnitude is the number
// of rounding midpoints m of E2M1 (0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5) with RN(|v| / s) > m.
// Each m has an even significand, so RN(q) > m exactly when q > m + ulp(m) / 2, i.e.
// |v| > m s + (ulp(m) / 2) s.  Both products are exact in fp32 (3 + 4 significant bits), and
// for an fp32 |v| the comparison with their real sum equals the comparison with that sum
// rounded down: seven thresholds per block, seven comparisons per element.  Most blocks never
// get there: a multiplication and the hardware converter give the same codes (see the kernel).
// A thread owns one block at a time (two per launch, their loads issued together): 32 or 64
// bytes in, 8 bytes of codes and one scale byte out.
// Four neighbouring lanes hold the four scales of one word of the tensor-core scale-factor
// layout, so the scale bytes leave as words.

#include "common.cuh"

namespace ls {
namespace {

constexpr int kThreads = 256;
constexpr int kBlocksPerThread = 2;

struct Nvfp4Out {
    uint8_t *packed;       // [rows, K/2]
    uint8_t *scale_u8;     // [rows, K/16] E4M3 bytes, or NULL
    float *scale_f32;      // [rows, K/16] the same scales as fp32, or NULL
    uint8_t *sf;           // scale-factor layout, or NULL
    uint32_t kblocks;      // K / 16
    uint32_t nblocks;      // rows * kblocks
    uint32_t div_mul, div_shift;   // row = block / kblocks by multiply-shift
};

// floor(b / kblocks) for any 32-bit b: t = hi(b * mul); q = (t + ((b - t) >> 1)) >> shift
__device__ __forceinline__ uint32_t row_of(const Nvfp4Out &o, uint32_t b)
{
    const uint32_t t = __umulhi(b, o.div_mul);
    return (t + ((b - t) >> 1)) >> o.div_shift;
}

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

struct Thresholds { float u[7]; };

// thresholds of one block: |v| > u[j]  <=>  RN(|v| / s) > midpoint j
__device__ __forceinline__ Thresholds thresholds_of(float s)
{
    const float mid[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
    // half an ulp above each midpoint: 2^-26, 2^-25, 2^-24, 2^-24, 2^-23, 2^-23, 2^-22
    const float half_ulp[7] = {1.4901161e-08f, 2.9802322e-08f, 5.9604645e-08f, 5.9604645e-08f,
                               1.1920929e-07f, 1.1920929e-07f, 2.3841858e-07f};
    Thresholds t;
#pragma unroll
    for (int j = 0; j < 7; j++) t.u[j] = __fadd_rd(__fmul_rn(mid[j], s), __fmul_rn(half_ulp[j], s));   // both products exact
    return t;
}

__device__ __forceinline__ uint32_t nearest_e2m1(float v, const Thresholds &t)
{
    const float a = fabsf(v);
    uint32_t c = 0;
#pragma unroll
    for (int j = 0; j < 7; j++) c += uint32_t(a > t.u[j]);
    if (a == __uint_as_float(kBitsInf)) c = 0;                 // every distance is infinite: the first candidate stays
    return c | (v < 0.0f ? 8u : 0u);
}

struct U8x32 { uint32_t w[8]; };

__device__ __forceinline__ U8x32 ld_stream32(const void *p)
{
    U8x32 v;
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]),
                   "=r"(v.w[6]), "=r"(v.w[7]) : "l"(p));
    return v;
}

// One block of 16 as loaded: bf16 in 8 words, fp32 in 16.
template <typename T> struct Raw;
template <> struct Raw<__nv_bfloat16> { uint32_t w[8]; };
template <> struct Raw<float> { uint32_t w[16]; };

__device__ __forceinline__ void load_raw(const __nv_bfloat16 *x, Raw<__nv_bfloat16> &r)
{
    const U8x32 a = ld_stream32(x);
#pragma unroll
    for (int i = 0; i < 8; i++) r.w[i] = a.w[i];
}
__device__ __forceinline__ void load_raw(const float *x, Raw<float> &r)
{
    const U8x32 a = ld_stream32(x), b = ld_stream32(x + 8);
#pragma unroll
    for (int i = 0; i < 8; i++) r.w[i] = a.w[i], r.w[8 + i] = b.w[i];
}
__device__ __forceinline__ float elem(const Raw<__nv_bfloat16> &r, int i)
{
    return __uint_as_float((i & 1) ? (r.w[i >> 1] & 0xFFFF0000u) : (r.w[i >> 1] << 16));
}
__device__ __forceinline__ float elem(const Raw<float> &r, int i) { return __uint_as_float(r.w[i]); }

// Bits of the block maximum of |v| as fp32, NaN-propagating: above 0x7F800000 if the block
// holds a NaN, equal to it if it holds an infinity and no NaN.
__device__ __forceinline__ uint32_t amax_bits(const Raw<__nv_bfloat16> &r)
{
    __nv_bfloat162 m = __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&r.w[0]));
#pragma unroll
    for (int i = 1; i < 8; i++) m = __hmax2_nan(m, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&r.w[i])));
    const uint32_t mb = *reinterpret_cast<const uint32_t *>(&m);
    return max(mb & 0xFFFF0000u, mb << 16);                    // a NaN pattern is the larger integer
}
__device__ __forceinline__ uint32_t amax_bits(const Raw<float> &r)
{
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 16; i++) m = max(m, r.w[i] & 0x7FFFFFFFu);
    return m;
}

__device__ __forceinline__ uint32_t scale_byte(float amax)      // amax >= 0, not NaN
{
    if (!(amax > 0.0f)) return 0x38u;                           // 1.0
    const uint32_t sb = e4m3_byte_sat(__fdiv_rn(amax, 6.0f));
    return sb ? sb : 1u;                                        // the smallest subnormal, 2^-9
}

// codes of eight elements (first = e0) from q = v * r through the hardware converter; the
// +0.0 addend turns a -0.0 input into +0.0 (the rule's sign is `v < 0`)
template <typename T>
__device__ __forceinline__ uint32_t convert8(const Raw<T> &raw, int e0, float r)
{
    float q[8];
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = __fmaf_rn(elem(raw, e0 + i), r, 0.0f);
    return cvt_e2m1x8(q);
}

// quant_sim.cuh:57-69 as written: the first candidate whose fp32 distance |a - m| is strictly the
// smallest.  Equal to "nearest, ties to the smaller magnitude" while a - m is exact (a < 2^23);
// beyond, the distances to several candidates round to the same float and a smaller code wins.
__device__ __forceinline__ uint32_t first_nearest_e2m1(float x)
{
    const float m[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    const float a = fabsf(x);
    uint32_t best = 0;
    float bd = fabsf(__fsub_rn(a, m[0]));
#pragma unroll
    for (int i = 1; i < 8; i++) {
        const float d = fabsf(__fsub_rn(a, m[i]));
        if (d < bd) bd = d, best = i;
    }
    return best | (x < 0.0f ? 8u : 0u);
}

constexpr uint32_t kBitsHuge = 0x4F000000u;    // 2^31: below, every quotient is < 2^23 (the scale is 448 from 2688 on)

// The rule for any input: by thresholds, or by division and the candidate loop where a quotient
// may reach 2^23.
template <typename T>
__device__ __forceinline__ void exact_block(const Raw<T> &raw, uint32_t &sb, uint32_t &lo, uint32_t &hi)
{
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(elem(raw, i)));     // fmaxf drops a NaN operand
    sb = scale_byte(amax);
    const float s = e4m3_value(sb);
    lo = hi = 0;
    if (__float_as_uint(amax) >= kBitsHuge) {
#pragma unroll                                           // (a rolled loop would index the registers of `raw`)
        for (int i = 0; i < 8; i++) {
            lo |= first_nearest_e2m1(__fdiv_rn(elem(raw, i), s)) << (4 * i);
            hi |= first_nearest_e2m1(__fdiv_rn(elem(raw, 8 + i), s)) << (4 * i);
        }
        return;
    }
    const Thresholds th = thresholds_of(s);
#pragma unroll
    for (int i = 0; i < 8; i++) {
        lo |= nearest_e2m1(elem(raw, i), th) << (4 * i);
        hi |= nearest_e2m1(elem(raw, 8 + i), th) << (4 * i);
    }
}

// Fast path.  With q' = v * r' for a reciprocal r' a little off 1 / s, the hardware converter
// (nearest, ties to even) gives the rule's code whenever no rounding midpoint lies between q'
// and the quotient the rule rounds:
//  * bf16 input: v has 8 significant bits and midpoint x scale at most 7, so v / s either is a
//    midpoint or is at least 2^-9 away from it in relative terms.  r' = (1 / s)(1 - 2^-12) moves
//    an exact midpoint just below itself (the rule's tie goes down) and nothing else across.
//  * fp32 input: two conversions with r' = (1 / s)(1 -+ 2^-21) bracket the quotient by far more
//    than the half ulp the rule's rounding can move it; equal codes are the rule's codes, unequal
//    codes (a value within 2^-20 of a midpoint) send the block to the literal evaluation.
// Blocks holding a NaN, an infinity or a value from 2^31 on always go there (the rule maps NaN
// and infinite quotients to magnitude 0, and its fp32 distances stop telling the candidates
// apart for quotients from 2^23 on).
template <typename T>
__global__ void __launch_bounds__(kThreads)
nvfp4_quantize_kernel(const T *__restrict__ x, Nvfp4Out o)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // kBlocksPerThread blocks per thread, all loads issued before the first is used
    Raw<T> raws[kBlocksPerThread];
#pragma unroll
    for (int u = 0; u < kBlocksPerThread; u++) {
        const uint32_t b = (blockIdx.x * kBlocksPerThread + u) * kThreads + threadIdx.x;
        if (b < o.nblocks) load_raw(x + size_t(b) * 16, raws[u]);
        else
#pragma unroll
            for (int i = 0; i < int(sizeof(raws[u].w) / 4); i++) raws[u].w[i] = 0u;
    }
#pragma unroll
    for (int u = 0; u < kBlocksPerThread; u++) {
    const Raw<T> &raw = raws[u];
    const uint32_t blk = (blockIdx.x * kBlocksPerThread + u) * kThreads + threadIdx.x;
    const bool in_range = blk < o.nblocks;
    const uint32_t ab = amax_bits(raw);
    bool literal = ab >= kBitsHuge;                            // also every block with an infinity or a NaN
    uint32_t sb = 0x38u, lo = 0, hi = 0;
    if (!literal) {
        sb = scale_byte(__uint_as_float(ab));
        const float r = __frcp_rn(e4m3_value(sb));
        if (sizeof(T) == 2) {
            const float rc = r * 0.999755859375f;                              // 1 - 2^-12
            lo = convert8(raw, 0, rc), hi = convert8(raw, 8, rc);
        } else {
            const float ra = r * 0.99999952316284f, rb = r * 1.00000047683716f; // 1 -+ 2^-21
            lo = convert8(raw, 0, ra), hi = convert8(raw, 8, ra);
            literal = lo != convert8(raw, 0, rb) || hi != convert8(raw, 8, rb);
        }
    }
    if (literal) exact_block(raw, sb, lo, hi);
    const float s = e4m3_value(sb);
    if (in_range) reinterpret_cast<uint2 *>(o.packed)[blk] = make_uint2(lo, hi);
    // scale bytes of 4 consecutive blocks (same row: K / 16 is a multiple of 8) as one word
    uint32_t w = sb;
    w |= __shfl_down_sync(0xFFFFFFFFu, sb, 1) << 8;
    w |= __shfl_down_sync(0xFFFFFFFFu, sb, 2) << 16;
    w |= __shfl_down_sync(0xFFFFFFFFu, sb, 3) << 24;
    if (in_range && (threadIdx.x & 3) == 0) {
        if (o.scale_u8) *reinterpret_cast<uint32_t *>(o.scale_u8 + blk) = w;
        if (o.sf) {
            const uint32_t row = row_of(o, blk), kb = blk - row * o.kblocks;
            *reinterpret_cast<uint32_t *>(o.sf + sf_offset(row, kb, o.kblocks / 4)) = w;
        }
    }
    if (in_range && o.scale_f32) o.scale_f32[blk] = s;
    }
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
    if ((reinterpret_cast<uintptr_t>(x) & 31) || (reinterpret_cast<uintptr_t>(packed) & 7) ||
        (reinterpret_cast<uintptr_t>(scale_u8) & 3) || (reinterpret_cast<uintptr_t>(scale_f32) & 3) ||
        (reinterpret_cast<uintptr_t>(sf) & 3))
        return fail(LS_EALIGN, "x must be 32-byte, packed 8-byte, scale buffers 4-byte aligned");
    Nvfp4Out o{packed, scale_u8, scale_f32, sf, uint32_t(K / 16), uint32_t(n / 16), 0u, 0u};
    {   // multiply-shift division by kblocks (>= 8 here)
        uint32_t d = o.kblocks, sh = 0;
        while ((1ull << sh) < d) sh++;
        o.div_mul = uint32_t(((1ull << 32) * ((1ull << sh) - d)) / d + 1);
        o.div_shift = sh - 1;
    }
    const int grid = int((o.nblocks + kThreads * kBlocksPerThread - 1) / (kThreads * kBlocksPerThread));
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

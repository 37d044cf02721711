// Shared helpers of the lockstep_b200 library: error reporting, device
// queries, bit-level MXFP4 arithmetic used by every kernel.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <mutex>
#include <stdint.h>

#include "../../include/lockstep_b200.h"

namespace ls {

// ---- host side ------------------------------------------------------------
int fail(int code, const char *fmt, ...);          // records the message, returns code
int check_device();                                 // LS_OK or LS_EARCH / LS_ECUDA
int sm_count();                                     // SMs of the current device
int current_device(int *dev);                       // index of the current device, checked against the per-device tables (64 entries)
std::mutex &state_mutex();                          // guards the library's per-device tables (attributes set, scratch, error words)
struct QuantEpilogue {              // optional MXFP4 output of act(C), per batch
    uint8_t *packed[2];
    uint8_t *sf[2];
    int act;                        // 0 none, 1 GELU (erf form)
};
int gemm_fused(int nbatch, const uint8_t *a0, const uint8_t *a1, const uint8_t *w, const uint8_t *sfa0,
               const uint8_t *sfa1, const uint8_t *sfb, void *c0, void *c1, int out_dtype, int64_t M,
               int64_t N, int64_t K, void *stream, int *err, const QuantEpilogue *qe);
int gemm_common(int nbatch, const uint8_t *a0, const uint8_t *a1, const uint8_t *w, const uint8_t *sfa0,
                const uint8_t *sfa1, const uint8_t *sfb, void *c0, void *c1, int out_dtype, int64_t M,
                int64_t N, int64_t K, void *stream, int *err);

#define LS_CUDA(expr)                                                              \
    do {                                                                           \
        cudaError_t e__ = (expr);                                                  \
        if (e__ != cudaSuccess)                                                    \
            return ::ls::fail(LS_ECUDA, "%s: %s", #expr, cudaGetErrorString(e__)); \
    } while (0)

#define LS_LAUNCH_CHECK(name)                                                          \
    do {                                                                               \
        cudaError_t e__ = cudaGetLastError();                                          \
        if (e__ != cudaSuccess)                                                        \
            return ::ls::fail(LS_ECUDA, "launch of %s: %s", name, cudaGetErrorString(e__)); \
    } while (0)

static inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---- device side ----------------------------------------------------------
#ifdef __CUDACC__

constexpr uint32_t kBitsOne = 0x3F800000u;      // 1.0f
constexpr uint32_t kBitsSix = 0x40C00000u;      // 6.0f
constexpr uint32_t kBitsClamp = 0x0DA24260u;    // 1e-30f, the floor of the block maximum
constexpr uint32_t kBitsInf = 0x7F800000u;

// Exponent E of the block scale 2^E from the bit pattern of the block maximum
// (sign cleared).  Returns the E8M0 byte E+127; 0xFF marks a NaN block.
//
// E = floor(log2(max(amax, 1e-30))) - 2 with log2 evaluated in fp32 and
// correctly rounded: for a maximum n ulps below 2^k the logarithm rounds to
// k itself when n <= 2^(j-1) ln 2, j = bit length of k-1 (k > 0) or of |k|
// (k < 0), so the exponent is then k, not k-1.  A zero block has E = 0 and an
// infinite maximum E = 127 (the clamp).
__device__ __forceinline__ uint32_t block_e8m0(uint32_t amax_bits)
{
    if (amax_bits == 0u) return 127u;
    if (amax_bits >= kBitsInf) return amax_bits == kBitsInf ? 254u : 255u;
    uint32_t a = max(amax_bits, kBitsClamp);
    int e = int(a >> 23) - 127;
    uint32_t mant = a & 0x7FFFFFu;
    int k = e + 1;
    uint32_t mag = k > 0 ? uint32_t(k - 1) : uint32_t(-k);
    int j = 32 - __clz(mag);                         // 0..7
    uint32_t nmax = uint32_t((0x2C160B0502010000ull >> (8 * j)) & 0xFFull);
    if (mant != 0u && (0x800000u - mant) <= nmax) e += 1;
    return uint32_t(e - 2 + 127);
}

// 2^(127-b) as fp32 bits: the factor that divides by the block scale 2^(b-127).
// b in [25, 254]; b = 254 needs the subnormal 2^-127.
__device__ __forceinline__ uint32_t inv_scale_bits(uint32_t e8m0)
{
    return e8m0 >= 254u ? 0x00400000u : ((254u - e8m0) << 23);
}

// fp32 bits of the scale 2^(b-127) (b >= 1 here), NaN for b = 255.
__device__ __forceinline__ uint32_t scale_bits(uint32_t e8m0)
{
    return e8m0 == 255u ? 0x7FC00000u : (e8m0 << 23);
}

// E2M1 code of q, a value halfway between two grid points keeping the smaller
// magnitude (RNE = false) or going to the even code (RNE = true).  NaN gives
// magnitude 7, as torch.bucketize does.  Integer arithmetic on the bit
// pattern: with one kept mantissa bit, adding (half - 1) and truncating
// rounds half down; below 1.0 the grid is uniform (0, 0.5, 1.0), so the value
// is first lifted into [1, 2] with a round-up add that cannot move it across
// or off a halfway point.
template <bool RNE>
__device__ __forceinline__ uint32_t e2m1_code(float q)
{
    uint32_t u = __float_as_uint(q);
    uint32_t a = min(u & 0x7FFFFFFFu, kBitsSix);
    bool small = a < kBitsOne;
    uint32_t v = small ? __float_as_uint(__fadd_ru(__uint_as_float(a), 1.0f)) : a;
    uint32_t code = ((v + 0x1FFFFFu) >> 22) - (small ? 254u : 252u);
    if (RNE) {
        // below 1.0 the lift may round, so halfway is tested on the value itself
        bool tie = small ? (a == 0x3E800000u || a == 0x3F400000u) : ((a & 0x3FFFFFu) == 0x200000u);
        code += (tie && (code & 1u)) ? 1u : 0u;
    }
    return code | ((u >> 28) & 8u);
}

// value of an E2M1 code as fp32 (code 8 is -0.0)
__device__ __forceinline__ float e2m1_value(uint32_t code)
{
    // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 = halves 0,1,2,3,4,6,8,12
    uint32_t halves = (0xC8643210u >> (4 * (code & 7u))) & 0xFu;
    float v = float(halves) * 0.5f;
    return __uint_as_float(__float_as_uint(v) | ((code & 8u) << 28));
}

// Four E2M1 codes (the low 16 bits of pk) -> their fp32 values, by two byte-permute
// table lookups: the upper 16 bits of the fp32 pattern of each magnitude are
// 0000 3F00 3F80 3FC0 4000 4040 4080 40C0, the lower 16 bits are zero.
__device__ __forceinline__ void e2m1x4_values(uint32_t pk, float (&v)[4])
{
    const uint32_t sel = pk & 0x7777u;
    const uint32_t tops = __byte_perm(0x3F3F3F00u, 0x40404040u, sel);     // byte i: bits 31..24 of value i
    const uint32_t secs = __byte_perm(0xC0800000u, 0xC0804000u, sel);     // byte i: bits 23..16 of value i
    const uint32_t a01 = __byte_perm(tops, secs, 0x1504u);                // value 1 in the high half, 0 in the low
    const uint32_t a23 = __byte_perm(tops, secs, 0x3726u);
    v[0] = __uint_as_float((a01 << 16) | ((pk << 28) & 0x80000000u));
    v[1] = __uint_as_float((a01 & 0xFFFF0000u) | ((pk << 24) & 0x80000000u));
    v[2] = __uint_as_float((a23 << 16) | ((pk << 20) & 0x80000000u));
    v[3] = __uint_as_float((a23 & 0xFFFF0000u) | ((pk << 16) & 0x80000000u));
}

// Eight E2M1 codes (one packed word, element 0 in the low nibble) -> their fp32 values,
// through the hardware converter to f16 pairs (every E2M1 value is exact in f16; code 8
// gives -0.0).
__device__ __forceinline__ void e2m1x8_values(uint32_t pk, float (&v)[8])
{
    uint32_t h[4];
    asm("{\n.reg .b8 b0, b1, b2, b3;\nmov.b32 {b0, b1, b2, b3}, %4;\n"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\ncvt.rn.f16x2.e2m1x2 %1, b1;\n"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\ncvt.rn.f16x2.e2m1x2 %3, b3;\n}\n"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3]) : "r"(pk));
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&h[i]));
        v[2 * i] = f.x, v[2 * i + 1] = f.y;
    }
}

// Two floats -> one byte of two E2M1 codes (lo in the low nibble), hardware
// round-to-nearest-even with saturation.
__device__ __forceinline__ uint32_t cvt_e2m1x8(const float (&q)[8])
{
    uint32_t out;
    asm("{\n"
        ".reg .b8 b0, b1, b2, b3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
        "mov.b32 %0, {b0, b1, b2, b3};\n"
        "}\n"
        : "=r"(out)
        : "f"(q[0]), "f"(q[1]), "f"(q[2]), "f"(q[3]), "f"(q[4]), "f"(q[5]), "f"(q[6]), "f"(q[7]));
    return out;
}

// Eight finite fp32 values -> eight E2M1 codes with the reference rule (halfway keeps
// the smaller magnitude), through the hardware converter.  The converter rounds
// halfway cases to even; the seven halfway points all have their low 21 mantissa
// bits clear, so every non-zero value with those bits clear is first moved one ulp
// toward zero: a halfway value then rounds down, and no other value changes its
// code (one ulp cannot carry a value with clear low bits across a halfway point).
__device__ __forceinline__ uint32_t cvt_ref_e2m1x8(const float (&q)[8])
{
    float r[8];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const uint32_t u = __float_as_uint(q[i]);
        const bool nudge = ((u << 11) == 0u) && ((u << 1) != 0u);
        r[i] = __uint_as_float(u - (nudge ? 1u : 0u));
    }
    return cvt_e2m1x8(r);
}

// byte offset of the scale factor of (row, kblock) in the tcgen05 layout:
// tiles of 128 rows x 4 k-blocks (512 B), k-tiles innermost; inside a tile
// row r sits at (r % 32) * 16 + (r / 32) * 4 + (kblock % 4).
__device__ __forceinline__ int64_t sf_offset(uint32_t row, uint32_t kb, uint32_t ktiles)
{
    uint32_t r = row & 127u;
    return (int64_t(row >> 7) * ktiles + (kb >> 2)) * 512 + (r & 31u) * 16 + (r >> 5) * 4 + (kb & 3u);
}

__device__ __forceinline__ uint4 ld_stream(const uint4 *p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

#endif  // __CUDACC__
}  // namespace ls

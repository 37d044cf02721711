// MXFP4 codec kernels: fused quantize (+pack, +E8M0, +tensor-core scale
// layout), pack, unpack, dequantize.  All are HBM-bound streaming kernels:
// 128-bit coalesced loads and stores, block maxima by warp shuffles, grids of
// a few CTAs per SM looping over the tensor.
#include "common.cuh"

namespace ls {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;          // 16-byte loads in flight per thread

struct QuantOut {
    uint8_t *codes, *packed, *e8m0, *sf;
    float *scale;
    uint32_t kblocks;               // blocks per row (K / BLOCK)
    uint32_t ktiles;                // K / 128 (scale-factor tiles per row)
    uint32_t div_mul, div_shift;    // row = block / kblocks by multiply-shift (scale-factor layout only)
    uint32_t nblocks;               // rows * kblocks
};

// floor(b / kblocks) for any 32-bit b: t = hi(b * mul); q = (t + ((b - t) >> 1)) >> shift
__device__ __forceinline__ uint32_t div_kblocks(const QuantOut &o, uint32_t b)
{
    uint32_t t = __umulhi(b, o.div_mul);
    return (t + ((b - t) >> 1)) >> o.div_shift;
}

// Stores the results of one 8-element group.  Lanes of a warp hold 32
// consecutive groups; a "quad" (16 lanes, BLOCK = 32) covers 4 consecutive
// blocks of one row, whose exponent bytes are contiguous in every scale
// output, so one lane per quad writes them as one word.
__device__ __forceinline__ uint32_t spread_codes(uint32_t h)   // 16 bits -> 4 code bytes
{
    return (h & 0xFu) | ((h & 0xF0u) << 4) | ((h & 0xF00u) << 8) | ((h & 0xF000u) << 12);
}

// Exponent bytes of 4 consecutive blocks -> every scale output, written by the lane
// that owns the first of the four.  LPB = lanes per block.
template <int LPB>
__device__ __forceinline__ void store_scales(const QuantOut &o, uint32_t blk_of_lane, uint32_t e8, bool in_range);

template <int BLOCK>
__device__ __forceinline__ void store_group(const QuantOut &o, uint32_t g8, uint32_t pk, uint32_t e8, bool in_range)
{
    constexpr int LPB = BLOCK / 8;
    if (in_range) {
        if (o.packed) reinterpret_cast<uint32_t *>(o.packed)[g8] = pk;
        if (o.codes) reinterpret_cast<uint2 *>(o.codes)[g8] = make_uint2(spread_codes(pk & 0xFFFFu), spread_codes(pk >> 16));
    }
    store_scales<LPB>(o, g8 / LPB, e8, in_range);
}

template <int LPB>
__device__ __forceinline__ void store_scales(const QuantOut &o, uint32_t blk_of_lane, uint32_t e8, bool in_range)
{
    // gather 4 consecutive blocks' exponent bytes into the first lane of each group of 4 blocks
    uint32_t w = e8;
    w |= __shfl_down_sync(0xFFFFFFFFu, e8, LPB) << 8;
    w |= __shfl_down_sync(0xFFFFFFFFu, e8, 2 * LPB) << 16;
    w |= __shfl_down_sync(0xFFFFFFFFu, e8, 3 * LPB) << 24;
    const uint32_t lane = threadIdx.x & 31;
    if (in_range && (lane & (4 * LPB - 1)) == 0) {
        const uint32_t blk = blk_of_lane;               // first of 4 blocks, blk % 4 == 0
        if (blk + 4 <= o.nblocks) {
            if (o.e8m0) *reinterpret_cast<uint32_t *>(o.e8m0 + blk) = w;
            if (o.scale) {
                uint4 sc;
                sc.x = scale_bits(w & 0xFFu), sc.y = scale_bits((w >> 8) & 0xFFu);
                sc.z = scale_bits((w >> 16) & 0xFFu), sc.w = scale_bits(w >> 24);
                *reinterpret_cast<uint4 *>(o.scale + blk) = sc;
            }
        } else {                                        // fewer than 4 blocks left in the tensor
            for (uint32_t i = 0; blk + i < o.nblocks; i++) {
                const uint32_t e = (w >> (8 * i)) & 0xFFu;
                if (o.e8m0) o.e8m0[blk + i] = uint8_t(e);
                if (o.scale) o.scale[blk + i] = __uint_as_float(scale_bits(e));
            }
        }
        if (o.sf) {
            const uint32_t row = div_kblocks(o, blk);
            const uint32_t kb = blk - row * o.kblocks;
            *reinterpret_cast<uint32_t *>(o.sf + sf_offset(row, kb, o.ktiles)) = w;
        }
    }
}

// Generic rounding of 8 values already divided by the scale.
template <bool RNE>
__device__ __forceinline__ uint32_t codes8(const float (&q)[8])
{
    uint32_t pk = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) pk |= e2m1_code<RNE>(q[i]) << (4 * i);
    return pk;
}

// ---- bf16 input -------------------------------------------------------------
// One thread owns 16 consecutive elements (one 32-byte load); two adjacent lanes
// share a block of 32 (a thread owns a whole block of 16).  The codes come from
// the hardware E2M1 converter (round-to-nearest-even).  For the reference rule
// (halfway keeps the smaller magnitude) the divisor carries a factor
// (1 - 2^-12): a bf16 value has 8 significant bits, the factor 12, so the
// product is exact in fp32, lies strictly below every halfway point the value
// sat on, and never crosses one it did not.  Each CTA handles kUnroll16 * 256
// groups; all of a thread's loads are issued before the first use.
constexpr int kUnroll16 = 2;

struct U8x32 { uint32_t w[8]; };

__device__ __forceinline__ U8x32 ld_stream32(const void *p)
{
    U8x32 v;
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v.w[0]), "=r"(v.w[1]), "=r"(v.w[2]), "=r"(v.w[3]), "=r"(v.w[4]), "=r"(v.w[5]),
                   "=r"(v.w[6]), "=r"(v.w[7]) : "l"(p));
    return v;
}

template <int BLOCK, bool RNE>
__global__ void __launch_bounds__(kThreads)
quantize_bf16_kernel(const uint8_t *__restrict__ x, uint32_t n16, QuantOut o)
{
    // lets a GEMM launched with programmatic stream serialization start its set-up under this
    // kernel; that GEMM waits for this grid to finish before it loads anything (no-op otherwise)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int LPB = BLOCK / 16;                    // 2 or 1 lanes per block
    const uint32_t base = blockIdx.x * (kThreads * kUnroll16) + threadIdx.x;
    U8x32 v[kUnroll16];
#pragma unroll
    for (int u = 0; u < kUnroll16; u++) {
        const uint32_t g = base + u * kThreads;
        if (g < n16) v[u] = ld_stream32(x + size_t(g) * 32);
        else
#pragma unroll
            for (int i = 0; i < 8; i++) v[u].w[i] = 0u;
    }
#pragma unroll
    for (int u = 0; u < kUnroll16; u++) {
        const uint32_t g = base + u * kThreads;
        const uint32_t(&w)[8] = v[u].w;
        // |x| maxima on packed bf16 pairs, NaN-propagating
        __nv_bfloat162 m = __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&w[0]));
#pragma unroll
        for (int i = 1; i < 8; i++)
            m = __hmax2_nan(m, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&w[i])));
        uint32_t mb = *reinterpret_cast<uint32_t *>(&m);
        if (LPB == 2) {
            uint32_t other = __shfl_xor_sync(0xFFFFFFFFu, mb, 1);
            __nv_bfloat162 mm = __hmax2_nan(*reinterpret_cast<__nv_bfloat162 *>(&mb),
                                            *reinterpret_cast<__nv_bfloat162 *>(&other));
            mb = *reinterpret_cast<uint32_t *>(&mm);
        }
        const uint32_t amax = max(mb & 0xFFFF0000u, mb << 16);      // as fp32 bits
        // a bf16 maximum is never within 44 ulps (fp32) below a power of two: plain exponent
        uint32_t e8 = (max(amax, kBitsClamp) >> 23) - 2u;
        if (amax == 0u) e8 = 127u;
        uint32_t pk[2];
        if (amax < kBitsInf) {
            const float c = __uint_as_float(RNE ? inv_scale_bits(e8) : (((253u - e8) << 23) | 0x7FF000u));
#pragma unroll
            for (int h = 0; h < 2; h++) {
                float q[8];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    q[2 * i] = __uint_as_float(w[4 * h + i] << 16) * c;
                    q[2 * i + 1] = __uint_as_float(w[4 * h + i] & 0xFFFF0000u) * c;
                }
                pk[h] = cvt_e2m1x8(q);
            }
        } else {                                   // infinite or NaN block maximum
            e8 = amax == kBitsInf ? 254u : 255u;
            const float c = __uint_as_float(e8 == 255u ? 0x7FC00000u : inv_scale_bits(e8));
#pragma unroll
            for (int h = 0; h < 2; h++) {
                float q[8];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    q[2 * i] = __uint_as_float(w[4 * h + i] << 16) * c;
                    q[2 * i + 1] = __uint_as_float(w[4 * h + i] & 0xFFFF0000u) * c;
                }
                pk[h] = codes8<RNE>(q);
            }
        }
        const bool in_range = g < n16;
        if (in_range) {
            if (o.packed) reinterpret_cast<uint2 *>(o.packed)[g] = make_uint2(pk[0], pk[1]);
            if (o.codes)
                reinterpret_cast<uint4 *>(o.codes)[g] = make_uint4(spread_codes(pk[0] & 0xFFFFu), spread_codes(pk[0] >> 16),
                                                                   spread_codes(pk[1] & 0xFFFFu), spread_codes(pk[1] >> 16));
        }
        store_scales<LPB>(o, g / LPB, e8, in_range);
    }
}

// ---- fp32 input -------------------------------------------------------------
// One thread owns 8 consecutive elements (one 32-byte load).  Integer rounding
// on the bit pattern; exact for every fp32 input.
template <int BLOCK, bool RNE>
__global__ void __launch_bounds__(kThreads)
quantize_f32_kernel(const uint8_t *__restrict__ x, uint32_t n8, QuantOut o)
{
    // lets a GEMM launched with programmatic stream serialization start its set-up under this
    // kernel; that GEMM waits for this grid to finish before it loads anything (no-op otherwise)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int LPB = BLOCK / 8;
    constexpr int U = kUnroll / 2;
    const uint32_t base = blockIdx.x * (kThreads * U) + threadIdx.x;
    U8x32 v[U];
#pragma unroll
    for (int u = 0; u < U; u++) {
        const uint32_t g8 = base + u * kThreads;
        if (g8 < n8) v[u] = ld_stream32(x + size_t(g8) * 32);
        else
#pragma unroll
            for (int i = 0; i < 8; i++) v[u].w[i] = 0u;
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
        const uint32_t g8 = base + u * kThreads;
        const uint32_t(&w)[8] = v[u].w;
        uint32_t amax = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) amax = max(amax, w[i] & 0x7FFFFFFFu);
#pragma unroll
        for (int off = 1; off < LPB; off <<= 1)
            amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
        const uint32_t e8 = block_e8m0(amax);
        const float c = __uint_as_float(e8 == 255u ? 0x7FC00000u : inv_scale_bits(e8));
        float q[8];
#pragma unroll
        for (int i = 0; i < 8; i++) q[i] = __uint_as_float(w[i]) * c;
        uint32_t pk;
        if (amax < kBitsInf) pk = RNE ? cvt_e2m1x8(q) : cvt_ref_e2m1x8(q);     // all quotients finite
        else pk = codes8<RNE>(q);
        store_group<BLOCK>(o, g8, pk, e8, g8 < n8);
    }
}

// ---- transposed quantizer -------------------------------------------------------
// x [R, C] row-major -> MXFP4 of x^T [C, R], blocks of 32 running down a column of x
// (what a GEMM that contracts over R needs).  A CTA walks tiles of 128 rows x 256 bytes:
// the rows are copied to shared memory with 16-byte asynchronous copies (the next tile
// is in flight while this one is quantized), then each thread walks one column segment
// of 32 values, so the packed output of a column is written in 64-byte pieces.
constexpr int kTR = 128;                  // tile rows = 4 blocks of 32
constexpr int kTRowBytes = 256;           // bytes of each row in a tile
constexpr int kTSmem = 2 * kTR * kTRowBytes;

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(uint32_t(__cvta_generic_to_shared(smem))),
                 "l"(__cvta_generic_to_global(gmem))
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ACT = 1 (bf16 only): the values quantized are GELU(x) rounded to bf16, as if an elementwise
// pass had come first -- applied to the tile once it is in shared memory, so that the
// activation of a feed-forward layer never has to exist in HBM for its weight gradient.
template <typename T, bool RNE, int ACT = 0>
__global__ void __launch_bounds__(kThreads)
quantize_t_kernel(const T *__restrict__ x, int64_t R, int64_t C, uint8_t *__restrict__ packed,
                  float *__restrict__ scale, uint8_t *__restrict__ sf, uint8_t *__restrict__ row_packed,
                  uint8_t *__restrict__ row_sf)
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // see quantize_bf16_kernel
    // A tile sits in shared memory as rows of 16-byte chunks.  Row r is rotated by
    // 2 * (r / 32) + r % 8 chunks: the column reads below (4 row groups x 8 columns per
    // warp, all lanes at the same r % 8) and the row reads of the row-wise outputs (8
    // consecutive rows per quarter warp) then fall on different banks without padding,
    // and the row writes stay 16-byte vectors.
    auto rot = [](int r) { return 2 * (r >> 5) + (r & 7); };
    constexpr int VEC = 16 / sizeof(T);                          // elements per 16-byte chunk
    constexpr int TC = kTRowBytes / sizeof(T);                   // tile columns
    constexpr int CHUNKS = TC / VEC;                             // per tile row
    extern __shared__ uint4 tile_smem[];                         // two tiles
    const int64_t tiles_x = (C + TC - 1) / TC, tiles = tiles_x * (R / kTR);
    const bool vec_ok = (C % VEC) == 0;

    auto stage = [&](int64_t t, uint4 *buf) {                    // tile t -> buf, asynchronously where it can be
        const int64_t r0 = (t / tiles_x) * kTR, c0 = (t % tiles_x) * TC;
#pragma unroll
        for (int i = threadIdx.x; i < kTR * CHUNKS; i += kThreads) {
            const int r = i / CHUNKS, ch = i % CHUNKS, cc = ch * VEC;
            uint4 *dst = buf + r * CHUNKS + ((ch + rot(r)) & (CHUNKS - 1));
            const T *src = x + (r0 + r) * C + c0 + cc;
            if (vec_ok && c0 + cc + VEC <= C) {
                cp_async16(dst, src);
            } else {                                             // ragged right edge, or rows not 16-byte aligned
                alignas(16) T e[VEC];
#pragma unroll
                for (int k = 0; k < VEC; k++) e[k] = c0 + cc + k < C ? src[k] : T(0.0f);
                *dst = *reinterpret_cast<uint4 *>(e);
            }
        }
        cp_async_commit();
    };

    int b = 0;
    if (int64_t(blockIdx.x) < tiles) stage(blockIdx.x, tile_smem);
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x, b ^= 1) {
        const int64_t next = t + gridDim.x;
        if (next < tiles) {
            stage(next, tile_smem + (b ^ 1) * kTR * CHUNKS);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if constexpr (ACT == 1 && sizeof(T) == 2) {
            uint32_t *words = reinterpret_cast<uint32_t *>(tile_smem + b * kTR * CHUNKS);
#pragma unroll 4
            for (int i = threadIdx.x; i < kTR * CHUNKS * 4; i += kThreads) {
                const uint32_t u = words[i];
                float lo = __uint_as_float(u << 16), hi = __uint_as_float(u & 0xFFFF0000u);
                lo = (lo * 0.5f) * (1.0f + erff(lo * 0.70710678118654752440f));
                hi = (hi * 0.5f) * (1.0f + erff(hi * 0.70710678118654752440f));
                const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                words[i] = *reinterpret_cast<const uint32_t *>(&h);
            }
            __syncthreads();
        }
        const T *tile = reinterpret_cast<const T *>(tile_smem + b * kTR * CHUNKS);
        const int64_t r0 = (t / tiles_x) * kTR, c0 = (t % tiles_x) * TC;
        auto emit = [&](int64_t col, int rb, uint32_t e8, const uint32_t (&pk)[4]) {
            // exponent bytes of this column's 4 blocks (lanes rb = 0..3) -> one word at lane rb = 0
            uint32_t w = e8;
            w |= __shfl_down_sync(0xFFFFFFFFu, e8, 1) << 8;
            w |= __shfl_down_sync(0xFFFFFFFFu, e8, 2) << 16;
            w |= __shfl_down_sync(0xFFFFFFFFu, e8, 3) << 24;
            if (col >= C) return;
            if (packed)
                *reinterpret_cast<uint4 *>(packed + col * (R / 2) + (r0 + rb * 32) / 2) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            if (rb == 0) {
                const int64_t kb = r0 / 32;                      // first of 4 blocks: one scale tile
                if (scale) {
                    uint4 sc;
                    sc.x = scale_bits(w & 0xFFu), sc.y = scale_bits((w >> 8) & 0xFFu);
                    sc.z = scale_bits((w >> 16) & 0xFFu), sc.w = scale_bits(w >> 24);
                    *reinterpret_cast<uint4 *>(scale + col * (R / 32) + kb) = sc;
                }
                if (sf) *reinterpret_cast<uint32_t *>(sf + sf_offset(uint32_t(col), uint32_t(kb), uint32_t(R / 128))) = w;
            }
        };
        if constexpr (sizeof(T) == 2) {
            // bf16: a thread takes two adjacent columns (one 32-bit word per row) of one row
            // group.  Maxima run on packed pairs; the reference's rounding of halfway values
            // comes from a reciprocal scale shortened by 2^-12 (the product is exact) and the
            // hardware's round-to-nearest-even conversion, as in the row-wise kernel.
            static_assert(sizeof(T) != 2 || 4 * (TC / 2) == kThreads, "one item per thread");
            const uint32_t *tile32 = reinterpret_cast<const uint32_t *>(tile);
            const int rb = threadIdx.x & 3, cp = threadIdx.x >> 2;
            uint32_t w[32];
#pragma unroll
            for (int i = 0; i < 32; i++)      // word of this column pair in row rb * 32 + i, rotated by 4 words per chunk
                w[i] = tile32[(rb * 32 + i) * (TC / 2) + ((cp + 4 * (2 * rb + (i & 7))) & (TC / 2 - 1))];
            __nv_bfloat162 m = __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&w[0]));
#pragma unroll
            for (int i = 1; i < 32; i++) m = __hmax2_nan(m, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&w[i])));
            const uint32_t mb = *reinterpret_cast<uint32_t *>(&m);
#pragma unroll
            for (int hi = 0; hi < 2; hi++) {
                const uint32_t amax = hi ? (mb & 0xFFFF0000u) : (mb << 16);       // as fp32 bits
                const uint32_t e8 = block_e8m0(amax);
                const bool finite = amax < kBitsInf;
                const float cmul = __uint_as_float(e8 == 255u      ? 0x7FC00000u
                                                   : (RNE || !finite) ? inv_scale_bits(e8)
                                                                      : (((253u - e8) << 23) | 0x7FF000u));
                uint32_t pk[4];
#pragma unroll
                for (int h = 0; h < 4; h++) {
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 8; i++)
                        v[i] = __uint_as_float(hi ? (w[8 * h + i] & 0xFFFF0000u) : (w[8 * h + i] << 16)) * cmul;
                    pk[h] = finite ? cvt_e2m1x8(v) : codes8<RNE>(v);
                }
                emit(c0 + 2 * cp + hi, rb, e8, pk);
            }
        } else {
#pragma unroll
            for (int item = threadIdx.x; item < 4 * TC; item += kThreads) {
                const int rb = item & 3, c = item >> 2;              // 4 blocks of 32 per column
                float q[32];
                uint32_t amax = 0;
#pragma unroll
                for (int i = 0; i < 32; i++) {                       // this column inside the rotated row rb * 32 + i
                    q[i] = float(tile[(rb * 32 + i) * TC + ((c + VEC * (2 * rb + (i & 7))) & (TC - 1))]);
                    amax = max(amax, __float_as_uint(q[i]) & 0x7FFFFFFFu);
                }
                const uint32_t e8 = block_e8m0(amax);
                const float inv = __uint_as_float(e8 == 255u ? 0x7FC00000u : inv_scale_bits(e8));
                uint32_t pk[4];
#pragma unroll
                for (int h = 0; h < 4; h++) {
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) v[i] = q[8 * h + i] * inv;
                    if (amax < kBitsInf) pk[h] = RNE ? cvt_e2m1x8(v) : cvt_ref_e2m1x8(v);
                    else pk[h] = codes8<RNE>(v);
                }
                emit(c0 + c, rb, e8, pk);
            }
        }
        if (row_packed) {
            // Row-wise MXFP4 of the same tile (blocks of 32 along a row), for callers that
            // need both orientations of one tensor: x is read from HBM once.
            constexpr int BLKS = TC / 32, CPB = 32 / VEC;            // blocks per tile row, chunks per block
            const uint4 *tile4 = tile_smem + b * kTR * CHUNKS;
#pragma unroll
            for (int item = threadIdx.x; item < kTR * BLKS; item += kThreads) {
                const int blk = item / kTR, r = item % kTR;          // a warp: 32 consecutive rows, one block each
                float q[32];
                uint32_t amax = 0;
                __nv_bfloat162 m2 = __floats2bfloat162_rn(0.0f, 0.0f);   // bf16: |x| maxima on packed pairs, NaN-propagating
#pragma unroll
                for (int j = 0; j < CPB; j++) {
                    const uint4 v = tile4[r * CHUNKS + ((blk * CPB + j + rot(r)) & (CHUNKS - 1))];
                    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        if constexpr (sizeof(T) == 2) {
                            m2 = __hmax2_nan(m2, __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&u[k])));
                            q[j * 8 + 2 * k] = __uint_as_float(u[k] << 16);
                            q[j * 8 + 2 * k + 1] = __uint_as_float(u[k] & 0xFFFF0000u);
                        } else {
                            q[j * 4 + k] = __uint_as_float(u[k]);
                            amax = max(amax, u[k] & 0x7FFFFFFFu);
                        }
                    }
                }
                if constexpr (sizeof(T) == 2) {
                    const uint32_t mb = *reinterpret_cast<uint32_t *>(&m2);
                    amax = max(mb & 0xFFFF0000u, mb << 16);              // as fp32 bits
                }
                const uint32_t e8 = block_e8m0(amax);
                const bool finite = amax < kBitsInf;
                // bf16 values: the shortened reciprocal scale gives the reference's rounding
                // through the round-to-nearest-even converter (see the column path above)
                const bool fold = sizeof(T) == 2 && !RNE && finite;
                const float inv = __uint_as_float(e8 == 255u ? 0x7FC00000u
                                                  : fold     ? (((253u - e8) << 23) | 0x7FF000u)
                                                             : inv_scale_bits(e8));
                uint32_t pk[4];
#pragma unroll
                for (int h = 0; h < 4; h++) {
                    float v[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) v[i] = q[8 * h + i] * inv;
                    if (!finite) pk[h] = codes8<RNE>(v);
                    else pk[h] = (RNE || sizeof(T) == 2) ? cvt_e2m1x8(v) : cvt_ref_e2m1x8(v);
                }
                const int64_t row = r0 + r, col = c0 + 32 * blk;
                if (col < C) {
                    *reinterpret_cast<uint4 *>(row_packed + row * (C / 2) + col / 2) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    row_sf[sf_offset(uint32_t(row), uint32_t(col / 32), uint32_t(C / 128))] = uint8_t(e8);
                }
            }
        }
        __syncthreads();                                         // this buffer is refilled by the next iteration's copies
    }
}

// ---- pack / unpack ----------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
pack_kernel(const uint4 *__restrict__ codes, uint2 *__restrict__ packed, int64_t n16,
            const uint8_t *codes_tail, uint8_t *packed_tail, int tail_bytes)
{
    const int64_t stride = int64_t(gridDim.x) * kThreads;
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < n16; i += stride) {
        uint4 c = ld_stream(codes + i);
        auto squeeze = [](uint32_t a) {      // 4 code bytes -> 16 bits
            uint32_t t = a | (a >> 4);       // byte0|byte1<<4 in bits 0-7, byte2|byte3<<4 in 16-23
            return (t & 0xFFu) | ((t >> 8) & 0xFF00u);
        };
        uint2 p;
        p.x = squeeze(c.x & 0x0F0F0F0Fu) | (squeeze(c.y & 0x0F0F0F0Fu) << 16);
        p.y = squeeze(c.z & 0x0F0F0F0Fu) | (squeeze(c.w & 0x0F0F0F0Fu) << 16);
        packed[i] = p;
    }
    if (blockIdx.x == 0 && threadIdx.x < tail_bytes)
        packed_tail[threadIdx.x] = uint8_t((codes_tail[2 * threadIdx.x] & 0xF) |
                                           (codes_tail[2 * threadIdx.x + 1] << 4));
}

__device__ __forceinline__ uint32_t spread4(uint32_t h)   // 16 bits -> 4 code bytes
{
    return (h & 0xFu) | ((h & 0xF0u) << 4) | ((h & 0xF00u) << 8) | ((h & 0xF000u) << 12);
}

__global__ void __launch_bounds__(kThreads)
unpack_kernel(const uint2 *__restrict__ packed, uint4 *__restrict__ codes, int64_t n8,
              const uint8_t *packed_tail, uint8_t *codes_tail, int tail_bytes)
{
    const int64_t stride = int64_t(gridDim.x) * kThreads;
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < n8; i += stride) {
        uint2 p = packed[i];
        uint4 c;
        c.x = spread4(p.x & 0xFFFFu);
        c.y = spread4(p.x >> 16);
        c.z = spread4(p.y & 0xFFFFu);
        c.w = spread4(p.y >> 16);
        codes[i] = c;
    }
    if (blockIdx.x == 0 && threadIdx.x < tail_bytes) {
        uint8_t b = packed_tail[threadIdx.x];
        codes_tail[2 * threadIdx.x] = b & 0xF;
        codes_tail[2 * threadIdx.x + 1] = b >> 4;
    }
}

// ---- dequantize ---------------------------------------------------------------
// One thread turns 4 codes (4 bytes, or 2 packed bytes) into 4 outputs per step, so
// that each load and each 16-byte (fp32) store of a warp is one contiguous segment.
template <bool PACKED, bool OUT_BF16>
__global__ void __launch_bounds__(kThreads)
dequantize_kernel(const uint8_t *__restrict__ q, const float *__restrict__ scale,
                  const uint8_t *__restrict__ e8m0, uint32_t n4, int block, void *__restrict__ out)
{
    constexpr int U = 4;
    const uint32_t stride = gridDim.x * kThreads;
    const uint32_t qpb = uint32_t(block) / 4;                 // quads per block
    for (uint32_t q0 = blockIdx.x * kThreads + threadIdx.x; q0 < n4; q0 += U * stride) {
        uint32_t pk[U];
        float sc[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint32_t i = q0 + u * stride;
            const bool ok = i < n4;
            if (PACKED) {
                pk[u] = ok ? reinterpret_cast<const uint16_t *>(q)[i] : 0u;
            } else {
                uint32_t c = ok ? reinterpret_cast<const uint32_t *>(q)[i] : 0u;
                c &= 0x0F0F0F0Fu;
                c |= c >> 4;
                pk[u] = (c & 0xFFu) | ((c >> 8) & 0xFF00u);
            }
            const uint32_t blk = i / qpb;
            sc[u] = !ok ? 0.0f : (scale ? scale[blk] : __uint_as_float(scale_bits(e8m0[blk])));
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint32_t i = q0 + u * stride;
            if (i >= n4) break;
            float f[4];
            e2m1x4_values(pk[u], f);
#pragma unroll
            for (int k = 0; k < 4; k++) f[k] *= sc[u];
            if (OUT_BF16) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(f[0], f[1]), hi = __floats2bfloat162_rn(f[2], f[3]);
                reinterpret_cast<uint2 *>(out)[i] = make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
            } else {
                reinterpret_cast<float4 *>(out)[i] = make_float4(f[0], f[1], f[2], f[3]);
            }
        }
    }
}

__global__ void __launch_bounds__(kThreads)
scales_to_sf_kernel(const float *__restrict__ scale, int64_t nblocks, uint32_t kblocks,
                    uint8_t *__restrict__ sf, int32_t *bad)
{
    const int64_t stride = int64_t(gridDim.x) * kThreads;
    for (int64_t b = int64_t(blockIdx.x) * kThreads + threadIdx.x; b < nblocks; b += stride) {
        uint32_t u = __float_as_uint(scale[b]);
        uint32_t e = (u >> 23) & 0xFFu;
        bool ok = (u & 0x807FFFFFu) == 0u && e >= 1u && e <= 254u;
        if (u == 0x00400000u) { ok = true; e = 0u; }          // 2^-127
        if (!ok) {
            if (bad) atomicAdd(bad, 1);
            e = 255u;
        }
        uint32_t row = uint32_t(b / kblocks);
        uint32_t kb = uint32_t(b - int64_t(row) * kblocks);
        sf[sf_offset(row, kb, kblocks / 4)] = uint8_t(e);
    }
}

template <bool RNE>
__global__ void __launch_bounds__(kThreads)
round_e2m1_kernel(const float *__restrict__ q, int64_t n, uint8_t *__restrict__ codes)
{
    const int64_t stride = int64_t(gridDim.x) * kThreads;
    for (int64_t i = int64_t(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride)
        codes[i] = uint8_t(e2m1_code<RNE>(q[i]));
}

int grid_for(int64_t work_items, int per_cta)
{
    int64_t want = (work_items + per_cta - 1) / per_cta;
    int64_t cap = int64_t(sm_count()) * 8;             // 8 CTAs of 256 threads fill an SM
    return int(want < 1 ? 1 : (want < cap ? want : cap));
}

}  // namespace
}  // namespace ls

using namespace ls;

extern "C" int64_t ls_sf_bytes(int64_t rows, int64_t K)
{
    if (rows < 0 || K < 0 || K % 128 != 0) return -1;
    return ((rows + 127) / 128) * (K / 128) * 512;
}

extern "C" int64_t ls_sf_bytes_block(int64_t rows, int64_t K, int block)
{
    if (rows < 0 || K < 0 || K % 128 != 0 || (block != 32 && block != 16)) return -1;
    return ((rows + 127) / 128) * (K / (4 * block)) * 512;
}

extern "C" int ls_quantize_mxfp4(const void *x, int x_dtype, int64_t rows, int64_t K, int block,
                                 int rounding, uint8_t *codes, uint8_t *packed, float *scale,
                                 uint8_t *e8m0, uint8_t *sf, void *stream)
{
    if (int rc = check_device()) return rc;
    if (block != 32 && block != 16) return fail(LS_EINVAL, "block must be 32 or 16, got %d", block);
    if (rows < 0 || K < 0 || K % block != 0)
        return fail(LS_EINVAL, "K=%lld must be a multiple of block=%d", (long long)K, block);
    if (x_dtype != LS_F32 && x_dtype != LS_BF16) return fail(LS_EINVAL, "unsupported dtype %d", x_dtype);
    if (rounding != LS_ROUND_REF && rounding != LS_ROUND_RNE) return fail(LS_EINVAL, "bad rounding %d", rounding);
    if (rows * K == 0) return LS_OK;
    if (!codes && !packed && !scale && !e8m0 && !sf) return fail(LS_EINVAL, "no output requested");
    if (sf && K % 128 != 0)
        return fail(LS_EINVAL, "scale-factor layout needs K %% 128 == 0 (K=%lld)", (long long)K);
    int64_t n = rows * K;
    if (n == 0) return LS_OK;
    if (!x) return fail(LS_EINVAL, "x is null");
    if (!aligned16(x) || (reinterpret_cast<uintptr_t>(codes) & 15) || (reinterpret_cast<uintptr_t>(packed) & 7) ||
        (reinterpret_cast<uintptr_t>(x) & 31))
        return fail(LS_EALIGN, "x must be 32-byte, codes 16-byte, packed 8-byte aligned");
    if (n / 8 >= (int64_t(1) << 31)) return fail(LS_EINVAL, "more than 2^34 elements in one call");
    if ((reinterpret_cast<uintptr_t>(scale) & 15) || (reinterpret_cast<uintptr_t>(e8m0) & 3) ||
        (reinterpret_cast<uintptr_t>(sf) & 3))
        return fail(LS_EALIGN, "scale must be 16-byte, e8m0 and sf 4-byte aligned");
    QuantOut o{codes, packed, e8m0, sf, scale, uint32_t(K / block), uint32_t(K / (4 * block)), 0u, 0u, uint32_t(n / block)};
    {   // multiply-shift division by kblocks (>= 4 whenever the scale-factor layout is requested)
        uint32_t d = o.kblocks, sh = 0;
        while ((1ull << sh) < d) sh++;
        if (d > 1) {
            o.div_mul = uint32_t(((1ull << 32) * ((1ull << sh) - d)) / d + 1);
            o.div_shift = sh - 1;
        }
    }
    uint32_t n8 = uint32_t(n / 8);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    bool rne = rounding == LS_ROUND_RNE;
    if (x_dtype == LS_BF16) {
        const uint32_t n16 = n8 / 2;
        const uint8_t *xb = static_cast<const uint8_t *>(x);
        int grid = int((n16 + kThreads * kUnroll16 - 1) / (kThreads * kUnroll16));
        if (block == 32) {
            if (rne) quantize_bf16_kernel<32, true><<<grid, kThreads, 0, st>>>(xb, n16, o);
            else quantize_bf16_kernel<32, false><<<grid, kThreads, 0, st>>>(xb, n16, o);
        } else {
            if (rne) quantize_bf16_kernel<16, true><<<grid, kThreads, 0, st>>>(xb, n16, o);
            else quantize_bf16_kernel<16, false><<<grid, kThreads, 0, st>>>(xb, n16, o);
        }
    } else {
        const uint8_t *xf = static_cast<const uint8_t *>(x);
        int grid = int((n8 + kThreads * kUnroll / 2 - 1) / (kThreads * kUnroll / 2));
        if (block == 32) {
            if (rne) quantize_f32_kernel<32, true><<<grid, kThreads, 0, st>>>(xf, n8, o);
            else quantize_f32_kernel<32, false><<<grid, kThreads, 0, st>>>(xf, n8, o);
        } else {
            if (rne) quantize_f32_kernel<16, true><<<grid, kThreads, 0, st>>>(xf, n8, o);
            else quantize_f32_kernel<16, false><<<grid, kThreads, 0, st>>>(xf, n8, o);
        }
    }
    LS_LAUNCH_CHECK("quantize_mxfp4");
    return LS_OK;
}

extern "C" int ls_pack_fp4(const uint8_t *codes, uint8_t *packed, int64_t n_codes, void *stream)
{
    if (int rc = check_device()) return rc;
    if (n_codes < 0 || (n_codes & 1)) return fail(LS_EINVAL, "n_codes must be even");
    if (n_codes == 0) return LS_OK;
    if (!codes || !packed) return fail(LS_EINVAL, "null pointer");
    if (!aligned16(codes) || (reinterpret_cast<uintptr_t>(packed) & 7)) return fail(LS_EALIGN, "codes 16-byte, packed 8-byte aligned");
    int64_t n16 = n_codes / 16;
    int tail = int((n_codes - n16 * 16) / 2);
    pack_kernel<<<grid_for(n16, kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint4 *>(codes), reinterpret_cast<uint2 *>(packed), n16,
        codes + n16 * 16, packed + n16 * 8, tail);
    LS_LAUNCH_CHECK("pack_fp4");
    return LS_OK;
}

extern "C" int ls_unpack_fp4(const uint8_t *packed, uint8_t *codes, int64_t n_bytes, void *stream)
{
    if (int rc = check_device()) return rc;
    if (n_bytes < 0) return fail(LS_EINVAL, "negative size");
    if (n_bytes == 0) return LS_OK;
    if (!codes || !packed) return fail(LS_EINVAL, "null pointer");
    if (!aligned16(codes) || (reinterpret_cast<uintptr_t>(packed) & 7)) return fail(LS_EALIGN, "codes 16-byte, packed 8-byte aligned");
    int64_t n8 = n_bytes / 8;
    int tail = int(n_bytes - n8 * 8);
    unpack_kernel<<<grid_for(n8, kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint2 *>(packed), reinterpret_cast<uint4 *>(codes), n8,
        packed + n8 * 8, codes + n8 * 16, tail);
    LS_LAUNCH_CHECK("unpack_fp4");
    return LS_OK;
}

extern "C" int ls_dequantize_mxfp4(const uint8_t *q, int is_packed, const float *scale,
                                   const uint8_t *e8m0, int64_t rows, int64_t K, int block,
                                   void *out, int out_dtype, void *stream)
{
    if (int rc = check_device()) return rc;
    if (block != 32 && block != 16) return fail(LS_EINVAL, "block must be 32 or 16, got %d", block);
    if (rows < 0 || K < 0 || K % block != 0) return fail(LS_EINVAL, "K must be a multiple of block");
    if (out_dtype != LS_F32 && out_dtype != LS_BF16) return fail(LS_EINVAL, "unsupported dtype %d", out_dtype);
    if (!scale == !e8m0) return fail(LS_EINVAL, "give exactly one of scale and e8m0");
    int64_t n = rows * K;
    if (n == 0) return LS_OK;
    if (!q || !out) return fail(LS_EINVAL, "null pointer");
    if (!aligned16(out) || (reinterpret_cast<uintptr_t>(q) & (is_packed ? 3 : 7))) return fail(LS_EALIGN, "misaligned buffer");
    if (n / 4 >= (int64_t(1) << 32)) return fail(LS_EINVAL, "more than 2^34 elements in one call");
    uint32_t n4 = uint32_t(n / 4);
    int grid = grid_for(n4, kThreads * 4);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (is_packed) {
        if (out_dtype == LS_BF16) dequantize_kernel<true, true><<<grid, kThreads, 0, st>>>(q, scale, e8m0, n4, block, out);
        else dequantize_kernel<true, false><<<grid, kThreads, 0, st>>>(q, scale, e8m0, n4, block, out);
    } else {
        if (out_dtype == LS_BF16) dequantize_kernel<false, true><<<grid, kThreads, 0, st>>>(q, scale, e8m0, n4, block, out);
        else dequantize_kernel<false, false><<<grid, kThreads, 0, st>>>(q, scale, e8m0, n4, block, out);
    }
    LS_LAUNCH_CHECK("dequantize_mxfp4");
    return LS_OK;
}

extern "C" int ls_scales_to_sf(const float *scale, int64_t rows, int64_t K, uint8_t *sf, int32_t *bad,
                               void *stream)
{
    if (int rc = check_device()) return rc;
    if (rows < 0 || K < 0 || K % 128 != 0) return fail(LS_EINVAL, "K must be a multiple of 128");
    int64_t nblocks = rows * (K / 32);
    if (nblocks == 0) return LS_OK;
    if (!scale || !sf) return fail(LS_EINVAL, "null pointer");
    scales_to_sf_kernel<<<grid_for(nblocks, kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        scale, nblocks, uint32_t(K / 32), sf, bad);
    LS_LAUNCH_CHECK("scales_to_sf");
    return LS_OK;
}

extern "C" int ls_scales_to_sf_block(const float *scale, int64_t rows, int64_t K, int block, uint8_t *sf,
                                     int32_t *bad, void *stream)
{
    if (int rc = check_device()) return rc;
    if (block != 32 && block != 16) return fail(LS_EINVAL, "block must be 32 or 16, got %d", block);
    if (rows < 0 || K < 0 || K % 128 != 0) return fail(LS_EINVAL, "K must be a multiple of 128");
    int64_t nblocks = rows * (K / block);
    if (nblocks == 0) return LS_OK;
    if (!scale || !sf) return fail(LS_EINVAL, "null pointer");
    scales_to_sf_kernel<<<grid_for(nblocks, kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        scale, nblocks, uint32_t(K / block), sf, bad);
    LS_LAUNCH_CHECK("scales_to_sf");
    return LS_OK;
}

extern "C" int ls_round_e2m1(const float *q, int64_t n, int rounding, uint8_t *codes, void *stream)
{
    if (int rc = check_device()) return rc;
    if (n < 0) return fail(LS_EINVAL, "negative size");
    if (n == 0) return LS_OK;
    if (!q || !codes) return fail(LS_EINVAL, "null pointer");
    int grid = grid_for(n, kThreads);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (rounding == LS_ROUND_RNE) round_e2m1_kernel<true><<<grid, kThreads, 0, st>>>(q, n, codes);
    else round_e2m1_kernel<false><<<grid, kThreads, 0, st>>>(q, n, codes);
    LS_LAUNCH_CHECK("round_e2m1");
    return LS_OK;
}

namespace {
int quantize_t_impl(const void *x, int x_dtype, int64_t R, int64_t C, int rounding, uint8_t *packed, float *scale,
                    uint8_t *sf, uint8_t *row_packed, uint8_t *row_sf, void *stream, int act = 0)
{
    if (act != 0 && (act != 1 || x_dtype != LS_BF16)) return fail(LS_EINVAL, "activation %d needs bf16 input (0 none, 1 GELU)", act);
    if (int rc = check_device()) return rc;
    if (x_dtype != LS_F32 && x_dtype != LS_BF16) return fail(LS_EINVAL, "unsupported dtype %d", x_dtype);
    if (rounding != LS_ROUND_REF && rounding != LS_ROUND_RNE) return fail(LS_EINVAL, "bad rounding %d", rounding);
    if (R < 0 || C < 0 || R % 128 != 0) return fail(LS_EINVAL, "R=%lld must be a multiple of 128", (long long)R);
    if (R == 0 || C == 0) return LS_OK;
    if (!x || (!packed && !scale && !sf)) return fail(LS_EINVAL, "null pointer");
    if (!aligned16(x) || !aligned16(packed) || !aligned16(scale) || (reinterpret_cast<uintptr_t>(sf) & 3))
        return fail(LS_EALIGN, "x, packed and scale must be 16-byte aligned, sf 4-byte");
    if (C >= (int64_t(1) << 31) || R >= (int64_t(1) << 31)) return fail(LS_EINVAL, "shape too large");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool rne = rounding == LS_ROUND_RNE;
    {
        static bool attr_set[64] = {};                           // the kernels need 64 KB of dynamic shared memory
        int dev = 0;
        if (int rc = current_device(&dev)) return rc;
        std::lock_guard<std::mutex> lk(state_mutex());
        if (!attr_set[dev]) {
            LS_CUDA(cudaFuncSetAttribute(quantize_t_kernel<__nv_bfloat16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTSmem));
            LS_CUDA(cudaFuncSetAttribute(quantize_t_kernel<__nv_bfloat16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTSmem));
            LS_CUDA(cudaFuncSetAttribute(quantize_t_kernel<float, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTSmem));
            LS_CUDA(cudaFuncSetAttribute(quantize_t_kernel<float, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTSmem));
            LS_CUDA(cudaFuncSetAttribute(quantize_t_kernel<__nv_bfloat16, true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTSmem));
            LS_CUDA(cudaFuncSetAttribute(quantize_t_kernel<__nv_bfloat16, false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTSmem));
            attr_set[dev] = true;
        }
    }
    auto launch = [&](auto kernel, auto xp, int tile_cols) -> int {
        const int64_t tiles = ((C + tile_cols - 1) / tile_cols) * (R / kTR);
        const int64_t cap = int64_t(sm_count()) * 3;             // three resident CTAs per SM (64 KB each)
        kernel<<<unsigned(tiles < cap ? tiles : cap), kThreads, kTSmem, st>>>(xp, R, C, packed, scale, sf, row_packed, row_sf);
        return LS_OK;
    };
    int rc;
    if (x_dtype == LS_BF16) {
        auto xp = static_cast<const __nv_bfloat16 *>(x);
        if (act == 1)
            rc = rne ? launch(quantize_t_kernel<__nv_bfloat16, true, 1>, xp, kTRowBytes / 2)
                     : launch(quantize_t_kernel<__nv_bfloat16, false, 1>, xp, kTRowBytes / 2);
        else
            rc = rne ? launch(quantize_t_kernel<__nv_bfloat16, true>, xp, kTRowBytes / 2)
                     : launch(quantize_t_kernel<__nv_bfloat16, false>, xp, kTRowBytes / 2);
    } else {
        auto xp = static_cast<const float *>(x);
        rc = rne ? launch(quantize_t_kernel<float, true>, xp, kTRowBytes / 4)
                 : launch(quantize_t_kernel<float, false>, xp, kTRowBytes / 4);
    }
    if (rc) return rc;
    LS_LAUNCH_CHECK("quantize_mxfp4_t");
    return LS_OK;
}
}  // namespace

extern "C" int ls_quantize_mxfp4_t(const void *x, int x_dtype, int64_t R, int64_t C, int rounding,
                                   uint8_t *packed, float *scale, uint8_t *sf, void *stream)
{
    return quantize_t_impl(x, x_dtype, R, C, rounding, packed, scale, sf, nullptr, nullptr, stream);
}

extern "C" int ls_quantize_mxfp4_t_act(const void *x, int x_dtype, int64_t R, int64_t C, int rounding, int act,
                                       uint8_t *packed, float *scale, uint8_t *sf, void *stream)
{
    return quantize_t_impl(x, x_dtype, R, C, rounding, packed, scale, sf, nullptr, nullptr, stream, act);
}

static int quantize_both_impl(const void *x, int x_dtype, int64_t R, int64_t C, int rounding, int act,
                              uint8_t *row_packed, uint8_t *row_sf, uint8_t *t_packed, uint8_t *t_sf, void *stream)
{
    if (C % 128 != 0) return fail(LS_EINVAL, "C=%lld must be a multiple of 128", (long long)C);
    if (!row_packed || !row_sf || !t_packed || !t_sf) return fail(LS_EINVAL, "null output");
    if (!aligned16(row_packed)) return fail(LS_EALIGN, "row_packed must be 16-byte aligned");
    return quantize_t_impl(x, x_dtype, R, C, rounding, t_packed, nullptr, t_sf, row_packed, row_sf, stream, act);
}

extern "C" int ls_quantize_mxfp4_both(const void *x, int x_dtype, int64_t R, int64_t C, int rounding,
                                      uint8_t *row_packed, uint8_t *row_sf, uint8_t *t_packed, uint8_t *t_sf,
                                      void *stream)
{
    return quantize_both_impl(x, x_dtype, R, C, rounding, 0, row_packed, row_sf, t_packed, t_sf, stream);
}

extern "C" int ls_quantize_mxfp4_both_act(const void *x, int x_dtype, int64_t R, int64_t C, int rounding, int act,
                                          uint8_t *row_packed, uint8_t *row_sf, uint8_t *t_packed, uint8_t *t_sf,
                                          void *stream)
{
    return quantize_both_impl(x, x_dtype, R, C, rounding, act, row_packed, row_sf, t_packed, t_sf, stream);
}

// Block-scaled MXFP4 GEMM on the 5th-generation tensor cores:
//   C[b][M,N] = A[b][M,K] * W[N,K]^T,  b = 0 (single) or 0,1 (dual batch, one W)
// A and W are packed E2M1 (two codes per byte, K-contiguous) with one UE8M0
// scale per 32 elements, held in the 128-row x 4-block tile layout that
// tcgen05.cp moves into tensor memory.  Accumulation is fp32 in tensor memory;
// the epilogue rounds to bf16 (nearest even) or writes fp32.
//
// One persistent CTA per SM, three roles:
//   warp 0      TMA producer: operand tiles (128-byte swizzle) and scale tiles
//               into a ring of shared-memory stages
//   warp 1      MMA issuer: scale tiles shared -> tensor memory, then four
//               K=64 MMAs per stage; commits free the stage / publish the tile
//   warps 2-5   epilogue: tensor memory -> registers -> global (warps 2-9 in the
//               CTA-pair kernel)
// Two accumulator buffers alternate between tiles.  With 256-column tiles they
// overlap by 32 columns (2 x 256 + scales would not fit in 512 columns): the
// epilogue drains the shared columns first and only then lets the next tile's
// MMAs start.
#include <cuda.h>
#include <algorithm>
#include <atomic>
#include <cstdlib>

#include "common.cuh"
#include "ptx.cuh"

namespace ls {
namespace {

constexpr int BM = 128;            // rows of A per tile (= tensor-memory lanes)
constexpr int BKB = 128;           // bytes of K per stage row = 256 E2M1 = one swizzle row
constexpr int kGemmThreads = 192;      // single-CTA kernel: producer, MMA issuer, 4 epilogue warps
constexpr int kPairThreads = 320;      // CTA-pair kernel: producer, MMA issuer, 8 epilogue warps
constexpr int kTmemCols = 512;

// VS = elements per scale (32: MXFP4 as lockstep quantizes by default; 16: the block-16 form of
// quantize_mxfp4(x, 16), UE8M0 scales on kind::mxf4nvf4).  A scale tile holds 128 rows x 4
// scales, i.e. 4 * VS elements of K, so a block-16 stage carries twice the scale tiles.
template <int BN, int VS = 32>
struct Cfg {
    static constexpr int SFT = 32 / VS;                    // scale tiles per 128 elements of K: 1 or 2
    // Narrow tiles (64 columns) are for short-M products, which are weight streams: the
    // number of SMs that load and the bytes each keeps in flight matter, the tile shape does
    // not.  Their stages are small, so there are more of them.
    static constexpr int STAGES = BN == 256 ? 4 : BN == 128 ? 6 : 8;
    static constexpr int A_BYTES = BM * BKB;
    static constexpr int B_BYTES = BN * BKB;
    static constexpr int SFA_BYTES = 1024 * SFT;           // 128 rows x 8 (16) scales
    static constexpr int SFB_TILES = BN >= 128 ? BN / 128 : 1;   // 128-row scale tiles of W that a tile touches
    static constexpr int SFB_BYTES = SFB_TILES * 1024 * SFT;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
    static constexpr int OVL = BN == 256 ? 32 : 0;        // columns shared by the two accumulators
    static constexpr int ACC1 = BN - OVL;                 // first column of the second accumulator
    static constexpr int SFA_COL = 2 * BN - OVL;          // 8 (16) columns
    static constexpr int SFB_COL = SFA_COL + 8 * SFT;     // 8 (16) columns per 128 rows of W
    static_assert(SFB_COL + SFB_TILES * 8 * SFT <= kTmemCols, "tensor memory overflow");
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;
    static_assert(SMEM <= 227 * 1024, "shared memory overflow");
};

struct GemmParams {
    const uint8_t *sfa[2];
    const uint8_t *sfb;
    void *c[2];
    int M, N, K;
    int nbatch;
    int out_bf16;
    int *err;                      // device int, set non-zero when a wait ran out
    int splits;                    // split-K factor of the single-CTA kernel (1 = off)
    int kt_per_split;              // k-tiles per split
    float *partial;                // [splits, M, N] fp32 partial sums when splits > 1
    // fused quantizing epilogue (the consumer of C is another MXFP4 GEMM): MXFP4 of act(C)
    uint8_t *q_packed[2];          // [M, N/2] packed codes, or NULL
    uint8_t *q_sf[2];              // scale-factor bytes of a [M, N] operand
    int act;                       // 0 none, 1 GELU (erf form)
    int store_c;                   // 0: C itself is not written (only its quantized form)
    int a_box_bytes;               // bytes one TMA load of an A tile delivers (single-CTA kernel: rows of the box x 128)
    int sf_e4m3;                   // block-16 kernel only: the scale bytes are E4M3 (NVFP4), not UE8M0
};

// MXFP4 of one row's 32 consecutive outputs (exactly one scale block), as the next GEMM
// reads it.  The values quantized are the ones a separate pass would see: the
// accumulator rounded to the output type, the activation applied in fp32 and rounded
// to the output type again.
// What an epilogue thread needs from the kernel parameters, read once into registers.
// (Indexing the parameter arrays with a run-time batch index makes the compiler keep a
// copy of the whole parameter struct in local memory and read it back on every use.)
struct Epi {
    int M, N;
    bool out_bf16, store_c;
    int act;
    uint8_t *q_packed, *q_sf;      // of this thread's batch
};
__device__ __forceinline__ Epi make_epi(const GemmParams &p, int b)
{
    Epi e;
    e.M = p.M, e.N = p.N;
    e.out_bf16 = p.out_bf16 != 0, e.store_c = p.store_c != 0;
    e.act = p.act;
    e.q_packed = b ? p.q_packed[1] : p.q_packed[0];
    e.q_sf = b ? p.q_sf[1] : p.q_sf[0];
    return e;
}

__device__ __forceinline__ void quant_chunk(const Epi &p, int row, int col0, const uint32_t (&r)[32])
{
    if (row >= p.M || col0 >= p.N) return;
    float v[32];
    uint32_t amax = 0;
#pragma unroll
    for (int i = 0; i < 32; i++) {
        float x = __uint_as_float(r[i]);
        if (p.out_bf16) x = __bfloat162float(__float2bfloat16_rn(x));
        if (p.act == 1) {
            x = (x * 0.5f) * (1.0f + erff(x * 0.70710678118654752440f));
            if (p.out_bf16) x = __bfloat162float(__float2bfloat16_rn(x));
        }
        v[i] = x;
        amax = max(amax, __float_as_uint(x) & 0x7FFFFFFFu);
    }
    const uint32_t e8 = block_e8m0(amax);
    const float inv = __uint_as_float(e8 == 255u ? 0x7FC00000u : inv_scale_bits(e8));
    uint32_t pk[4];
#pragma unroll
    for (int h = 0; h < 4; h++) {
        float t[8];
#pragma unroll
        for (int i = 0; i < 8; i++) t[i] = v[8 * h + i] * inv;
        if (amax < kBitsInf) {
            pk[h] = cvt_ref_e2m1x8(t);
        } else {
            pk[h] = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) pk[h] |= e2m1_code<false>(t[i]) << (4 * i);
        }
    }
    *reinterpret_cast<uint4 *>(p.q_packed + int64_t(row) * (p.N / 2) + col0 / 2) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    p.q_sf[sf_offset(uint32_t(row), uint32_t(col0 / 32), uint32_t(p.N / 128))] = uint8_t(e8);
}

// 4 x 4 transpose of 16-byte items inside each group of four lanes: afterwards item k of
// lane 4g + j is what lane 4g + k held as item j.
__device__ __forceinline__ void transpose4(uint4 (&it)[4], int lane)
{
#pragma unroll
    for (int b = 0; b < 2; b++) {
        const bool up = (lane >> b) & 1;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            if (i & (1 << b)) continue;
            const int hi = i | (1 << b);
            uint4 send = up ? it[i] : it[hi], recv;
            recv.x = __shfl_xor_sync(0xFFFFFFFFu, send.x, 1 << b);
            recv.y = __shfl_xor_sync(0xFFFFFFFFu, send.y, 1 << b);
            recv.z = __shfl_xor_sync(0xFFFFFFFFu, send.z, 1 << b);
            recv.w = __shfl_xor_sync(0xFFFFFFFFu, send.w, 1 << b);
            if (up) it[i] = recv;
            else it[hi] = recv;
        }
    }
}

// Ragged edge of the output (N not a multiple of the vector width, or the last columns of
// a tile): element-wise stores from a private copy of the chunk.  Kept out of line, and fed
// from a copy, so that neither its loop nor its run-time index touches the epilogue's
// accumulator registers (a run-time index into them would move them to local memory) or
// its code size (a tile's epilogue runs once per tile; short tiles pay for every
// instruction fetched).
__device__ __noinline__ void store_tail_impl(void *dst, bool bf16, int n, const uint32_t *v)
{
    if (bf16)
        for (int j = 0; j < n; j++) static_cast<__nv_bfloat16 *>(dst)[j] = __float2bfloat16_rn(__uint_as_float(v[j]));
    else
        for (int j = 0; j < n; j++) static_cast<float *>(dst)[j] = __uint_as_float(v[j]);
}
__device__ __forceinline__ void store_tail(void *dst, bool bf16, int n, const uint32_t (&r)[32])
{
    uint32_t v[32];
#pragma unroll
    for (int j = 0; j < 32; j++) v[j] = r[j];
    store_tail_impl(dst, bf16, n, v);
}

// Stores one accumulator chunk: lane l of the warp holds the 32 consecutive outputs
// (columns col0 .. col0 + 31) of row row0 + l.  Called by the whole warp.  Storing each
// lane's own row would touch 32 rows per instruction (one 16-byte piece each); the
// pieces are transposed inside groups of four lanes first, so that four adjacent lanes
// write 64 contiguous bytes of one row and an instruction touches 8 rows.
__device__ __forceinline__ void store_chunk(const Epi &p, void *cbase, bool bf16, int row0, int lane, int col0,
                                            const uint32_t (&r)[32])
{
    if (row0 >= p.M || col0 >= p.N) return;                       // uniform over the warp
    const int row = row0 + lane;
    const int trow = row0 + (lane & ~3), tq = lane & 3;            // first row / piece of this lane after a transpose
    if (bf16) {
        __nv_bfloat16 *base = static_cast<__nv_bfloat16 *>(cbase);
        if (col0 + 32 <= p.N && (p.N & 7) == 0) {
            uint4 it[4];
#pragma unroll
            for (int v = 0; v < 4; v++) {
                uint32_t *ow = &it[v].x;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[8 * v + 2 * j]),
                                                             __uint_as_float(r[8 * v + 2 * j + 1]));
                    ow[j] = *reinterpret_cast<uint32_t *>(&h);
                }
            }
            transpose4(it, lane);
#pragma unroll
            for (int k = 0; k < 4; k++)
                if (trow + k < p.M)
                    *reinterpret_cast<uint4 *>(base + int64_t(trow + k) * p.N + col0 + 8 * tq) = it[k];
        } else if (row < p.M) {
            store_tail(base + int64_t(row) * p.N + col0, true, min(32, p.N - col0), r);
        }
    } else {
        float *base = static_cast<float *>(cbase);
        if (col0 + 32 <= p.N && (p.N & 3) == 0) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                uint4 it[4];
#pragma unroll
                for (int v = 0; v < 4; v++)
                    it[v] = make_uint4(r[16 * h + 4 * v], r[16 * h + 4 * v + 1], r[16 * h + 4 * v + 2], r[16 * h + 4 * v + 3]);
                transpose4(it, lane);
#pragma unroll
                for (int k = 0; k < 4; k++)
                    if (trow + k < p.M)
                        *reinterpret_cast<uint4 *>(base + int64_t(trow + k) * p.N + col0 + 16 * h + 4 * tq) = it[k];
            }
        } else if (row < p.M) {
            store_tail(base + int64_t(row) * p.N + col0, false, min(32, p.N - col0), r);
        }
    }
}

// One pipeline stage on the tensor pipe: scale tiles shared -> tensor memory, then the
// K = 64 MMAs.  ATOMS = number of 128-element k-tiles in the stage (2, or 1 at the K
// tail); everything else is a compile-time offset so that the issuing thread spends
// its time on the tcgen05 instructions, not on address arithmetic.
template <int CTAS, int ATOMS, int SFB_ATOMS>
__device__ __forceinline__ void issue_stage(uint32_t acc, uint64_t adesc, uint64_t bdesc, uint64_t sfa_desc,
                                            uint64_t sfb_desc, uint32_t sfa_t, uint32_t sfb_t, uint32_t idesc,
                                            bool first_of_tile, bool skip_cp, bool skip_mma, uint32_t sfb_sub = 0)
{
    constexpr int SFB_COLS = 4 * SFB_ATOMS;                 // columns per k-tile
    if (!skip_cp) {
#pragma unroll
        for (int j = 0; j < ATOMS; j++) {
            ptx::tmem_cp_sf<CTAS>(sfa_t + 4 * j, sfa_desc + 32 * j);
#pragma unroll
            for (int r = 0; r < SFB_ATOMS; r++)
                ptx::tmem_cp_sf<CTAS>(sfb_t + SFB_COLS * j + 4 * r, sfb_desc + 64 * r + 32 * j);
        }
    }
    if (!skip_mma) {
#pragma unroll
        for (int kb = 0; kb < 2 * ATOMS; kb++) {
            constexpr uint32_t kId[2] = {0u, 2u};           // byte of the scale column used by this MMA
            const uint32_t id = kId[kb & 1];
            ptx::mma_mxf4<CTAS>(acc, adesc + 2 * kb, bdesc + 2 * kb, idesc | (id << 29) | (id << 4),
                                sfa_t + 4 * (kb >> 1) + (id << 30), sfb_t + sfb_sub + SFB_COLS * (kb >> 1) + (id << 30),
                                (kb == 0 && first_of_tile) ? 0u : 1u);
        }
    }
}

// The same for block-16 scales: every K = 64 MMA has a scale tile of its own (4 scales per row).
template <int CTAS, int ATOMS, int SFB_ATOMS>
__device__ __forceinline__ void issue_stage16(uint32_t acc, uint64_t adesc, uint64_t bdesc, uint64_t sfa_desc,
                                              uint64_t sfb_desc, uint32_t sfa_t, uint32_t sfb_t, uint32_t idesc,
                                              bool first_of_tile, uint32_t sfb_sub)
{
    constexpr int T = 2 * ATOMS;                            // scale tiles = MMAs in this stage
    constexpr int SFB_COLS = 4 * SFB_ATOMS;                 // columns per scale tile index
#pragma unroll
    for (int j = 0; j < T; j++) {
        ptx::tmem_cp_sf<CTAS>(sfa_t + 4 * j, sfa_desc + 32 * j);
#pragma unroll
        for (int r = 0; r < SFB_ATOMS; r++)
            ptx::tmem_cp_sf<CTAS>(sfb_t + SFB_COLS * j + 4 * r, sfb_desc + 128 * r + 32 * j);
    }
#pragma unroll
    for (int kb = 0; kb < T; kb++)
        ptx::mma_mxf4_block16<CTAS>(acc, adesc + 2 * kb, bdesc + 2 * kb, idesc, sfa_t + 4 * kb, sfb_t + sfb_sub + SFB_COLS * kb,
                              (kb == 0 && first_of_tile) ? 0u : 1u);
}

template <int BN, int VS>
__global__ void __launch_bounds__(kGemmThreads, 1)
mxfp4_gemm_kernel(const __grid_constant__ CUtensorMap tm_a0, const __grid_constant__ CUtensorMap tm_a1,
                  const __grid_constant__ CUtensorMap tm_b, const GemmParams p)
{
    using C = Cfg<BN, VS>;
    constexpr int SFT = C::SFT;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + C::STAGES * C::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (C::STAGES + s); };
    const uint32_t acc_full_bar = bar_base + 8u * (2 * C::STAGES);
    const uint32_t acc_free_bar = acc_full_bar + 8u;
    const uint32_t tmem_slot = acc_free_bar + 8u;
    uint8_t *gen_base = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    volatile uint32_t *tmem_slot_p = reinterpret_cast<volatile uint32_t *>(gen_base + C::STAGES * C::STAGE_BYTES + 8 * (2 * C::STAGES + 2));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot_p + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
    const int total_tiles = m_tiles * n_tiles * p.nbatch * p.splits;
    const int k_tiles = (p.K / 2 + BKB - 1) / BKB;
    const int k_atoms = p.K / 128;                    // scale tiles (4 k-blocks each) per row tile
    const int n_atoms = (p.N + 127) / 128;            // 128-row scale tiles of W
    // tile index -> (split, batch, row tile, column tile); a split covers k-tiles [kt0, kt1)
    auto split_of = [&](int t) { return t % p.splits; };
    auto kt_begin = [&](int ks) { return ks * p.kt_per_split; };
    auto kt_end = [&](int ks) { return min(k_tiles, (ks + 1) * p.kt_per_split); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        ptx::mbar_init(acc_full_bar, 1);
        ptx::mbar_init(acc_free_bar, 4);
        *abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc<1>(tmem_slot, kTmemCols);
        ptx::tmem_relinquish<1>();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_p;
    // Programmatic dependent launch: this grid may have started while the kernel before it in
    // the stream was still running (its set-up above overlaps that kernel's tail), and the
    // kernel after it may start its own set-up now.  Nothing that depends on earlier kernels
    // has been touched so far; the producer waits for them before its first load, and every
    // store of this kernel follows from those loads.  (Both are no-ops in an ordinary launch.)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (ptx::elect_one()) {
            ptx::prefetch_tmap(&tm_a0);
            ptx::prefetch_tmap(&tm_a1);
            ptx::prefetch_tmap(&tm_b);
            asm volatile("griddepcontrol.wait;" ::: "memory");
            uint32_t it = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                const int ks = split_of(t), tt = t / p.splits;
                const int b = tt % p.nbatch, rest = tt / p.nbatch;
                const int mt = rest % m_tiles, nt = rest / m_tiles;
                const CUtensorMap *tma = b ? &tm_a1 : &tm_a0;
                const uint8_t *sfa = (b ? p.sfa[1] : p.sfa[0]) + int64_t(mt) * k_atoms * SFT * 512;
                for (int kt = kt_begin(ks); kt < kt_end(ks); kt++, it++) {
                    const int s = it % C::STAGES;
                    const uint32_t ph = (it / C::STAGES) & 1;
                    if (!(ok = ptx::mbar_wait(empty_bar(s), ph ^ 1, abort_flag))) break;
                    const int atoms = min(2, k_atoms - 2 * kt);           // scale tiles in this stage
                    const uint32_t sf_bytes = 512u * SFT * atoms;
                    const uint32_t st = smem_base + s * C::STAGE_BYTES;
                    // scale tiles of W rows past N do not exist; their products are never stored
                    const int sfb_tile0 = nt * BN / 128;                  // first 128-row scale tile of this column tile
                    const int b_atoms = min(C::SFB_TILES, n_atoms - sfb_tile0);
                    ptx::mbar_expect_tx(full_bar(s), uint32_t(p.a_box_bytes) + C::B_BYTES + sf_bytes * (1 + b_atoms));
                    ptx::tma_load_2d(st, tma, kt * BKB, mt * BM, full_bar(s));
                    ptx::tma_load_2d(st + C::A_BYTES, &tm_b, kt * BKB, nt * BN, full_bar(s));
                    ptx::bulk_load(st + C::A_BYTES + C::B_BYTES, sfa + int64_t(kt) * 1024 * SFT, sf_bytes, full_bar(s));
                    for (int r = 0; r < b_atoms; r++)
                        ptx::bulk_load(st + C::A_BYTES + C::B_BYTES + C::SFA_BYTES + r * 1024 * SFT,
                                       p.sfb + (int64_t(sfb_tile0 + r) * k_atoms + 2 * kt) * SFT * 512,
                                       sf_bytes, full_bar(s));
                }
            }
            // do not leave while the MMA side may still arrive on this CTA's barriers
            for (int i = 0; i < C::STAGES && ok; i++, it++)
                ok = ptx::mbar_wait(empty_bar(it % C::STAGES), ((it / C::STAGES) & 1) ^ 1, abort_flag);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        if (ptx::elect_one()) {
            // bit 23 of the instruction descriptor: scale type (1 = UE8M0, 0 = UE4M3)
            const uint32_t idesc = (VS == 16 && p.sf_e4m3) ? (ptx::idesc_mxf4(BM, BN) & ~(1u << 23)) : ptx::idesc_mxf4(BM, BN);
            const uint64_t adesc0 = ptx::desc_sw128(smem_base), bdesc0 = ptx::desc_sw128(smem_base + C::A_BYTES);
            const uint64_t sfadesc0 = ptx::desc_sf(smem_base + C::A_BYTES + C::B_BYTES);
            const uint64_t sfbdesc0 = ptx::desc_sf(smem_base + C::A_BYTES + C::B_BYTES + C::SFA_BYTES);
            uint32_t it = 0;
            int lt = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, lt++) {
                if (lt > 0 && !(ok = ptx::mbar_wait(acc_free_bar, (lt - 1) & 1, abort_flag))) break;
                ptx::tc_fence_after();
                const uint32_t acc = tmem_base + ((lt & 1) ? C::ACC1 : 0);
                const int kt0 = kt_begin(split_of(t)), kt1 = kt_end(split_of(t));
                // A 64-column tile uses one half of a 128-row scale tile of W: the rows 32 c .. 32 c + 31
                // of a scale tile sit in column c of its group of four, so the second half starts at
                // column 2.
                const int nt_of = (t / p.splits) / p.nbatch / m_tiles;
                const uint32_t sfb_sub = BN >= 128 ? 0u : uint32_t((nt_of * BN) % 128) / 32u;
                for (int kt = kt0; kt < kt1; kt++, it++) {
                    const int s = it % C::STAGES;
                    const uint32_t ph = (it / C::STAGES) & 1;
                    if (!(ok = ptx::mbar_wait(full_bar(s), ph, abort_flag))) break;
                    ptx::tc_fence_after();
                    const uint32_t st16 = uint32_t(s) * (C::STAGE_BYTES >> 4);       // stage offset in 16-byte units
                    if constexpr (VS == 32) {
                        if (2 * kt + 2 <= k_atoms)
                            issue_stage<1, 2, C::SFB_TILES>(acc, adesc0 + st16, bdesc0 + st16, sfadesc0 + st16, sfbdesc0 + st16,
                                                            tmem_base + C::SFA_COL, tmem_base + C::SFB_COL, idesc, kt == kt0, false, false, sfb_sub);
                        else
                            issue_stage<1, 1, C::SFB_TILES>(acc, adesc0 + st16, bdesc0 + st16, sfadesc0 + st16, sfbdesc0 + st16,
                                                            tmem_base + C::SFA_COL, tmem_base + C::SFB_COL, idesc, kt == kt0, false, false, sfb_sub);
                    } else {
                        if (2 * kt + 2 <= k_atoms)
                            issue_stage16<1, 2, C::SFB_TILES>(acc, adesc0 + st16, bdesc0 + st16, sfadesc0 + st16, sfbdesc0 + st16,
                                                           tmem_base + C::SFA_COL, tmem_base + C::SFB_COL, idesc, kt == kt0, sfb_sub);
                        else
                            issue_stage16<1, 1, C::SFB_TILES>(acc, adesc0 + st16, bdesc0 + st16, sfadesc0 + st16, sfbdesc0 + st16,
                                                           tmem_base + C::SFA_COL, tmem_base + C::SFB_COL, idesc, kt == kt0, sfb_sub);
                    }
                    ptx::tc_commit(empty_bar(s));
                }
                if (ok) ptx::tc_commit(acc_full_bar);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const int q = warp & 3;                        // tensor-memory lane quarter of this warp
        const int splits = p.splits;
        int lt = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, lt++) {
            const int ks = split_of(t), tt = t / p.splits;
            const int b = tt % p.nbatch, rest = tt / p.nbatch;
            const int mt = rest % m_tiles, nt = rest / m_tiles;
            // split-K: fp32 partial sums into the scratch slab of (batch, split)
            const Epi ep = make_epi(p, b);
            void *dst = p.splits > 1 ? static_cast<void *>(p.partial + int64_t(b * p.splits + ks) * p.M * p.N)
                                     : (b ? p.c[1] : p.c[0]);
            const bool dst_bf16 = p.splits > 1 ? false : ep.out_bf16;
            if (!(ok = ptx::mbar_wait(acc_full_bar, lt & 1, abort_flag))) break;
            ptx::tc_fence_after();
            const uint32_t acc = tmem_base + ((lt & 1) ? C::ACC1 : 0) + (uint32_t(32 * q) << 16);
            const int row = mt * BM + 32 * q + lane;
            constexpr int CH = BN / 32;
            // first chunk: the columns shared with the other accumulator
            const int first = (C::OVL && !(lt & 1)) ? CH - 1 : 0;
            // two register sets: the load of the next chunk is in flight while this one is stored
            auto emit = [&](int c, const uint32_t (&r)[32]) {
                if (ep.store_c || splits > 1) store_chunk(ep, dst, dst_bf16, row - lane, lane, nt * BN + 32 * c, r);
                if (ep.q_packed) quant_chunk(ep, row, nt * BN + 32 * c, r);
            };
            uint32_t ra[32], rb[32];
            ptx::tmem_ld32(acc + 32 * first, ra);
#pragma unroll 1                                    // code size: the body already holds two chunks
            for (int i = 0; i < CH; i += 2) {
                ptx::tmem_ld_wait(ra);
                if (i + 1 < CH) ptx::tmem_ld32(acc + 32 * ((first + i + 1) % CH), rb);
                if (i == 0) {                               // first chunk drained: the next tile may start
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(acc_free_bar);
                }
                emit((first + i) % CH, ra);
                if (i + 1 < CH) {
                    ptx::tmem_ld_wait(rb);
                    if (i + 2 < CH) ptx::tmem_ld32(acc + 32 * ((first + i + 2) % CH), ra);
                    emit((first + i + 1) % CH, rb);
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    if (*abort_flag) {
        // give copies and MMAs still in flight time to land before memory is released
        for (int i = 0; i < 4096; i++) __nanosleep(256);
        if (threadIdx.x == 0) atomicExch(p.err, 1);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc<1>(tmem_base, kTmemCols);
    }
}

// Sums the split-K partial slabs in ascending split order and writes the output type.
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float *__restrict__ partial, void *__restrict__ out, int64_t mn, int splits, int out_bf16)
{
    const int64_t stride = int64_t(gridDim.x) * 256;
    const bool vec = (mn & 3) == 0;
    if (vec) {
        for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < mn / 4; i += stride) {
            float4 acc = reinterpret_cast<const float4 *>(partial)[i];
            for (int s = 1; s < splits; s++) {
                const float4 v = reinterpret_cast<const float4 *>(partial + int64_t(s) * mn)[i];
                acc.x += v.x, acc.y += v.y, acc.z += v.z, acc.w += v.w;
            }
            if (out_bf16) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
                reinterpret_cast<uint2 *>(out)[i] = make_uint2(*reinterpret_cast<uint32_t *>(&lo), *reinterpret_cast<uint32_t *>(&hi));
            } else {
                reinterpret_cast<float4 *>(out)[i] = acc;
            }
        }
    } else {
        for (int64_t i = int64_t(blockIdx.x) * 256 + threadIdx.x; i < mn; i += stride) {
            float acc = partial[i];
            for (int s = 1; s < splits; s++) acc += partial[int64_t(s) * mn + i];
            if (out_bf16) static_cast<__nv_bfloat16 *>(out)[i] = __float2bfloat16_rn(acc);
            else static_cast<float *>(out)[i] = acc;
        }
    }
}

// ---- CTA-pair kernel ---------------------------------------------------------------
// Two CTAs of a cluster work on one 256 x 256 tile with cta_group::2 MMAs: each
// CTA stages its own 128 rows of A and its own 128 rows (half) of the W tile,
// the tensor cores of both SMs read both halves of W, and each CTA's tensor
// memory receives the accumulator of its own 128 rows.  Per SM this halves the
// shared-memory traffic of the W operand and makes room for six stages.
// Dual batch: CTA 0 takes batch 0's row tile, CTA 1 batch 1's, against the same
// W tile -- the two activation batches share one weight stream inside the MMA.
// Single batch: the pair takes two consecutive row tiles.
//
// Roles per CTA: warp 0 lane: TMA producer for this CTA's stage halves (every
// load of either CTA completes on CTA 0's barrier).  Warp 1 lane of CTA 0: the
// MMA issuer for the pair (warp 1 of CTA 1 only takes part in the tensor-memory
// allocation).  Warps 2-9: epilogue, two warps per quarter of the rows.
template <int VS, int BNP = 256>
struct PairCfg {
    static constexpr int SFT = 32 / VS;                    // scale tiles per 128 elements of K
    static constexpr int BN = BNP;                         // tile columns (BN / 2 rows of W per CTA): 256 or 192
    static_assert(BN == 256 || BN == 192, "tile widths: 256 or 192");
    static constexpr int A_BYTES = BM * BKB;               // 16 KB
    static constexpr int B_BYTES = (BN / 2) * BKB;         // this CTA's half of the W tile
    static constexpr int SFA_BYTES = 1024 * SFT;
    static constexpr int SFB_BYTES = 2048 * SFT;           // scales of the two 128-row scale tiles the W tile touches, in both CTAs
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
    static constexpr int STAGES = (227 * 1024 - 1024 - 256) / STAGE_BYTES;    // 6 (5 with scales per 16); 7 (6) at 192 columns
    // Tensor memory, 256-column tiles: accumulators [0,256) and [224,480) share 32 columns; scale
    // columns at 480 (8 for A, 16 for W).  A second set of scale columns (tried with a 64-column
    // overlap) did not speed the kernel up.  Scales per 16 elements take 48 columns: the
    // accumulators then share 64 columns, [0,256) and [192,448).
    // 192-column tiles: [0,192) and [192,384) share nothing, and the MMAs of a tile can start
    // while the tile before it is still being read out.
    static constexpr int OVL = BN == 192 ? 0 : VS == 32 ? 32 : 64;
    static constexpr int ACC1 = BN - OVL;                  // 224 (192)
    static constexpr int SF_COL = 2 * BN - OVL;            // 480 (448, 384)
    static_assert(SF_COL + 24 * SFT <= kTmemCols, "tensor memory overflow");
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 256;
    static_assert(SMEM <= 227 * 1024, "shared memory overflow");
};

__device__ __forceinline__ void cluster_sync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

template <int VS, int BNP>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
mxfp4_gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a0, const __grid_constant__ CUtensorMap tm_a1,
                       const __grid_constant__ CUtensorMap tm_b, const __grid_constant__ CUtensorMap tm_sfa0,
                       const __grid_constant__ CUtensorMap tm_sfa1, const __grid_constant__ CUtensorMap tm_sfb,
                       const GemmParams p)
{
    using C = PairCfg<VS, BNP>;
    constexpr int SFT = C::SFT;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bar_base = smem_base + C::STAGES * C::STAGE_BYTES;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (C::STAGES + s); };
    const uint32_t acc_full_bar = bar_base + 8u * (2 * C::STAGES);
    const uint32_t acc_free_bar = acc_full_bar + 8u;                                    // used in CTA 0; a second one follows it
    const uint32_t tmem_slot = acc_free_bar + 16u;
    uint8_t *gen_base = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    volatile uint32_t *tmem_slot_p =
        reinterpret_cast<volatile uint32_t *>(gen_base + C::STAGES * C::STAGE_BYTES + 8 * (2 * C::STAGES + 3));
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot_p + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = cluster_ctarank();                 // 0 = leader
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + C::BN - 1) / C::BN;
    const int mp_tiles = p.nbatch == 2 ? m_tiles : (m_tiles + 1) / 2;   // row-tile pairs
    const int total = mp_tiles * n_tiles * p.splits;       // work items: (pair tile, K split)
    const int k_tiles = (p.K / 2 + BKB - 1) / BKB;
    const int k_atoms = p.K / 128;
    auto kt_begin = [&](int t) { return (t % p.splits) * p.kt_per_split; };
    auto kt_end = [&](int t) { return min(k_tiles, (t % p.splits + 1) * p.kt_per_split); };
    // this CTA's batch and row tile inside pair-tile index mp
    const int my_batch = p.nbatch == 2 ? int(cta) : 0;
    auto my_mtile = [&](int mp) { return p.nbatch == 2 ? mp : 2 * mp + int(cta); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; s++) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        ptx::mbar_init(acc_full_bar, 1);
        ptx::mbar_init(acc_free_bar, 16);                   // 8 epilogue warps of each CTA
        ptx::mbar_init(acc_free_bar + 8u, 16);              // accumulators that share nothing: one barrier each
        *abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc<2>(tmem_slot, kTmemCols);
        ptx::tmem_relinquish<2>();
    }
    ptx::tc_fence_before();
    __syncthreads();
    cluster_sync();                                         // both CTAs' barriers exist before any remote arrive
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_p;
    // programmatic dependent launch, as in the single-CTA kernel: the set-up above may have
    // overlapped the tail of the kernel before this one (typically the quantizer of A)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        // ------------------------------------------------------------ producer (both CTAs)
        // Every load of either CTA completes on CTA 0's "full" barrier of the stage: the
        // MMA thread there waits once for both halves.  All boxes have a fixed size
        // (rows or scale tiles outside the tensors are zero-filled), so the byte count
        // per stage is constant.
        if (ptx::elect_one()) {
            const CUtensorMap *tma = my_batch ? &tm_a1 : &tm_a0;
            const CUtensorMap *tsfa = my_batch ? &tm_sfa1 : &tm_sfa0;
            ptx::prefetch_tmap(tma);
            ptx::prefetch_tmap(&tm_b);
            ptx::prefetch_tmap(tsfa);
            ptx::prefetch_tmap(&tm_sfb);
            asm volatile("griddepcontrol.wait;" ::: "memory");
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = pair; t < total && ok; t += npairs) {
                const int tt = t / p.splits;
                const int mp = tt % mp_tiles, nt = tt / mp_tiles;
                const int mt = my_mtile(mp);
                for (int kt = kt_begin(t), kte = kt_end(t); kt < kte; kt++) {
                    if (!(ok = ptx::mbar_wait(empty_bar(s), ph ^ 1, abort_flag))) break;
                    const uint32_t st = smem_base + s * C::STAGE_BYTES;
                    const uint32_t bar = ptx::map_to_cta(full_bar(s), 0);
                    if (cta == 0) ptx::mbar_expect_tx(full_bar(s), 2 * C::STAGE_BYTES);
                    ptx::tma_load_2d_pair(st, tma, kt * BKB, mt * BM, bar);
                    ptx::tma_load_2d_pair(st + C::A_BYTES, &tm_b, kt * BKB, nt * C::BN + int(cta) * (C::BN / 2), bar);
                    ptx::tma_load_2d_pair(st + C::A_BYTES + C::B_BYTES, tsfa, 0, (mt * k_atoms + 2 * kt) * SFT, bar);
                    const int sfb_tile0 = nt * C::BN / 128;       // first of the two 128-row scale tiles of W under this tile
                    ptx::tma_load_2d_pair(st + C::A_BYTES + C::B_BYTES + C::SFA_BYTES, &tm_sfb, 0,
                                          (sfb_tile0 * k_atoms + 2 * kt) * SFT, bar);
                    ptx::tma_load_2d_pair(st + C::A_BYTES + C::B_BYTES + C::SFA_BYTES + 1024 * SFT, &tm_sfb, 0,
                                          ((sfb_tile0 + 1) * k_atoms + 2 * kt) * SFT, bar);
                    if (++s == C::STAGES) s = 0, ph ^= 1;
                }
            }
            for (int i = 0; i < C::STAGES && ok; i++) {     // wait until the MMA side is done with every stage
                ok = ptx::mbar_wait(empty_bar(s), ph ^ 1, abort_flag);
                if (++s == C::STAGES) s = 0, ph ^= 1;
            }
        }
    } else if (warp == 1 && cta == 0) {
        // ------------------------------------------------------------ MMA issuer (CTA 0, for the pair)
        if (ptx::elect_one()) {
            const uint32_t idesc = (VS == 16 && p.sf_e4m3) ? (ptx::idesc_mxf4(256, C::BN) & ~(1u << 23)) : ptx::idesc_mxf4(256, C::BN);
            const uint64_t adesc0 = ptx::desc_sw128(smem_base), bdesc0 = ptx::desc_sw128(smem_base + C::A_BYTES);
            const uint64_t sfadesc0 = ptx::desc_sf(smem_base + C::A_BYTES + C::B_BYTES);
            const uint64_t sfbdesc0 = ptx::desc_sf(smem_base + C::A_BYTES + C::B_BYTES + C::SFA_BYTES);
            int s = 0, lt = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int t = pair; t < total && ok; t += npairs, lt++) {
                if (C::OVL > 0) {
                    // the tile before this one has been read out of the columns the two accumulators share
                    if (lt > 0 && !(ok = ptx::mbar_wait(acc_free_bar, (lt - 1) & 1, abort_flag))) break;
                } else {
                    // this accumulator's previous tile (two tiles back) has been read out
                    if (lt > 1 && !(ok = ptx::mbar_wait(acc_free_bar + 8u * (lt & 1), ((lt >> 1) - 1) & 1, abort_flag))) break;
                }
                ptx::tc_fence_after();
                const uint32_t acc = tmem_base + ((lt & 1) ? C::ACC1 : 0);
                const int kt0 = kt_begin(t), kt1 = kt_end(t);
                // a 192-column tile starts at row 0 or 64 of its first scale tile of W: scale column 0 or 2
                const uint32_t sfb_sub = uint32_t(((t / p.splits) / mp_tiles) * C::BN % 128) / 32u;
                for (int kt = kt0; kt < kt1; kt++) {
                    if (!(ok = ptx::mbar_wait(full_bar(s), ph, abort_flag))) break;
                    ptx::tc_fence_after();
                    const uint32_t st16 = uint32_t(s) * (C::STAGE_BYTES >> 4);
                    const uint32_t sfa_t = tmem_base + C::SF_COL, sfb_t = sfa_t + 8 * SFT;
                    if constexpr (VS == 32) {
                        if (2 * kt + 2 <= k_atoms)
                            issue_stage<2, 2, 2>(acc, adesc0 + st16, bdesc0 + st16, sfadesc0 + st16, sfbdesc0 + st16, sfa_t,
                                                 sfb_t, idesc, kt == kt0, false, false, sfb_sub);
                        else
                            issue_stage<2, 1, 2>(acc, adesc0 + st16, bdesc0 + st16, sfadesc0 + st16, sfbdesc0 + st16, sfa_t,
                                                 sfb_t, idesc, kt == kt0, false, false, sfb_sub);
                    } else {
                        if (2 * kt + 2 <= k_atoms)
                            issue_stage16<2, 2, 2>(acc, adesc0 + st16, bdesc0 + st16, sfadesc0 + st16, sfbdesc0 + st16, sfa_t,
                                                   sfb_t, idesc, kt == kt0, sfb_sub);
                        else
                            issue_stage16<2, 1, 2>(acc, adesc0 + st16, bdesc0 + st16, sfadesc0 + st16, sfbdesc0 + st16, sfa_t,
                                                   sfb_t, idesc, kt == kt0, sfb_sub);
                    }
                    ptx::tc_commit_pair(empty_bar(s), 3);      // frees the stage in both CTAs
                    if (++s == C::STAGES) s = 0, ph ^= 1;
                }
                if (ok) ptx::tc_commit_pair(acc_full_bar, 3);  // publishes the tile to both epilogues
            }
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogue (both CTAs)
        // Eight warps: warp w reads the tensor-memory lanes of quarter w % 4 (the hardware
        // ties a warp to that quarter) and one half of the tile's columns, four chunks of
        // 32.  The stores of a 128 x 256 tile keep one warp busy for longer than a short-K
        // tile takes on the tensor cores, so two warps share each row quarter.
        const int q = warp & 3, half = (warp - 2) >> 2;
        const Epi ep = make_epi(p, my_batch);
        const int splits = p.splits;
        int lt = 0;
        bool ok = true;
        for (int t = pair; t < total && ok; t += npairs, lt++) {
            const int ks = t % splits, tt = t / splits;
            const int mp = tt % mp_tiles, nt = tt / mp_tiles;
            const int mt = my_mtile(mp);
            // split-K: fp32 partial sums into the scratch slab of (batch, split)
            void *dst = splits > 1 ? static_cast<void *>(p.partial + int64_t(my_batch * splits + ks) * ep.M * ep.N)
                                   : (my_batch ? p.c[1] : p.c[0]);
            const bool dst_bf16 = splits > 1 ? false : ep.out_bf16;
            constexpr int CH = C::BN / 32 / 2;              // chunks per warp: 4 or 3
            constexpr int SH = C::OVL / 32;                 // chunks shared with the other accumulator: 0, 1 or 2
            static_assert(SH == 0 || CH == 4, "the drain order below reads the shared chunks as the first pair of four");
            auto release_next_tile = [&]() {
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_cluster(acc_free_bar, 0);
            };
            // Accumulators that share nothing: a warp frees this tile's accumulator (one barrier per
            // accumulator, so that a fast warp's arrival cannot be counted for the other one) as soon
            // as its last load of the tile has landed in registers.
            auto release_accumulator = [&]() {
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_cluster(acc_free_bar + 8u * (lt & 1), 0);
            };
            if (!(ok = ptx::mbar_wait(acc_full_bar, lt & 1, abort_flag))) break;
            ptx::tc_fence_after();
            const uint32_t acc = tmem_base + ((lt & 1) ? C::ACC1 : 0) + (uint32_t(32 * q) << 16);
            const int row = mt * BM + 32 * q + lane;
            // The columns shared with the other accumulator are the last chunk(s) of accumulator 0
            // and the first of accumulator 1.  The warps that own them read them first and
            // then release the next tile; the other warps release it at once: being here,
            // they have finished every load of the tiles before this one.
            const bool owner = SH > 0 && ((lt & 1) ? half == 0 : half == 1);
            const int start = (owner && !(lt & 1)) ? CH - SH : 0;
            auto chunk = [&](int i) { return CH * half + (SH > 0 ? ((start + i) & (CH - 1)) : i); };
            if (SH > 0 && !owner) release_next_tile();
            auto emit = [&](int c, const uint32_t (&r)[32]) {
                if (ep.store_c || splits > 1) store_chunk(ep, dst, dst_bf16, row - lane, lane, nt * C::BN + 32 * c, r);
                if (ep.q_packed) quant_chunk(ep, row, nt * C::BN + 32 * c, r);
            };
            // two register sets: the load of the next chunk is in flight while this one is stored
            uint32_t ra[32], rb[32];
            ptx::tmem_ld32(acc + 32 * chunk(0), ra);
#pragma unroll 1                                    // code size: the body already holds two chunks
            for (int i = 0; i < CH; i += 2) {
                ptx::tmem_ld_wait(ra);
                if (i + 1 < CH) ptx::tmem_ld32(acc + 32 * chunk(i + 1), rb);
                else if (SH == 0) release_accumulator();    // the last chunk is in registers
                if (SH == 2 && i == 0 && owner) ptx::tmem_ld_wait(rb);
                if (i == 0 && owner) release_next_tile();   // shared columns drained
                emit(chunk(i), ra);
                if (i + 1 < CH) {
                    ptx::tmem_ld_wait(rb);
                    if (i + 2 < CH) ptx::tmem_ld32(acc + 32 * chunk(i + 2), ra);
                    else if (SH == 0) release_accumulator();
                    emit(chunk(i + 1), rb);
                }
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    if (*abort_flag) {
        for (int i = 0; i < 4096; i++) __nanosleep(256);
        if (threadIdx.x == 0) atomicExch(p.err, 1);
    }
    ptx::tc_fence_before();
    __syncthreads();
    cluster_sync();                                         // neither CTA leaves while the other may still signal it
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc<2>(tmem_base, kTmemCols);
    }
}

// ---- host ---------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                              const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is a driver entry point and wants a current context.  A host thread
// that has only made calls that do not need one (cudaGetDevice) has none bound yet, and the
// encode fails with CUDA_ERROR_INVALID_CONTEXT; cudaSetDevice binds the device's primary
// context to the calling thread.  Once per thread.
void bind_primary_context()
{
    static thread_local bool bound = false;
    if (bound) return;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess) bound = true;
}

EncodeFn encode_fn()
{
    bind_primary_context();
    static EncodeFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

int encode_operand_map(CUtensorMap *m, const void *base, int64_t rows, int64_t kbytes, int box_rows)
{
    EncodeFn fn = encode_fn();
    if (!fn) return fail(LS_ECUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {cuuint64_t(kbytes), cuuint64_t(rows)};
    cuuint64_t strides[1] = {cuuint64_t(kbytes)};
    cuuint32_t box[2] = {cuuint32_t(BKB), cuuint32_t(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LS_ECUDA, "cuTensorMapEncodeTiled failed with %d", int(r));
    return LS_OK;
}

// Encoded tensor maps are pure functions of (base, shape, box): a small per-thread,
// direct-mapped cache keeps the last ones, so that a layer called every step with the
// same buffers (weights, a caching allocator's recycled activations) does not pay the
// driver's encoding on every launch.  kind 0: operand map, 1: scale-factor map.
struct MapKey {
    const void *base;
    int64_t rows, inner;
    int box_rows, kind;
    bool operator==(const MapKey &o) const
    {
        return base == o.base && rows == o.rows && inner == o.inner && box_rows == o.box_rows && kind == o.kind;
    }
};
struct MapSlot { MapKey key; CUtensorMap map; bool used; };
constexpr int kMapSlots = 256;
MapSlot *map_slot(const MapKey &k)
{
    static thread_local MapSlot slots[kMapSlots] = {};
    uint64_t h = reinterpret_cast<uintptr_t>(k.base) >> 4;
    h ^= uint64_t(k.rows) * 0x9E3779B97F4A7C15ull + uint64_t(k.inner) * 0xC2B2AE3D27D4EB4Full + uint64_t(k.box_rows) * 31 + uint64_t(k.kind);
    h ^= h >> 29;
    return &slots[h % kMapSlots];
}

// [rows, kbytes] bytes, K-contiguous; box = 128 bytes x box_rows, 128-byte swizzle
int make_operand_map(CUtensorMap *m, const void *base, int64_t rows, int64_t kbytes, int box_rows)
{
    const MapKey key{base, rows, kbytes, box_rows, 0};
    MapSlot *slot = map_slot(key);
    if (slot->used && slot->key == key) {
        *m = slot->map;
        return LS_OK;
    }
    if (int rc = encode_operand_map(m, base, rows, kbytes, box_rows)) return rc;
    slot->key = key, slot->map = *m, slot->used = true;
    return LS_OK;
}

std::atomic<int> g_gemm_pdl{1};       // 1: the GEMM kernels are launched with programmatic stream serialization

template <int BN, int VS = 32>
int launch(const CUtensorMap &ta0, const CUtensorMap &ta1, const CUtensorMap &tb, const GemmParams &p,
           cudaStream_t st)
{
    using C = Cfg<BN, VS>;
    static bool attr_set[64] = {};
    int dev = 0;
    if (int rc = current_device(&dev)) return rc;
    {
        std::lock_guard<std::mutex> lk(state_mutex());
        if (!attr_set[dev]) {
            LS_CUDA(cudaFuncSetAttribute(mxfp4_gemm_kernel<BN, VS>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
            attr_set[dev] = true;
        }
    }
    int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * p.nbatch * p.splits;
    int grid = tiles < sm_count() ? tiles : sm_count();
    // launched with programmatic stream serialization: see the note in the kernel
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(grid), 1, 1);
    cfg.blockDim = dim3(kGemmThreads, 1, 1);
    cfg.dynamicSmemBytes = C::SMEM;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = g_gemm_pdl.load(std::memory_order_relaxed) ? 1 : 0;
    cfg.attrs = at, cfg.numAttrs = 1;
    LS_CUDA(cudaLaunchKernelEx(&cfg, mxfp4_gemm_kernel<BN, VS>, ta0, ta1, tb, p));
    return LS_OK;
}

// Scale-factor buffer as [tiles, 128] 32-bit words (512 bytes per 128-row x 4-block tile);
// one box = two consecutive k-tiles of one row tile.
int make_sf_map(CUtensorMap *m, const void *base, int64_t rows, int64_t K, int sft)
{
    const MapKey key{base, rows, K, 2 * sft, 1};
    MapSlot *slot = map_slot(key);
    if (slot->used && slot->key == key) {
        *m = slot->map;
        return LS_OK;
    }
    EncodeFn fn = encode_fn();
    if (!fn) return fail(LS_ECUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {128, cuuint64_t(((rows + 127) / 128) * (K / 128) * sft)};
    cuuint64_t strides[1] = {512};
    cuuint32_t box[2] = {128, cuuint32_t(2 * sft)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(LS_ECUDA, "cuTensorMapEncodeTiled (scales) failed with %d", int(r));
    slot->key = key, slot->map = *m, slot->used = true;
    return LS_OK;
}

template <int VS = 32, int BNP = 256>
int launch_pair(const CUtensorMap &ta0, const CUtensorMap &ta1, const CUtensorMap &tb, const GemmParams &p,
                cudaStream_t st)
{
    using C = PairCfg<VS, BNP>;
    CUtensorMap tsa0, tsa1, tsb;
    if (int rc = make_sf_map(&tsa0, p.sfa[0], p.M, p.K, C::SFT)) return rc;
    if (int rc = make_sf_map(&tsa1, p.sfa[1], p.M, p.K, C::SFT)) return rc;
    if (int rc = make_sf_map(&tsb, p.sfb, p.N, p.K, C::SFT)) return rc;
    static int resident_pairs[64] = {};
    int dev = 0;
    if (int rc = current_device(&dev)) return rc;
    std::unique_lock<std::mutex> lk(state_mutex());
    if (!resident_pairs[dev]) {
        LS_CUDA(cudaFuncSetAttribute(mxfp4_gemm_pair_kernel<VS, BNP>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM));
        // The kernel is persistent: the grid must not exceed the CTA pairs that can be
        // resident at once (fewer than SMs / 2 when a TPC has a single SM enabled).
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(unsigned(sm_count() & ~1), 1, 1);
        cfg.blockDim = dim3(kPairThreads, 1, 1);
        cfg.dynamicSmemBytes = C::SMEM;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2, at[0].val.clusterDim.y = 1, at[0].val.clusterDim.z = 1;
        cfg.attrs = at, cfg.numAttrs = 1;
        int n = 0;
        LS_CUDA(cudaOccupancyMaxActiveClusters(&n, mxfp4_gemm_pair_kernel<VS, BNP>, &cfg));
        if (n < 1) return fail(LS_ECUDA, "no CTA pair of the GEMM kernel fits on this device");
        resident_pairs[dev] = n;
    }
    const int max_pairs = resident_pairs[dev];
    lk.unlock();
    int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + C::BN - 1) / C::BN;
    int pairs = (p.nbatch == 2 ? m_tiles : (m_tiles + 1) / 2) * n_tiles * p.splits;
    int grid = 2 * (pairs < max_pairs ? pairs : max_pairs);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(grid), 1, 1);
    cfg.blockDim = dim3(kPairThreads, 1, 1);
    cfg.dynamicSmemBytes = C::SMEM;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = g_gemm_pdl.load(std::memory_order_relaxed) ? 1 : 0;
    cfg.attrs = at, cfg.numAttrs = 1;
    LS_CUDA(cudaLaunchKernelEx(&cfg, mxfp4_gemm_pair_kernel<VS, BNP>, ta0, ta1, tb, tsa0, tsa1, tsb, p));
    return LS_OK;
}

std::atomic<int> g_gemm_variant{0};   // 0 = choose by shape, 1 = single-CTA kernel (256-column tiles), 2 = CTA-pair kernel,
                                      // 3 / 5 = single-CTA kernel with 128- / 64-column tiles, 6 = CTA-pair kernel with 192-column tiles
std::atomic<int> g_gemm_splits{0};    // 0 = choose by shape, n = split K n ways where splitting is allowed

// Per-device scratch for split-K partial sums, shared by every K-split GEMM of the device.
// Two such GEMMs on different streams are ordered by an event: the later one waits for the
// earlier one's summation kernel before its own partial sums may overwrite the slabs.  A
// request larger than the buffer gets a new, larger buffer; the old one may still be in use
// by a launch in flight, so it is kept until the process ends (a handful of doublings at most).
struct SplitScratch {
    float *buf = nullptr;
    size_t cap = 0;
    cudaEvent_t last_use = nullptr;     // recorded after the summation kernel of the last K-split GEMM
    cudaStream_t last_stream = nullptr;
    bool used = false;
};
SplitScratch g_split[64];

// Returns the scratch (>= bytes) after making `st` wait for the previous user on another stream.
float *splitk_acquire(size_t bytes, cudaStream_t st)
{
    int dev = 0;
    if (current_device(&dev)) return nullptr;
    std::lock_guard<std::mutex> lk(state_mutex());
    SplitScratch &sc = g_split[dev];
    if (!sc.last_use && cudaEventCreateWithFlags(&sc.last_use, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    if (sc.cap < bytes) {
        size_t want = bytes < (size_t(32) << 20) ? (size_t(32) << 20) : bytes;
        float *fresh = nullptr;
        if (cudaMalloc(&fresh, want) != cudaSuccess) return nullptr;
        sc.buf = fresh, sc.cap = want, sc.used = false;            // the old buffer stays allocated
    }
    if (sc.used && sc.last_stream != st && cudaStreamWaitEvent(st, sc.last_use, 0) != cudaSuccess) return nullptr;
    return sc.buf;
}
void splitk_release(cudaStream_t st)
{
    int dev = 0;
    if (current_device(&dev)) return;
    std::lock_guard<std::mutex> lk(state_mutex());
    SplitScratch &sc = g_split[dev];
    if (cudaEventRecord(sc.last_use, st) == cudaSuccess) sc.last_stream = st, sc.used = true;
}

}  // namespace

int *error_word()
{
    // one device int per device, allocated on first use and kept for the process
    static int *words[64] = {};
    int dev = 0;
    if (current_device(&dev)) return nullptr;
    std::lock_guard<std::mutex> lk(state_mutex());
    if (!words[dev]) {
        if (cudaMalloc(&words[dev], sizeof(int)) != cudaSuccess) return nullptr;
        cudaMemset(words[dev], 0, sizeof(int));
    }
    return words[dev];
}

// Shared by the public entry points.  `err` = device int that a kernel sets when
// a bounded wait runs out; NULL selects the per-device word that
// ls_gemm_status reads (allocated on first use).
int gemm_common(int nbatch, const uint8_t *a0, const uint8_t *a1, const uint8_t *w, const uint8_t *sfa0,
                const uint8_t *sfa1, const uint8_t *sfb, void *c0, void *c1, int out_dtype, int64_t M,
                int64_t N, int64_t K, void *stream, int *err)
{
    return gemm_fused(nbatch, a0, a1, w, sfa0, sfa1, sfb, c0, c1, out_dtype, M, N, K, stream, err, nullptr);
}

int gemm_fused(int nbatch, const uint8_t *a0, const uint8_t *a1, const uint8_t *w, const uint8_t *sfa0,
               const uint8_t *sfa1, const uint8_t *sfb, void *c0, void *c1, int out_dtype, int64_t M,
               int64_t N, int64_t K, void *stream, int *err, const QuantEpilogue *qe)
{
    if (int rc = check_device()) return rc;
    if (M < 0 || N < 0 || K < 0 || K % 128 != 0) return fail(LS_EINVAL, "K=%lld must be a multiple of 128", (long long)K);
    if (out_dtype != LS_F32 && out_dtype != LS_BF16) return fail(LS_EINVAL, "unsupported output dtype %d", out_dtype);
    if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return fail(LS_EINVAL, "dimension too large");
    if (M == 0 || N == 0) return LS_OK;
    if (K == 0) return fail(LS_EINVAL, "K must be positive");
    const bool fused = qe && qe->packed[0];
    const void *ptrs[] = {a0, w, sfa0, sfb};
    for (const void *q : ptrs)
        if (!q) return fail(LS_EINVAL, "null pointer");
    if (!c0 && !fused) return fail(LS_EINVAL, "null output");
    if (nbatch == 2 && (!a1 || !sfa1 || (!c1 && !fused))) return fail(LS_EINVAL, "null pointer (second batch)");
    if (fused) {
        if (N % 128 != 0) return fail(LS_EINVAL, "quantizing epilogue needs N %% 128 == 0 (N=%lld)", (long long)N);
        if (!qe->sf[0] || (nbatch == 2 && (!qe->packed[1] || !qe->sf[1]))) return fail(LS_EINVAL, "null quantized output");
        if (qe->act != 0 && qe->act != 1) return fail(LS_EINVAL, "unknown activation %d", qe->act);
        if (!aligned16(qe->packed[0]) || (nbatch == 2 && !aligned16(qe->packed[1])))
            return fail(LS_EALIGN, "quantized outputs must be 16-byte aligned");
    }
    if (!aligned16(a0) || !aligned16(w) || !aligned16(sfa0) || !aligned16(sfb) || !aligned16(c0) ||
        (nbatch == 2 && (!aligned16(a1) || !aligned16(sfa1) || !aligned16(c1))))    // NULL counts as aligned
        return fail(LS_EALIGN, "GEMM operands, scale buffers and outputs must be 16-byte aligned");
    const bool caller_err = err != nullptr;
    if (!err) err = error_word();
    if (!err) return fail(LS_ECUDA, "could not allocate the device error word");
    CUtensorMap ta0, ta1, tb;
    const int variant = g_gemm_variant.load(std::memory_order_relaxed), forced_splits = g_gemm_splits.load(std::memory_order_relaxed);
    const bool pair = variant == 2 || variant == 6 || (variant == 0 && (nbatch == 2 || M > BM));
    const int pair_bn = variant == 6 ? 192 : 256;
    // A tile of the single-CTA kernel: the box has only as many rows (16, 32, 64 or 128) as
    // A has.  The other rows of the stage keep whatever shared memory held; an output row
    // depends on its own row of A only, and rows past M are never stored.  (A 128-row box
    // that is almost entirely out of bounds still fills 16 KB of shared memory per k-tile:
    // 16384-squared went 36 -> 28 us at M = 1, 8192-squared 14.7 -> 10.0 us.)
    int a_box_rows = BM;
    if (!pair)
        for (a_box_rows = 16; a_box_rows < M && a_box_rows < BM; a_box_rows *= 2) {}
    if (int rc = make_operand_map(&ta0, a0, M, K / 2, a_box_rows)) return rc;
    if (int rc = make_operand_map(&ta1, nbatch == 2 ? a1 : a0, M, K / 2, a_box_rows)) return rc;
    // Single-CTA kernel: 128-column tiles when 256-column tiles would leave more than half
    // the SMs without one (the weight stream of a short-M product needs the SMs' loads in
    // flight more than it needs wide tiles).
    // Narrower still (64 columns) while the tiles of the wider shape would not occupy half
    // the SMs: N = K = 4096 has 32 tiles of 128 columns but 64 of 64.
    const int64_t m_tiles_ = (M + BM - 1) / BM;
    auto tiles_of = [&](int w_) { return m_tiles_ * ((N + w_ - 1) / w_) * nbatch; };
    int bn = 256;
    if (!pair) {
        if (variant == 3) bn = 128;
        else if (variant == 5) bn = 64;
        else if (variant == 0) {
            if (tiles_of(256) * 2 <= sm_count()) bn = 128;
            if (bn == 128 && tiles_of(128) * 2 <= sm_count()) bn = 64;
        }
    }
    if (int rc = make_operand_map(&tb, w, N, K / 2, pair ? pair_bn / 2 : bn)) return rc;
    GemmParams p{};
    p.sfa[0] = sfa0;
    p.sfa[1] = nbatch == 2 ? sfa1 : sfa0;
    p.sfb = sfb;
    p.c[0] = c0;
    p.c[1] = nbatch == 2 ? c1 : c0;
    p.M = int(M), p.N = int(N), p.K = int(K);
    p.nbatch = nbatch;
    p.out_bf16 = out_dtype == LS_BF16;
    p.err = err;
    p.splits = 1;
    p.kt_per_split = int((K / 2 + BKB - 1) / BKB);
    p.partial = nullptr;
    p.store_c = c0 != nullptr;
    p.a_box_bytes = a_box_rows * BKB;
    p.act = fused ? qe->act : 0;
    for (int b = 0; b < 2; b++) {
        p.q_packed[b] = fused ? qe->packed[nbatch == 2 ? b : 0] : nullptr;
        p.q_sf[b] = fused ? qe->sf[nbatch == 2 ? b : 0] : nullptr;
    }
    // Few output tiles and a long K (decode-like shapes, weight gradients): split K over
    // otherwise idle SMs into fp32 partial slabs that a second kernel sums in ascending
    // order.  Not on the allocation-free path (caller-supplied error word), which must
    // not touch an allocator, and not with the quantizing epilogue.
    const int k_tiles = p.kt_per_split;
    const int tiles = pair ? int((nbatch == 2 ? (M + BM - 1) / BM : (M + 2 * BM - 1) / (2 * BM)) * ((N + pair_bn - 1) / pair_bn))
                           : int(((M + BM - 1) / BM) * ((N + bn - 1) / bn)) * nbatch;
    const int slots = pair ? sm_count() / 2 : sm_count();       // work items that run at once
    int s = 1;
    // A stream that is being captured into a CUDA graph cannot wait for the scratch's last user
    // outside the capture, and a replay may run beside other users: no K split inside a capture.
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(static_cast<cudaStream_t>(stream), &capture) != cudaSuccess) capture = cudaStreamCaptureStatusNone;
    if (!caller_err && !fused && capture == cudaStreamCaptureStatusNone) {
        if (forced_splits > 0) {
            s = forced_splits;
        } else if (pair) {
            // Pays only with a quarter of the CTA pairs busy and a long K (weight gradients
            // of small layers): the partial slabs and the second kernel cost about 10 us.
            if (tiles * 4 <= slots && k_tiles >= 32) s = std::min(slots / tiles, k_tiles / 8);
        }
        // The single-CTA kernel does not split by itself: with 128-column tiles and an A box
        // of M rows the unsplit launch was as fast or faster at every short-M shape measured
        // (N = K = 2048 ... 16384; an in-kernel summation by the tile's last CTA was slower
        // still: one CTA reads all slabs).
        s = std::max(1, std::min(std::min(s, 16), k_tiles));
    }
    if (s > 1) {
        p.kt_per_split = (k_tiles + s - 1) / s;
        p.splits = (k_tiles + p.kt_per_split - 1) / p.kt_per_split;
    }
    // The scratch of a device has one user at a time: the next user's stream waits for the event
    // recorded after this one's summation.  Calls from several host threads must not interleave
    // between that wait and that record, hence the lock over the (asynchronous) launches.
    static std::mutex split_calls;
    std::unique_lock<std::mutex> split_lk;
    if (p.splits > 1) {
        split_lk = std::unique_lock<std::mutex>(split_calls);
        p.partial = splitk_acquire(size_t(p.splits) * nbatch * M * N * sizeof(float), static_cast<cudaStream_t>(stream));
        if (!p.partial) return fail(LS_ECUDA, "could not allocate split-K scratch");
    }
    if (pair) {
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        if (int rc = pair_bn == 192 ? launch_pair<32, 192>(ta0, ta1, tb, p, st) : launch_pair<32, 256>(ta0, ta1, tb, p, st)) return rc;
    } else {
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        if (int rc = bn == 64 ? launch<64>(ta0, ta1, tb, p, st)
                   : bn == 128 ? launch<128>(ta0, ta1, tb, p, st) : launch<256>(ta0, ta1, tb, p, st))
            return rc;
    }
    if (p.splits > 1) {
        for (int b = 0; b < nbatch; b++) {
            const int64_t mn = M * N;
            int64_t want = (mn / 4 + 255) / 256;
            int grid = int(want < 1 ? 1 : (want > sm_count() * 8 ? sm_count() * 8 : want));
            splitk_reduce_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
                p.partial + int64_t(b) * p.splits * mn, p.c[b], mn, p.splits, p.out_bf16);
        }
        splitk_release(static_cast<cudaStream_t>(stream));
        LS_LAUNCH_CHECK("splitk_reduce");
    }
    return LS_OK;
}

// Operands quantized with blocks of 16 (fp4.py:57, quantize_mxfp4(x, 16)): the single-CTA
// kernels with one scale tile per K = 64 MMA.  The single-CTA kernel takes tiles of 128 or 64
// columns (two 256-column accumulators sharing 32 columns leave no room for 48 scale columns);
// the CTA-pair kernel lets its accumulators share 64 columns.  No K split.
int gemm_block16(int nbatch, const uint8_t *a0, const uint8_t *a1, const uint8_t *w, const uint8_t *sfa0,
                 const uint8_t *sfa1, const uint8_t *sfb, void *c0, void *c1, int out_dtype, int64_t M,
                 int64_t N, int64_t K, void *stream, bool e4m3_scales)
{
    if (int rc = check_device()) return rc;
    if (M < 0 || N < 0 || K < 0 || K % 128 != 0) return fail(LS_EINVAL, "K=%lld must be a multiple of 128", (long long)K);
    if (out_dtype != LS_F32 && out_dtype != LS_BF16) return fail(LS_EINVAL, "unsupported output dtype %d", out_dtype);
    if (M > (1 << 30) || N > (1 << 30) || K > (1 << 30)) return fail(LS_EINVAL, "dimension too large");
    if (M == 0 || N == 0) return LS_OK;
    if (K == 0) return fail(LS_EINVAL, "K must be positive");
    if (!a0 || !w || !sfa0 || !sfb || !c0 || (nbatch == 2 && (!a1 || !sfa1 || !c1))) return fail(LS_EINVAL, "null pointer");
    if (!aligned16(a0) || !aligned16(w) || !aligned16(sfa0) || !aligned16(sfb) || !aligned16(c0) ||
        (nbatch == 2 && (!aligned16(a1) || !aligned16(sfa1) || !aligned16(c1))))
        return fail(LS_EALIGN, "GEMM operands, scale buffers and outputs must be 16-byte aligned");
    int *err = error_word();
    if (!err) return fail(LS_ECUDA, "could not allocate the device error word");
    CUtensorMap ta0, ta1, tb;
    // as for blocks of 32: CTA pairs for two batches or more than one row tile, else one CTA per
    // tile with a box of A no taller than A (ls_gemm_set_variant 2 / 1, 3, 5 force either)
    const int variant = g_gemm_variant.load(std::memory_order_relaxed);
    const bool pair = variant == 2 || variant == 6 || (variant == 0 && (nbatch == 2 || M > BM));
    const int pair_bn = variant == 6 ? 192 : 256;
    int a_box_rows = BM;
    if (!pair)
        for (a_box_rows = 16; a_box_rows < M && a_box_rows < BM; a_box_rows *= 2) {}
    const int64_t tiles128 = ((M + BM - 1) / BM) * ((N + 127) / 128) * nbatch;
    const int bn = variant == 5 || (variant != 3 && tiles128 * 2 <= sm_count()) ? 64 : 128;
    if (int rc = make_operand_map(&ta0, a0, M, K / 2, a_box_rows)) return rc;
    if (int rc = make_operand_map(&ta1, nbatch == 2 ? a1 : a0, M, K / 2, a_box_rows)) return rc;
    if (int rc = make_operand_map(&tb, w, N, K / 2, pair ? pair_bn / 2 : bn)) return rc;
    GemmParams p{};
    p.sfa[0] = sfa0;
    p.sfa[1] = nbatch == 2 ? sfa1 : sfa0;
    p.sfb = sfb;
    p.c[0] = c0;
    p.c[1] = nbatch == 2 ? c1 : c0;
    p.M = int(M), p.N = int(N), p.K = int(K);
    p.nbatch = nbatch;
    p.out_bf16 = out_dtype == LS_BF16;
    p.err = err;
    p.splits = 1;
    p.kt_per_split = int((K / 2 + BKB - 1) / BKB);
    p.partial = nullptr;
    p.store_c = true;
    p.a_box_bytes = a_box_rows * BKB;
    p.sf_e4m3 = e4m3_scales;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (pair) return pair_bn == 192 ? launch_pair<16, 192>(ta0, ta1, tb, p, st) : launch_pair<16, 256>(ta0, ta1, tb, p, st);
    return bn == 64 ? launch<64, 16>(ta0, ta1, tb, p, st) : launch<128, 16>(ta0, ta1, tb, p, st);
}

}  // namespace ls

using namespace ls;

extern "C" int ls_mxfp4_gemm_block16(const uint8_t *a_pk, const uint8_t *bt_pk, const uint8_t *sfa, const uint8_t *sfb,
                                     void *c, int out_dtype, int64_t M, int64_t N, int64_t K, void *stream)
{
    return gemm_block16(1, a_pk, nullptr, bt_pk, sfa, nullptr, sfb, c, nullptr, out_dtype, M, N, K, stream, false);
}

extern "C" int ls_mxfp4_gemm_dual_block16(const uint8_t *a1_pk, const uint8_t *a2_pk, const uint8_t *bt_pk,
                                          const uint8_t *sfa1, const uint8_t *sfa2, const uint8_t *sfb, void *c1,
                                          void *c2, int out_dtype, int64_t M, int64_t N, int64_t K, void *stream)
{
    return gemm_block16(2, a1_pk, a2_pk, bt_pk, sfa1, sfa2, sfb, c1, c2, out_dtype, M, N, K, stream, false);
}

extern "C" int ls_nvfp4_gemm(const uint8_t *a_pk, const uint8_t *bt_pk, const uint8_t *sfa, const uint8_t *sfb,
                             void *c, int out_dtype, int64_t M, int64_t N, int64_t K, void *stream)
{
    return gemm_block16(1, a_pk, nullptr, bt_pk, sfa, nullptr, sfb, c, nullptr, out_dtype, M, N, K, stream, true);
}

extern "C" int ls_nvfp4_gemm_dual(const uint8_t *a1_pk, const uint8_t *a2_pk, const uint8_t *bt_pk,
                                  const uint8_t *sfa1, const uint8_t *sfa2, const uint8_t *sfb, void *c1,
                                  void *c2, int out_dtype, int64_t M, int64_t N, int64_t K, void *stream)
{
    return gemm_block16(2, a1_pk, a2_pk, bt_pk, sfa1, sfa2, sfb, c1, c2, out_dtype, M, N, K, stream, true);
}

extern "C" int ls_mxfp4_gemm(const uint8_t *a_pk, const uint8_t *bt_pk, const uint8_t *sfa, const uint8_t *sfb,
                             void *c, int out_dtype, int64_t M, int64_t N, int64_t K, void *stream)
{
    return gemm_common(1, a_pk, nullptr, bt_pk, sfa, nullptr, sfb, c, nullptr, out_dtype, M, N, K, stream, nullptr);
}

extern "C" int ls_mxfp4_gemm_dual(const uint8_t *a1_pk, const uint8_t *a2_pk, const uint8_t *bt_pk,
                                  const uint8_t *sfa1, const uint8_t *sfa2, const uint8_t *sfb, void *c1,
                                  void *c2, int out_dtype, int64_t M, int64_t N, int64_t K, void *stream)
{
    return gemm_common(2, a1_pk, a2_pk, bt_pk, sfa1, sfa2, sfb, c1, c2, out_dtype, M, N, K, stream, nullptr);
}

extern "C" int ls_gemm_status(int *status_host)
{
    if (int rc = check_device()) return rc;
    int *err = ls::error_word();
    if (!err) return fail(LS_ECUDA, "could not allocate the device error word");
    int v = 0;
    LS_CUDA(cudaMemcpy(&v, err, sizeof(int), cudaMemcpyDeviceToHost));
    if (v) LS_CUDA(cudaMemset(err, 0, sizeof(int)));
    if (status_host) *status_host = v;
    if (v & 1) return fail(LS_ETIMEOUT, "a GEMM kernel gave up waiting on a barrier");
    if (v & 2) return fail(LS_EINVAL, "an E4M3 operand held a byte that is not an E2M1 value");
    return LS_OK;
}

extern "C" int ls_gemm_set_variant(int variant)
{
    if (variant < 0 || variant > 6 || variant == 4) return fail(LS_EINVAL, "variant must be 0..3, 5 or 6");
    g_gemm_variant.store(variant, std::memory_order_relaxed);
    return LS_OK;
}

extern "C" int ls_gemm_set_pdl(int on)
{
    g_gemm_pdl.store(on ? 1 : 0, std::memory_order_relaxed);
    return LS_OK;
}

extern "C" int ls_gemm_set_splits(int splits)
{
    if (splits < 0 || splits > 16) return fail(LS_EINVAL, "splits must be 0 (choose by shape) or 1..16");
    g_gemm_splits.store(splits, std::memory_order_relaxed);
    return LS_OK;
}

extern "C" int ls_mxfp4_gemm_quant(const uint8_t *a_pk, const uint8_t *bt_pk, const uint8_t *sfa, const uint8_t *sfb,
                                   void *c, int out_dtype, int act, uint8_t *q_packed, uint8_t *q_sf, int64_t M,
                                   int64_t N, int64_t K, void *stream)
{
    if (!q_packed || !q_sf) return fail(LS_EINVAL, "null quantized output");
    QuantEpilogue qe{{q_packed, nullptr}, {q_sf, nullptr}, act};
    return gemm_fused(1, a_pk, nullptr, bt_pk, sfa, nullptr, sfb, c, nullptr, out_dtype, M, N, K, stream, nullptr, &qe);
}

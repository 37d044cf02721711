// Measured ceiling of the block-scaled FP4 tensor pipe: the MMA instruction stream of the
// CTA-pair GEMM (cta_group::2, 256 x 256 x 64 per instruction, kind::mxf4.block_scale) on
// operands that already sit in shared memory, with no loads, no scale copies and no
// epilogue.  What this kernel reaches at the clock the power cap allows is what a GEMM
// kernel could reach if everything but the MMAs were free; the benchmark times it between
// launches of the real kernel so that both see the same power state.
#include "common.cuh"
#include "ptx.cuh"

namespace ls {
namespace {

constexpr int kPeakThreads = 128;
constexpr int kA = 128 * 128, kB = 128 * 128, kSfa = 1024, kSfb = 2048;      // one pipeline stage of the pair kernel
constexpr int kPeakSmem = kA + kB + kSfa + kSfb + 1024 + 64;

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPeakThreads, 1)
fp4_mma_peak_kernel(int rounds, int *err)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
    const uint32_t done_bar = smem_base + kA + kB + kSfa + kSfb;
    const uint32_t tmem_slot = done_bar + 8u;
    volatile uint32_t *tmem_slot_p = reinterpret_cast<volatile uint32_t *>(gen + kA + kB + kSfa + kSfb + 8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot_p + 1);
    const int warp = threadIdx.x >> 5;
    uint32_t cta;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cta));

    // operands: pseudo-random nibbles; scale bytes 2^-3 .. 2^3 around 1.0
    uint32_t x = 0x9E3779B9u * (blockIdx.x * kPeakThreads + threadIdx.x + 1u);
    for (int i = threadIdx.x; i < (kA + kB) / 4; i += kPeakThreads) {
        x ^= x << 13, x ^= x >> 17, x ^= x << 5;
        reinterpret_cast<uint32_t *>(gen)[i] = x;
    }
    for (int i = threadIdx.x; i < kSfa + kSfb; i += kPeakThreads) {
        x ^= x << 13, x ^= x >> 17, x ^= x << 5;
        gen[kA + kB + i] = uint8_t(124u + x % 7u);
    }
    if (threadIdx.x == 0) {
        ptx::mbar_init(done_bar, 1);
        *abort_flag = 0;
        ptx::fence_mbar_init();
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // generic-proxy writes -> tensor-core reads
    if (warp == 1) {
        ptx::tmem_alloc<2>(tmem_slot, 512);
        ptx::tmem_relinquish<2>();
    }
    ptx::tc_fence_before();
    __syncthreads();
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_p;

    if (warp == 1 && cta == 0 && ptx::elect_one()) {
        constexpr uint32_t idesc = ptx::idesc_mxf4(256, 256);
        const uint64_t adesc = ptx::desc_sw128(smem_base), bdesc = ptx::desc_sw128(smem_base + kA);
        const uint64_t sfadesc = ptx::desc_sf(smem_base + kA + kB), sfbdesc = ptx::desc_sf(smem_base + kA + kB + kSfa);
        const uint32_t sfa_t = tmem_base + 480, sfb_t = sfa_t + 8;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            ptx::tmem_cp_sf<2>(sfa_t + 4 * j, sfadesc + 32 * j);
            ptx::tmem_cp_sf<2>(sfb_t + 8 * j, sfbdesc + 32 * j);
            ptx::tmem_cp_sf<2>(sfb_t + 8 * j + 4, sfbdesc + 64 + 32 * j);
        }
        for (int r = 0; r < rounds; r++) {
            const uint32_t acc = tmem_base + ((r >> 5) & 1 ? 224u : 0u);          // a new "tile" every 32 stages
#pragma unroll
            for (int kb = 0; kb < 4; kb++) {
                const uint32_t id = (kb & 1) ? 2u : 0u;
                ptx::mma_mxf4<2>(acc, adesc + 2 * kb, bdesc + 2 * kb, idesc | (id << 29) | (id << 4),
                                 sfa_t + 4 * (kb >> 1) + (id << 30), sfb_t + 8 * (kb >> 1) + (id << 30),
                                 ((r & 31) == 0 && kb == 0) ? 0u : 1u);
            }
        }
        ptx::tc_commit_pair(done_bar, 1);
        if (!ptx::mbar_wait(done_bar, 0, abort_flag)) atomicExch(err, 1);
    }
    ptx::tc_fence_before();
    __syncthreads();
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc<2>(tmem_base, 512);
    }
}

}  // namespace
int *error_word();
}  // namespace ls

using namespace ls;

// Launches the MMA-only kernel on every CTA pair the device holds: `rounds` pipeline stages
// (4 MMAs of 256 x 256 x 64 each) per pair.  *flop_out receives the FLOPs of the launch.
// The caller times it (CUDA events on `stream`).
extern "C" int ls_fp4_mma_peak(int rounds, double *flop_out, void *stream)
{
    if (int rc = check_device()) return rc;
    if (rounds < 1 || rounds > (1 << 20)) return fail(LS_EINVAL, "rounds must be 1 .. 2^20");
    static bool attr_set[64] = {};
    int dev = 0;
    if (int rc = current_device(&dev)) return rc;
    {
        std::lock_guard<std::mutex> lk(state_mutex());
        if (!attr_set[dev]) {
            LS_CUDA(cudaFuncSetAttribute(fp4_mma_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPeakSmem));
            attr_set[dev] = true;
        }
    }
    int *err = error_word();
    if (!err) return fail(LS_ECUDA, "could not allocate the device error word");
    const int pairs = sm_count() / 2;
    fp4_mma_peak_kernel<<<2 * pairs, kPeakThreads, kPeakSmem, static_cast<cudaStream_t>(stream)>>>(rounds, err);
    LS_LAUNCH_CHECK("fp4_mma_peak");
    if (flop_out) *flop_out = double(pairs) * rounds * 4.0 * 2.0 * 256.0 * 256.0 * 64.0;
    return LS_OK;
}

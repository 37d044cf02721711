// FP4-compressed gradient all-reduce: reduce-scatter + all-gather by direct
// peer stores over NVLink, one process per GPU.
//
// Protocol (lockstep wire.py:104-138 with the fp4.py codec in place of the
// integer grid; every rank owns one contiguous shard of the padded buffer):
//   send    v = g + res; encode v to MXFP4 (16 packed bytes + 1 exponent byte
//           per 32 values); res = v - decode; store shard o's bytes straight
//           into owner o's receive slot [my rank]; raise flag[my rank] on o
//   reduce  owner: wait for every sender's flag; val = sum of the decoded
//           slots in ascending sender order from +0.0 (each add rounded to
//           fp32); val += ores; encode; ores = val - decode; store the result
//           into every rank's gather slot [my rank]; raise the gather flag
//   finish  wait for every owner's gather flag; g = decode(all shards) / world
// NCCL/gloo only carries the 64-byte IPC handles at set-up.
//
// Two ways to run a step.  Three launches on the caller's stream (send, reduce,
// finish): a kernel then only ever waits for kernels of OTHER GPUs.  Or one
// cooperative launch that cuts every shard into S sub-ranges and walks them as
// a pipeline -- send(t), reduce(t-1), finish(t-2) -- with one flag per
// sub-range, sender and phase, so that the owner's work on a sub-range and the
// decode of the one before overlap the memory passes of the next send instead
// of queueing behind a kernel boundary.  The cooperative launch guarantees that
// all CTAs are resident, which the waits inside one kernel rely on.
//
// Senders walk the owners starting at their right-hand neighbour (rank + 1),
// so at any moment every owner receives from one sender only instead of all
// ranks storing into owner 0 first.  A thread owns 8 consecutive values (one
// 32-byte load per operand, one 4-byte packed store); four adjacent lanes share
// a block of 32, so every instruction of a warp reads or writes whole 128-byte
// lines, locally and across NVLink.
//
// Every wait is bounded by a wall-clock limit (%globaltimer).  A CTA whose wait
// runs out records it in the status word, stores nothing more and raises no
// further flag, so the ranks that depend on it run out too: a lost peer becomes
// an error on every rank of that step instead of a silently different average.
// All arithmetic uses explicitly rounded intrinsics so that no multiply-add
// contraction changes a bit against the CPU oracle.
#include <cstring>
#include <new>

#include "common.cuh"

namespace ls {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kThreads = 256;
constexpr int kMaxSub = 8;                                  // sub-ranges a shard may be cut into
constexpr uint64_t kDefaultTimeoutNs = 20ull * 1000 * 1000 * 1000;   // a wait gives up after 20 s

struct Header {                 // start of every rank's arena
    uint32_t rs_flag[kMaxSub][kMaxWorld];       // epoch of the last completed send of sub-range c from rank s
    uint32_t ag_flag[kMaxSub][kMaxWorld];       // epoch of the last completed reduce of sub-range c by owner o
    uint32_t counter[kMaxSub][2];               // CTA completion counters (send, reduce)
    uint32_t work[2][kMaxSub][3];               // next group of (sub-range, phase) to hand out; set epoch & 1 is in
                                                // use, the other one is cleared for the next step
    uint32_t status;                // non-zero: a wait ran out
    uint32_t mx_flag[kMaxWorld];    // integer wires: epoch of rank s's last published chunk maxima
    uint32_t counter_mx;
};
constexpr size_t kHeaderBytes = 1024;
static_assert(sizeof(Header) <= kHeaderBytes, "header does not fit");

// The same sub-range [first, first + count) of every owner's shard, in groups of 8
// elements; both are multiples of 32 groups, so a warp never straddles a sub-range.
struct Sub {
    int index;
    uint32_t first, count;
};

struct Peers { uint8_t *arena[kMaxWorld]; };

struct WireGeom {
    int rank, world;
    int64_t padded, shard;          // elements
    int64_t slot_bytes;             // packed + exponent bytes of one shard, 256-aligned
    int64_t rs_off, ag_off;         // byte offsets of the slot arrays in an arena
    uint64_t timeout_ns;            // how long a wait on a peer's flag may last
    uint32_t *host_status;          // mapped pinned host word of this rank: set to 1 when a wait ran out
    int bits;                       // 0: MXFP4 payload; 8 / 16: integer payload (wire.py's int8 / int16)
    int dynamic;                    // 1: groups are handed out in chunks from a counter; 0: fixed shares per warp
    int64_t mx_off;                 // integer wires: [world][padded / 64] fp32 chunk maxima of every rank
};

struct Wire {
    WireGeom g;
    int dev;
    size_t arena_bytes;
    uint8_t *arena;
    Peers peers;
    bool mapped, opened[kMaxWorld];
    uint32_t epoch;
    int mode;                       // 0 = choose, 1 = three launches, 2 = one cooperative launch
    int subs;                       // sub-ranges of the cooperative launch (0 = choose)
    int fused_ctas;                 // CTAs of the cooperative kernel that fit the device at once (0 = not asked yet)
    int *status_host;               // pinned and mapped: a kernel whose wait ran out writes 1 here
};

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t global_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Thread s of the CTA polls rank s's flag until it reaches `epoch`.  Returns true (to
// every thread of the CTA) when all `world` flags arrived, false when the time limit ran
// out first; the time-out is recorded in the status word of this rank's arena.
__device__ __forceinline__ bool wait_flags(Header *h, const uint32_t *flags, int world, uint32_t epoch,
                                           uint64_t timeout_ns, uint32_t *host_status)
{
    bool ok = true;
    if (int(threadIdx.x) < world && int32_t(ld_acquire_sys(flags + threadIdx.x) - epoch) < 0) {
        const uint64_t t0 = global_ns();
        uint32_t polls = 0;
        while (int32_t(ld_acquire_sys(flags + threadIdx.x) - epoch) < 0) {
            if ((++polls & 15u) == 0 && global_ns() - t0 > timeout_ns) {
                atomicExch(&h->status, 1u);
                *reinterpret_cast<volatile uint32_t *>(host_status) = 1u;      // the host sees it without a copy or a sync
                __threadfence_system();
                ok = false;
                break;
            }
            __nanosleep(100);
        }
    }
    return __syncthreads_and(ok) != 0;
}

// After this CTA's stores: the last of the `ncta` CTAs that work for this rank raises
// flag[rank] = epoch on every peer.
__device__ __forceinline__ void signal_done(uint32_t *counter, uint32_t ncta, const Peers &peers, int world,
                                            int rank, size_t flag_off, uint32_t epoch)
{
    // The CTA's stores are ordered before thread 0's fence by the barrier; the fence (system
    // scope, cumulative) then orders them before the counter update and the flag stores.
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        uint32_t done = atomicAdd(counter, 1u);
        if (done == ncta - 1) {
            *counter = 0;
            __threadfence_system();
            for (int p = 0; p < world; p++)
                st_release_sys(reinterpret_cast<uint32_t *>(peers.arena[p] + flag_off) + rank, epoch);
        }
    }
}

// ---- 8 values per thread ---------------------------------------------------------------
// One thread owns 8 consecutive values (one 32-byte load or store), four adjacent lanes
// share a block of 32, so every load and store instruction of a warp covers whole 128-byte
// lines: 1 KB of fp32 values, 128 bytes of packed nibbles.
__device__ __forceinline__ void ld8(const float *p, float *v)
{
    asm volatile("ld.global.L1::no_allocate.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7])
                 : "l"(p) : "memory");
}
__device__ __forceinline__ void st8(float *p, const float *v)
{
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"l"(p), "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]) : "memory");
}
__device__ __forceinline__ void load8v(const float *p, int64_t i0, int64_t n, float (&v)[8])
{
    if (i0 + 8 <= n && (reinterpret_cast<uintptr_t>(p + i0) & 31) == 0) {
        ld8(p + i0, v);
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = i0 + i < n ? p[i0 + i] : 0.0f;
    }
}
__device__ __forceinline__ void store8v(float *p, int64_t i0, int64_t n, const float (&v)[8])
{
    if (i0 + 8 <= n && (reinterpret_cast<uintptr_t>(p + i0) & 31) == 0) {
        st8(p + i0, v);
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (i0 + i < n) p[i0 + i] = v[i];
    }
}

// Encodes the 8 values of this thread; lanes 4k .. 4k + 3 hold one block of 32.  Returns the
// packed nibbles; e8 = exponent byte of the block; dq[] = decoded values.
__device__ __forceinline__ uint32_t encode8(const float (&v)[8], uint32_t &e8, float (&dq)[8])
{
    uint32_t amax = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) amax = max(amax, __float_as_uint(v[i]) & 0x7FFFFFFFu);
    amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 1));
    amax = max(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, 2));
    e8 = block_e8m0(amax);
    const float inv = __uint_as_float(e8 == 255u ? 0x7FC00000u : inv_scale_bits(e8));
    const float sc = __uint_as_float(scale_bits(e8));
    float q[8];
#pragma unroll
    for (int i = 0; i < 8; i++) q[i] = __fmul_rn(v[i], inv);
    uint32_t pk;
    if (amax < kBitsInf) {
        pk = cvt_ref_e2m1x8(q);                          // all quotients finite: hardware converter
    } else {
        pk = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) pk |= e2m1_code<false>(q[i]) << (4 * i);
    }
    e2m1x8_values(pk, dq);
#pragma unroll
    for (int i = 0; i < 8; i++) dq[i] = __fmul_rn(dq[i], sc);
    return pk;
}

// val[i] += decode(pk)[i] * 2^(e8 - 127), each add rounded to fp32
__device__ __forceinline__ void add_decoded8(uint32_t pk, uint32_t e8, float (&val)[8])
{
    const float sc = __uint_as_float(scale_bits(e8));
    float d[8];
    e2m1x8_values(pk, d);
#pragma unroll
    for (int i = 0; i < 8; i++) val[i] = __fadd_rn(val[i], __fmul_rn(d[i], sc));
}

// ---- work distribution -----------------------------------------------------------------
// The groups of a part are handed out in chunks of kRows rows of 32 (one row = one group per
// lane) from a counter in the rank's arena: a warp takes the next chunk when it is done with
// its last.  Against a fixed share per thread this keeps every SM busy until the part ends,
// whichever SMs the memory system happens to serve slower (a sender of 64 Mi elements:
// 141 -> 134 us).  `total` is a multiple of 32, so rows are whole: body(base, rows, lane) is
// called by all 32 lanes of the warp for `rows` rows starting at group `base`.
constexpr uint32_t kRows = 8;

template <class F>
__device__ __forceinline__ void for_each_row(uint32_t total, uint32_t *work, uint32_t cta, uint32_t ncta, F body)
{
    const uint32_t lane = threadIdx.x & 31;
    if (!work) {                                    // fixed shares: warp w of CTA c takes rows c * 8 + w, + ncta * 8, ...
        constexpr uint32_t kWarps = kThreads / 32;
        for (uint32_t r = cta * kWarps + (threadIdx.x >> 5); r * 32u < total; r += ncta * kWarps) body(r * 32u, 1u, lane);
        return;
    }
    for (;;) {
        uint32_t base = 0;
        if (lane == 0) base = atomicAdd(work, kRows * 32u);
        base = __shfl_sync(0xFFFFFFFFu, base, 0);
        if (base >= total) break;
        const uint32_t rows = min(kRows, (total - base) / 32u);
        body(base, rows, lane);
    }
}

// ---- phase 1: sender ---------------------------------------------------------------
// Position j of a sub-range's flat group index belongs to step i = j / count, and step i goes
// to owner rank + 1 + i (this rank's own shard comes last).  A row of 32 never straddles two
// owners (count is a multiple of 32).
__device__ __forceinline__ void send_part(const float *g, int64_t n, float *res, const WireGeom &geo,
                                          const Peers &peers, Sub sub, uint32_t *work, uint32_t cta, uint32_t ncta)
{
    const uint32_t per_shard = uint32_t(geo.shard / 8);        // groups of 8 per shard: a multiple of 32
    const int64_t exp_off = geo.shard / 2;
    const bool first_of_block = (threadIdx.x & 3) == 0;
    for_each_row(uint32_t(geo.world) * sub.count, work, cta, ncta, [&](uint32_t base, uint32_t rows, uint32_t lane) {
        for (uint32_t c = 0; c < rows; c++) {
            const uint32_t row = base + 32u * c;
            const uint32_t i = row / sub.count;                        // uniform over the warp
            uint32_t o = uint32_t(geo.rank) + 1u + i;
            if (o >= uint32_t(geo.world)) o -= uint32_t(geo.world);
            const uint32_t in_shard = sub.first + (row - i * sub.count) + lane;
            uint8_t *slot = peers.arena[o] + geo.rs_off + int64_t(geo.rank) * geo.slot_bytes;
            const int64_t i0 = (int64_t(o) * per_shard + in_shard) * 8;
            float v[8], dq[8];
            load8v(g, i0, n, v);
            if (res) {
                float r[8];
                load8v(res, i0, geo.padded, r);
#pragma unroll
                for (int t = 0; t < 8; t++) v[t] = __fadd_rn(v[t], r[t]);
            }
            uint32_t e8;
            const uint32_t pk = encode8(v, e8, dq);
            if (res) {
#pragma unroll
                for (int t = 0; t < 8; t++) dq[t] = __fsub_rn(v[t], dq[t]);
                store8v(res, i0, geo.padded, dq);
            }
            reinterpret_cast<uint32_t *>(slot)[in_shard] = pk;
            if (first_of_block) slot[exp_off + in_shard / 4] = uint8_t(e8);   // a warp's 8 exponent bytes are contiguous
        }
    });
}

// ---- phase 2: owner ------------------------------------------------------------------
// WORLD > 0: the world size as a compile-time constant, so that the loads of up to four
// senders' slots are issued together before the first decode.  WORLD = 0: any size.
template <int WORLD>
__device__ __forceinline__ void reduce_part(float *ores, const WireGeom &geo, const Peers &peers, int reverse, Sub sub,
                                            uint32_t *work, uint32_t cta, uint32_t ncta)
{
    const int world = WORLD ? WORLD : geo.world;
    const uint8_t *rs = peers.arena[geo.rank] + geo.rs_off;
    const int64_t exp_off = geo.shard / 2;
    const bool first_of_block = (threadIdx.x & 3) == 0;
    for_each_row(sub.count, work, cta, ncta, [&](uint32_t base, uint32_t rows, uint32_t lane) {
        for (uint32_t c = 0; c < rows; c++) {
            const uint32_t g8 = sub.first + base + 32u * c + lane;
            float val[8], dq[8], r[8];
#pragma unroll
            for (int i = 0; i < 8; i++) val[i] = 0.0f;
            if (ores) load8v(ores, int64_t(g8) * 8, geo.shard, r);
            if (WORLD) {
                constexpr int B = WORLD < 4 ? (WORLD ? WORLD : 1) : 4;     // senders whose loads are in flight together
#pragma unroll
                for (int t0 = 0; t0 < WORLD; t0 += B) {
                    uint32_t pk[B], eb[B];
#pragma unroll
                    for (int t = 0; t < B; t++) {
                        const uint8_t *slot = rs + int64_t(reverse ? WORLD - 1 - (t0 + t) : t0 + t) * geo.slot_bytes;
                        pk[t] = reinterpret_cast<const uint32_t *>(slot)[g8];
                        eb[t] = slot[exp_off + g8 / 4];
                    }
#pragma unroll
                    for (int t = 0; t < B; t++) add_decoded8(pk[t], eb[t], val);
                }
            } else {
                for (int t = 0; t < world; t++) {
                    const uint8_t *slot = rs + int64_t(reverse ? world - 1 - t : t) * geo.slot_bytes;
                    add_decoded8(reinterpret_cast<const uint32_t *>(slot)[g8], slot[exp_off + g8 / 4], val);
                }
            }
            if (ores) {
#pragma unroll
                for (int i = 0; i < 8; i++) val[i] = __fadd_rn(val[i], r[i]);
            }
            uint32_t e8;
            const uint32_t pk2 = encode8(val, e8, dq);
            if (ores) {
#pragma unroll
                for (int i = 0; i < 8; i++) dq[i] = __fsub_rn(val[i], dq[i]);
                store8v(ores, int64_t(g8) * 8, geo.shard, dq);
            }
            // every rank's gather slot, starting at the right-hand neighbour
#pragma unroll
            for (int i = 0; i < (WORLD ? WORLD : kMaxWorld); i++) {
                if (i >= world) break;
                int p = geo.rank + 1 + i;
                if (p >= world) p -= world;
                uint8_t *slot = peers.arena[p] + geo.ag_off + int64_t(geo.rank) * geo.slot_bytes;
                reinterpret_cast<uint32_t *>(slot)[g8] = pk2;
                if (first_of_block) slot[exp_off + g8 / 4] = uint8_t(e8);
            }
        }
    });
}

__device__ __forceinline__ void reduce_any(float *ores, const WireGeom &geo, const Peers &peers, int reverse, Sub sub,
                                           uint32_t *work, uint32_t cta, uint32_t ncta)
{
    switch (geo.world) {
    case 1: reduce_part<1>(ores, geo, peers, reverse, sub, work, cta, ncta); break;
    case 2: reduce_part<2>(ores, geo, peers, reverse, sub, work, cta, ncta); break;
    case 4: reduce_part<4>(ores, geo, peers, reverse, sub, work, cta, ncta); break;
    case 8: reduce_part<8>(ores, geo, peers, reverse, sub, work, cta, ncta); break;
    default: reduce_part<0>(ores, geo, peers, reverse, sub, work, cta, ncta); break;
    }
}

// ---- phase 3: everyone ---------------------------------------------------------------
// One thread decodes 8 values (one packed word) and writes one 32-byte word; the loads of
// four rows are in flight together.  POW2: the world size is a power of two, so dividing by
// it is an exact multiplication that folds into the block scale.  Otherwise an IEEE division
// (wire.py:138 `.div_(world)`).
template <bool POW2>
__device__ __forceinline__ void finish_part(float *g, int64_t n, const WireGeom &geo, const Peers &peers, Sub sub,
                                            uint32_t *work, uint32_t cta, uint32_t ncta)
{
    constexpr uint32_t U = 4;
    static_assert(kRows % U == 0, "rows are decoded four at a time");
    const uint8_t *my = peers.arena[geo.rank];
    const float w = float(geo.world), rw = 1.0f / w;
    const int64_t exp_off = geo.shard / 2;
    for_each_row(uint32_t(geo.world) * sub.count, work, cta, ncta, [&](uint32_t base, uint32_t rows, uint32_t lane) {
        for (uint32_t c0 = 0; c0 < rows; c0 += U) {
            uint32_t pk[U], e8[U], q[U];
            int o[U];
#pragma unroll
            for (uint32_t u = 0; u < U; u++) {
                const uint32_t row = base + 32u * (c0 + u);
                o[u] = int(row / sub.count);                            // owner of this row's shard
                q[u] = sub.first + (row - uint32_t(o[u]) * sub.count) + lane;
                const bool ok = c0 + u < rows && int64_t(o[u]) * geo.shard + int64_t(q[u]) * 8 < n;
                const uint8_t *slot = my + geo.ag_off + int64_t(ok ? o[u] : 0) * geo.slot_bytes;
                pk[u] = ok ? reinterpret_cast<const uint32_t *>(slot)[q[u]] : 0u;
                e8[u] = ok ? slot[exp_off + (q[u] >> 2)] : 127u;
                if (!ok) o[u] = -1;
            }
#pragma unroll
            for (uint32_t u = 0; u < U; u++) {
                if (o[u] < 0) continue;
                float sc = __uint_as_float(scale_bits(e8[u]));
                if (POW2) sc = __fmul_rn(sc, rw);
                float t[8];
                e2m1x8_values(pk[u], t);
#pragma unroll
                for (int i = 0; i < 8; i++) t[i] = POW2 ? __fmul_rn(t[i], sc) : __fdiv_rn(__fmul_rn(t[i], sc), w);
                const int64_t first = int64_t(o[u]) * geo.shard;
                store8v(g + first, int64_t(q[u]) * 8, n - first, t);
            }
        }
    });
}

// The first kernel of a step clears the work counters of the NEXT step (the other set): the
// step before this one, which used them last, is complete on this GPU by stream order, and
// no other GPU touches them.
__device__ __forceinline__ void clear_next_work(Header *mine, uint32_t epoch, uint32_t cta)
{
    if (cta == 0 && threadIdx.x < kMaxSub * 3) (&mine->work[(epoch + 1) & 1][0][0])[threadIdx.x] = 0;
}

// ---- the three phases as separate launches ---------------------------------------------
__global__ void __launch_bounds__(kThreads, 5)
wire_send_kernel(const float *g, int64_t n, float *res, const __grid_constant__ WireGeom geo,
                 const __grid_constant__ Peers peers, uint32_t epoch, Sub sub)
{
    Header *mine = reinterpret_cast<Header *>(peers.arena[geo.rank]);
    clear_next_work(mine, epoch, blockIdx.x);
    send_part(g, n, res, geo, peers, sub, geo.dynamic ? &mine->work[epoch & 1][sub.index][0] : nullptr, blockIdx.x, gridDim.x);
    signal_done(&mine->counter[sub.index][0], gridDim.x, peers, geo.world, geo.rank,
                offsetof(Header, rs_flag) + sub.index * sizeof(mine->rs_flag[0]), epoch);
}

__global__ void __launch_bounds__(kThreads, 4)
wire_reduce_kernel(float *ores, const __grid_constant__ WireGeom geo, const __grid_constant__ Peers peers,
                   uint32_t epoch, int reverse, Sub sub)
{
    Header *mine = reinterpret_cast<Header *>(peers.arena[geo.rank]);
    if (!wait_flags(mine, mine->rs_flag[sub.index], geo.world, epoch, geo.timeout_ns, geo.host_status)) return;
    reduce_any(ores, geo, peers, reverse, sub, geo.dynamic ? &mine->work[epoch & 1][sub.index][1] : nullptr, blockIdx.x, gridDim.x);
    signal_done(&mine->counter[sub.index][1], gridDim.x, peers, geo.world, geo.rank,
                offsetof(Header, ag_flag) + sub.index * sizeof(mine->ag_flag[0]), epoch);
}

__global__ void __launch_bounds__(kThreads)
wire_finish_kernel(float *g, int64_t n, const __grid_constant__ WireGeom geo, const __grid_constant__ Peers peers,
                   uint32_t epoch, Sub sub)
{
    Header *mine = reinterpret_cast<Header *>(peers.arena[geo.rank]);
    if (!wait_flags(mine, mine->ag_flag[sub.index], geo.world, epoch, geo.timeout_ns, geo.host_status)) return;
    uint32_t *work = geo.dynamic ? &mine->work[epoch & 1][sub.index][2] : nullptr;
    if ((geo.world & (geo.world - 1)) == 0) finish_part<true>(g, n, geo, peers, sub, work, blockIdx.x, gridDim.x);
    else finish_part<false>(g, n, geo, peers, sub, work, blockIdx.x, gridDim.x);
}

// ---- one cooperative launch ---------------------------------------------------------
// The grid serves `nranks` ranks (one on a real multi-GPU run; all of them when several
// ranks are emulated on one GPU, which is how the single-GPU tests exercise the waits
// between ranks: all CTAs of a cooperative launch are resident together).  Rank v gets
// CTAs [v * ctas, (v + 1) * ctas).
struct RankArgs {
    float *g, *res, *ores;
    int64_t n;
    uint32_t epoch;
    WireGeom geo;
    Peers peers;
};
struct FusedArgs {
    RankArgs r[kMaxWorld];
    int nranks, ctas, subs, reverse, stagger;
};

template <int WORLD>
__global__ void __launch_bounds__(kThreads, 4)
wire_fused_kernel(const __grid_constant__ FusedArgs a)
{
    const uint32_t vr = blockIdx.x / uint32_t(a.ctas), cta = blockIdx.x - vr * uint32_t(a.ctas), ncta = uint32_t(a.ctas);
    const RankArgs &ra = a.r[vr];
    const WireGeom &geo = ra.geo;
    Header *mine = reinterpret_cast<Header *>(ra.peers.arena[geo.rank]);
    const int S = a.subs;
    const uint32_t per = uint32_t(geo.shard / 8) / uint32_t(S);
    const bool pow2 = (geo.world & (geo.world - 1)) == 0;
    // Within pipeline step t the three items are independent of each other (each depends on
    // items of step t - 1 at most), so CTAs may take them in different orders: with `stagger`
    // a third of the CTAs starts each step with the send, a third with the owner's part and a
    // third with the decode, which keeps the HBM-bound and the link-bound work mixed on every SM.
    const int rot = a.stagger ? int(cta % 3u) : 0;
    clear_next_work(mine, ra.epoch, cta);
    bool alive = true;
    for (int t = 0; t < S + 2 && alive; t++) {
        for (int q = 0; q < 3 && alive; q++) {
            const int item = (q + rot) % 3;
            if (item == 0 && t < S) {
                const Sub sub{t, uint32_t(t) * per, per};
                send_part(ra.g, ra.n, ra.res, geo, ra.peers, sub, geo.dynamic ? &mine->work[ra.epoch & 1][t][0] : nullptr, cta, ncta);
                signal_done(&mine->counter[t][0], ncta, ra.peers, geo.world, geo.rank,
                            offsetof(Header, rs_flag) + t * sizeof(mine->rs_flag[0]), ra.epoch);
            } else if (item == 1 && t >= 1 && t - 1 < S) {
                const int c = t - 1;
                const Sub sub{c, uint32_t(c) * per, per};
                alive = wait_flags(mine, mine->rs_flag[c], geo.world, ra.epoch, geo.timeout_ns, geo.host_status);
                if (alive) {
                    reduce_part<WORLD>(ra.ores, geo, ra.peers, a.reverse, sub, geo.dynamic ? &mine->work[ra.epoch & 1][c][1] : nullptr, cta, ncta);
                    signal_done(&mine->counter[c][1], ncta, ra.peers, geo.world, geo.rank,
                                offsetof(Header, ag_flag) + c * sizeof(mine->ag_flag[0]), ra.epoch);
                }
            } else if (item == 2 && t >= 2) {
                const int c = t - 2;
                const Sub sub{c, uint32_t(c) * per, per};
                alive = wait_flags(mine, mine->ag_flag[c], geo.world, ra.epoch, geo.timeout_ns, geo.host_status);
                if (alive) {
                    uint32_t *work = geo.dynamic ? &mine->work[ra.epoch & 1][c][2] : nullptr;
                    if (pow2) finish_part<true>(ra.g, ra.n, geo, ra.peers, sub, work, cta, ncta);
                    else finish_part<false>(ra.g, ra.n, geo, ra.peers, sub, work, cta, ncta);
                }
            }
        }
    }
}

// ======================================================================================
// Integer wires of the reference (wire.py:104-138): one fp32 scale per chunk of 64, shared
// by all ranks (maximum over ranks), exact int32 sum at the owner, owner re-encodes with its
// own grid, gather.  Same transport as above; every fp32 operation is the one torch runs,
// explicitly rounded (division by IEEE divide, rounding to nearest even integer).
// One thread owns 8 consecutive elements; 8 adjacent lanes share a chunk.
// ======================================================================================
constexpr int kChunk = 64;

__device__ __forceinline__ void load8(const float *p, int64_t i0, int64_t n, float (&v)[8])
{
    if (i0 + 8 <= n && (reinterpret_cast<uintptr_t>(p + i0) & 15) == 0) {
        float4 a = *reinterpret_cast<const float4 *>(p + i0), b = *reinterpret_cast<const float4 *>(p + i0 + 4);
        v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = i0 + i < n ? p[i0 + i] : 0.0f;
    }
}
__device__ __forceinline__ void store8(float *p, int64_t i0, int64_t n, const float (&v)[8])
{
    if (i0 + 8 <= n && (reinterpret_cast<uintptr_t>(p + i0) & 15) == 0) {
        *reinterpret_cast<float4 *>(p + i0) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(p + i0 + 4) = make_float4(v[4], v[5], v[6], v[7]);
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++)
            if (i0 + i < n) p[i0 + i] = v[i];
    }
}

__device__ __forceinline__ float chunk_max8(const float (&v)[8])
{
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) m = max(m, __float_as_uint(v[i]) & 0x7FFFFFFFu);
    m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 1));
    m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 2));
    m = max(m, __shfl_xor_sync(0xFFFFFFFFu, m, 4));
    return __uint_as_float(m);
}
// torch evaluates `lim / m` (Python scalar over tensor) as m.reciprocal() * lim: two roundings
__device__ __forceinline__ float grid_scale(float m, float lim) { return m > 0.0f ? __fmul_rn(__frcp_rn(m), lim) : 1.0f; }
__device__ __forceinline__ int quant_int(float x, float s, int lim)
{
    return max(-lim, min(lim, __float2int_rn(__fmul_rn(x, s))));       // torch.round: half to even
}
template <int BITS>
__device__ __forceinline__ void store_q8(uint8_t *slot, uint32_t g8, const int (&q)[8])
{
    if (BITS == 8) {
        uint2 w;
        w.x = (q[0] & 0xFF) | ((q[1] & 0xFF) << 8) | ((q[2] & 0xFF) << 16) | (uint32_t(q[3] & 0xFF) << 24);
        w.y = (q[4] & 0xFF) | ((q[5] & 0xFF) << 8) | ((q[6] & 0xFF) << 16) | (uint32_t(q[7] & 0xFF) << 24);
        reinterpret_cast<uint2 *>(slot)[g8] = w;
    } else {
        uint4 w;
        w.x = (q[0] & 0xFFFF) | (uint32_t(q[1] & 0xFFFF) << 16), w.y = (q[2] & 0xFFFF) | (uint32_t(q[3] & 0xFFFF) << 16);
        w.z = (q[4] & 0xFFFF) | (uint32_t(q[5] & 0xFFFF) << 16), w.w = (q[6] & 0xFFFF) | (uint32_t(q[7] & 0xFFFF) << 16);
        reinterpret_cast<uint4 *>(slot)[g8] = w;
    }
}
template <int BITS>
__device__ __forceinline__ void load_q8(const uint8_t *slot, uint32_t g8, int (&q)[8])
{
    if (BITS == 8) {
        const uint2 w = reinterpret_cast<const uint2 *>(slot)[g8];
#pragma unroll
        for (int i = 0; i < 4; i++) q[i] = int(int8_t(w.x >> (8 * i))), q[4 + i] = int(int8_t(w.y >> (8 * i)));
    } else {
        const uint4 w = reinterpret_cast<const uint4 *>(slot)[g8];
        const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int i = 0; i < 4; i++) q[2 * i] = int(int16_t(u[i] & 0xFFFF)), q[2 * i + 1] = int(int16_t(u[i] >> 16));
    }
}
// maximum over ranks of the published chunk maxima (chunk index c of the padded buffer)
__device__ __forceinline__ float shared_max(const uint8_t *my, const WireGeom &geo, int64_t c)
{
    const float *mx = reinterpret_cast<const float *>(my + geo.mx_off);
    const int64_t chunks = geo.padded / kChunk;
    float m = 0.0f;
    for (int s = 0; s < geo.world; s++) m = fmaxf(m, mx[s * chunks + c]);
    return m;
}

// phase 0: publish this rank's chunk maxima of v = g + res to every rank
__global__ void __launch_bounds__(kThreads)
wire_int_max_kernel(const float *__restrict__ g, int64_t n, const float *__restrict__ res, const __grid_constant__ WireGeom geo, const __grid_constant__ Peers peers,
                    uint32_t epoch)
{
    const uint32_t groups = uint32_t(geo.padded / 8), stride = gridDim.x * kThreads;
    const int64_t chunks = geo.padded / kChunk;
    for (uint32_t g8 = blockIdx.x * kThreads + threadIdx.x; g8 < groups; g8 += stride) {
        float v[8];
        load8(g, int64_t(g8) * 8, n, v);
        if (res) {
            float r[8];
            load8(res, int64_t(g8) * 8, geo.padded, r);
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = __fadd_rn(v[i], r[i]);
        }
        const float m = chunk_max8(v);
        if ((threadIdx.x & 7) == 0)
            for (int p = 0; p < geo.world; p++)
                reinterpret_cast<float *>(peers.arena[p] + geo.mx_off)[geo.rank * chunks + g8 / 8] = m;
    }
    Header *mine = reinterpret_cast<Header *>(peers.arena[geo.rank]);
    signal_done(&mine->counter_mx, gridDim.x, peers, geo.world, geo.rank, offsetof(Header, mx_flag), epoch);
}

// phase 1: quantize on the shared grid, update the sender residual, push to the owners
template <int BITS>
__global__ void __launch_bounds__(kThreads)
wire_int_send_kernel(const float *__restrict__ g, int64_t n, float *__restrict__ res, const __grid_constant__ WireGeom geo, const __grid_constant__ Peers peers,
                     uint32_t epoch)
{
    constexpr int LIM = (1 << (BITS - 1)) - 1;
    uint8_t *my = peers.arena[geo.rank];
    Header *mine = reinterpret_cast<Header *>(my);
    if (!wait_flags(mine, mine->mx_flag, geo.world, epoch, geo.timeout_ns, geo.host_status)) return;
    const uint32_t groups = uint32_t(geo.padded / 8), stride = gridDim.x * kThreads;
    const uint32_t g_per_shard = uint32_t(geo.shard / 8);
    uint32_t g8 = blockIdx.x * kThreads + threadIdx.x;
    uint32_t o = g8 / g_per_shard, in_shard = g8 - o * g_per_shard;
    for (; g8 < groups; g8 += stride, in_shard += stride) {
        while (in_shard >= g_per_shard) in_shard -= g_per_shard, o++;
        float v[8];
        load8(g, int64_t(g8) * 8, n, v);
        if (res) {
            float r[8];
            load8(res, int64_t(g8) * 8, geo.padded, r);
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = __fadd_rn(v[i], r[i]);
        }
        const float s = grid_scale(shared_max(my, geo, g8 / 8), float(LIM));
        int q[8];
#pragma unroll
        for (int i = 0; i < 8; i++) q[i] = quant_int(v[i], s, LIM);
        if (res) {
            float r[8];
#pragma unroll
            for (int i = 0; i < 8; i++) r[i] = __fsub_rn(v[i], __fdiv_rn(float(q[i]), s));
            store8(res, int64_t(g8) * 8, geo.padded, r);
        }
        store_q8<BITS>(peers.arena[o] + geo.rs_off + int64_t(geo.rank) * geo.slot_bytes, in_shard, q);
    }
    signal_done(&mine->counter[0][0], gridDim.x, peers, geo.world, geo.rank, offsetof(Header, rs_flag), epoch);
}

// phase 2: exact integer sum at the owner, owner grid, owner residual, push to everyone
template <int BITS>
__global__ void __launch_bounds__(kThreads)
wire_int_reduce_kernel(float *__restrict__ ores, const __grid_constant__ WireGeom geo, const __grid_constant__ Peers peers, uint32_t epoch)
{
    constexpr int LIM = (1 << (BITS - 1)) - 1;
    uint8_t *my = peers.arena[geo.rank];
    Header *mine = reinterpret_cast<Header *>(my);
    if (!wait_flags(mine, mine->rs_flag[0], geo.world, epoch, geo.timeout_ns, geo.host_status)) return;
    const uint32_t groups = uint32_t(geo.shard / 8), stride = gridDim.x * kThreads;
    const int64_t first_chunk = int64_t(geo.rank) * (geo.shard / kChunk);
    const int64_t payload = geo.shard * (BITS / 8);
    for (uint32_t g8 = blockIdx.x * kThreads + threadIdx.x; g8 < groups; g8 += stride) {
        int sum[8];
#pragma unroll
        for (int i = 0; i < 8; i++) sum[i] = 0;
        for (int t = 0; t < geo.world; t++) {
            int q[8];
            load_q8<BITS>(my + geo.rs_off + int64_t(t) * geo.slot_bytes, g8, q);
#pragma unroll
            for (int i = 0; i < 8; i++) sum[i] += q[i];
        }
        const float s = grid_scale(shared_max(my, geo, first_chunk + g8 / 8), float(LIM));
        float val[8], r[8];
#pragma unroll
        for (int i = 0; i < 8; i++) val[i] = __fdiv_rn(float(sum[i]), s);
        if (ores) {
            load8(ores, int64_t(g8) * 8, geo.shard, r);
#pragma unroll
            for (int i = 0; i < 8; i++) val[i] = __fadd_rn(val[i], r[i]);
        }
        const float s2 = grid_scale(chunk_max8(val), float(LIM));
        int q2[8];
#pragma unroll
        for (int i = 0; i < 8; i++) q2[i] = quant_int(val[i], s2, LIM);
        if (ores) {
#pragma unroll
            for (int i = 0; i < 8; i++) r[i] = __fsub_rn(val[i], __fdiv_rn(float(q2[i]), s2));
            store8(ores, int64_t(g8) * 8, geo.shard, r);
        }
        for (int p = 0; p < geo.world; p++) {
            uint8_t *slot = peers.arena[p] + geo.ag_off + int64_t(geo.rank) * geo.slot_bytes;
            store_q8<BITS>(slot, g8, q2);
            if ((threadIdx.x & 7) == 0) reinterpret_cast<float *>(slot + payload)[g8 / 8] = s2;
        }
    }
    signal_done(&mine->counter[0][1], gridDim.x, peers, geo.world, geo.rank, offsetof(Header, ag_flag), epoch);
}

// phase 3: decode the gathered shards, divide by the world size
template <int BITS>
__global__ void __launch_bounds__(kThreads)
wire_int_finish_kernel(float *__restrict__ g, int64_t n, const __grid_constant__ WireGeom geo, const __grid_constant__ Peers peers, uint32_t epoch)
{
    uint8_t *my = peers.arena[geo.rank];
    Header *mine = reinterpret_cast<Header *>(my);
    if (!wait_flags(mine, mine->ag_flag[0], geo.world, epoch, geo.timeout_ns, geo.host_status)) return;
    const uint32_t groups = uint32_t((n + 7) / 8), stride = gridDim.x * kThreads;
    const uint32_t g_per_shard = uint32_t(geo.shard / 8);
    const int64_t payload = geo.shard * (BITS / 8);
    const float w = float(geo.world);
    for (uint32_t g8 = blockIdx.x * kThreads + threadIdx.x; g8 < groups; g8 += stride) {
        const uint32_t o = g8 / g_per_shard, in_shard = g8 - o * g_per_shard;
        const uint8_t *slot = my + geo.ag_off + int64_t(o) * geo.slot_bytes;
        int q[8];
        load_q8<BITS>(slot, in_shard, q);
        const float s2 = reinterpret_cast<const float *>(slot + payload)[in_shard / 8];
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = __fdiv_rn(__fdiv_rn(float(q[i]), s2), w);
        store8(g, int64_t(g8) * 8, n, v);
    }
}

int grid_for(int64_t groups, int ctas_per_sm = 8)
{
    int64_t want = (groups + kThreads - 1) / kThreads;
    int64_t cap = int64_t(sm_count()) * ctas_per_sm;           // one resident wave: flags are polled once per CTA
    return int(want < 1 ? 1 : (want < cap ? want : cap));
}

Wire *as_wire(void *h) { return static_cast<Wire *>(h); }

int check_call(Wire *w, const float *g, int64_t numel)
{
    if (!w) return fail(LS_EINVAL, "null wire handle");
    if (!w->mapped) return fail(LS_ESTATE, "wire peers are not mapped yet");
    if (w->g.bits) return fail(LS_ESTATE, "this handle carries an integer wire");
    if (!g || numel <= 0 || numel > w->g.padded) return fail(LS_EINVAL, "numel %lld does not fit the wire (padded %lld)", (long long)numel, (long long)w->g.padded);
    return LS_OK;
}

// A step's epoch is a kernel argument that the host advances on every call: a CUDA graph would
// replay one epoch for ever and its waits would pass on stale flags.  Calls on a stream under
// capture are refused.
int refuse_capture(void *stream)
{
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(static_cast<cudaStream_t>(stream), &cs) == cudaSuccess && cs != cudaStreamCaptureStatusNone)
        return fail(LS_ESTATE, "a wire step cannot be captured into a CUDA graph (its epoch advances on the host)");
    return LS_OK;
}

}  // namespace
}  // namespace ls

using namespace ls;

extern "C" int64_t ls_wire_handle_bytes(void) { return int64_t(sizeof(cudaIpcMemHandle_t)); }

static int wire_create(int rank, int world, int64_t padded, int bits, void **out);
extern "C" int ls_wire_create(int rank, int world, int64_t padded, void **out)
{
    return wire_create(rank, world, padded, 0, out);
}
extern "C" int ls_wire_create_int(int rank, int world, int64_t padded, int bits, void **out)
{
    if (bits != 8 && bits != 16) return fail(LS_EINVAL, "integer wire has 8 or 16 bits, got %d", bits);
    return wire_create(rank, world, padded, bits, out);
}
static int wire_create(int rank, int world, int64_t padded, int bits, void **out)
{
    if (int rc = check_device()) return rc;
    if (!out) return fail(LS_EINVAL, "null output");
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return fail(LS_EINVAL, "rank %d / world %d unsupported (world <= %d)", rank, world, kMaxWorld);
    if (padded <= 0 || padded % (int64_t(world) * 256) != 0)
        return fail(LS_EINVAL, "padded=%lld must be a positive multiple of world*256", (long long)padded);
    if (padded / 4 > int64_t(0xFFFFFFFFu) - (int64_t(1) << 24))
        return fail(LS_EINVAL, "padded=%lld exceeds the 32-bit group index of the wire kernels", (long long)padded);
    Wire *w = new (std::nothrow) Wire();
    if (!w) return fail(LS_ECUDA, "out of host memory");
    w->g.rank = rank, w->g.world = world, w->g.padded = padded, w->g.shard = padded / world;
    int64_t raw = bits ? w->g.shard * (bits / 8) + (w->g.shard / kChunk) * 4 : w->g.shard / 2 + w->g.shard / 32;
    w->g.slot_bytes = (raw + 255) / 256 * 256;
    w->g.rs_off = int64_t(kHeaderBytes);
    w->g.ag_off = w->g.rs_off + w->g.slot_bytes * world;
    w->g.timeout_ns = kDefaultTimeoutNs;
    w->g.bits = bits;
    // groups handed out in chunks from a counter instead of fixed shares per warp: nothing on
    // one to four ranks (277 vs 281 us on four), 9 % on eight (292 vs 324 us)
    w->g.dynamic = world >= 8 ? 1 : 0;
    w->g.mx_off = w->g.ag_off + w->g.slot_bytes * world;
    w->arena_bytes = size_t(w->g.mx_off + (bits ? int64_t(world) * (padded / kChunk) * 4 : 0));
    w->mapped = false;
    w->epoch = 0;
    w->mode = 0, w->subs = 0, w->fused_ctas = 0;
    w->status_host = nullptr;
    for (int i = 0; i < kMaxWorld; i++) w->opened[i] = false, w->peers.arena[i] = nullptr;
    cudaError_t e = cudaGetDevice(&w->dev);
    if (e == cudaSuccess) e = cudaMalloc(&w->arena, w->arena_bytes);
    if (e == cudaSuccess) e = cudaMemset(w->arena, 0, w->arena_bytes);
    if (e == cudaSuccess) e = cudaHostAlloc(reinterpret_cast<void **>(&w->status_host), sizeof(int), cudaHostAllocMapped);
    if (e == cudaSuccess) e = cudaHostGetDevicePointer(reinterpret_cast<void **>(&w->g.host_status), w->status_host, 0);
    if (e != cudaSuccess) {
        size_t bytes = w->arena_bytes;
        if (w->arena) cudaFree(w->arena);
        delete w;
        return fail(LS_ECUDA, "wire arena of %zu bytes: %s", bytes, cudaGetErrorString(e));
    }
    *w->status_host = 0;
    w->peers.arena[rank] = w->arena;
    if (world == 1) w->mapped = true;
    *out = w;
    return LS_OK;
}

extern "C" int ls_wire_destroy(void *h)
{
    Wire *w = as_wire(h);
    if (!w) return LS_OK;
    cudaDeviceSynchronize();
    for (int i = 0; i < kMaxWorld; i++)
        if (w->opened[i]) cudaIpcCloseMemHandle(w->peers.arena[i]);
    cudaFree(w->arena);
    if (w->status_host) cudaFreeHost(w->status_host);
    delete w;
    return LS_OK;
}

extern "C" int ls_wire_local_handle(void *h, void *out)
{
    Wire *w = as_wire(h);
    if (!w || !out) return fail(LS_EINVAL, "null argument");
    cudaIpcMemHandle_t mh;
    LS_CUDA(cudaIpcGetMemHandle(&mh, w->arena));
    memcpy(out, &mh, sizeof mh);
    return LS_OK;
}

extern "C" int ls_wire_map_peers(void *h, const void *all_handles)
{
    Wire *w = as_wire(h);
    if (!w || !all_handles) return fail(LS_EINVAL, "null argument");
    if (w->mapped) return LS_OK;
    const cudaIpcMemHandle_t *hs = static_cast<const cudaIpcMemHandle_t *>(all_handles);
    for (int p = 0; p < w->g.world; p++) {
        if (p == w->g.rank) continue;
        void *ptr = nullptr;
        LS_CUDA(cudaIpcOpenMemHandle(&ptr, hs[p], cudaIpcMemLazyEnablePeerAccess));
        w->peers.arena[p] = static_cast<uint8_t *>(ptr);
        w->opened[p] = true;
    }
    w->mapped = true;
    return LS_OK;
}

extern "C" int ls_wire_map_local(void *h, void *const *wires)
{
    Wire *w = as_wire(h);
    if (!w || !wires) return fail(LS_EINVAL, "null argument");
    for (int p = 0; p < w->g.world; p++) {
        Wire *o = as_wire(wires[p]);
        if (!o || o->g.world != w->g.world || o->g.rank != p || o->g.padded != w->g.padded)
            return fail(LS_EINVAL, "wire %d does not match", p);
        w->peers.arena[p] = o->arena;
    }
    w->mapped = true;
    return LS_OK;
}

namespace {
Sub whole_shard(const Wire *w) { return Sub{0, 0u, uint32_t(w->g.shard / 8)}; }

// Sub-ranges of the cooperative launch: the requested number, lowered until it divides the
// shard into pieces of whole warps (multiples of 256 elements).
int subs_of(const Wire *w, int want)
{
    const int64_t units = w->g.shard / 256;
    // default: two sub-ranges, one on two ranks.  Every part boundary drains the CTA (barrier,
    // fence, flag), so more sub-ranges cost more than their overlap wins.  Measured, 64 Mi
    // elements with error feedback, 1 / 2 / 4 sub-ranges: one rank 321 / 306 / 345 us, two
    // ranks 268 / 288 / 341 us, four ranks 281 / 294 / 358 us and 266 us for two sub-ranges
    // with the CTAs taking a step's three items in rotated orders (the default from three
    // ranks up), eight ranks 315 / 327 / 442 us (312 / 318 / 440 with rotated orders; with the
    // groups handed out from a counter, the default there, 304 / 292 / 398 and 292 for three).
    // Letting the warps of a CTA pass the boundaries on their own (no barrier) was slower
    // still: the early warps' polling competes with the others' memory traffic.
    int s = want > 0 ? want : (w->g.world == 2 ? 1 : 2);
    if (s > kMaxSub) s = kMaxSub;
    while (s > 1 && units % s != 0) s--;
    return s;
}

const void *fused_entry(int world)
{
    switch (world) {
    case 1: return reinterpret_cast<const void *>(wire_fused_kernel<1>);
    case 2: return reinterpret_cast<const void *>(wire_fused_kernel<2>);
    case 4: return reinterpret_cast<const void *>(wire_fused_kernel<4>);
    case 8: return reinterpret_cast<const void *>(wire_fused_kernel<8>);
    default: return reinterpret_cast<const void *>(wire_fused_kernel<0>);
    }
}

// Rotated item orders: asked for explicitly, or by default from three ranks up when the
// number of sub-ranges was left to the library too.
int stagger_of(const Wire *w)
{
    if (w->mode & 0x100) return 1;
    return (w->subs == 0 && w->g.world >= 3) ? 1 : 0;
}

// CTAs of the cooperative kernel that can be resident on this device at once.
int fused_capacity(Wire *w)
{
    if (!w->fused_ctas) {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fused_entry(w->g.world), kThreads, 0) != cudaSuccess || per_sm < 1)
            return 0;
        w->fused_ctas = per_sm * sm_count();
    }
    return w->fused_ctas;
}

void fill_rank(RankArgs &r, Wire *w, float *g, int64_t numel, float *res, float *ores)
{
    r.g = g, r.res = res, r.ores = ores, r.n = numel, r.epoch = w->epoch, r.geo = w->g, r.peers = w->peers;
}

int launch_fused(FusedArgs &a, int capacity, cudaStream_t st)
{
    const int64_t groups = int64_t(a.r[0].geo.world) * (a.r[0].geo.shard / 8) / a.subs;     // send work of one sub-range
    int ctas = capacity / a.nranks;
    const int64_t want = (groups + kThreads - 1) / kThreads;
    if (want < ctas) ctas = int(want < 1 ? 1 : want);
    if (ctas < 1) return fail(LS_ECUDA, "the cooperative wire kernel does not fit %d ranks on this device", a.nranks);
    a.ctas = ctas;
    void *params[] = {&a};
    LS_CUDA(cudaLaunchCooperativeKernel(fused_entry(a.r[0].geo.world), dim3(unsigned(ctas * a.nranks)),
                                        dim3(kThreads), params, 0, st));
    return LS_OK;
}

}  // namespace

extern "C" int ls_wire_send(void *h, const float *g, int64_t numel, float *res, void *stream)
{
    Wire *w = as_wire(h);
    if (int rc = check_call(w, g, numel)) return rc;
    if (int rc = refuse_capture(stream)) return rc;
    w->epoch++;
    const Sub sub = whole_shard(w);
    wire_send_kernel<<<grid_for(int64_t(w->g.world) * sub.count, 5), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        g, numel, res, w->g, w->peers, w->epoch, sub);
    LS_LAUNCH_CHECK("wire_send");
    return LS_OK;
}

extern "C" int ls_wire_reduce(void *h, float *ores, int reverse, void *stream)
{
    Wire *w = as_wire(h);
    if (!w || !w->mapped || w->g.bits) return fail(LS_ESTATE, "wire not ready");
    if (int rc = refuse_capture(stream)) return rc;
    const Sub sub = whole_shard(w);
    wire_reduce_kernel<<<grid_for(sub.count, 4), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        ores, w->g, w->peers, w->epoch, reverse, sub);
    LS_LAUNCH_CHECK("wire_reduce");
    return LS_OK;
}

extern "C" int ls_wire_finish(void *h, float *g, int64_t numel, void *stream)
{
    Wire *w = as_wire(h);
    if (int rc = check_call(w, g, numel)) return rc;
    if (int rc = refuse_capture(stream)) return rc;
    const Sub sub = whole_shard(w);
    // four groups per thread and step
    wire_finish_kernel<<<grid_for((int64_t(w->g.world) * sub.count + 3) / 4, 8), kThreads, 0,
                         static_cast<cudaStream_t>(stream)>>>(g, numel, w->g, w->peers, w->epoch, sub);
    LS_LAUNCH_CHECK("wire_finish");
    return LS_OK;
}

extern "C" int ls_wire_set_mode(void *h, int mode, int subs, int stagger)
{
    Wire *w = as_wire(h);
    if (!w) return fail(LS_EINVAL, "null wire handle");
    if (mode < 0 || mode > 2) return fail(LS_EINVAL, "mode must be 0 (choose), 1 (three launches) or 2 (one cooperative launch)");
    if (subs < 0 || subs > kMaxSub) return fail(LS_EINVAL, "sub-ranges must be 0 (choose) or 1..%d", kMaxSub);
    w->mode = mode | (stagger ? 0x100 : 0), w->subs = subs;
    return LS_OK;
}

// 1 = three launches, 2 = one cooperative launch: what ls_wire_allreduce runs on this handle.
extern "C" int ls_wire_mode(void *h)
{
    Wire *w = as_wire(h);
    if (!w) return 0;
    const int m = w->mode & 0xFF;
    return m ? m : 2;
}

extern "C" int ls_wire_allreduce(void *h, float *g, int64_t numel, float *res, float *ores, int reverse,
                                 void *stream)
{
    Wire *w = as_wire(h);
    if (int rc = check_call(w, g, numel)) return rc;
    if (int rc = refuse_capture(stream)) return rc;
    if (ls_wire_mode(h) == 1) {
        if (int rc = ls_wire_send(h, g, numel, res, stream)) return rc;
        if (int rc = ls_wire_reduce(h, ores, reverse, stream)) return rc;
        return ls_wire_finish(h, g, numel, stream);
    }
    const int capacity = fused_capacity(w);
    if (!capacity) return fail(LS_ECUDA, "could not size the cooperative wire kernel");
    w->epoch++;
    FusedArgs a{};
    fill_rank(a.r[0], w, g, numel, res, ores);
    a.nranks = 1, a.subs = subs_of(w, w->subs), a.reverse = reverse, a.stagger = stagger_of(w);
    return launch_fused(a, capacity, static_cast<cudaStream_t>(stream));
}

// All ranks of a group created in ONE process on one GPU (ls_wire_map_local), one step, one
// cooperative launch: every rank's CTAs are resident together, so the waits between ranks
// are met inside the launch.  handles / gs / ress / oress: arrays of `world` entries in
// rank order (ress / oress or their entries may be NULL).
extern "C" int ls_wire_allreduce_group(void *const *handles, float *const *gs, int64_t numel, float *const *ress,
                                       float *const *oress, int reverse, void *stream)
{
    if (!handles || !gs) return fail(LS_EINVAL, "null argument");
    Wire *w0 = as_wire(handles[0]);
    if (int rc = check_call(w0, gs[0], numel)) return rc;
    if (int rc = refuse_capture(stream)) return rc;
    const int world = w0->g.world;
    const int capacity = fused_capacity(w0);
    if (!capacity) return fail(LS_ECUDA, "could not size the cooperative wire kernel");
    FusedArgs a{};
    for (int r = 0; r < world; r++) {
        Wire *w = as_wire(handles[r]);
        if (int rc = check_call(w, gs[r], numel)) return rc;
        if (w->g.rank != r || w->g.world != world || w->g.padded != w0->g.padded || w->dev != w0->dev)
            return fail(LS_EINVAL, "handle %d does not belong to this group", r);
        w->epoch++;
        fill_rank(a.r[r], w, gs[r], numel, ress ? ress[r] : nullptr, oress ? oress[r] : nullptr);
    }
    a.nranks = world, a.subs = subs_of(w0, w0->subs), a.reverse = reverse, a.stagger = stagger_of(w0);
    return launch_fused(a, capacity, static_cast<cudaStream_t>(stream));
}

// Integer wires: phase 0 publish maxima, 1 send, 2 reduce, 3 finish.
extern "C" int ls_wire_int_phase(void *h, int phase, float *g, int64_t numel, float *res, float *ores, void *stream)
{
    Wire *w = as_wire(h);
    if (!w || !w->mapped || !w->g.bits) return fail(LS_ESTATE, "not a ready integer wire");
    if (int rc = refuse_capture(stream)) return rc;
    if ((phase == 0 || phase == 1 || phase == 3) && (!g || numel <= 0 || numel > w->g.padded))
        return fail(LS_EINVAL, "numel %lld does not fit the wire", (long long)numel);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool b8 = w->g.bits == 8;
    switch (phase) {
    case 0:
        w->epoch++;
        wire_int_max_kernel<<<grid_for(w->g.padded / 8), kThreads, 0, st>>>(g, numel, res, w->g, w->peers, w->epoch);
        break;
    case 1:
        if (b8) wire_int_send_kernel<8><<<grid_for(w->g.padded / 8, 5), kThreads, 0, st>>>(g, numel, res, w->g, w->peers, w->epoch);
        else wire_int_send_kernel<16><<<grid_for(w->g.padded / 8, 5), kThreads, 0, st>>>(g, numel, res, w->g, w->peers, w->epoch);
        break;
    case 2:
        if (b8) wire_int_reduce_kernel<8><<<grid_for(w->g.shard / 8, 4), kThreads, 0, st>>>(ores, w->g, w->peers, w->epoch);
        else wire_int_reduce_kernel<16><<<grid_for(w->g.shard / 8, 4), kThreads, 0, st>>>(ores, w->g, w->peers, w->epoch);
        break;
    case 3:
        if (b8) wire_int_finish_kernel<8><<<grid_for((numel + 7) / 8), kThreads, 0, st>>>(g, numel, w->g, w->peers, w->epoch);
        else wire_int_finish_kernel<16><<<grid_for((numel + 7) / 8), kThreads, 0, st>>>(g, numel, w->g, w->peers, w->epoch);
        break;
    default:
        return fail(LS_EINVAL, "phase must be 0..3");
    }
    LS_LAUNCH_CHECK("wire_int_phase");
    return LS_OK;
}

extern "C" int ls_wire_int_allreduce(void *h, float *g, int64_t numel, float *res, float *ores, void *stream)
{
    for (int phase = 0; phase < 4; phase++)
        if (int rc = ls_wire_int_phase(h, phase, g, numel, res, ores, stream)) return rc;
    return LS_OK;
}

extern "C" int ls_wire_set_dynamic(void *h, int on)
{
    Wire *w = as_wire(h);
    if (!w) return fail(LS_EINVAL, "null wire handle");
    w->g.dynamic = on ? 1 : 0;
    return LS_OK;
}

extern "C" int ls_wire_set_timeout_us(void *h, int64_t microseconds)
{
    Wire *w = as_wire(h);
    if (!w || microseconds < 1 || microseconds > int64_t(3600) * 1000 * 1000)
        return fail(LS_EINVAL, "bad wire handle or time limit (1 us .. 1 h)");
    w->g.timeout_ns = uint64_t(microseconds) * 1000u;
    return LS_OK;
}

extern "C" int ls_wire_status(void *h, int *status_host)
{
    Wire *w = as_wire(h);
    if (!w) return fail(LS_EINVAL, "null wire handle");
    uint32_t v = 0;
    Header *hd = reinterpret_cast<Header *>(w->arena);
    LS_CUDA(cudaMemcpy(&v, &hd->status, sizeof v, cudaMemcpyDeviceToHost));
    if (v) LS_CUDA(cudaMemset(&hd->status, 0, sizeof v));
    *w->status_host = 0;
    if (status_host) *status_host = int(v);
    return v ? fail(LS_ETIMEOUT, "a wire kernel gave up waiting for a peer's flag") : LS_OK;
}

// Non-blocking: a kernel whose wait ran out also writes a word of mapped pinned host memory;
// this reads it.  Kernels still in flight are not waited for, so a time-out shows up as soon
// as it happened, at the next call that looks.
extern "C" int ls_wire_poll_status(void *h, int *status_host)
{
    Wire *w = as_wire(h);
    if (!w) return fail(LS_EINVAL, "null wire handle");
    const int v = *static_cast<volatile int *>(w->status_host);
    if (status_host) *status_host = v;
    return v ? fail(LS_ETIMEOUT, "a wire kernel gave up waiting for a peer's flag") : LS_OK;
}

// After a time-out: waits for this device, clears flags, counters and the status word and
// rewinds the epoch.  Every rank of the wire must call it (and meet in a host-side barrier
// before and after) before the wire is used again; error-feedback residuals are the
// caller's to clear.
extern "C" int ls_wire_reset(void *h)
{
    Wire *w = as_wire(h);
    if (!w) return fail(LS_EINVAL, "null wire handle");
    LS_CUDA(cudaDeviceSynchronize());
    LS_CUDA(cudaMemset(w->arena, 0, kHeaderBytes));
    LS_CUDA(cudaDeviceSynchronize());
    w->epoch = 0;
    *w->status_host = 0;
    return LS_OK;
}

// Raw bytes of the arena, for byte-exact checks of what crossed the wire:
// which = 0 receive slots (world x slot), 1 gather slots.  Copies to a device buffer.
extern "C" int ls_wire_debug_slots(void *h, int which, uint8_t *out, int64_t *slot_bytes, void *stream)
{
    Wire *w = as_wire(h);
    if (!w) return fail(LS_EINVAL, "null wire handle");
    if (slot_bytes) *slot_bytes = w->g.slot_bytes;
    if (out)
        LS_CUDA(cudaMemcpyAsync(out, w->arena + (which ? w->g.ag_off : w->g.rs_off), size_t(w->g.slot_bytes) * w->g.world,
                                cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)));
    return LS_OK;
}

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
// NCCL/gloo only carries the 64-byte IPC handles at set-up.  The three phases
// are three launches on the caller's stream; a phase only ever waits for
// kernels of OTHER GPUs (bounded, reported through the status word).
// All arithmetic uses explicitly rounded intrinsics so that no multiply-add
// contraction changes a bit against the CPU oracle.
#include <cstring>
#include <new>

#include "common.cuh"

namespace ls {
namespace {

constexpr int kMaxWorld = 8;
constexpr int kThreads = 256;
constexpr uint32_t kPollLimit = 1u << 22;     // default polls (x ~100 ns sleep each) before a wait gives up

constexpr int kMaxChunks = 8;   // pieces an all-reduce call may be cut into (each with its own flags)
struct Header {                 // start of every rank's arena
    uint32_t rs_flag[kMaxChunks][kMaxWorld];    // epoch of the last completed send of chunk c from rank s
    uint32_t ag_flag[kMaxChunks][kMaxWorld];    // epoch of the last completed reduce of chunk c by owner o
    uint32_t counter[kMaxChunks][2];            // CTA completion counters (send, reduce)
    uint32_t status;                // non-zero: a wait ran out
    uint32_t mx_flag[kMaxWorld];    // integer wires: epoch of rank s's last published chunk maxima
    uint32_t counter_mx;
};
constexpr size_t kHeaderBytes = 1024;
static_assert(sizeof(Header) <= kHeaderBytes, "header does not fit");

// A piece of one all-reduce: the same sub-range [first, first + count) (in groups of 8
// elements) of every owner's shard.  Pieces of one call run as separate launches on three
// streams, so that one piece's exchange overlaps the memory passes of the others.
struct Chunk {
    int index;
    uint32_t first, count;      // multiples of 32: a warp never straddles a piece
};

struct Peers { uint8_t *arena[kMaxWorld]; };

struct WireGeom {
    int rank, world;
    int64_t padded, shard;          // elements
    int64_t slot_bytes;             // packed + exponent bytes of one shard, 256-aligned
    int64_t rs_off, ag_off;         // byte offsets of the slot arrays in an arena
    uint32_t poll_limit;            // polls before a wait on a peer's flag gives up
    int bits;                       // 0: MXFP4 payload; 8 / 16: integer payload (wire.py's int8 / int16)
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
    // pipelined all-reduce: pieces of a call run on the caller's stream (send) and on two
    // streams of the wire (owner phase, decode), chained by events
    int chunks;                     // 0 = choose by size and world, n = cut every call into n pieces
    cudaStream_t s_reduce, s_finish;
    cudaEvent_t ev_start, ev_done, ev_sent[kMaxChunks], ev_reduced[kMaxChunks];
    bool pipe_ready;
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

// Thread s of every CTA polls rank s's flag; returns after all `world` flags reached `epoch`
// (or after poll_limit polls, recording the time-out).
__device__ __forceinline__ void wait_flags(Header *h, const uint32_t *flags, int world, uint32_t epoch,
                                           uint32_t poll_limit)
{
    if (int(threadIdx.x) < world) {
        uint32_t polls = 0;
        while (int32_t(ld_acquire_sys(flags + threadIdx.x) - epoch) < 0) {
            if (++polls > poll_limit) {
                atomicExch(&h->status, 1u);
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
}

// After this CTA's stores: the last CTA of the grid raises flag[rank] = epoch on every peer.
__device__ __forceinline__ void signal_done(Header *mine, uint32_t *counter, const Peers &peers, int world,
                                            int rank, size_t flag_off, uint32_t epoch)
{
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t done = atomicAdd(counter, 1u);
        if (done == gridDim.x - 1) {
            *counter = 0;
            __threadfence_system();
            for (int p = 0; p < world; p++)
                st_release_sys(reinterpret_cast<uint32_t *>(peers.arena[p] + flag_off) + rank, epoch);
        }
    }
}

// Encodes 8 values held by this thread (4 adjacent lanes share a block of 32).
// Returns packed nibbles; e8 = exponent byte of the block; dq[] = decoded values.
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
    float lo[4], hi[4];
    e2m1x4_values(pk, lo);
    e2m1x4_values(pk >> 16, hi);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        dq[i] = __fmul_rn(lo[i], sc);
        dq[4 + i] = __fmul_rn(hi[i], sc);
    }
    return pk;
}

// The 8 exponent bytes of a warp's 8 blocks, gathered into lane 0 as one 64-bit word.
__device__ __forceinline__ uint2 gather_exponents(uint32_t e8)
{
    uint2 w = make_uint2(0, 0);
#pragma unroll
    for (int b = 0; b < 4; b++) w.x |= __shfl_sync(0xFFFFFFFFu, e8, 4 * b) << (8 * b);
#pragma unroll
    for (int b = 0; b < 4; b++) w.y |= __shfl_sync(0xFFFFFFFFu, e8, 16 + 4 * b) << (8 * b);
    return w;
}

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

// ---- phase 1: sender ---------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
wire_send_kernel(const float *__restrict__ g, int64_t n, float *__restrict__ res, const __grid_constant__ WireGeom geo, const __grid_constant__ Peers peers,
                 uint32_t epoch, Chunk ch)
{
    const uint32_t stride = gridDim.x * kThreads;
    const int lane = threadIdx.x & 31;
    const uint32_t g_per_shard = uint32_t(geo.shard / 8);      // a multiple of 32: warps never straddle shards
    const uint32_t total = uint32_t(geo.world) * ch.count;
    // one flat loop over the piece's groups of all owners; the owner index advances with the position
    uint32_t j = blockIdx.x * kThreads + threadIdx.x;
    uint32_t o = j / ch.count, k = j - o * ch.count;
    for (; j < total; j += stride, k += stride) {
        while (k >= ch.count) k -= ch.count, o++;
        const uint32_t in_shard = ch.first + k, g8 = o * g_per_shard + in_shard;
        uint8_t *slot = peers.arena[o] + geo.rs_off + int64_t(geo.rank) * geo.slot_bytes;
        const int64_t i0 = int64_t(g8) * 8;
        float v[8], dq[8];
        load8(g, i0, n, v);
        if (res) {
            float r[8];
            load8(res, i0, geo.padded, r);
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = __fadd_rn(v[i], r[i]);
        }
        uint32_t e8;
        const uint32_t pk = encode8(v, e8, dq);
        if (res) {
            float r[8];
#pragma unroll
            for (int i = 0; i < 8; i++) r[i] = __fsub_rn(v[i], dq[i]);
            store8(res, i0, geo.padded, r);
        }
        reinterpret_cast<uint32_t *>(slot)[in_shard] = pk;
        const uint2 ex = gather_exponents(e8);
        if (lane == 0) *reinterpret_cast<uint2 *>(slot + geo.shard / 2 + in_shard / 4) = ex;
    }
    Header *mine = reinterpret_cast<Header *>(peers.arena[geo.rank]);
    signal_done(mine, &mine->counter[ch.index][0], peers, geo.world, geo.rank,
                offsetof(Header, rs_flag) + ch.index * sizeof(mine->rs_flag[0]), epoch);
}

// ---- phase 2: owner ------------------------------------------------------------------
// WORLD > 0: the world size as a compile-time constant, so that the loads of all
// senders' slots are issued together before the first decode.  WORLD = 0: any size.
template <int WORLD>
__global__ void __launch_bounds__(kThreads)
wire_reduce_kernel(float *__restrict__ ores, const __grid_constant__ WireGeom geo, const __grid_constant__ Peers peers, uint32_t epoch, int reverse,
                   Chunk ch)
{
    uint8_t *my = peers.arena[geo.rank];
    Header *mine = reinterpret_cast<Header *>(my);
    const int world = WORLD ? WORLD : geo.world;
    wait_flags(mine, mine->rs_flag[ch.index], world, epoch, geo.poll_limit);
    const uint32_t groups = ch.first + ch.count;               // end of this piece inside the shard
    const uint32_t stride = gridDim.x * kThreads;
    const int lane = threadIdx.x & 31;
    const uint8_t *rs = my + geo.rs_off;
    const int64_t exp_off = geo.shard / 2;
    for (uint32_t g8 = ch.first + blockIdx.x * kThreads + threadIdx.x; g8 < groups; g8 += stride) {
        float val[8], dq[8], r[8];
#pragma unroll
        for (int i = 0; i < 8; i++) val[i] = 0.0f;
        if (ores) load8(ores, int64_t(g8) * 8, geo.shard, r);
        if (WORLD) {
            uint32_t pk[WORLD ? WORLD : 1], eb[WORLD ? WORLD : 1];
#pragma unroll
            for (int t = 0; t < WORLD; t++) {
                const uint8_t *slot = rs + int64_t(reverse ? WORLD - 1 - t : t) * geo.slot_bytes;
                pk[t] = reinterpret_cast<const uint32_t *>(slot)[g8];
                eb[t] = slot[exp_off + g8 / 4];
            }
#pragma unroll
            for (int t = 0; t < WORLD; t++) {
                const float sc = __uint_as_float(scale_bits(eb[t]));
                float lo[4], hi[4];
                e2m1x4_values(pk[t], lo);
                e2m1x4_values(pk[t] >> 16, hi);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    val[i] = __fadd_rn(val[i], __fmul_rn(lo[i], sc));
                    val[4 + i] = __fadd_rn(val[4 + i], __fmul_rn(hi[i], sc));
                }
            }
        } else {
            for (int t = 0; t < world; t++) {
                const uint8_t *slot = rs + int64_t(reverse ? world - 1 - t : t) * geo.slot_bytes;
                const uint32_t pk = reinterpret_cast<const uint32_t *>(slot)[g8];
                const float sc = __uint_as_float(scale_bits(slot[exp_off + g8 / 4]));
                float lo[4], hi[4];
                e2m1x4_values(pk, lo);
                e2m1x4_values(pk >> 16, hi);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    val[i] = __fadd_rn(val[i], __fmul_rn(lo[i], sc));
                    val[4 + i] = __fadd_rn(val[4 + i], __fmul_rn(hi[i], sc));
                }
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
            for (int i = 0; i < 8; i++) r[i] = __fsub_rn(val[i], dq[i]);
            store8(ores, int64_t(g8) * 8, geo.shard, r);
        }
        const uint2 ex = gather_exponents(e8);
#pragma unroll
        for (int p = 0; p < (WORLD ? WORLD : kMaxWorld); p++) {
            if (p >= world) break;
            uint8_t *slot = peers.arena[p] + geo.ag_off + int64_t(geo.rank) * geo.slot_bytes;
            reinterpret_cast<uint32_t *>(slot)[g8] = pk2;
            if (lane == 0) *reinterpret_cast<uint2 *>(slot + exp_off + g8 / 4) = ex;
        }
    }
    signal_done(mine, &mine->counter[ch.index][1], peers, world, geo.rank,
                offsetof(Header, ag_flag) + ch.index * sizeof(mine->ag_flag[0]), epoch);
}

// ---- phase 3: everyone ---------------------------------------------------------------
// One thread decodes 4 values (two packed bytes) per step and writes one 16-byte
// word, so every load and store of a warp is one contiguous segment.  POW2: the
// world size is a power of two, so dividing by it is an exact multiplication that
// folds into the block scale.  Otherwise an IEEE division (wire.py:138 `.div_(world)`).
template <bool POW2>
__global__ void __launch_bounds__(kThreads)
wire_finish_kernel(float *__restrict__ g, int64_t n, const __grid_constant__ WireGeom geo, const __grid_constant__ Peers peers, uint32_t epoch,
                   Chunk ch)
{
    constexpr int U = 4;                                        // independent quads in flight per thread
    uint8_t *my = peers.arena[geo.rank];
    Header *mine = reinterpret_cast<Header *>(my);
    wait_flags(mine, mine->ag_flag[ch.index], geo.world, epoch, geo.poll_limit);
    const uint32_t stride = gridDim.x * kThreads;
    const uint32_t q_first = 2 * ch.first, q_end = 2 * (ch.first + ch.count);   // this piece in quads of 4 elements
    const float w = float(geo.world), rw = 1.0f / w;
    const bool vec = (reinterpret_cast<uintptr_t>(g) & 15) == 0;
    for (int o = 0; o < geo.world; o++) {
        const uint8_t *slot = my + geo.ag_off + int64_t(o) * geo.slot_bytes;
        const uint8_t *slot_e = slot + geo.shard / 2;
        const int64_t first = int64_t(o) * geo.shard;
        if (first >= n) break;
        const int64_t left = (n - first + 3) / 4;
        const uint32_t count = left < int64_t(q_end) ? uint32_t(left) : q_end;
        float *gs = g + first;
        const int64_t ns = n - first;                           // elements of g in this shard and beyond
        for (uint32_t q0 = q_first + blockIdx.x * kThreads + threadIdx.x; q0 < count; q0 += U * stride) {
            uint32_t pk[U], e8[U];
#pragma unroll
            for (int u = 0; u < U; u++) {
                const uint32_t q = q0 + u * stride;
                const bool ok = q < count;
                pk[u] = ok ? reinterpret_cast<const uint16_t *>(slot)[q] : 0u;
                e8[u] = ok ? slot_e[q >> 3] : 127u;
            }
#pragma unroll
            for (int u = 0; u < U; u++) {
                const uint32_t q = q0 + u * stride;
                if (q >= count) break;
                float sc = __uint_as_float(scale_bits(e8[u]));
                if (POW2) sc = __fmul_rn(sc, rw);
                float t[4];
                e2m1x4_values(pk[u], t);
#pragma unroll
                for (int i = 0; i < 4; i++) t[i] = POW2 ? __fmul_rn(t[i], sc) : __fdiv_rn(__fmul_rn(t[i], sc), w);
                const int64_t i0 = int64_t(q) * 4;
                if (vec && i0 + 4 <= ns) {
                    *reinterpret_cast<float4 *>(gs + i0) = make_float4(t[0], t[1], t[2], t[3]);
                } else {
                    for (int i = 0; i < 4; i++)
                        if (i0 + i < ns) gs[i0 + i] = t[i];
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
    signal_done(mine, &mine->counter_mx, peers, geo.world, geo.rank, offsetof(Header, mx_flag), epoch);
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
    wait_flags(mine, mine->mx_flag, geo.world, epoch, geo.poll_limit);
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
    signal_done(mine, &mine->counter[0][0], peers, geo.world, geo.rank, offsetof(Header, rs_flag), epoch);
}

// phase 2: exact integer sum at the owner, owner grid, owner residual, push to everyone
template <int BITS>
__global__ void __launch_bounds__(kThreads)
wire_int_reduce_kernel(float *__restrict__ ores, const __grid_constant__ WireGeom geo, const __grid_constant__ Peers peers, uint32_t epoch)
{
    constexpr int LIM = (1 << (BITS - 1)) - 1;
    uint8_t *my = peers.arena[geo.rank];
    Header *mine = reinterpret_cast<Header *>(my);
    wait_flags(mine, mine->rs_flag[0], geo.world, epoch, geo.poll_limit);
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
    signal_done(mine, &mine->counter[0][1], peers, geo.world, geo.rank, offsetof(Header, ag_flag), epoch);
}

// phase 3: decode the gathered shards, divide by the world size
template <int BITS>
__global__ void __launch_bounds__(kThreads)
wire_int_finish_kernel(float *__restrict__ g, int64_t n, const __grid_constant__ WireGeom geo, const __grid_constant__ Peers peers, uint32_t epoch)
{
    uint8_t *my = peers.arena[geo.rank];
    Header *mine = reinterpret_cast<Header *>(my);
    wait_flags(mine, mine->ag_flag[0], geo.world, epoch, geo.poll_limit);
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
    Wire *w = new (std::nothrow) Wire();
    if (!w) return fail(LS_ECUDA, "out of host memory");
    w->g.rank = rank, w->g.world = world, w->g.padded = padded, w->g.shard = padded / world;
    int64_t raw = bits ? w->g.shard * (bits / 8) + (w->g.shard / kChunk) * 4 : w->g.shard / 2 + w->g.shard / 32;
    w->g.slot_bytes = (raw + 255) / 256 * 256;
    w->g.rs_off = int64_t(kHeaderBytes);
    w->g.ag_off = w->g.rs_off + w->g.slot_bytes * world;
    w->g.poll_limit = kPollLimit;
    w->g.bits = bits;
    w->g.mx_off = w->g.ag_off + w->g.slot_bytes * world;
    w->arena_bytes = size_t(w->g.mx_off + (bits ? int64_t(world) * (padded / kChunk) * 4 : 0));
    w->mapped = false;
    w->epoch = 0;
    w->chunks = 0;
    w->pipe_ready = false;
    for (int i = 0; i < kMaxWorld; i++) w->opened[i] = false, w->peers.arena[i] = nullptr;
    cudaError_t e = cudaGetDevice(&w->dev);
    if (e == cudaSuccess) e = cudaMalloc(&w->arena, w->arena_bytes);
    if (e == cudaSuccess) e = cudaMemset(w->arena, 0, w->arena_bytes);
    if (e != cudaSuccess) {
        size_t bytes = w->arena_bytes;
        delete w;
        return fail(LS_ECUDA, "wire arena of %zu bytes: %s", bytes, cudaGetErrorString(e));
    }
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
    if (w->pipe_ready) {
        cudaStreamDestroy(w->s_reduce), cudaStreamDestroy(w->s_finish);
        cudaEventDestroy(w->ev_start), cudaEventDestroy(w->ev_done);
        for (int c = 0; c < kMaxChunks; c++) cudaEventDestroy(w->ev_sent[c]), cudaEventDestroy(w->ev_reduced[c]);
    }
    cudaFree(w->arena);
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
Chunk whole_shard(const Wire *w) { return Chunk{0, 0u, uint32_t(w->g.shard / 8)}; }

int launch_send(Wire *w, const float *g, int64_t numel, float *res, Chunk ch, int ctas_per_sm, cudaStream_t st)
{
    wire_send_kernel<<<grid_for(int64_t(w->g.world) * ch.count, ctas_per_sm), kThreads, 0, st>>>(g, numel, res, w->g, w->peers,
                                                                                               w->epoch, ch);
    LS_LAUNCH_CHECK("wire_send");
    return LS_OK;
}

int launch_reduce(Wire *w, float *ores, int reverse, Chunk ch, int ctas_per_sm, cudaStream_t st)
{
    const int grid = grid_for(ch.count, ctas_per_sm);
    switch (w->g.world) {
    case 1: wire_reduce_kernel<1><<<grid, kThreads, 0, st>>>(ores, w->g, w->peers, w->epoch, reverse, ch); break;
    case 2: wire_reduce_kernel<2><<<grid, kThreads, 0, st>>>(ores, w->g, w->peers, w->epoch, reverse, ch); break;
    case 4: wire_reduce_kernel<4><<<grid, kThreads, 0, st>>>(ores, w->g, w->peers, w->epoch, reverse, ch); break;
    case 8: wire_reduce_kernel<8><<<grid, kThreads, 0, st>>>(ores, w->g, w->peers, w->epoch, reverse, ch); break;
    default: wire_reduce_kernel<0><<<grid, kThreads, 0, st>>>(ores, w->g, w->peers, w->epoch, reverse, ch); break;
    }
    LS_LAUNCH_CHECK("wire_reduce");
    return LS_OK;
}

int launch_finish(Wire *w, float *g, int64_t numel, Chunk ch, int ctas_per_sm, cudaStream_t st)
{
    const bool pow2 = (w->g.world & (w->g.world - 1)) == 0;
    const int grid = grid_for((int64_t(w->g.world) * ch.count + 1) / 2, ctas_per_sm);    // four quads per thread and step
    if (pow2) wire_finish_kernel<true><<<grid, kThreads, 0, st>>>(g, numel, w->g, w->peers, w->epoch, ch);
    else wire_finish_kernel<false><<<grid, kThreads, 0, st>>>(g, numel, w->g, w->peers, w->epoch, ch);
    LS_LAUNCH_CHECK("wire_finish");
    return LS_OK;
}

int pipe_setup(Wire *w)
{
    if (w->pipe_ready) return LS_OK;
    LS_CUDA(cudaStreamCreateWithFlags(&w->s_reduce, cudaStreamNonBlocking));
    LS_CUDA(cudaStreamCreateWithFlags(&w->s_finish, cudaStreamNonBlocking));
    LS_CUDA(cudaEventCreateWithFlags(&w->ev_start, cudaEventDisableTiming));
    LS_CUDA(cudaEventCreateWithFlags(&w->ev_done, cudaEventDisableTiming));
    for (int c = 0; c < kMaxChunks; c++) {
        LS_CUDA(cudaEventCreateWithFlags(&w->ev_sent[c], cudaEventDisableTiming));
        LS_CUDA(cudaEventCreateWithFlags(&w->ev_reduced[c], cudaEventDisableTiming));
    }
    w->pipe_ready = true;
    return LS_OK;
}

// Pieces per call.  One unless the caller asks for more: on 1 and 2 GPUs the three phases
// of concurrent pieces compete for HBM (64 Mi elements, error feedback on: 312 -> 356 us
// alone, 284 -> 349 us with one peer at four pieces), which costs more than the hidden
// exchange latency saves.
int pieces_of(const Wire *w)
{
    const int64_t groups = w->g.shard / 8;
    int c = w->chunks > 0 ? w->chunks : 1;
    while (c > 1 && groups % (int64_t(c) * 32) != 0) c--;
    return c;
}
}  // namespace

extern "C" int ls_wire_send(void *h, const float *g, int64_t numel, float *res, void *stream)
{
    Wire *w = as_wire(h);
    if (int rc = check_call(w, g, numel)) return rc;
    w->epoch++;
    return launch_send(w, g, numel, res, whole_shard(w), 5, static_cast<cudaStream_t>(stream));
}

extern "C" int ls_wire_reduce(void *h, float *ores, int reverse, void *stream)
{
    Wire *w = as_wire(h);
    if (!w || !w->mapped) return fail(LS_ESTATE, "wire not ready");
    return launch_reduce(w, ores, reverse, whole_shard(w), 4, static_cast<cudaStream_t>(stream));
}

extern "C" int ls_wire_finish(void *h, float *g, int64_t numel, void *stream)
{
    Wire *w = as_wire(h);
    if (int rc = check_call(w, g, numel)) return rc;
    return launch_finish(w, g, numel, whole_shard(w), 8, static_cast<cudaStream_t>(stream));
}

extern "C" int ls_wire_set_chunks(void *h, int chunks)
{
    Wire *w = as_wire(h);
    if (!w) return fail(LS_EINVAL, "null wire handle");
    if (chunks < 0 || chunks > kMaxChunks) return fail(LS_EINVAL, "chunks must be 0 (choose) or 1..%d", kMaxChunks);
    w->chunks = chunks;
    return LS_OK;
}

extern "C" int ls_wire_allreduce(void *h, float *g, int64_t numel, float *res, float *ores, int reverse,
                                 void *stream)
{
    Wire *w = as_wire(h);
    if (int rc = check_call(w, g, numel)) return rc;
    const int pieces = pieces_of(w);
    if (pieces == 1) {
        if (int rc = ls_wire_send(h, g, numel, res, stream)) return rc;
        if (int rc = ls_wire_reduce(h, ores, reverse, stream)) return rc;
        return ls_wire_finish(h, g, numel, stream);
    }
    // Send pieces follow each other on the caller's stream; the owner phase of piece c
    // runs on a second stream once piece c is sent, its decode on a third once it is
    // reduced here.  The grids leave room for the three kernels to be resident together:
    // a kernel that waits for its peers must not keep the others off the SMs.
    if (int rc = pipe_setup(w)) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    w->epoch++;
    const uint32_t per = uint32_t(w->g.shard / 8 / pieces);
    LS_CUDA(cudaEventRecord(w->ev_start, st));
    LS_CUDA(cudaStreamWaitEvent(w->s_reduce, w->ev_start, 0));     // residuals and g are ready when the caller's stream says so
    LS_CUDA(cudaStreamWaitEvent(w->s_finish, w->ev_start, 0));
    for (int c = 0; c < pieces; c++) {
        const Chunk ch{c, uint32_t(c) * per, per};
        if (int rc = launch_send(w, g, numel, res, ch, 3, st)) return rc;
        LS_CUDA(cudaEventRecord(w->ev_sent[c], st));
        LS_CUDA(cudaStreamWaitEvent(w->s_reduce, w->ev_sent[c], 0));
        if (int rc = launch_reduce(w, ores, reverse, ch, 2, w->s_reduce)) return rc;
        LS_CUDA(cudaEventRecord(w->ev_reduced[c], w->s_reduce));
        LS_CUDA(cudaStreamWaitEvent(w->s_finish, w->ev_reduced[c], 0));
        if (int rc = launch_finish(w, g, numel, ch, 2, w->s_finish)) return rc;
    }
    LS_CUDA(cudaEventRecord(w->ev_done, w->s_finish));
    LS_CUDA(cudaStreamWaitEvent(st, w->ev_done, 0));
    return LS_OK;
}

// Integer wires: phase 0 publish maxima, 1 send, 2 reduce, 3 finish.
extern "C" int ls_wire_int_phase(void *h, int phase, float *g, int64_t numel, float *res, float *ores, void *stream)
{
    Wire *w = as_wire(h);
    if (!w || !w->mapped || !w->g.bits) return fail(LS_ESTATE, "not a ready integer wire");
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

extern "C" int ls_wire_set_poll_limit(void *h, int64_t polls)
{
    Wire *w = as_wire(h);
    if (!w || polls < 1 || polls > (int64_t(1) << 31)) return fail(LS_EINVAL, "bad wire handle or poll limit");
    w->g.poll_limit = uint32_t(polls);
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
    if (status_host) *status_host = int(v);
    return v ? fail(LS_ETIMEOUT, "a wire kernel gave up waiting for a peer's flag") : LS_OK;
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

// Kernels of the sharded step that talk to the other GPUs directly over
// NVLink through peer-mapped pointers (plain loads and stores, no multicast):
//
//   reduce_stat_kernel      reduce-scatter + statistics in one pass: for every
//                           element of this rank's shard, load the FP16 gradient
//                           from every rank's pool, add in FP32 in rank order,
//                           round once to FP16, store it in the local pool and
//                           accumulate its square for the global norm.
//   adamw_table_peer_kernel update + all-gather in one pass: the update kernel
//                           of the single-GPU path, with every new FP16 parameter
//                           also stored at the same offset of every peer's pool.
//
// Neither kernel waits on another GPU: ordering between ranks comes from the
// small NCCL collectives the host code enqueues around them (zero1.cu).
#include "zero1_p2p.h"

#include <cstdlib>
#include <mutex>

#include "adamw_bulk.cuh"
#include "adamw_update.cuh"
#include "host_util.h"
#include "tensor_list.h"

namespace rlcu {

namespace {

__device__ __forceinline__ void add_h8(uint4 x, F8& acc, bool bf) {
    const F8 f = x8_to_f8(x, bf);
#pragma unroll
    for (int i = 0; i < 8; i++) acc.a[i] = __fadd_rn(acc.a[i], f.a[i]);
}

// x holds the reduced gradients as stored (already rounded to 16 bits): they are what the
// update will use, so a sum that overflowed the 16-bit format counts as non-finite.
__device__ __forceinline__ void square_accumulate(const F8& x, float unscale, float (&acc)[4], float& probe) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
        probe = __fmaf_rn(x.a[i], 0.0f, probe);        // NaN once any value is inf or NaN
        const float a = x.a[i] * unscale;
        acc[i & 3] = fmaf(a, a, acc[i & 3]);
    }
}

// UB groups of 8 elements per thread: all loads (UB per rank) are issued before any
// arithmetic; each group is summed over the ranks in rank order (FP32) and rounded
// once to FP16.  Group u of the thread is `stride` groups after group u-1.
template <int WORLD, int UB>
__device__ __forceinline__ void reduce_groups(const PeerIn& peers, ptrdiff_t off, __half* dst,
                                              ptrdiff_t stride, float unscale, float (&acc)[4], bool bf,
                                              float& probe) {
    constexpr int W = WORLD > 0 ? WORLD : kMaxWorld;
    const int n = WORLD > 0 ? WORLD : peers.n;
    uint4 x[UB][W];
#pragma unroll
    for (int u = 0; u < UB; u++)
#pragma unroll
        for (int j = 0; j < W; j++)
            if (j < n) x[u][j] = ld_h8(peers.base[j] + off + u * stride * kGroup);
#pragma unroll
    for (int u = 0; u < UB; u++) {
        F8 sum = x8_to_f8(x[u][0], bf);
#pragma unroll
        for (int j = 1; j < W; j++)
            if (j < n) add_h8(x[u][j], sum, bf);
        const uint4 r = f8_to_x8(sum, bf);
        *reinterpret_cast<uint4*>(dst + u * stride * kGroup) = r;   // default policy: the update pass reads it next
        square_accumulate(x8_to_f8(r, bf), unscale, acc, probe);
    }
}

struct __align__(32) U8 { uint32_t w[8]; };
__device__ __forceinline__ U8 ld_h16(const __half* p) {
    U8 r;
    asm volatile("ld.global.cs.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.w[0]), "=r"(r.w[1]), "=r"(r.w[2]), "=r"(r.w[3]),
                   "=r"(r.w[4]), "=r"(r.w[5]), "=r"(r.w[6]), "=r"(r.w[7])
                 : "l"(p));
    return r;
}
// 16 consecutive elements per thread with 256-bit loads from every rank.
template <int WORLD, int UB>
__device__ __forceinline__ void reduce_wide(const PeerIn& peers, ptrdiff_t off, __half* dst,
                                            ptrdiff_t stride, float unscale, float (&acc)[4], bool bf,
                                            float& probe) {
    constexpr int W = WORLD > 0 ? WORLD : kMaxWorld;
    const int n = WORLD > 0 ? WORLD : peers.n;
    U8 x[UB][W];
#pragma unroll
    for (int u = 0; u < UB; u++)
#pragma unroll
        for (int j = 0; j < W; j++)
            if (j < n) x[u][j] = ld_h16(peers.base[j] + off + u * stride * 16);
#pragma unroll
    for (int u = 0; u < UB; u++) {
#pragma unroll
        for (int h = 0; h < 2; h++) {
            F8 sum = x8_to_f8(make_uint4(x[u][0].w[4 * h], x[u][0].w[4 * h + 1], x[u][0].w[4 * h + 2], x[u][0].w[4 * h + 3]), bf);
#pragma unroll
            for (int j = 1; j < W; j++)
                if (j < n) add_h8(make_uint4(x[u][j].w[4 * h], x[u][j].w[4 * h + 1], x[u][j].w[4 * h + 2], x[u][j].w[4 * h + 3]), sum, bf);
            const uint4 r = f8_to_x8(sum, bf);
            *reinterpret_cast<uint4*>(dst + u * stride * 16 + h * 8) = r;
            square_accumulate(x8_to_f8(r, bf), unscale, acc, probe);
        }
    }
}

// loads in flight per thread are capped at eight 16-byte vectors
template <int WORLD>
struct ReduceBatch {
    static constexpr int value = WORLD == 1 ? 4 : WORLD == 2 ? 4 : WORLD == 4 ? 2 : 1;
};

// The kernel waits on NVLink round trips, so residency matters more than registers: the
// 4-rank instantiation is held to the register count that lets three CTAs share an SM
// (a minimum of 0 leaves the others to the compiler).
template <int WORLD>
__global__ void __launch_bounds__(kThreads, WORLD == 4 ? 3 : 0)
reduce_stat_kernel(const WorkItem* __restrict__ table, uint32_t n_items,
                   const __grid_constant__ PeerIn peers, float unscale_arg,
                   const rlcu_scaler_state* scaler, rlcu_stat* out, float* partials,
                   unsigned int* counter) {
    __shared__ float warp_sums[kThreads / 32];
    __shared__ bool is_last;
    float unscale = unscale_arg;
    if (scaler) {
        const float mul = scaler->grad_mul == 0.0f ? 1.0f : scaler->grad_mul;
        unscale = __fmul_rn(mul, __fdiv_rn(1.0f, scaler->scale));
    }
    const int n = WORLD > 0 ? WORLD : peers.n;
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float probe = 0.0f;
    for (uint32_t idx = blockIdx.x; idx < n_items; idx += gridDim.x) {
        const WorkItem* wi = table + idx;
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(wi));        // p, g
        const uint4 d = __ldg(reinterpret_cast<const uint4*>(wi) + 2);    // master, count, wd
        const uint4 e = __ldg(reinterpret_cast<const uint4*>(wi) + 3);    // flags
        __half* g = reinterpret_cast<__half*>(((uint64_t)a.w << 32) | a.z);
        const uint32_t count = d.z;
        const uint32_t fl = e.x;
        if (fl & RLCU_TENSOR_GRAD_ZERO) continue;
        const bool bf = (fl & kItemBF16) != 0;
        const ptrdiff_t base_off = g - peers.local_base;
        const uint32_t groups = (fl & kItemVec16) ? count / kGroup : 0;
        // full items whose addresses are 32-byte aligned on every rank: 256-bit loads
        // (sm_100), 16 consecutive elements per thread (measured 5 % faster over NVLink
        // than 128-bit loads)
        bool wide = count == kChunk;
        for (int j = 0; j < n; j++) wide = wide && ((reinterpret_cast<uintptr_t>(peers.base[j] + base_off) & 31) == 0);
        if (wide) {
#ifdef RLCU_RS_WIDE_UB
            constexpr int UB = RLCU_RS_WIDE_UB;
#else
            constexpr int UB = WORLD == 8 ? 1 : 2;       // 512 wide groups per item, 2 per thread
#endif
#pragma unroll
            for (int b = 0; b < 2 / UB; b++) {
                const ptrdiff_t first = (ptrdiff_t)(threadIdx.x + b * UB * kThreads) * 16;
                reduce_wide<WORLD, UB>(peers, base_off + first, g + first, kThreads, unscale, acc, bf, probe);
            }
            continue;
        }
        if (count == kChunk && (fl & kItemVec16)) {
            constexpr int UB = ReduceBatch<WORLD>::value;
#pragma unroll
            for (int b = 0; b < kGroupsPerThread / UB; b++) {
                const ptrdiff_t first = (ptrdiff_t)(threadIdx.x + b * UB * kThreads) * kGroup;
                reduce_groups<WORLD, UB>(peers, base_off + first, g + first, kThreads, unscale, acc, bf, probe);
            }
            continue;
        }
        // partial item (head or tail of a tensor): batches of groups while enough are left
        {
            constexpr int UB = ReduceBatch<WORLD>::value;
            uint32_t grp = threadIdx.x;
            for (; grp + (UB - 1) * kThreads < groups; grp += UB * kThreads)
                reduce_groups<WORLD, UB>(peers, base_off + (ptrdiff_t)grp * kGroup, g + (size_t)grp * kGroup, kThreads,
                                         unscale, acc, bf, probe);
            for (; grp < groups; grp += kThreads)
                reduce_groups<WORLD, 1>(peers, base_off + (ptrdiff_t)grp * kGroup, g + (size_t)grp * kGroup, 0, unscale, acc, bf, probe);
        }
        for (uint32_t i = groups * kGroup + threadIdx.x; i < count; i += kThreads) {
            float s = x_to_f(__half_as_ushort(peers.base[0][base_off + i]), bf);
            for (int j = 1; j < n; j++) s = __fadd_rn(s, x_to_f(__half_as_ushort(peers.base[j][base_off + i]), bf));
            const __half r = __ushort_as_half(f_to_x(s, bf));
            g[i] = r;
            const float raw = x_to_f(__half_as_ushort(r), bf);
            probe = __fmaf_rn(raw, 0.0f, probe);
            const float x = raw * unscale;
            acc[0] = fmaf(x, x, acc[0]);
        }
    }
    float mine = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    if (isnan(probe)) mine = __int_as_float(0x7FC00000);     // NaN total = a non-finite gradient (see finalize_stat)
    const float block_total = block_sum(mine, warp_sums);
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = block_total;
        __threadfence();
        is_last = (atomicAdd(counter, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (threadIdx.x < 32) {
        double s = 0.0;
        for (uint32_t i = threadIdx.x; i < gridDim.x; i += 32) s += (double)__ldcg(partials + i);
#pragma unroll
        for (int mask = 16; mask >= 1; mask >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, mask);
        if (threadIdx.x == 0) {
            *counter = 0;
            out->sum_sq = s;      // this rank's share; the host code all-reduces it
        }
    }
}

// ---------------------------------------------------------------------------
// reduce-scatter + statistics over FP32 gradient pools (RLCU_ZERO1_GRADS_F32)
// ---------------------------------------------------------------------------
// For 16-bit parameters whose gradients were accumulated in FP32.  Every element of the shard
// is loaded from all ranks' pools, added in FP32 in rank order and stored as FP32: unlike the
// 16-bit wire nothing is rounded, and twice the bytes cross NVLink.
__global__ void __launch_bounds__(kThreads)
reduce_stat_f32_kernel(const WorkItem* __restrict__ table, uint32_t n_items,
                       const __grid_constant__ PeerIn peers, float unscale_arg,
                       const rlcu_scaler_state* scaler, rlcu_stat* out, float* partials,
                       unsigned int* counter) {
    __shared__ float warp_sums[kThreads / 32];
    __shared__ bool is_last;
    float unscale = unscale_arg;
    if (scaler) {
        const float mul = scaler->grad_mul == 0.0f ? 1.0f : scaler->grad_mul;
        unscale = __fmul_rn(mul, __fdiv_rn(1.0f, scaler->scale));
    }
    const int n = peers.n;
    const float* local_base = reinterpret_cast<const float*>(peers.local_base);
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float probe = 0.0f;
    for (uint32_t idx = blockIdx.x; idx < n_items; idx += gridDim.x) {
        const WorkItem* wi = table + idx;
        const uint4 a = __ldg(reinterpret_cast<const uint4*>(wi));        // p, g
        const uint4 d = __ldg(reinterpret_cast<const uint4*>(wi) + 2);    // master, count, wd
        const uint4 e = __ldg(reinterpret_cast<const uint4*>(wi) + 3);    // flags
        float* g = reinterpret_cast<float*>(((uint64_t)a.w << 32) | a.z);
        const uint32_t count = d.z;
        const uint32_t fl = e.x;
        if (fl & RLCU_TENSOR_GRAD_ZERO) continue;
        const ptrdiff_t base_off = g - local_base;
        const uint32_t quads = (fl & kItemVec16) ? count / 4 : 0;
        // two 16-byte vectors per rank in flight per thread
        uint32_t q = threadIdx.x;
        for (; q + kThreads < quads; q += 2 * kThreads) {
            float4 x0[kMaxWorld], x1[kMaxWorld];
#pragma unroll
            for (int j = 0; j < kMaxWorld; j++) {
                if (j < n) {
                    const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(peers.base[j]) + base_off);
                    x0[j] = __ldcs(src + q);
                    x1[j] = __ldcs(src + q + kThreads);
                }
            }
            float4 s0 = x0[0], s1 = x1[0];
#pragma unroll
            for (int j = 1; j < kMaxWorld; j++) {
                if (j < n) {
                    s0.x = __fadd_rn(s0.x, x0[j].x); s0.y = __fadd_rn(s0.y, x0[j].y);
                    s0.z = __fadd_rn(s0.z, x0[j].z); s0.w = __fadd_rn(s0.w, x0[j].w);
                    s1.x = __fadd_rn(s1.x, x1[j].x); s1.y = __fadd_rn(s1.y, x1[j].y);
                    s1.z = __fadd_rn(s1.z, x1[j].z); s1.w = __fadd_rn(s1.w, x1[j].w);
                }
            }
            reinterpret_cast<float4*>(g)[q] = s0;
            reinterpret_cast<float4*>(g)[q + kThreads] = s1;
            const float v[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
            for (int k = 0; k < 8; k++) {
                probe = __fmaf_rn(v[k], 0.0f, probe);
                const float t = v[k] * unscale;
                acc[k & 3] = fmaf(t, t, acc[k & 3]);
            }
        }
        for (; q < quads; q += kThreads) {
            float4 s0 = __ldcs(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(peers.base[0]) + base_off) + q);
            for (int j = 1; j < n; j++) {
                const float4 x = __ldcs(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(peers.base[j]) + base_off) + q);
                s0.x = __fadd_rn(s0.x, x.x); s0.y = __fadd_rn(s0.y, x.y);
                s0.z = __fadd_rn(s0.z, x.z); s0.w = __fadd_rn(s0.w, x.w);
            }
            reinterpret_cast<float4*>(g)[q] = s0;
            const float v[4] = {s0.x, s0.y, s0.z, s0.w};
#pragma unroll
            for (int k = 0; k < 4; k++) {
                probe = __fmaf_rn(v[k], 0.0f, probe);
                const float t = v[k] * unscale;
                acc[k] = fmaf(t, t, acc[k]);
            }
        }
        for (uint32_t i = quads * 4 + threadIdx.x; i < count; i += kThreads) {
            float sum = reinterpret_cast<const float*>(peers.base[0])[base_off + i];
            for (int j = 1; j < n; j++) sum = __fadd_rn(sum, reinterpret_cast<const float*>(peers.base[j])[base_off + i]);
            g[i] = sum;
            probe = __fmaf_rn(sum, 0.0f, probe);
            const float t = sum * unscale;
            acc[0] = fmaf(t, t, acc[0]);
        }
    }
    float mine = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    if (isnan(probe)) mine = __int_as_float(0x7FC00000);
    const float block_total = block_sum(mine, warp_sums);
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = block_total;
        __threadfence();
        is_last = (atomicAdd(counter, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (threadIdx.x < 32) {
        double s = 0.0;
        for (uint32_t i = threadIdx.x; i < gridDim.x; i += 32) s += (double)__ldcg(partials + i);
#pragma unroll
        for (int mask = 16; mask >= 1; mask >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, mask);
        if (threadIdx.x == 0) {
            *counter = 0;
            out->sum_sq = s;
        }
    }
}

// ---------------------------------------------------------------------------
// reduce-scatter + statistics with the peers' gradients fetched by the bulk-copy engine
// ---------------------------------------------------------------------------
// Same result as reduce_stat_kernel, bit for bit in the reduced gradients (FP32 sum in rank
// order, one rounding).  One CTA per SM: a producer thread keeps kRbDepth tiles in flight,
// each tile being kRbTile consecutive elements fetched from every rank's pool with one
// cp.async.bulk per rank (plain bulk loads from peer-mapped memory, no multicast), and
// kBulkThreads consumer threads add the ranks' copies out of shared memory.  Large requests
// from the copy engine use the links better than per-thread loads do.
constexpr int kRbTile = 2048;                          // elements per rank per stage
constexpr int kRbTileBytes = kRbTile * 2;
constexpr int kRbStageBytes = kMaxWorld * kRbTileBytes;   // 32 KB: every rank's copy of one tile
constexpr int kRbStages = 6;
constexpr int kRbDepth = kRbStages - 1;
constexpr int kRbSmemBytes = kRbStages * kRbStageBytes;
constexpr int kRbTilesPerItem = kChunk / kRbTile;
static_assert(kRbTile == kBulkThreads * 4 && kChunk % kRbTile == 0, "tile geometry");

__device__ __forceinline__ bool reduce_bulk_eligible(uint32_t count, uint32_t fl) {
    return count == (uint32_t)kChunk && (fl & kItemVec16) && !(fl & RLCU_TENSOR_GRAD_ZERO);
}

// Items the bulk path does not take (ragged tails, unaligned tensors): per-thread loads, the
// ranks one after the other.  Rare, so simple.
__device__ __forceinline__ void reduce_item_simple(const PeerIn& peers, __half* g, uint32_t count, uint32_t fl,
                                                   float unscale, float (&acc)[4], float& probe, int threads) {
    const int n = peers.n;
    const bool bf = (fl & kItemBF16) != 0;
    const ptrdiff_t base_off = g - peers.local_base;
    const uint32_t groups = (fl & kItemVec16) ? count / kGroup : 0;
    for (uint32_t grp = threadIdx.x; grp < groups; grp += threads) {
        const ptrdiff_t off = base_off + (ptrdiff_t)grp * kGroup;
        F8 sum = x8_to_f8(ld_h8(peers.base[0] + off), bf);
        for (int j = 1; j < n; j++) add_h8(ld_h8(peers.base[j] + off), sum, bf);
        const uint4 r = f8_to_x8(sum, bf);
        *reinterpret_cast<uint4*>(g + (size_t)grp * kGroup) = r;
        square_accumulate(x8_to_f8(r, bf), unscale, acc, probe);
    }
    for (uint32_t i = groups * kGroup + threadIdx.x; i < count; i += threads) {
        float s = x_to_f(__half_as_ushort(peers.base[0][base_off + i]), bf);
        for (int j = 1; j < n; j++) s = __fadd_rn(s, x_to_f(__half_as_ushort(peers.base[j][base_off + i]), bf));
        const __half r = __ushort_as_half(f_to_x(s, bf));
        g[i] = r;
        const float raw = x_to_f(__half_as_ushort(r), bf);
        probe = __fmaf_rn(raw, 0.0f, probe);
        const float x = raw * unscale;
        acc[0] = fmaf(x, x, acc[0]);
    }
}

__global__ void __launch_bounds__(kBulkThreads + 32, 1)
reduce_stat_bulk_kernel(const WorkItem* __restrict__ table, uint32_t n_items,
                        const __grid_constant__ PeerIn peers, float unscale_arg,
                        const rlcu_scaler_state* scaler, rlcu_stat* out, float* partials,
                        unsigned int* counter, unsigned int* error_word) {
    extern __shared__ __align__(128) unsigned char ring[];
    __shared__ __align__(8) unsigned long long full_bar[kRbStages];
    __shared__ __align__(8) unsigned long long empty_bar[kRbStages];
    __shared__ float warp_sums[(kBulkThreads + 32) / 32];
    __shared__ bool is_last;
    float unscale = unscale_arg;
    if (scaler) {
        const float mul = scaler->grad_mul == 0.0f ? 1.0f : scaler->grad_mul;
        unscale = __fmul_rn(mul, __fdiv_rn(1.0f, scaler->scale));
    }
    const int n = peers.n;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kRbStages; s++) {
            mbar_init(smem_u32(&full_bar[s]), 1);                    // the producer's expect_tx
            mbar_init(smem_u32(&empty_bar[s]), kBulkThreads / 32);   // one arrival per consumer warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    float probe = 0.0f;
    if (threadIdx.x >= kBulkThreads) {
        // ---------------- producer: one thread issues every bulk load ----------------
        if (threadIdx.x == kBulkThreads) {
            uint32_t issued = 0;
            bool bail = false;
            for (uint32_t idx = blockIdx.x; idx < n_items && !bail; idx += gridDim.x) {
                const WorkItem* wi = table + idx;
                const uint4 a = __ldg(reinterpret_cast<const uint4*>(wi));
                const uint4 d = __ldg(reinterpret_cast<const uint4*>(wi) + 2);
                const uint4 e = __ldg(reinterpret_cast<const uint4*>(wi) + 3);
                if (!reduce_bulk_eligible(d.z, e.x)) continue;
                const __half* g = reinterpret_cast<const __half*>(((uint64_t)a.w << 32) | a.z);
                const ptrdiff_t base_off = g - peers.local_base;
                for (int sub = 0; sub < kRbTilesPerItem; sub++) {
                    const int stage = issued % kRbStages;
                    // the consumers are done with what this stage held kRbStages tiles ago
                    if (issued >= (uint32_t)kRbStages &&
                        !mbar_wait(smem_u32(&empty_bar[stage]), ((issued / kRbStages) - 1) & 1u)) {
                        bail = true;
                        break;
                    }
                    const uint32_t bar = smem_u32(&full_bar[stage]);
                    const uint32_t dst = smem_u32(ring + (size_t)stage * kRbStageBytes);
                    mbar_expect_tx(bar, (uint32_t)n * kRbTileBytes);
                    for (int j = 0; j < n; j++)
                        bulk_load(dst + j * kRbTileBytes, peers.base[j] + base_off + (ptrdiff_t)sub * kRbTile, kRbTileBytes, bar);
                    issued++;
                }
            }
            if (bail) atomicExch(error_word, 1u);
            // Loads already issued land in this CTA's shared memory whatever the consumers do: the
            // CTA must not end before they have (bounded waits on the stages still filling).
            const uint32_t first = issued > (uint32_t)kRbStages ? issued - kRbStages : 0;
            for (uint32_t t = first; t < issued; t++)
                mbar_wait(smem_u32(&full_bar[t % kRbStages]), (t / kRbStages) & 1u);
        }
    } else {
        // ---------------- consumers ----------------
        uint32_t tiles = 0;
        bool bail = false;
        for (uint32_t idx = blockIdx.x; idx < n_items && !bail; idx += gridDim.x) {
            const WorkItem* wi = table + idx;
            const uint4 a = __ldg(reinterpret_cast<const uint4*>(wi));
            const uint4 d = __ldg(reinterpret_cast<const uint4*>(wi) + 2);
            const uint4 e = __ldg(reinterpret_cast<const uint4*>(wi) + 3);
            __half* g = reinterpret_cast<__half*>(((uint64_t)a.w << 32) | a.z);
            const uint32_t count = d.z, fl = e.x;
            if (fl & RLCU_TENSOR_GRAD_ZERO) continue;
            if (!reduce_bulk_eligible(count, fl)) {
                reduce_item_simple(peers, g, count, fl, unscale, acc, probe, kBulkThreads);
                continue;
            }
            const bool bf = (fl & kItemBF16) != 0;
            for (int sub = 0; sub < kRbTilesPerItem; sub++) {
                const int stage = tiles % kRbStages;
                if (!mbar_wait(smem_u32(&full_bar[stage]), (tiles / kRbStages) & 1u)) {
                    atomicExch(error_word, 1u);       // stop arriving: the producer's wait runs out too
                    bail = true;
                    break;
                }
                const unsigned char* st = ring + (size_t)stage * kRbStageBytes + (size_t)threadIdx.x * 8;
                uint2 x = *reinterpret_cast<const uint2*>(st);
                float s4[4];
                {
                    const uint32_t w[2] = {x.x, x.y};
#pragma unroll
                    for (int k = 0; k < 2; k++) {
                        s4[2 * k] = x_to_f((unsigned short)(w[k] & 0xFFFFu), bf);
                        s4[2 * k + 1] = x_to_f((unsigned short)(w[k] >> 16), bf);
                    }
                }
                for (int j = 1; j < n; j++) {
                    x = *reinterpret_cast<const uint2*>(st + (size_t)j * kRbTileBytes);
                    const uint32_t w[2] = {x.x, x.y};
#pragma unroll
                    for (int k = 0; k < 2; k++) {
                        s4[2 * k] = __fadd_rn(s4[2 * k], x_to_f((unsigned short)(w[k] & 0xFFFFu), bf));
                        s4[2 * k + 1] = __fadd_rn(s4[2 * k + 1], x_to_f((unsigned short)(w[k] >> 16), bf));
                    }
                }
                __syncwarp();
                if ((threadIdx.x & 31) == 0) mbar_arrive(smem_u32(&empty_bar[stage]));
                uint2 r;
                r.x = (uint32_t)f_to_x(s4[0], bf) | ((uint32_t)f_to_x(s4[1], bf) << 16);
                r.y = (uint32_t)f_to_x(s4[2], bf) | ((uint32_t)f_to_x(s4[3], bf) << 16);
                *reinterpret_cast<uint2*>(g + (size_t)sub * kRbTile + (size_t)threadIdx.x * 4) = r;
                const uint32_t rw[2] = {r.x, r.y};
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    const float lo = x_to_f((unsigned short)(rw[k] & 0xFFFFu), bf), hi = x_to_f((unsigned short)(rw[k] >> 16), bf);
                    probe = __fmaf_rn(lo, 0.0f, probe);
                    probe = __fmaf_rn(hi, 0.0f, probe);
                    const float a0 = lo * unscale, a1 = hi * unscale;
                    acc[2 * k] = fmaf(a0, a0, acc[2 * k]);
                    acc[2 * k + 1] = fmaf(a1, a1, acc[2 * k + 1]);
                }
                tiles++;
            }
        }
    }

    // ---------------- the CTA's partial, then the last CTA's total ----------------
    float mine = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    if (isnan(probe)) mine = __int_as_float(0x7FC00000);
#pragma unroll
    for (int mask = 16; mask >= 1; mask >>= 1) mine += __shfl_xor_sync(0xFFFFFFFFu, mine, mask);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int w = 0; w < (kBulkThreads + 32) / 32; w++) total += warp_sums[w];
        partials[blockIdx.x] = total;
        __threadfence();
        is_last = (atomicAdd(counter, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (threadIdx.x < 32) {
        double s = 0.0;
        for (uint32_t i = threadIdx.x; i < gridDim.x; i += 32) s += (double)__ldcg(partials + i);
#pragma unroll
        for (int mask = 16; mask >= 1; mask >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, mask);
        if (threadIdx.x == 0) {
            *counter = 0;
            out->sum_sq = s;      // this rank's share; the host code all-reduces it
        }
    }
}

// Clears share `part` of `parts` of the gradient pool outside the shard (RLCU_STEP_ZERO_GRADS).
// `threads` = how many threads of the CTA (the first ones) take part.
__device__ __forceinline__ void zero_slice(const ZeroSpan& z, uint64_t part, uint64_t parts, uint32_t threads) {
    const uint64_t total = z.a_vecs + z.b_vecs;
    const uint64_t lo = total * part / parts, hi = total * (part + 1) / parts;
    for (uint64_t i = lo + threadIdx.x; i < hi; i += threads)
        __stcs(i < z.a_vecs ? z.a + i : z.b + (i - z.a_vecs), make_uint4(0u, 0u, 0u, 0u));
}

template <bool GF32>
__global__ void __launch_bounds__(kThreads)
adamw_table_peer_kernel(const WorkItem* __restrict__ table, uint32_t n_items, StepConsts c,
                        const rlcu_stat* __restrict__ stat, uint32_t step_flags,
                        const __grid_constant__ PeerOut peers, const __grid_constant__ ZeroSpan zero) {
    GradXform xf;
    const bool clear = (step_flags & RLCU_STEP_ZERO_GRADS) != 0;
    // a skipped (overflowed) step leaves parameters as they are on every rank, so there is
    // nothing to deliver either; stale gradients are still cleared if that was asked for
    if (!resolve_step(stat, step_flags, c, xf)) {
        if (!clear) return;
        clear_gradients(table, n_items);
        zero_slice(zero, blockIdx.x, gridDim.x, kThreads);
        return;
    }
    uint32_t idx = blockIdx.x;
    if (idx >= n_items) return;
    WorkItem next = load_item(table, idx);
    while (true) {
        const WorkItem it = next;
        const uint32_t nidx = idx + gridDim.x;
        if (nidx < n_items) next = load_item(table, nidx);
        process_item<true, GF32>(it, c, xf, peers);
        if (clear) zero_slice(zero, idx, n_items, kThreads);      // spread over the items: rides under the NVLink stores
        if (nidx >= n_items) break;
        idx = nidx;
    }
}

// The same pass with the traffic, the peers' copies included, issued by the bulk-copy engine:
// each finished 4 KB tile of parameters leaves shared memory once per destination.
__global__ void __launch_bounds__(kBulkThreads + 32, 1)
adamw_table_bulk_peer_kernel(const WorkItem* __restrict__ table, uint32_t n_items, StepConsts c,
                             const rlcu_stat* __restrict__ stat, uint32_t step_flags,
                             unsigned int* error_word, const __grid_constant__ PeerOut peers,
                             const __grid_constant__ ZeroSpan zero) {
    bulk_table_body<true>(TableItems{table}, n_items, c, stat, step_flags, error_word, peers);
    // the rest of the gradient pool (RLCU_STEP_ZERO_GRADS): by the consumer threads, after
    // their tiles; the shard's own gradients were cleared tile by tile
    if ((step_flags & RLCU_STEP_ZERO_GRADS) && threadIdx.x < kBulkThreads) zero_slice(zero, blockIdx.x, gridDim.x, kBulkThreads);
}

struct Geometry {
    int sms = 0, occ_reduce[5] = {0, 0, 0, 0, 0}, occ_update = 0;   // reduce: generic, 1, 2, 4, 8 ranks
    int occ_update_gf32 = 0, occ_reduce_f32 = 0;
};

int geometry(Geometry* out) {
    static Geometry cache[64];
    static bool have[64] = {};
    static std::mutex mu;
    int dev = 0;
    RLCU_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return set_error(RLCU_ERR_UNSUPPORTED, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!have[dev]) {
        Geometry g;
        RLCU_CUDA(cudaDeviceGetAttribute(&g.sms, cudaDevAttrMultiProcessorCount, dev));
        RLCU_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&g.occ_reduce[0], reduce_stat_kernel<0>, kThreads, 0));
        RLCU_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&g.occ_reduce[1], reduce_stat_kernel<1>, kThreads, 0));
        RLCU_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&g.occ_reduce[2], reduce_stat_kernel<2>, kThreads, 0));
        RLCU_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&g.occ_reduce[3], reduce_stat_kernel<4>, kThreads, 0));
        RLCU_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&g.occ_reduce[4], reduce_stat_kernel<8>, kThreads, 0));
        RLCU_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&g.occ_update, adamw_table_peer_kernel<false>, kThreads, 0));
        RLCU_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&g.occ_update_gf32, adamw_table_peer_kernel<true>, kThreads, 0));
        RLCU_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&g.occ_reduce_f32, reduce_stat_f32_kernel, kThreads, 0));
        RLCU_CUDA(cudaFuncSetAttribute(adamw_table_bulk_peer_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kBulkSmemBytes));
        RLCU_CUDA(cudaFuncSetAttribute(reduce_stat_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kRbSmemBytes));
        for (int occ : g.occ_reduce)
            if (occ < 1) return set_error(RLCU_ERR_CUDA, "kernel does not fit on an SM");
        if (g.occ_update < 1 || g.occ_update_gf32 < 1 || g.occ_reduce_f32 < 1) return set_error(RLCU_ERR_CUDA, "kernel does not fit on an SM");
        // measurement knobs: cap the resident CTAs per SM of the two exchange kernels
        if (const char* e = getenv("RLCU_P2P_REDUCE_CTAS_PER_SM")) {
            const int cap = atoi(e);
            for (int& occ : g.occ_reduce)
                if (cap >= 1 && cap < occ) occ = cap;
        }
        if (const char* e = getenv("RLCU_P2P_UPDATE_CTAS_PER_SM")) {
            const int cap = atoi(e);
            if (cap >= 1 && cap < g.occ_update) g.occ_update = cap;
        }
        cache[dev] = g;
        have[dev] = true;
    }
    *out = cache[dev];
    return RLCU_OK;
}

}  // namespace

int launch_reduce_stat(rlcu_tensor_list* list, const PeerIn& peers, float unscale,
                       const rlcu_scaler_state* scaler, rlcu_stat* stat, bool bulk, cudaStream_t stream) {
    if (!list || !stat) return set_error(RLCU_ERR_INVALID, "null list or stat");
    if (peers.n < 1 || peers.n > kMaxWorld) return set_error(RLCU_ERR_INVALID, "world size %d not supported", peers.n);
    Geometry g;
    const int rc = geometry(&g);
    if (rc) return rc;
    if (bulk) {
        int grid = g.sms;
        if (grid > list->grid_stat) grid = list->grid_stat;
        if ((uint32_t)grid > list->n_items) grid = list->n_items ? (int)list->n_items : 1;
        reduce_stat_bulk_kernel<<<grid, kBulkThreads + 32, kRbSmemBytes, stream>>>(
            list->d_items, list->n_items, peers, unscale, scaler, stat, list->d_partials, list->d_counter,
            list->d_counter + 16);
        RLCU_CUDA(cudaGetLastError());
        return RLCU_OK;
    }
    // the scratch of the list was sized for the statistics kernel's grid; stay within it
    const int variant = peers.n == 1 ? 1 : peers.n == 2 ? 2 : peers.n == 4 ? 3 : peers.n == 8 ? 4 : 0;
    int grid = g.sms * g.occ_reduce[variant];
    if (grid > list->grid_stat) grid = list->grid_stat;
    if ((uint32_t)grid > list->n_items) grid = list->n_items ? (int)list->n_items : 1;
#define RLCU_LAUNCH_REDUCE(W)                                                                   \
    reduce_stat_kernel<W><<<grid, kThreads, 0, stream>>>(list->d_items, list->n_items, peers,   \
                                                         unscale, scaler, stat, list->d_partials, \
                                                         list->d_counter)
    switch (peers.n) {
        case 1: RLCU_LAUNCH_REDUCE(1); break;
        case 2: RLCU_LAUNCH_REDUCE(2); break;
        case 4: RLCU_LAUNCH_REDUCE(4); break;
        case 8: RLCU_LAUNCH_REDUCE(8); break;
        default: RLCU_LAUNCH_REDUCE(0); break;
    }
#undef RLCU_LAUNCH_REDUCE
    RLCU_CUDA(cudaGetLastError());
    return RLCU_OK;
}

int launch_reduce_stat_f32(rlcu_tensor_list* list, const PeerIn& peers, float unscale,
                           const rlcu_scaler_state* scaler, rlcu_stat* stat, cudaStream_t stream) {
    if (!list || !stat) return set_error(RLCU_ERR_INVALID, "null list or stat");
    if (peers.n < 1 || peers.n > kMaxWorld) return set_error(RLCU_ERR_INVALID, "world size %d not supported", peers.n);
    Geometry g;
    const int rc = geometry(&g);
    if (rc) return rc;
    int grid = g.sms * g.occ_reduce_f32;
    if (grid > list->grid_stat) grid = list->grid_stat;
    if ((uint32_t)grid > list->n_items) grid = list->n_items ? (int)list->n_items : 1;
    reduce_stat_f32_kernel<<<grid, kThreads, 0, stream>>>(list->d_items, list->n_items, peers, unscale, scaler, stat,
                                                          list->d_partials, list->d_counter);
    RLCU_CUDA(cudaGetLastError());
    return RLCU_OK;
}

int launch_update_peers(rlcu_tensor_list* list, const rlcu_hparams* hp, const rlcu_stat* stat,
                        uint32_t step_flags, const PeerOut& peers, const ZeroSpan& zero, cudaStream_t stream) {
    if (!list || !hp) return set_error(RLCU_ERR_INVALID, "null list or hparams");
    if (peers.n < 0 || peers.n > kMaxPeers) return set_error(RLCU_ERR_INVALID, "%d peers not supported", peers.n);
    if (list->n_items == 0) {
        // a rank whose shard lies wholly in the padding still owns the clearing of its pool
        if ((step_flags & RLCU_STEP_ZERO_GRADS) && zero.a_vecs + zero.b_vecs) {
            RLCU_CUDA(cudaMemsetAsync(zero.a, 0, zero.a_vecs * 16, stream));
            if (zero.b_vecs) RLCU_CUDA(cudaMemsetAsync(zero.b, 0, zero.b_vecs * 16, stream));
        }
        return RLCU_OK;
    }
    Geometry g;
    const int rc = geometry(&g);
    if (rc) return rc;
    int grid = g.sms * g.occ_update;
    if ((uint32_t)grid > list->n_items) grid = (int)list->n_items;
    StepConsts c;
    c.lr = hp->lr; c.b1 = hp->beta1; c.b2 = hp->beta2; c.eps = hp->eps;
    c.bc1_inv = 1.0f / hp->bias_correction1;
    c.bc2_inv = 1.0f / hp->bias_correction2;
    // same choice as the single-GPU update: shards that are mostly FP16 weights with FP32
    // masters go through the bulk-copy kernel unless the caller says otherwise
    if ((step_flags & RLCU_STEP_BULK_COPY) && (step_flags & RLCU_STEP_DIRECT))
        return set_error(RLCU_ERR_INVALID, "RLCU_STEP_BULK_COPY and RLCU_STEP_DIRECT exclude each other");
    if (!(step_flags & RLCU_STEP_DIRECT) && list->prefer_bulk) step_flags |= RLCU_STEP_BULK_COPY;
    step_flags &= ~(uint32_t)RLCU_STEP_DIRECT;
    if (step_flags & RLCU_STEP_BULK_COPY) {
        grid = (uint32_t)g.sms > list->n_items ? (int)list->n_items : g.sms;
        adamw_table_bulk_peer_kernel<<<grid, kBulkThreads + 32, kBulkSmemBytes, stream>>>(
            list->d_items, list->n_items, c, stat, step_flags & ~(uint32_t)RLCU_STEP_BULK_COPY,
            list->d_counter + 16, peers, zero);
        RLCU_CUDA(cudaGetLastError());
        return RLCU_OK;
    }
    if (list->has_grad_f32) {
        grid = g.sms * g.occ_update_gf32;
        if ((uint32_t)grid > list->n_items) grid = (int)list->n_items;
        adamw_table_peer_kernel<true><<<grid, kThreads, 0, stream>>>(list->d_items, list->n_items, c, stat,
                                                                     step_flags, peers, zero);
    } else {
        adamw_table_peer_kernel<false><<<grid, kThreads, 0, stream>>>(list->d_items, list->n_items, c, stat,
                                                                      step_flags, peers, zero);
    }
    RLCU_CUDA(cudaGetLastError());
    return RLCU_OK;
}

}  // namespace rlcu

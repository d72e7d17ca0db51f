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

#include <mutex>

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
            constexpr int UB = WORLD == 8 ? 1 : 2;       // 512 wide groups per item, 2 per thread
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
        for (uint32_t grp = threadIdx.x; grp < groups; grp += kThreads)
            reduce_groups<WORLD, 1>(peers, base_off + (ptrdiff_t)grp * kGroup, g + (size_t)grp * kGroup, 0, unscale, acc, bf, probe);
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

__global__ void __launch_bounds__(kThreads)
adamw_table_peer_kernel(const WorkItem* __restrict__ table, uint32_t n_items, StepConsts c,
                        const rlcu_stat* __restrict__ stat, uint32_t step_flags,
                        const __grid_constant__ PeerOut peers) {
    GradXform xf;
    // a skipped (overflowed) step leaves parameters as they are on every rank, so
    // there is nothing to deliver either
    if (!resolve_step(stat, step_flags, c, xf)) return;
    uint32_t idx = blockIdx.x;
    if (idx >= n_items) return;
    WorkItem next = load_item(table, idx);
    while (true) {
        const WorkItem it = next;
        const uint32_t nidx = idx + gridDim.x;
        if (nidx < n_items) next = load_item(table, nidx);
        process_item<true>(it, c, xf, peers);
        if (nidx >= n_items) break;
        idx = nidx;
    }
}

struct Geometry {
    int sms = 0, occ_reduce[5] = {0, 0, 0, 0, 0}, occ_update = 0;   // reduce: generic, 1, 2, 4, 8 ranks
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
        RLCU_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&g.occ_update, adamw_table_peer_kernel, kThreads, 0));
        for (int occ : g.occ_reduce)
            if (occ < 1) return set_error(RLCU_ERR_CUDA, "kernel does not fit on an SM");
        if (g.occ_update < 1) return set_error(RLCU_ERR_CUDA, "kernel does not fit on an SM");
        cache[dev] = g;
        have[dev] = true;
    }
    *out = cache[dev];
    return RLCU_OK;
}

}  // namespace

int launch_reduce_stat(rlcu_tensor_list* list, const PeerIn& peers, float unscale,
                       const rlcu_scaler_state* scaler, rlcu_stat* stat, cudaStream_t stream) {
    if (!list || !stat) return set_error(RLCU_ERR_INVALID, "null list or stat");
    if (peers.n < 1 || peers.n > kMaxWorld) return set_error(RLCU_ERR_INVALID, "world size %d not supported", peers.n);
    Geometry g;
    const int rc = geometry(&g);
    if (rc) return rc;
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

int launch_update_peers(rlcu_tensor_list* list, const rlcu_hparams* hp, const rlcu_stat* stat,
                        uint32_t step_flags, const PeerOut& peers, cudaStream_t stream) {
    if (!list || !hp) return set_error(RLCU_ERR_INVALID, "null list or hparams");
    if (peers.n < 0 || peers.n > kMaxPeers) return set_error(RLCU_ERR_INVALID, "%d peers not supported", peers.n);
    if (list->n_items == 0) return RLCU_OK;
    Geometry g;
    const int rc = geometry(&g);
    if (rc) return rc;
    int grid = g.sms * g.occ_update;
    if ((uint32_t)grid > list->n_items) grid = (int)list->n_items;
    StepConsts c;
    c.lr = hp->lr; c.b1 = hp->beta1; c.b2 = hp->beta2; c.eps = hp->eps;
    c.bc1_inv = 1.0f / hp->bias_correction1;
    c.bc2_inv = 1.0f / hp->bias_correction2;
    adamw_table_peer_kernel<<<grid, kThreads, 0, stream>>>(list->d_items, list->n_items, c, stat,
                                                           step_flags, peers);
    RLCU_CUDA(cudaGetLastError());
    return RLCU_OK;
}

}  // namespace rlcu

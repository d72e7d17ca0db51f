// The update pass with its HBM traffic moved by the bulk-copy engine (TMA, 1-D
// cp.async.bulk) through a ring of shared-memory stages instead of per-thread
// loads and stores: one elected thread keeps several tiles of p/g/m/v in flight
// per SM, the other threads only touch shared memory.
//
// Only full, 16-byte aligned FP16 work items (FP16 or FP32 gradients, with or without
// a master copy) take this route; everything else in the table (partial items, FP32
// and bfloat16 tensors, statistics-only entries) is handled by the direct code of
// adamw_update.cuh inside the same kernel.
//
// Waits on the load barriers are bounded: when a wait gives up the CTA records it
// in the error word, drains its own copies (again bounded) and returns.
#pragma once

#include "adamw_update.cuh"

namespace rlcu {

constexpr int kBulkThreads = 512;
constexpr int kBulkTile = 2048;                       // elements per stage
constexpr int kBulkTilesPerItem = kChunk / kBulkTile;
constexpr int kBulkStages = 6;
constexpr int kBulkDepth = kBulkStages - 2;           // tiles loading ahead of the one in use
constexpr int kBulkStageBytes = 36864;                // [m 8K][v 8K][master 8K][p 4K][g 8K: FP16 uses the first 4K]
constexpr int kBulkSmemBytes = kBulkStages * kBulkStageBytes;
constexpr uint32_t kBulkWaitTries = 1u << 18;
constexpr int kBulkPendingCap = 1024;                 // items per CTA remembered for the direct code
static_assert(kChunk % kBulkTile == 0 && kBulkTile == kBulkThreads * 4, "tile geometry");

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}

// Bounded wait for the phase with the given parity.  false = gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t tries = kBulkWaitTries) {
    for (uint32_t i = 0; i < tries; i++) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

// global -> shared, completion counted in bytes on the stage's barrier
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// shared -> global, tracked by the issuing thread's bulk groups
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                 :: "l"(dst), "r"(src_smem), "r"(bytes) : "memory");
}

__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ bool bulk_eligible(const WorkItem& it) {
    const uint32_t kind = it.flags & kItemKindMask;
    return it.count == (uint32_t)kChunk && (it.flags & kItemVec16) && kind != kItemKindF32 &&
           !(it.flags & (RLCU_TENSOR_NORM_ONLY | kItemBF16));
}

// Issues the loads of one tile into a stage (one thread).
__device__ __forceinline__ void bulk_issue_tile(const WorkItem& it, int sub, unsigned char* stage, uint32_t bar) {
    const size_t e = (size_t)sub * kBulkTile;
    const bool master = (it.flags & kItemKindMask) == kItemKindF16Master;
    const bool zero = (it.flags & RLCU_TENSOR_GRAD_ZERO) != 0;
    const uint32_t gbytes = (it.flags & kItemGradF32) ? kBulkTile * 4u : kBulkTile * 2u;
    const uint32_t bytes = 2u * kBulkTile * 4u + (master ? kBulkTile * 4u : kBulkTile * 2u) + (zero ? 0u : gbytes);
    mbar_expect_tx(bar, bytes);
    const uint32_t s = smem_u32(stage);
    bulk_load(s, it.m + e, kBulkTile * 4, bar);
    bulk_load(s + 8192, it.v + e, kBulkTile * 4, bar);
    if (master) bulk_load(s + 16384, it.master + e, kBulkTile * 4, bar);
    else bulk_load(s + 24576, static_cast<const __half*>(it.p) + e, kBulkTile * 2, bar);
    if (!zero) bulk_load(s + 28672, static_cast<const char*>(it.g) + e * (gbytes / kBulkTile), gbytes, bar);
}

// Issues the stores of one finished tile (one thread) and commits them as one group.
template <bool PEERS>
__device__ __forceinline__ void bulk_store_tile(const WorkItem& it, int sub, unsigned char* stage, bool zero_grads,
                                                const PeerOut& peers) {
    const size_t e = (size_t)sub * kBulkTile;
    const bool master = (it.flags & kItemKindMask) == kItemKindF16Master;
    const uint32_t s = smem_u32(stage);
    bulk_store(it.m + e, s, kBulkTile * 4);
    bulk_store(it.v + e, s + 8192, kBulkTile * 4);
    if (master) bulk_store(it.master + e, s + 16384, kBulkTile * 4);
    bulk_store(static_cast<__half*>(it.p) + e, s + 24576, kBulkTile * 2);
    if constexpr (PEERS) {
        // the same 4 KB of new parameters into every peer's pool, over NVLink
        const ptrdiff_t off = (static_cast<__half*>(it.p) + e) - peers.local_base;
        for (int j = 0; j < peers.n; j++) bulk_store(peers.base[j] + off, s + 24576, kBulkTile * 2);
    }
    if (zero_grads && !(it.flags & RLCU_TENSOR_GRAD_ZERO)) {
        const uint32_t gbytes = (it.flags & kItemGradF32) ? kBulkTile * 4u : kBulkTile * 2u;
        bulk_store(const_cast<char*>(static_cast<const char*>(it.g)) + e * (gbytes / kBulkTile), s + 28672, gbytes);
    }
    bulk_commit();
}

// Four elements of the tile per thread, in place in shared memory.
__device__ __forceinline__ void bulk_compute_tile(const WorkItem& it, unsigned char* stage, const StepConsts& c,
                                                  const GradXform& xf) {
    const bool master = (it.flags & kItemKindMask) == kItemKindF16Master;
    const bool zero = (it.flags & RLCU_TENSOR_GRAD_ZERO) != 0;
    const bool gf32 = (it.flags & kItemGradF32) != 0;
    const float decay = decay_factor(c.lr, it.wd);
    const int t = threadIdx.x;
    float4* sm = reinterpret_cast<float4*>(stage) + t;
    float4* sv = reinterpret_cast<float4*>(stage + 8192) + t;
    float4* sw = reinterpret_cast<float4*>(stage + 16384) + t;
    uint2* sp = reinterpret_cast<uint2*>(stage + 24576) + t;
    uint2* sg = reinterpret_cast<uint2*>(stage + 28672) + t;
    float4 m = *sm, v = *sv;
    float w[4], g[4];
    if (master) {
        const float4 x = *sw;
        w[0] = x.x; w[1] = x.y; w[2] = x.z; w[3] = x.w;
    } else {
        const uint2 x = *sp;
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&x.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&x.y));
        w[0] = a.x; w[1] = a.y; w[2] = b.x; w[3] = b.y;
    }
    float4* sg32 = reinterpret_cast<float4*>(stage + 28672) + t;
    if (zero) {
        g[0] = g[1] = g[2] = g[3] = 0.0f;
    } else if (gf32) {
        const float4 x = *sg32;
        g[0] = x.x; g[1] = x.y; g[2] = x.z; g[3] = x.w;
    } else {
        const uint2 x = *sg;
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&x.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&x.y));
        g[0] = a.x; g[1] = a.y; g[2] = b.x; g[3] = b.y;
    }
    float mm[4] = {m.x, m.y, m.z, m.w}, vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float x = __fmul_rn(g[i], xf.coef);
        if (xf.round_half && !gf32) x = round_through_half(x);     // FP32 gradients are scaled in FP32 (trainer.h:144)
        w[i] = adamw_element(w[i], x, mm[i], vv[i], c, decay);
    }
    *sm = make_float4(mm[0], mm[1], mm[2], mm[3]);
    *sv = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (master) *sw = make_float4(w[0], w[1], w[2], w[3]);
    __half2 lo = __floats2half2_rn(w[0], w[1]), hi = __floats2half2_rn(w[2], w[3]);
    uint2 out;
    out.x = *reinterpret_cast<uint32_t*>(&lo);
    out.y = *reinterpret_cast<uint32_t*>(&hi);
    *sp = out;
    if (xf.zero_grads && !zero) {
        if (gf32) *sg32 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        else *sg = make_uint2(0u, 0u);
    }
}

// Body of the bulk-copy update kernels (launch: kBulkThreads + 32 threads, one CTA per SM,
// kBulkSmemBytes of dynamic shared memory): kBulkThreads consumer threads do the arithmetic
// in shared memory while one thread of the extra warp drives cp.async.bulk loads and stores
// through a ring of kBulkStages stages.  Producer and consumers meet only at the stages'
// full/empty barriers.  With PEERS every finished tile of FP16 parameters is also stored,
// by the same engine, at the same offset of each peer GPU's parameter pool (the all-gather
// of the sharded step); a skipped step then stores nothing anywhere.
// Where the work items come from: a table in device memory (tensor lists), or one tensor
// cut into kChunk-element items on the fly (the single-tensor entry points).
using TableItems = TableRef;
struct FlatItems {
    WorkItem base;      // pointers at the tensor's first element; flags carry kind and alignment
    uint64_t n;         // elements in the tensor
    __device__ __forceinline__ WorkItem get(uint32_t idx) const {
        const uint64_t off = (uint64_t)idx * kChunk;
        WorkItem it = base;
        it.count = (uint32_t)((n - off) < (uint64_t)kChunk ? (n - off) : (uint64_t)kChunk);
        it.m += off;
        it.v += off;
        if (it.master) it.master += off;
        const size_t esz = (base.flags & kItemKindMask) == kItemKindF32 ? 4 : 2;
        it.p = static_cast<char*>(base.p) + off * esz;
        it.g = static_cast<const char*>(base.g) + off * esz;
        return it;
    }
};

template <bool PEERS, class Items>
__device__ __forceinline__ void bulk_table_body(const Items items, uint32_t n_items, StepConsts c,
                                                const rlcu_stat* __restrict__ stat, uint32_t step_flags,
                                                unsigned int* error_word, const PeerOut& peers) {
    extern __shared__ __align__(128) unsigned char ring[];
    __shared__ __align__(8) unsigned long long full_bar[kBulkStages];
    __shared__ __align__(8) unsigned long long empty_bar[kBulkStages];
    __shared__ uint32_t pending[kBulkPendingCap];     // items left to the direct code
    GradXform xf;
    if (!resolve_step(stat, step_flags, c, xf)) {
        if (!(step_flags & RLCU_STEP_ZERO_GRADS)) return;
        clear_gradients(items, n_items);
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < kBulkStages; s++) {
            mbar_init(smem_u32(&full_bar[s]), 1);                    // the producer's expect_tx
            mbar_init(smem_u32(&empty_bar[s]), kBulkThreads / 32);   // one arrival per consumer warp
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (threadIdx.x >= kBulkThreads) {
        // ---------------- producer warp: one thread issues every bulk copy ----------------
        if (threadIdx.x != kBulkThreads) return;
        uint32_t load_item_idx = blockIdx.x, loaded = 0;     // next tile to load
        uint32_t store_item_idx = blockIdx.x, stored = 0;    // next tile to store
        int load_sub = 0, store_sub = 0;
        WorkItem lit, sit;
        bool have_l = false, have_s = false, bail = false;
        auto next_eligible = [&](uint32_t& idx, WorkItem& it, bool& have) {
            while (!have && idx < n_items) {
                it = items.get(idx);
                if (bulk_eligible(it)) have = true;
                else idx += gridDim.x;
            }
            return have;
        };
        auto load_upto = [&](uint32_t upto) {
            while (loaded < upto && next_eligible(load_item_idx, lit, have_l)) {
                const int stage = loaded % kBulkStages;
                bulk_issue_tile(lit, load_sub, ring + (size_t)stage * kBulkStageBytes, smem_u32(&full_bar[stage]));
                loaded++;
                if (++load_sub == kBulkTilesPerItem) {
                    load_sub = 0;
                    load_item_idx += gridDim.x;
                    have_l = false;
                }
            }
        };
        load_upto(kBulkDepth);
        while (next_eligible(store_item_idx, sit, have_s)) {
            const int stage = stored % kBulkStages;
            // the consumers have finished tile `stored` in this stage
            if (!mbar_wait(smem_u32(&empty_bar[stage]), (stored / kBulkStages) & 1u)) {
                bail = true;
                break;
            }
            bulk_store_tile<PEERS>(sit, store_sub, ring + (size_t)stage * kBulkStageBytes, xf.zero_grads, peers);
            stored++;
            if (++store_sub == kBulkTilesPerItem) {
                store_sub = 0;
                store_item_idx += gridDim.x;
                have_s = false;
            }
            bulk_wait_read<1>();                 // the stage refilled next was stored two tiles ago
            load_upto(stored + kBulkDepth);
        }
        if (bail) {
            atomicExch(error_word, 1u);
            // loads already issued still land in this CTA's shared memory: wait for them (bounded)
            for (uint32_t t = stored; t < loaded; t++)
                mbar_wait(smem_u32(&full_bar[t % kBulkStages]), (t / kBulkStages) & 1u);
        }
        bulk_wait_all();
        return;
    }

    // ---------------- consumer warps ----------------
    // The items that go through the ring first; the ones that do not (partial items, FP32
    // tensors) are noted on the way and run afterwards with the direct code, which keeps that
    // code's registers out of the tile loop.
    uint32_t tiles = 0, n_pending = 0;       // n_pending is the same in every consumer thread
    bool ok = true;
    for (uint32_t idx = blockIdx.x; idx < n_items && ok; idx += gridDim.x) {
        const WorkItem it = items.get(idx);
        if (!bulk_eligible(it)) {
            if (threadIdx.x == 0 && n_pending < (uint32_t)kBulkPendingCap) pending[n_pending] = idx;
            n_pending++;
            continue;
        }
        for (int sub = 0; sub < kBulkTilesPerItem; sub++) {
            const int stage = tiles % kBulkStages;
            if (!mbar_wait(smem_u32(&full_bar[stage]), (tiles / kBulkStages) & 1u)) {
                atomicExch(error_word, 1u);      // stop arriving: the producer's wait runs out too
                ok = false;
                break;
            }
            bulk_compute_tile(it, ring + (size_t)stage * kBulkStageBytes, c, xf);
            fence_async_smem();                  // results visible to the bulk store
            __syncwarp();
            if ((threadIdx.x & 31) == 0) mbar_arrive(smem_u32(&empty_bar[stage]));
            tiles++;
        }
    }
    // consumer-only barrier: the list written by thread 0 is visible to the others
    asm volatile("bar.sync 1, %0;" :: "n"(kBulkThreads) : "memory");
    if (!ok || threadIdx.x >= kThreads) return;      // the direct code is written for kThreads threads
    const uint32_t listed = n_pending < (uint32_t)kBulkPendingCap ? n_pending : (uint32_t)kBulkPendingCap;
    for (uint32_t i = 0; i < listed; i++) process_item<PEERS, true>(items.get(pending[i]), c, xf, peers);
    if (n_pending > listed) {
        // more than the list holds: walk the rest of this CTA's items again
        for (uint32_t idx = pending[listed - 1] + gridDim.x; idx < n_items; idx += gridDim.x) {
            const WorkItem it = items.get(idx);
            if (!bulk_eligible(it)) process_item<PEERS, true>(it, c, xf, peers);
        }
    }
}

}  // namespace rlcu

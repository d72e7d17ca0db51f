// The update pass as device code shared by the single-GPU kernels and the
// sharded (peer-writing) kernel: one work item = at most kChunk consecutive
// elements of one tensor.
#pragma once

#include "adamw_device.cuh"
#include "rlcu_adamw.h"

namespace rlcu {

struct GradXform {
    float coef;        // multiply every gradient by this
    bool round_half;   // then round FP16 gradients through binary16
    bool zero_grads;   // write zeros over the gradient after reading it
};

// Where the sharded step also delivers each updated FP16 parameter: the same
// offset in every peer GPU's parameter pool (plain stores through peer-mapped
// pointers; the all-gather of the step happens inside the update kernel).
constexpr int kMaxPeers = 7;
struct PeerOut {
    int n;                         // number of peers (0..kMaxPeers)
    const __half* local_base;      // this GPU's parameter pool
    __half* base[kMaxPeers];       // peers' parameter pools, mapped into this process
};

// 256-bit peer stores (lane pairs merged by shuffle) were measured on 4 GPUs and gave
// nothing over these 128-bit ones (640 GB/s per direction either way), so they are not used.
template <bool PEERS>
__device__ __forceinline__ void store_param_h8(__half* dst, uint4 val, const PeerOut& peers) {
    st_h8(dst, val);
    if constexpr (PEERS) {
        const ptrdiff_t off = dst - peers.local_base;
        for (int j = 0; j < peers.n; j++) *reinterpret_cast<uint4*>(peers.base[j] + off) = val;
    }
}

template <bool PEERS>
__device__ __forceinline__ void store_param_h(__half* dst, __half val, const PeerOut& peers) {
    *dst = val;
    if constexpr (PEERS) {
        const ptrdiff_t off = dst - peers.local_base;
        for (int j = 0; j < peers.n; j++) peers.base[j][off] = val;
    }
}

template <bool ROUND>
__device__ __forceinline__ float xform_h(float g, float coef, bool bf) {
    float x = __fmul_rn(g, coef);
    if constexpr (ROUND) x = round_through_16(x, bf);
    return x;
}

__device__ __forceinline__ F8 f8_zero() {
    F8 z;
#pragma unroll
    for (int i = 0; i < 8; i++) z.a[i] = 0.0f;
    return z;
}

// One group of 8 FP16 elements with every access vectorised.
//   KIND 0: weight read from the FP16 parameter; KIND 1: from the FP32 master.
//   GF32: the gradient is FP32 (16-bit parameter whose gradient was accumulated in FP32);
//         it is scaled in FP32 like RL.cu's scale_float_kernel (trainer.h:142-145), never
//         rounded through 16 bits.
template <int KIND, bool V32, bool ROUND, int U, bool PEERS, bool GF32 = false>
__device__ __forceinline__ void f16_groups(const WorkItem& it, int first_group, int group_stride,
                                           const StepConsts& c, float decay, const GradXform& xf,
                                           const PeerOut& peers) {
    static_assert(!(GF32 && ROUND), "FP32 gradients are not rounded through 16 bits");
    uint4 gw[U], pw[U];
    F8 gf[U], m[U], v[U], w[U];
    const bool zero = (it.flags & RLCU_TENSOR_GRAD_ZERO) != 0;
    const bool bf = (it.flags & kItemBF16) != 0;
#pragma unroll
    for (int u = 0; u < U; u++) {
        const size_t e = (size_t)(first_group + u * group_stride) * kGroup;
        if constexpr (GF32) gf[u] = zero ? f8_zero() : ld_f8<V32>(static_cast<const float*>(it.g) + e);
        else gw[u] = zero ? make_uint4(0, 0, 0, 0) : ld_h8(static_cast<const __half*>(it.g) + e);
        if constexpr (KIND == 0) pw[u] = ld_h8(static_cast<const __half*>(it.p) + e);
        else w[u] = ld_f8<V32>(it.master + e);
        m[u] = ld_f8<V32>(it.m + e);
        v[u] = ld_f8<V32>(it.v + e);
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
        const size_t e = (size_t)(first_group + u * group_stride) * kGroup;
        F8 g;
        if constexpr (GF32) g = gf[u];
        else g = x8_to_f8(gw[u], bf);
        if constexpr (KIND == 0) w[u] = x8_to_f8(pw[u], bf);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float x;
            if constexpr (GF32) x = __fmul_rn(g.a[i], xf.coef);          // trainer.h:144
            else x = xform_h<ROUND>(g.a[i], xf.coef, bf);
            w[u].a[i] = adamw_element(w[u].a[i], x, m[u].a[i], v[u].a[i], c, decay);
        }
        st_f8<V32>(it.m + e, m[u]);
        st_f8<V32>(it.v + e, v[u]);
        if constexpr (KIND == 1) st_f8<V32>(it.master + e, w[u]);
        store_param_h8<PEERS>(static_cast<__half*>(it.p) + e, f8_to_x8(w[u], bf), peers);
        if (xf.zero_grads && !zero) {
            if constexpr (GF32) st_f8<V32>(const_cast<float*>(static_cast<const float*>(it.g)) + e, f8_zero());
            else st_h8(const_cast<__half*>(static_cast<const __half*>(it.g)) + e, make_uint4(0, 0, 0, 0));
        }
    }
}

template <bool V32, int U>
__device__ __forceinline__ void f32_groups(const WorkItem& it, int first_group, int group_stride,
                                           const StepConsts& c, float decay, const GradXform& xf) {
    F8 g[U], m[U], v[U], w[U];
    const bool zero = (it.flags & RLCU_TENSOR_GRAD_ZERO) != 0;
#pragma unroll
    for (int u = 0; u < U; u++) {
        const size_t e = (size_t)(first_group + u * group_stride) * kGroup;
        if (zero) {
#pragma unroll
            for (int i = 0; i < 8; i++) g[u].a[i] = 0.0f;
        } else {
            g[u] = ld_f8<V32>(static_cast<const float*>(it.g) + e);
        }
        w[u] = ld_f8<V32>(static_cast<const float*>(it.p) + e);
        m[u] = ld_f8<V32>(it.m + e);
        v[u] = ld_f8<V32>(it.v + e);
    }
#pragma unroll
    for (int u = 0; u < U; u++) {
        const size_t e = (size_t)(first_group + u * group_stride) * kGroup;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float x = __fmul_rn(g[u].a[i], xf.coef);   // trainer.h:144
            w[u].a[i] = adamw_element(w[u].a[i], x, m[u].a[i], v[u].a[i], c, decay);
        }
        st_f8<V32>(it.m + e, m[u]);
        st_f8<V32>(it.v + e, v[u]);
        st_f8<V32>(static_cast<float*>(it.p) + e, w[u]);
        if (xf.zero_grads && !zero) {
            F8 z;
#pragma unroll
            for (int i = 0; i < 8; i++) z.a[i] = 0.0f;
            st_f8<V32>(const_cast<float*>(static_cast<const float*>(it.g)) + e, z);
        }
    }
}

// Element-at-a-time path: ragged tails and tensors whose pointers are not
// 16-byte aligned.  Same arithmetic, scalar accesses.
template <bool PEERS>
__device__ __forceinline__ void scalar_range(const WorkItem& it, uint32_t begin, uint32_t end,
                                             const StepConsts& c, float decay, const GradXform& xf,
                                             const PeerOut& peers) {
    const uint32_t kind = it.flags & kItemKindMask;
    const bool zero = (it.flags & RLCU_TENSOR_GRAD_ZERO) != 0;
    for (uint32_t i = begin + threadIdx.x; i < end; i += kThreads) {
        float m = it.m[i], v = it.v[i];
        if (kind == kItemKindF32) {
            float* p = static_cast<float*>(it.p);
            float* g = const_cast<float*>(static_cast<const float*>(it.g));
            const float x = zero ? 0.0f : __fmul_rn(g[i], xf.coef);
            p[i] = adamw_element(p[i], x, m, v, c, decay);
            if (xf.zero_grads && !zero) g[i] = 0.0f;
        } else {
            __half* p = static_cast<__half*>(it.p);
            const bool bf = (it.flags & kItemBF16) != 0;
            float x;
            if (it.flags & kItemGradF32) {
                float* g = const_cast<float*>(static_cast<const float*>(it.g));
                x = zero ? 0.0f : __fmul_rn(g[i], xf.coef);
                if (xf.zero_grads && !zero) g[i] = 0.0f;
            } else {
                __half* g = const_cast<__half*>(static_cast<const __half*>(it.g));
                x = zero ? 0.0f : __fmul_rn(x_to_f(__half_as_ushort(g[i]), bf), xf.coef);
                if (xf.round_half) x = round_through_16(x, bf);
                if (xf.zero_grads && !zero) g[i] = __float2half_rn(0.0f);
            }
            const float w0 = (kind == kItemKindF16Master) ? it.master[i] : x_to_f(__half_as_ushort(p[i]), bf);
            const float w = adamw_element(w0, x, m, v, c, decay);
            if (kind == kItemKindF16Master) it.master[i] = w;
            store_param_h<PEERS>(p + i, __ushort_as_half(f_to_x(w, bf)), peers);
        }
        it.m[i] = m;
        it.v[i] = v;
    }
}

template <int KIND, bool V32, bool ROUND, bool PEERS, bool GF32 = false>
__device__ __forceinline__ void vector_item(const WorkItem& it, const StepConsts& c, float decay,
                                            const GradXform& xf, const PeerOut& peers) {
    const int groups = it.count / kGroup;
    if (it.count == kChunk) {
        // full item: every thread owns kGroupsPerThread groups, loads issued kUnroll groups deep
        constexpr int U = kUnroll;
#pragma unroll
        for (int b = 0; b < kGroupsPerThread / U; b++) {
            const int first = threadIdx.x + b * U * kThreads;
            if constexpr (KIND == 2) f32_groups<V32, U>(it, first, kThreads, c, decay, xf);
            else f16_groups<KIND, V32, ROUND, U, PEERS, GF32>(it, first, kThreads, c, decay, xf, peers);
        }
    } else {
        // partial item (the head or the tail of a tensor): kUnroll groups per thread at a time
        // while that many are left, then one at a time, then the last few elements one by one
        constexpr int U = kUnroll;
        int grp = threadIdx.x;
        for (; grp + (U - 1) * kThreads < groups; grp += U * kThreads) {
            if constexpr (KIND == 2) f32_groups<V32, U>(it, grp, kThreads, c, decay, xf);
            else f16_groups<KIND, V32, ROUND, U, PEERS, GF32>(it, grp, kThreads, c, decay, xf, peers);
        }
        for (; grp < groups; grp += kThreads) {
            if constexpr (KIND == 2) f32_groups<V32, 1>(it, grp, 0, c, decay, xf);
            else f16_groups<KIND, V32, ROUND, 1, PEERS, GF32>(it, grp, 0, c, decay, xf, peers);
        }
        scalar_range<PEERS>(it, groups * kGroup, it.count, c, decay, xf, peers);
    }
}

// GF32 says whether the table may hold 16-bit parameters with FP32 gradients; kernels are
// instantiated both ways so that lists without such tensors run the code they always ran.
template <bool PEERS, bool GF32 = false>
__device__ __forceinline__ void process_item(const WorkItem& it, const StepConsts& c,
                                             const GradXform& xf, const PeerOut& peers) {
    if (it.flags & RLCU_TENSOR_NORM_ONLY) return;
    const float decay = decay_factor(c.lr, it.wd);
    const uint32_t kind = it.flags & kItemKindMask;
    if (!(it.flags & kItemVec16)) {
        scalar_range<PEERS>(it, 0, it.count, c, decay, xf, peers);
        return;
    }
    const bool v32 = (it.flags & kItemVec32) != 0;
    if constexpr (GF32) {
        if (it.flags & kItemGradF32) {
            if (kind == kItemKindF16) {
                if (v32) vector_item<0, true, false, PEERS, true>(it, c, decay, xf, peers);
                else vector_item<0, false, false, PEERS, true>(it, c, decay, xf, peers);
            } else {
                if (v32) vector_item<1, true, false, PEERS, true>(it, c, decay, xf, peers);
                else vector_item<1, false, false, PEERS, true>(it, c, decay, xf, peers);
            }
            return;
        }
    }
    if (kind == kItemKindF16) {
        if (xf.round_half) {
            if (v32) vector_item<0, true, true, PEERS>(it, c, decay, xf, peers);
            else vector_item<0, false, true, PEERS>(it, c, decay, xf, peers);
        } else {
            if (v32) vector_item<0, true, false, PEERS>(it, c, decay, xf, peers);
            else vector_item<0, false, false, PEERS>(it, c, decay, xf, peers);
        }
    } else if (kind == kItemKindF16Master) {
        if (xf.round_half) {
            if (v32) vector_item<1, true, true, PEERS>(it, c, decay, xf, peers);
            else vector_item<1, false, true, PEERS>(it, c, decay, xf, peers);
        } else {
            if (v32) vector_item<1, true, false, PEERS>(it, c, decay, xf, peers);
            else vector_item<1, false, false, PEERS>(it, c, decay, xf, peers);
        }
    } else {
        if (v32) vector_item<2, true, false, PEERS>(it, c, decay, xf, peers);
        else vector_item<2, false, false, PEERS>(it, c, decay, xf, peers);
    }
}

__device__ __forceinline__ WorkItem load_item(const WorkItem* table, uint32_t idx) {
    // four 16-byte loads through the read-only path; the table is re-read every
    // step and shared by all CTAs, so it is left to the default cache policy
    WorkItem it;
    const uint4* src = reinterpret_cast<const uint4*>(table + idx);
    uint4* dst = reinterpret_cast<uint4*>(&it);
#pragma unroll
    for (int i = 0; i < 4; i++) dst[i] = __ldg(src + i);
    return it;
}

struct TableRef {     // a work table in device memory
    const WorkItem* table;
    __device__ __forceinline__ WorkItem get(uint32_t idx) const { return load_item(table, idx); }
};
__device__ __forceinline__ void clear_gradients(const WorkItem* table, uint32_t n_items);

// What a skipped (overflowed) step still does when RLCU_STEP_ZERO_GRADS is set: the stale
// gradients are cleared, parameters and moments stay untouched.
template <class Items>
__device__ __forceinline__ void clear_gradients(const Items& items, uint32_t n_items) {
    for (uint32_t idx = blockIdx.x; idx < n_items; idx += gridDim.x) {
        const WorkItem it = items.get(idx);
        if (it.flags & (RLCU_TENSOR_NORM_ONLY | RLCU_TENSOR_GRAD_ZERO)) continue;
        const bool f32 = (it.flags & kItemKindMask) == kItemKindF32 || (it.flags & kItemGradF32);
        const uint32_t per_vec = f32 ? 4u : 8u;          // elements in 16 bytes
        uint32_t done = 0;
        if (it.flags & kItemVec16) {                     // the gradient pointer is 16-byte aligned
            uint4* g = reinterpret_cast<uint4*>(const_cast<void*>(it.g));
            const uint32_t vecs = it.count / per_vec;
            for (uint32_t i = threadIdx.x; i < vecs; i += blockDim.x) __stcs(g + i, make_uint4(0, 0, 0, 0));
            done = vecs * per_vec;
        }
        if (f32) {
            float* g = const_cast<float*>(static_cast<const float*>(it.g));
            for (uint32_t i = done + threadIdx.x; i < it.count; i += blockDim.x) g[i] = 0.0f;
        } else {
            __half* g = const_cast<__half*>(static_cast<const __half*>(it.g));
            for (uint32_t i = done + threadIdx.x; i < it.count; i += blockDim.x) g[i] = __float2half_rn(0.0f);
        }
    }
}

__device__ __forceinline__ void clear_gradients(const WorkItem* table, uint32_t n_items) {
    clear_gradients(TableRef{table}, n_items);
}

// Resolves the per-launch constants from the statistics record (if any).
// Returns false when the step must be skipped.
__device__ __forceinline__ bool resolve_step(const rlcu_stat* stat, uint32_t step_flags,
                                             StepConsts& c, GradXform& xf) {
    xf.coef = 1.0f;
    xf.round_half = false;
    xf.zero_grads = (step_flags & RLCU_STEP_ZERO_GRADS) != 0;
    if (stat) {
        if (stat->found_inf) return false;
        xf.coef = stat->coef;
        xf.round_half = (step_flags & RLCU_STEP_ROUND_CLIP_FP16) && stat->clip_active;
        if (step_flags & RLCU_STEP_DEVICE_BIAS_CORRECTION) {
            c.bc1_inv = __fdiv_rn(1.0f, stat->bias_correction1);
            c.bc2_inv = __fdiv_rn(1.0f, stat->bias_correction2);
        }
    }
    return true;
}

}  // namespace rlcu

// Device-side building blocks of the sm_100a optimizer step: wide global
// accesses, FP16 packing, the AdamW element update and the block reduction.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rlcu {

// Tuning knobs (the defaults are the measured best on B200; the macros exist so that
// variants can be built side by side and timed).
#ifndef RLCU_CHUNK
#define RLCU_CHUNK 8192
#endif
#ifndef RLCU_UNROLL
#define RLCU_UNROLL 2
#endif
#ifndef RLCU_POLICY
#define RLCU_POLICY 0      // 0 streaming (.cs), 1 default, 2 L1::no_allocate + L2::evict_first loads
#endif

constexpr int kThreads = 256;          // threads per CTA for every kernel here
constexpr int kGroup = 8;              // elements one thread moves per access set
constexpr int kChunk = RLCU_CHUNK;     // elements per work item (= 4 groups per thread)
constexpr int kGroupsPerThread = kChunk / (kThreads * kGroup);
constexpr int kUnroll = RLCU_UNROLL;   // groups whose loads are issued before any arithmetic
static_assert(kChunk % (kThreads * kGroup) == 0 && kGroupsPerThread % kUnroll == 0, "chunk geometry");

// Internal per-item bits kept above the public RLCU_TENSOR_* flags.
constexpr uint32_t kItemKindMask = 0x3u << 8;   // 0 F16, 1 F16+master, 2 F32
constexpr uint32_t kItemKindF16 = 0u << 8;
constexpr uint32_t kItemKindF16Master = 1u << 8;
constexpr uint32_t kItemKindF32 = 2u << 8;
constexpr uint32_t kItemVec16 = 1u << 10;       // every pointer 16-byte aligned
constexpr uint32_t kItemVec32 = 1u << 11;       // FP32 pointers 32-byte aligned too
constexpr uint32_t kItemBF16 = 1u << 12;        // the 16-bit data of an F16-kind item is bfloat16
constexpr uint32_t kItemGradF32 = 1u << 13;     // an F16-kind item whose gradient is FP32

// One unit of work: at most kChunk consecutive elements of one tensor, with
// every pointer already advanced to the first of them.  64 bytes so that a
// thread fetches it with four 16-byte loads.
struct __align__(64) WorkItem {
    void* p;
    const void* g;
    float* m;
    float* v;
    float* master;
    uint32_t count;
    float wd;
    uint32_t flags;      // RLCU_TENSOR_* | kItem*
    uint32_t pad[3];
};
static_assert(sizeof(WorkItem) == 64, "WorkItem must be 64 bytes");

struct StepConsts {
    float lr, b1, b2, eps, bc1_inv, bc2_inv;
};

struct __align__(32) F8 {
    float a[8];
};

// ---- global memory access -------------------------------------------------
// m, v and the master copy are read once and written once per step and the
// working set is far beyond L2, so every access is marked streaming (.cs).
// B200 has 256-bit global loads and stores (ld/st.global.v8.f32, sm_100+);
// they need 32-byte alignment, otherwise two 128-bit accesses are used.

template <bool V32>
__device__ __forceinline__ F8 ld_f8(const float* p) {
    F8 r;
    if constexpr (V32) {
#if RLCU_POLICY == 1
        asm volatile("ld.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
#elif RLCU_POLICY == 2
        asm volatile("ld.global.L1::no_allocate.L2::evict_first.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
#else
        asm volatile("ld.global.cs.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
#endif
                     : "=f"(r.a[0]), "=f"(r.a[1]), "=f"(r.a[2]), "=f"(r.a[3]),
                       "=f"(r.a[4]), "=f"(r.a[5]), "=f"(r.a[6]), "=f"(r.a[7])
                     : "l"(p));
    } else {
        float4 x = __ldcs(reinterpret_cast<const float4*>(p));
        float4 y = __ldcs(reinterpret_cast<const float4*>(p) + 1);
        r.a[0] = x.x; r.a[1] = x.y; r.a[2] = x.z; r.a[3] = x.w;
        r.a[4] = y.x; r.a[5] = y.y; r.a[6] = y.z; r.a[7] = y.w;
    }
    return r;
}

template <bool V32>
__device__ __forceinline__ void st_f8(float* p, const F8& r) {
    if constexpr (V32) {
#if RLCU_POLICY == 1
        asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
#else
        asm volatile("st.global.cs.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
#endif
                     :: "l"(p), "f"(r.a[0]), "f"(r.a[1]), "f"(r.a[2]), "f"(r.a[3]),
                        "f"(r.a[4]), "f"(r.a[5]), "f"(r.a[6]), "f"(r.a[7])
                     : "memory");
    } else {
        __stcs(reinterpret_cast<float4*>(p), make_float4(r.a[0], r.a[1], r.a[2], r.a[3]));
        __stcs(reinterpret_cast<float4*>(p) + 1, make_float4(r.a[4], r.a[5], r.a[6], r.a[7]));
    }
}

__device__ __forceinline__ uint4 ld_h8(const void* p) {
#if RLCU_POLICY == 1
    return *reinterpret_cast<const uint4*>(p);
#else
    return __ldcs(reinterpret_cast<const uint4*>(p));
#endif
}

__device__ __forceinline__ void st_h8(void* p, uint4 x) {
#if RLCU_POLICY == 1
    *reinterpret_cast<uint4*>(p) = x;
#else
    __stcs(reinterpret_cast<uint4*>(p), x);
#endif
}

__device__ __forceinline__ F8 h8_to_f8(uint4 x) {
    F8 r;
    const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
        float2 f = __half22float2(h);
        r.a[2 * i] = f.x;
        r.a[2 * i + 1] = f.y;
    }
    return r;
}

__device__ __forceinline__ uint4 f8_to_h8(const F8& r) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        __half2 h = __floats2half2_rn(r.a[2 * i], r.a[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// bfloat16 twins of the two packers above
__device__ __forceinline__ F8 b8_to_f8(uint4 x) {
    F8 r;
    const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        r.a[2 * i] = __uint_as_float(w[i] << 16);            // bfloat16 is the top half of an FP32
        r.a[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
    return r;
}

__device__ __forceinline__ uint4 f8_to_b8(const F8& r) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        __nv_bfloat162 h = __floats2bfloat162_rn(r.a[2 * i], r.a[2 * i + 1]);
        w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ F8 x8_to_f8(uint4 x, bool bf) { return bf ? b8_to_f8(x) : h8_to_f8(x); }
__device__ __forceinline__ uint4 f8_to_x8(const F8& r, bool bf) { return bf ? f8_to_b8(r) : f8_to_h8(r); }

// scalar forms on raw 16-bit patterns
__device__ __forceinline__ float x_to_f(unsigned short bits, bool bf) {
    return bf ? __uint_as_float((uint32_t)bits << 16) : __half2float(__ushort_as_half(bits));
}
__device__ __forceinline__ unsigned short f_to_x(float x, bool bf) {
    return bf ? __bfloat16_as_ushort(__float2bfloat16_rn(x)) : __half_as_ushort(__float2half_rn(x));
}

// ---- arithmetic -------------------------------------------------------------
// The AdamW element update of RL.cu (src/kernels/adamw.cu:25-36).  Every
// operation is spelled with an explicit round-to-nearest intrinsic, in exactly
// the shape the reference's kernel has when that file is built for sm_100a with
// CUDA 12.9 at its default -fmad=true (established by matching its output bit
// for bit on a B200), so the result depends neither on this compiler's
// contraction choices nor on how the loop around it is unrolled:
//   m  = fma(1-b1, g, b1*m)            v  = fma((1-b2)*g, g, b2*v)
//   w' = w*(1 - lr*wd) - (lr*m_hat) / (sqrt(v_hat) + eps)     (no fma here)
// with IEEE division and square root (the reference is built without fast-math).
__device__ __forceinline__ float adamw_element(float w, float g, float& m, float& v,
                                               const StepConsts& c, float decay) {
    const float mi = __fmaf_rn(__fsub_rn(1.0f, c.b1), g, __fmul_rn(c.b1, m));
    const float vi = __fmaf_rn(__fmul_rn(__fsub_rn(1.0f, c.b2), g), g, __fmul_rn(c.b2, v));
    m = mi;
    v = vi;
    const float m_hat = __fmul_rn(mi, c.bc1_inv);
    const float v_hat = __fmul_rn(vi, c.bc2_inv);
    const float q = __fdiv_rn(__fmul_rn(c.lr, m_hat), __fadd_rn(__fsqrt_rn(v_hat), c.eps));
    return __fsub_rn(__fmul_rn(w, decay), q);
}

__device__ __forceinline__ float decay_factor(float lr, float wd) {
    return __fsub_rn(1.0f, __fmul_rn(lr, wd));   // 1 - lr*wd
}

// What RL.cu's scale_half_kernel leaves in memory: g*scale rounded to FP16
// (include/training/trainer.h:136-139).
__device__ __forceinline__ float round_through_half(float x) {
    return __half2float(__float2half_rn(x));
}
// the same for bfloat16 gradients
__device__ __forceinline__ float round_through_16(float x, bool bf) {
    return bf ? __bfloat162float(__float2bfloat16_rn(x)) : round_through_half(x);
}

// ---- non-finite detection ---------------------------------------------------
// x*0 is NaN exactly when x is inf or NaN, and NaN is sticky under addition, so one
// multiply-add per value (per pair, for packed 16-bit data) into an accumulator that
// starts at zero records whether any value seen was non-finite.  The test is on the
// stored gradient itself, not on its square: a finite FP32 gradient whose square
// overflows FP32 is not an overflowed step.
struct NanProbe {
    float f = 0.0f;        // FP32 values
    uint32_t h = 0u;       // a half2 (+0, +0)
    uint32_t b = 0u;       // a bfloat162 (+0, +0)

    __device__ __forceinline__ void add(float x) { f = __fmaf_rn(x, 0.0f, f); }
    __device__ __forceinline__ void add_pair16(uint32_t w, bool bf) {
        if (bf) {
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&w);
            __nv_bfloat162 acc = *reinterpret_cast<const __nv_bfloat162*>(&b);
            acc = __hfma2(a, __float2bfloat162_rn(0.0f), acc);
            b = *reinterpret_cast<const uint32_t*>(&acc);
        } else {
            const __half2 a = *reinterpret_cast<const __half2*>(&w);
            __half2 acc = *reinterpret_cast<const __half2*>(&h);
            acc = __hfma2(a, __float2half2_rn(0.0f), acc);
            h = *reinterpret_cast<const uint32_t*>(&acc);
        }
    }
    __device__ __forceinline__ void add_h8(uint4 x, bool bf) {
        add_pair16(x.x, bf);
        add_pair16(x.y, bf);
        add_pair16(x.z, bf);
        add_pair16(x.w, bf);
    }
    __device__ __forceinline__ bool bad() const {
        const float2 hf = __half22float2(*reinterpret_cast<const __half2*>(&h));
        const float b0 = __uint_as_float(b << 16), b1 = __uint_as_float(b & 0xFFFF0000u);
        return isnan(f) || isnan(hf.x) || isnan(hf.y) || isnan(b0) || isnan(b1);
    }
};

// ---- reduction --------------------------------------------------------------
// Fixed-order sum over the CTA: xor-shuffle tree inside each warp, then the
// warp results are added in warp order by thread 0.  Result valid in thread 0.
__device__ __forceinline__ float block_sum(float x, float* smem /* kThreads/32 floats */) {
#pragma unroll
    for (int mask = 16; mask >= 1; mask >>= 1) x += __shfl_xor_sync(0xFFFFFFFFu, x, mask);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) smem[warp] = x;
    __syncthreads();
    float s = 0.0f;
    if (threadIdx.x == 0) {
#pragma unroll
        for (int w = 0; w < kThreads / 32; w++) s += smem[w];
    }
    return s;
}

}  // namespace rlcu

// sm_100a optimizer step for RL.cu: kernels and the C ABI declared in
// include/rlcu_adamw.h.
//
// Two kernels carry the step:
//   gradstat_kernel : reads every gradient once (2 B/param for FP16), produces
//                     sum of squares, non-finite flag, norm and clip factor in
//                     device memory.  Replaces RL.cu's sum_sq_* kernels, its
//                     blocking read-back and host sqrtf
//                     (include/training/trainer.h:103-133, 324-344).
//   adamw_table_kernel : one persistent launch over a table of work items that
//                     covers every tensor; reads p/g/m/v (12 B/param) and
//                     writes p/m/v (10 B/param).  Replaces RL.cu's three
//                     launch_adamw_* calls and its two scale kernels
//                     (include/training/optimizer.h:119-147,
//                      src/kernels/adamw.cu, trainer.h:136-145, 345-349).
//                     adamw_table_bulk_kernel is the same pass with the traffic
//                     issued by cp.async.bulk; adamw_flat_kernel serves the
//                     single-tensor entry points.
// All are pure streaming kernels bound by HBM bandwidth: CUDA cores only,
// 128/256-bit coalesced accesses, grids sized to the SM count.
#include "rlcu_adamw.h"

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "adamw_bulk.cuh"
#include "adamw_update.cuh"
#include "host_util.h"
#include "tensor_list.h"

namespace rlcu {

// ---------------------------------------------------------------------------
// update pass
// ---------------------------------------------------------------------------

// Multi-tensor update: persistent CTAs walk the work table with a grid stride.
// GF32 = the table holds 16-bit parameters with FP32 gradients (a second instantiation, so
// that every other list runs exactly the code it ran before that kind existed).
template <bool GF32>
#ifdef RLCU_MIN_CTAS
__global__ void __launch_bounds__(kThreads, RLCU_MIN_CTAS)
#else
__global__ void __launch_bounds__(kThreads)
#endif
adamw_table_kernel(const WorkItem* __restrict__ table, uint32_t n_items, StepConsts c,
                   const rlcu_stat* __restrict__ stat, uint32_t step_flags) {
    GradXform xf;
    if (!resolve_step(stat, step_flags, c, xf)) {
        // overflowed step: parameters and moments stay as they are; stale
        // gradients are still cleared if the caller asked for that
        if (!(step_flags & RLCU_STEP_ZERO_GRADS)) return;
        clear_gradients(table, n_items);
        return;
    }
    uint32_t idx = blockIdx.x;
    if (idx >= n_items) return;
    WorkItem next = load_item(table, idx);
    while (true) {
        const WorkItem it = next;
        const uint32_t nidx = idx + gridDim.x;
        if (nidx < n_items) next = load_item(table, nidx);   // fetched under the data loads
        process_item<false, GF32>(it, c, xf, PeerOut{});
        if (nidx >= n_items) break;
        idx = nidx;
    }
}

// Multi-tensor update, bulk-copy variant: one CTA per SM; kBulkThreads consumer threads do
// the arithmetic in shared memory while one thread of an extra warp drives cp.async.bulk
// loads and stores through a ring of kBulkStages stages (bulk_table_body in adamw_bulk.cuh).
__global__ void __launch_bounds__(kBulkThreads + 32, 1)
adamw_table_bulk_kernel(const WorkItem* __restrict__ table, uint32_t n_items, StepConsts c,
                        const rlcu_stat* __restrict__ stat, uint32_t step_flags,
                        unsigned int* error_word) {
    bulk_table_body<false>(TableItems{table}, n_items, c, stat, step_flags, error_word, PeerOut{});
}

// The same for one tensor (RL.cu's launch_adamw_fp16 shape): items are cut on the fly.
__global__ void __launch_bounds__(kBulkThreads + 32, 1)
adamw_flat_bulk_kernel(const __grid_constant__ FlatItems items, uint32_t n_items, StepConsts c,
                       unsigned int* error_word) {
    bulk_table_body<false>(items, n_items, c, nullptr, 0u, error_word, PeerOut{});
}

// Error word of the launches that have no tensor list to keep one in (the single-tensor entry
// points): set when a bounded wait of adamw_flat_bulk_kernel gives up, read and cleared by
// rlcu_tensor_list_check(NULL).  In host code this name is only a handle for
// cudaGetSymbolAddress.
static __device__ unsigned int flat_error_word;

// Exercises the give-up path of the bounded barrier wait: waits on a barrier that
// nothing will ever complete, with a small try budget, and records the outcome the way
// the bulk-copy update does.  The kernel returns normally; the context stays usable.
__global__ void bounded_wait_probe_kernel(unsigned int* error_word, uint32_t tries) {
    __shared__ __align__(8) unsigned long long bar;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (!mbar_wait(smem_u32(&bar), 0u, tries)) atomicExch(error_word, 1u);
    }
}

// Single-tensor update (RL.cu's launch_adamw_* shape): the work items are
// computed from one descriptor instead of being read from a table.
__global__ void __launch_bounds__(kThreads)
adamw_flat_kernel(WorkItem base, uint64_t n, StepConsts c) {
    GradXform xf;
    xf.coef = 1.0f;
    xf.round_half = false;
    xf.zero_grads = false;
    const uint64_t n_items = (n + kChunk - 1) / kChunk;
    const uint32_t kind = base.flags & kItemKindMask;
    for (uint64_t idx = blockIdx.x; idx < n_items; idx += gridDim.x) {
        const uint64_t off = idx * kChunk;
        WorkItem it = base;
        it.count = (uint32_t)((n - off) < (uint64_t)kChunk ? (n - off) : (uint64_t)kChunk);
        it.m += off;
        it.v += off;
        if (it.master) it.master += off;
        if (kind == kItemKindF32) {
            it.p = static_cast<float*>(base.p) + off;
            it.g = static_cast<const float*>(base.g) + off;
        } else {
            it.p = static_cast<__half*>(base.p) + off;
            it.g = static_cast<const __half*>(base.g) + off;
        }
        process_item<false>(it, c, xf, PeerOut{});
    }
}

__global__ void __launch_bounds__(kThreads)
half_to_float_kernel(float* __restrict__ dst, const __half* __restrict__ src, uint64_t n, bool vec) {
    const uint64_t stride = (uint64_t)gridDim.x * kThreads;
    uint64_t tid = (uint64_t)blockIdx.x * kThreads + threadIdx.x;
    if (vec) {
        const uint64_t groups = n / kGroup;
        for (uint64_t gi = tid; gi < groups; gi += stride) {
            F8 f = h8_to_f8(ld_h8(src + gi * kGroup));
            st_f8<false>(dst + gi * kGroup, f);
        }
        for (uint64_t i = groups * kGroup + tid; i < n; i += stride) dst[i] = __half2float(src[i]);
    } else {
        for (uint64_t i = tid; i < n; i += stride) dst[i] = __half2float(src[i]);
    }
}

// ---------------------------------------------------------------------------
// statistics pass
// ---------------------------------------------------------------------------

// 1 - beta^t as the host computes it (optimizer.h:121-122: FP32 powf).  pow is
// evaluated in FP64 and rounded once, i.e. the correctly rounded FP32 power.  Checked
// for beta in {0.8, 0.9, 0.95, 0.99, 0.999} and every t up to 100,000: equal to the C
// library's powf except where that powf is itself one ulp off the correctly rounded
// value (glibc 2.39: beta 0.999 at t = 2958 and 3606), a 6e-8 relative difference.
__device__ __forceinline__ float bias_correction_dev(float beta, int step) {
    const float p = (float)pow((double)beta, (double)step);
    return __fsub_rn(1.0f, p);
}

// Turns a total sum of squares into the finished record and advances the
// scaler state.  Runs in one thread.
__device__ void finalize_stat(rlcu_stat* out, double sum_sq, float unscale, float max_norm,
                              rlcu_scaler_state* scaler) {
    // A non-finite gradient reaches this point as a NaN sum (the statistics kernels turn their
    // partial into NaN when they see one).  An infinite sum is something else: finite
    // gradients whose squares overflow FP32; the norm is then +inf and a clip scales the
    // gradients to zero, which is what RL.cu's own sequence does with such values.
    const float s = (float)sum_sq;
    const bool bad = isnan(sum_sq);
    const float norm = __fsqrt_rn(s);                       // trainer.h:341
    float coef = unscale;
    uint32_t clip = 0;
    if (!bad && max_norm > 0.0f && norm > max_norm) {      // trainer.h:280, 343
        coef = __fmul_rn(unscale, __fdiv_rn(max_norm, __fadd_rn(norm, 1e-6f)));
        clip = 1;
    }
    out->sum_sq = sum_sq;
    out->norm = norm;
    out->coef = coef;
    out->found_inf = bad ? 1u : 0u;
    out->clip_active = clip;
    if (scaler) {
        out->loss_scale = scaler->scale;
        if (bad) {
            scaler->scale = scaler->scale * 0.5f;
            scaler->growth_tracker = 0;
            scaler->skipped += 1;
        } else {
            scaler->step += 1;
            scaler->growth_tracker += 1;
            if (scaler->growth_tracker >= scaler->growth_interval) {
                scaler->scale = scaler->scale * 2.0f;
                scaler->growth_tracker = 0;
            }
        }
        const int t = scaler->step > 0 ? scaler->step : 1;
        out->step = t;
        out->bias_correction1 = bias_correction_dev(scaler->beta1, t);
        out->bias_correction2 = bias_correction_dev(scaler->beta2, t);
    }
}

__device__ __forceinline__ float scaler_unscale(const rlcu_scaler_state* scaler) {
    const float mul = scaler->grad_mul == 0.0f ? 1.0f : scaler->grad_mul;
    return __fmul_rn(mul, __fdiv_rn(1.0f, scaler->scale));
}

__device__ __forceinline__ void accum_h8(uint4 x, float unscale, float (&acc)[4], bool bf, NanProbe& probe) {
    probe.add_h8(x, bf);
    const F8 f = x8_to_f8(x, bf);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float a = f.a[2 * i] * unscale, b = f.a[2 * i + 1] * unscale;
        acc[i] = fmaf(a, a, acc[i]);
        acc[i] = fmaf(b, b, acc[i]);
    }
}

// Scratch layout: partials[grid] floats, then one uint32 arrival counter kept at
// zero between launches (the last CTA to arrive resets it).
// 40 registers, six CTAs per SM.  The kernel is bound by loads in flight (0.330 / 0.239 / 0.201 /
// 0.192 ms at 2 / 3 / 4 / 6 CTAs per SM); forcing eight CTAs through 32 registers spills and
// runs 0.241 ms, so the compiler's choice stands.
__global__ void __launch_bounds__(kThreads)
gradstat_kernel(const WorkItem* __restrict__ table, uint32_t n_items, float unscale_arg,
                float max_norm, rlcu_scaler_state* scaler, rlcu_stat* out, uint32_t flags,
                float* partials, unsigned int* counter) {
    __shared__ float warp_sums[kThreads / 32];
    __shared__ bool is_last;
    const float unscale = scaler ? scaler_unscale(scaler) : unscale_arg;

    // A thread that saw an inf or NaN gradient turns its partial into NaN, which the sums
    // carry to the total (see NanProbe and finalize_stat).
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    NanProbe probe;
    // only g, count and flags of an item are needed: words 0-1 (p, g), 2 (master, count, wd)
    // and 3 (flags).  The next item's words are fetched before the current item's data, so
    // that their latency hides under the gradient loads.
    uint4 na = make_uint4(0, 0, 0, 0), nd = na, ne = na;
    if (blockIdx.x < n_items) {
        const uint4* wi = reinterpret_cast<const uint4*>(table + blockIdx.x);
        na = __ldg(wi);
        nd = __ldg(wi + 2);
        ne = __ldg(wi + 3);
    }
    for (uint32_t idx = blockIdx.x; idx < n_items; idx += gridDim.x) {
        const uint4 a = na, d = nd, e = ne;
        if (idx + gridDim.x < n_items) {
            const uint4* wi = reinterpret_cast<const uint4*>(table + idx + gridDim.x);
            na = __ldg(wi);
            nd = __ldg(wi + 2);
            ne = __ldg(wi + 3);
        }
        const void* g = reinterpret_cast<const void*>(((uint64_t)a.w << 32) | a.z);
        const uint32_t count = d.z;
        const uint32_t fl = e.x;
        if (fl & RLCU_TENSOR_GRAD_ZERO) continue;
        const bool f32 = (fl & kItemKindMask) == kItemKindF32 || (fl & kItemGradF32);
        const bool bf = (fl & kItemBF16) != 0;
        if (!(fl & kItemVec16)) {
            for (uint32_t i = threadIdx.x; i < count; i += kThreads) {
                const float raw = f32 ? static_cast<const float*>(g)[i]
                                      : x_to_f(static_cast<const unsigned short*>(g)[i], bf);
                probe.add(raw);
                const float x = raw * unscale;
                acc[0] = fmaf(x, x, acc[0]);
            }
        } else if (!f32) {
            const __half* gh = static_cast<const __half*>(g);
            if (count == kChunk) {
                uint4 x[kGroupsPerThread];
#pragma unroll
                for (int u = 0; u < kGroupsPerThread; u++)
                    x[u] = ld_h8(gh + (size_t)(threadIdx.x + u * kThreads) * kGroup);
#pragma unroll
                for (int u = 0; u < kGroupsPerThread; u++) accum_h8(x[u], unscale, acc, bf, probe);
            } else {
                const uint32_t groups = count / kGroup;
                for (uint32_t grp = threadIdx.x; grp < groups; grp += kThreads)
                    accum_h8(ld_h8(gh + (size_t)grp * kGroup), unscale, acc, bf, probe);
                for (uint32_t i = groups * kGroup + threadIdx.x; i < count; i += kThreads) {
                    const float raw = x_to_f(__half_as_ushort(gh[i]), bf);
                    probe.add(raw);
                    const float x = raw * unscale;
                    acc[0] = fmaf(x, x, acc[0]);
                }
            }
        } else {
            const float* gf = static_cast<const float*>(g);
            const uint32_t quads = count / 4;
            for (uint32_t q = threadIdx.x; q < quads; q += kThreads) {
                const float4 x = __ldcs(reinterpret_cast<const float4*>(gf) + q);
                probe.add(x.x);
                probe.add(x.y);
                probe.add(x.z);
                probe.add(x.w);
                const float a0 = x.x * unscale, a1 = x.y * unscale, a2 = x.z * unscale, a3 = x.w * unscale;
                acc[0] = fmaf(a0, a0, acc[0]);
                acc[1] = fmaf(a1, a1, acc[1]);
                acc[2] = fmaf(a2, a2, acc[2]);
                acc[3] = fmaf(a3, a3, acc[3]);
            }
            for (uint32_t i = quads * 4 + threadIdx.x; i < count; i += kThreads) {
                probe.add(gf[i]);
                const float x = gf[i] * unscale;
                acc[0] = fmaf(x, x, acc[0]);
            }
        }
    }
    float mine = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    if (probe.bad()) mine = __int_as_float(0x7FC00000);
    const float block_total = block_sum(mine, warp_sums);

    if (threadIdx.x == 0) {
        partials[blockIdx.x] = block_total;
        __threadfence();
        const unsigned int ticket = atomicAdd(counter, 1u);
        is_last = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;

    // last CTA to arrive: add the per-CTA partials in FP64, in a fixed order (every thread a
    // strided few, so that the loads are independent; then the warp tree; then the warps in order)
    __threadfence();
    __shared__ double warp_totals[kThreads / 32];
    double s = 0.0;
    for (uint32_t i = threadIdx.x; i < gridDim.x; i += kThreads) s += (double)__ldcg(partials + i);
#pragma unroll
    for (int mask = 16; mask >= 1; mask >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, mask);
    if ((threadIdx.x & 31) == 0) warp_totals[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double total = 0.0;
#pragma unroll
        for (int w = 0; w < kThreads / 32; w++) total += warp_totals[w];
        *counter = 0;
        if (flags & RLCU_STAT_PARTIAL) out->sum_sq = total;
        else finalize_stat(out, total, unscale, max_norm, scaler);
    }
}

__global__ void finalize_kernel(rlcu_stat* stat, float unscale_arg, float max_norm,
                                rlcu_scaler_state* scaler) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        const float unscale = scaler ? scaler_unscale(scaler) : unscale_arg;
        finalize_stat(stat, stat->sum_sq, unscale, max_norm, scaler);
    }
}

}  // namespace rlcu

// ===========================================================================
// host side
// ===========================================================================

using namespace rlcu;

namespace {

struct DeviceInfo {
    unsigned int* flat_error = nullptr;   // device address of flat_error_word
    int sms = 0;
    int occ_table = 0, occ_table_gf32 = 0, occ_flat = 0, occ_stat = 0;
};

// per-device launch geometry, looked up once per device
int device_info(DeviceInfo* out) {
    static DeviceInfo cache[64];
    static bool have[64] = {};
    static std::mutex mu;
    int dev = 0;
    RLCU_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return set_error(RLCU_ERR_UNSUPPORTED, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!have[dev]) {
        DeviceInfo di;
        RLCU_CUDA(cudaDeviceGetAttribute(&di.sms, cudaDevAttrMultiProcessorCount, dev));
        RLCU_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&di.occ_table, adamw_table_kernel<false>, kThreads, 0));
        RLCU_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&di.occ_table_gf32, adamw_table_kernel<true>, kThreads, 0));
        RLCU_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&di.occ_flat, adamw_flat_kernel, kThreads, 0));
        RLCU_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&di.occ_stat, gradstat_kernel, kThreads, 0));
        // the bulk-copy variant needs its 192 KB ring opted in once per device
        RLCU_CUDA(cudaFuncSetAttribute(adamw_table_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kBulkSmemBytes));
        RLCU_CUDA(cudaFuncSetAttribute(adamw_flat_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       kBulkSmemBytes));
        void* word = nullptr;
        RLCU_CUDA(cudaGetSymbolAddress(&word, flat_error_word));
        di.flat_error = static_cast<unsigned int*>(word);
        if (di.occ_table < 1 || di.occ_table_gf32 < 1 || di.occ_flat < 1 || di.occ_stat < 1)
            return set_error(RLCU_ERR_CUDA, "kernel does not fit on an SM");
        if (const char* e = getenv("RLCU_STAT_CTAS_PER_SM")) {      // measurement knob
            const int cap = atoi(e);
            if (cap >= 1 && cap < di.occ_stat) di.occ_stat = cap;
        }
        cache[dev] = di;
        have[dev] = true;
    }
    *out = cache[dev];
    return RLCU_OK;
}

// RLCU_DIRECT_ONLY=1 in the environment keeps every launch on the per-thread load/store
// kernels (for measurements, and as a switch should the bulk-copy engine misbehave).
bool direct_only() {
    static const bool on = [] {
        const char* e = getenv("RLCU_DIRECT_ONLY");
        return e && e[0] && e[0] != '0';
    }();
    return on;
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

inline size_t grad_elem_size(const rlcu_tensor_desc& d) {
    return (d.dtype == RLCU_F32 || d.grad_dtype == RLCU_GRAD_F32) ? 4 : 2;
}

// kind bits of one tensor, after checking its descriptor
int classify(const rlcu_tensor_desc& d, uint32_t* bits) {
    uint32_t kind;
    if (d.dtype == RLCU_F32) {
        if (d.master) return set_error(RLCU_ERR_INVALID, "FP32 tensor with a master copy");
        kind = kItemKindF32;
    } else if (d.dtype == RLCU_F16 || d.dtype == RLCU_BF16) {
        kind = (d.master ? kItemKindF16Master : kItemKindF16) | (d.dtype == RLCU_BF16 ? kItemBF16 : 0u);
    } else {
        return set_error(RLCU_ERR_INVALID, "unknown dtype %u", d.dtype);
    }
    if (d.grad_dtype != RLCU_GRAD_AS_PARAM && d.grad_dtype != RLCU_GRAD_F32)
        return set_error(RLCU_ERR_INVALID, "unknown grad_dtype %u", d.grad_dtype);
    if (d.grad_dtype == RLCU_GRAD_F32 && d.dtype != RLCU_F32) kind |= kItemGradF32;
    const bool norm_only = d.flags & RLCU_TENSOR_NORM_ONLY;
    const bool grad_zero = d.flags & RLCU_TENSOR_GRAD_ZERO;
    if (!grad_zero && !d.grad) return set_error(RLCU_ERR_INVALID, "null gradient");
    if (!norm_only && (!d.param || !d.m || !d.v)) return set_error(RLCU_ERR_INVALID, "null param/m/v");
    const size_t esz = d.dtype == RLCU_F32 ? 4 : 2;
    const size_t gesz = grad_elem_size(d);
    if ((d.grad && !aligned(d.grad, gesz)) || (d.param && !aligned(d.param, esz)) ||
        !aligned(d.m, 4) || !aligned(d.v, 4) || !aligned(d.master, 4))
        return set_error(RLCU_ERR_INVALID, "pointer not aligned to its element size");
    *bits = kind;
    return RLCU_OK;
}

// vector-path bits of one work item, from where its pointers actually are
uint32_t item_alignment(const WorkItem& it, const rlcu_tensor_desc& d) {
    const bool norm_only = d.flags & RLCU_TENSOR_NORM_ONLY;
    bool v16 = aligned(it.g, 16), v32 = true;
    if (!norm_only) {
        v16 = v16 && aligned(it.p, 16) && aligned(it.m, 16) && aligned(it.v, 16) && aligned(it.master, 16);
        v32 = aligned(it.m, 32) && aligned(it.v, 32) && aligned(it.master, 32);
        if (d.dtype == RLCU_F32) v32 = v32 && aligned(it.p, 32);
        if (grad_elem_size(d) == 4) v32 = v32 && aligned(it.g, 32);
    }
    return (v16 ? kItemVec16 : 0u) | ((v16 && v32) ? kItemVec32 : 0u);
}

// Where to cut the first work item of a tensor so that the following ones start on a common
// grid in every stream.  A grid of E elements is usable when all of the tensor's pointers sit
// at the same element phase modulo E; then, after `head` elements, every pointer is a multiple
// of E elements of its own type (16 KB for FP16 data and 32 KB for FP32 state at E = 8192).
// Returns the head for the largest usable power of two E between one 128-byte line of the
// narrowest stream and kChunk that the tensor is long enough for (at least four
// grids), or 0 when the tensor already starts on it or no common grid exists.
// Why: full items that start on 16/32 KB boundaries run at 0.985 of the measured HBM bandwidth
// on 20,000 ragged tensors packed into one arena, items that only start on a 128-byte line at
// 0.91, items that straddle lines at 0.86.
uint64_t grid_head(const rlcu_tensor_desc& d, size_t esz) {
    struct Stream { const void* p; size_t sz; };
    const Stream streams[5] = {{d.param, esz}, {d.grad, grad_elem_size(d)}, {d.m, 4}, {d.v, 4}, {d.master, 4}};
    size_t narrow = 4;
    for (const Stream& st : streams)
        if (st.p && st.sz < narrow) narrow = st.sz;
    const uint64_t line_elems = 128 / narrow;
    // measurement knob: RLCU_ITEM_GRID caps the grid (64 = line alignment only)
    static const uint64_t max_grid = [] {
        const char* e = getenv("RLCU_ITEM_GRID");
        const long v = e ? atol(e) : 0;
        return v > 0 ? (uint64_t)v : (uint64_t)kChunk;
    }();
    uint64_t top = kChunk;
    while (top > max_grid && top > line_elems) top >>= 1;
    for (uint64_t E = top; E >= line_elems; E >>= 1) {
        if (d.n < 4 * E && E > line_elems) continue;
        bool have = false, same = true;
        uint64_t phase = 0;
        for (const Stream& st : streams) {
            if (!st.p) continue;
            const uint64_t ph = (reinterpret_cast<uintptr_t>(st.p) / st.sz) % E;
            if (!have) { phase = ph; have = true; }
            else if (ph != phase) same = false;
        }
        if (!have || !same) continue;
        const uint64_t head = phase ? E - phase : 0;
        return head < d.n ? head : 0;
    }
    return 0;
}

StepConsts make_consts(float lr, float b1, float b2, float eps, float bc1, float bc2) {
    StepConsts c;
    c.lr = lr; c.b1 = b1; c.b2 = b2; c.eps = eps;
    c.bc1_inv = 1.0f / bc1;    // FP32 on the host, as src/kernels/adamw.cu:52-53
    c.bc2_inv = 1.0f / bc2;
    return c;
}

int launch_flat(const rlcu_tensor_desc& d, int64_t n, float lr, float b1, float b2, float eps,
                float bc1, float bc2, void* stream) {
    if (n <= 0) return RLCU_OK;                // adamw.cu:49, :99
    uint32_t bits = 0;
    int rc = classify(d, &bits);
    if (rc) return rc;
    DeviceInfo di;
    rc = device_info(&di);
    if (rc) return rc;
    WorkItem base;
    std::memset(&base, 0, sizeof(base));
    base.p = d.param; base.g = d.grad; base.m = d.m; base.v = d.v; base.master = d.master;
    base.wd = d.weight_decay;
    // every later item starts kChunk elements further on, which keeps whatever 16- and
    // 32-byte alignment the tensor's first element has
    base.flags = bits | item_alignment(base, d);
    const uint64_t items = ((uint64_t)n + kChunk - 1) / kChunk;
    // FP16 weights with an FP32 master copy (what RL.cu's launch_adamw_fp16 is) move 28 bytes per
    // element in eight streams; issued as 4-8 KB bulk copies they reach 0.98 of the measured
    // HBM bandwidth where per-thread accesses reach 0.93, so large tensors of that kind take
    // the bulk-copy kernel.  Small ones, and every other kind, take the direct kernel.
    const bool bulk = d.master && d.dtype == RLCU_F16 && (base.flags & kItemVec16) &&
                      items >= 4ull * (uint64_t)di.sms && items <= 0xFFFFFFFFull && !direct_only();
    if (bulk) {
        FlatItems fi;
        fi.base = base;
        fi.n = (uint64_t)n;
        adamw_flat_bulk_kernel<<<di.sms, kBulkThreads + 32, kBulkSmemBytes, (cudaStream_t)stream>>>(
            fi, (uint32_t)items, make_consts(lr, b1, b2, eps, bc1, bc2), di.flat_error);
        RLCU_CUDA(cudaGetLastError());
        return RLCU_OK;
    }
    const uint64_t cap = (uint64_t)di.sms * di.occ_flat;
    const int grid = (int)(items < cap ? items : cap);
    adamw_flat_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(
        base, (uint64_t)n, make_consts(lr, b1, b2, eps, bc1, bc2));
    RLCU_CUDA(cudaGetLastError());
    return RLCU_OK;
}

}  // namespace

extern "C" {

int rlcu_abi_version(void) { return RLCU_ABI_VERSION; }

const char* rlcu_last_error(void) { return rlcu::last_error(); }

float rlcu_bias_correction(float beta, int step) {
    return 1.0f - powf(beta, (float)step);     // optimizer.h:121-122
}

int rlcu_adamw_fp16_master(float* master_w, void* model_w, const void* grad, float* m, float* v,
                           int64_t n, float lr, float beta1, float beta2, float eps,
                           float weight_decay, float bc1, float bc2, void* stream) {
    if (n <= 0) return RLCU_OK;
    if (!master_w) return set_error(RLCU_ERR_INVALID, "null master");
    rlcu_tensor_desc d = {model_w, grad, m, v, master_w, (uint64_t)n, weight_decay, RLCU_F16, 0, 0};
    return launch_flat(d, n, lr, beta1, beta2, eps, bc1, bc2, stream);
}

int rlcu_adamw_fp16(void* param, const void* grad, float* m, float* v,
                    int64_t n, float lr, float beta1, float beta2, float eps,
                    float weight_decay, float bc1, float bc2, void* stream) {
    if (n <= 0) return RLCU_OK;
    rlcu_tensor_desc d = {param, grad, m, v, nullptr, (uint64_t)n, weight_decay, RLCU_F16, 0, 0};
    return launch_flat(d, n, lr, beta1, beta2, eps, bc1, bc2, stream);
}

int rlcu_adamw_bf16_master(float* master_w, void* model_w, const void* grad, float* m, float* v,
                           int64_t n, float lr, float beta1, float beta2, float eps,
                           float weight_decay, float bc1, float bc2, void* stream) {
    if (n <= 0) return RLCU_OK;
    if (!master_w) return set_error(RLCU_ERR_INVALID, "null master");
    rlcu_tensor_desc d = {model_w, grad, m, v, master_w, (uint64_t)n, weight_decay, RLCU_BF16, 0, 0};
    return launch_flat(d, n, lr, beta1, beta2, eps, bc1, bc2, stream);
}

int rlcu_adamw_bf16(void* param, const void* grad, float* m, float* v,
                    int64_t n, float lr, float beta1, float beta2, float eps,
                    float weight_decay, float bc1, float bc2, void* stream) {
    if (n <= 0) return RLCU_OK;
    rlcu_tensor_desc d = {param, grad, m, v, nullptr, (uint64_t)n, weight_decay, RLCU_BF16, 0, 0};
    return launch_flat(d, n, lr, beta1, beta2, eps, bc1, bc2, stream);
}

int rlcu_adamw_fp32(float* w, const float* grad, float* m, float* v,
                    int64_t n, float lr, float beta1, float beta2, float eps,
                    float weight_decay, float bc1, float bc2, void* stream) {
    if (n <= 0) return RLCU_OK;
    rlcu_tensor_desc d = {w, grad, m, v, nullptr, (uint64_t)n, weight_decay, RLCU_F32, 0, 0};
    return launch_flat(d, n, lr, beta1, beta2, eps, bc1, bc2, stream);
}

int rlcu_half_to_float(float* dst, const void* src, int64_t n, void* stream) {
    if (n <= 0) return RLCU_OK;
    if (!dst || !src) return set_error(RLCU_ERR_INVALID, "null pointer");
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc) return rc;
    const bool vec = aligned(dst, 16) && aligned(src, 16);
    const uint64_t want = ((uint64_t)n + (uint64_t)kThreads * kGroup - 1) / ((uint64_t)kThreads * kGroup);
    const uint64_t cap = (uint64_t)di.sms * 8;
    half_to_float_kernel<<<(int)(want < cap ? want : cap), kThreads, 0, (cudaStream_t)stream>>>(
        dst, static_cast<const __half*>(src), (uint64_t)n, vec);
    RLCU_CUDA(cudaGetLastError());
    return RLCU_OK;
}

int rlcu_tensor_list_create(const rlcu_tensor_desc* descs, uint64_t count, rlcu_tensor_list** out) {
    if (!out) return set_error(RLCU_ERR_INVALID, "null out");
    *out = nullptr;
    if (count && !descs) return set_error(RLCU_ERR_INVALID, "null descriptor array");
    DeviceInfo di;
    int rc = device_info(&di);
    if (rc) return rc;

    std::vector<WorkItem> items;
    uint64_t numel = 0, stat_numel = 0, master_numel = 0;
    bool any_grad_f32 = false;
    for (uint64_t k = 0; k < count; k++) {
        const rlcu_tensor_desc& d = descs[k];
        if (d.flags & ~(uint32_t)(RLCU_TENSOR_NORM_ONLY | RLCU_TENSOR_GRAD_ZERO))
            return set_error(RLCU_ERR_INVALID, "tensor %llu: unknown flags", (unsigned long long)k);
        if (d.n == 0) continue;
        uint32_t bits = 0;
        rc = classify(d, &bits);
        if (rc) return rc;
        if (!(d.flags & RLCU_TENSOR_NORM_ONLY)) numel += d.n;
        if (!(d.flags & RLCU_TENSOR_GRAD_ZERO)) stat_numel += d.n;
        const size_t esz = d.dtype == RLCU_F32 ? 4 : 2;
        const size_t gesz = grad_elem_size(d);
        if (bits & kItemGradF32) any_grad_f32 = true;
        // streams per element beyond the five of the plain FP16 update: a master copy, an FP32 gradient
        if (!(d.flags & RLCU_TENSOR_NORM_ONLY) && d.dtype == RLCU_F16 && (d.master || (bits & kItemGradF32))) master_numel += d.n;
        // Work items are cut so that, from the second one on, every pointer sits on a
        // common grid in every stream: a tensor that starts off it (ragged sizes packed into
        // one arena) gets a partial head item first (see grid_head)
        const uint64_t head = grid_head(d, esz);
        uint64_t off = 0;
        while (off < d.n) {
            const uint64_t want = (off == 0 && head) ? head : (uint64_t)kChunk;
            WorkItem it;
            std::memset(&it, 0, sizeof(it));
            it.p = d.param ? static_cast<char*>(d.param) + off * esz : nullptr;
            it.g = d.grad ? static_cast<const char*>(d.grad) + off * gesz : nullptr;
            it.m = d.m ? d.m + off : nullptr;
            it.v = d.v ? d.v + off : nullptr;
            it.master = d.master ? d.master + off : nullptr;
            it.count = (uint32_t)((d.n - off) < want ? (d.n - off) : want);
            it.wd = d.weight_decay;
            it.flags = d.flags | (bits & (kItemKindMask | kItemBF16 | kItemGradF32)) | item_alignment(it, d);
            items.push_back(it);
            off += it.count;
        }
    }
    if (items.size() > 0xFFFFFFFFull) return set_error(RLCU_ERR_UNSUPPORTED, "too many work items");

    rlcu_tensor_list* L = new (std::nothrow) rlcu_tensor_list();
    if (!L) return set_error(RLCU_ERR_INVALID, "out of host memory");
    RLCU_CUDA(cudaGetDevice(&L->device));
    L->n_items = (uint32_t)items.size();
    L->numel = numel;
    L->stat_numel = stat_numel;
    L->has_grad_f32 = any_grad_f32;
    // lists that are mostly FP16 weights with FP32 masters run faster through the bulk-copy
    // kernel (see launch_flat); the others through the direct one
    L->prefer_bulk = master_numel * 2 > numel && items.size() >= 4ull * (uint64_t)di.sms;
    const uint64_t cap_u = (uint64_t)di.sms * (any_grad_f32 ? di.occ_table_gf32 : di.occ_table), cap_s = (uint64_t)di.sms * di.occ_stat;
    L->grid_update = (int)(L->n_items < cap_u ? (L->n_items ? L->n_items : 1) : cap_u);
    L->grid_stat = (int)(L->n_items < cap_s ? (L->n_items ? L->n_items : 1) : cap_s);

    cudaError_t e = cudaSuccess;
    if (L->n_items) {
        e = cudaMalloc(&L->d_items, (size_t)L->n_items * sizeof(WorkItem));
        if (e == cudaSuccess)
            e = cudaMemcpy(L->d_items, items.data(), (size_t)L->n_items * sizeof(WorkItem), cudaMemcpyHostToDevice);
    }
    // scratch of the statistics pass: one float per CTA, then the arrival counter
    const size_t part_bytes = (((size_t)cap_s * sizeof(float) + 255) / 256) * 256;
    if (e == cudaSuccess) e = cudaMalloc(&L->d_partials, part_bytes + 256);
    if (e == cudaSuccess) {
        L->d_counter = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(L->d_partials) + part_bytes);
        e = cudaMemset(L->d_partials, 0, part_bytes + 256);
    }
    if (e != cudaSuccess) {
        cudaFree(L->d_items);
        cudaFree(L->d_partials);
        delete L;
        return set_error(RLCU_ERR_CUDA, "tensor list allocation: %s", cudaGetErrorString(e));
    }
    *out = L;
    return RLCU_OK;
}

int rlcu_tensor_list_destroy(rlcu_tensor_list* list) {
    if (!list) return RLCU_OK;
    cudaError_t e1 = cudaFree(list->d_items);
    cudaError_t e2 = cudaFree(list->d_partials);
    delete list;
    if (e1 != cudaSuccess || e2 != cudaSuccess)
        return set_error(RLCU_ERR_CUDA, "cudaFree: %s", cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
    return RLCU_OK;
}

int rlcu_tensor_list_check(rlcu_tensor_list* list) {
    unsigned int word = 0;
    if (!list) {
        // the single-tensor entry points keep their error word in the library image
        DeviceInfo di;
        const int rc = device_info(&di);
        if (rc) return rc;
        RLCU_CUDA(cudaDeviceSynchronize());
        RLCU_CUDA(cudaMemcpy(&word, di.flat_error, sizeof(word), cudaMemcpyDeviceToHost));
        if (word) {
            cudaMemset(di.flat_error, 0, sizeof(word));
            return set_error(RLCU_ERR_TIMEOUT, "a bulk-copy wait in a single-tensor update gave up; that update is incomplete");
        }
        return RLCU_OK;
    }
    // A blocking copy on the legacy stream does not wait for streams created with
    // cudaStreamNonBlocking, so wait for the whole device first.
    RLCU_CUDA(cudaDeviceSynchronize());
    RLCU_CUDA(cudaMemcpy(&word, list->d_counter + 16, sizeof(word), cudaMemcpyDeviceToHost));
    if (word) {
        cudaMemset(list->d_counter + 16, 0, sizeof(word));
        return set_error(RLCU_ERR_TIMEOUT, "a bulk-copy wait in the update kernel gave up; the step is incomplete");
    }
    return RLCU_OK;
}

int rlcu_selftest_bounded_wait(rlcu_tensor_list* list, void* stream) {
    if (!list) return set_error(RLCU_ERR_INVALID, "null list");
    bounded_wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(list->d_counter + 16, 64u);
    RLCU_CUDA(cudaGetLastError());
    return rlcu_tensor_list_check(list);
}

uint64_t rlcu_tensor_list_numel(const rlcu_tensor_list* list) { return list ? list->numel : 0; }
uint64_t rlcu_tensor_list_stat_numel(const rlcu_tensor_list* list) { return list ? list->stat_numel : 0; }
uint64_t rlcu_tensor_list_work_items(const rlcu_tensor_list* list) { return list ? list->n_items : 0; }

int rlcu_gradstat(rlcu_tensor_list* list, float unscale, float max_norm,
                  rlcu_scaler_state* scaler, rlcu_stat* stat_out, uint32_t flags, void* stream) {
    if (!list || !stat_out) return set_error(RLCU_ERR_INVALID, "null list or stat");
    if (flags & ~(uint32_t)RLCU_STAT_PARTIAL) return set_error(RLCU_ERR_INVALID, "unknown flags");
    if (!aligned(stat_out, 16)) return set_error(RLCU_ERR_INVALID, "stat record must be 16-byte aligned");
    NvtxRange range("rlcu: gradient statistics");
    gradstat_kernel<<<list->grid_stat, kThreads, 0, (cudaStream_t)stream>>>(
        list->d_items, list->n_items, unscale, max_norm, scaler, stat_out, flags,
        list->d_partials, list->d_counter);
    RLCU_CUDA(cudaGetLastError());
    return RLCU_OK;
}

int rlcu_gradstat_finalize(rlcu_stat* stat, float unscale, float max_norm,
                           rlcu_scaler_state* scaler, void* stream) {
    if (!stat) return set_error(RLCU_ERR_INVALID, "null stat");
    finalize_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(stat, unscale, max_norm, scaler);
    RLCU_CUDA(cudaGetLastError());
    return RLCU_OK;
}

int rlcu_adamw_multi_step(rlcu_tensor_list* list, const rlcu_hparams* hp,
                          const rlcu_stat* stat, uint32_t step_flags, void* stream) {
    if (!list || !hp) return set_error(RLCU_ERR_INVALID, "null list or hparams");
    const uint32_t known = RLCU_STEP_ROUND_CLIP_FP16 | RLCU_STEP_DEVICE_BIAS_CORRECTION | RLCU_STEP_ZERO_GRADS |
                           RLCU_STEP_BULK_COPY | RLCU_STEP_DIRECT;
    if (step_flags & ~known) return set_error(RLCU_ERR_INVALID, "unknown step flags");
    if ((step_flags & RLCU_STEP_DEVICE_BIAS_CORRECTION) && !stat)
        return set_error(RLCU_ERR_INVALID, "device bias correction needs a statistics record");
    if (list->n_items == 0) return RLCU_OK;
    NvtxRange range("rlcu: AdamW update");
    if ((step_flags & RLCU_STEP_BULK_COPY) && (step_flags & RLCU_STEP_DIRECT))
        return set_error(RLCU_ERR_INVALID, "RLCU_STEP_BULK_COPY and RLCU_STEP_DIRECT exclude each other");
    if (!(step_flags & RLCU_STEP_DIRECT) && list->prefer_bulk && !direct_only()) step_flags |= RLCU_STEP_BULK_COPY;
    step_flags &= ~(uint32_t)RLCU_STEP_DIRECT;
    if (step_flags & RLCU_STEP_BULK_COPY) {
        DeviceInfo di;
        const int rc = device_info(&di);
        if (rc) return rc;
        const int grid = (int)(list->n_items < (uint32_t)di.sms ? list->n_items : (uint32_t)di.sms);
        adamw_table_bulk_kernel<<<grid, kBulkThreads + 32, kBulkSmemBytes, (cudaStream_t)stream>>>(
            list->d_items, list->n_items,
            make_consts(hp->lr, hp->beta1, hp->beta2, hp->eps, hp->bias_correction1, hp->bias_correction2),
            stat, step_flags & ~(uint32_t)RLCU_STEP_BULK_COPY, list->d_counter + 16);
        RLCU_CUDA(cudaGetLastError());
        return RLCU_OK;
    }
    const StepConsts consts =
        make_consts(hp->lr, hp->beta1, hp->beta2, hp->eps, hp->bias_correction1, hp->bias_correction2);
    if (list->has_grad_f32)
        adamw_table_kernel<true><<<list->grid_update, kThreads, 0, (cudaStream_t)stream>>>(
            list->d_items, list->n_items, consts, stat, step_flags);
    else
        adamw_table_kernel<false><<<list->grid_update, kThreads, 0, (cudaStream_t)stream>>>(
            list->d_items, list->n_items, consts, stat, step_flags);
    RLCU_CUDA(cudaGetLastError());
    return RLCU_OK;
}

}  // extern "C"

// rlcu_gradstat_flat_noalloc: the gradient statistics pass for callers that must
// not allocate device memory.
//
// Who needs this.  RL.cu's GRPO loop shares one GPU between the trainer and an
// inference engine that sizes its KV cache from whatever device memory is free
// (the engine is put to sleep and woken around every training phase).  Code that
// runs once the engine has claimed that memory cannot count on cudaMalloc
// succeeding, and code on a latency-critical path may simply be forbidden to
// enter the allocator.  The list-based rlcu_gradstat() keeps its reduction
// scratch in memory allocated by rlcu_tensor_list_create(); this variant keeps it
// in a fixed array that is part of the library image instead, and takes the
// gradients as one flat buffer (RL.cu's half_pool or float_pool), so no list and
// no allocation are involved at any point.
//
// One call covers one buffer.  RL.cu's clip norm runs over two (the FP16 pool and the
// FP32 pool, trainer.h:331-337): call once on the first buffer with RLCU_STAT_PARTIAL,
// which leaves only its sum in the record, then on the second with RLCU_STAT_ACCUMULATE,
// which adds its own sum to the one in the record and writes the finished record.  The
// two calls go on the same stream, in that order.
//
// Cost and limits.  The array below (1 MiB + 256 B) is resident on every GPU that
// loads the library until the process exits.  It holds one FP32 partial per 8192
// gradient elements, which caps one call at RLCU_NOALLOC_MAX_ELEMS = 2^31
// elements; larger calls are rejected with RLCU_ERR_INVALID.  All calls on a
// device share the array: two calls that overlap on the GPU (different streams
// without ordering, or different host threads) race on it and give wrong
// results.  The array keeps whatever the previous call left; the only word that
// has to start at zero, the arrival counter, is cleared on the caller's stream
// before each launch, and every partial that is read has been written by the same
// launch.
//
// The first call on each device looks up the array's device address
// (cudaGetSymbolAddress) and the kernel's residency; make that first call during
// set-up, outside any stream capture.  Later calls only enqueue a 4-byte memset
// and one kernel on `stream`.  Nothing here calls cudaMalloc, cudaFree or any
// allocating library routine.
#include "rlcu_adamw.h"

#include <mutex>

#include "adamw_device.cuh"
#include "host_util.h"

namespace rlcu {
namespace {

constexpr uint32_t kNoAllocSlots = 262144;                  // one per 8192-element chunk
constexpr uint64_t kNoAllocMaxElems = (uint64_t)kNoAllocSlots * kChunk;
static_assert(kNoAllocMaxElems == RLCU_NOALLOC_MAX_ELEMS, "header and kernel disagree on the limit");

// [0, kNoAllocSlots): per-chunk partial sums; [kNoAllocSlots]: arrival counter.
// In host code this name is only a handle for cudaGetSymbolAddress, never a
// pointer to pass to a kernel.
static __device__ __align__(256) float noalloc_scratch[kNoAllocSlots + 64];

__device__ __forceinline__ void accum8(uint4 x, float unscale, float (&acc)[4], NanProbe& probe) {
    probe.add_h8(x, false);
    const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        const float a = f.x * unscale, b = f.y * unscale;
        acc[i] = fmaf(a, a, acc[i]);
        acc[i] = fmaf(b, b, acc[i]);
    }
}

// `scratch` is the device address of noalloc_scratch, resolved on the host.
__global__ void __launch_bounds__(kThreads)
gradstat_flat_kernel(const void* __restrict__ grad, int is_f32, int vec_ok, uint64_t n,
                     float unscale, float max_norm, rlcu_stat* out, uint32_t flags, float* scratch) {
    __shared__ float warp_sums[kThreads / 32];
    __shared__ double warp_sums_d[kThreads / 32];
    __shared__ bool is_last;
    const uint32_t n_chunks = (uint32_t)((n + kChunk - 1) / kChunk);
    unsigned int* counter = reinterpret_cast<unsigned int*>(scratch + kNoAllocSlots);

    for (uint32_t c = blockIdx.x; c < n_chunks; c += gridDim.x) {
        const uint64_t base = (uint64_t)c * kChunk;
        const uint32_t count = (uint32_t)((n - base) < (uint64_t)kChunk ? (n - base) : (uint64_t)kChunk);
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        NanProbe probe;
        if (is_f32) {
            const float* g = static_cast<const float*>(grad) + base;
            const uint32_t quads = vec_ok ? count / 4 : 0;
            for (uint32_t q = threadIdx.x; q < quads; q += kThreads) {
                const float4 x = __ldcs(reinterpret_cast<const float4*>(g) + q);
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
                probe.add(g[i]);
                const float x = g[i] * unscale;
                acc[0] = fmaf(x, x, acc[0]);
            }
        } else {
            const __half* g = static_cast<const __half*>(grad) + base;
            const uint32_t groups = vec_ok ? count / kGroup : 0;
            for (uint32_t grp = threadIdx.x; grp < groups; grp += kThreads)
                accum8(ld_h8(g + (size_t)grp * kGroup), unscale, acc, probe);
            for (uint32_t i = groups * kGroup + threadIdx.x; i < count; i += kThreads) {
                const float raw = __half2float(g[i]);
                probe.add(raw);
                const float x = raw * unscale;
                acc[0] = fmaf(x, x, acc[0]);
            }
        }
        // an inf or NaN gradient turns the chunk's partial, and so the total, into NaN
        float mine = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        if (probe.bad()) mine = __int_as_float(0x7FC00000);
        const float total = block_sum(mine, warp_sums);
        if (threadIdx.x == 0) scratch[c] = total;
        __syncthreads();                       // warp_sums is reused by the next chunk
    }

    if (threadIdx.x == 0) {
        __threadfence();
        is_last = (atomicAdd(counter, 1u) == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;

    // last CTA to arrive: add every chunk's partial in index order, in FP64
    __threadfence();
    double s = 0.0;
    for (uint32_t i = threadIdx.x; i < n_chunks; i += kThreads) s += (double)__ldcg(scratch + i);
#pragma unroll
    for (int mask = 16; mask >= 1; mask >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, mask);
    if ((threadIdx.x & 31) == 0) warp_sums_d[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        double sum_sq = 0.0;
#pragma unroll
        for (int w = 0; w < kThreads / 32; w++) sum_sq += warp_sums_d[w];
        // a second buffer of the same step: add what the earlier RLCU_STAT_PARTIAL call left
        if (flags & RLCU_STAT_ACCUMULATE) sum_sq += out->sum_sq;
        if (flags & RLCU_STAT_PARTIAL) {
            out->sum_sq = sum_sq;
            *counter = 0;
            return;
        }
        // same rule as the list-based pass: RL.cu's trainer.h:341-344; a NaN total means
        // that some gradient was inf or NaN
        const float sf = (float)sum_sq;
        const bool bad = isnan(sum_sq);
        const float norm = __fsqrt_rn(sf);
        float coef = unscale;
        uint32_t clip = 0;
        if (!bad && max_norm > 0.0f && norm > max_norm) {
            coef = __fmul_rn(unscale, __fdiv_rn(max_norm, __fadd_rn(norm, 1e-6f)));
            clip = 1;
        }
        rlcu_stat r;
        r.sum_sq = sum_sq;
        r.norm = norm;
        r.coef = coef;
        r.found_inf = bad ? 1u : 0u;
        r.clip_active = clip;
        r.bias_correction1 = 0.0f;
        r.bias_correction2 = 0.0f;
        r.step = 0;
        r.loss_scale = 0.0f;
        for (int i = 0; i < 6; i++) r.reserved[i] = 0;
        *out = r;
        *counter = 0;
    }
}

struct NoAllocDevice {
    float* scratch = nullptr;   // device address of noalloc_scratch on this device
    int grid_cap = 0;
};

// One-time set-up per device, with that device current.
int noalloc_device(NoAllocDevice* out) {
    static NoAllocDevice cache[64];
    static bool have[64] = {};
    static std::mutex mu;
    int dev = 0;
    RLCU_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return set_error(RLCU_ERR_UNSUPPORTED, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!have[dev]) {
        NoAllocDevice d;
        void* addr = nullptr;
        RLCU_CUDA(cudaGetSymbolAddress(&addr, noalloc_scratch));
        d.scratch = static_cast<float*>(addr);
        int sms = 0, occ = 0;
        RLCU_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        RLCU_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, gradstat_flat_kernel, kThreads, 0));
        if (occ < 1) return set_error(RLCU_ERR_CUDA, "kernel does not fit on an SM");
        d.grid_cap = sms * occ;
        cache[dev] = d;
        have[dev] = true;
    }
    *out = cache[dev];
    return RLCU_OK;
}

}  // namespace
}  // namespace rlcu

extern "C" int rlcu_gradstat_flat_noalloc(const void* grad, uint32_t dtype, uint64_t n,
                                          float unscale, float max_norm,
                                          rlcu_stat* stat_out, uint32_t flags, void* stream) {
    using namespace rlcu;
    if (!stat_out) return set_error(RLCU_ERR_INVALID, "null statistics record");
    if (flags & ~(uint32_t)(RLCU_STAT_PARTIAL | RLCU_STAT_ACCUMULATE)) return set_error(RLCU_ERR_INVALID, "unknown flags");
    if (dtype != RLCU_F16 && dtype != RLCU_F32) return set_error(RLCU_ERR_INVALID, "unknown dtype %u", dtype);
    if (n > kNoAllocMaxElems)
        return set_error(RLCU_ERR_INVALID,
                         "rlcu_gradstat_flat_noalloc: %llu elements exceed the fixed scratch (limit %llu); "
                         "use rlcu_gradstat with a tensor list",
                         (unsigned long long)n, (unsigned long long)kNoAllocMaxElems);
    if (n && !grad) return set_error(RLCU_ERR_INVALID, "null gradient buffer");
    const size_t esz = dtype == RLCU_F32 ? 4 : 2;
    if (reinterpret_cast<uintptr_t>(grad) % esz) return set_error(RLCU_ERR_INVALID, "gradient pointer not aligned to its element size");
    if (reinterpret_cast<uintptr_t>(stat_out) % 16) return set_error(RLCU_ERR_INVALID, "stat record must be 16-byte aligned");

    NoAllocDevice d;
    const int rc = noalloc_device(&d);
    if (rc) return rc;
    const uint64_t chunks = (n + kChunk - 1) / kChunk;
    const int grid = (int)(chunks < (uint64_t)d.grid_cap ? (chunks ? chunks : 1) : (uint64_t)d.grid_cap);
    const int vec_ok = reinterpret_cast<uintptr_t>(grad) % 16 == 0;
    cudaStream_t s = (cudaStream_t)stream;
    // the arrival counter must start at zero whatever an earlier call left behind
    RLCU_CUDA(cudaMemsetAsync(d.scratch + kNoAllocSlots, 0, sizeof(unsigned int), s));
    gradstat_flat_kernel<<<grid, kThreads, 0, s>>>(grad, dtype == RLCU_F32, vec_ok, n, unscale, max_norm,
                                                   stat_out, flags, d.scratch);
    RLCU_CUDA(cudaGetLastError());
    return RLCU_OK;
}

// Test infrastructure: exposes the reference's own gradient-norm / clip kernels
// (static __global__ functions in include/training/trainer.h:96-145 of RL.cu)
// through a C ABI so the GPU parity tests can run them beside the new kernels.
//
// This file contains no reference code.  It #includes the reference header from
// the reference tree at build time and only restates the host-side launch
// sequence of Trainer::clip_grad_norm_ (trainer.h:323-352), which is a
// protected member of an abstract class and cannot be called on its own.
// The compiled object goes to oracle/_ref/ and is never committed.
#include "training/trainer.h"

#include <algorithm>

extern "C" {

// trainer.h:324-341: zero the accumulator, two sum-of-squares launches, blocking read-back.
int ref_grad_sum_sq(const half* half_pool, int n16, const float* float_pool, int n32,
                    float* d_acc, float* sum_sq_out) {
    if (cudaMemset(d_acc, 0, sizeof(float)) != cudaSuccess) return 1;
    const int block = 256;
    const int max_grid = 2048;
    int grid16 = std::min(max_grid, (n16 + block - 1) / block);
    int grid32 = std::min(max_grid, (n32 + block - 1) / block);
    if (n16 > 0) sum_sq_half_kernel<<<grid16, block>>>(half_pool, d_acc, n16);
    if (n32 > 0) sum_sq_float_kernel<<<grid32, block>>>(float_pool, d_acc, n32);
    if (cudaMemcpy(sum_sq_out, d_acc, sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) return 2;
    return 0;
}

// trainer.h:323-352 in full: returns the pre-clip norm through *norm_out.
int ref_clip_grad_norm(half* half_pool, int n16, float* float_pool, int n32,
                       float max_norm, float* d_acc, float* norm_out) {
    float sum_sq = 0.0f;
    int rc = ref_grad_sum_sq(half_pool, n16, float_pool, n32, d_acc, &sum_sq);
    if (rc) return rc;
    float total_norm = sqrtf(sum_sq);
    if (total_norm > max_norm) {
        float scale = max_norm / (total_norm + 1e-6f);
        const int block = 256;
        int g16 = (n16 + block - 1) / block;
        int g32 = (n32 + block - 1) / block;
        if (n16 > 0) scale_half_kernel<<<g16, block>>>(half_pool, scale, n16);
        if (n32 > 0) scale_float_kernel<<<g32, block>>>(float_pool, scale, n32);
    }
    *norm_out = total_norm;
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// trainer.h:345-349 alone: the reference's two scale kernels with a scale chosen by the caller.
int ref_scale_grads(half* half_pool, int n16, float* float_pool, int n32, float scale) {
    const int block = 256;
    int g16 = (n16 + block - 1) / block;
    int g32 = (n32 + block - 1) / block;
    if (n16 > 0) scale_half_kernel<<<g16, block>>>(half_pool, scale, n16);
    if (n32 > 0) scale_float_kernel<<<g32, block>>>(float_pool, scale, n32);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // extern "C"

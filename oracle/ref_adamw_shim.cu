// Test infrastructure: C-ABI doorway to the reference's AdamW launchers
// (launch_adamw_fp16 / launch_adamw_fp32, include/kernels/adamw.cuh:24-57 of
// RL.cu), which have C++ linkage.  Contains no reference code: it includes the
// reference header from the reference tree at build time and is linked with
// the reference's src/kernels/adamw.cu compiled unmodified from where it lies.
// The result goes to oracle/_ref/ and is never committed.
#include "kernels/adamw.cuh"

extern "C" {

int ref_launch_adamw_fp16(float* master_w, half* model_w, const half* grad, float* m, float* v,
                          int n, float lr, float beta1, float beta2, float eps, float weight_decay,
                          float bias_correction1, float bias_correction2, cudaStream_t stream) {
    launch_adamw_fp16(master_w, model_w, grad, m, v, n, lr, beta1, beta2, eps, weight_decay,
                      bias_correction1, bias_correction2, stream);
    return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

int ref_launch_adamw_fp32(float* w, const float* grad, float* m, float* v,
                          int n, float lr, float beta1, float beta2, float eps, float weight_decay,
                          float bias_correction1, float bias_correction2, cudaStream_t stream) {
    launch_adamw_fp32(w, grad, m, v, n, lr, beta1, beta2, eps, weight_decay,
                      bias_correction1, bias_correction2, stream);
    return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

}  // extern "C"

// C++-linkage launchers with RL.cu's exact signatures
// (include/kernels/adamw.cuh:24-57 of RL.cu), forwarding to the C ABI.
#include "kernels/adamw.cuh"

#include <cstdio>

#include "rlcu_adamw.h"

void launch_adamw_fp16(float* master_w, half* model_w, const half* grad, float* m, float* v, int n,
                       float lr, float beta1, float beta2, float eps, float weight_decay,
                       float bias_correction1, float bias_correction2, cudaStream_t stream) {
    const int rc = rlcu_adamw_fp16_master(master_w, model_w, grad, m, v, n, lr, beta1, beta2, eps,
                                          weight_decay, bias_correction1, bias_correction2, stream);
    if (rc != RLCU_OK) fprintf(stderr, "launch_adamw_fp16: %s\n", rlcu_last_error());
}

void launch_adamw_fp32(float* w, const float* grad, float* m, float* v, int n,
                       float lr, float beta1, float beta2, float eps, float weight_decay,
                       float bias_correction1, float bias_correction2, cudaStream_t stream) {
    const int rc = rlcu_adamw_fp32(w, grad, m, v, n, lr, beta1, beta2, eps, weight_decay,
                                   bias_correction1, bias_correction2, stream);
    if (rc != RLCU_OK) fprintf(stderr, "launch_adamw_fp32: %s\n", rlcu_last_error());
}

// Source-compatible stand-in for RL.cu's include/kernels/adamw.cuh.
//
// The two launchers below have the same names, parameter lists and C++ linkage
// as RL.cu's (include/kernels/adamw.cuh:24-57), so AdamWOptimizer::step
// (include/training/optimizer.h:126-146), train_sft, train_grpo and test_adamw
// compile and link against this library without a change.  They forward to the
// C ABI in rlcu_adamw.h, which runs the vectorised sm_100a kernels.
//
// Behaviour kept from RL.cu: asynchronous on `stream`, no allocation, no
// device synchronisation, `n <= 0` returns at once, nothing is returned.  A
// failed launch is reported on stderr (RL.cu does not check it at all).
//
// bias_correction1 / bias_correction2 are 1 - beta^t, not their inverses.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

// FP16 weight with an FP32 master copy: master_w, m, v are updated in place,
// model_w receives the rounded master, grad is read.
void launch_adamw_fp16(float* master_w, half* model_w, const half* grad, float* m, float* v, int n,
                       float lr, float beta1, float beta2, float eps, float weight_decay,
                       float bias_correction1, float bias_correction2, cudaStream_t stream = 0);

// FP32 weight updated in place from an FP32 gradient.
void launch_adamw_fp32(float* w, const float* grad, float* m, float* v, int n,
                       float lr, float beta1, float beta2, float eps, float weight_decay,
                       float bias_correction1, float bias_correction2, cudaStream_t stream = 0);

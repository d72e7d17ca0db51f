// Drop-in for RL.cu's include/training/optimizer.h: the same AdamWOptimizer
// class name and interface (constructor, public hyper-parameters, set_lr,
// get_step, state accessors, step), implemented over librlcu_b200.  Put this
// repository's include/ directory before RL.cu's on the include path; RL.cu's
// own model/qwen3.h is still the one that defines Qwen3Model and Qwen3Gradients.
//
// Beyond RL.cu's interface the class offers clip_and_step(), which replaces the
// clip_grad_norm_ + step pair of Trainer::training_step
// (include/training/trainer.h:279-286) and GRPOTrainer::grpo_training_step
// (include/training/GRPO_trainer.h:507-514) with two launches and no host
// round trip in the middle of the step.
#pragma once

#include "model/qwen3.h"

#include "training/optimizer_impl.h"

#ifndef CUDA_CHECK
#define CUDA_CHECK(x)                                                                               \
    do {                                                                                            \
        cudaError_t err_ = (x);                                                                     \
        if (err_ != cudaSuccess) {                                                                  \
            fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(err_), __FILE__, __LINE__); \
            exit(1);                                                                                \
        }                                                                                           \
    } while (0)
#endif

using AdamWOptimizer = rlcu_host::BasicAdamWOptimizer<Qwen3Model, Qwen3Gradients>;

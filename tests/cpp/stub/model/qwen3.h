// Test stand-in for RL.cu's model/qwen3.h: just the members that the optimizer
// mirror reads (names as in RL.cu's include/model/config.h:5-33,
// include/model/weights.h:43-61 and include/model/qwen3.h:35-37, 190-198), so that
// include/training/optimizer.h can be built and exercised without RL.cu's tree.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>

struct Qwen3Config {
    int vocab_size = 1000;
    int hidden_size = 256;
    int intermediate_size = 768;
    int num_hidden_layers = 2;
    int num_attention_heads = 4;
    int num_key_value_heads = 2;
    int head_dim = 128;
    int q_dim = 0, kv_dim = 0;
    void compute_derived() {
        q_dim = num_attention_heads * head_dim;
        kv_dim = num_key_value_heads * head_dim;
    }
};

struct Qwen3Weights {
    half* fp16_pool = nullptr;
    float* fp32_pool = nullptr;
    size_t fp16_pool_elems = 0;
    size_t fp32_pool_elems = 0;
};

struct Qwen3Model {
    Qwen3Config config;
    Qwen3Weights weights;
};

struct Qwen3Gradients {
    half* half_pool = nullptr;
    float* float_pool = nullptr;
    size_t half_pool_bytes = 0;
    size_t float_pool_bytes = 0;
};

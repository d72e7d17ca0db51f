// Internal layout of the tensor-list handle, shared by the translation units of
// the library (not part of the public ABI).
#pragma once

#include "adamw_device.cuh"

struct rlcu_tensor_list {
    int device = -1;
    rlcu::WorkItem* d_items = nullptr;
    uint32_t n_items = 0;
    uint64_t numel = 0;        // elements the update pass touches
    uint64_t stat_numel = 0;   // elements the statistics pass reads
    bool prefer_bulk = false;  // mostly FP16 weights with FP32 masters: the bulk-copy kernel is the faster one
    bool has_grad_f32 = false; // some 16-bit parameter has FP32 gradients (selects the kernel instantiation)
    float* d_partials = nullptr;
    unsigned int* d_counter = nullptr;
    int grid_update = 0;
    int grid_stat = 0;
};

// Internal interface between the ZeRO-1 host code (zero1.cu) and the kernels
// that reach the other GPUs through peer-mapped pointers (zero1_p2p.cu).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "adamw_update.cuh"
#include "rlcu_adamw.h"

namespace rlcu {

constexpr int kMaxWorld = kMaxPeers + 1;

// Every rank's FP16 gradient pool in rank order (this rank's own included),
// mapped into this process.
struct PeerIn {
    int n;
    const __half* local_base;
    const __half* base[kMaxWorld];
};

// Fused reduce-scatter + statistics over this rank's shard; writes the rank's
// share of the sum of squares to stat->sum_sq.
int launch_reduce_stat(rlcu_tensor_list* list, const PeerIn& peers, float unscale,
                       const rlcu_scaler_state* scaler, rlcu_stat* stat, cudaStream_t stream);

// Fused update + all-gather: the update pass with every new FP16 parameter also
// stored into the peers' pools.
int launch_update_peers(rlcu_tensor_list* list, const rlcu_hparams* hp, const rlcu_stat* stat,
                        uint32_t step_flags, const PeerOut& peers, cudaStream_t stream);

}  // namespace rlcu

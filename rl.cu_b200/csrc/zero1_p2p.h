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

// The same for an FP32 gradient pool (peers.base / local_base then point at floats): FP32 sum in
// rank order, stored as FP32, nothing rounded.
int launch_reduce_stat_f32(rlcu_tensor_list* list, const PeerIn& peers, float unscale,
                           const rlcu_scaler_state* scaler, rlcu_stat* stat, cudaStream_t stream);

// The part of this rank's gradient pool that lies outside its shard, as two runs of 16-byte
// vectors (before and after the shard).  With RLCU_STEP_ZERO_GRADS the update kernel clears
// it while it works: once the norm has been all-reduced no other rank reads this pool any
// more, and the local HBM is mostly idle while the parameters cross NVLink.
struct ZeroSpan {
    uint4* a;
    uint64_t a_vecs;
    uint4* b;
    uint64_t b_vecs;
};

// Fused reduce-scatter + statistics over this rank's shard; writes the rank's
// share of the sum of squares to stat->sum_sq.
// `bulk`: fetch the ranks' gradients with the bulk-copy engine instead of per-thread loads.
int launch_reduce_stat(rlcu_tensor_list* list, const PeerIn& peers, float unscale,
                       const rlcu_scaler_state* scaler, rlcu_stat* stat, bool bulk, cudaStream_t stream);

// Fused update + all-gather: the update pass with every new FP16 parameter also
// stored into the peers' pools.
int launch_update_peers(rlcu_tensor_list* list, const rlcu_hparams* hp, const rlcu_stat* stat,
                        uint32_t step_flags, const PeerOut& peers, const ZeroSpan& zero, cudaStream_t stream);

}  // namespace rlcu

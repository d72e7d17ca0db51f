// ZeRO-1 sharded optimizer step over the GPUs of one node (rlcu_zero1_* in
// include/rlcu_adamw.h).  RL.cu has no multi-GPU code; the contract comes from
// the step's definition: the result equals the single-GPU step on the mean of the
// ranks' gradients.
//
// NCCL is bound at run time (dlopen/dlsym), not at link time: a host program that
// has already loaded an NCCL (PyTorch bundles its own libnccl.so.2) must keep
// using that copy, and the library must load on machines without NCCL for the
// single-GPU entry points.
#include "rlcu_adamw.h"

#include <dlfcn.h>
#include <nccl.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "host_util.h"
#include "zero1_p2p.h"

namespace {

using rlcu::set_error;

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*CommAbort)(ncclComm_t);
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*);
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    const char* (*GetErrorString)(ncclResult_t);
    bool ok = false;
};

int nccl_api(const NcclApi** out) {
    static NcclApi api;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!api.ok) {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return set_error(RLCU_ERR_NCCL, "cannot load libnccl.so.2: %s", dlerror());
        bool all = true;
        auto sym = [&](const char* name) {
            void* p = dlsym(h, name);
            if (!p) all = false;
            return p;
        };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
        api.CommAbort = reinterpret_cast<decltype(api.CommAbort)>(sym("ncclCommAbort"));
        api.CommGetAsyncError = reinterpret_cast<decltype(api.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
        api.ReduceScatter = reinterpret_cast<decltype(api.ReduceScatter)>(sym("ncclReduceScatter"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
        api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
        if (!all) return set_error(RLCU_ERR_NCCL, "libnccl.so.2 lacks a required symbol");
        api.ok = true;
    }
    *out = &api;
    return RLCU_OK;
}

#define RLCU_NCCL(api, call)                                                                  \
    do {                                                                                      \
        ncclResult_t rlcu_n_ = (call);                                                        \
        if (rlcu_n_ != ncclSuccess && rlcu_n_ != ncclInProgress)                              \
            return set_error(RLCU_ERR_NCCL, "%s: %s", #call, (api)->GetErrorString(rlcu_n_)); \
    } while (0)

constexpr uint64_t kShardAlign = 1024;   // elements: keeps every shard edge 32-byte aligned in FP32 state

struct Piece {
    uint64_t pool_offset, state_offset, n;
    float wd;
    uint32_t flags;
};

int check_geometry(const rlcu_zero1_segment* segs, uint64_t nsegs, int rank, int world) {
    if (world < 1 || rank < 0 || rank >= world) return set_error(RLCU_ERR_INVALID, "rank %d of %d", rank, world);
    if (nsegs && !segs) return set_error(RLCU_ERR_INVALID, "null segments");
    for (uint64_t k = 0; k < nsegs; k++)
        if (segs[k].flags & ~(uint32_t)RLCU_TENSOR_GRAD_ZERO)
            return set_error(RLCU_ERR_INVALID, "segment %llu: unsupported flags", (unsigned long long)k);
    return RLCU_OK;
}

void make_plan(const rlcu_zero1_segment* segs, uint64_t nsegs, int rank, int world,
               rlcu_zero1_plan* plan, std::vector<Piece>* pieces) {
    uint64_t total = 0;
    for (uint64_t k = 0; k < nsegs; k++) total += segs[k].n;
    uint64_t shard = (total + (uint64_t)world - 1) / (uint64_t)world;
    shard = (shard + kShardAlign - 1) / kShardAlign * kShardAlign;
    if (shard == 0) shard = kShardAlign;
    plan->total = total;
    plan->shard_elems = shard;
    plan->padded_elems = shard * (uint64_t)world;
    const uint64_t lo = shard * (uint64_t)rank;
    const uint64_t hi = lo + shard;
    plan->lo = lo < total ? lo : total;
    plan->hi = hi < total ? hi : total;
    uint64_t count = 0, begin = 0;
    for (uint64_t k = 0; k < nsegs; k++) {
        const uint64_t end = begin + segs[k].n;
        const uint64_t a = begin > plan->lo ? begin : plan->lo;
        const uint64_t b = end < plan->hi ? end : plan->hi;
        if (a < b) {
            count++;
            if (pieces) pieces->push_back({a, a - lo, b - a, segs[k].weight_decay, segs[k].flags});
        }
        begin = end;
    }
    plan->pieces = count;
}

}  // namespace

struct rlcu_zero1 {
    const NcclApi* api = nullptr;
    ncclComm_t comm = nullptr;
    int rank = 0, world = 1;
    uint32_t mode = RLCU_ZERO1_NCCL;
    ncclDataType_t wire_type = ncclHalf;   // element type of the parameter pool on the wire (NCCL mode)
    bool grads_f32 = false;                // the gradient pool holds FP32 (RLCU_ZERO1_GRADS_F32)
    rlcu_zero1_plan plan{};
    void* param_pool = nullptr;
    void* grad_pool = nullptr;
    rlcu_tensor_list* list = nullptr;
    // peer-to-peer mode: the other ranks' pools mapped into this process
    int* d_barrier = nullptr;
    rlcu::PeerIn grads_in{};
    rlcu::PeerOut params_out{};
    std::vector<void*> mapped;     // what cudaIpcOpenMemHandle returned, to be closed
};

namespace {

// what each rank tells the others about its two pools
struct PoolExport {
    cudaIpcMemHandle_t grad_handle, param_handle;
    uint64_t grad_offset, param_offset;     // of the pool inside its allocation
    int32_t ok, pad;
};

// base address of the allocation that contains `ptr` (the IPC handle names the
// whole allocation, and callers hand in pointers carved out of larger blocks)
int allocation_base(const void* ptr, void** base) {
    typedef int (*GetRange)(unsigned long long*, size_t*, unsigned long long);
    static GetRange fn = nullptr;
    if (!fn) {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qr;
        RLCU_CUDA(cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &qr));
        if (!f || qr != cudaDriverEntryPointSuccess)
            return set_error(RLCU_ERR_CUDA, "cuMemGetAddressRange is not available");
        fn = reinterpret_cast<GetRange>(f);
    }
    unsigned long long b = 0;
    size_t size = 0;
    if (fn(&b, &size, (unsigned long long)reinterpret_cast<uintptr_t>(ptr)) != 0)
        return set_error(RLCU_ERR_CUDA, "cuMemGetAddressRange failed for %p", ptr);
    *base = reinterpret_cast<void*>((uintptr_t)b);
    return RLCU_OK;
}

int barrier(rlcu_zero1* z, cudaStream_t s) {
    RLCU_NCCL(z->api, z->api->AllReduce(z->d_barrier, z->d_barrier, 1, ncclInt32, ncclSum, z->comm, s));
    return RLCU_OK;
}

// Collective: every rank reports whether its own preparation worked (`local_rc`), and all
// return an error if any rank failed, so that no rank goes on to a collective the others
// will never join.  Needs only the communicator and z->d_barrier (which may be null on a
// rank whose allocation failed: that rank then cannot take part, and says so by aborting
// the communicator, which ends the others' wait with an error instead of a hang).
int agree(rlcu_zero1* z, int local_rc, const char* what) {
    if (!z->d_barrier) {
        z->api->CommAbort(z->comm);
        z->comm = nullptr;
        return local_rc ? local_rc : set_error(RLCU_ERR_CUDA, "%s: no device memory for the agreement word", what);
    }
    int flag = local_rc ? 1 : 0;
    cudaError_t ce = cudaMemcpy(z->d_barrier, &flag, sizeof(int), cudaMemcpyHostToDevice);
    ncclResult_t nr = ncclSuccess;
    if (ce == cudaSuccess) {
        nr = z->api->AllReduce(z->d_barrier, z->d_barrier, 1, ncclInt32, ncclSum, z->comm, 0);
        ce = cudaStreamSynchronize(0);
    }
    int failed = 1;
    if (nr == ncclSuccess && ce == cudaSuccess) ce = cudaMemcpy(&failed, z->d_barrier, sizeof(int), cudaMemcpyDeviceToHost);
    cudaMemset(z->d_barrier, 0, 256);
    if (local_rc) return local_rc;                       // this rank's own message stays in place
    if (nr != ncclSuccess) return set_error(RLCU_ERR_NCCL, "%s: %s", what, z->api->GetErrorString(nr));
    if (ce != cudaSuccess) return set_error(RLCU_ERR_CUDA, "%s: %s", what, cudaGetErrorString(ce));
    if (failed) return set_error(RLCU_ERR_CUDA, "%s: another rank failed", what);
    return RLCU_OK;
}

// Maps every peer's gradient and parameter pool into this process.  Collective; no early
// return before a collective the other ranks take part in.
int setup_p2p(rlcu_zero1* z) {
    const int W = z->world;
    if (W > rlcu::kMaxWorld) return set_error(RLCU_ERR_UNSUPPORTED, "peer-to-peer mode supports at most %d ranks", rlcu::kMaxWorld);

    PoolExport mine{};
    void *gbase = nullptr, *pbase = nullptr;
    int rc = allocation_base(z->grad_pool, &gbase);
    if (!rc) rc = allocation_base(z->param_pool, &pbase);
    bool ok = rc == RLCU_OK;
    if (ok && W > 1) {
        ok = cudaIpcGetMemHandle(&mine.grad_handle, gbase) == cudaSuccess &&
             cudaIpcGetMemHandle(&mine.param_handle, pbase) == cudaSuccess;
        if (!ok) set_error(RLCU_ERR_CUDA, "cudaIpcGetMemHandle failed (pools must come from cudaMalloc): %s",
                           cudaGetErrorString(cudaGetLastError()));
    }
    mine.grad_offset = ok ? (uint64_t)((char*)z->grad_pool - (char*)gbase) : 0;
    mine.param_offset = ok ? (uint64_t)((char*)z->param_pool - (char*)pbase) : 0;
    mine.ok = ok ? 1 : 0;

    PoolExport* d_all = nullptr;
    const cudaError_t alloc_e = cudaMalloc(&d_all, sizeof(PoolExport) * W);
    rc = agree(z, alloc_e == cudaSuccess ? RLCU_OK : set_error(RLCU_ERR_CUDA, "handle exchange buffer: %s", cudaGetErrorString(alloc_e)),
               "handle exchange set-up");
    if (rc) {
        cudaFree(d_all);
        return rc;
    }
    std::vector<PoolExport> all(W);
    cudaError_t ce = cudaMemcpy(d_all + z->rank, &mine, sizeof(PoolExport), cudaMemcpyHostToDevice);
    ncclResult_t nr = ncclSuccess;
    if (ce == cudaSuccess) {
        nr = z->api->AllGather(d_all + z->rank, d_all, sizeof(PoolExport), ncclInt8, z->comm, 0);
        ce = cudaStreamSynchronize(0);
    }
    if (nr == ncclSuccess && ce == cudaSuccess)
        ce = cudaMemcpy(all.data(), d_all, sizeof(PoolExport) * W, cudaMemcpyDeviceToHost);
    cudaFree(d_all);
    if (nr != ncclSuccess) return set_error(RLCU_ERR_NCCL, "handle exchange: %s", z->api->GetErrorString(nr));
    if (ce != cudaSuccess) return set_error(RLCU_ERR_CUDA, "handle exchange: %s", cudaGetErrorString(ce));
    for (int j = 0; j < W; j++)
        if (!all[j].ok) return ok ? set_error(RLCU_ERR_CUDA, "rank %d could not export its pools", j) : RLCU_ERR_CUDA;

    z->grads_in.n = W;
    z->grads_in.local_base = static_cast<const __half*>(z->grad_pool);
    z->params_out.n = 0;
    z->params_out.local_base = static_cast<const __half*>(z->param_pool);
    bool opened_all = true;
    for (int j = 0; j < W && opened_all; j++) {
        if (j == z->rank) {
            z->grads_in.base[j] = static_cast<const __half*>(z->grad_pool);
            continue;
        }
        void *g = nullptr, *p = nullptr;
        if (cudaIpcOpenMemHandle(&g, all[j].grad_handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            set_error(RLCU_ERR_CUDA, "cudaIpcOpenMemHandle(rank %d gradients): %s", j, cudaGetErrorString(cudaGetLastError()));
            opened_all = false;
            break;
        }
        z->mapped.push_back(g);
        if (memcmp(&all[j].grad_handle, &all[j].param_handle, sizeof(cudaIpcMemHandle_t)) == 0) {
            p = g;                      // both pools live in one allocation
        } else if (cudaIpcOpenMemHandle(&p, all[j].param_handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            set_error(RLCU_ERR_CUDA, "cudaIpcOpenMemHandle(rank %d parameters): %s", j, cudaGetErrorString(cudaGetLastError()));
            opened_all = false;
            break;
        } else {
            z->mapped.push_back(p);
        }
        z->grads_in.base[j] = reinterpret_cast<const __half*>((char*)g + all[j].grad_offset);
        z->params_out.base[z->params_out.n++] = reinterpret_cast<__half*>((char*)p + all[j].param_offset);
    }
    // every rank must agree that the mapping worked before anyone relies on it
    return agree(z, opened_all ? RLCU_OK : RLCU_ERR_CUDA, "mapping the peers' pools");
}

void release_p2p(rlcu_zero1* z) {
    for (void* p : z->mapped) cudaIpcCloseMemHandle(p);
    z->mapped.clear();
    if (z->d_barrier) cudaFree(z->d_barrier);
    z->d_barrier = nullptr;
}

}  // namespace

extern "C" {

int rlcu_zero1_make_plan(const rlcu_zero1_segment* segs, uint64_t nsegs, int rank, int world,
                         rlcu_zero1_plan* out) {
    if (!out) return set_error(RLCU_ERR_INVALID, "null plan");
    const int rc = check_geometry(segs, nsegs, rank, world);
    if (rc) return rc;
    make_plan(segs, nsegs, rank, world, out, nullptr);
    return RLCU_OK;
}

int rlcu_zero1_plan_pieces(const rlcu_zero1_segment* segs, uint64_t nsegs, int rank, int world,
                           uint64_t* pool_offset, uint64_t* state_offset, uint64_t* n,
                           float* weight_decay, uint32_t* flags) {
    const int rc = check_geometry(segs, nsegs, rank, world);
    if (rc) return rc;
    rlcu_zero1_plan plan;
    std::vector<Piece> pieces;
    make_plan(segs, nsegs, rank, world, &plan, &pieces);
    for (size_t i = 0; i < pieces.size(); i++) {
        if (pool_offset) pool_offset[i] = pieces[i].pool_offset;
        if (state_offset) state_offset[i] = pieces[i].state_offset;
        if (n) n[i] = pieces[i].n;
        if (weight_decay) weight_decay[i] = pieces[i].wd;
        if (flags) flags[i] = pieces[i].flags;
    }
    return RLCU_OK;
}

int rlcu_zero1_unique_id(void* id_out) {
    static_assert(RLCU_UNIQUE_ID_BYTES == NCCL_UNIQUE_ID_BYTES, "unique id size");
    if (!id_out) return set_error(RLCU_ERR_INVALID, "null id buffer");
    const NcclApi* api;
    const int rc = nccl_api(&api);
    if (rc) return rc;
    RLCU_NCCL(api, api->GetUniqueId(static_cast<ncclUniqueId*>(id_out)));
    return RLCU_OK;
}

int rlcu_zero1_create(const void* unique_id, int rank, int world,
                      void* param_pool, void* grad_pool,
                      const rlcu_zero1_segment* segs, uint64_t nsegs,
                      float* m_shard, float* v_shard, float* master_shard,
                      uint32_t mode, rlcu_zero1** out) {
    if (!out) return set_error(RLCU_ERR_INVALID, "null out");
    const bool bf16 = (mode & RLCU_ZERO1_POOLS_BF16) != 0;
    const bool grads_f32 = (mode & RLCU_ZERO1_GRADS_F32) != 0;
    mode &= ~(uint32_t)(RLCU_ZERO1_POOLS_BF16 | RLCU_ZERO1_GRADS_F32);
    if (mode != RLCU_ZERO1_NCCL && mode != RLCU_ZERO1_P2P) return set_error(RLCU_ERR_INVALID, "unknown mode %u", mode);
    *out = nullptr;
    if (!unique_id || !param_pool || !grad_pool || !m_shard || !v_shard)
        return set_error(RLCU_ERR_INVALID, "null pointer");
    int rc = check_geometry(segs, nsegs, rank, world);
    if (rc) return rc;
    const NcclApi* api;
    rc = nccl_api(&api);
    if (rc) return rc;

    rlcu_zero1* z = new (std::nothrow) rlcu_zero1();
    if (!z) return set_error(RLCU_ERR_INVALID, "out of host memory");
    z->api = api;
    z->rank = rank;
    z->world = world;
    z->mode = mode;
    z->wire_type = bf16 ? ncclBfloat16 : ncclHalf;
    z->grads_f32 = grads_f32;
    z->param_pool = param_pool;
    z->grad_pool = grad_pool;
    std::vector<Piece> pieces;
    make_plan(segs, nsegs, rank, world, &z->plan, &pieces);

    std::vector<rlcu_tensor_desc> descs;
    for (const Piece& p : pieces) {
        rlcu_tensor_desc d{};
        d.param = static_cast<char*>(param_pool) + p.pool_offset * 2;
        d.grad = static_cast<const char*>(grad_pool) + p.pool_offset * (grads_f32 ? 4 : 2);
        d.grad_dtype = grads_f32 ? RLCU_GRAD_F32 : RLCU_GRAD_AS_PARAM;
        d.m = m_shard + p.state_offset;
        d.v = v_shard + p.state_offset;
        d.master = master_shard ? master_shard + p.state_offset : nullptr;
        d.n = p.n;
        d.weight_decay = p.wd;
        d.dtype = bf16 ? RLCU_BF16 : RLCU_F16;
        d.flags = p.flags;
        descs.push_back(d);
    }
    // Join the communicator before any rank-local work that can fail: a rank that returned
    // early would leave the others waiting in ncclCommInitRank for good.
    ncclUniqueId id;
    memcpy(&id, unique_id, sizeof(id));
    ncclResult_t nr = api->CommInitRank(&z->comm, world, id, rank);
    if (nr != ncclSuccess) {
        delete z;
        return set_error(RLCU_ERR_NCCL, "ncclCommInitRank: %s", api->GetErrorString(nr));
    }
    // Rank-local checks and set-up, then every rank learns whether all of them got through.
    if (reinterpret_cast<uintptr_t>(param_pool) % 16 || reinterpret_cast<uintptr_t>(grad_pool) % 16 ||
        reinterpret_cast<uintptr_t>(m_shard) % 32 || reinterpret_cast<uintptr_t>(v_shard) % 32 ||
        reinterpret_cast<uintptr_t>(master_shard) % 32)
        rc = set_error(RLCU_ERR_INVALID, "pools must be 16-byte aligned, shard state 32-byte aligned");
    else
        rc = rlcu_tensor_list_create(descs.data(), descs.size(), &z->list);
    if (cudaMalloc(&z->d_barrier, 256) != cudaSuccess || cudaMemset(z->d_barrier, 0, 256) != cudaSuccess) {
        if (!rc) rc = set_error(RLCU_ERR_CUDA, "agreement word: %s", cudaGetErrorString(cudaGetLastError()));
        if (z->d_barrier) cudaFree(z->d_barrier);
        z->d_barrier = nullptr;
    }
    rc = agree(z, rc, "sharded step set-up");
    if (!rc && mode == RLCU_ZERO1_P2P) rc = setup_p2p(z);
    if (rc) {
        release_p2p(z);
        if (z->comm) api->CommAbort(z->comm);
        rlcu_tensor_list_destroy(z->list);
        delete z;
        return rc;
    }
    *out = z;
    return RLCU_OK;
}

int rlcu_zero1_step(rlcu_zero1* z, const rlcu_hparams* hp, float unscale, float max_norm,
                    rlcu_scaler_state* scaler, rlcu_stat* stat, uint32_t step_flags,
                    uint32_t phases, void* stream) {
    if (!z || !hp || !stat) return set_error(RLCU_ERR_INVALID, "null argument");
    if (phases == 0) phases = 15;
    const uint32_t step_flags_in = step_flags;      // as the caller gave them
    cudaStream_t s = (cudaStream_t)stream;
    const uint64_t S = z->plan.shard_elems;
    const uint64_t gsz = z->grads_f32 ? 4 : 2;         // bytes per gradient element
    char* gshard = static_cast<char*>(z->grad_pool) + (uint64_t)z->rank * S * gsz;
    char* pshard = static_cast<char*>(z->param_pool) + (uint64_t)z->rank * S * 2;
    // gradients are summed, not averaged, on the wire (FP16 would lose the small
    // ones to the division); 1/world goes into the factor applied in registers
    const float unscale_all = unscale / (float)z->world;
    int rc;
    const uint32_t known_flags = RLCU_STEP_ROUND_CLIP_FP16 | RLCU_STEP_DEVICE_BIAS_CORRECTION | RLCU_STEP_ZERO_GRADS |
                                 RLCU_STEP_BULK_COPY | RLCU_STEP_DIRECT;
    if (step_flags & ~known_flags)
        return set_error(RLCU_ERR_INVALID, "step flags 0x%x are not available in the sharded step", step_flags & ~known_flags);
    if ((step_flags & RLCU_STEP_DEVICE_BIAS_CORRECTION) && !scaler)
        return set_error(RLCU_ERR_INVALID, "device bias correction needs a scaler state");
    // RLCU_STEP_ZERO_GRADS clears the WHOLE local gradient pool: the shard inside the update
    // kernel (each gradient after it was read), the rest beside it.
    const uint64_t total_bytes = z->plan.padded_elems * gsz, shard_lo = (uint64_t)z->rank * S * gsz, shard_hi = shard_lo + S * gsz;
    rlcu::ZeroSpan zero{};
    zero.a = reinterpret_cast<uint4*>(z->grad_pool);
    zero.a_vecs = shard_lo / 16;
    zero.b = reinterpret_cast<uint4*>(static_cast<char*>(z->grad_pool) + shard_hi);
    zero.b_vecs = (total_bytes - shard_hi) / 16;
    if (z->mode == RLCU_ZERO1_P2P) {
        if ((step_flags & RLCU_STEP_BULK_COPY) && (step_flags & RLCU_STEP_DIRECT))
            return set_error(RLCU_ERR_INVALID, "RLCU_STEP_BULK_COPY and RLCU_STEP_DIRECT exclude each other");
        // Which pair of exchange kernels: with FP16 pools on more than one rank the bulk-copy pair
        // is the default (1-2 % faster over NVLink at 2 and at 8 ranks); bfloat16 pools and a single
        // rank keep the per-thread pair.  The flags force either.
        static const bool env_direct = [] {
            const char* e = getenv("RLCU_DIRECT_ONLY");
            return e && e[0] && e[0] != '0';
        }();
        const bool bulk = (step_flags & RLCU_STEP_BULK_COPY) ||
                          (!(step_flags & RLCU_STEP_DIRECT) && !env_direct && z->world > 1 && z->wire_type == ncclHalf);
        // (FP32 gradient pools are always reduced by the per-thread kernel; the flag then only
        // selects the update kernel)
        if (bulk) step_flags |= RLCU_STEP_BULK_COPY;
        if (phases & 1u) {
            rlcu::NvtxRange range("rlcu zero1: reduce-scatter + statistics (peer loads)");
            // every rank's gradients are complete before anyone reads them remotely
            rc = barrier(z, s);
            if (rc) return rc;
            // When the library chooses (no flag given), four ranks keep the per-thread reduce kernel:
            // its three CTAs per SM with 256-bit loads measured 651 GB/s per direction there against
            // 636 for the bulk-copy one (at two and at eight ranks the bulk-copy kernel is ahead).
            const bool bulk_reduce = (step_flags_in & RLCU_STEP_BULK_COPY) || (bulk && z->world != 4);
            rc = z->grads_f32
                     ? rlcu::launch_reduce_stat_f32(z->list, z->grads_in, unscale_all, scaler, stat, s)
                     : rlcu::launch_reduce_stat(z->list, z->grads_in, unscale_all, scaler, stat, bulk_reduce, s);
            if (rc) return rc;
        }
        if (phases & 2u) {
            rlcu::NvtxRange range("rlcu zero1: norm all-reduce + finalize");
            // the sum over ranks doubles as "all remote reads of my gradients are done"
            RLCU_NCCL(z->api, z->api->AllReduce(&stat->sum_sq, &stat->sum_sq, 1, ncclDouble, ncclSum, z->comm, s));
            rc = rlcu_gradstat_finalize(stat, unscale_all, max_norm, scaler, s);
            if (rc) return rc;
        }
        if (phases & (4u | 8u)) {
            rlcu::NvtxRange range("rlcu zero1: update + all-gather (peer stores)");
            rc = rlcu::launch_update_peers(z->list, hp, stat, step_flags, z->params_out, zero, s);
            if (rc) return rc;
            // every rank's stores into my pool have landed before I use the parameters
            rc = barrier(z, s);
            if (rc) return rc;
        }
        return RLCU_OK;
    }
    if (phases & 1u) {
        rlcu::NvtxRange range("rlcu zero1: ncclReduceScatter");
        RLCU_NCCL(z->api, z->api->ReduceScatter(z->grad_pool, gshard, S, z->grads_f32 ? ncclFloat : z->wire_type,
                                                ncclSum, z->comm, s));
    }
    if (phases & 2u) {
        rlcu::NvtxRange range("rlcu zero1: statistics + norm all-reduce");
        rc = rlcu_gradstat(z->list, unscale_all, max_norm, scaler, stat, RLCU_STAT_PARTIAL, s);
        if (rc) return rc;
        RLCU_NCCL(z->api, z->api->AllReduce(&stat->sum_sq, &stat->sum_sq, 1, ncclDouble, ncclSum, z->comm, s));
        rc = rlcu_gradstat_finalize(stat, unscale_all, max_norm, scaler, s);
        if (rc) return rc;
    }
    if (phases & 4u) {
        rc = rlcu_adamw_multi_step(z->list, hp, stat, step_flags, s);
        if (rc) return rc;
        if (step_flags & RLCU_STEP_ZERO_GRADS) {      // the stale partial sums outside the shard
            if (zero.a_vecs) RLCU_CUDA(cudaMemsetAsync(zero.a, 0, zero.a_vecs * 16, s));
            if (zero.b_vecs) RLCU_CUDA(cudaMemsetAsync(zero.b, 0, zero.b_vecs * 16, s));
        }
    }
    if (phases & 8u) {
        rlcu::NvtxRange range("rlcu zero1: ncclAllGather");
        RLCU_NCCL(z->api, z->api->AllGather(pshard, z->param_pool, S, z->wire_type, z->comm, s));
    }
    return RLCU_OK;
}

int rlcu_zero1_poll_error(rlcu_zero1* z) {
    if (!z) return set_error(RLCU_ERR_INVALID, "null context");
    ncclResult_t async = ncclSuccess;
    RLCU_NCCL(z->api, z->api->CommGetAsyncError(z->comm, &async));
    if (async != ncclSuccess && async != ncclInProgress)
        return set_error(RLCU_ERR_NCCL, "asynchronous NCCL error: %s", z->api->GetErrorString(async));
    return RLCU_OK;
}

int rlcu_zero1_check(rlcu_zero1* z) {
    if (!z) return set_error(RLCU_ERR_INVALID, "null context");
    const int rc = rlcu_tensor_list_check(z->list);      // waits for the device; a bounded wait that gave up
    if (rc) return rc;
    return rlcu_zero1_poll_error(z);
}

int rlcu_zero1_destroy(rlcu_zero1* z, int abort) {
    if (!z) return RLCU_OK;
    int rc = RLCU_OK;
    if (z->comm) {
        ncclResult_t nr = abort ? z->api->CommAbort(z->comm) : z->api->CommDestroy(z->comm);
        if (nr != ncclSuccess) rc = set_error(RLCU_ERR_NCCL, "communicator teardown: %s", z->api->GetErrorString(nr));
    }
    release_p2p(z);
    const int rc2 = rlcu_tensor_list_destroy(z->list);
    delete z;
    return rc ? rc : rc2;
}

}  // extern "C"

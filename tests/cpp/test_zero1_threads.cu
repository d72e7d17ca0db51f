// The sharded optimizer step driven from plain C++ through the C ABI, with no
// Python and no PyTorch: one host thread per GPU, an NCCL unique id handed from
// thread 0 to the others through a promise, pools from cudaMalloc.
//
// Checks the contract of the sharded step without an oracle: after one step every
// rank's FP16 parameter pool is identical, and it equals the pool a single-GPU
// step (same library, one list over the whole pool) produces from the summed
// gradients with 1/world as the unscale factor.
//
// Uses the NCCL exchange because every rank lives in one process here (the
// peer-to-peer mode maps the other ranks' pools with CUDA IPC, which needs one
// process per GPU).  Prints [PASS]/[FAIL] lines and returns the failure count.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <future>
#include <thread>
#include <vector>

#include "rlcu_adamw.h"

#define CHECK_CUDA(x)                                                                      \
    do {                                                                                   \
        cudaError_t e_ = (x);                                                              \
        if (e_ != cudaSuccess) {                                                           \
            fprintf(stderr, "CUDA %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); \
            exit(2);                                                                       \
        }                                                                                  \
    } while (0)
#define CHECK_RLCU(x)                                                             \
    do {                                                                          \
        int rc_ = (x);                                                            \
        if (rc_ != RLCU_OK) {                                                     \
            fprintf(stderr, "%s: %s\n", #x, rlcu_last_error());                   \
            exit(3);                                                              \
        }                                                                         \
    } while (0)

static unsigned lcg_state = 2024u;
static float lcg() {
    lcg_state = lcg_state * 1664525u + 1013904223u;
    return (float)(lcg_state >> 8) / 8388608.0f - 1.0f;
}

int main() {
    int world = 0;
    if (cudaGetDeviceCount(&world) != cudaSuccess || world < 2) {
        printf("needs at least 2 GPUs (found %d)\n", world);
        return 99;
    }
    if (world > 8) world = 8;
    const rlcu_zero1_segment segs[3] = {{300000, 0.01f, 0}, {200037, 0.0f, 0}, {8192, 0.02f, 0}};
    rlcu_zero1_plan plan;
    CHECK_RLCU(rlcu_zero1_make_plan(segs, 3, 0, world, &plan));
    const size_t total = plan.total, padded = plan.padded_elems, S = plan.shard_elems;

    std::vector<half> p0(padded, __float2half(0.0f));
    std::vector<std::vector<half>> g(world, std::vector<half>(padded, __float2half(0.0f)));
    for (size_t i = 0; i < total; i++) p0[i] = __float2half(0.02f * lcg());
    for (int r = 0; r < world; r++)
        for (size_t i = 0; i < total; i++) g[r][i] = __float2half(0.005f * lcg());
    const rlcu_hparams hp = {1e-4f, 0.9f, 0.999f, 1e-8f, rlcu_bias_correction(0.9f, 1), rlcu_bias_correction(0.999f, 1)};

    std::promise<std::vector<char>> id_promise;
    std::shared_future<std::vector<char>> id_future = id_promise.get_future().share();
    std::vector<std::vector<half>> p_after(world, std::vector<half>(padded));
    std::vector<std::vector<half>> g_after(world, std::vector<half>(padded));
    std::vector<rlcu_stat> stats(world);

    auto rank_main = [&](int rank) {
        CHECK_CUDA(cudaSetDevice(rank));
        if (rank == 0) {
            std::vector<char> id(RLCU_UNIQUE_ID_BYTES);
            CHECK_RLCU(rlcu_zero1_unique_id(id.data()));
            id_promise.set_value(id);
        }
        const std::vector<char> id = id_future.get();
        half *p, *gr;
        float *m, *v;
        rlcu_stat* stat;
        CHECK_CUDA(cudaMalloc(&p, padded * sizeof(half)));
        CHECK_CUDA(cudaMalloc(&gr, padded * sizeof(half)));
        CHECK_CUDA(cudaMalloc(&m, S * sizeof(float)));
        CHECK_CUDA(cudaMalloc(&v, S * sizeof(float)));
        CHECK_CUDA(cudaMalloc(&stat, sizeof(rlcu_stat)));
        CHECK_CUDA(cudaMemcpy(p, p0.data(), padded * sizeof(half), cudaMemcpyHostToDevice));
        CHECK_CUDA(cudaMemcpy(gr, g[rank].data(), padded * sizeof(half), cudaMemcpyHostToDevice));
        CHECK_CUDA(cudaMemset(m, 0, S * sizeof(float)));
        CHECK_CUDA(cudaMemset(v, 0, S * sizeof(float)));
        rlcu_zero1* z;
        CHECK_RLCU(rlcu_zero1_create(id.data(), rank, world, p, gr, segs, 3, m, v, nullptr, RLCU_ZERO1_NCCL, &z));
        CHECK_RLCU(rlcu_zero1_step(z, &hp, 1.0f, 1.0f, nullptr, stat, RLCU_STEP_ROUND_CLIP_FP16, 0, nullptr));
        CHECK_CUDA(cudaDeviceSynchronize());
        CHECK_RLCU(rlcu_zero1_poll_error(z));
        CHECK_CUDA(cudaMemcpy(p_after[rank].data(), p, padded * sizeof(half), cudaMemcpyDeviceToHost));
        CHECK_CUDA(cudaMemcpy(g_after[rank].data(), gr, padded * sizeof(half), cudaMemcpyDeviceToHost));
        CHECK_CUDA(cudaMemcpy(&stats[rank], stat, sizeof(rlcu_stat), cudaMemcpyDeviceToHost));
        CHECK_RLCU(rlcu_zero1_destroy(z, 0));
        cudaFree(p); cudaFree(gr); cudaFree(m); cudaFree(v); cudaFree(stat);
    };
    std::vector<std::thread> threads;
    for (int r = 0; r < world; r++) threads.emplace_back(rank_main, r);
    for (auto& t : threads) t.join();

    int failures = 0;
    auto expect = [&](bool ok, const char* name) {
        printf("[%s] %s\n", ok ? "PASS" : "FAIL", name);
        if (!ok) failures++;
    };
    bool same = true, norms = true;
    for (int r = 1; r < world; r++) {
        same = same && memcmp(p_after[0].data(), p_after[r].data(), padded * sizeof(half)) == 0;
        norms = norms && stats[r].norm == stats[0].norm && stats[r].coef == stats[0].coef;
    }
    expect(same, "every rank holds the same parameters after the all-gather");
    expect(norms && stats[0].found_inf == 0 && stats[0].clip_active == 1, "every rank computed the same global norm");

    // single-GPU step on the reduce-scattered gradients (each rank's shard of its own pool)
    CHECK_CUDA(cudaSetDevice(0));
    std::vector<half> g_sum(padded, __float2half(0.0f));
    for (int r = 0; r < world; r++) memcpy(&g_sum[r * S], &g_after[r][r * S], S * sizeof(half));
    half *p, *gr;
    float *m, *v;
    rlcu_stat* stat;
    CHECK_CUDA(cudaMalloc(&p, padded * sizeof(half)));
    CHECK_CUDA(cudaMalloc(&gr, padded * sizeof(half)));
    CHECK_CUDA(cudaMalloc(&m, padded * sizeof(float)));
    CHECK_CUDA(cudaMalloc(&v, padded * sizeof(float)));
    CHECK_CUDA(cudaMalloc(&stat, sizeof(rlcu_stat)));
    CHECK_CUDA(cudaMemcpy(p, p0.data(), padded * sizeof(half), cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(gr, g_sum.data(), padded * sizeof(half), cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemset(m, 0, padded * sizeof(float)));
    CHECK_CUDA(cudaMemset(v, 0, padded * sizeof(float)));
    rlcu_tensor_desc d[3];
    memset(d, 0, sizeof(d));
    size_t off = 0;
    for (int k = 0; k < 3; k++) {
        d[k].param = p + off; d[k].grad = gr + off; d[k].m = m + off; d[k].v = v + off;
        d[k].n = segs[k].n; d[k].weight_decay = segs[k].weight_decay; d[k].dtype = RLCU_F16;
        off += segs[k].n;
    }
    rlcu_tensor_list* list;
    CHECK_RLCU(rlcu_tensor_list_create(d, 3, &list));
    CHECK_RLCU(rlcu_gradstat(list, 1.0f / (float)world, 1.0f, nullptr, stat, 0, nullptr));
    CHECK_RLCU(rlcu_adamw_multi_step(list, &hp, stat, RLCU_STEP_ROUND_CLIP_FP16, nullptr));
    CHECK_CUDA(cudaDeviceSynchronize());
    std::vector<half> p_single(padded);
    rlcu_stat s1;
    CHECK_CUDA(cudaMemcpy(p_single.data(), p, padded * sizeof(half), cudaMemcpyDeviceToHost));
    CHECK_CUDA(cudaMemcpy(&s1, stat, sizeof(rlcu_stat), cudaMemcpyDeviceToHost));
    const float rel = fabsf(s1.norm - stats[0].norm) / s1.norm;
    expect(rel <= 1e-5f, "global norm equals the single-GPU norm of the summed gradients (1e-5 relative)");
    size_t worst = 0;
    for (size_t i = 0; i < total; i++) {
        const int a = (int)__half_as_ushort(p_single[i]), b = (int)__half_as_ushort(p_after[0][i]);
        const size_t dist = (size_t)(a > b ? a - b : b - a);
        if (((a ^ b) & 0x8000) == 0 && dist > worst) worst = dist;
    }
    // the two norms are summed in a different order, so the clip factor may differ in its last
    // bit: parameters within 1 FP16 ulp
    expect(worst <= 1, "parameters equal the single-GPU step on the summed gradients (1 ulp)");
    CHECK_RLCU(rlcu_tensor_list_destroy(list));
    printf("%d failure(s) on %d GPUs\n", failures, world);
    return failures;
}

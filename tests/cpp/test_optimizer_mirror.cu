// Exercises the AdamWOptimizer mirror (include/training/optimizer.h) the way
// RL.cu's tests/test_adamw.cu exercises the original: construct over a model,
// step, read the state back through the accessors -- here on a small synthetic
// model, and checked against the reference's own call sequence issued through
// the launch_adamw_* launchers (optimizer.h:119-147 of RL.cu).
// Prints [PASS]/[FAIL] lines and returns the number of failures.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "kernels/adamw.cuh"
#include "training/optimizer.h"

static int failures = 0;
#define EXPECT(cond, name)                          \
    do {                                            \
        if (cond) printf("[PASS] %s\n", name);      \
        else { printf("[FAIL] %s\n", name); failures++; } \
    } while (0)

static unsigned lcg_state = 12345u;
static float lcg() {   // uniform in [-1, 1)
    lcg_state = lcg_state * 1664525u + 1013904223u;
    return (float)(lcg_state >> 8) / 8388608.0f - 1.0f;
}

template <class T>
static std::vector<T> download(const T* d, size_t n) {
    std::vector<T> h(n);
    CUDA_CHECK(cudaMemcpy(h.data(), d, n * sizeof(T), cudaMemcpyDeviceToHost));
    return h;
}

template <class T>
static bool same(const std::vector<T>& a, const std::vector<T>& b) {
    return a.size() == b.size() && memcmp(a.data(), b.data(), a.size() * sizeof(T)) == 0;
}

int main() {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
        printf("no CUDA device\n");
        return 99;
    }
    Qwen3Model model;
    model.config.compute_derived();
    const Qwen3Config& c = model.config;
    const size_t H = c.hidden_size;
    const size_t layer16 = (size_t)c.q_dim * H * 2 + (size_t)c.kv_dim * H * 2 + (size_t)c.intermediate_size * H * 3;
    const size_t proj_n = layer16 * c.num_hidden_layers;
    const size_t n16 = proj_n + (size_t)c.vocab_size * H;
    const size_t n32 = (2 * H + 2 * c.head_dim) * c.num_hidden_layers + H;
    const size_t workspace = 777;                      // floats behind the norm gradients
    model.weights.fp16_pool_elems = n16;
    model.weights.fp32_pool_elems = n32;

    std::vector<half> w16(n16), g16(n16);
    std::vector<float> w32(n32), g32(n32 + workspace);
    for (auto& x : w16) x = __float2half(0.02f * lcg());
    for (auto& x : g16) x = __float2half(0.01f * lcg());
    for (auto& x : w32) x = 1.0f + 0.01f * lcg();
    for (auto& x : g32) x = 0.01f * lcg();

    Qwen3Gradients grads;
    grads.half_pool_bytes = n16 * sizeof(half);
    grads.float_pool_bytes = (n32 + workspace) * sizeof(float);
    CUDA_CHECK(cudaMalloc(&model.weights.fp16_pool, n16 * sizeof(half)));
    CUDA_CHECK(cudaMalloc(&model.weights.fp32_pool, n32 * sizeof(float)));
    CUDA_CHECK(cudaMalloc(&grads.half_pool, grads.half_pool_bytes));
    CUDA_CHECK(cudaMalloc(&grads.float_pool, grads.float_pool_bytes));
    auto upload = [&]() {
        CUDA_CHECK(cudaMemcpy(model.weights.fp16_pool, w16.data(), n16 * sizeof(half), cudaMemcpyHostToDevice));
        CUDA_CHECK(cudaMemcpy(model.weights.fp32_pool, w32.data(), n32 * sizeof(float), cudaMemcpyHostToDevice));
        CUDA_CHECK(cudaMemcpy(grads.half_pool, g16.data(), grads.half_pool_bytes, cudaMemcpyHostToDevice));
        CUDA_CHECK(cudaMemcpy(grads.float_pool, g32.data(), grads.float_pool_bytes, cudaMemcpyHostToDevice));
    };
    upload();

    // ---- construction: defaults, sizes, master initialised from the FP16 pool
    {
        AdamWOptimizer opt(&model);
        EXPECT(opt.lr == 1e-4f && opt.beta1 == 0.9f && opt.beta2 == 0.999f && opt.eps == 1e-8f && opt.weight_decay == 0.01f,
               "constructor defaults");
        EXPECT(opt.num_fp16_params() == n16 && opt.num_fp32_params() == n32 && opt.get_step() == 0, "pool sizes and step counter");
        auto master = download(opt.fp16_master(), n16);
        bool ok = true;
        for (size_t i = 0; i < n16; i++) ok = ok && master[i] == __half2float(w16[i]);
        EXPECT(ok, "master weights start as the FP16 weights");
        EXPECT(opt.get_fp16_m(1, 2) == opt.fp16_m() + layer16 + (size_t)c.q_dim * H + (size_t)c.kv_dim * H, "per-projection accessor offsets");
        EXPECT(opt.get_final_norm_v() == opt.fp32_v() + n32 - H, "final-norm accessor offset");
    }

    // ---- three steps through the mirror vs the reference's three-launch sequence
    std::vector<half> p_a;
    std::vector<float> master_a, m_a, v_a, w32_a, m32_a, v32_a;
    {
        AdamWOptimizer opt(&model, 1e-3f, 0.9f, 0.999f, 1e-8f, 0.01f);
        for (int s = 0; s < 3; s++) opt.step(&grads);
        CUDA_CHECK(cudaDeviceSynchronize());
        EXPECT(opt.get_step() == 3, "step counter counts steps");
        p_a = download(model.weights.fp16_pool, n16);
        master_a = download(opt.fp16_master(), n16);
        m_a = download(opt.fp16_m(), n16);
        v_a = download(opt.fp16_v(), n16);
        w32_a = download(model.weights.fp32_pool, n32);
        m32_a = download(opt.fp32_m(), n32);
        v32_a = download(opt.fp32_v(), n32);
    }
    upload();
    {
        float *master, *m, *v, *m32, *v32;
        CUDA_CHECK(cudaMalloc(&master, n16 * 4)); CUDA_CHECK(cudaMalloc(&m, n16 * 4)); CUDA_CHECK(cudaMalloc(&v, n16 * 4));
        CUDA_CHECK(cudaMalloc(&m32, n32 * 4)); CUDA_CHECK(cudaMalloc(&v32, n32 * 4));
        CUDA_CHECK(cudaMemset(m, 0, n16 * 4)); CUDA_CHECK(cudaMemset(v, 0, n16 * 4));
        CUDA_CHECK(cudaMemset(m32, 0, n32 * 4)); CUDA_CHECK(cudaMemset(v32, 0, n32 * 4));
        std::vector<float> mh(n16);
        for (size_t i = 0; i < n16; i++) mh[i] = __half2float(w16[i]);
        CUDA_CHECK(cudaMemcpy(master, mh.data(), n16 * 4, cudaMemcpyHostToDevice));
        for (int s = 1; s <= 3; s++) {
            const float bc1 = 1.0f - powf(0.9f, (float)s), bc2 = 1.0f - powf(0.999f, (float)s);
            launch_adamw_fp16(master, model.weights.fp16_pool, grads.half_pool, m, v, (int)proj_n,
                              1e-3f, 0.9f, 0.999f, 1e-8f, 0.01f, bc1, bc2);
            launch_adamw_fp16(master + proj_n, model.weights.fp16_pool + proj_n, grads.half_pool + proj_n,
                              m + proj_n, v + proj_n, (int)(n16 - proj_n), 1e-3f, 0.9f, 0.999f, 1e-8f, 0.0f, bc1, bc2);
            launch_adamw_fp32(model.weights.fp32_pool, grads.float_pool, m32, v32, (int)n32,
                              1e-3f, 0.9f, 0.999f, 1e-8f, 0.0f, bc1, bc2);
        }
        CUDA_CHECK(cudaDeviceSynchronize());
        EXPECT(same(p_a, download(model.weights.fp16_pool, n16)) && same(master_a, download(master, n16)) &&
               same(m_a, download(m, n16)) && same(v_a, download(v, n16)), "step(): FP16 pools equal the three-launch sequence bit for bit");
        EXPECT(same(w32_a, download(model.weights.fp32_pool, n32)) && same(m32_a, download(m32, n32)) &&
               same(v32_a, download(v32, n32)), "step(): FP32 pool equals the three-launch sequence bit for bit");
        cudaFree(master); cudaFree(m); cudaFree(v); cudaFree(m32); cudaFree(v32);
    }

    // ---- clip_and_step: norm against a host FP64 sum, gradients untouched, switches
    upload();
    {
        AdamWOptimizer opt(&model, 1e-3f);
        double ss = 0.0, ss_ws = 0.0;
        for (size_t i = 0; i < n16; i++) ss += (double)__half2float(g16[i]) * __half2float(g16[i]);
        for (size_t i = 0; i < n32; i++) ss += (double)g32[i] * g32[i];
        for (size_t i = n32; i < n32 + workspace; i++) ss_ws += (double)g32[i] * g32[i];
        const float norm = opt.clip_and_step(&grads, 1.0f);
        EXPECT(fabs(norm - sqrt(ss)) <= 1e-5 * sqrt(ss), "clip_and_step(): pre-clip norm over parameters");
        EXPECT(same(g16, download(grads.half_pool, n16)), "clip_and_step(): gradients are not modified");
        EXPECT(opt.get_step() == 1, "clip_and_step(): advances the step counter");
        opt.norm_includes_workspace = true;
        const float norm_ws = opt.clip_and_step(&grads, 1.0f);
        EXPECT(fabs(norm_ws - sqrt(ss + ss_ws)) <= 1e-5 * sqrt(ss + ss_ws), "clip_and_step(): norm with the workspace counted in");
        opt.norm_includes_workspace = false;
        opt.freeze_embed = true;
        double ss_frozen = 0.0;
        for (size_t i = 0; i < proj_n; i++) ss_frozen += (double)__half2float(g16[i]) * __half2float(g16[i]);
        for (size_t i = 0; i < n32; i++) ss_frozen += (double)g32[i] * g32[i];
        const float norm_frozen = opt.clip_and_step(&grads, 1.0f);
        EXPECT(fabs(norm_frozen - sqrt(ss_frozen)) <= 1e-5 * sqrt(ss_frozen), "clip_and_step(): frozen embedding leaves the norm");
        // move construction keeps the state usable
        AdamWOptimizer moved(std::move(opt));
        moved.step(&grads);
        CUDA_CHECK(cudaDeviceSynchronize());
        EXPECT(moved.get_step() == 4, "move construction keeps state and step counter");
    }

    // ---- weight_decay is a public field: a change between steps takes effect, as in RL.cu,
    //      which hands the field to the launcher on every step (optimizer.h:126-129)
    upload();
    {
        AdamWOptimizer opt(&model, 1e-3f, 0.9f, 0.999f, 1e-8f, 0.01f);
        opt.step(&grads);
        opt.weight_decay = 0.1f;
        opt.step(&grads);
        CUDA_CHECK(cudaDeviceSynchronize());
        auto p_b = download(model.weights.fp16_pool, n16);
        auto master_b = download(opt.fp16_master(), n16);
        upload();
        float *master, *m, *v;
        CUDA_CHECK(cudaMalloc(&master, n16 * 4)); CUDA_CHECK(cudaMalloc(&m, n16 * 4)); CUDA_CHECK(cudaMalloc(&v, n16 * 4));
        CUDA_CHECK(cudaMemset(m, 0, n16 * 4)); CUDA_CHECK(cudaMemset(v, 0, n16 * 4));
        std::vector<float> mh(n16);
        for (size_t i = 0; i < n16; i++) mh[i] = __half2float(w16[i]);
        CUDA_CHECK(cudaMemcpy(master, mh.data(), n16 * 4, cudaMemcpyHostToDevice));
        const float wds[2] = {0.01f, 0.1f};
        for (int s = 1; s <= 2; s++) {
            const float bc1 = 1.0f - powf(0.9f, (float)s), bc2 = 1.0f - powf(0.999f, (float)s);
            launch_adamw_fp16(master, model.weights.fp16_pool, grads.half_pool, m, v, (int)proj_n,
                              1e-3f, 0.9f, 0.999f, 1e-8f, wds[s - 1], bc1, bc2);
            launch_adamw_fp16(master + proj_n, model.weights.fp16_pool + proj_n, grads.half_pool + proj_n,
                              m + proj_n, v + proj_n, (int)(n16 - proj_n), 1e-3f, 0.9f, 0.999f, 1e-8f, 0.0f, bc1, bc2);
        }
        CUDA_CHECK(cudaDeviceSynchronize());
        EXPECT(same(p_b, download(model.weights.fp16_pool, n16)) && same(master_b, download(master, n16)),
               "weight_decay changed between steps is honoured");
        cudaFree(master); cudaFree(m); cudaFree(v);
    }

    // ---- a step with a non-finite gradient writes nothing and does not count
    upload();
    {
        AdamWOptimizer opt(&model, 1e-3f);
        opt.clip_and_step(&grads, 1.0f);
        auto p_before = download(model.weights.fp16_pool, n16);
        const half inf = __float2half(INFINITY);
        CUDA_CHECK(cudaMemcpy(grads.half_pool + 5, &inf, sizeof(half), cudaMemcpyHostToDevice));
        opt.clip_and_step_async(&grads, 1.0f);
        EXPECT(opt.last_step_skipped() && opt.get_step() == 1, "skipped step leaves the step counter");
        EXPECT(same(p_before, download(model.weights.fp16_pool, n16)), "skipped step leaves the weights");
        CUDA_CHECK(cudaMemcpy(grads.half_pool + 5, &g16[5], sizeof(half), cudaMemcpyHostToDevice));
        opt.clip_and_step(&grads, 1.0f);
        EXPECT(!opt.last_step_skipped() && opt.get_step() == 2, "the next clean step is step 2");
    }

    printf("%d failure(s)\n", failures);
    return failures;
}

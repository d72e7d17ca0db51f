// AdamW optimizer object over librlcu_b200, with the public interface of RL.cu's
// AdamWOptimizer (include/training/optimizer.h:59-274 of RL.cu): same constructor,
// same public hyper-parameter fields, same accessors, same step() call.  What is
// different is underneath: step() is one launch over a three-entry tensor list
// instead of three launches, and clip_and_step() folds Trainer::clip_grad_norm_
// (include/training/trainer.h:323-352) into two launches without the blocking
// read-back in the middle of the step.
//
// The class is a template over the model and gradient types so that it can be
// built without RL.cu's headers; include/training/optimizer.h instantiates it for
// RL.cu's Qwen3Model / Qwen3Gradients.  Only these members are used:
//   model->config.{num_hidden_layers, hidden_size, q_dim, kv_dim,
//                  intermediate_size, vocab_size, head_dim}
//   model->weights.{fp16_pool, fp32_pool, fp16_pool_elems, fp32_pool_elems}
//   grads->{half_pool, float_pool, float_pool_bytes}
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "rlcu_adamw.h"

namespace rlcu_host {

// RL.cu's call sites stop the process on a CUDA error (optimizer.h:13-22); the
// mirror does the same for a failed library call.
inline void check(int rc, const char* what) {
    if (rc != RLCU_OK) {
        fprintf(stderr, "[AdamW] %s failed: %s\n", what, rlcu_last_error());
        exit(1);
    }
}

inline void check_cuda(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        fprintf(stderr, "[AdamW] %s failed: %s\n", what, cudaGetErrorString(e));
        exit(1);
    }
}

template <class Model, class Grads>
class BasicAdamWOptimizer {
public:
    // hyper-parameters, public as in RL.cu
    float lr;
    float beta1;
    float beta2;
    float eps;
    float weight_decay;

    // Treat the embedding gradient as zero without reading it (RL.cu zeroes it with
    // a 311 MB memset when freeze_embed is set, trainer.h:271-277).
    bool freeze_embed = false;
    // Count the attention workspace that follows the norm gradients in RL.cu's FP32
    // gradient pool in the clip norm, as RL.cu's clip does (trainer.h:331).
    bool norm_includes_workspace = false;

    BasicAdamWOptimizer() : lr(1e-5f), beta1(0.9f), beta2(0.999f), eps(1e-8f), weight_decay(0.01f) {}

    BasicAdamWOptimizer(Model* model, float lr = 1e-4f, float beta1 = 0.9f, float beta2 = 0.999f,
                        float eps = 1e-8f, float weight_decay = 0.01f)
        : lr(lr), beta1(beta1), beta2(beta2), eps(eps), weight_decay(weight_decay) {
        init(model);
    }

    ~BasicAdamWOptimizer() { release(); }

    BasicAdamWOptimizer(const BasicAdamWOptimizer&) = delete;
    BasicAdamWOptimizer& operator=(const BasicAdamWOptimizer&) = delete;
    BasicAdamWOptimizer(BasicAdamWOptimizer&& o) noexcept { take(o); }
    BasicAdamWOptimizer& operator=(BasicAdamWOptimizer&& o) noexcept {
        if (this != &o) {
            release();
            take(o);
        }
        return *this;
    }

    void set_lr(float new_lr) { lr = new_lr; }
    // Adam step counter t.  A step that clip_and_step found non-finite gradients in wrote
    // nothing and does not count; the counter is settled when that step's record is read.
    int get_step() const {
        settle();
        return step_;
    }

    float* fp16_master() { return master_; }
    float* fp16_m() { return m16_; }
    float* fp16_v() { return v16_; }
    float* fp32_m() { return m32_; }
    float* fp32_v() { return v32_; }
    size_t num_fp16_params() const { return n16_; }
    size_t num_fp32_params() const { return n32_; }

    // proj: 0=q 1=k 2=v 3=o 4=gate 5=up 6=down;  norm: 0=input 1=q 2=k 3=post_attn
    float* get_fp16_master(int layer, int proj) const { return master_ + offset16(layer, proj); }
    float* get_fp16_m(int layer, int proj) const { return m16_ + offset16(layer, proj); }
    float* get_fp16_v(int layer, int proj) const { return v16_ + offset16(layer, proj); }
    float* get_fp32_m_norm(int layer, int norm) const { return m32_ + offset32(layer, norm); }
    float* get_fp32_v_norm(int layer, int norm) const { return v32_ + offset32(layer, norm); }
    float* get_final_norm_m() const { return m32_ + layer32_ * layers_; }
    float* get_final_norm_v() const { return v32_ + layer32_ * layers_; }

    // AdamWOptimizer::step of RL.cu (optimizer.h:119-147): no clipping here.
    void step(Grads* grads, cudaStream_t stream = 0) {
        settle();
        bind(grads);
        step_++;
        const rlcu_hparams hp = hparams();
        check(rlcu_adamw_multi_step(list_, &hp, nullptr, 0, stream), "rlcu_adamw_multi_step");
    }

    // clip_grad_norm_ + step in two launches.  The gradients are left as they
    // are (RL.cu scales them in place); the clip factor is applied in registers
    // with the same FP16 re-rounding.  max_norm <= 0 disables the clip
    // (trainer.h:280).  Nothing here waits for the GPU.
    void clip_and_step_async(Grads* grads, float max_norm, cudaStream_t stream = 0) {
        settle();
        bind(grads);
        step_++;
        const rlcu_hparams hp = hparams();
        check(rlcu_gradstat(list_, 1.0f, max_norm, nullptr, d_stat_, 0, stream), "rlcu_gradstat");
        check(rlcu_adamw_multi_step(list_, &hp, d_stat_, RLCU_STEP_ROUND_CLIP_FP16, stream),
              "rlcu_adamw_multi_step");
        check_cuda(cudaMemcpyAsync(h_stat_, d_stat_, sizeof(rlcu_stat), cudaMemcpyDeviceToHost, stream),
                   "statistics read-back");
        check_cuda(cudaEventRecord(stat_ready_, stream), "cudaEventRecord");
        pending_ = true;
    }

    // The pre-clip gradient norm of the last clip_and_step_async (what RL.cu logs
    // as grad_norm, trainer.h:322, 351).  Waits only for that step's record.
    float last_grad_norm() {
        settle();
        return h_stat_->norm;
    }
    // Whether the last clip_and_step found an inf/NaN gradient and therefore wrote nothing.
    bool last_step_skipped() {
        settle();
        return h_stat_->found_inf != 0;
    }

    // Same, returning the norm at once like Trainer::clip_grad_norm_ does.
    float clip_and_step(Grads* grads, float max_norm, cudaStream_t stream = 0) {
        clip_and_step_async(grads, max_norm, stream);
        return last_grad_norm();
    }

    const rlcu_stat* device_stat() const { return d_stat_; }

private:
    Model* model_ = nullptr;
    mutable int step_ = 0;
    int layers_ = 0;
    float* state16_ = nullptr;   // one allocation: [master | m | v], as optimizer.h:224-236
    float* state32_ = nullptr;   // one allocation: [m | v]
    float *master_ = nullptr, *m16_ = nullptr, *v16_ = nullptr, *m32_ = nullptr, *v32_ = nullptr;
    size_t n16_ = 0, n32_ = 0, proj_n_ = 0, layer16_ = 0, layer32_ = 0;
    size_t proj_[7] = {}, norm_[4] = {};
    rlcu_tensor_list* list_ = nullptr;
    const void* bound_half_ = nullptr;
    const void* bound_float_ = nullptr;
    bool bound_freeze_ = false, bound_workspace_ = false;
    float bound_wd_ = 0.0f;
    mutable bool pending_ = false;             // a clip_and_step record has not been looked at yet
    rlcu_stat* d_stat_ = nullptr;
    rlcu_stat* h_stat_ = nullptr;      // pinned
    cudaEvent_t stat_ready_ = nullptr;

    // Waits for the record of the last clip_and_step (already there in a training loop, which
    // logs the norm of every step) and takes a skipped step back out of the counter, so that
    // bias correction follows the steps that were applied.
    void settle() const {
        if (!pending_) return;
        check_cuda(cudaEventSynchronize(stat_ready_), "cudaEventSynchronize");
        pending_ = false;
        if (h_stat_->found_inf) step_--;
    }

    rlcu_hparams hparams() const {
        rlcu_hparams hp;
        hp.lr = lr; hp.beta1 = beta1; hp.beta2 = beta2; hp.eps = eps;
        hp.bias_correction1 = rlcu_bias_correction(beta1, step_);     // optimizer.h:121-122
        hp.bias_correction2 = rlcu_bias_correction(beta2, step_);
        return hp;
    }

    size_t offset16(int layer, int proj) const {
        size_t off = (size_t)layer * layer16_;
        for (int p = 0; p < proj; p++) off += proj_[p];
        return off;
    }
    size_t offset32(int layer, int norm) const {
        size_t off = (size_t)layer * layer32_;
        for (int k = 0; k < norm; k++) off += norm_[k];
        return off;
    }

    void init(Model* model) {
        model_ = model;
        const auto& c = model->config;
        layers_ = c.num_hidden_layers;
        const size_t H = (size_t)c.hidden_size;
        // pool order: per layer [q k v o gate up down], then the embedding (weights.h:43-61)
        proj_[0] = (size_t)c.q_dim * H;
        proj_[1] = proj_[2] = (size_t)c.kv_dim * H;
        proj_[3] = H * (size_t)c.q_dim;
        proj_[4] = proj_[5] = (size_t)c.intermediate_size * H;
        proj_[6] = H * (size_t)c.intermediate_size;
        layer16_ = 0;
        for (size_t s : proj_) layer16_ += s;
        proj_n_ = layer16_ * (size_t)layers_;
        n16_ = proj_n_ + (size_t)c.vocab_size * H;
        norm_[0] = norm_[3] = H;
        norm_[1] = norm_[2] = (size_t)c.head_dim;
        layer32_ = 0;
        for (size_t s : norm_) layer32_ += s;
        n32_ = layer32_ * (size_t)layers_ + H;
        if (n16_ != model->weights.fp16_pool_elems || n32_ != model->weights.fp32_pool_elems) {
            fprintf(stderr, "[AdamW] pool sizes (%zu, %zu) do not match the configuration (%zu, %zu)\n",
                    (size_t)model->weights.fp16_pool_elems, (size_t)model->weights.fp32_pool_elems, n16_, n32_);
            exit(1);
        }
        check_cuda(cudaMalloc(&state16_, n16_ * 3 * sizeof(float)), "cudaMalloc");
        check_cuda(cudaMalloc(&state32_, n32_ * 2 * sizeof(float)), "cudaMalloc");
        check_cuda(cudaMemset(state16_, 0, n16_ * 3 * sizeof(float)), "cudaMemset");
        check_cuda(cudaMemset(state32_, 0, n32_ * 2 * sizeof(float)), "cudaMemset");
        master_ = state16_;
        m16_ = master_ + n16_;
        v16_ = m16_ + n16_;
        m32_ = state32_;
        v32_ = m32_ + n32_;
        check(rlcu_half_to_float(master_, model->weights.fp16_pool, (int64_t)n16_, 0), "rlcu_half_to_float");
        check_cuda(cudaMalloc(&d_stat_, sizeof(rlcu_stat)), "cudaMalloc");
        check_cuda(cudaMallocHost(&h_stat_, sizeof(rlcu_stat)), "cudaMallocHost");
        memset(h_stat_, 0, sizeof(rlcu_stat));
        check_cuda(cudaEventCreateWithFlags(&stat_ready_, cudaEventDisableTiming), "cudaEventCreate");
        check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        printf("[AdamW] optimizer state ready: %zu FP16 parameters with FP32 master/m/v (%.1f MB), "
               "%zu FP32 parameters with m/v (%.2f MB); lr %.1e, weight decay %.2f\n",
               n16_, n16_ * 12 / (1024.0 * 1024.0), n32_, n32_ * 8 / (1024.0 * 1024.0), lr, weight_decay);
    }

    // (Re)builds the tensor list when the gradient pools or a switch changed.
    // RL.cu allocates its gradient pools once, so this runs on the first step only.
    void bind(Grads* grads) {
        if (list_ && bound_half_ == grads->half_pool && bound_float_ == grads->float_pool &&
            bound_freeze_ == freeze_embed && bound_workspace_ == norm_includes_workspace &&
            bound_wd_ == weight_decay)
            return;
        if (list_) check(rlcu_tensor_list_destroy(list_), "rlcu_tensor_list_destroy");
        list_ = nullptr;
        half* w16 = model_->weights.fp16_pool;
        half* g16 = grads->half_pool;
        float* w32 = model_->weights.fp32_pool;
        float* g32 = (float*)grads->float_pool;
        rlcu_tensor_desc d[4];
        memset(d, 0, sizeof(d));
        // projections, with weight decay (optimizer.h:125-129)
        d[0].param = w16; d[0].grad = g16; d[0].m = m16_; d[0].v = v16_; d[0].master = master_;
        d[0].n = proj_n_; d[0].weight_decay = weight_decay; d[0].dtype = RLCU_F16;
        // embedding, no weight decay (optimizer.h:131-140)
        d[1].param = w16 + proj_n_; d[1].grad = g16 + proj_n_; d[1].m = m16_ + proj_n_; d[1].v = v16_ + proj_n_;
        d[1].master = master_ + proj_n_; d[1].n = n16_ - proj_n_; d[1].weight_decay = 0.0f; d[1].dtype = RLCU_F16;
        d[1].flags = freeze_embed ? RLCU_TENSOR_GRAD_ZERO : 0;
        // norm weights, FP32, no weight decay (optimizer.h:142-146)
        d[2].param = w32; d[2].grad = g32; d[2].m = m32_; d[2].v = v32_; d[2].n = n32_; d[2].dtype = RLCU_F32;
        uint64_t count = 3;
        const size_t pool32 = grads->float_pool_bytes / sizeof(float);
        if (norm_includes_workspace && pool32 > n32_) {
            d[3].grad = g32 + n32_; d[3].n = pool32 - n32_; d[3].dtype = RLCU_F32;
            d[3].flags = RLCU_TENSOR_NORM_ONLY;
            count = 4;
        }
        // the weight-decay value is baked into the list, so a change of the public field
        // rebuilds it (RL.cu passes weight_decay to the launcher on every step, optimizer.h:126-129)
        check(rlcu_tensor_list_create(d, count, &list_), "rlcu_tensor_list_create");
        bound_wd_ = weight_decay;
        bound_half_ = grads->half_pool;
        bound_float_ = grads->float_pool;
        bound_freeze_ = freeze_embed;
        bound_workspace_ = norm_includes_workspace;
    }

    void release() {
        if (list_) rlcu_tensor_list_destroy(list_);
        if (state16_) cudaFree(state16_);
        if (state32_) cudaFree(state32_);
        if (d_stat_) cudaFree(d_stat_);
        if (h_stat_) cudaFreeHost(h_stat_);
        if (stat_ready_) cudaEventDestroy(stat_ready_);
        list_ = nullptr;
        state16_ = state32_ = master_ = m16_ = v16_ = m32_ = v32_ = nullptr;
        d_stat_ = h_stat_ = nullptr;
        stat_ready_ = nullptr;
    }

    void take(BasicAdamWOptimizer& o) {
        memcpy((void*)this, (void*)&o, sizeof(*this));
        o.list_ = nullptr;
        o.state16_ = o.state32_ = o.master_ = o.m16_ = o.v16_ = o.m32_ = o.v32_ = nullptr;
        o.d_stat_ = o.h_stat_ = nullptr;
        o.stat_ready_ = nullptr;
    }
};

}  // namespace rlcu_host

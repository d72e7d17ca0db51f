/*
 * CPU oracle for the AdamW / gradient-clip optimizer path of RL.cu.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the reference's
 * algorithm, used as the checker in the test-suite, in the smoke check and as
 * the timed CPU baseline of the benchmark.  No product code path may call it:
 * the CUDA library never links or loads this file.
 *
 * Parity status.  The AdamW update functions are pinned against outputs of the
 * reference's own CUDA kernels (src/kernels/adamw.cu compiled unmodified and
 * run on a B200; fixtures under tests/golden/).  The gradient norm / clip
 * functions are pinned the same way against the reference's static kernels in
 * include/training/trainer.h.  The loss-scale state machine, the non-finite
 * skip and the sharded step have NO counterpart in the reference: for those
 * rows the header says "parity unpinned" and the oracle restates the published
 * dynamic-loss-scaling recipe (halve on overflow, double after a growth
 * interval of clean steps, skipped steps do not advance the Adam step counter).
 *
 * Reference lines restated (paths inside the RL.cu tree):
 *   src/kernels/adamw.cu:22-39      FP16-with-master element update
 *   src/kernels/adamw.cu:52-53      host-side 1/bias_correction in FP32
 *   src/kernels/adamw.cu:77-90      FP32 element update
 *   include/training/optimizer.h:120-122  step counter and powf bias correction
 *   include/training/trainer.h:103-133    sum of squares (FP32 accumulate)
 *   include/training/trainer.h:136-145    in-place scale (FP16 re-rounded)
 *   include/training/trainer.h:339-349    sqrtf, clip threshold, +1e-6
 *   tests/test_adamw.cu:195-206, 283-293  the reference's own CPU check loops
 */
#ifndef RLCU_ADAMW_ORACLE_H
#define RLCU_ADAMW_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Rounding model of the expression tree of adamw.cu:25-36.  A bit field: which
 * of the four multiply-add sites is contracted into a single fma.
 *   bits 0-1  m = b1*m + (1-b1)*g     0 two roundings, 1 fma(b1,m,.), 2 fma(1-b1,g,.)
 *   bits 2-3  v = b2*v + (1-b2)*g*g   0 two roundings, 1 fma(b2,v,.), 2 fma((1-b2)*g,g,.)
 *   bit  4    w*decay - q             1 fma(w,decay,-q)
 *   bit  5    decay = 1 - lr*wd       1 fma(-lr,wd,1)
 * ORC_UNFUSED is the reference's host-side check loop (tests/test_adamw.cu:283-293,
 * built without FMA contraction).  ORC_NVCC is what the reference's CUDA kernel
 * computes when src/kernels/adamw.cu is built for sm_100a with CUDA 12.9 at its
 * default -fmad=true; it was found by matching that binary's output bit for bit
 * on a B200 (fixtures under tests/golden/), not by reading machine code.  Bit 5
 * cannot be told apart by any input tried (1 - lr*wd rounds the same both ways). */
#define ORC_ROUNDING(m_mode, v_mode, w_fused, d_fused) \
    ((m_mode) | ((v_mode) << 2) | ((w_fused) << 4) | ((d_fused) << 5))
enum { ORC_UNFUSED = 0, ORC_NVCC = ORC_ROUNDING(2, 2, 0, 0) };

/* element kinds and flags; binary-compatible with rlcu_tensor_desc */
enum { ORC_F16 = 0, ORC_F32 = 1, ORC_BF16 = 2 };   /* BF16: no reference counterpart, parity unpinned */
enum { ORC_FLAG_NORM_ONLY = 1u, ORC_FLAG_GRAD_ZERO = 2u };
/* gradient kind: as the parameter, or FP32 for a 16-bit parameter (no reference counterpart:
 * the reference accumulates FP16 gradients, src/kernels/linear.cu:85-98; parity unpinned) */
enum { ORC_GRAD_AS_PARAM = 0u, ORC_GRAD_F32 = 1u };
enum { ORC_STEP_ROUND_CLIP_FP16 = 1u };

typedef struct orc_tensor {
    void*       param;    /* uint16_t* (IEEE binary16 bits) or float*          */
    const void* grad;     /* same element kind as param, or float* (ORC_GRAD_F32) */
    float*      m;
    float*      v;
    float*      master;   /* FP32 master copy or NULL (F16 only)               */
    uint64_t    n;
    float       weight_decay;
    uint32_t    dtype;
    uint32_t    flags;
    uint32_t    grad_dtype;
} orc_tensor;

typedef struct orc_hparams {
    float lr, beta1, beta2, eps;
    float bias_correction1;   /* 1 - beta1^t, NOT its inverse (adamw.cuh:36-37) */
    float bias_correction2;
} orc_hparams;

typedef struct orc_stat {
    double   sum_sq;       /* sum of (g * unscale)^2 over every listed tensor   */
    float    norm;         /* sqrtf((float)sum_sq)                              */
    float    coef;         /* factor the update multiplies each gradient by     */
    uint32_t found_inf;    /* 1 if any gradient element is inf or NaN           */
    uint32_t clip_active;  /* 1 if norm > max_norm                              */
} orc_stat;

typedef struct orc_scaler {
    float   scale;
    int32_t growth_tracker;
    int32_t step;          /* Adam step counter t; advanced on clean steps only */
    int32_t skipped;       /* count of skipped (overflowed) steps               */
} orc_scaler;

/* binary16 <-> binary32, round-to-nearest-even, subnormals preserved */
uint16_t orc_f2h(float f);
float    orc_h2f(uint16_t h);
void     orc_f2h_array(const float* src, uint16_t* dst, int64_t n);
void     orc_h2f_array(const uint16_t* src, float* dst, int64_t n);
/* The same two conversions through the CPU's F16C instructions when the build and the CPU
 * have them (else they fall back to the functions above).  The update and norm loops use
 * these by default; orc_use_hw_half(0) switches them to the bit-level definition. */
uint16_t orc_f2h_hw(float f);
float    orc_h2f_hw(uint16_t h);
int      orc_hw_half_available(void);
void     orc_use_hw_half(int on);
/* bfloat16 <-> binary32, round-to-nearest-even (NaN kept quiet) */
uint16_t orc_f2bf(float f);
float    orc_bf2f(uint16_t b);
void     orc_f2bf_array(const float* src, uint16_t* dst, int64_t n);
void     orc_bf2f_array(const uint16_t* src, float* dst, int64_t n);

/* include/training/optimizer.h:121-122 */
float orc_bias_correction(float beta, int step);

/* src/kernels/adamw.cu:7-58 (launch_adamw_fp16) */
void orc_adamw_fp16_master(float* master_w, uint16_t* model_w, const uint16_t* grad,
                           float* m, float* v, int64_t n,
                           float lr, float beta1, float beta2, float eps, float weight_decay,
                           float bias_correction1, float bias_correction2,
                           int rounding, int threads);
/* same arithmetic, weight read from the FP16 parameter instead of a master copy */
void orc_adamw_fp16(uint16_t* param, const uint16_t* grad, float* m, float* v, int64_t n,
                    float lr, float beta1, float beta2, float eps, float weight_decay,
                    float bias_correction1, float bias_correction2,
                    int rounding, int threads);
/* src/kernels/adamw.cu:63-108 (launch_adamw_fp32) */
void orc_adamw_fp32(float* w, const float* grad, float* m, float* v, int64_t n,
                    float lr, float beta1, float beta2, float eps, float weight_decay,
                    float bias_correction1, float bias_correction2,
                    int rounding, int threads);

/* include/training/trainer.h:103-133; accumulation in FP64 (the reference's
 * FP32 atomic order is unspecified, so the oracle gives the exact sum) of squares
 * taken in FP32 as the reference takes them.  Elements that are inf or NaN are left
 * out of the sum and reported by orc_count_nonfinite_*; a finite FP32 element whose
 * square overflows FP32 makes the sum +inf (norm +inf, a clip then scales to zero),
 * which is what the reference's kernels do with it, and is NOT an overflowed step. */
double orc_sum_sq_half(const uint16_t* g, int64_t n, float unscale, int threads);
double orc_sum_sq_float(const float* g, int64_t n, float unscale, int threads);
double orc_sum_sq_bf16(const uint16_t* g, int64_t n, float unscale, int threads);
int64_t orc_count_nonfinite_half(const uint16_t* g, int64_t n);
int64_t orc_count_nonfinite_float(const float* g, int64_t n);
/* include/training/trainer.h:136-145 */
void orc_scale_half(uint16_t* g, int64_t n, float scale, int threads);
void orc_scale_float(float* g, int64_t n, float scale, int threads);
/* include/training/trainer.h:323-352: returns the pre-clip norm, scales in place */
float orc_clip_grad_norm(uint16_t* half_pool, int64_t n16, float* float_pool, int64_t n32,
                         float max_norm, int threads);

/* fused statistics pass over a tensor list (unscale, non-finite, norm, clip factor).
 * extra_sum_sq / extra_found_inf carry other ranks' contributions in the sharded step. */
void orc_gradstat(const orc_tensor* t, uint64_t count, float unscale, float max_norm,
                  double extra_sum_sq, uint32_t extra_found_inf, int threads,
                  orc_stat* out);
/* finish a statistics record from a total sum and flag (trainer.h:341-344) */
void orc_gradstat_finalize(double sum_sq, uint32_t found_inf, float unscale, float max_norm,
                           orc_stat* out);
/* multi-tensor update consuming the statistics record; returns 1 if skipped */
int orc_multi_step(const orc_tensor* t, uint64_t count, const orc_hparams* hp,
                   const orc_stat* stat, uint32_t step_flags, int rounding, int threads);
/* dynamic loss scale: halve on overflow, double after growth_interval clean steps */
void orc_scaler_update(orc_scaler* s, uint32_t found_inf, int growth_interval);

#ifdef __cplusplus
}
#endif
#endif

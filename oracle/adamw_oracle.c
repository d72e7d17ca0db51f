/*
 * CPU oracle for the AdamW / gradient-clip optimizer path of RL.cu.
 * TEST INFRASTRUCTURE ONLY -- see adamw_oracle.h for the parity status and the
 * list of reference lines each function restates.
 *
 * Build: gcc -O2 -ffp-contract=off -mavx2 -mfma -mf16c -fopenmp -shared -fPIC
 * (-ffp-contract=off keeps the compiler from fusing on its own; the rounding
 * models call fmaf() explicitly at the sites they contract.)
 */
#include "adamw_oracle.h"

#include <math.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif
#ifdef __F16C__
#include <immintrin.h>
#endif

/* ------------------------------------------------------------------ */
/* binary16 <-> binary32                                               */
/* ------------------------------------------------------------------ */

static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

float orc_h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0x1Fu) return bits_f32(sign | 0x7F800000u | (man << 13));   /* inf / NaN */
    if (exp != 0) return bits_f32(sign | ((exp + 112u) << 23) | (man << 13));
    if (man == 0) return bits_f32(sign);
    /* subnormal: value = man * 2^-24, exact in binary32 */
    float mag = (float)man * 5.9604644775390625e-08f;
    return bits_f32(sign | f32_bits(mag));
}

uint16_t orc_f2h(float f) {
    uint32_t x = f32_bits(f);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) {                       /* inf or NaN */
        if (ax == 0x7F800000u) return (uint16_t)(sign | 0x7C00u);
        return (uint16_t)(sign | 0x7FFFu);         /* canonical NaN, as __float2half */
    }
    if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);  /* rounds to >= 65520 -> inf */
    if (ax < 0x33000001u) return sign;             /* <= 2^-25 rounds to zero (tie to even) */
    uint32_t e = ax >> 23;
    uint32_t man = (ax & 0x7FFFFFu) | 0x800000u;   /* 24-bit significand */
    uint32_t shift, half_exp;
    if (e >= 113u) { shift = 13u; half_exp = e - 112u; }       /* normal binary16 */
    else { shift = 126u - e; half_exp = 0u; }                  /* subnormal: 14..24 */
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1u);
    if (rem > halfway || (rem == halfway && (q & 1u))) q++;
    /* normal: q has the implicit bit at 1<<10; adding (half_exp-1)<<10 merges it
       and lets a mantissa carry bump the exponent.  subnormal: q is the field,
       a carry to 1<<10 is exactly the smallest normal. */
    uint32_t h = half_exp ? (((half_exp - 1u) << 10) + q) : q;
    return (uint16_t)(sign | h);
}

/* The loops below convert through H2F / F2H.  When the build has F16C and the CPU running
 * it does too, these use the hardware conversion instructions (what any tuned CPU code
 * would use, so that the timed CPU baseline is not slowed down by bit arithmetic); the
 * bit-level functions above remain the definition, and tests/test_oracle.py checks the
 * two against each other on every binary16 value and on a large sample of floats.
 * orc_use_hw_half(0) forces the bit-level path. */
static int g_hw_half = -1;

int orc_hw_half_available(void) {
#ifdef __F16C__
    return __builtin_cpu_supports("f16c") ? 1 : 0;
#else
    return 0;
#endif
}

void orc_use_hw_half(int on) { g_hw_half = (on && orc_hw_half_available()) ? 1 : 0; }

static inline int hw_half(void) {
    if (g_hw_half < 0) g_hw_half = orc_hw_half_available();
    return g_hw_half;
}

#ifdef __F16C__
static inline float hw_h2f(uint16_t h) { return _cvtsh_ss(h); }
static inline uint16_t hw_f2h(float f) {
    if (f != f) return (uint16_t)(((f32_bits(f) >> 16) & 0x8000u) | 0x7FFFu);   /* canonical NaN, as __float2half */
    return (uint16_t)_cvtss_sh(f, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC);
}
#define H2F(h) (hw ? hw_h2f(h) : orc_h2f(h))
#define F2H(f) (hw ? hw_f2h(f) : orc_f2h(f))
#else
#define H2F(h) orc_h2f(h)
#define F2H(f) orc_f2h(f)
#endif

uint16_t orc_f2h_hw(float f) {
#ifdef __F16C__
    if (orc_hw_half_available()) return hw_f2h(f);
#endif
    return orc_f2h(f);
}
float orc_h2f_hw(uint16_t h) {
#ifdef __F16C__
    if (orc_hw_half_available()) return hw_h2f(h);
#endif
    return orc_h2f(h);
}

void orc_f2h_array(const float* src, uint16_t* dst, int64_t n) {
    for (int64_t i = 0; i < n; i++) dst[i] = orc_f2h(src[i]);
}
void orc_h2f_array(const uint16_t* src, float* dst, int64_t n) {
    for (int64_t i = 0; i < n; i++) dst[i] = orc_h2f(src[i]);
}

float orc_bf2f(uint16_t b) { return bits_f32((uint32_t)b << 16); }

uint16_t orc_f2bf(float f) {
    uint32_t x = f32_bits(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)0x7FFFu;      /* NaN, as __float2bfloat16_rn */
    x += 0x7FFFu + ((x >> 16) & 1u);                                    /* round to nearest even */
    return (uint16_t)(x >> 16);
}

void orc_f2bf_array(const float* src, uint16_t* dst, int64_t n) {
    for (int64_t i = 0; i < n; i++) dst[i] = orc_f2bf(src[i]);
}
void orc_bf2f_array(const uint16_t* src, float* dst, int64_t n) {
    for (int64_t i = 0; i < n; i++) dst[i] = orc_bf2f(src[i]);
}

/* ------------------------------------------------------------------ */
/* the element update                                                  */
/* ------------------------------------------------------------------ */

float orc_bias_correction(float beta, int step) {
    return 1.0f - powf(beta, (float)step);         /* optimizer.h:121-122 */
}

typedef struct { float lr, b1, b2, eps, wd, bc1_inv, bc2_inv; } orc_k;

static inline orc_k make_k(float lr, float b1, float b2, float eps, float wd, float bc1, float bc2) {
    orc_k k = { lr, b1, b2, eps, wd, 1.0f / bc1, 1.0f / bc2 };   /* adamw.cu:52-53 */
    return k;
}

/* adamw.cu:24-36 under a rounding model (see ORC_* in the header): each of the
 * four multiply-add sites is either rounded twice or contracted into one fma. */
static inline float upd(float w, float g, float* m, float* v, const orc_k* k, int rounding) {
    const int m_mode = rounding & 3, v_mode = (rounding >> 2) & 3;
    const int w_fused = (rounding >> 4) & 1, d_fused = (rounding >> 5) & 1;
    const float omb1 = 1.0f - k->b1, omb2 = 1.0f - k->b2;
    float mi, vi;
    if (m_mode == 1) mi = fmaf(k->b1, *m, omb1 * g);          /* fma(b1, m, (1-b1)*g)   */
    else if (m_mode == 2) mi = fmaf(omb1, g, k->b1 * *m);     /* fma(1-b1, g, b1*m)     */
    else mi = k->b1 * *m + omb1 * g;
    const float t = omb2 * g;                                 /* (1-b2)*g*g is left-assoc */
    if (v_mode == 1) vi = fmaf(k->b2, *v, t * g);             /* fma(b2, v, t*g)        */
    else if (v_mode == 2) vi = fmaf(t, g, k->b2 * *v);        /* fma(t, g, b2*v)        */
    else vi = k->b2 * *v + t * g;
    *m = mi; *v = vi;
    const float m_hat = mi * k->bc1_inv;
    const float v_hat = vi * k->bc2_inv;
    const float decay = d_fused ? fmaf(-k->lr, k->wd, 1.0f) : 1.0f - k->lr * k->wd;
    const float q = (k->lr * m_hat) / (sqrtf(v_hat) + k->eps);
    return w_fused ? fmaf(w, decay, -q) : w * decay - q;
}

static int pick_threads(int threads) {
#ifdef _OPENMP
    if (threads <= 0) return omp_get_max_threads();
    return threads;
#else
    (void)threads; return 1;
#endif
}

void orc_adamw_fp16_master(float* master_w, uint16_t* model_w, const uint16_t* grad,
                           float* m, float* v, int64_t n,
                           float lr, float beta1, float beta2, float eps, float weight_decay,
                           float bc1, float bc2, int rounding, int threads) {
    if (n <= 0) return;                            /* adamw.cu:49 */
    orc_k k = make_k(lr, beta1, beta2, eps, weight_decay, bc1, bc2);
    int nt = pick_threads(threads);
    const int hw = hw_half(); (void)hw;
    #pragma omp parallel for num_threads(nt) schedule(static)
    for (int64_t i = 0; i < n; i++) {
        float w = upd(master_w[i], H2F(grad[i]), &m[i], &v[i], &k, rounding);
        master_w[i] = w;
        model_w[i] = F2H(w);
    }
}

void orc_adamw_fp16(uint16_t* param, const uint16_t* grad, float* m, float* v, int64_t n,
                    float lr, float beta1, float beta2, float eps, float weight_decay,
                    float bc1, float bc2, int rounding, int threads) {
    if (n <= 0) return;
    orc_k k = make_k(lr, beta1, beta2, eps, weight_decay, bc1, bc2);
    int nt = pick_threads(threads);
    const int hw = hw_half(); (void)hw;
    #pragma omp parallel for num_threads(nt) schedule(static)
    for (int64_t i = 0; i < n; i++) {
        float w = upd(H2F(param[i]), H2F(grad[i]), &m[i], &v[i], &k, rounding);
        param[i] = F2H(w);
    }
}

void orc_adamw_fp32(float* w, const float* grad, float* m, float* v, int64_t n,
                    float lr, float beta1, float beta2, float eps, float weight_decay,
                    float bc1, float bc2, int rounding, int threads) {
    if (n <= 0) return;                            /* adamw.cu:99 */
    orc_k k = make_k(lr, beta1, beta2, eps, weight_decay, bc1, bc2);
    int nt = pick_threads(threads);
    #pragma omp parallel for num_threads(nt) schedule(static)
    for (int64_t i = 0; i < n; i++)
        w[i] = upd(w[i], grad[i], &m[i], &v[i], &k, rounding);
}

/* ------------------------------------------------------------------ */
/* gradient norm and clip                                              */
/* ------------------------------------------------------------------ */

double orc_sum_sq_half(const uint16_t* g, int64_t n, float unscale, int threads) {
    double s = 0.0;
    int nt = pick_threads(threads);
    const int hw = hw_half(); (void)hw;
    #pragma omp parallel for num_threads(nt) schedule(static) reduction(+:s)
    for (int64_t i = 0; i < n; i++) {
        float raw = H2F(g[i]);
        float x = raw * unscale;                   /* trainer.h:108-109, FP32 product */
        float sq = x * x;
        if (isfinite(raw)) s += (double)sq;        /* inf/NaN elements are reported through found_inf */
    }
    return s;
}

double orc_sum_sq_bf16(const uint16_t* g, int64_t n, float unscale, int threads) {
    double s = 0.0;
    int nt = pick_threads(threads);
    #pragma omp parallel for num_threads(nt) schedule(static) reduction(+:s)
    for (int64_t i = 0; i < n; i++) {
        float raw = orc_bf2f(g[i]);
        float x = raw * unscale;
        float sq = x * x;
        if (isfinite(raw)) s += (double)sq;
    }
    return s;
}

double orc_sum_sq_float(const float* g, int64_t n, float unscale, int threads) {
    double s = 0.0;
    int nt = pick_threads(threads);
    #pragma omp parallel for num_threads(nt) schedule(static) reduction(+:s)
    for (int64_t i = 0; i < n; i++) {
        float x = g[i] * unscale;                  /* trainer.h:125-126 */
        float sq = x * x;                          /* FP32: a finite element's square may be +inf, */
        if (isfinite(g[i])) s += (double)sq;       /* as in the reference's FP32 accumulation       */
    }
    return s;
}

int64_t orc_count_nonfinite_half(const uint16_t* g, int64_t n) {
    int64_t c = 0;
    for (int64_t i = 0; i < n; i++) c += ((g[i] & 0x7C00u) == 0x7C00u);
    return c;
}

int64_t orc_count_nonfinite_float(const float* g, int64_t n) {
    int64_t c = 0;
    for (int64_t i = 0; i < n; i++) c += ((f32_bits(g[i]) & 0x7F800000u) == 0x7F800000u);
    return c;
}

void orc_scale_half(uint16_t* g, int64_t n, float scale, int threads) {
    int nt = pick_threads(threads);
    const int hw = hw_half(); (void)hw;
    #pragma omp parallel for num_threads(nt) schedule(static)
    for (int64_t i = 0; i < n; i++) g[i] = F2H(H2F(g[i]) * scale);   /* trainer.h:138 */
}

void orc_scale_float(float* g, int64_t n, float scale, int threads) {
    int nt = pick_threads(threads);
    #pragma omp parallel for num_threads(nt) schedule(static)
    for (int64_t i = 0; i < n; i++) g[i] *= scale;                           /* trainer.h:144 */
}

float orc_clip_grad_norm(uint16_t* half_pool, int64_t n16, float* float_pool, int64_t n32,
                         float max_norm, int threads) {
    double s = 0.0;
    if (n16 > 0) s += orc_sum_sq_half(half_pool, n16, 1.0f, threads);
    if (n32 > 0) s += orc_sum_sq_float(float_pool, n32, 1.0f, threads);
    float sum_sq = (float)s;                       /* the device scalar is FP32, trainer.h:339 */
    float total_norm = sqrtf(sum_sq);              /* trainer.h:341 */
    if (total_norm > max_norm) {                   /* trainer.h:343 */
        float scale = max_norm / (total_norm + 1e-6f);
        if (n16 > 0) orc_scale_half(half_pool, n16, scale, threads);
        if (n32 > 0) orc_scale_float(float_pool, n32, scale, threads);
    }
    return total_norm;
}

/* ------------------------------------------------------------------ */
/* fused multi-tensor step (statistics pass + update pass)             */
/* ------------------------------------------------------------------ */

void orc_gradstat_finalize(double sum_sq, uint32_t found_inf, float unscale, float max_norm,
                           orc_stat* out) {
    out->sum_sq = sum_sq;
    out->found_inf = found_inf ? 1u : 0u;
    out->norm = sqrtf((float)sum_sq);
    out->clip_active = 0u;
    out->coef = unscale;
    if (max_norm > 0.0f && out->norm > max_norm) {         /* trainer.h:280, 343-344 */
        float scale = max_norm / (out->norm + 1e-6f);
        out->coef = unscale * scale;
        out->clip_active = 1u;
    }
}

void orc_gradstat(const orc_tensor* t, uint64_t count, float unscale, float max_norm,
                  double extra_sum_sq, uint32_t extra_found_inf, int threads,
                  orc_stat* out) {
    double s = extra_sum_sq;
    uint32_t inf = extra_found_inf;
    for (uint64_t k = 0; k < count; k++) {
        if (t[k].n == 0 || (t[k].flags & ORC_FLAG_GRAD_ZERO)) continue;
        if (t[k].grad_dtype == ORC_GRAD_F32 && t[k].dtype != ORC_F32) {
            /* 16-bit parameter with an FP32 gradient: the FP32 rules (trainer.h:120-133) */
            s += orc_sum_sq_float((const float*)t[k].grad, (int64_t)t[k].n, unscale, threads);
            inf |= orc_count_nonfinite_float((const float*)t[k].grad, (int64_t)t[k].n) != 0;
        } else if (t[k].dtype == ORC_F16) {
            s += orc_sum_sq_half((const uint16_t*)t[k].grad, (int64_t)t[k].n, unscale, threads);
            inf |= orc_count_nonfinite_half((const uint16_t*)t[k].grad, (int64_t)t[k].n) != 0;
        } else if (t[k].dtype == ORC_BF16) {
            const uint16_t* g = (const uint16_t*)t[k].grad;
            s += orc_sum_sq_bf16(g, (int64_t)t[k].n, unscale, threads);
            for (uint64_t i = 0; i < t[k].n; i++) inf |= (g[i] & 0x7F80u) == 0x7F80u;
        } else {
            s += orc_sum_sq_float((const float*)t[k].grad, (int64_t)t[k].n, unscale, threads);
            inf |= orc_count_nonfinite_float((const float*)t[k].grad, (int64_t)t[k].n) != 0;
        }
    }
    orc_gradstat_finalize(s, inf, unscale, max_norm, out);
}

int orc_multi_step(const orc_tensor* t, uint64_t count, const orc_hparams* hp,
                   const orc_stat* stat, uint32_t step_flags, int rounding, int threads) {
    float coef = 1.0f;
    int round_clip = 0;
    if (stat) {
        if (stat->found_inf) return 1;             /* overflow: nothing is written */
        coef = stat->coef;
        round_clip = (step_flags & ORC_STEP_ROUND_CLIP_FP16) && stat->clip_active;
    }
    int nt = pick_threads(threads);
    for (uint64_t k = 0; k < count; k++) {
        const orc_tensor* d = &t[k];
        if (d->n == 0 || (d->flags & ORC_FLAG_NORM_ONLY)) continue;
        orc_k kk = make_k(hp->lr, hp->beta1, hp->beta2, hp->eps, d->weight_decay,
                          hp->bias_correction1, hp->bias_correction2);
        int zero = (d->flags & ORC_FLAG_GRAD_ZERO) != 0;
        int64_t n = (int64_t)d->n;
        if (d->dtype == ORC_F16 || d->dtype == ORC_BF16) {
            const int hw = hw_half(); (void)hw;
            const int bf = d->dtype == ORC_BF16;
            const int gf32 = d->grad_dtype == ORC_GRAD_F32;
            uint16_t* p = (uint16_t*)d->param;
            const uint16_t* g = (const uint16_t*)d->grad;
            const float* gf = (const float*)d->grad;
            #pragma omp parallel for num_threads(nt) schedule(static)
            for (int64_t i = 0; i < n; i++) {
                float x;
                if (gf32) {
                    x = zero ? 0.0f : gf[i] * coef;                                   /* trainer.h:144 */
                } else {
                    x = zero ? 0.0f : (bf ? orc_bf2f(g[i]) : H2F(g[i])) * coef;
                    if (round_clip) x = bf ? orc_bf2f(orc_f2bf(x)) : H2F(F2H(x));   /* trainer.h:138 */
                }
                float w0 = d->master ? d->master[i] : (bf ? orc_bf2f(p[i]) : H2F(p[i]));
                float w = upd(w0, x, &d->m[i], &d->v[i], &kk, rounding);
                if (d->master) d->master[i] = w;
                p[i] = bf ? orc_f2bf(w) : F2H(w);
            }
        } else {
            float* p = (float*)d->param;
            const float* g = (const float*)d->grad;
            #pragma omp parallel for num_threads(nt) schedule(static)
            for (int64_t i = 0; i < n; i++) {
                float x = zero ? 0.0f : g[i] * coef;       /* trainer.h:144 */
                p[i] = upd(p[i], x, &d->m[i], &d->v[i], &kk, rounding);
            }
        }
    }
    return 0;
}

void orc_scaler_update(orc_scaler* s, uint32_t found_inf, int growth_interval) {
    if (found_inf) {
        s->scale *= 0.5f;
        s->growth_tracker = 0;
        s->skipped += 1;
    } else {
        s->step += 1;
        s->growth_tracker += 1;
        if (s->growth_tracker >= growth_interval) {
            s->scale *= 2.0f;
            s->growth_tracker = 0;
        }
    }
}

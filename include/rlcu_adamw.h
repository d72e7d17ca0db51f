/*
 * rlcu_adamw.h -- C ABI of the B200 (sm_100a) optimizer step for RL.cu.
 *
 * Scope: the mixed-precision fused AdamW update and the gradient unscale /
 * non-finite check / global L2 norm / clip around it, i.e. what RL.cu runs at
 * the end of every SFT and GRPO optimizer step.  Each entry point names the
 * RL.cu interface it stands in for (paths inside the RL.cu tree).
 *
 * Conventions
 *   - Every function returns an int status (RLCU_OK == 0).  Nothing here exits
 *     the process, throws, or synchronises the device unless it says so.
 *   - All data pointers are DEVICE pointers on the current device unless a
 *     parameter is documented as a host pointer.  Buffers are owned by the
 *     caller and must not alias each other.
 *   - `stream` is a cudaStream_t passed as void* so that this header needs no
 *     CUDA headers; NULL is the legacy default stream, which is what RL.cu uses.
 *   - FP16 data is IEEE binary16 (`__half`), BF16 data is bfloat16; both are passed as void*.
 *   - Sizes are 64-bit element counts.  RL.cu's `int n` launchers are kept
 *     separately in include/kernels/adamw.cuh for source compatibility.
 *   - There is no CPU fallback: without a CUDA device every compute entry
 *     point fails with RLCU_ERR_CUDA.
 */
#ifndef RLCU_ADAMW_H
#define RLCU_ADAMW_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RLCU_ABI_VERSION 2

/* status codes */
enum {
    RLCU_OK = 0,
    RLCU_ERR_INVALID = 1,   /* bad argument (null, size, alignment, kind)      */
    RLCU_ERR_CUDA = 2,      /* a CUDA runtime call failed                      */
    RLCU_ERR_NCCL = 3,      /* an NCCL call failed                             */
    RLCU_ERR_TIMEOUT = 4,   /* a bounded device-side wait gave up              */
    RLCU_ERR_UNSUPPORTED = 5
};

/* element kinds.  RL.cu trains in FP16 (RLCU_F16) with FP32 norm weights (RLCU_F32).
 * RLCU_BF16 (bfloat16 parameters and gradients, same arithmetic in FP32, same options)
 * has no counterpart in RL.cu; its results are checked against the CPU restatement only. */
enum { RLCU_F16 = 0, RLCU_F32 = 1, RLCU_BF16 = 2 };

/* kind of a tensor's gradient (rlcu_tensor_desc.grad_dtype).  RL.cu keeps FP16 gradients for
 * FP16 parameters, accumulated by cuBLAS with beta = 1 (src/kernels/linear.cu:85-98) and by
 * FP16 atomics for the embedding (src/kernels/embedding.cu:62-67), which is where small
 * gradients are lost before the optimizer sees them.  RLCU_GRAD_F32 lets a 16-bit parameter
 * take its gradient from an FP32 buffer instead: 4 bytes read per element where the 16-bit
 * gradient has 2, scaled in FP32 (never rounded through 16 bits).  No RL.cu counterpart. */
enum { RLCU_GRAD_AS_PARAM = 0, RLCU_GRAD_F32 = 1 };

/* per-tensor flags */
enum {
    RLCU_TENSOR_NORM_ONLY = 1u, /* counted in the gradient norm, never updated.
                                   RL.cu's clip covers the whole FP32 gradient pool,
                                   which ends with an attention workspace that is not
                                   a parameter (trainer.h:331, qwen3.cu:1038-1042).   */
    RLCU_TENSOR_GRAD_ZERO = 2u  /* gradient is taken as zero without being read:
                                   RL.cu's freeze_embed memset (trainer.h:271-277).   */
};

/* flags of the update pass */
enum {
    RLCU_STEP_ROUND_CLIP_FP16 = 1u, /* when the clip is active, round g*coef to FP16
                                       (BF16 for BF16 tensors) before use, as RL.cu's
                                       scale_half_kernel stores it (trainer.h:136-139).
                                       FP32 tensors are scaled in FP32.                   */
    RLCU_STEP_DEVICE_BIAS_CORRECTION = 2u, /* take 1-beta^t from the statistics record
                                       (written by the statistics pass when a device-side
                                       scaler state is attached) instead of rlcu_hparams.
                                       The device value is the correctly rounded FP32 power;
                                       it equals rlcu_bias_correction (the host's powf) except
                                       at the rare steps where the C library's powf is one ulp
                                       off (beta 0.999: t = 2958, 3606 with glibc 2.39)      */
    RLCU_STEP_ZERO_GRADS = 4u,      /* write zeros over each gradient after reading it:
                                       folds RL.cu's qwen3_gradients_zero (qwen3.cu:1109-1112)
                                       into the update                                   */
    RLCU_STEP_BULK_COPY = 8u,       /* move the update's HBM traffic with the bulk-copy engine
                                       (cp.async.bulk through shared-memory stages) instead of
                                       per-thread loads and stores; same results.  Without this
                                       flag or the next the library picks: lists that are mostly
                                       FP16 weights with FP32 masters or with FP32 gradients (24
                                       to 30 bytes per element in eight or more streams) take the
                                       bulk-copy kernel, which is 5-7 % faster there; all others
                                       the direct kernel.                                     */
    RLCU_STEP_DIRECT = 16u          /* force the per-thread load/store kernel                 */
};

/* flags of the statistics pass */
enum {
    RLCU_STAT_PARTIAL = 1u,   /* only write sum_sq (this rank's or this buffer's share); the
                                 caller all-reduces it and calls rlcu_gradstat_finalize, or
                                 follows with an RLCU_STAT_ACCUMULATE call                */
    RLCU_STAT_ACCUMULATE = 2u /* rlcu_gradstat_flat_noalloc only: add this buffer's sum to
                                 the sum_sq an earlier PARTIAL call left in the record     */
};

/* One parameter tensor.  Mirrors one slice of RL.cu's flat pools: param/grad
 * from Qwen3Weights / Qwen3Gradients (weights.h:43-61, qwen3.h:190-218), m / v /
 * master from AdamWOptimizer's state (optimizer.h:150-156). 64 bytes. */
typedef struct rlcu_tensor_desc {
    void*       param;        /* __half*, bfloat16* or float* by dtype; updated in place */
    const void* grad;         /* same kind as param, or float* with RLCU_GRAD_F32; may be
                                 NULL with GRAD_ZERO                                   */
    float*      m;            /* first moment                                          */
    float*      v;            /* second moment                                         */
    float*      master;       /* FP32 master copy (F16/BF16 only) or NULL.  With a master,
                                 param is write-only, as in launch_adamw_fp16.         */
    uint64_t    n;            /* elements                                              */
    float       weight_decay; /* decoupled; RL.cu uses 0 for embedding and norms
                                 (optimizer.h:131-146)                                 */
    uint32_t    dtype;        /* RLCU_F16 / RLCU_F32 / RLCU_BF16                       */
    uint32_t    flags;        /* RLCU_TENSOR_*                                         */
    uint32_t    grad_dtype;   /* RLCU_GRAD_AS_PARAM (0) or RLCU_GRAD_F32               */
} rlcu_tensor_desc;

/* Step hyper-parameters: AdamWOptimizer's public fields (optimizer.h:62-66) and
 * the two bias corrections it computes per step (optimizer.h:121-122). */
typedef struct rlcu_hparams {
    float lr, beta1, beta2, eps;
    float bias_correction1;   /* 1 - beta1^t (NOT the inverse, adamw.cuh:36-37)        */
    float bias_correction2;   /* 1 - beta2^t                                            */
} rlcu_hparams;

/* Statistics record in device memory, produced by the statistics pass and read
 * by the update pass without a host round trip (RL.cu reads the sum back to the
 * host in the middle of the step, trainer.h:340). 64 bytes, 16-byte aligned. */
typedef struct rlcu_stat {
    double   sum_sq;       /* sum over all listed gradients of (g*unscale)^2; NaN when some
                              gradient was inf or NaN (that is how a partial sum carries
                              the overflow through an all-reduce); +inf when finite FP32
                              gradients have squares beyond FP32, which is not an overflow:
                              norm is then +inf and a clip scales the gradients to zero   */
    float    norm;         /* sqrtf((float)sum_sq): the PRE-clip norm RL.cu logs        */
    float    coef;         /* what each gradient is multiplied by: unscale, times
                              max_norm/(norm+1e-6) when norm > max_norm (trainer.h:343-344) */
    uint32_t found_inf;    /* 1: some gradient is inf/NaN (tested on the stored value, not on
                              its square) -> the update writes nothing                  */
    uint32_t clip_active;  /* 1: norm > max_norm                                        */
    float    bias_correction1; /* valid when a scaler state was attached                */
    float    bias_correction2;
    int32_t  step;         /* Adam step t the update pass belongs to (scaler attached)  */
    float    loss_scale;   /* scale the gradients of THIS step carried                  */
    uint32_t reserved[6];
} rlcu_stat;

/* Dynamic loss-scale and step-counter state in device memory.  No counterpart
 * in RL.cu (it has no loss scaling): halve on overflow, double after
 * growth_interval consecutive clean steps; an overflowed step is skipped and
 * does not advance the Adam step counter. 32 bytes. */
typedef struct rlcu_scaler_state {
    float   scale;
    int32_t growth_tracker;
    int32_t step;             /* Adam step counter t (clean steps so far)              */
    int32_t skipped;          /* overflowed steps so far                               */
    int32_t growth_interval;
    float   beta1, beta2;     /* for the device-side 1-beta^t                          */
    float   grad_mul;         /* extra factor folded into unscale (1/world after a
                                 summed reduce-scatter); 0 is read as 1                */
} rlcu_scaler_state;

typedef struct rlcu_tensor_list rlcu_tensor_list;

/* -------- library ------------------------------------------------------ */
int         rlcu_abi_version(void);
/* message of the last failure on the calling thread (never NULL) */
const char* rlcu_last_error(void);

/* -------- single tensor: RL.cu's launchers ----------------------------- */
/* launch_adamw_fp16 (include/kernels/adamw.cuh:24-39, src/kernels/adamw.cu:42-58):
 * FP32 master/m/v updated in place, FP16 model weight written, FP16 grad read.
 * n <= 0 is a silent no-op as in adamw.cu:49. */
int rlcu_adamw_fp16_master(float* master_w, void* model_w, const void* grad, float* m, float* v,
                           int64_t n, float lr, float beta1, float beta2, float eps,
                           float weight_decay, float bias_correction1, float bias_correction2,
                           void* stream);
/* Same arithmetic without a master copy: the weight is read from the FP16
 * parameter (12 bytes read + 10 written per element).  No RL.cu counterpart. */
int rlcu_adamw_fp16(void* param, const void* grad, float* m, float* v,
                    int64_t n, float lr, float beta1, float beta2, float eps,
                    float weight_decay, float bias_correction1, float bias_correction2,
                    void* stream);
/* The two calls above for bfloat16 parameters and gradients (no RL.cu counterpart). */
int rlcu_adamw_bf16_master(float* master_w, void* model_w, const void* grad, float* m, float* v,
                           int64_t n, float lr, float beta1, float beta2, float eps,
                           float weight_decay, float bias_correction1, float bias_correction2,
                           void* stream);
int rlcu_adamw_bf16(void* param, const void* grad, float* m, float* v,
                    int64_t n, float lr, float beta1, float beta2, float eps,
                    float weight_decay, float bias_correction1, float bias_correction2,
                    void* stream);
/* launch_adamw_fp32 (include/kernels/adamw.cuh:43-57, src/kernels/adamw.cu:93-108) */
int rlcu_adamw_fp32(float* w, const float* grad, float* m, float* v,
                    int64_t n, float lr, float beta1, float beta2, float eps,
                    float weight_decay, float bias_correction1, float bias_correction2,
                    void* stream);
/* fp16_to_fp32 master initialisation (include/training/optimizer.h:46-57) */
int rlcu_half_to_float(float* dst, const void* src, int64_t n, void* stream);

/* -------- tensor list --------------------------------------------------- */
/* Builds the device-side work table for `count` tensors (host array `descs`).
 * Allocates device memory (table + reduction scratch) on the current device and
 * copies synchronously; call it at set-up, like AdamWOptimizer::init
 * (optimizer.h:188-250).  Tensors with n == 0 are allowed and ignored. */
int rlcu_tensor_list_create(const rlcu_tensor_desc* descs, uint64_t count, rlcu_tensor_list** out);
int rlcu_tensor_list_destroy(rlcu_tensor_list* list);
/* Waits for every stream of the device (cudaDeviceSynchronize) and reports whether a
 * bounded wait inside a kernel launched on this list gave up since the last check
 * (RLCU_ERR_TIMEOUT); only the RLCU_STEP_BULK_COPY update has such waits.  Clears the
 * condition. */
/* list == NULL checks the single-tensor entry points instead (rlcu_adamw_fp16_master takes the
 * bulk-copy kernel for large tensors). */
int rlcu_tensor_list_check(rlcu_tensor_list* list);
/* Runs a one-thread kernel whose bounded wait is certain to run out (it waits on a
 * barrier nothing completes) and reports it through the same path: the expected
 * return value is RLCU_ERR_TIMEOUT, and the device stays usable afterwards. */
int rlcu_selftest_bounded_wait(rlcu_tensor_list* list, void* stream);
/* elements the update pass touches / elements the statistics pass reads */
uint64_t rlcu_tensor_list_numel(const rlcu_tensor_list* list);
uint64_t rlcu_tensor_list_stat_numel(const rlcu_tensor_list* list);
uint64_t rlcu_tensor_list_work_items(const rlcu_tensor_list* list);

/* -------- statistics pass: Trainer::clip_grad_norm_ without the host sync ---- */
/* One launch over every gradient in the list: x = g * unscale, sum of x^2 in a
 * fixed (deterministic) order, non-finite detection, and -- unless
 * RLCU_STAT_PARTIAL -- the finished record {norm, coef, found_inf, clip_active}
 * written to `stat_out` (device).  Stands in for sum_sq_half_kernel /
 * sum_sq_float_kernel + the blocking read-back + host sqrtf
 * (include/training/trainer.h:103-133, 324-344); the scale kernels
 * (trainer.h:136-145, 345-349) are folded into the update pass through `coef`.
 *   unscale   : 1/loss_scale (times 1/world when gradients were summed); 1 for RL.cu
 *   max_norm  : clip threshold; <= 0 disables clipping (trainer.h:280)
 *   scaler    : optional device state; when given, unscale is taken as
 *               grad_mul/scale from it (the `unscale` argument is ignored) and the
 *               finished record also carries the step's bias corrections, after
 *               which the scale / step counter are advanced.
 * Calls on the same list must not overlap on the GPU (they share its scratch).
 * The sum is taken in a fixed order for a given list, so the same list gives the same bits run
 * after run; the order follows the work items, which are cut by address, so a copy of the same
 * data at other addresses may differ in the last bits of sum_sq. */
int rlcu_gradstat(rlcu_tensor_list* list, float unscale, float max_norm,
                  rlcu_scaler_state* scaler, rlcu_stat* stat_out, uint32_t flags, void* stream);
/* The statistics pass for callers that cannot allocate device memory: one flat
 * gradient buffer in (RL.cu's half_pool or float_pool), the finished record
 * {sum_sq, norm, coef, found_inf, clip_active} out, no tensor list and no
 * allocation anywhere -- the reduction scratch is a fixed 1 MiB array inside the
 * library image, resident on every GPU that loads the library.  This entry
 * point has no counterpart in RL.cu.  It exists because RL.cu's trainer runs
 * beside an inference engine that claims the free device memory for its KV
 * cache, so an optimizer step issued at that point cannot rely on cudaMalloc,
 * and because some hot paths are not allowed to enter the allocator at all.
 *   n      : at most RLCU_NOALLOC_MAX_ELEMS; more is refused with RLCU_ERR_INVALID
 *   dtype  : RLCU_F16 or RLCU_F32
 *   flags  : 0 for a single buffer.  The record covers exactly the one buffer of the call;
 *            RL.cu's clip norm covers two pools (trainer.h:331-337), so for those call
 *            once on half_pool with RLCU_STAT_PARTIAL (leaves only sum_sq in the record)
 *            and then, on the same stream, on float_pool with RLCU_STAT_ACCUMULATE (adds
 *            its sum to the record's and writes the finished record).
 * Calls on one device share the scratch: calls that overlap on the GPU race.
 * The first call on a device resolves the scratch address; make it at set-up,
 * before any stream capture.  Sums are taken per 8192-element chunk and added in
 * chunk order, so the result does not depend on the GPU's SM count; it agrees
 * with rlcu_gradstat to rounding (1e-5 relative on the norm), not bit for bit. */
#define RLCU_NOALLOC_MAX_ELEMS 2147483648ull
int rlcu_gradstat_flat_noalloc(const void* grad, uint32_t dtype, uint64_t n,
                               float unscale, float max_norm,
                               rlcu_stat* stat_out, uint32_t flags, void* stream);
/* Completes a PARTIAL record after the caller has all-reduced stat->sum_sq. */
int rlcu_gradstat_finalize(rlcu_stat* stat, float unscale, float max_norm,
                           rlcu_scaler_state* scaler, void* stream);

/* -------- update pass: AdamWOptimizer::step as one launch ---------------- */
/* One launch over every tensor of the list (optimizer.h:119-147 issues three).
 * `stat` may be NULL (no clip, no skip: the plain RL.cu update).  With `stat`,
 * nothing is written when stat->found_inf, and every gradient is multiplied by
 * stat->coef in registers first. */
int rlcu_adamw_multi_step(rlcu_tensor_list* list, const rlcu_hparams* hp,
                          const rlcu_stat* stat, uint32_t step_flags, void* stream);

/* -------- ZeRO-1: optimizer state partitioned over the GPUs of one node ----- */
/* No counterpart in RL.cu (single GPU, no NCCL).  One process (or host thread) per
 * GPU.  All parameters live in one flat FP16 pool and all gradients in another
 * (RL.cu's fp16_pool / half_pool layout, include/model/weights.h:43-61), both
 * padded to rlcu_zero1_plan.padded_elems.  The flat element space is cut into
 * `world` equal contiguous shards; rank r keeps m / v (/ master) for shard r only.
 * One step:
 *   reduce-scatter (sum) of the FP16 gradients, in place       NCCL over NVLink
 *   statistics pass on the shard, all-reduce of one double     norm over all ranks
 *   update pass on the shard (1/world folded into the factor)
 *   all-gather of the FP16 parameters, in place                NCCL over NVLink
 * Result: every rank holds the parameters a single GPU would hold after a step
 * on the mean of the ranks' gradients. */
typedef struct rlcu_zero1 rlcu_zero1;

/* One run of consecutive pool elements with the same weight decay and flags
 * (RL.cu: projections with decay, then the embedding without, optimizer.h:125-140). */
typedef struct rlcu_zero1_segment {
    uint64_t n;
    float    weight_decay;
    uint32_t flags;            /* RLCU_TENSOR_GRAD_ZERO allowed */
} rlcu_zero1_segment;

/* What rank `rank` owns; pure host arithmetic, usable without a GPU. */
typedef struct rlcu_zero1_plan {
    uint64_t total;            /* sum of segment sizes                               */
    uint64_t shard_elems;      /* ceil(total/world) rounded up to 1024               */
    uint64_t padded_elems;     /* shard_elems * world: required pool length          */
    uint64_t lo, hi;           /* this rank's element range, clipped to total        */
    uint64_t pieces;           /* segments (or parts of segments) inside [lo, hi)    */
} rlcu_zero1_plan;

#define RLCU_UNIQUE_ID_BYTES 128

/* how the two exchanges of the step are carried out */
enum {
    RLCU_ZERO1_NCCL = 0,  /* ncclReduceScatter / ncclAllGather around the single-GPU kernels    */
    RLCU_ZERO1_P2P = 1    /* fused: the statistics kernel pulls every rank's gradients over
                             NVLink through peer-mapped pointers (FP32 sum in rank order, one
                             rounding), the update kernel pushes each new FP16 parameter into
                             every peer's pool.  One process per GPU, pools from cudaMalloc,
                             at most 8 ranks.  Rank ordering uses 8-byte NCCL collectives.      */
};
/* OR this into `mode` when the two pools hold bfloat16 instead of FP16 */
#define RLCU_ZERO1_POOLS_BF16 0x100u
/* OR this into `mode` when the GRADIENT pool holds FP32 (padded_elems floats) for the 16-bit
 * parameters: gradients are summed in FP32 in rank order and never rounded to 16 bits; twice the
 * bytes cross NVLink in the reduce-scatter.  See RLCU_GRAD_F32. */
#define RLCU_ZERO1_GRADS_F32 0x200u
int rlcu_zero1_make_plan(const rlcu_zero1_segment* segs, uint64_t nsegs, int rank, int world,
                         rlcu_zero1_plan* out);
/* The descriptors rank `rank` would update, with pointers expressed as element
 * offsets from the pool / shard-state bases (param, grad: offset into the pools;
 * m, v, master: offset into the rank's shard arrays).  `out` has room for
 * plan.pieces entries.  Host arithmetic only. */
int rlcu_zero1_plan_pieces(const rlcu_zero1_segment* segs, uint64_t nsegs, int rank, int world,
                           uint64_t* pool_offset, uint64_t* state_offset, uint64_t* n,
                           float* weight_decay, uint32_t* flags);
/* NCCL unique id for rank 0 to hand to the other ranks (host buffer of
 * RLCU_UNIQUE_ID_BYTES), by whatever channel the caller has. */
int rlcu_zero1_unique_id(void* id_out);
/* Collective over all ranks: joins the communicator and builds the shard's work
 * table.  m_shard / v_shard / master_shard have plan.shard_elems floats
 * (master_shard may be NULL: weights are read from the FP16 pool).  Allocates;
 * synchronises the device. */
int rlcu_zero1_create(const void* unique_id, int rank, int world,
                      void* param_pool, void* grad_pool,
                      const rlcu_zero1_segment* segs, uint64_t nsegs,
                      float* m_shard, float* v_shard, float* master_shard,
                      uint32_t mode, rlcu_zero1** out);
/* One sharded optimizer step, enqueued on `stream` (no host synchronisation).
 * `unscale` is 1/loss_scale (1 without loss scaling); the division by `world` is
 * added inside.  With a `scaler` the factor is taken from it instead
 * (grad_mul/scale): set its grad_mul to 1/world.  `stat` is a device record that
 * receives the global norm etc.
 * phases: bit mask for measurements, 0 = all.  NCCL mode: 1 reduce-scatter, 2
 * statistics + all-reduce, 4 update, 8 all-gather.  P2P mode: 1 fused
 * reduce-scatter + statistics, 2 all-reduce + finalize, 4 (or 8) fused update +
 * all-gather.  With RLCU_STEP_ZERO_GRADS the whole local gradient pool is zero after the step
 * (in P2P mode cleared inside the update kernel, under its NVLink traffic).
 * In P2P mode with FP16 pools on more than one rank the two exchange kernels move their NVLink
 * traffic with the bulk-copy engine (cp.async.bulk, no multicast) by default, which is 1-2 %
 * faster than per-thread loads and stores; RLCU_STEP_DIRECT forces the latter (bfloat16 pools
 * always use it), RLCU_STEP_BULK_COPY the former. */
int rlcu_zero1_step(rlcu_zero1* z, const rlcu_hparams* hp, float unscale, float max_norm,
                    rlcu_scaler_state* scaler, rlcu_stat* stat, uint32_t step_flags,
                    uint32_t phases, void* stream);
/* Reports an asynchronous NCCL failure (a peer that died, a timed-out
 * collective) without blocking: RLCU_OK or RLCU_ERR_NCCL. */
int rlcu_zero1_poll_error(rlcu_zero1* z);
/* Blocking check after one or more steps: waits for the device, then reports a bounded wait
 * of the bulk-copy exchange kernels that gave up (RLCU_ERR_TIMEOUT: that step is incomplete) or
 * an asynchronous NCCL failure. */
int rlcu_zero1_check(rlcu_zero1* z);
/* Tears the communicator down; `abort` != 0 uses ncclCommAbort (after a failure). */
int rlcu_zero1_destroy(rlcu_zero1* z, int abort);

/* -------- optimizer-state checkpoint ------------------------------------- */
/* RL.cu's Trainer::save_checkpoint is a stub (include/training/trainer.h:317-319;
 * the configuration already carries save_dir / save_steps, trainer.h:35, 47-48).
 * One file per rank holds what is needed to continue bit-identically: the Adam
 * step counter, the loss-scale state and the rank's m / v (/ master) arrays.
 * Layout: 128-byte little-endian header, then m, v, master as raw FP32, then a
 * 64-bit FNV-1a checksum of the payload.  Both calls block until the copy is done. */
typedef struct rlcu_checkpoint_info {
    uint64_t state_elems;     /* floats in each of m, v (and master)                   */
    int32_t  step;            /* Adam step counter t                                   */
    float    loss_scale;
    int32_t  growth_tracker;
    int32_t  skipped;
    int32_t  rank, world;     /* which shard this is (0 of 1 without sharding)         */
    uint32_t has_master;
    uint32_t reserved;
} rlcu_checkpoint_info;

int rlcu_checkpoint_save(const char* path, const rlcu_checkpoint_info* info,
                         const float* m, const float* v, const float* master, void* stream);
/* header only; touches no device */
int rlcu_checkpoint_peek(const char* path, rlcu_checkpoint_info* info_out);
/* m / v / master must hold `capacity_elems` >= the file's state_elems floats; a
 * file written with a master needs `master`, and the other way round. */
int rlcu_checkpoint_load(const char* path, rlcu_checkpoint_info* info_out,
                         float* m, float* v, float* master, uint64_t capacity_elems, void* stream);

/* -------- host-side helpers --------------------------------------------- */
/* 1 - powf(beta, t) in FP32 exactly as AdamWOptimizer::step (optimizer.h:121-122) */
float rlcu_bias_correction(float beta, int step);

#ifdef __cplusplus
}
#endif
#endif /* RLCU_ADAMW_H */

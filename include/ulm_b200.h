/*
 * ulm_b200.h -- C ABI of libulm_b200.so, the sm_100a (B200) implementation of the
 * Universal-LM-Trainer training hot path: causal FlashAttention-2 forward and
 * backward, fused RoPE, RMSNorm and the row kernels of the chunked cross-entropy.
 *
 * Conventions
 *   - Plain C types only; every pointer named *_dev* or typed as a tensor is a
 *     CUDA device pointer owned by the caller.  The library allocates no device
 *     memory: outputs and scratch are passed in.
 *   - Strides are in ELEMENTS of the tensor's dtype.  The innermost dimension is
 *     always contiguous.
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 *     Calls only enqueue work; they never synchronise.
 *   - Return value 0 = success.  Negative = error; the text is available from
 *     ulm_last_error() on the calling thread.  Nothing throws, exits or traps.
 *   - Kernels that wait on hardware barriers bound every wait; on expiry they set
 *     a bit in the caller's `status_dev` word (may be NULL) and return.
 *
 * Each entry point names the reference code it replaces (paths relative to the
 * root of sunyi9161/Universal-LM-Trainer).
 */
#ifndef ULM_B200_H
#define ULM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ULM_ABI_VERSION 4

enum { ULM_F16 = 0, ULM_BF16 = 1, ULM_F32 = 2 };
/* dtype of RMSNorm's y (forward) and dy (backward) relative to x */
enum { ULM_Y_SAME = 0, ULM_Y_F16 = 1, ULM_Y_BF16 = 2 };

enum {
  ULM_OK = 0,
  ULM_ERR_ARG = -1,       /* bad shape / stride / alignment / dtype           */
  ULM_ERR_CUDA = -2,      /* a CUDA runtime or driver call failed             */
  ULM_ERR_DEVICE = -3,    /* device is not compute capability 10.0            */
  ULM_ERR_TOO_LARGE = -4  /* size beyond a documented fixed maximum           */
};

/* bits a kernel may set in *status_dev */
enum {
  ULM_STATUS_TIMEOUT_LOAD = 1,   /* a wait for a TMA load ran out      */
  ULM_STATUS_TIMEOUT_MMA = 2,    /* a wait for the tensor core ran out */
  ULM_STATUS_TIMEOUT_SOFTMAX = 4 /* a wait for the softmax warps ran out */
};

/* ---- library ----------------------------------------------------------- */
int ulm_abi_version(void);
const char* ulm_last_error(void);
/* 0 if `device` is an sm_100 part this library can run on. */
int ulm_device_ok(int device);
/* Number of kernels this library has launched in this process (all threads). */
uint64_t ulm_launch_count(void);

/* ---- RoPE ---------------------------------------------------------------
 * Replaces rope_fwd / rope_bwd of csrc/flash_attn_v100/fast_ops.cu:189-216
 * (kernel rope_kernel<BACKWARD>, fast_ops.cu:70-101), bound in the reference at
 * flash_attn_v100.cu:395-396 and called from flash_attn_v100_cuda.py:117,137.
 * q,k: (B,H,S,64) views, any b/h/s strides; cos,sin: fp32 [S,64] with a row
 * stride (the tables are d_model wide, only the first 64 columns are read).
 * fp32 multiply, multiply, add without contraction, one rounding to `dtype`.
 * backward != 0 computes the adjoint (inputs are the output gradients).
 * head_dim is fixed at 64 like the reference (fast_ops.cu:27).
 * Either tensor may be left out by passing NULL for both its input and its output
 * (K alone is what the attention forward with fused Q rotation needs beside it).
 */
typedef struct {
  const void* q; const void* k;        /* inputs (or dqo, dko when backward)  */
  void* qo; void* ko;                  /* outputs                             */
  const float* cos_tab; const float* sin_tab;
  int64_t q_sb, q_sh, q_ss;
  int64_t k_sb, k_sh, k_ss;
  int64_t qo_sb, qo_sh, qo_ss;
  int64_t ko_sb, ko_sh, ko_ss;
  int64_t cos_stride, sin_stride;      /* row strides of the tables (floats)  */
  int32_t B, H, S;
  int32_t dtype;                       /* ULM_F16 or ULM_BF16                 */
  int32_t backward;
  void* stream;
} ulm_rope_args;
int ulm_rope(const ulm_rope_args* a);

/* ---- attention forward ---------------------------------------------------
 * Replaces fa_fwd (csrc/flash_attn_v100/flash_attn_v100.cu:337-364, kernel
 * fa_fwd_kernel :40-309), called from flash_attn_v100_cuda.py:76.
 * q,k,v: (B,H,S,64) 16-bit, innermost contiguous, strides multiples of 8
 * elements, base pointers 16-byte aligned.  o: same shape, caller-chosen strides.
 * lse: fp32 (B,H,S) contiguous, natural log.  softmax_scale is applied to QK^T.
 * dropout_p > 0 uses the reference's stateless hash (fa_common.cuh:21-38) keyed
 * by (seed, row, col, b*H+h).
 *
 * Fused RoPE (replaces the rope_fwd call in front of fa_fwd for Q; train.py:1913,
 * fast_ops.cu:70-101): with cos_tab and sin_tab non-NULL, q is the tensor BEFORE
 * rotation; each CTA rotates its resident Q tile after loading it, with the same
 * arithmetic as ulm_rope (bit-identical), and, when q_rot is non-NULL, also
 * writes the rotated tile there (the backward needs it).  k must already be
 * rotated (ulm_rope with q = qo = NULL).  cos_tab = sin_tab = NULL: q is used as is.
 */
typedef struct {
  const void* q; const void* k; const void* v;
  void* o; float* lse;
  int64_t q_sb, q_sh, q_ss;
  int64_t k_sb, k_sh, k_ss;
  int64_t v_sb, v_sh, v_ss;
  int64_t o_sb, o_sh, o_ss;
  int32_t B, H, S;
  int32_t dtype;                       /* ULM_F16 or ULM_BF16                 */
  int32_t causal;
  float softmax_scale;
  float dropout_p;
  uint32_t seed;
  uint32_t* status_dev;                /* optional, see ULM_STATUS_*          */
  void* stream;
  const float* cos_tab; const float* sin_tab;   /* fp32 [S,64] tables, or NULL: no fused rotation */
  int64_t cos_stride, sin_stride;      /* row strides of the tables (floats, multiples of 4) */
  void* q_rot;                         /* optional output: rotated q, same dtype            */
  int64_t qr_sb, qr_sh, qr_ss;
} ulm_attn_fwd_args;
int ulm_attn_fwd(const ulm_attn_fwd_args* a);

/* ---- attention backward --------------------------------------------------
 * Replaces fa_bwd (csrc/flash_attn_v100/flash_attn_v100_bwd.cu:433-506; kernels
 * fa_bwd_delta_kernel :42, fa_bwd_dq_kernel :66, fa_bwd_dkv_kernel :224), called
 * from flash_attn_v100_cuda.py:91.  `mode` is the reference's bitmask
 * (1 = delta, 2 = dQ, 4 = dK/dV; 7 = all).
 * o and d_o may be strided (the reference forces contiguous copies).
 * delta: fp32 scratch (B,H,S) contiguous, written when mode&1, read otherwise.
 * With both mode&1 and mode&2 the dQ pass computes delta from its resident O and dO
 * tiles (no separate delta launch); delta is complete when the dQ pass has run, so a
 * later mode=4 call on the same stream may read it.
 * dq, dk, dv: caller-chosen strides.
 *
 * Fused RoPE adjoint (replaces the rope_bwd call behind fa_bwd,
 * flash_attn_v100_cuda.py:137, fast_ops.cu:51-68): with cos_tab and sin_tab
 * non-NULL, q and k are the ROTATED tensors the forward used, and the dQ and dK
 * epilogues round their result to the 16-bit type and apply the adjoint rotation
 * before storing, so dq and dk are the gradients of the tensors BEFORE rotation,
 * bit-identical to ulm_attn_bwd followed by ulm_rope(backward).
 */
typedef struct {
  const void* q; const void* k; const void* v;
  const void* o; const void* d_o; const float* lse;
  float* delta;
  void* dq; void* dk; void* dv;
  int64_t q_sb, q_sh, q_ss;
  int64_t k_sb, k_sh, k_ss;
  int64_t v_sb, v_sh, v_ss;
  int64_t o_sb, o_sh, o_ss;
  int64_t do_sb, do_sh, do_ss;
  int64_t dq_sb, dq_sh, dq_ss;
  int64_t dk_sb, dk_sh, dk_ss;
  int64_t dv_sb, dv_sh, dv_ss;
  int32_t B, H, S;
  int32_t dtype;
  int32_t causal;
  int32_t mode;
  float softmax_scale;
  float dropout_p;
  uint32_t seed;
  uint32_t* status_dev;
  void* stream;
  const float* cos_tab; const float* sin_tab;   /* fp32 [S,64] tables, or NULL: no fused adjoint */
  int64_t cos_stride, sin_stride;
} ulm_attn_bwd_args;
int ulm_attn_bwd(const ulm_attn_bwd_args* a);

/* ---- RMSNorm --------------------------------------------------------------
 * The reference calls F.rms_norm (train.py:1862-1875; manual form
 * inf.py:58-67): y = w * x * rsqrt(mean(x^2) + eps), fp32 reduction, output in
 * x's dtype.  x: [rows, d] with a row stride; w: [d] of dtype w_dtype.
 * rstd (optional, fp32 [rows]) is written by fwd and may be passed to bwd.
 *
 * Fused residual add (train.py:1989, 1993: x = x + branch, followed by the next
 * norm at :1991 / :1988 / :2054): with `branch` non-NULL -- x fp32, branch and y
 * of the 16-bit y_kind -- the kernel forms x + branch in fp32, writes it to x_out
 * and normalises it in the same pass.  Rows of at most 1024 elements.
 */
typedef struct {
  const void* x; const void* w; void* y; float* rstd;
  int64_t x_stride, y_stride;
  int64_t rows; int32_t d;
  int32_t x_dtype, w_dtype;            /* ULM_F16 / ULM_BF16 / ULM_F32        */
  float eps;
  void* stream;
  int32_t y_kind;                      /* ULM_Y_SAME, or with fp32 x: ULM_Y_F16 / ULM_Y_BF16 -- y is rounded
                                          once from the fp32 result, which is what autocast's cast of an fp32
                                          F.rms_norm output in front of the next Linear produces              */
  int32_t reserved;
  const void* branch; void* x_out;     /* fused residual add (both NULL: none)                                */
  int64_t branch_stride, xout_stride;
} ulm_rmsnorm_fwd_args;
int ulm_rmsnorm_fwd(const ulm_rmsnorm_fwd_args* a);

/* Backward of the above (autograd's rms_norm backward in the reference).
 * dx has x's dtype; dw is fp32 [d] and is OVERWRITTEN.  `partial` is fp32
 * scratch of at least ulm_rmsnorm_bwd_partial_rows(rows) * d floats.
 * Backward of the fused residual add (x = the forward's x_out): g_add (fp32, may
 * be NULL) is the gradient that reaches x_out from later layers; dx receives
 * rms_norm's gradient plus g_add -- the gradient of both inputs of the add -- and
 * d_branch (16-bit of dy_kind, may be NULL) the same values rounded, which is what
 * autograd hands the 16-bit branch.  Needs an fp32 x and a 16-bit dy_kind. */
typedef struct {
  const void* x; const void* w; const void* dy; const float* rstd; /* rstd may be NULL */
  void* dx; float* dw; float* partial;
  int64_t x_stride, dy_stride, dx_stride;
  int64_t rows; int32_t d;
  int32_t x_dtype, w_dtype;
  float eps;
  void* stream;
  int32_t dy_kind;                     /* dtype of dy like y_kind above; dx always has x's dtype */
  int32_t reserved;
  const void* g_add; void* d_branch;   /* fused gradient add (both NULL: none)                   */
  int64_t gadd_stride, dbranch_stride;
} ulm_rmsnorm_bwd_args;
int ulm_rmsnorm_bwd(const ulm_rmsnorm_bwd_args* a);
int64_t ulm_rmsnorm_bwd_partial_rows(int64_t rows);

/* Same computation and results as ulm_rmsnorm_bwd, for callers that cannot
 * allocate device memory (a frozen memory pool, a stream being captured, a
 * binding without an allocator).  No counterpart in the reference.
 * `a->partial` is ignored: the per-CTA partial sums go to a fixed 1.16 MiB array
 * built into the library (296 x 1024 floats; it exists on every GPU that loads
 * the library, for the life of the process).  Limits: d <= 1024; larger sizes
 * return ULM_ERR_TOO_LARGE.  The device that owns the tensors must be current.
 * The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress) and keeps it; make that first call before starting a
 * stream capture.  The kept address does not survive a cudaDeviceReset: a process
 * that resets a device must not use this entry point on it afterwards.
 * This entry point calls no cudaMalloc / cudaFree and no allocating library
 * routine.  All calls on a device share the one array and it keeps the previous
 * call's contents; every value read is rewritten first within the same call, so
 * nothing needs clearing, but two calls that overlap on the GPU (different
 * streams) race on it: keep them on one stream or order them with events. */
int ulm_rmsnorm_bwd_static(const ulm_rmsnorm_bwd_args* a);

/* ---- SwiGLU gate ----------------------------------------------------------
 * The reference computes F.silu(w1 x) * (w3 x) with separate PyTorch kernels
 * (train.py:1966-1975); no custom kernel exists there.  a = w1 x, b = w3 x, all
 * tensors contiguous with n elements of one dtype.
 * fwd: y = silu(a) * b.   bwd: da = dy * b * silu'(a), db = dy * silu(a).
 * Intermediate values are rounded to the dtype where eager PyTorch rounds them.
 */
typedef struct {
  const void* a; const void* b;
  void* y;                             /* fwd output                           */
  const void* dy; void* da; void* db;  /* bwd input and outputs                */
  int64_t n;
  int32_t dtype;                       /* ULM_F16 / ULM_BF16 / ULM_F32        */
  int32_t reserved;
  void* stream;
} ulm_swiglu_args;
int ulm_swiglu_fwd(const ulm_swiglu_args* a);
int ulm_swiglu_bwd(const ulm_swiglu_args* a);

/* ---- chunked cross-entropy row kernels -----------------------------------
 * The reference loops fc_out + F.cross_entropy(reduction='sum') over chunks of
 * rows (train.py:2075-2079).  These kernels are the softmax part over one
 * 16-bit (or fp32) logits tile [rows, V] produced by the lm-head GEMM.
 * fwd : lse[r] = logsumexp(logits[r,:]) (fp32), loss[r] = lse - logits[r,t]
 *       (0 where target[r] == ignore_index).
 * bwd : logits[r,:] <- (softmax - onehot(t)) * g   in place, in the tile's dtype,
 *       with g = *gscale_dev * gscale (0 for ignored rows).  gscale_dev may be
 *       NULL (treated as 1).
 */
typedef struct {
  const void* logits; const int64_t* target;
  float* lse; float* loss;
  int64_t row_stride; int64_t rows; int32_t V;
  int32_t dtype; int64_t ignore_index;
  void* stream;
} ulm_ce_fwd_args;
int ulm_ce_fwd(const ulm_ce_fwd_args* a);

typedef struct {
  void* logits; const int64_t* target; const float* lse;
  const float* gscale_dev; float gscale;
  int64_t row_stride; int64_t rows; int32_t V;
  int32_t dtype; int64_t ignore_index;
  void* stream;
} ulm_ce_bwd_args;
int ulm_ce_bwd(const ulm_ce_bwd_args* a);

/* ---- lm-head GEMM with the loss statistics in its epilogue -----------------
 * Forward of the reference's `F.cross_entropy(self.fc_out(h), t)` (train.py:2075-2079) as ONE tensor-core
 * kernel plus a per-row finishing kernel: z = h w^T rounded to the 16-bit dtype (what the autocast linear
 * returns), lse[r] = logsumexp(z[r,:]) in fp32, loss[r] = lse[r] - z[r, target[r]] (0 where target[r] ==
 * ignore_index) -- ulm_ce_fwd's outputs without a separate pass over the logits.
 * h [rows, d], w [V, d]: fp16 or bf16, rows h_stride / w_stride elements apart (multiples of 8), d a
 * multiple of 64, base pointers 16-byte aligned.  logits: optional [rows, V] buffer of the same dtype that
 * receives z for the backward (needs V % 64 == 0, z_stride a multiple of 8); NULL: nothing is stored and
 * loss must be NULL too (lse only).  part_m, part_s: fp32 scratch of rows * ulm_lmhead_lse_parts(V) floats
 * each.  status_dev: optional, see ULM_STATUS_*.
 */
typedef struct {
  const void* h; const void* w;
  void* logits;
  const int64_t* target;
  float* lse; float* loss;
  float* part_m; float* part_s;
  int64_t h_stride, w_stride, z_stride;
  int64_t rows; int32_t V; int32_t d;
  int32_t dtype; int32_t reserved;
  int64_t ignore_index;
  uint32_t* status_dev;
  void* stream;
} ulm_lmhead_lse_args;
int ulm_lmhead_lse(const ulm_lmhead_lse_args* a);
int64_t ulm_lmhead_lse_parts(int32_t V);

/* ---- gradient post-processing after the data-parallel all-reduce ----------
 * No counterpart kernel in the reference: fuses what scaler.unscale_ and
 * clip_grad_norm_ do in separate passes (train.py:2364-2365) over one flat fp32
 * gradient bucket: g *= inv_scale; out[0] += sum(g^2); out[1] = 1 if any
 * element is inf/nan.  `out` is a 2-float device array the caller zeroes.
 * `partial` is fp32 scratch of ulm_grad_sumsq_partial_count() floats: every CTA
 * writes its partial sum there and a second one-CTA kernel adds them in a fixed
 * order, so the result is bit-identical from run to run and from rank to rank
 * (data-parallel ranks derive the clip factor from it and must agree exactly).
 */
int ulm_grad_unscale_sumsq(float* grad, int64_t n, const float* inv_scale_dev,
                           float* out, float* partial, void* stream);
int64_t ulm_grad_sumsq_partial_count(void);

/* ---- diagnostics ------------------------------------------------------------
 * No counterpart in the reference.
 * ulm_tensor_map_cache_stats: hits and misses of the host-side cache of encoded
 * TMA tensor maps since the library was loaded.
 * ulm_selftest_wait_timeout: launches a one-CTA kernel whose only work is a
 * bounded wait of `limit_ns` nanoseconds on a hardware barrier that nothing ever
 * arrives at -- the same wait routine the attention kernels use, with a short
 * limit instead of their 2 s.  The kernel returns normally and ORs
 * ULM_STATUS_TIMEOUT_LOAD into *status_dev, which is how a caller can check, with
 * no fault and no hang, that an expired wait is reported and leaves the context
 * usable.  limit_ns must be between 1 and 100 000 000.
 */
void ulm_tensor_map_cache_stats(uint64_t* hits, uint64_t* misses);
int ulm_selftest_wait_timeout(uint64_t limit_ns, uint32_t* status_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ULM_B200_H */

/* toner_b200 -- C ABI of the B200 (sm_100a) kernels behind the Toner optimizer step.
 *
 * The reference project is pure Python (PyTorch + Triton); it has no FFI of its own.  Each entry point
 * below therefore names the reference *operator* it stands in for (path inside the reference project
 * and line range), which is the seam a maintainer would rebind.
 *
 * Conventions
 *   - plain pointers and sizes only; every pointer is a CUDA device pointer unless said otherwise
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, nothing synchronises
 *     unless documented
 *   - return value 0 = ok, > 0 = host-detected error (toner_last_error() gives the text)
 *   - numerical / device conditions are reported through int status words in device memory
 *   - the library never allocates caller-visible memory: scratch is a caller-provided workspace whose
 *     size comes from the matching *_workspace_bytes query.  (The per-device context keeps one small
 *     private arena for TMA tensor maps, created on first use.)
 *   - streams and the tensor-map arena: the first product that reads an operand (address, shape, strides)
 *     encodes its TMA tensor maps on the host and uploads them with an asynchronous copy on that call's
 *     stream; later products find them by that key.  A product launched on ANOTHER stream before the upload
 *     has finished is made to wait for it (an event recorded after the copy), so any stream may be passed
 *     to any call.  The arena holds 32768 maps; when it is full the library synchronises the device once
 *     and starts over (not allowed during stream capture: a captured region should reuse operand addresses,
 *     which costs no new map)
 *   - matrices are row-major FP32 unless said otherwise; "stack" means `batch` equally shaped matrices
 *     stored back to back
 *   - there is no CPU fallback: without a CUDA device every compute entry point fails
 */
#ifndef TONER_B200_H_
#define TONER_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ library */
int toner_init(int device);               /* create the context of `device` (optional: created on first use) */
const char* toner_last_error(void);       /* text of the last host-side failure on this thread */
int toner_sm_count(void);                 /* SM count of the current device (0 on failure) */
long long toner_launch_count(void);       /* kernels launched by this library so far (for launch accounting) */
/* Synchronise `stream`, then read and clear the device status word that kernels set when one of their
 * bounded waits runs out (0 = healthy). */
int toner_device_status(void* stream, int* status_out);
/* The same word without a synchronisation: an asynchronous copy into `host_out` (pinned HOST memory, one int32)
 * enqueued on `stream`; the word is not cleared.  A host that already waits for something later on that stream (the
 * factor engine's status flags, an event after the update) reads it then, and so learns of a product that gave up
 * a wait before it uses the product's result.  The reference has no counterpart (its kernels do not wait). */
int toner_status_snapshot(int32_t* host_out, void* stream);
/* CTAs the persistent GEMM kernel launches from now on (this device): 0 = one per SM (default), else at most `sms`
 * (rounded down to an even count).  The kernel assigns its tiles to CTAs up front, so a CTA that finds no free SM --
 * because a collective running on another stream holds some -- starts only when a whole CTA's share of tiles has
 * finished elsewhere.  A host that overlaps collectives with these products leaves the collective's SMs free
 * instead.  Host-side state read at launch time; no counterpart in the reference (its kernels are not persistent). */
int toner_set_gemm_sm_limit(int32_t sms);
/* Self-test of that mechanism (the reference has no device-side waits): launches a one-warp kernel whose wait can
 * never be satisfied and gives up after `limit_cycles` SM cycles (at most 2e9).  The kernel returns normally, the
 * next toner_device_status reports 199, and the context stays usable. */
int toner_selftest_bounded_wait(long long limit_cycles, void* stream);

/* ------------------------------------------------------------------ generic tensor-core product
 * D[b] = alpha * sum_s A_s[b] * B_s[b]^T (+ beta * C[b]), 16-bit operands, FP32 accumulation in tensor
 * memory.  This is the one contraction kernel under every operator below; it is exported for tests and
 * for callers that want to fuse differently.  Replaces torch.mm/bmm(out_dtype=float32)
 * (src/toner/linalg.py:18, src/toner/fast/muon.py:9-33), mm16 / apply16_raw (src/toner/fast/roots.py:95-119)
 * and the Triton symmetric product (src/toner/fast/symm16.py:16-127). */
typedef struct toner_operand {
  const void* base;         /* first element of z-slice 0 (FP16 or BF16) */
  const void* const* list;  /* optional HOST array of `batch` device pointers: separately allocated matrices */
  int32_t rows, cols;       /* stored shape of one slice, cols contiguous */
  int64_t ld;               /* elements between stored rows (multiple of 8) */
  int64_t z_stride;         /* elements between z-slices */
  int32_t nz;               /* number of z-slices reachable from base */
  int32_t mn_major;         /* 0: stored as (M or N) x K;  1: stored as K x (M or N), i.e. a transposed view */
  int32_t seg_z[3];         /* z-slice of batch 0 for each K segment */
  int32_t z_step;           /* batch b reads z-slice seg_z[s] + b * z_step (0: every batch reads the same slice) */
} toner_operand;

typedef struct toner_gemm_desc {
  toner_operand a, b;
  int32_t m, n, k, batch;
  int32_t segs;             /* 1..3 operand-plane pairs accumulated into one result */
  int32_t fmt;              /* operand format: 0 FP16, 1 BF16 */
  int32_t tri;              /* 1: result symmetric (m == n); compute only tiles meeting the upper triangle */
  int32_t mirror;           /* with tri: also store the transposed element (full symmetric result) */
  int32_t packed;           /* with tri: C / D are packed upper triangles, row r starts at r*n - r(r+1)/2 + r */
  float alpha, beta;
  const float* alpha_a;     /* optional per-batch factors multiplied into alpha */
  const float* alpha_b;     /*   alpha_b is read at alpha_b[b * alpha_b_step] (0 means 1) */
  const float* beta_v;      /* optional per-batch factor multiplied into beta */
  int32_t alpha_b_step;
  const float* c; int64_t ldc, c_bs;
  float* d;       int64_t ldd, d_bs;       /* optional FP32 result */
  void* d16;      int64_t ld16, d16_bs;    /* optional 16-bit copy of the result */
  int32_t d16_fmt;                         /* 0 FP16, 1 BF16 */
  float* sumsq;             /* optional per-batch accumulators (caller zeroes them): sum d^2, */
  uint32_t* maxabs;         /*   max |d| as FP32 bits, */
  uint32_t* maxaff;         /*   max |aff_a*[r==c] + aff_b*d| as FP32 bits */
  float aff_a, aff_b;
  int32_t tile_n;           /* 0 = choose; else 128 or 256 (128-row tiles), 512 = 256 x 256 tiles on CTA pairs,
                               1024 = 256 x 512 tiles on CTA pairs (no chained accumulation) */
  int32_t promote;          /* > 0: k-blocks (64 deep) per tensor-core accumulation chain; chains are summed in
                               FP32 registers with round-to-nearest (the tensor core truncates).  0: one chain */
  int32_t raster;           /* tile columns per rasterisation group for full schedules (0: default 8) */
  int32_t promote_all;      /* 0: chain only the first segment (later segments of a split product are 2^-11 of
                               it and form one chain each); 1: chain every segment */
  /* Optional FP16 hi/lo operand planes of the result, written by the same kernel so that the next
   * split-precision product needs no separate splitting pass:
   *   split0: planes of split0_scale * d
   *   split1: planes of split1_scale * (split1_aff_a * [r==c] + split1_aff_b * d)
   * hi plane element (b, r, c) at split + b*split_bs + r*split_ld + c, lo plane split_plane elements further.
   * The scales are the caller's (powers of two chosen from a bound on |d|; FP16 overflows above 65504). */
  void* split0;
  void* split1;
  int64_t split_ld, split_bs, split_plane;
  float split0_scale, split1_scale, split1_aff_a, split1_aff_b;
  uint32_t* maxres;         /* optional per-batch accumulator: max |[r==c] - d| as FP32 bits */
  int32_t upper_d;          /* with tri + mirror: write the FP32 result d on and above the diagonal only (the 16-bit copy
                               and the operand planes are still mirrored) -- for a result whose FP32 form is read back
                               as the upper-triangle `c` of another symmetric product and nowhere else */
} toner_gemm_desc;

int toner_gemm(const toner_gemm_desc* desc, void* stream);

/* Diagnostics (the reference has none at this level; its engine reports phase times only,
 * src/toner/fast/adapter.py:536-545).  While enabled, every toner_gemm launch adds cycle counts, summed over
 * its CTAs, to eight counters: [0] MMA warp busy in its tile loop, [1] MMA warp waiting for a free accumulator,
 * [2] MMA warp waiting for operands, [3] TMA warp waiting for a free stage, [4] first epilogue warp waiting for an
 * accumulator, [5] that warp writing results, [6] that warp summing chains, [7] number of CTAs.
 * The call synchronises `stream`, copies the counters to out8 (HOST, may be NULL), clears them, then switches
 * the counting on or off.  Off by default; enabling allocates 64 bytes of device memory. */
int toner_gemm_phase_cycles(int enable, void* stream, unsigned long long* out8);

/* ------------------------------------------------------------------ input statistics
 * Upper-triangle SYRK  S_b = X_b^T X_b  over BF16 row buffers, FP32 accumulation.
 *   mode 0  PACKED      out (k, n(n+1)/2) = S           replaces syrk_list_packed(acc=False)  src/toner/fast/syrk.py:192-217
 *   mode 1  PACKED_ACC  out += S                        replaces syrk_list_packed(acc=True)   src/toner/fast/syrk.py:144-146,192-217
 *   mode 2  EMA_FULL    out (k, n, n) = beta*out + gamma*S, mirrored   replaces syrk_ema     src/toner/fast/syrk.py:250-304
 * Row buffers: either `x_list` (HOST array of k device pointers, as list_offsets() addresses separately
 * allocated buffers, src/toner/fast/syrk.py:62-69) or a stack at `x_base` with `x_batch_stride` elements
 * between buffers.  Each buffer is (rows, n) BF16 with `ld` elements between rows; n and ld multiples of 8. */
int toner_syrk_upper(const void* const* x_list, const void* x_base, int64_t x_batch_stride, int32_t k,
                     int32_t rows, int32_t n, int64_t ld, float* out, int32_t mode, float beta, float gamma,
                     void* stream);

/* Sampled-row capture: dst[(b*count + j), :] = BF16(x[b, positions[j], :]) for a (batch, seq, n) activation tensor
 * (BF16, or FP32 when x_is_fp32: rounded to BF16 as autocast would), `positions` a DEVICE array of `count` token
 * indices (toner's head-then-stride sample).  dst is (batch*count, n) BF16, typically a slice of the statistic's
 * row buffer.  Strides in elements; rows 16-byte aligned; n a multiple of 8; positions are not range-checked.
 * Replaces x.index_select(1, positions) + copy in the capture hooks (src/toner/fast/adapter.py:398-402,
 * src/toner/statistics.py:68-80) and the row-gather capture kernel (reproduce/marin/ops.py:10-27). */
int toner_gather_rows(const void* x, int32_t x_is_fp32, int32_t batch, int32_t seq, int32_t n, int64_t batch_stride,
                      int64_t row_stride, const int32_t* positions, int32_t count, void* dst, void* stream);

/* Row capture for a whole model in one launch: every job writes the sampled rows of one micro-batch into one
 * statistic's row buffer, copied or recomputed from tensors the forward pass keeps anyway.  For job j and sampled
 * row r = b * positions + p:   src = a + b * batch_stride + idx[p] * row_stride;   dst row = at[r]  (width elements)
 *   TONER_CAPTURE_COPY      dst = a row                                         (a BF16)
 *   TONER_CAPTURE_RMSNORM   out = bf16(x * rsqrt(mean(x^2) + eps)); dst = bf16(float(bf16(w)) * float(out))
 *                           (a = x BF16, b = w FP32 of `width` elements: the model's BF16-residual RMSNorm)
 *   TONER_CAPTURE_SILU_MUL  dst = bf16(g * (1 / (1 + exp(-g))) * u) in FP32     (a = g, b = u, both BF16, same strides)
 *   TONER_CAPTURE_COPY_F32  dst = bf16(a row)                                   (a FP32: the input of a projection that
 *                           runs under BF16 autocast, rounded as autocast rounds it; strides in FP32 elements)
 * The job table is passed twice: `jobs_host` is validated, `jobs_device` (the same n_jobs entries in device memory)
 * is what the kernel reads; a caller keeps both for as long as the tensors' addresses repeat.  `at` and `idx` are
 * DEVICE int64 arrays of batch*positions and positions entries (not range-checked).  Widths and strides in
 * elements, multiples of 8; pointers 16-byte aligned; destination buffers are (capacity, width) BF16, contiguous.
 * Replaces capture_rows / capture_recomputed and their kernels _gather_rows, _norm_rows, _silu_mul_rows
 * (reproduce/marin/ops.py:10-27,30-54,63-100,107-163), four launches per micro-batch there. */
enum { TONER_CAPTURE_COPY = 0, TONER_CAPTURE_RMSNORM = 1, TONER_CAPTURE_SILU_MUL = 2, TONER_CAPTURE_COPY_F32 = 3 };
typedef struct toner_capture_job {
  const void* a;
  const void* b;
  void* dst;
  int64_t batch_stride, row_stride;
  int32_t width;
  int32_t kind;
} toner_capture_job;
int toner_capture(const toner_capture_job* jobs_device, const toner_capture_job* jobs_host, int32_t n_jobs,
                  const int64_t* at, const int64_t* idx, int32_t batch, int32_t positions, float eps, void* stream);

/* C_b <- beta*C_b + gamma*S_b with S_b read from its packed upper triangle and mirrored.
 * Replaces unpack_ema_ (src/toner/fast/syrk.py:220-247); general-path EMA src/toner/reference.py:79. */
int toner_unpack_ema(const float* packed, float* ema, int32_t k, int32_t n, float beta, float gamma, void* stream);

/* ------------------------------------------------------------------ FP32-accurate operand preparation
 * Split an FP32 stack into FP16 hi/lo planes of x*scale, scale = power of two putting max|x| of each
 * matrix in [2^13, 2^14); planes layout [2][batch][rows][cols] (hi plane first), inv_scale[b] = 1/scale.
 * Optionally the source is  aff_a*I + aff_b*x  (used to form T = alpha*I - beta*M on the fly).
 * `x_list` (DEVICE array of batch pointers) may replace x for separately allocated matrices.
 * `maxabs` (DEVICE, FP32 bits, batch entries) must hold max|source|; pass NULL to have it computed here
 * into the first `batch` words of `scratch` (DEVICE, >= 4*batch bytes).
 * Replaces _hi_lo / _cols_hi_scaled / rows_lo (src/toner/fast/roots.py:47-81). */
int toner_split16(const float* x, const float* const* x_list, int32_t batch, int32_t rows, int32_t cols,
                  int64_t ld, int64_t bs, float aff_a, float aff_b, const uint32_t* maxabs, void* scratch,
                  void* planes, float* inv_scale, void* stream);

/* ------------------------------------------------------------------ factor engine
 * Inverse roots of the damped, trace-normalised statistics, as the general path computes them with eigh
 * (input_factors, src/toner/linalg.py:54-89) and the fast path with exact_eigh_powers / its cached-basis
 * iteration (src/toner/fast/roots.py:293-336,466-482):
 *     A_b = sym(C_b) / mean(diag C_b) + damping * I
 *     root_lo[b] = A_b^(-1/p)          root_hi[b] = A_b^(-q/p)   (q a power of two dividing p; q == 1: not written)
 *     fro2_lo[b] = ||root_lo[b]||_F^2  (gives the decay normalisation n / ||R||_F^2, src/toner/linalg.py:87-88)
 * Method: coupled Newton iteration T = a I - b M, X <- X T, M <- T^p M with minimax-scaled (a, b), batched
 * over the k statistics, all products FP32-accurate on tensor cores (FP16 hi/lo planes, three plane products
 * per accumulator).  The last of the `iters` steps applies a polynomial q(R) ~ (I - R)^(-1/p), R = I - M, to X
 * alone: the Chebyshev interpolant of (1 - r)^(-1/p) on [-0.02, 1.15 e + 1e-3] of the smallest degree with relative
 * error below 3e-6, e being the bound on R the schedule guarantees (toner_inv_roots_finish_order_for,
 * toner_inv_roots_schedule); its degree - 1 products are single passes over FP16 planes of R.
 * `iters` <= 0 selects toner_inv_roots_iterations(n, damping, p), which depends only on
 * its arguments (8 for p = 8, 8 for p = 4, 10 for p = 2 at n = 5632, damping 1e-3): the count with the fewest
 * plane passes, Newton steps and series together.
 * status[b] (DEVICE, optional): 0 converged, 1 residual max|I - M| above 0.5 before the last step,
 * 2 non-finite, 3 / 4 a caller's spectrum bound that did not hold (toner_inv_roots_ex / _tracked).  The caller decides what to do with a non-zero status (the Python host recomputes that
 * statistic with an eigendecomposition, as the reference's fallback does, src/toner/fast/engine.py:714-731).
 * Workspace: toner_inv_roots_workspace_bytes(chunk, n) lets `chunk` statistics be processed at once; a
 * smaller workspace makes the call loop over chunks (it must hold at least one statistic). */
size_t toner_inv_roots_workspace_bytes(int32_t chunk, int32_t n);
int toner_inv_roots_iterations(int32_t n, float damping, int32_t p);
int toner_inv_roots_iterations_for(float lower, int32_t p);   /* the count for a given spectrum lower bound */
/* degree of the finishing polynomial for that bound and count (iters <= 0: the default count); 0 on bad arguments */
int toner_inv_roots_finish_order_for(float lower, int32_t p, int32_t iters);
/* The whole schedule the engine runs for a spectrum lower bound (host only, no device needed): returns the step count
 * (iters <= 0: the default), and writes the (a_k, b_k) of its count - 1 Newton steps (ab_out: pairs of doubles, as many
 * as ab_capacity holds), the degree of the finishing polynomial (order_out), its coefficients c_0 .. c_degree in powers
 * of r (coef_out, as many as coef_capacity holds; at most 13), and the distance e of the last M from I it is cut for
 * (e_out).  Every output pointer is optional.  0 on bad arguments.  With these a scalar can be taken through exactly
 * what the engine does to every eigenvalue: x = 1, mu = lambda; per step t = a - b mu, x *= t, mu *= t^p; finally
 * x * q(1 - mu) = lambda^(-1/p). */
int toner_inv_roots_schedule(float lower, int32_t p, int32_t iters, double* ab_out, int32_t ab_capacity, double* coef_out,
                             int32_t coef_capacity, int32_t* order_out, double* e_out);
int toner_inv_roots(const float* ema, int32_t k, int32_t n, float damping, int32_t p, int32_t q, int32_t iters,
                    float* root_lo, float* root_hi, float* fro2_lo, int32_t* status, void* workspace,
                    size_t workspace_bytes, void* stream);
/* The same with what a caller that factors slowly changing statistics every step can add:
 *   lower     lower bound of the spectrum of A' / ||A'||_F valid for every statistic of the call (0: use the bound
 *             damping / (n (1 + damping)) that always holds).  A larger bound means fewer Newton steps
 *             (toner_inv_roots_iterations_for).  The bound is checked on the device: status[b] = 3 where
 *             damping / norm_out[b] lies below it, and the caller recomputes that statistic.
 *   norm_out  (DEVICE, optional, k floats) the bound of lambda_max(A'_b) the engine normalised by: the smallest of ||A'||_F
 *             and 1.03 ||A'||_F ||P^(2^j)||_F^(1/2^j), j = 1, 2, 3, with P = A' / ||A'||_F (three extra single-pass
 *             products; (sum lambda^16)^(1/16) bounds lambda_max far more tightly than the Frobenius norm when the spectrum
 *             is flat).  The caller derives next step's bound from it: lower = margin * damping / max_b norm_out[b].
 * A' is A with its dominant eigen-direction deflated: six power-iteration steps find (lambda_1, v); where they
 * converged (residual below 1e-5) and lambda_1 stands above 8x the mean of the rest, the engine factors
 * A' = A - (lambda_1 - c) v v^T and adds (lambda_1^(-1/p) - c^(-1/p)) v v^T back to the root.  This is what the
 * reference's eigendecomposition does implicitly for the mean-activation direction of an input statistic
 * (src/toner/linalg.py:72-86); toner_inv_roots deflates too. */
int toner_inv_roots_ex(const float* ema, int32_t k, int32_t n, float damping, int32_t p, int32_t q, int32_t iters,
                       float lower, float* root_lo, float* root_hi, float* fro2_lo, int32_t* status, float* norm_out,
                       void* workspace, size_t workspace_bytes, void* stream);

/* The same for a caller that factors the same slowly changing statistics step after step and wants the schedule to
 * follow the actual spectrum instead of the bound damping / norm that always holds (the reference's engine exploits
 * the same slowness with a cached eigenbasis and two warm iterations, src/toner/fast/engine.py:504-553):
 *   track          (DEVICE, k * n floats, kept by the caller between calls) for each statistic a unit vector along the
 *                  eigenvector of the smallest eigenvalue of A.  After the roots are computed the call advances it by
 *                  `track_sweeps` power-iteration steps on the highest inverse power (A^(-q/p)), where that eigenvalue
 *                  is the dominant one however small it is next to lambda_max(A); track_sweeps + 256 starts from a
 *                  fixed vector instead of the buffer's content (first call, or after the statistics were replaced).
 *   lmin_out       (DEVICE, optional, k floats) the estimate of lambda_min(A_b) that comes with it: a Rayleigh quotient,
 *                  so it errs on the high side (by 5-25 % after 8 sweeps from scratch, less once tracking).
 *   lower, lower_is_estimate
 *                  with lower_is_estimate = 1, `lower` is the caller's ESTIMATE of the lower end of the spectrum of
 *                  A' / norm, typically margin * min_b lmin_out[b] / norm_out[b] of the previous call.  Such a bound
 *                  cannot be checked in advance; it is verified after the chain: four power-iteration steps on
 *                  R = I - M of the last M, from the tracked direction, estimate ||R||_2, and status[b] = 4 where that
 *                  exceeds what the finishing series was cut for (by 15 % + 1e-3).  The caller recomputes such a
 *                  statistic with the bound that always holds.  resid_out (DEVICE, optional, k floats) receives the
 *                  estimate.  With lower_is_estimate = 0 the call is toner_inv_roots_ex (plus tracking).
 *   deflate, deflate_rank, deflated_out
 *                  `deflate` (DEVICE, k * 8 * n floats, kept by the caller between calls; optional): eight vector slots
 *                  per statistic for the dominant eigen-directions.  With it the engine looks for deflate_rank (1..8)
 *                  directions instead of one, by block power iteration with Rayleigh-Ritz (one pass over the statistic
 *                  per sweep whatever the rank; four sweeps from the buffer's vectors, eight from fixed ones when 256 is
 *                  added to deflate_rank), and deflates those that converged (residual below 1e-5) and stand above 8x
 *                  the mean of everything else, in descending order.  deflated_out (DEVICE, optional, k ints): how many, in
 *                  bits 0..7; bits 8..15: how many Ritz values stand above that mark whether converged or not.
 *                  Outlier features of an activation statistic are such directions; each one deflated lowers
 *                  lambda_max(A') and with it the number of Newton steps.
 * The upper end: norm_out is a certified bound, the smallest of ||A'||_F times ||P^2||_F^(1/2), ||P^4||_F^(1/4),
 * ||P^8||_F^(1/8) (three single-pass squarings).  With 512 added to deflate_rank (only with lower_is_estimate = 1 and
 * without 256) it is an estimate instead and the squarings are skipped: 1.4 times the largest Ritz value of the block
 * iteration that was NOT deflated, never above ||A'||_F.  That value errs low, by up to a fifth at the dense edge of
 * a bulk, once its vector is a few calls old (the caller's business: a fresh slot's value sits near the mean
 * eigenvalue).  An eigenvalue of
 * A' / norm above 1 comes out of the first Newton step below the lower bound and lags like one below `lower`; the
 * verification looks for it with four more steps from that Ritz vector, status 4 as above. */
int toner_inv_roots_tracked(const float* ema, int32_t k, int32_t n, float damping, int32_t p, int32_t q, int32_t iters,
                            float lower, int32_t lower_is_estimate, float* root_lo, float* root_hi, float* fro2_lo,
                            int32_t* status, float* norm_out, float* track, float* lmin_out, float* resid_out,
                            int32_t track_sweeps, float* deflate, int32_t deflate_rank, int32_t* deflated_out,
                            void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------ Newton-Schulz polar iteration
 * x = u / (||u||_F + eps); `steps` times  A = x x^T (on the short side),  x <- a x + (b A + c A A) x  with
 * (a, b, c) = (3.4445, -4.7750, 2.0315); every product takes BF16-rounded operands and accumulates /
 * outputs FP32 ("tpu" mode), x itself is carried in FP32.  Tall matrices are iterated through x^T x and
 * x (b A + c A A), which is the same arithmetic as transposing first.
 * Replaces newton_schulz_batched (src/toner/fast/muon.py:36-50) and newton_schulz(mode="tpu")
 * (src/toner/linalg.py:22-51).  u and x_out are (batch, m, n) stacks and may alias; m, n multiples of 8.
 * maxabs_out (optional, DEVICE, batch words): max |x| of the result as FP32 bits. */
size_t toner_ns_polar_workspace_bytes(int32_t batch, int32_t m, int32_t n);
int toner_ns_polar(const float* u, int32_t batch, int32_t m, int32_t n, int32_t steps, float eps, float* x_out,
                   uint32_t* maxabs_out, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------ elementwise update kernels
 * Stacks are `count` matrices of `per` elements each (per a multiple of 4); gradient and weight tensors
 * are caller-owned and separately allocated, so they come as DEVICE arrays of `count` device pointers. */

/* out[b] = sum of squares of matrix b; bitwise reproducible (fixed reduction tree, no float atomics).
 * Stands in for Tensor.norm()/matrix_norm (src/toner/reference.py:207,309-311; src/toner/linalg.py:41).
 * scratch: toner_sumsq_scratch_bytes(batch) bytes. */
size_t toner_sumsq_scratch_bytes(int32_t batch);
int toner_sumsq(const float* x, int32_t batch, int32_t rows, int32_t cols, int64_t ld, int64_t bs, float* scratch,
                float* out, void* stream);

/* toner_sumsq without caller scratch (no counterpart in the reference: it exists for hosts that cannot hand
 * this library device memory to work in -- for instance an embedding whose every device byte is budgeted and
 * owned by its own pool, so that neither a scratch tensor for the caller nor a cudaMalloc inside a library is
 * acceptable).  The partial sums go to an array that is part of the library image: 296 KB on every device that
 * loads the library, held until the process exits.  Limit: batch <= toner_sumsq_static_max_batch() (256);
 * larger batches are refused with an error, not truncated.  The result has the same bits as toner_sumsq.
 * The call allocates and frees nothing (no cudaMalloc / cudaFree, no allocating library routine) and does not
 * create the library's per-device context.  The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current); make that first call before any stream capture begins.
 * All calls on a device share the one array: two calls whose kernels may overlap on the GPU (different
 * streams without an ordering between them) race on it -- keep them on one stream or order them with events.
 * Nothing needs clearing between calls: each call overwrites every partial sum before reading it. */
int toner_sumsq_static_max_batch(void);
int toner_sumsq_static(const float* x, int32_t batch, int32_t rows, int32_t cols, int64_t ld, int64_t bs, float* out,
                       void* stream);

/* m <- mu*m + g ; u = nesterov ? g + mu*m : m ; maxabs[b] = max|u| (FP32 bits, optional).
 * Replaces src/toner/reference.py:197-202 and _muont_in's momentum (src/toner/fast/engine.py:35-39). */
int toner_muont_momentum(const float* const* grad_ptrs, float* m, float* u, int32_t count, int64_t per, float mu,
                         int32_t nesterov, uint32_t* maxabs, void* stream);

/* Per-matrix scalars of the MuonT update, from ||R_out||_F^2 of the statistic first + b*step:
 * c1[b] = lr*wd*n/||R||^2 (shaped decay W R^2 / mean diag R^2), c2[b] = lr*scale*sqrt(n)/||R|| (R-hat).
 * Replaces the scalar part of _muont_out (src/toner/fast/engine.py:42-51; src/toner/reference.py:206-215). */
int toner_muont_coeffs(const float* fro2, int32_t first, int32_t step, int32_t count, int32_t n, float lr, float wd,
                       float scale, float* c1, float* c2, void* stream);

/* a[b] *= b[b]: folds a per-matrix scalar into an operand's inverse scale. */
int toner_scale_vec(float* a, const float* b, int32_t count, void* stream);

/* m <- beta1*m + (1-beta1)*g.  Replaces src/toner/reference.py:304 / _adamt (src/toner/fast/engine.py:21). */
int toner_adamt_first_moment(const float* const* grad_ptrs, float* m, int32_t count, int64_t per, float beta1,
                             void* stream);

/* v <- beta2*v + (1-beta2)*t^2 ; num <- num / (sqrt(v/bc2) + eps) in place (num holds (m/bc1) R);
 * maxabs[b] = max|num| afterwards.  Replaces src/toner/reference.py:306-308 / engine.py:23-24. */
int toner_adamt_ratio(const float* t, float* v, float* num, int32_t count, int64_t per, float beta2, float bc2,
                      float eps, uint32_t* maxabs, void* stream);

/* c1[b] = lr*wd*n/||R||^2 ; c2[b] = -lr*||U||_F / max(||U R||_F, 1e-30) from the two sums of squares.
 * Replaces the scalar part of src/toner/reference.py:309-313 / engine.py:26-32. */
int toner_adamt_coeffs(const float* fro2, int32_t first, int32_t step, int32_t count, int32_t n, float lr, float wd,
                       const float* ss_before, const float* ss_after, float* c1, float* c2, void* stream);

/* out = a*x + b*y over n FP32 elements (16-byte aligned pointers).  The general path's statistic EMA
 * C <- beta*C + (1-beta)*S on full matrices (src/toner/reference.py:79). */
int toner_axpby(const float* x, const float* y, float* out, int64_t n, float a, float b, void* stream);

/* out_b = coeff[b] * x_b (used for the AdamT change when weight_decay is zero: -lr ||U||/||U R|| U R). */
int toner_scale_stack(const float* x, const float* coeff, float* out, int32_t count, int64_t per, void* stream);

/* W_b += delta_b.  Replaces torch._foreach_add_ (src/toner/fast/engine.py:875). */
int toner_apply_delta(float* const* weight_ptrs, const float* delta, int32_t count, int64_t per, void* stream);
/* W_b <- weight_scale * W_b + delta_scale * delta_b: the plain Muon baseline's decoupled decay p.mul_(1 - lr wd)
 * and p.add_(o, alpha = -lr sqrt(max(1, rows / cols))) in one pass (src/toner/fast/muon.py:118-119,160-164). */
int toner_apply_scaled(float* const* weight_ptrs, const float* delta, int32_t count, int64_t per, float weight_scale,
                       float delta_scale, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TONER_B200_H_ */

// Factor engine: inverse p-th roots of damped, trace-normalised input statistics by a coupled Newton
// iteration with minimax scaling, every product on the tcgen05 GEMM in FP32-accurate split precision.
//
//   A   = sym(C) / mean(diag C) + damping * I                 (what the reference factors by eigh)
//   A'  = A - (lambda_1 - c) v v^T                            (dominant direction deflated when power iteration finds it)
//   M_0 = A' / beta,  beta >= lambda_max(A')                  (beta = min(||A'||_F, 1.04 ||A'||_F ||P^2||_F^(1/2)), P = A'/||A'||_F)
//   T_k = a_k I - b_k M_k ;  X_{k+1} = X_k T_k ;  M_{k+1} = T_k^p M_k          (X_0 = I)
//   X_K = X_{K-1} (c0 I + c1 R + c2 R^2 + ... ),  R = I - M_{K-1}               (Chebyshev fit of (1 - r)^(-1/p))
//   X_K ~ M_0^{-1/p}  =>  A^{-1/p} = X_K beta^{-1/p} + (lambda_1^{-1/p} - c^{-1/p}) v v^T
// (a_k, b_k) map the interval [l_k, 1] known to contain the spectrum of M_k onto [l_{k+1}, 1] with
// l_{k+1} as large as a linear T allows (the ends of the interval and the interior maximum of
// mu (a - b mu)^p are levelled, subject to a cap on b/a that bounds the dynamic range of T^p); once
// l_k is close to 1 they become the Newton values ((p+1)/p, 1/p).
// l_0 is the caller's lower bound of the spectrum of M_0 (checked per statistic on the device), or
// damping / (n (1 + damping)), which always holds; the schedule and the iteration count depend only on
// (l_0, p), so they are fixed before anything is launched and stated by toner_inv_roots_iterations[_for].
// Every operand of every product is a pair of FP16 hi/lo planes written by the epilogue of the product that
// made it, scaled by a power of two taken from a norm bound known in advance.
#include <cmath>
#include <cstdlib>
#include <vector>

#include "runtime.cuh"

namespace toner {

struct NewtonStep {
  double a, b, lower;
};

// Dynamic range allowed for T^p.  The unconstrained minimax step sends the top of the spectrum (mu = 1)
// down to the new lower bound, i.e. T = a I - b M gets an eigenvalue (a - b) << a and T^p spans
// (a / (a - b))^p; a component that small relative to ||T^p|| is lost in operand rounding and can come
// out negative, after which the iteration diverges.  Capping b / a keeps every eigen-component of T^p
// above 1e-3 of its norm, at the price of one more iteration.
constexpr double kMaxPowerRange = 1e3;

// Minimax-scaled schedule; returns the steps and the final lower bound of the spectrum.
static std::vector<NewtonStep> newton_schedule(double l0, int p, int iters, double* lower_out) {
  std::vector<NewtonStep> out;
  const double max_ratio = 1.0 - std::pow(kMaxPowerRange, -1.0 / p);
  double l = l0;
  for (int k = 0; k < iters; ++k) {
    NewtonStep s;
    s.lower = l;
    const double r = std::pow(l, 1.0 / p);
    double ratio = (l < 1.0 - 1e-9) ? (1.0 - r) / (1.0 - r * l) : 0.0;  // b/a levelling f(l) = f(1)
    if (ratio > max_ratio) ratio = max_ratio;
    const double mu_star = ratio > 0 ? 1.0 / (ratio * (p + 1)) : 2.0;   // interior maximum of f
    if (mu_star < 1.0 && mu_star > l) {
      const double fmax = mu_star * std::pow((double)p / (p + 1), p);    // with a = 1
      const double f_low = l * std::pow(1.0 - ratio * l, p), f_top = std::pow(1.0 - ratio, p);
      s.a = std::pow(fmax, -1.0 / p);                                    // rescale so that max f = 1
      s.b = s.a * ratio;
      l = (f_low < f_top ? f_low : f_top) / fmax;
    } else {
      s.a = (p + 1.0) / p;
      s.b = 1.0 / p;
      l = l * std::pow((p + 1.0 - l) / p, p);
    }
    if (l > 1.0) l = 1.0;
    out.push_back(s);
  }
  if (lower_out) *lower_out = l;
  return out;
}

// k-blocks (64 deep) per tensor-core accumulation chain for the products that update M, given the lower
// bound of M's spectrum (0 = one chain over the whole product, the fastest kernel).  Truncation costs about
// 1.2e-7 per k-block on same-sign sums, i.e. up to 1e-5 over a whole product of depth 5632; the damage to the
// result is that divided by the smallest eigenvalue of M.
static int chain_length(double lower) {
  if (lower < 5e-3) return kPromoteAccurate;
  if (lower < 5e-2) return kPromoteLinear;
  return 0;
}

// Products applied to X (and the final squarings) pass their error on linearly: one chain, about 1e-5.
constexpr int kPromoteX = 0;

// power-iteration steps spent on the dominant direction (each one pass over the statistic)
constexpr int kPowerSteps = 6;

// The last step does not square the error once more; it finishes with a polynomial q(R) ~ (I - R)^(-1/p), R = I - M:
// X <- X q(R).  The spectrum of R lies in [0, e] with e known from the schedule, so q is fixed in advance: the
// Chebyshev interpolant of (1 - r)^(-1/p) on [kFinishLow, kFinishGrow e + kFinishPad] (the margins cover rounding
// at the lower end and the allowance an estimated bound is verified with at the upper end) of the smallest degree
// whose relative error stays below kFinishTail there.  Spreading the error over the interval takes about half
// the degree of the binomial series, whose error sits at r = e alone (e = 0.5, p = 8: degree 6 instead of 12).
// The powers come from m - 1 single-pass products of FP16 planes in Horner form (a third of a split-precision
// product each; R is small, so its rounding to FP16 costs about 5e-4 c_2 e^2), which is cheaper than the log2(p) + 2
// split-precision products of one more Newton step; the step count is the one with the fewest plane passes in total.
constexpr double kFinishRadius = 0.6;
constexpr int kMaxFinishOrder = 12;
constexpr double kFinishTail = 3e-6;
constexpr double kFinishLow = -0.02, kFinishGrow = 1.15, kFinishPad = 1e-3;

struct FinishPoly {
  int order = 0;                       // 0: no degree up to the cap reaches the bound at this distance
  double c[kMaxFinishOrder + 1] = {};  // q(r) = sum_j c[j] r^j
};

// Degree-m Chebyshev interpolant of (1 - r)^(-1/p) on [lo, hi] as monomial coefficients; returns its largest
// relative error on the interval.
static double finish_fit(int p, double lo, double hi, int m, double* c) {
  const double kPi = 3.14159265358979323846;
  double cheb[kMaxFinishOrder + 1];
  for (int j = 0; j <= m; ++j) {
    double acc = 0.0;
    for (int k = 0; k <= m; ++k) {
      const double th = kPi * (k + 0.5) / (m + 1);
      const double r = lo + (hi - lo) * (std::cos(th) + 1.0) * 0.5;
      acc += std::pow(1.0 - r, -1.0 / p) * std::cos(j * th);
    }
    cheb[j] = acc * (j == 0 ? 1.0 : 2.0) / (m + 1);
  }
  // sum_j cheb[j] T_j(x) in powers of x (T_{j+1} = 2 x T_j - T_{j-1}) ...
  double t0[kMaxFinishOrder + 1] = {1.0}, t1[kMaxFinishOrder + 1] = {0.0, 1.0}, px[kMaxFinishOrder + 1] = {};
  px[0] = cheb[0];
  for (int i = 0; i <= m; ++i) px[i] += (m >= 1 ? cheb[1] : 0.0) * t1[i];
  for (int j = 2; j <= m; ++j) {
    double t2[kMaxFinishOrder + 1] = {};
    for (int i = 0; i <= m; ++i) t2[i] = (i > 0 ? 2.0 * t1[i - 1] : 0.0) - t0[i];
    for (int i = 0; i <= m; ++i) {
      px[i] += cheb[j] * t2[i];
      t0[i] = t1[i];
      t1[i] = t2[i];
    }
  }
  // ... then in powers of r, x = alpha r + beta (Horner over the polynomial in x)
  const double alpha = 2.0 / (hi - lo), beta = -(hi + lo) / (hi - lo);
  for (int i = 0; i <= m; ++i) c[i] = 0.0;
  for (int j = m; j >= 0; --j) {
    for (int i = m; i >= 1; --i) c[i] = c[i] * beta + c[i - 1] * alpha;
    c[0] = c[0] * beta + px[j];
  }
  double worst = 0.0;
  const int samples = 256;
  for (int i = 0; i <= samples; ++i) {
    const double r = lo + (hi - lo) * i / samples;
    double q = 0.0;
    for (int j = m; j >= 0; --j) q = q * r + c[j];
    worst = std::fmax(worst, std::fabs(q * std::pow(1.0 - r, 1.0 / p) - 1.0));
  }
  return worst;
}

// In powers of r the fit's coefficients grow as the interval approaches the singularity at r = 1 (sooner for small p):
// sums with cancellation, which single-pass FP16 products would not survive and whose Horner intermediates
// W_j = sum_{k >= j} c_k r^(k-j+1) would leave the range the operand planes are scaled for.  Such a fit is not used.
constexpr double kFinishMaxCond = 2.5;   // sum_k |c_k| hi^k, against q(r) <= 1.8
constexpr double kFinishMaxTerm = 3.5;   // bound of every W_j (planes hold |x| <= 4)

static bool finish_usable(const FinishPoly& f, double hi) {
  double cond = 0.0;
  for (int k = f.order; k >= 0; --k) cond = cond * hi + std::fabs(f.c[k]);   // Horner of sum |c_k| hi^k
  if (cond > kFinishMaxCond) return false;
  double w = 0.0;
  for (int j = f.order; j >= 1; --j) {
    w = (w + std::fabs(f.c[j])) * hi;
    if (w > kFinishMaxTerm) return false;
  }
  return true;
}

static FinishPoly finish_poly(int p, double e) {
  FinishPoly f;
  if (!(e < kFinishRadius)) return f;
  const double hi = kFinishGrow * e + kFinishPad;
  for (int m = 2; m <= kMaxFinishOrder; ++m) {
    if (finish_fit(p, kFinishLow, hi, m, f.c) < kFinishTail) {
      f.order = m;
      if (!finish_usable(f, hi)) f.order = 0;
      return f;
    }
  }
  return f;
}
static int finish_order_or_zero(int p, double e) { return finish_poly(p, e).order; }
// A caller's own (too small) step count leaves M too far from I for a usable fit: the binomial series of
// (1 - r)^(-1/p) at the cap (all coefficients positive and below 1); status reports the statistic.
static FinishPoly finish_poly_or_best(int p, double e) {
  FinishPoly f = finish_poly(p, e);
  if (f.order) return f;
  f.order = kMaxFinishOrder;
  f.c[0] = 1.0;
  for (int j = 1; j <= kMaxFinishOrder; ++j) f.c[j] = f.c[j - 1] * (1.0 / p + j - 1) / j;
  return f;
}
static int finish_order(int p, double e) { return finish_poly_or_best(p, e).order; }

static int default_iterations(double l0, int p) {
  // k steps of M, then the finishing step on X alone: the k with the fewest plane passes,
  // 3 (log2 p + 2) per step of M and order - 1 for the series, among those the series can finish
  int log2p = 0;
  while ((1 << log2p) < p) ++log2p;
  int best = 0;
  long best_cost = 0;
  for (int k = 1; k < 64; ++k) {
    double l;
    newton_schedule(l0, p, k, &l);
    const double e = 1.0 - l;
    const int m = finish_order_or_zero(p, e);
    if (m) {
      const long cost = 3L * k * (log2p + 2) + (m - 1);
      if (!best || cost < best_cost) {
        best = k + 1;
        best_cost = cost;
      }
      if (m == 2) break;  // further steps only add cost
    }
  }
  return best ? best : 64;
}

// ------------------------------------------------------------------ elementwise helpers
__global__ void __launch_bounds__(256) trace_kernel(const float* __restrict__ c, int n, float* __restrict__ trace) {
  const int b = blockIdx.x;
  const float* C = c + (long long)b * n * n;
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += C[(long long)i * n + i];
  __shared__ float red[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    trace[b] = t;
  }
}

// A = sym(C) / max(trace/n, 1e-30) + damping I, written to `a`.
// 32x32 tile pairs so that C and C^T are both read along rows.
__global__ void __launch_bounds__(256) damp_kernel(const float* __restrict__ c, float* __restrict__ a, int n, float damping,
                                                   const float* __restrict__ trace) {
  const int ti = blockIdx.y, tj = blockIdx.x;
  if (ti > tj) return;
  __shared__ float up[32][33], lo[32][33];
  const long long b = blockIdx.z;
  const float* C = c + b * (long long)n * n;
  float* A = a + b * (long long)n * n;
  const float inv = 1.f / fmaxf(trace[b] / n, 1e-30f);
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int lr = ty + 8 * i;
    const int r = ti * 32 + lr, cc = tj * 32 + tx;
    up[lr][tx] = (r < n && cc < n) ? C[(long long)r * n + cc] : 0.f;
    const int r2 = tj * 32 + lr, c2 = ti * 32 + tx;
    lo[lr][tx] = (r2 < n && c2 < n) ? C[(long long)r2 * n + c2] : 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int lr = ty + 8 * i;
    {
      const int r = ti * 32 + lr, cc = tj * 32 + tx;
      if (r < n && cc < n) A[(long long)r * n + cc] = 0.5f * (up[lr][tx] + lo[tx][lr]) * inv + (r == cc ? damping : 0.f);
    }
    if (ti != tj) {
      const int r = tj * 32 + lr, cc = ti * 32 + tx;
      if (r < n && cc < n) A[(long long)r * n + cc] = 0.5f * (lo[lr][tx] + up[tx][lr]) * inv;
    }
  }
}

// FP16 hi/lo planes of the two operands the iteration starts from, from A (FP32, damped and normalised):
//   M_0 = A / ||A||_F  (scaled by s_m)      T_0 = a I - b M_0  (scaled by s_t)      X_1 = T_0
// planes layout [2][batch][n][n], hi plane first.  With t_planes == nullptr only the hi plane of M_0 is written (all
// that the single-pass squarings of the norm bound read).
// With defl_v the input is A and the deflation A' = A + sum_j coef[j] v_j v_j^T is applied on the way (the terms of
// rankr_update_kernel, in its order), so that A' is never written.
__global__ void __launch_bounds__(256) init_planes_kernel(const float* __restrict__ a32, int n, int batch,
                                                          const float* __restrict__ sumsq, float a, float b, float s_m,
                                                          float s_t, __half* __restrict__ m_planes,
                                                          __half* __restrict__ t_planes, __half* __restrict__ x_planes,
                                                          const float* __restrict__ defl_v = nullptr,
                                                          const float* __restrict__ defl_coef = nullptr, int defl_r = 0,
                                                          int vstride = 0) {
  const int bi = blockIdx.y;
  float cf[8];
  bool any = false;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    cf[j] = (defl_v != nullptr && j < defl_r) ? defl_coef[bi * 8 + j] : 0.f;
    any = any || cf[j] != 0.f;
  }
  const float* DV = defl_v ? defl_v + (long long)bi * vstride * n : nullptr;
  const long long nn = (long long)n * n;
  const float4* A = reinterpret_cast<const float4*>(a32 + bi * nn);
  const float f = rsqrtf(fmaxf(sumsq[bi], 1e-60f));
  __half* mh = m_planes + bi * nn;
  __half* ml = m_planes + ((long long)batch + bi) * nn;
  __half* th = t_planes + bi * nn;
  __half* tl = t_planes + ((long long)batch + bi) * nn;
  __half* xh = x_planes + bi * nn;  // X_1 = T_0: a second copy, because T's buffer is rewritten by the first step
  __half* xl = x_planes + ((long long)batch + bi) * nn;
  const int n4 = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nn / 4; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / n4), c = (int)(i - (long long)r * n4) * 4;
    float4 v = A[i];
    if (any) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (cf[j] != 0.f) {
          const float vr = DV[(long long)j * n + r];
          const float4 vc = *reinterpret_cast<const float4*>(DV + (long long)j * n + c);
          v.x = fmaf(cf[j], vr * vc.x, v.x); v.y = fmaf(cf[j], vr * vc.y, v.y);
          v.z = fmaf(cf[j], vr * vc.z, v.z); v.w = fmaf(cf[j], vr * vc.w, v.w);
        }
      }
    }
    const float m[4] = {v.x * f, v.y * f, v.z * f, v.w * f};
    __half h[4], l[4], g[4], k[4];
    if (t_planes == nullptr) {
#pragma unroll
      for (int e = 0; e < 4; ++e) h[e] = __float2half_rn(m[e] * s_m);
      *reinterpret_cast<uint2*>(mh + i * 4) = *reinterpret_cast<uint2*>(h);
      continue;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float x = m[e] * s_m;
      h[e] = __float2half_rn(x);
      l[e] = __float2half_rn(x - __half2float(h[e]));
      const float t = (((c + e) == r ? a : 0.f) - b * m[e]) * s_t;
      g[e] = __float2half_rn(t);
      k[e] = __float2half_rn(t - __half2float(g[e]));
    }
    *reinterpret_cast<uint2*>(mh + i * 4) = *reinterpret_cast<uint2*>(h);
    *reinterpret_cast<uint2*>(ml + i * 4) = *reinterpret_cast<uint2*>(l);
    *reinterpret_cast<uint2*>(th + i * 4) = *reinterpret_cast<uint2*>(g);
    *reinterpret_cast<uint2*>(tl + i * 4) = *reinterpret_cast<uint2*>(k);
    *reinterpret_cast<uint2*>(xh + i * 4) = *reinterpret_cast<uint2*>(g);
    *reinterpret_cast<uint2*>(xl + i * 4) = *reinterpret_cast<uint2*>(k);
  }
}

// ------------------------------------------------------------------ deflation of a dominant direction
// Activation statistics usually have one eigenvalue far above the rest (the mean activation).  It sets ||A||
// and with it the spectrum's lower bound after normalisation, i.e. the number of Newton steps and the
// attainable accuracy.  A few power-iteration steps find that eigenpair (lambda_1, v) to working accuracy when
// the gap is large; then  A' = A - (lambda_1 - c) v v^T  (c = mean of the remaining eigenvalues) has the same
// eigenvectors, and  A^{-s} = A'^{-s} + (lambda_1^{-s} - c^{-s}) v v^T.  When the iteration has not converged
// (no dominant direction) nothing is deflated.

// v_0: a fixed pattern of +-1 / sqrt(n)
__global__ void power_start_kernel(float* __restrict__ v, int n) {
  const int b = blockIdx.y;
  const float s = rsqrtf((float)n);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
    v[(long long)b * n + i] = (((unsigned)i * 2654435761u) >> 15) & 1u ? s : -s;
}

// y = A v, one warp per row, FP64 accumulation
__global__ void __launch_bounds__(256) gemv_kernel(const float* __restrict__ a, const float* __restrict__ v,
                                                   float* __restrict__ y, int n) {
  const int b = blockIdx.y;
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n) return;
  const float* A = a + ((long long)b * n + row) * n;
  const float* X = v + (long long)b * n;
  // Four products at a time are summed in FP32 (their rounding, 6e-8 of the partial sum, is that of the FP32 result
  // itself) and the partial sums in FP64: one conversion per four elements instead of eight -- conversions to FP64 run
  // at a quarter of the FP64 rate and were what bound this kernel.
  double acc = 0.0;
  for (int c = lane * 4; c < n; c += 128) {
    const float4 av = *reinterpret_cast<const float4*>(A + c);
    const float4 xv = *reinterpret_cast<const float4*>(X + c);
    acc += (double)fmaf(av.x, xv.x, fmaf(av.y, xv.y, fmaf(av.z, xv.z, av.w * xv.w)));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) y[(long long)b * n + row] = (float)acc;
}

// lambda = v.y / v.v (Rayleigh quotient), res = ||y - lambda v|| / ||lambda v||, then v <- y / ||y||.
// The residual is summed term by term: the shortcut ||y||^2 - lambda^2 cancels catastrophically.
__global__ void __launch_bounds__(256) power_norm_kernel(float* __restrict__ v, const float* __restrict__ y, int n,
                                                         float* __restrict__ lam, float* __restrict__ res) {
  const int b = blockIdx.x;
  float* V = v + (long long)b * n;
  const float* Y = y + (long long)b * n;
  __shared__ double red[3][8];
  __shared__ double tot[3];
  auto block_sum3 = [&](double a0, double a1, double a2) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      a0 += __shfl_xor_sync(0xffffffffu, a0, o);
      a1 += __shfl_xor_sync(0xffffffffu, a1, o);
      a2 += __shfl_xor_sync(0xffffffffu, a2, o);
    }
    __syncthreads();  // the previous round's totals have been read
    if ((threadIdx.x & 31) == 0) {
      red[0][threadIdx.x >> 5] = a0;
      red[1][threadIdx.x >> 5] = a1;
      red[2][threadIdx.x >> 5] = a2;
    }
    __syncthreads();
    if (threadIdx.x < 3) {
      double t = 0.0;
      for (int w = 0; w < 8; ++w) t += red[threadIdx.x][w];
      tot[threadIdx.x] = t;
    }
    __syncthreads();
  };
  double yy = 0.0, vy = 0.0, vv = 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const double t = Y[i], u = V[i];
    yy += t * t;
    vy += t * u;
    vv += u * u;
  }
  block_sum3(yy, vy, vv);
  yy = tot[0];
  vy = tot[1];
  vv = tot[2];
  const double l = vv > 0.0 ? vy / vv : 0.0;
  double rr = 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const double d = (double)Y[i] - l * (double)V[i];
    rr += d * d;
  }
  block_sum3(rr, 0.0, 0.0);
  rr = tot[0];
  const double inv = yy > 0.0 ? 1.0 / sqrt(yy) : 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) V[i] = (float)(Y[i] * inv);
  if (threadIdx.x == 0) {
    lam[b] = (float)l;
    res[b] = (l > 0.0 && vv > 0.0) ? (float)(sqrt(rr) / (l * sqrt(vv))) : INFINITY;
  }
}

// sigma = lambda_1 - c if the pair converged and stands well above the rest, else 0;  corr = lambda_1^{-1/p} - c^{-1/p}
__global__ void deflate_decide_kernel(const float* __restrict__ lam, const float* __restrict__ res, int k, int n,
                                      float damping, int p, float* __restrict__ neg_sigma, float* __restrict__ corr) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= k) return;
  const float l1 = lam[b];
  const float tr = (float)n * (1.f + damping);  // A has unit mean diagonal plus the damping
  const float c = (tr - l1) / (float)(n - 1);
  const bool ok = n > 1 && isfinite(l1) && isfinite(res[b]) && res[b] < 1e-5f && c > 0.f && l1 > 8.f * c;
  neg_sigma[b] = ok ? -(l1 - c) : 0.f;
  corr[b] = ok ? powf(l1, -1.f / p) - powf(c, -1.f / p) : 0.f;
}

// A_b += coef[b] v_b v_b^T  (skipped where coef is zero)
__global__ void __launch_bounds__(256) rank1_update_kernel(float* __restrict__ a, const float* __restrict__ v,
                                                           const float* __restrict__ coef, int n) {
  const int b = blockIdx.y;
  const float cf = coef[b];
  if (cf == 0.f) return;
  float* A = a + (long long)b * n * n;
  const float* V = v + (long long)b * n;
  const int n4 = n / 4;
  const long long total = (long long)n * n4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / n4), c = (int)(i - (long long)r * n4) * 4;
    const float vr = V[r];
    const float4 vc = *reinterpret_cast<const float4*>(V + c);
    float4 x = *reinterpret_cast<float4*>(A + (long long)r * n + c);
    // cf * (v_r v_c): the product v_r v_c is the same bits at (r, c) and (c, r), so symmetry is kept exactly
    x.x = fmaf(cf, vr * vc.x, x.x); x.y = fmaf(cf, vr * vc.y, x.y); x.z = fmaf(cf, vr * vc.z, x.z); x.w = fmaf(cf, vr * vc.w, x.w);
    *reinterpret_cast<float4*>(A + (long long)r * n + c) = x;
  }
}


// ------------------------------------------------------------------ deflation of several dominant directions
// Statistics of real activations often have a handful of directions far above the rest (outlier features), not just
// the mean.  Block power iteration with Rayleigh-Ritz finds r <= kMaxDeflate of them at the cost of one pass over the
// statistic per sweep, whatever r is, and converges with the ratio of the (r+1)-th eigenvalue to the wanted one, so
// close pairs among the dominant ones do not slow it down; the vectors are kept by the caller between calls.
// Vectors are stored vector-major: v[(b * vstride + j) * n + c].
constexpr int kMaxDeflate = 8;  // (init_planes_kernel keeps that many coefficients in registers)

// Y_j = A v_j, j < R: one pass over A.  A block takes 32 rows (four per warp) and walks the columns 256 at a time; the
// 256-column slice of the vectors is staged in shared memory once per block, so the vectors are read from L2 once per
// 32 rows instead of once per row pair (that traffic, not the pass over A, bounded the first version of this kernel).
// The products of four slices (32 per lane) are summed in FP32 before they join the FP64 sums: conversions and FP64
// additions run at a fraction of the FP32 rate, and with one per eight products they, not the pass over A, set the
// pace.  R (the number of vectors, rounded up to even) is a template argument so that absent vectors cost nothing.
constexpr int kBlockGemvRows = 32;
template <int R>
__global__ void __launch_bounds__(256) block_gemv_kernel(const float* __restrict__ a, const float* __restrict__ v,
                                                         float* __restrict__ y, int n, int r, int vstride) {
  __shared__ float4 sv[R][64];
  const int b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * kBlockGemvRows + warp * 4;
  const float* V = v + (long long)b * vstride * n;
  const float* A = a + (long long)b * n * n;
  double acc[4][R];
  float part[4][R];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < R; ++j) {
      acc[i][j] = 0.0;
      part[i][j] = 0.f;
    }
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  int slice = 0;
  for (int c0 = 0; c0 < n; c0 += 256, ++slice) {
    __syncthreads();  // the previous slice has been read
    for (int i = threadIdx.x; i < R * 64; i += 256) {
      const int j = i >> 6, col = c0 + (i & 63) * 4;
      sv[j][i & 63] = (j < r && col < n) ? *reinterpret_cast<const float4*>(V + (long long)j * n + col) : zero;
    }
    __syncthreads();
    const int ca = c0 + lane * 4, cb = ca + 128;
    // this lane's eight columns of every vector, read from shared memory once for the warp's four rows (read per
    // row, the shared-memory traffic is R times the traffic of A and sets the pace from four vectors on)
    float4 x0[R], x1[R];
#pragma unroll
    for (int j = 0; j < R; ++j) {
      x0[j] = sv[j][lane];
      x1[j] = sv[j][lane + 32];
    }
    float4 p0[4], p1[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = row0 + i;
      const float* Ar = A + (long long)row * n;
      p0[i] = (row < n && ca < n) ? *reinterpret_cast<const float4*>(Ar + ca) : zero;
      p1[i] = (row < n && cb < n) ? *reinterpret_cast<const float4*>(Ar + cb) : zero;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
      for (int j = 0; j < R; ++j) {
        const float s0 = fmaf(p0[i].x, x0[j].x, fmaf(p0[i].y, x0[j].y, fmaf(p0[i].z, x0[j].z, p0[i].w * x0[j].w)));
        const float s1 = fmaf(p1[i].x, x1[j].x, fmaf(p1[i].y, x1[j].y, fmaf(p1[i].z, x1[j].z, p1[i].w * x1[j].w)));
        part[i][j] += s0 + s1;
      }
    }
    if ((slice & 3) == 3) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < R; ++j) {
          acc[i][j] += (double)part[i][j];
          part[i][j] = 0.f;
        }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
#pragma unroll
    for (int j = 0; j < R; ++j) {
      double t = acc[i][j] + (double)part[i][j];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
      if (lane == 0 && j < r && row0 + i < n) y[((long long)b * vstride + j) * n + row0 + i] = (float)t;
    }
  }
}

// Sum over the block of one double per thread; every thread gets the total.  256 threads.
__device__ __forceinline__ double block_sum(double x, double* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  __syncthreads();  // the previous total has been read by everyone
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = x;
  __syncthreads();
  double t = 0.0;
#pragma unroll
  for (int w = 0; w < 8; ++w) t += red[w];
  return t;
}
__device__ __forceinline__ double block_dot(const float* x, const float* y, int n, double* red) {
  double s = 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += (double)x[i] * (double)y[i];
  return block_sum(s, red);
}

// Sums over the block of K doubles per thread (256 threads): out[i] holds the total of acc[i] afterwards (shared
// memory, valid for every thread after the call).  `part` is 8 * K doubles of shared scratch.
template <int K>
__device__ __forceinline__ void block_sum_many(double (&acc)[K], double* part, double* out) {
#pragma unroll
  for (int i = 0; i < K; ++i) {
    double x = acc[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    acc[i] = x;
  }
  __syncthreads();  // earlier readers of part / out are done
  if ((threadIdx.x & 31) == 0) {
#pragma unroll
    for (int i = 0; i < K; ++i) part[(threadIdx.x >> 5) * K + i] = acc[i];
  }
  __syncthreads();
  if (threadIdx.x < K) {
    double t = 0.0;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += part[w * K + threadIdx.x];
    out[threadIdx.x] = t;
  }
  __syncthreads();
}

constexpr int kPairs = kMaxDeflate * (kMaxDeflate + 1) / 2;  // entries of a symmetric r x r matrix, r = 8
__device__ __forceinline__ int pair_index(int i, int j) { return i * (i + 1) / 2 + j; }  // j <= i

// Cholesky-QR of the r vectors held in Y (r x n, vector-major): G = Y Y^T = L L^T (FP64, one thread), V = L^-1 Y.
// `gram` holds G's lower triangle (pair_index order) on entry.  A vector that is (numerically) a combination of the
// earlier ones comes out as zero; its slot is seeded afresh by the next call.
__device__ void cholesky_orthonormalise(const float* Y, float* V, int n, int r, const double* gram, double (*L)[kMaxDeflate]) {
  if (threadIdx.x == 0) {
    for (int i = 0; i < r; ++i) {
      for (int j = 0; j <= i; ++j) {
        double sum = gram[pair_index(i, j)];
        for (int k = 0; k < j; ++k) sum -= L[i][k] * L[j][k];
        if (i == j) {
          L[i][i] = (sum > 1e-24 * gram[pair_index(i, i)] && sum > 0.0) ? sqrt(sum) : 0.0;
        } else {
          L[i][j] = L[j][j] > 0.0 ? sum / L[j][j] : 0.0;
        }
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    double out[kMaxDeflate];
#pragma unroll
    for (int j = 0; j < kMaxDeflate; ++j) {
      if (j < r) {
        double sum = (double)Y[(long long)j * n + c];
#pragma unroll
        for (int i = 0; i < kMaxDeflate; ++i)
          if (i < j) sum -= L[j][i] * out[i];
        out[j] = L[j][j] > 0.0 ? sum / L[j][j] : 0.0;
      } else {
        out[j] = 0.0;
      }
    }
#pragma unroll
    for (int j = 0; j < kMaxDeflate; ++j)
      if (j < r) V[(long long)j * n + c] = (float)out[j];
  }
  __syncthreads();
}

// start vectors: the caller's vectors (warm), or r different fixed +-1 patterns (cold, and for a slot that holds
// nothing yet because the rank grew since the last call), orthonormalised
__global__ void __launch_bounds__(256) block_start_kernel(float* __restrict__ v, int n, int r, int vstride, int cold) {
  __shared__ double red[8];
  __shared__ double part[8 * kPairs], gram[kPairs];
  __shared__ double L[kMaxDeflate][kMaxDeflate];
  const int b = blockIdx.x;
  float* V = v + (long long)b * vstride * n;
  const float s = rsqrtf((float)n);
  for (int j = 0; j < r; ++j) {
    float* vj = V + (long long)j * n;
    const bool seed = cold || !(block_dot(vj, vj, n, red) > 0.0);
    if (seed)
      for (int c = threadIdx.x; c < n; c += blockDim.x)
        vj[c] = ((((unsigned)c + 977u * (unsigned)j) * 2654435761u) >> (15 + (j & 7))) & 1u ? s : -s;
    __syncthreads();
  }
  double acc[kPairs];
#pragma unroll
  for (int i = 0; i < kPairs; ++i) acc[i] = 0.0;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    double x[kMaxDeflate];
#pragma unroll
    for (int i = 0; i < kMaxDeflate; ++i) x[i] = i < r ? (double)V[(long long)i * n + c] : 0.0;
#pragma unroll
    for (int i = 0; i < kMaxDeflate; ++i)
#pragma unroll
      for (int j = 0; j <= i; ++j) acc[i * (i + 1) / 2 + j] += x[i] * x[j];
  }
  block_sum_many<kPairs>(acc, part, gram);
  cholesky_orthonormalise(V, V, n, r, gram, L);
}

// Rayleigh-Ritz on span(V) with Y = A V (V orthonormal): H = V Y^T, H = Q diag(theta) Q^T (Jacobi, FP64, one thread),
// V <- Q^T V, Y <- Q^T Y (Ritz vectors, descending theta), res_j = ||Y_j - theta_j V_j|| / |theta_j|.  Unless this is
// the last sweep, V is then replaced by the orthonormalised Y (one more step of the power iteration).  Three passes
// over the two blocks of vectors; every reduction is taken for all pairs at once.
__global__ void __launch_bounds__(256) ritz_kernel(float* __restrict__ v, float* __restrict__ y, int n, int r, int vstride,
                                                   int last, float* __restrict__ theta, float* __restrict__ res) {
  constexpr int R = kMaxDeflate;
  __shared__ double part[8 * R * R], sums[R * R];
  __shared__ double H[R][R], Q[R][R], lam[R], L[R][R];
  const int b = blockIdx.x;
  float* V = v + (long long)b * vstride * n;
  float* Y = y + (long long)b * vstride * n;
  {
    double acc[R * R];
#pragma unroll
    for (int i = 0; i < R * R; ++i) acc[i] = 0.0;
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
      double vv[R], yy[R];
#pragma unroll
      for (int i = 0; i < R; ++i) {
        vv[i] = i < r ? (double)V[(long long)i * n + c] : 0.0;
        yy[i] = i < r ? (double)Y[(long long)i * n + c] : 0.0;
      }
#pragma unroll
      for (int i = 0; i < R; ++i)
#pragma unroll
        for (int j = 0; j < R; ++j) acc[i * R + j] += vv[i] * yy[j];
    }
    block_sum_many<R * R>(acc, part, sums);
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < r; ++i)
      for (int j = 0; j < r; ++j) {
        H[i][j] = 0.5 * (sums[i * R + j] + sums[j * R + i]);
        Q[i][j] = i == j ? 1.0 : 0.0;
      }
    for (int sweep = 0; sweep < 12; ++sweep) {
      double off = 0.0;
      for (int pp = 0; pp < r; ++pp)
        for (int qq = pp + 1; qq < r; ++qq) off += H[pp][qq] * H[pp][qq];
      double diag = 0.0;
      for (int pp = 0; pp < r; ++pp) diag += H[pp][pp] * H[pp][pp];
      if (!(off > 1e-30 * diag)) break;   // off-diagonal part below FP64 rounding of the diagonal: converged
      for (int pp = 0; pp < r; ++pp)
        for (int qq = pp + 1; qq < r; ++qq) {
          const double apq = H[pp][qq];
          if (apq == 0.0) continue;
          const double tau = (H[qq][qq] - H[pp][pp]) / (2.0 * apq);
          const double t = (tau >= 0.0 ? 1.0 : -1.0) / (fabs(tau) + sqrt(1.0 + tau * tau));
          const double cs = 1.0 / sqrt(1.0 + t * t), sn = t * cs;
          for (int k = 0; k < r; ++k) {  // columns pp, qq of H and Q
            const double hp = H[k][pp], hq = H[k][qq];
            H[k][pp] = cs * hp - sn * hq;
            H[k][qq] = sn * hp + cs * hq;
            const double qp = Q[k][pp], qv = Q[k][qq];
            Q[k][pp] = cs * qp - sn * qv;
            Q[k][qq] = sn * qp + cs * qv;
          }
          for (int k = 0; k < r; ++k) {  // rows pp, qq of H
            const double hp = H[pp][k], hq = H[qq][k];
            H[pp][k] = cs * hp - sn * hq;
            H[qq][k] = sn * hp + cs * hq;
          }
        }
    }
    for (int i = 0; i < r; ++i) lam[i] = H[i][i];
    for (int i = 0; i < r; ++i) {  // selection sort, descending, columns of Q follow
      int best = i;
      for (int j = i + 1; j < r; ++j)
        if (lam[j] > lam[best]) best = j;
      if (best != i) {
        const double t = lam[i]; lam[i] = lam[best]; lam[best] = t;
        for (int k = 0; k < r; ++k) {
          const double q = Q[k][i]; Q[k][i] = Q[k][best]; Q[k][best] = q;
        }
      }
    }
  }
  __syncthreads();
  {
    // rotate both blocks (new vector j = sum_i Q[i][j] old vector i); on the way: the squared residuals and the Gram
    // matrix of the rotated Y (for its orthonormalisation)
    double acc[kPairs + R];
#pragma unroll
    for (int i = 0; i < kPairs + R; ++i) acc[i] = 0.0;
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
      double vv[R], yy[R], nv[R], ny[R];
#pragma unroll
      for (int i = 0; i < R; ++i) {
        vv[i] = i < r ? (double)V[(long long)i * n + c] : 0.0;
        yy[i] = i < r ? (double)Y[(long long)i * n + c] : 0.0;
      }
#pragma unroll
      for (int j = 0; j < R; ++j) {
        double sv = 0.0, sy = 0.0;
        if (j < r) {
#pragma unroll
          for (int i = 0; i < R; ++i) {
            if (i < r) {
              sv += Q[i][j] * vv[i];
              sy += Q[i][j] * yy[i];
            }
          }
          // what is stored is what later passes read: round before the sums
          const float fv = (float)sv, fy = (float)sy;
          V[(long long)j * n + c] = fv;
          Y[(long long)j * n + c] = fy;
          sv = fv;
          sy = fy;
        }
        nv[j] = sv;
        ny[j] = sy;
      }
#pragma unroll
      for (int i = 0; i < R; ++i) {
#pragma unroll
        for (int j = 0; j <= i; ++j) acc[i * (i + 1) / 2 + j] += ny[i] * ny[j];
        const double d = i < r ? ny[i] - lam[i] * nv[i] : 0.0;
        acc[kPairs + i] += d * d;
      }
    }
    block_sum_many<kPairs + R>(acc, part, sums);
  }
  if (threadIdx.x < r) {
    const double l = lam[threadIdx.x];
    theta[b * R + threadIdx.x] = (float)l;
    res[b * R + threadIdx.x] = l > 0.0 ? (float)(sqrt(sums[kPairs + threadIdx.x]) / l) : INFINITY;
  }
  if (!last) cholesky_orthonormalise(Y, V, n, r, sums, L);
}

// Which of the r Ritz pairs are deflated: in descending order, as long as each has converged and stands above eight
// times the mean c of everything that would remain; all accepted directions are moved to that common c.
//   coef[b][j] = -(theta_j - c)  (0 where not deflated)      corr[b][j] = theta_j^(-1/p) - c^(-1/p)
// rest_top[b] / rest_idx[b]: the largest Ritz value that stays in A' and its vector's index (0 / -1 when every vector of
// the block was deflated: nothing is known about the remainder then).
__global__ void block_decide_kernel(const float* __restrict__ theta, const float* __restrict__ res, int k, int n, int r,
                                    float damping, int p, float* __restrict__ coef, float* __restrict__ corr,
                                    int* __restrict__ count, float* __restrict__ rest_top, int* __restrict__ rest_idx,
                                    float* __restrict__ rest_trace) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= k) return;
  const double tr = (double)n * (1.0 + (double)damping);  // A has unit mean diagonal plus the damping
  double sum = 0.0;
  int m = 0;
  for (int j = 0; j < r && n - (j + 1) > 0; ++j) {
    const double t = theta[b * kMaxDeflate + j];
    const double e = res[b * kMaxDeflate + j];
    const double c = (tr - sum - t) / (double)(n - (m + 1));
    if (!(isfinite(t) && isfinite(e) && e < 1e-5 && c > 0.0 && t > 8.0 * c)) break;
    sum += t;
    ++m;
  }
  const double c = (tr - sum) / (double)(n - m);
  for (int j = 0; j < kMaxDeflate; ++j) {
    const bool on = j < m;
    const double t = on ? (double)theta[b * kMaxDeflate + j] : 0.0;
    coef[b * kMaxDeflate + j] = on ? (float)-(t - c) : 0.f;
    corr[b * kMaxDeflate + j] = on ? (float)(pow(t, -1.0 / p) - pow(c, -1.0 / p)) : 0.f;
  }
  // also reported (bits 8..15): how many Ritz values stand above 8x the rest whether converged or not -- directions
  // that look like outliers; a caller that iterates fewer vectors than there are of those widens its block
  int cand = 0;
  for (int j = 0; j < r; ++j)
    if ((double)theta[b * kMaxDeflate + j] > 8.0 * c) ++cand;
  if (count) count[b] = m | (cand << 8);
  const float rest = m < r ? theta[b * kMaxDeflate + m] : 0.f;
  const bool known = m < r && isfinite(rest) && rest > 0.f;
  rest_top[b] = known ? rest : 0.f;
  rest_idx[b] = known ? m : -1;
  rest_trace[b] = (float)(c * (double)n);   // trace of A' (every deflated direction moved to c): above its Frobenius norm
}

// An ESTIMATE of lambda_max(A') in place of the certified bound: kRitzGrow times the largest Ritz value that was not
// deflated, never above the trace of A' (which bounds its Frobenius norm).  A Rayleigh quotient errs low, and at the dense upper
// edge of an activation statistic's bulk it stays low however long the block has followed the statistic: 17-20 % on
// the benchmark's statistics (Marchenko-Pastur edges 1.36 and 1.63, Ritz values 1.08 and 1.30).  The factor leaves
// ten percent above that.  Three squarings give n^(1/16) = 1.7 times lambda_max for a flat spectrum and cost three
// passes; what the estimate risks -- eigenvalues of M_0 above 1, which the first Newton step sends BELOW the new lower
// bound -- is looked for after the chain (see the verification).
constexpr float kRitzGrow = 1.4f;
__global__ void ritz_norm_kernel(float* __restrict__ bound2, const float* __restrict__ rest_top,
                                 const float* __restrict__ rest_trace, int k) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= k) return;
  const float cap = rest_trace[b];      // ||A'||_F <= trace(A') for a positive matrix: costs no pass over A'
  const float t = kRitzGrow * rest_top[b];
  bound2[b] = (t > 0.f && t < cap) ? t * t : cap * cap;
}

// v2[b] = the Ritz vector rest_idx[b] of statistic b (zero where there is none)
// out[b][0] = first[b] (the tracked direction), out[b][1] = the Ritz vector rest_idx[b] of statistic b (zero where there
// is none): the two starting vectors of the verification, side by side for the two-vector pass over M
__global__ void __launch_bounds__(256) pick_vector_kernel(const float* __restrict__ first, const float* __restrict__ v,
                                                          const int* __restrict__ idx, float* __restrict__ out, int n,
                                                          int vstride) {
  const int b = blockIdx.y;
  const int j = idx[b];
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
    out[((long long)b * 2) * n + i] = first[(long long)b * n + i];
    out[((long long)b * 2 + 1) * n + i] = j >= 0 ? v[((long long)b * vstride + j) * n + i] : 0.f;
  }
}

// A_b += sum_j coef[b][j] v_bj v_bj^T  (terms with a zero coefficient are skipped; exact symmetry is kept: the
// product v_r v_c has the same bits at (r, c) and (c, r) and the terms are added in the same order)
__global__ void __launch_bounds__(256) rankr_update_kernel(float* __restrict__ a, const float* __restrict__ v,
                                                           const float* __restrict__ coef, int n, int r, int vstride) {
  const int b = blockIdx.y;
  float cf[kMaxDeflate];
  bool any = false;
#pragma unroll
  for (int j = 0; j < kMaxDeflate; ++j) {
    cf[j] = j < r ? coef[b * kMaxDeflate + j] : 0.f;
    any = any || cf[j] != 0.f;
  }
  if (!any) return;
  float* A = a + (long long)b * n * n;
  const float* V = v + (long long)b * vstride * n;
  const int n4 = n / 4;
  const long long total = (long long)n * n4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(i / n4), c = (int)(i - (long long)row * n4) * 4;
    float4 x = *reinterpret_cast<float4*>(A + (long long)row * n + c);
#pragma unroll
    for (int j = 0; j < kMaxDeflate; ++j) {
      if (cf[j] != 0.f) {
        const float vr = V[(long long)j * n + row];
        const float4 vc = *reinterpret_cast<const float4*>(V + (long long)j * n + c);
        x.x = fmaf(cf[j], vr * vc.x, x.x); x.y = fmaf(cf[j], vr * vc.y, x.y);
        x.z = fmaf(cf[j], vr * vc.z, x.z); x.w = fmaf(cf[j], vr * vc.w, x.w);
      }
    }
    *reinterpret_cast<float4*>(A + (long long)row * n + c) = x;
  }
}

// With P = A' / ||A'||_F:  lambda_max(P) <= ||P^(2^j)||_F^(1 / 2^j) = (sum lambda^(2^(j+1)))^(1 / 2^(j+1))  for every j, and
// the bound tightens with j (for a flat spectrum it is n^(-1/2) times n^(1/4), n^(1/8), n^(1/16) for j = 1, 2, 3).
// bound^2 <- bound^2 * t^2 with t the smallest of the three, 3 % above it for the single-pass products' rounding.
__global__ void tighten_bound_kernel(float* __restrict__ bound2, const float* __restrict__ ss2, const float* __restrict__ ss4,
                                     const float* __restrict__ ss8, int k) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= k) return;
  float t = 1.f;
  const float t2 = powf(fmaxf(ss2[b], 0.f), 0.25f);
  if (isfinite(t2) && t2 > 0.f) t = fminf(t, 1.03f * t2);
  if (ss4) {
    const float t4 = powf(fmaxf(ss4[b], 0.f), 0.125f);
    if (isfinite(t4) && t4 > 0.f) t = fminf(t, 1.03f * t4);
  }
  if (ss8) {
    const float t8 = powf(fmaxf(ss8[b], 0.f), 0.0625f);
    if (isfinite(t8) && t8 > 0.f) t = fminf(t, 1.03f * t8);
  }
  if (t < 1.f) bound2[b] *= t * t;
}

// v <- (v - y) / ||v - y||  with y = M v:  one power-iteration step on R = I - M;  e[b] = the Rayleigh quotient of R at
// the incoming v, 1 - v.y / v.v (0 where v is zero: nothing is known).
// Vector j = blockIdx.y of statistic b sits at (b * vs + j) * n; its quotient goes to e[j * e_stride + b].
__global__ void __launch_bounds__(256) power_shift_kernel(float* __restrict__ v, const float* __restrict__ y, int n,
                                                          float* __restrict__ e, int vs = 1, long long e_stride = 0) {
  const int b = blockIdx.x;
  float* V = v + ((long long)b * vs + blockIdx.y) * n;
  const float* Y = y + ((long long)b * vs + blockIdx.y) * n;
  e += (long long)blockIdx.y * e_stride;
  __shared__ double red[3][8];
  __shared__ double tot[3];
  double vy = 0.0, vv = 0.0, tt = 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const double yi = Y[i], vi = V[i], d = vi - yi;
    vy += vi * yi;
    vv += vi * vi;
    tt += d * d;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    vy += __shfl_xor_sync(0xffffffffu, vy, o);
    vv += __shfl_xor_sync(0xffffffffu, vv, o);
    tt += __shfl_xor_sync(0xffffffffu, tt, o);
  }
  if ((threadIdx.x & 31) == 0) {
    red[0][threadIdx.x >> 5] = vy;
    red[1][threadIdx.x >> 5] = vv;
    red[2][threadIdx.x >> 5] = tt;
  }
  __syncthreads();
  if (threadIdx.x < 3) {
    double t = 0.0;
    for (int w = 0; w < 8; ++w) t += red[threadIdx.x][w];
    tot[threadIdx.x] = t;
  }
  __syncthreads();
  const double inv = tot[2] > 0.0 ? 1.0 / sqrt(tot[2]) : 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) V[i] = (float)(((double)V[i] - (double)Y[i]) * inv);
  if (threadIdx.x == 0) e[b] = tot[1] > 0.0 ? (float)(1.0 - tot[0] / tot[1]) : 0.f;
}

// status 4 where the distance of the last M from the identity, estimated by power iteration on I - M, exceeds what the
// schedule was built for: the caller's estimate of the spectrum's lower end was too high for this statistic.
__global__ void verify_kernel(const float* __restrict__ e_est, const float* __restrict__ e_top, float e_allowed,
                              int* __restrict__ status, float* __restrict__ e_out, int k) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= k) return;
  float e = e_est[b];
  if (e_top) e = isfinite(e_top[b]) ? fmaxf(e, e_top[b]) : e_top[b];
  if (e_out) e_out[b] = e;
  if (status && status[b] == 0 && (!isfinite(e) || e > e_allowed)) status[b] = 4;
}

// lmin[b] = theta^(-power): the smallest eigenvalue of A from the largest eigenvalue theta (a Rayleigh quotient, so a
// lower estimate) of its computed inverse root A^(-1/power).
__global__ void lmin_from_root_kernel(const float* __restrict__ theta, float power, float* __restrict__ lmin, int k) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= k) return;
  const float t = theta[b];
  lmin[b] = (isfinite(t) && t > 0.f) ? powf(t, -power) : 0.f;
}

// Per statistic: the scale that turns M_0^{-1/p} into A^{-1/p}, and the convergence status from the
// distance max|I - M| gathered when the last M was produced (0 converged, 1 above tol, 2 non-finite).
// 3: the statistic's spectrum reaches below the lower bound the schedule was built for (caller's bound too high).
// Also the bound of the finished root's entries for its operand planes: a symmetric positive matrix has no entry above
// its largest eigenvalue, and A >= damping I by construction, so |A^(-1/p)|_ij <= damping^(-1/p) -- known without a
// pass over the result.
__global__ void finish_kernel(const unsigned int* __restrict__ resid, const float* __restrict__ sumsq_a,
                              float* root_scale_lo, int* status, float* norm_out, int k, int p, float tol, float damping,
                              float lower_used, unsigned int* __restrict__ root_max_bits, float root_bound) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= k) return;
  root_max_bits[b] = __float_as_uint(root_bound);
  const float ub = sqrtf(fmaxf(sumsq_a[b], 1e-60f));
  root_scale_lo[b] = powf(ub, -1.f / p);
  if (norm_out) norm_out[b] = ub;
  const float r = __uint_as_float(resid[b]);
  int st = !isfinite(r) ? 2 : (r > tol ? 1 : 0);
  // lower_used < 0: the bound is an estimate, verified after the chain instead (verify_kernel)
  if (st == 0 && lower_used > 0.f && damping / ub < lower_used * 0.999f) st = 3;
  if (status) status[b] = st;
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static size_t per_statistic_bytes(int n) {
  // A (FP32) + seven FP16 hi/lo plane pairs (T, M x2, X x2, two powers of T) = 8 FP32-sized matrices
  return align_up((size_t)n * n * 4, 256) * 8;
}
static size_t small_bytes(int chunk, int n) {
  // twenty per-statistic scalars, four blocks of eight scalars per statistic (Ritz values, residuals, deflation
  // coefficients, root corrections), the reduction scratch, and two blocks of eight n-vectors per statistic
  // (block power iteration: V and A V)
  return align_up((size_t)chunk * 4, 256) * 20 + 4 * align_up((size_t)chunk * 32, 256) +
         align_up(sumsq_scratch_bytes(chunk), 256) + 2 * align_up((size_t)chunk * 8 * n * 4, 256);
}

// Largest power of two s with s * bound <= 2^14: FP16 planes of s * x then stay a factor four below overflow
// for |x| <= bound, and elements down to 2^-16 of the bound keep all 22 bits of the hi/lo pair.
static float plane_scale(double bound) {
  return (float)std::ldexp(1.0, (int)std::floor(std::log2(16384.0 / bound)));
}

}  // namespace toner

extern "C" {

size_t toner_inv_roots_workspace_bytes(int32_t chunk, int32_t n) {
  if (chunk <= 0 || n <= 0) return 0;
  return toner::per_statistic_bytes(n) * (size_t)chunk + toner::small_bytes(chunk, n);
}

int toner_inv_roots_iterations(int32_t n, float damping, int32_t p) {
  if (n <= 0 || !(damping > 0) || p < 1) return 0;
  return toner::default_iterations((double)damping / ((double)n * (1.0 + damping)), p);
}

int toner_inv_roots_iterations_for(float lower, int32_t p) {
  if (!(lower > 0.f) || !(lower < 1.f) || p < 1) return 0;
  return toner::default_iterations((double)lower, p);
}

int toner_inv_roots_finish_order_for(float lower, int32_t p, int32_t iters) {
  if (!(lower > 0.f) || !(lower < 1.f) || p < 1) return 0;
  if (iters <= 0) iters = toner::default_iterations((double)lower, p);
  if (iters < 2) return 0;
  double l_last;
  toner::newton_schedule((double)lower, p, iters - 1, &l_last);
  return toner::finish_order(p, 1.0 - l_last);
}

int toner_inv_roots_schedule(float lower, int32_t p, int32_t iters, double* ab_out, int32_t ab_capacity, double* coef_out,
                             int32_t coef_capacity, int32_t* order_out, double* e_out) {
  if (!(lower > 0.f) || !(lower < 1.f) || p < 1) return 0;
  if (iters <= 0) iters = toner::default_iterations((double)lower, p);
  if (iters < 2) return 0;
  const std::vector<toner::NewtonStep> sched = toner::newton_schedule((double)lower, p, iters, nullptr);
  double l_last;
  toner::newton_schedule((double)lower, p, iters - 1, &l_last);
  const toner::FinishPoly fin = toner::finish_poly_or_best(p, 1.0 - l_last);
  if (ab_out) {
    for (int k = 0; k < iters - 1 && 2 * k + 1 < ab_capacity; ++k) {
      ab_out[2 * k] = sched[k].a;
      ab_out[2 * k + 1] = sched[k].b;
    }
  }
  if (coef_out)
    for (int j = 0; j <= fin.order && j < coef_capacity; ++j) coef_out[j] = fin.c[j];
  if (order_out) *order_out = fin.order;
  if (e_out) *e_out = 1.0 - l_last;
  return iters;
}

int toner_inv_roots(const float* ema, int32_t k, int32_t n, float damping, int32_t p, int32_t q, int32_t iters,
                    float* root_lo, float* root_hi, float* fro2_lo, int32_t* status, void* workspace,
                    size_t workspace_bytes, void* stream_) {
  return toner_inv_roots_ex(ema, k, n, damping, p, q, iters, 0.f, root_lo, root_hi, fro2_lo, status, nullptr, workspace,
                            workspace_bytes, stream_);
}

int toner_inv_roots_ex(const float* ema, int32_t k, int32_t n, float damping, int32_t p, int32_t q, int32_t iters,
                       float lower, float* root_lo, float* root_hi, float* fro2_lo, int32_t* status, float* norm_out,
                       void* workspace, size_t workspace_bytes, void* stream_) {
  return toner_inv_roots_tracked(ema, k, n, damping, p, q, iters, lower, 0, root_lo, root_hi, fro2_lo, status, norm_out,
                                 nullptr, nullptr, nullptr, 0, nullptr, 0, nullptr, workspace, workspace_bytes, stream_);
}

int toner_inv_roots_tracked(const float* ema, int32_t k, int32_t n, float damping, int32_t p, int32_t q, int32_t iters,
                            float lower, int32_t lower_is_estimate, float* root_lo, float* root_hi, float* fro2_lo,
                            int32_t* status, float* norm_out, float* track, float* lmin_out, float* resid_out,
                            int32_t track_sweeps, float* deflate, int32_t deflate_rank, int32_t* deflated_out,
                            void* workspace, size_t workspace_bytes, void* stream_) {
  using namespace toner;
  Context* ctx = context();
  if (!ctx) return kErrCuda;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!ema || !root_lo || !workspace) return fail(kErrArg, "inv_roots: null pointer");
  if (k <= 0 || n <= 0) return fail(kErrArg, "inv_roots: sizes must be positive");
  if (n % 8 != 0) return fail(kErrUnsupported, "inv_roots: n must be a multiple of 8");
  if (!(damping > 0.f)) return fail(kErrArg, "inv_roots: damping must be positive");
  if (p < 1 || p > 32 || (p & (p - 1))) return fail(kErrUnsupported, "inv_roots: root order p must be a power of two <= 32");
  if (q < 1 || q > p || (q & (q - 1))) return fail(kErrUnsupported, "inv_roots: q must be a power of two <= p");
  if (q > 1 && !root_hi) return fail(kErrArg, "inv_roots: root_hi is required when q > 1");
  // Lower bound of the normalised spectrum the schedule is built for: the caller's (checked per statistic, status 3
  // where it does not hold), else the bound that holds for every statistic, damping / (n (1 + damping)).
  const double l_worst = (double)damping / ((double)n * (1.0 + damping));
  if (lower != 0.f && !(lower > 0.f && lower < 1.f)) return fail(kErrArg, "inv_roots: lower must be 0 or inside (0, 1)");
  const double l0 = (lower > 0.f && (double)lower > l_worst) ? (double)lower : l_worst;
  const bool estimated = lower_is_estimate != 0 && l0 > l_worst;
  if (estimated && !track) return fail(kErrArg, "inv_roots: an estimated bound needs the tracking vectors to verify it");
  if (track_sweeps < 0 || (track_sweeps & ~(63 | 256))) return fail(kErrArg, "inv_roots: track_sweeps is 0..63, plus 256 to start afresh");
  const int defl_r = deflate ? (deflate_rank & 15) : 0;      // directions the block iteration looks for (0: one, the old way)
  const bool defl_cold = deflate && (deflate_rank & 256);
  const bool ritz_norm = deflate && (deflate_rank & 512);   // norm from the block iteration instead of three squarings
  if (deflate && (defl_r < 1 || defl_r > kMaxDeflate || (deflate_rank & ~(15 | 256 | 512))))
    return fail(kErrArg, "inv_roots: deflate_rank is 1..8, plus 256 to start from fixed vectors, plus 512 to take the "
                         "norm from the block iteration");
  if (ritz_norm && (defl_cold || !estimated))
    return fail(kErrArg, "inv_roots: the norm estimate needs vectors from an earlier call and an estimated lower bound "
                         "(both are verified together after the chain)");
  // > 0: certified bound, checked against damping / norm per statistic; < 0: estimate, verified after the chain
  const float lower_used = l0 > l_worst ? (estimated ? -(float)l0 : (float)l0) : 0.f;
  if (iters <= 0) iters = default_iterations(l0, p);
  if (iters < 2) return fail(kErrArg, "inv_roots: at least two iterations are required");
  const std::vector<NewtonStep> sched = newton_schedule(l0, p, iters, nullptr);
  double l_last;  // lower bound of the spectrum of the last M, i.e. after iters - 1 updates
  newton_schedule(l0, p, iters - 1, &l_last);
  const FinishPoly fin = finish_poly_or_best(p, 1.0 - l_last);
  const int order = fin.order;
  int log2p = 0;
  while ((1 << log2p) < p) ++log2p;

  const size_t per = per_statistic_bytes(n);
  long long chunk_cap = 0;
  for (long long c = k; c >= 1; --c) {
    if (per * (size_t)c + small_bytes((int)c, n) <= workspace_bytes) {
      chunk_cap = c;
      break;
    }
  }
  if (chunk_cap < 1) return fail(kErrWorkspace, "inv_roots: workspace holds less than one statistic");
  const long long nn = (long long)n * n;
  const size_t mat = align_up((size_t)nn * 4, 256);
  const int ew_blocks = (int)std::min<long long>((nn / 4 + 255) / 256, 8LL * ctx->num_sms / (k < 8 ? k : 8) + 1);

  // Plane scales from norm bounds known in advance (no pass over the data is needed to find them):
  // ||M_k|| <= 1, ||T_k|| <= a_k, ||T_k^(2^j)|| <= a_k^(2^j), ||X_k|| <= min(prod_{j<k} a_j, l0^(-1/p)),
  // ||A^(-1/p)|| <= damping^(-1/p).
  const float s_m = plane_scale(1.0);
  const double x_cap = 1.01 * std::pow(l0, -1.0 / p);
  const double root_bound = 1.01 * std::pow((double)damping, -1.0 / p);

  for (int k0 = 0; k0 < k; k0 += (int)chunk_cap) {
    const int kc = (int)std::min<long long>(chunk_cap, k - k0);
    char* w = static_cast<char*>(workspace);
    float* A32 = reinterpret_cast<float*>(w); w += mat * kc;
    __half* Tb[2];
    __half* Mb[2];
    __half* Xb[2];
    __half* Pb[2];
    Tb[0] = reinterpret_cast<__half*>(w); w += mat * kc;
    Mb[0] = reinterpret_cast<__half*>(w); w += mat * kc;
    Mb[1] = reinterpret_cast<__half*>(w); w += mat * kc;
    Xb[0] = reinterpret_cast<__half*>(w); w += mat * kc;
    Xb[1] = reinterpret_cast<__half*>(w); w += mat * kc;
    Pb[0] = reinterpret_cast<__half*>(w); w += mat * kc;
    Pb[1] = reinterpret_cast<__half*>(w); w += mat * kc;
    Tb[1] = Pb[0];  // p == 1 has no powers of T to store: the next T is written beside the current one
    const size_t sm = align_up((size_t)kc * 4, 256);
    auto small = [&](int i) { return reinterpret_cast<float*>(w + sm * i); };
    float* trace = small(0);
    float* sumsq_a = small(1);
    unsigned int* resid = reinterpret_cast<unsigned int*>(small(2));
    float* scale_lo = small(3);
    float* fro_tmp = small(4);
    float* lam = small(5);
    float* pres = small(6);
    float* neg_sigma = small(7);
    float* corr = small(8);
    float* inv_r = small(9);
    unsigned int* max_r = reinterpret_cast<unsigned int*>(small(10));
    float* ss2 = small(11);
    float* ss4 = small(12);
    float* ss8 = small(13);
    float* e_est = small(14);
    float* theta = small(15);
    float* rest_top = small(16);
    int* rest_idx = reinterpret_cast<int*>(small(17));
    float* e_top = small(18);
    float* rest_trace = small(19);
    const size_t sm8 = align_up((size_t)kc * 32, 256);
    char* wp = w + sm * 20;
    float* th8 = reinterpret_cast<float*>(wp); wp += sm8;     // Ritz values, residuals, deflation coefficients and
    float* res8 = reinterpret_cast<float*>(wp); wp += sm8;    // root corrections of the block deflation: eight per statistic
    float* coef8 = reinterpret_cast<float*>(wp); wp += sm8;
    float* corr8 = reinterpret_cast<float*>(wp); wp += sm8;
    float* partials = reinterpret_cast<float*>(wp); wp += align_up(sumsq_scratch_bytes(kc), 256);
    const size_t vec = align_up((size_t)kc * 8 * n * 4, 256);
    float* pv = reinterpret_cast<float*>(wp);
    float* py = reinterpret_cast<float*>(wp + vec);
    float* dv = deflate ? deflate + (long long)k0 * kMaxDeflate * n : nullptr;
    TONER_CUDA(cudaMemsetAsync(w, 0, sm * 20 + 4 * sm8, stream));

    const float* C = ema + (long long)k0 * nn;
    const int t32 = (n + 31) / 32;
    trace_kernel<<<kc, 256, 0, stream>>>(C, n, trace);
    count_launch();
    damp_kernel<<<dim3(t32, t32, kc), 256, 0, stream>>>(C, A32, n, damping, trace);
    count_launch();
    if (defl_r > 0) {
      // dominant directions: block power iteration with Rayleigh-Ritz on the caller's vectors (eight sweeps from fixed
      // vectors -- the first three or four only find the subspace --, four from last call's), then deflate those that
      // converged and stand above the rest
      block_start_kernel<<<kc, 256, 0, stream>>>(dv, n, defl_r, kMaxDeflate, defl_cold ? 1 : 0);
      count_launch();
      const int sweeps = defl_cold ? 8 : 4;
      for (int sw = 0; sw < sweeps; ++sw) {
        const dim3 bg((n + kBlockGemvRows - 1) / kBlockGemvRows, kc);
        if (defl_r <= 2) block_gemv_kernel<2><<<bg, 256, 0, stream>>>(A32, dv, py, n, defl_r, kMaxDeflate);
        else if (defl_r <= 4) block_gemv_kernel<4><<<bg, 256, 0, stream>>>(A32, dv, py, n, defl_r, kMaxDeflate);
        else if (defl_r <= 6) block_gemv_kernel<6><<<bg, 256, 0, stream>>>(A32, dv, py, n, defl_r, kMaxDeflate);
        else block_gemv_kernel<8><<<bg, 256, 0, stream>>>(A32, dv, py, n, defl_r, kMaxDeflate);
        count_launch();
        ritz_kernel<<<kc, 256, 0, stream>>>(dv, py, n, defl_r, kMaxDeflate, sw == sweeps - 1 ? 1 : 0, th8, res8);
        count_launch();
      }
      block_decide_kernel<<<(kc + 127) / 128, 128, 0, stream>>>(th8, res8, kc, n, defl_r, damping, p, coef8, corr8,
                                                               deflated_out ? deflated_out + k0 : nullptr, rest_top, rest_idx,
                                                               rest_trace);
      count_launch();
      if (!ritz_norm) {   // (with the norm estimate the deflation is applied where the operand planes are formed)
        rankr_update_kernel<<<dim3(ew_blocks, kc), 256, 0, stream>>>(A32, dv, coef8, n, defl_r, kMaxDeflate);
        count_launch();
      }
    } else {
      // dominant direction: six power-iteration steps, then deflate where they converged
      power_start_kernel<<<dim3(8, kc), 256, 0, stream>>>(pv, n);
      count_launch();
      for (int pi = 0; pi < kPowerSteps; ++pi) {
        gemv_kernel<<<dim3((n + 7) / 8, kc), 256, 0, stream>>>(A32, pv, py, n);
        count_launch();
        power_norm_kernel<<<kc, 256, 0, stream>>>(pv, py, n, lam, pres);
        count_launch();
      }
      deflate_decide_kernel<<<(kc + 127) / 128, 128, 0, stream>>>(lam, pres, kc, n, damping, p, neg_sigma, corr);
      count_launch();
      rank1_update_kernel<<<dim3(ew_blocks, kc), 256, 0, stream>>>(A32, pv, neg_sigma, n);
      count_launch();
    }
    TONER_CUDA(cudaGetLastError());
    if (!ritz_norm) {
      int rc0 = sumsq_det(A32, kc, n, n, n, nn, partials, sumsq_a, stream);
      if (rc0) return rc0;
    }
    float s_t = plane_scale(sched[0].a);
    if (ritz_norm) {
      // Neither A' nor its Frobenius norm is formed: the norm is the estimate (capped by the trace), and the planes of
      // M_0 and T_0 are made from A with the deflation applied on the way.
      ritz_norm_kernel<<<(kc + 127) / 128, 128, 0, stream>>>(sumsq_a, rest_top, rest_trace, kc);
      count_launch();
      init_planes_kernel<<<dim3(ew_blocks, kc), 256, 0, stream>>>(A32, n, kc, sumsq_a, (float)sched[0].a, (float)sched[0].b,
                                                                  s_m, s_t, Mb[0], Tb[0], Xb[1], dv, coef8, defl_r,
                                                                  kMaxDeflate);
      count_launch();
      TONER_CUDA(cudaGetLastError());
    } else {
    init_planes_kernel<<<dim3(ew_blocks, kc), 256, 0, stream>>>(A32, n, kc, sumsq_a, (float)sched[0].a, (float)sched[0].b, s_m,
                                                                s_t, Mb[0], nullptr, nullptr);
    count_launch();
    TONER_CUDA(cudaGetLastError());
    {
      // A tighter bound of the largest eigenvalue than ||A'||_F: with P = A' / ||A'||_F, lambda_max(P) <= ||P^2||_F^(1/2)
      // = (sum lambda^4)^(1/4), and likewise ||P^4||_F^(1/4), ||P^8||_F^(1/8).  For a flat spectrum these are n^(-1/4),
      // n^(-3/8), n^(-7/16) instead of 1, which raises the spectrum's lower bound after normalisation by the same factor
      // and saves Newton steps (each costs fifteen plane passes; these three squarings cost one pass each).  Single-pass
      // products of hi planes are accurate enough for a bound (3 % is added); the FP32 results and the planes of P^2
      // and P^4 (written by the epilogues, entries at most 1) go to buffers that are free here.
      float* P2 = reinterpret_cast<float*>(Pb[0]);
      const float s_w = plane_scale(1.0);
      toner_gemm_desc g = {};
      toner_operand op = {};
      op.base = Mb[0];
      op.rows = n; op.cols = n; op.ld = n; op.z_stride = nn; op.nz = 2 * kc; op.z_step = 1;
      g.a = op; g.b = op;
      g.m = n; g.n = n; g.k = n; g.batch = kc; g.segs = 1; g.fmt = 0;
      g.tri = 1; g.mirror = 1;
      g.alpha = (float)(1.0 / ((double)s_m * (double)s_m));
      g.d = P2; g.ldd = n; g.d_bs = nn;
      g.split0 = Pb[1]; g.split0_scale = s_w; g.split_ld = n; g.split_bs = nn; g.split_plane = (long long)kc * nn;
      int rc1 = launch_gemm(g, stream);
      if (rc1) return rc1;
      rc1 = sumsq_det(P2, kc, n, n, n, nn, partials, ss2, stream);
      if (rc1) return rc1;
      float* P4 = reinterpret_cast<float*>(Xb[0]);
      toner_gemm_desc g4 = g;
      g4.a.base = Pb[1]; g4.b.base = Pb[1];
      g4.alpha = (float)(1.0 / ((double)s_w * (double)s_w));
      g4.d = P4; g4.split0 = Mb[1];
      rc1 = launch_gemm(g4, stream);
      if (rc1) return rc1;
      rc1 = sumsq_det(P4, kc, n, n, n, nn, partials, ss4, stream);
      if (rc1) return rc1;
      toner_gemm_desc g8 = g4;
      g8.a.base = Mb[1]; g8.b.base = Mb[1];
      g8.d = P2; g8.split0 = nullptr;
      rc1 = launch_gemm(g8, stream);
      if (rc1) return rc1;
      rc1 = sumsq_det(P2, kc, n, n, n, nn, partials, ss8, stream);
      if (rc1) return rc1;
      tighten_bound_kernel<<<(kc + 127) / 128, 128, 0, stream>>>(sumsq_a, ss2, ss4, ss8, kc);
      count_launch();
      init_planes_kernel<<<dim3(ew_blocks, kc), 256, 0, stream>>>(A32, n, kc, sumsq_a, (float)sched[0].a, (float)sched[0].b,
                                                                  s_m, s_t, Mb[0], Tb[0], Xb[1]);
      count_launch();
      TONER_CUDA(cudaGetLastError());
    }
    }

    // D = (A planes) * (B planes)^T / (sa * sb): symmetric result, FP32-accurate; outputs as requested
    struct Out {
      float* d = nullptr;           // FP32 result
      const float* alpha_a = nullptr;  // optional per-statistic factors of the result
      const float* alpha_b = nullptr;
      __half* s0 = nullptr; float s0_scale = 0.f;
      __half* s1 = nullptr; float s1_scale = 0.f, s1_a = 0.f, s1_b = 0.f;
      unsigned int* maxres = nullptr;
      const float* c = nullptr; float beta = 0.f;  // result = gain * product + beta * c (c symmetric, FP32)
      double gain = 1.0;
      int segs = 3;                                // 1: hi planes only (a single pass)
    };
    auto sym_product = [&](const __half* ap, float sa, const __half* bp, float sb, const Out& o, int promote) -> int {
      toner_gemm_desc g = {};
      toner_operand op = {};
      op.rows = n; op.cols = n; op.ld = n; op.z_stride = nn; op.nz = 2 * kc; op.z_step = 1;
      g.a = op; g.a.base = ap;
      g.b = op; g.b.base = bp;
      g.a.seg_z[0] = 0; g.a.seg_z[1] = 0; g.a.seg_z[2] = kc;   // Ah Ah Al
      g.b.seg_z[0] = 0; g.b.seg_z[1] = kc; g.b.seg_z[2] = 0;   // Bh Bl Bh
      g.m = n; g.n = n; g.k = n; g.batch = kc; g.segs = o.segs; g.fmt = 0;
      g.tri = 1; g.mirror = 1;
      g.alpha = (float)(o.gain / ((double)sa * (double)sb));
      g.c = o.c; g.ldc = n; g.c_bs = nn; g.beta = o.beta;
      g.alpha_a = o.alpha_a;
      g.alpha_b = o.alpha_b;
      g.d = o.d; g.ldd = n; g.d_bs = nn;
      g.split0 = o.s0; g.split0_scale = o.s0_scale;
      g.split1 = o.s1; g.split1_scale = o.s1_scale; g.split1_aff_a = o.s1_a; g.split1_aff_b = o.s1_b;
      g.split_ld = n; g.split_bs = nn; g.split_plane = (long long)kc * nn;
      g.maxres = o.maxres;
      g.promote = promote;
      return launch_gemm(g, stream);
    };
    int rc = 0;
    const __half* Xcur = Xb[1];  // X_1 = T_0
    float s_x = s_t;
    double x_bound = sched[0].a;
    int xi = 0, mi = 0, ti = 0;

    for (int it = 0; it < iters; ++it) {
      const bool last = (it == iters - 1);
      const __half* Tcur = Tb[ti];
      if (it > 0) {
        x_bound = std::min(x_bound * sched[it].a, x_cap);
        if (last) {
          // fold ||A||_F^{-1/p} into the product; the distance of M from I was gathered when M was produced
          finish_kernel<<<(kc + 127) / 128, 128, 0, stream>>>(resid, sumsq_a, scale_lo, status ? status + k0 : nullptr,
                                                            norm_out ? norm_out + k0 : nullptr, kc, p, 0.5f, damping,
                                                            lower_used, max_r, (float)root_bound);
          count_launch();
          TONER_CUDA(cudaGetLastError());
          // Tcur holds planes of R = I - M and A32 the FP32 M (both from the last update of M).  Horner steps
          // W_j = c_j R + R W_{j+1} (W_m = c_m R) build q(R) = c_0 I + W_1; the terms linear in M enter in FP32 as
          // beta * c.
          const float s_w = plane_scale(1.0), s_f = plane_scale(2.0);
          const __half* wcur = Tcur;
          float s_cur = s_t;
          double gain = fin.c[order];
          for (int j = order - 1; j >= 1; --j) {
            const double aj = fin.c[j];
            Out w;
            w.segs = 1;
            w.gain = gain;
            w.c = A32; w.beta = (float)-aj;
            w.s1 = Mb[j & 1];
            w.s1_scale = (j == 1) ? s_f : s_w;
            w.s1_a = (float)(j == 1 ? fin.c[0] + aj : aj);
            w.s1_b = 1.f;
            rc = sym_product(Tcur, s_t, wcur, s_cur, w, 0);
            if (rc) return rc;
            wcur = w.s1;
            s_cur = w.s1_scale;
            gain = 1.0;
          }
          float* R = root_lo + (long long)k0 * nn;
          Out o;
          o.d = R;
          o.alpha_a = scale_lo;
          rc = sym_product(Xcur, s_x, Mb[1], s_f, o, kPromoteX);
          if (rc) return rc;
          // put the deflated direction back: A^{-1/p} = A'^{-1/p} + (lambda_1^{-1/p} - c^{-1/p}) v v^T
          if (defl_r > 0) rankr_update_kernel<<<dim3(ew_blocks, kc), 256, 0, stream>>>(R, dv, corr8, n, defl_r, kMaxDeflate);
          else rank1_update_kernel<<<dim3(ew_blocks, kc), 256, 0, stream>>>(R, pv, corr, n);
          count_launch();
          TONER_CUDA(cudaGetLastError());
          rc = sumsq_det(R, kc, n, n, n, nn, partials, fro_tmp, stream);
          if (rc) return rc;
          if (q > 1) {  // operand planes of the finished root for the squarings below
            rc = split16(R, nullptr, kc, n, n, n, nn, 0.f, 1.f, max_r, nullptr, Xb[xi], inv_r, stream);
            if (rc) return rc;
          }
          Xcur = Xb[xi];
          break;
        }
        Out o;
        o.s0 = Xb[xi];
        o.s0_scale = plane_scale(x_bound);
        rc = sym_product(Xcur, s_x, Tcur, s_t, o, kPromoteX);
        if (rc) return rc;
        Xcur = Xb[xi];
        s_x = o.s0_scale;
        xi ^= 1;
      }
      // M_{k+1} = T^p M_k.  The tensor core adds into its accumulator by truncation, a one-sided error that
      // grows with the length of the accumulation chain and, unlike rounding noise, does not average out over
      // the sum; a relative error e of M matters as e / (smallest eigenvalue of M), so the chains are kept
      // short while the spectrum's lower bound is small and lengthened as it approaches 1.
      const int chain = chain_length(sched[it].lower);
      const __half* pw = Tcur;
      float s_pw = s_t;
      double pw_bound = sched[it].a;
      for (int j = 0; j < log2p; ++j) {
        pw_bound *= pw_bound;
        Out o;
        o.s0 = Pb[j & 1];
        o.s0_scale = plane_scale(pw_bound);
        rc = sym_product(pw, s_pw, pw, s_pw, o, chain);
        if (rc) return rc;
        pw = o.s0;
        s_pw = o.s0_scale;
      }
      {
        const float na = (float)sched[it + 1].a, nb = (float)sched[it + 1].b;
        const int tn = (log2p == 0) ? (ti ^ 1) : ti;  // with p == 1 the product reads T itself
        Out o;
        o.s1 = Tb[tn];
        if (it == iters - 2) {
          // the last M: kept in FP32 with planes of R = I - M for the finishing series, and its distance from I
          o.d = A32;
          o.s1_scale = s_m;
          o.s1_a = 1.f;
          o.s1_b = -1.f;
          o.maxres = resid;
        } else {
          o.s0 = Mb[mi ^ 1];
          o.s0_scale = s_m;
          o.s1_scale = plane_scale(na);
          o.s1_a = na;
          o.s1_b = -nb;
        }
        rc = sym_product(pw, s_pw, Mb[mi], s_m, o, chain);
        if (rc) return rc;
        mi ^= 1;
        ti = tn;
        s_t = o.s1_scale;
      }
    }
    if (fro2_lo) TONER_CUDA(cudaMemcpyAsync(fro2_lo + k0, fro_tmp, sizeof(float) * kc, cudaMemcpyDeviceToDevice, stream));

    if (q > 1) {
      // A^{-q/p} by repeated squaring of A^{-1/p} (its planes came with the last product)
      int have = 1;
      double bound = root_bound;
      int pi = 0;
      s_x = 1.f;  // the root's planes carry per-statistic scales (inv_r), applied below
      while (have < q) {
        const bool first = (have == 1);
        have *= 2;
        bound *= bound;
        Out o;
        if (first) {
          o.alpha_a = inv_r;
          o.alpha_b = inv_r;
        }
        if (have == q) {
          o.d = root_hi + (long long)k0 * nn;
        } else {
          o.s0 = Pb[pi];
          o.s0_scale = plane_scale(bound);
        }
        rc = sym_product(Xcur, s_x, Xcur, s_x, o, kPromoteX);
        if (rc) return rc;
        Xcur = Pb[pi];
        s_x = o.s0_scale;
        pi ^= 1;
      }
    }

    if (track) {
      float* vt = track + (long long)k0 * n;
      if (lower_used < 0.f) {
        // The schedule was built for an ESTIMATE of the spectrum's lower end.  If the estimate was too high for a
        // statistic, its smallest eigenvalues have not reached the distance from 1 the finishing series was cut for,
        // and they are the dominant eigenvalues of R = I - M of the last M (kept in FP32): four power-iteration steps
        // on R from the tracked direction (the eigenvector of the smallest eigenvalue, as of the previous call) find
        // them.  The allowance: the assumed distance with 15 % and the noise floor of the estimate.
        if (ritz_norm) {
          // The norm was an estimate too.  Eigenvalues of M_0 above 1 (the estimate was too low for them) come out of
          // the first Newton step BELOW the lower bound the schedule continues from -- T = a I - b M is small there --
          // and lag the same way; they belong to the top of A', so the same four steps from the largest Ritz vector
          // that stayed in A' find them.  (An eigenvalue beyond a / b, where T changes sign, makes M grow instead and
          // fails the convergence test.)  Both starting vectors go through M in one pass per step.
          pick_vector_kernel<<<dim3(8, kc), 256, 0, stream>>>(vt, dv, rest_idx, pv, n, kMaxDeflate);
          count_launch();
          const dim3 bg((n + kBlockGemvRows - 1) / kBlockGemvRows, kc);
          for (int sw = 0; sw < 4; ++sw) {
            block_gemv_kernel<2><<<bg, 256, 0, stream>>>(A32, pv, py, n, 2, 2);
            count_launch();
            power_shift_kernel<<<dim3(kc, 2), 256, 0, stream>>>(pv, py, n, e_est, 2, (long long)(e_top - e_est));
            count_launch();
          }
        } else {
          TONER_CUDA(cudaMemcpyAsync(pv, vt, sizeof(float) * (size_t)kc * n, cudaMemcpyDeviceToDevice, stream));
          for (int sw = 0; sw < 4; ++sw) {
            gemv_kernel<<<dim3((n + 7) / 8, kc), 256, 0, stream>>>(A32, pv, py, n);
            count_launch();
            power_shift_kernel<<<kc, 256, 0, stream>>>(pv, py, n, e_est);
            count_launch();
          }
        }
        verify_kernel<<<(kc + 127) / 128, 128, 0, stream>>>(e_est, ritz_norm ? e_top : nullptr,
                                                          (float)(1.15 * (1.0 - l_last) + 1e-3),
                                                          status ? status + k0 : nullptr,
                                                          resid_out ? resid_out + k0 : nullptr, kc);
        count_launch();
        TONER_CUDA(cudaGetLastError());
      }
      const int sweeps = track_sweeps & 63;
      if (sweeps > 0) {
        // Track the direction of the smallest eigenvalue of A for the next call: it is the dominant eigenvector of the
        // highest inverse power just computed, where it stands out however small it is next to lambda_max(A).
        const float* top = (q > 1 ? root_hi : root_lo) + (long long)k0 * nn;
        if (track_sweeps & 256) {
          power_start_kernel<<<dim3(8, kc), 256, 0, stream>>>(vt, n);
          count_launch();
        }
        for (int sw = 0; sw < sweeps; ++sw) {
          gemv_kernel<<<dim3((n + 7) / 8, kc), 256, 0, stream>>>(top, vt, py, n);
          count_launch();
          power_norm_kernel<<<kc, 256, 0, stream>>>(vt, py, n, theta, pres);
          count_launch();
        }
        if (lmin_out) {
          lmin_from_root_kernel<<<(kc + 127) / 128, 128, 0, stream>>>(theta, (float)p / (float)q, lmin_out + k0, kc);
          count_launch();
        }
        TONER_CUDA(cudaGetLastError());
      }
    }
  }
  return 0;
}

}  // extern "C"

// Factor engine: inverse p-th roots of damped, trace-normalised input statistics by a coupled Newton
// iteration with minimax scaling, every product on the tcgen05 GEMM in FP32-accurate split precision.
//
//   A   = sym(C) / mean(diag C) + damping * I                 (what the reference factors by eigh)
//   M_0 = A / ||A||_F         (spectrum inside [l_0, 1],  l_0 >= damping / (n (1 + damping)))
//   T_k = a_k I - b_k M_k ;  X_{k+1} = X_k T_k ;  M_{k+1} = T_k^p M_k          (X_0 = I)
//   X_K ~ M_0^{-1/p}  =>  A^{-1/p} = X_K ||A||_F^{-1/p}
// (a_k, b_k) map the interval [l_k, 1] known to contain the spectrum of M_k onto [l_{k+1}, 1] with
// l_{k+1} as large as a linear T allows (the ends of the interval and the interior maximum of
// mu (a - b mu)^p are levelled, subject to a cap on b/a that bounds the dynamic range of T^p); once
// l_k is close to 1 they become the Newton values ((p+1)/p, 1/p).
// The schedule depends only on (n, damping, p), so the iteration count is fixed and stated.
#include <cmath>
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

static int default_iterations(double l0, int p) {
  // steps until the spectrum is within 3e-4 of 1, plus one Newton step (which squares that distance)
  for (int k = 1; k < 64; ++k) {
    double l;
    newton_schedule(l0, p, k, &l);
    if (1.0 - l < 3e-4) return k + 1;
  }
  return 64;
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

// x <- x * factor[b] (factor = 1/sqrt(sumsq) when rsqrt_of_sumsq), with max|x| and max|aff_a I + aff_b x|.
__global__ void __launch_bounds__(256) scale_stats_kernel(float* __restrict__ x, int n, const float* __restrict__ sumsq,
                                                          float aff_a, float aff_b, unsigned int* __restrict__ maxabs,
                                                          unsigned int* __restrict__ maxaff) {
  const int b = blockIdx.y;
  float* X = x + (long long)b * n * n;
  const float f = rsqrtf(fmaxf(sumsq[b], 1e-60f));
  const long long total = (long long)n * n;
  float m0 = 0.f, m1 = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / n), c = (int)(i - (long long)r * n);
    const float v = X[i] * f;
    X[i] = v;
    m0 = fmaxf(m0, fabsf(v));
    m1 = fmaxf(m1, fabsf(aff_b * v + (r == c ? aff_a : 0.f)));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, o));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, o));
  }
  if ((threadIdx.x & 31) == 0) {
    atomicMax(maxabs + b, __float_as_uint(m0));
    atomicMax(maxaff + b, __float_as_uint(m1));
  }
}

// y = aff_a I + aff_b x (FP32 copy; used for X_1 = T_0)
__global__ void __launch_bounds__(256) affine_copy_kernel(const float* __restrict__ x, float* __restrict__ y, int n,
                                                          float aff_a, float aff_b) {
  const int b = blockIdx.y;
  const float* X = x + (long long)b * n * n;
  float* Y = y + (long long)b * n * n;
  const long long total = (long long)n * n;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / n), c = (int)(i - (long long)r * n);
    Y[i] = aff_b * X[i] + (r == c ? aff_a : 0.f);
  }
}

// status[b]: 0 converged, 1 residual max|I - M| above tol, 2 non-finite
__global__ void __launch_bounds__(256) residual_kernel(const float* __restrict__ m, int n, unsigned int* __restrict__ resid) {
  const int b = blockIdx.y;
  const float* M = m + (long long)b * n * n;
  const long long total = (long long)n * n;
  float r0 = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / n), c = (int)(i - (long long)r * n);
    const float v = fabsf((r == c ? 1.f : 0.f) - M[i]);
    r0 = (v == v) ? fmaxf(r0, v) : INFINITY;  // NaN counts as infinite residual
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, o));
  if ((threadIdx.x & 31) == 0) atomicMax(resid + b, __float_as_uint(r0));
}

__global__ void finish_kernel(const unsigned int* __restrict__ resid, const float* __restrict__ sumsq_a, float* inv_x,
                              float* root_scale_lo, float* root_scale_hi, int* status, int k, int p, int q, float tol) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= k) return;
  const float ub = sqrtf(fmaxf(sumsq_a[b], 1e-60f));
  const float s_lo = powf(ub, -1.f / p);
  root_scale_lo[b] = s_lo;
  root_scale_hi[b] = powf(ub, -(float)q / p);
  inv_x[b] *= s_lo;  // the last X product applies the inverse operand scales: fold the root's scale in
  const float r = __uint_as_float(resid[b]);
  if (status) status[b] = !isfinite(r) ? 2 : (r > tol ? 1 : 0);
}

__global__ void mul_vec_kernel(float* a, const float* b, int k) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < k) a[i] *= b[i];
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static size_t per_statistic_bytes(int n) {
  // M, X, F (FP32) + five FP16 hi/lo plane pairs (T, M, X, P0, P1) = 8 FP32-sized matrices
  return align_up((size_t)n * n * 4, 256) * 8;
}
static size_t small_bytes(int chunk) { return align_up((size_t)chunk * 4, 256) * 16 + align_up(sumsq_scratch_bytes(chunk), 256); }

}  // namespace toner

extern "C" {

size_t toner_inv_roots_workspace_bytes(int32_t chunk, int32_t n) {
  if (chunk <= 0 || n <= 0) return 0;
  return toner::per_statistic_bytes(n) * (size_t)chunk + toner::small_bytes(chunk);
}

int toner_inv_roots_iterations(int32_t n, float damping, int32_t p) {
  if (n <= 0 || !(damping > 0) || p < 1) return 0;
  return toner::default_iterations((double)damping / ((double)n * (1.0 + damping)), p);
}

int toner_inv_roots(const float* ema, int32_t k, int32_t n, float damping, int32_t p, int32_t q, int32_t iters,
                    float* root_lo, float* root_hi, float* fro2_lo, int32_t* status, void* workspace,
                    size_t workspace_bytes, void* stream_) {
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
  const double l0 = (double)damping / ((double)n * (1.0 + damping));
  if (iters <= 0) iters = default_iterations(l0, p);
  if (iters < 2) return fail(kErrArg, "inv_roots: at least two iterations are required");
  const std::vector<NewtonStep> sched = newton_schedule(l0, p, iters, nullptr);
  int log2p = 0;
  while ((1 << log2p) < p) ++log2p;

  const size_t per = per_statistic_bytes(n);
  long long chunk_cap = 0;
  for (long long c = k; c >= 1; --c) {
    if (per * (size_t)c + small_bytes((int)c) <= workspace_bytes) {
      chunk_cap = c;
      break;
    }
  }
  if (chunk_cap < 1) return fail(kErrWorkspace, "inv_roots: workspace holds less than one statistic");
  const long long nn = (long long)n * n;
  const size_t mat = align_up((size_t)nn * 4, 256);
  const int ew_blocks = (int)std::min<long long>((nn + 1023) / 1024, 4LL * ctx->num_sms);

  for (int k0 = 0; k0 < k; k0 += (int)chunk_cap) {
    const int kc = (int)std::min<long long>(chunk_cap, k - k0);
    char* w = static_cast<char*>(workspace);
    float* M = reinterpret_cast<float*>(w); w += mat * kc;
    float* X = reinterpret_cast<float*>(w); w += mat * kc;
    float* F = reinterpret_cast<float*>(w); w += mat * kc;
    __half* Tp = reinterpret_cast<__half*>(w); w += mat * kc;
    __half* Mp = reinterpret_cast<__half*>(w); w += mat * kc;
    __half* Xp = reinterpret_cast<__half*>(w); w += mat * kc;
    __half* P0 = reinterpret_cast<__half*>(w); w += mat * kc;
    __half* P1 = reinterpret_cast<__half*>(w); w += mat * kc;
    const size_t sm = align_up((size_t)kc * 4, 256);
    auto small = [&](int i) { return reinterpret_cast<float*>(w + sm * i); };
    float* trace = small(0);
    float* sumsq_a = small(1);
    unsigned int* max_m = reinterpret_cast<unsigned int*>(small(2));
    unsigned int* max_t = reinterpret_cast<unsigned int*>(small(3));
    unsigned int* max_x = reinterpret_cast<unsigned int*>(small(4));
    unsigned int* max_f = reinterpret_cast<unsigned int*>(small(5));
    unsigned int* resid = reinterpret_cast<unsigned int*>(small(6));
    float* inv_t = small(7);
    float* inv_m = small(8);
    float* inv_x = small(9);
    float* inv_p0 = small(10);
    float* inv_p1 = small(11);
    float* scale_lo = small(12);
    float* scale_hi = small(13);
    float* fro_tmp = small(14);
    float* partials = small(16);
    TONER_CUDA(cudaMemsetAsync(w, 0, sm * 16, stream));

    const float* C = ema + (long long)k0 * nn;
    const int t32 = (n + 31) / 32;
    trace_kernel<<<kc, 256, 0, stream>>>(C, n, trace);
    count_launch();
    damp_kernel<<<dim3(t32, t32, kc), 256, 0, stream>>>(C, M, n, damping, trace);
    count_launch();
    {
      int rc0 = sumsq_det(M, kc, n, n, n, nn, partials, sumsq_a, stream);
      if (rc0) return rc0;
    }
    scale_stats_kernel<<<dim3(ew_blocks, kc), 256, 0, stream>>>(M, n, sumsq_a, (float)sched[0].a, (float)-sched[0].b, max_m, max_t);
    count_launch();
    TONER_CUDA(cudaGetLastError());

    auto planes_op = [&](const __half* planes, int hi_lo_first) {
      toner_operand op = {};
      op.base = planes;
      op.rows = n; op.cols = n; op.ld = n; op.z_stride = nn; op.nz = 2 * kc; op.z_step = 1;
      return op;
    };
    // D = (A planes) * (B planes)^T, symmetric result, FP32-accurate
    auto sym_product = [&](const __half* ap, const float* ainv, const __half* bp, const float* binv, float* d,
                           unsigned int* maxabs, unsigned int* maxaff, float aff_a, float aff_b, float* sumsq) -> int {
      toner_gemm_desc g = {};
      g.a = planes_op(ap, 0);
      g.b = planes_op(bp, 0);
      g.a.seg_z[0] = 0; g.a.seg_z[1] = 0; g.a.seg_z[2] = kc;   // Ah Ah Al
      g.b.seg_z[0] = 0; g.b.seg_z[1] = kc; g.b.seg_z[2] = 0;   // Bh Bl Bh
      g.m = n; g.n = n; g.k = n; g.batch = kc; g.segs = 3; g.fmt = 0;
      g.tri = 1; g.mirror = 1;
      g.alpha = 1.f; g.alpha_a = ainv; g.alpha_b = binv;
      g.d = d; g.ldd = n; g.d_bs = nn;
      g.maxabs = maxabs; g.maxaff = maxaff; g.aff_a = aff_a; g.aff_b = aff_b; g.sumsq = sumsq;
      g.promote = kPromoteAccurate;
      return launch_gemm(g, stream);
    };
    auto zero = [&](void* ptr) { return cudaMemsetAsync(ptr, 0, sm, stream); };
    int rc = 0;

    for (int it = 0; it < iters; ++it) {
      const float a = (float)sched[it].a, b = (float)sched[it].b;
      const bool last = (it == iters - 1);
      // T_k planes from M_k (max|T_k| was gathered when M_k was produced)
      rc = split16(M, nullptr, kc, n, n, n, nn, a, -b, max_t, nullptr, Tp, inv_t, stream);
      if (rc) return rc;
      if (it == 0) {
        affine_copy_kernel<<<dim3(ew_blocks, kc), 256, 0, stream>>>(M, X, n, a, -b);  // X_1 = T_0
        TONER_CUDA(cudaGetLastError());
        count_launch();
        TONER_CUDA(cudaMemcpyAsync(max_x, max_t, sm, cudaMemcpyDeviceToDevice, stream));
      } else {
        rc = split16(X, nullptr, kc, n, n, n, nn, 0.f, 1.f, max_x, nullptr, Xp, inv_x, stream);
        if (rc) return rc;
        if (last) {
          // fold ||A||_F^{-1/p} into the product, take the residual of M before it stops being updated
          TONER_CUDA(zero(resid));
          residual_kernel<<<dim3(ew_blocks, kc), 256, 0, stream>>>(M, n, resid);
          count_launch();
          finish_kernel<<<(kc + 127) / 128, 128, 0, stream>>>(resid, sumsq_a, inv_x, scale_lo, scale_hi,
                                                            status ? status + k0 : nullptr, kc, p, q, 0.05f);
          count_launch();
          TONER_CUDA(cudaGetLastError());
          TONER_CUDA(zero(max_x));
          rc = sym_product(Xp, inv_x, Tp, inv_t, root_lo + (long long)k0 * nn, max_x, nullptr, 0.f, 1.f, nullptr);
          if (rc) return rc;
          rc = sumsq_det(root_lo + (long long)k0 * nn, kc, n, n, n, nn, partials, fro_tmp, stream);
          if (rc) return rc;
          break;
        }
        TONER_CUDA(zero(max_x));
        rc = sym_product(Xp, inv_x, Tp, inv_t, X, max_x, nullptr, 0.f, 1.f, nullptr);
        if (rc) return rc;
      }
      // M_{k+1} = T^p M_k
      rc = split16(M, nullptr, kc, n, n, n, nn, 0.f, 1.f, max_m, nullptr, Mp, inv_m, stream);
      if (rc) return rc;
      const __half* pw = Tp;
      const float* pw_inv = inv_t;
      for (int j = 0; j < log2p; ++j) {
        TONER_CUDA(zero(max_f));
        rc = sym_product(pw, pw_inv, pw, pw_inv, F, max_f, nullptr, 0.f, 1.f, nullptr);
        if (rc) return rc;
        __half* dst = (j & 1) ? P1 : P0;
        float* dst_inv = (j & 1) ? inv_p1 : inv_p0;
        rc = split16(F, nullptr, kc, n, n, n, nn, 0.f, 1.f, max_f, nullptr, dst, dst_inv, stream);
        if (rc) return rc;
        pw = dst;
        pw_inv = dst_inv;
      }
      TONER_CUDA(zero(max_m));
      TONER_CUDA(zero(max_t));
      const float na = (float)sched[it + 1].a, nb = (float)sched[it + 1].b;
      rc = sym_product(pw, pw_inv, Mp, inv_m, M, max_m, max_t, na, -nb, nullptr);
      if (rc) return rc;
    }
    if (fro2_lo) TONER_CUDA(cudaMemcpyAsync(fro2_lo + k0, fro_tmp, sizeof(float) * kc, cudaMemcpyDeviceToDevice, stream));

    if (q > 1) {
      // A^{-q/p} by repeated squaring of A^{-1/p}
      const float* src = root_lo + (long long)k0 * nn;
      int have = 1;
      while (have < q) {
        __half* pl = (have == 1) ? Xp : P0;
        float* pl_inv = (have == 1) ? inv_x : inv_p0;
        const unsigned int* mx = (have == 1) ? max_x : max_f;
        rc = split16(src, nullptr, kc, n, n, n, nn, 0.f, 1.f, mx, nullptr, pl, pl_inv, stream);
        if (rc) return rc;
        have *= 2;
        float* dst = (have == q) ? root_hi + (long long)k0 * nn : F;
        TONER_CUDA(zero(max_f));
        rc = sym_product(pl, pl_inv, pl, pl_inv, dst, max_f, nullptr, 0.f, 1.f, nullptr);
        if (rc) return rc;
        src = dst;
      }
    }
  }
  return 0;
}

}  // extern "C"

// Update path: Muon Newton-Schulz polar iteration on the tcgen05 GEMM, and the elementwise
// momentum / Adam-moment / apply kernels (vectorised, coalesced, HBM-bound).
#include <cuda_bf16.h>

#include "runtime.cuh"

namespace toner {

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
static int ew_grid(long long elems4, int num_sms) {
  long long b = (elems4 + 255) / 256;
  const long long cap = 8LL * num_sms;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

// ------------------------------------------------------------------ Newton-Schulz helpers
// x = u / (sqrt(sumsq[b]) + eps), written as FP32 and as BF16 (the operand the products read)
__global__ void __launch_bounds__(256) ns_scale_kernel(const float* __restrict__ u, const float* __restrict__ sumsq,
                                                       float eps, long long per, float* __restrict__ x,
                                                       __nv_bfloat16* __restrict__ xb) {
  const int b = blockIdx.y;
  const float f = 1.f / (sqrtf(sumsq[b]) + eps);
  const float4* U = reinterpret_cast<const float4*>(u + (long long)b * per);
  float4* X = reinterpret_cast<float4*>(x + (long long)b * per);
  uint2* XB = reinterpret_cast<uint2*>(xb + (long long)b * per);
  const long long n4 = per / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 v = U[i];
    v.x *= f; v.y *= f; v.z *= f; v.w *= f;
    X[i] = v;
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), c = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&a);
    o.y = *reinterpret_cast<uint32_t*>(&c);
    XB[i] = o;
  }
}

// ------------------------------------------------------------------ MuonT momentum
// m <- mu m + g ;  u = nesterov ? g + mu m : m ;  maxabs[b] = max |u|
__global__ void __launch_bounds__(256) muont_momentum_kernel(const float* const* __restrict__ grads, float* __restrict__ m,
                                                             float* __restrict__ u, long long per, float mu, int nesterov,
                                                             unsigned int* __restrict__ maxabs) {
  const int b = blockIdx.y;
  const float4* G = reinterpret_cast<const float4*>(grads[b]);
  float4* M = reinterpret_cast<float4*>(m + (long long)b * per);
  float4* U = reinterpret_cast<float4*>(u + (long long)b * per);
  const long long n4 = per / 4;
  float mx = 0.f;
  auto update = [&](const float4 g, float4 mm, long long i) {
    mm.x = fmaf(mu, mm.x, g.x); mm.y = fmaf(mu, mm.y, g.y); mm.z = fmaf(mu, mm.z, g.z); mm.w = fmaf(mu, mm.w, g.w);
    M[i] = mm;
    float4 d = mm;
    if (nesterov) {
      d.x = fmaf(mu, mm.x, g.x); d.y = fmaf(mu, mm.y, g.y); d.z = fmaf(mu, mm.z, g.z); d.w = fmaf(mu, mm.w, g.w);
    }
    U[i] = d;
    mx = fmaxf(fmaxf(fmaxf(mx, fabsf(d.x)), fabsf(d.y)), fmaxf(fabsf(d.z), fabsf(d.w)));
  };
  // four independent 16-byte loads in flight per thread before the first store
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + stride < n4; i += 2 * stride) {
    const float4 g0 = G[i], g1 = G[i + stride];
    const float4 m0 = M[i], m1 = M[i + stride];
    update(g0, m0, i);
    update(g1, m1, i + stride);
  }
  if (i < n4) update(G[i], M[i], i);
  if (maxabs) block_atomic_max(mx, maxabs + b);
}

// c1[b] = lr wd n / ||R||_F^2 ,  c2[b] = lr scale sqrt(n) / ||R||_F   with ||R||_F^2 = fro2[first + b*step]
__global__ void muont_coeff_kernel(const float* __restrict__ fro2, int first, int step, int count, int n, float lr, float wd,
                                   float scale, float* __restrict__ c1, float* __restrict__ c2) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= count) return;
  const float f2 = fro2[first + b * step];
  c1[b] = lr * wd * (float)n / fmaxf(f2, 1e-60f);
  c2[b] = lr * scale * sqrtf((float)n) / fmaxf(sqrtf(f2), 1e-30f);
}

__global__ void mul_vec_kernel2(float* a, const float* b, int k) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < k) a[i] *= b[i];
}

// ------------------------------------------------------------------ AdamT elementwise
// m <- b1 m + (1-b1) g
__global__ void __launch_bounds__(256) adamt_m_kernel(const float* const* __restrict__ grads, float* __restrict__ m,
                                                      long long per, float b1) {
  const int b = blockIdx.y;
  const float4* G = reinterpret_cast<const float4*>(grads[b]);
  float4* M = reinterpret_cast<float4*>(m + (long long)b * per);
  const long long n4 = per / 4;
  const float w = 1.f - b1;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 g = G[i];
    float4 mm = M[i];
    mm.x = mm.x * b1 + g.x * w; mm.y = mm.y * b1 + g.y * w; mm.z = mm.z * b1 + g.z * w; mm.w = mm.w * b1 + g.w * w;
    M[i] = mm;
  }
}

// v <- b2 v + (1-b2) t^2 ;  ratio = num / (sqrt(v / bc2) + eps)  (num already holds (m / bc1) R), in place in num
__global__ void __launch_bounds__(256) adamt_ratio_kernel(const float* __restrict__ t, float* __restrict__ v,
                                                          float* __restrict__ num, long long per, float b2, float bc2,
                                                          float eps, unsigned int* __restrict__ maxabs) {
  const int b = blockIdx.y;
  const float4* T = reinterpret_cast<const float4*>(t + (long long)b * per);
  float4* V = reinterpret_cast<float4*>(v + (long long)b * per);
  float4* N = reinterpret_cast<float4*>(num + (long long)b * per);
  const long long n4 = per / 4;
  const float w = 1.f - b2;
  float mx = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 tt = T[i];
    float4 vv = V[i];
    vv.x = vv.x * b2 + tt.x * tt.x * w; vv.y = vv.y * b2 + tt.y * tt.y * w;
    vv.z = vv.z * b2 + tt.z * tt.z * w; vv.w = vv.w * b2 + tt.w * tt.w * w;
    V[i] = vv;
    float4 nn = N[i];
    nn.x = nn.x / (sqrtf(vv.x / bc2) + eps); nn.y = nn.y / (sqrtf(vv.y / bc2) + eps);
    nn.z = nn.z / (sqrtf(vv.z / bc2) + eps); nn.w = nn.w / (sqrtf(vv.w / bc2) + eps);
    N[i] = nn;
    mx = fmaxf(fmaxf(fmaxf(mx, fabsf(nn.x)), fabsf(nn.y)), fmaxf(fabsf(nn.z), fabsf(nn.w)));
  }
  if (maxabs) block_atomic_max(mx, maxabs + b);
}

// c1[b] = lr wd n / ||R||_F^2 ;  c2[b] = -lr ||U||_F / max(||U R||_F, 1e-30)
__global__ void adamt_coeff_kernel(const float* __restrict__ fro2, int first, int step, int count, int n, float lr, float wd,
                                   const float* __restrict__ ss_before, const float* __restrict__ ss_after,
                                   float* __restrict__ c1, float* __restrict__ c2) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= count) return;
  c1[b] = lr * wd * (float)n / fmaxf(fro2[first + b * step], 1e-60f);
  c2[b] = -lr * sqrtf(ss_before[b]) / fmaxf(sqrtf(ss_after[b]), 1e-30f);
}

// ------------------------------------------------------------------ apply
// W_b += delta_b for separately allocated weights
__global__ void __launch_bounds__(256) apply_delta_kernel(float* const* __restrict__ weights, const float* __restrict__ delta,
                                                          long long per) {
  const int b = blockIdx.y;
  float4* W = reinterpret_cast<float4*>(weights[b]);
  const float4* D = reinterpret_cast<const float4*>(delta + (long long)b * per);
  const long long n4 = per / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 w = W[i];
    const float4 d = D[i];
    w.x += d.x; w.y += d.y; w.z += d.z; w.w += d.w;
    W[i] = w;
  }
}

// W_b <- ws * W_b + ds * delta_b (decoupled weight decay and a scaled change in one pass)
__global__ void __launch_bounds__(256) apply_scaled_kernel(float* const* __restrict__ weights, const float* __restrict__ delta,
                                                           long long per, float ws, float ds) {
  const int b = blockIdx.y;
  float4* W = reinterpret_cast<float4*>(weights[b]);
  const float4* D = reinterpret_cast<const float4*>(delta + (long long)b * per);
  const long long n4 = per / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 w = W[i];
    const float4 d = D[i];
    w.x = fmaf(ds, d.x, ws * w.x); w.y = fmaf(ds, d.y, ws * w.y);
    w.z = fmaf(ds, d.z, ws * w.z); w.w = fmaf(ds, d.w, ws * w.w);
    W[i] = w;
  }
}

__global__ void __launch_bounds__(256) scale_stack_kernel(const float* __restrict__ x, const float* __restrict__ coeff,
                                                          float* __restrict__ out, long long per) {
  const int b = blockIdx.y;
  const float c = coeff[b];
  const float4* X = reinterpret_cast<const float4*>(x + (long long)b * per);
  float4* O = reinterpret_cast<float4*>(out + (long long)b * per);
  const long long n4 = per / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 v = X[i];
    v.x *= c; v.y *= c; v.z *= c; v.w *= c;
    O[i] = v;
  }
}

// out = a x + b y
__global__ void __launch_bounds__(256) axpby_kernel(const float* __restrict__ x, const float* __restrict__ y,
                                                    float* __restrict__ out, long long n, float a, float b) {
  const long long n4 = n / 4;
  const float4* X = reinterpret_cast<const float4*>(x);
  const float4* Y = reinterpret_cast<const float4*>(y);
  float4* O = reinterpret_cast<float4*>(out);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 p = X[i], q = Y[i];
    O[i] = make_float4(fmaf(a, p.x, b * q.x), fmaf(a, p.y, b * q.y), fmaf(a, p.z, b * q.z), fmaf(a, p.w, b * q.w));
  }
  for (long long i = n4 * 4 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = fmaf(a, x[i], b * y[i]);
}

}  // namespace toner

extern "C" {

using namespace toner;

int toner_axpby(const float* x, const float* y, float* out, int64_t n, float a, float b, void* stream) {
  Context* ctx = context();
  if (!ctx) return kErrCuda;
  if (!x || !y || !out || n <= 0) return fail(kErrArg, "axpby: bad arguments");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(out)) & 15u)
    return fail(kErrArg, "axpby: pointers must be 16-byte aligned");
  axpby_kernel<<<ew_grid(n / 4 + 1, ctx->num_sms), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, y, out, n, a, b);
  count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

int toner_scale_stack(const float* x, const float* coeff, float* out, int32_t count, int64_t per, void* stream) {
  Context* ctx = context();
  if (!ctx) return kErrCuda;
  if (!x || !coeff || !out || count <= 0 || per <= 0 || per % 4) return fail(kErrArg, "scale_stack: bad arguments");
  scale_stack_kernel<<<dim3(ew_grid(per / 4, ctx->num_sms), count), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, coeff, out, per);
  count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

size_t toner_ns_polar_workspace_bytes(int32_t batch, int32_t m, int32_t n) {
  if (batch <= 0 || m <= 0 || n <= 0) return 0;
  const size_t a = (size_t)(m < n ? m : n);
  const size_t mn = (size_t)m * n;
  return align_up(sumsq_scratch_bytes(batch), 256) + align_up((size_t)batch * 4, 256) +
         2 * align_up(mn * 2 * batch, 256) +                 // two BF16 copies of X (read one, write the other)
         align_up(a * a * 4 * batch, 256) +                  // Gram, FP32
         2 * align_up(a * a * 2 * batch, 256);               // Gram and polynomial, BF16
}

int toner_ns_polar(const float* u, int32_t batch, int32_t m, int32_t n, int32_t steps, float eps, float* x_out,
                   uint32_t* maxabs_out, void* workspace, size_t workspace_bytes, void* stream_) {
  Context* ctx = context();
  if (!ctx) return kErrCuda;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!u || !x_out || !workspace) return fail(kErrArg, "ns_polar: null pointer");
  if (batch <= 0 || m <= 0 || n <= 0 || steps < 1 || !(eps > 0.f)) return fail(kErrArg, "ns_polar: bad sizes");
  if (m % 8 != 0 || n % 8 != 0) return fail(kErrUnsupported, "ns_polar: matrix dimensions must be multiples of 8");
  if (workspace_bytes < toner_ns_polar_workspace_bytes(batch, m, n)) return fail(kErrWorkspace, "ns_polar: workspace too small");
  const bool wide = m <= n;
  const int a = wide ? m : n;
  const long long mn = (long long)m * n, aa = (long long)a * a;
  char* w = static_cast<char*>(workspace);
  float* partial = reinterpret_cast<float*>(w); w += align_up(sumsq_scratch_bytes(batch), 256);
  float* ss = reinterpret_cast<float*>(w); w += align_up((size_t)batch * 4, 256);
  __nv_bfloat16* xb[2];
  xb[0] = reinterpret_cast<__nv_bfloat16*>(w); w += align_up((size_t)mn * 2 * batch, 256);
  xb[1] = reinterpret_cast<__nv_bfloat16*>(w); w += align_up((size_t)mn * 2 * batch, 256);
  float* gram = reinterpret_cast<float*>(w); w += align_up((size_t)aa * 4 * batch, 256);
  __nv_bfloat16* gram_b = reinterpret_cast<__nv_bfloat16*>(w); w += align_up((size_t)aa * 2 * batch, 256);
  __nv_bfloat16* poly_b = reinterpret_cast<__nv_bfloat16*>(w);

  int rc = sumsq_det(u, batch, m, n, n, mn, partial, ss, stream);
  if (rc) return rc;
  ns_scale_kernel<<<dim3(ew_grid(mn / 4, ctx->num_sms), batch), 256, 0, stream>>>(u, ss, eps, mn, x_out, xb[0]);
  count_launch();
  TONER_CUDA(cudaGetLastError());

  const float ca = 3.4445f, cb = -4.7750f, cc = 2.0315f;  // src/toner/linalg.py:9
  auto op16 = [&](const __nv_bfloat16* base, int rows, int cols, int mn_major) {
    toner_operand op = {};
    op.base = base;
    op.rows = rows; op.cols = cols; op.ld = cols; op.z_stride = (long long)rows * cols; op.nz = batch;
    op.mn_major = mn_major; op.z_step = 1;
    return op;
  };
  for (int s = 0; s < steps; ++s) {
    const __nv_bfloat16* cur = xb[s & 1];
    __nv_bfloat16* nxt = xb[(s + 1) & 1];
    const bool last = (s == steps - 1);
    {  // A = x x^T on the short side (symmetric): FP32 and BF16 copies
      toner_gemm_desc g = {};
      g.a = op16(cur, m, n, wide ? 0 : 1);
      g.b = g.a;
      g.m = a; g.n = a; g.k = wide ? n : m; g.batch = batch; g.segs = 1; g.fmt = 1;
      g.tri = 1; g.mirror = 1; g.alpha = 1.f;
      g.upper_d = 1;  // the FP32 Gram is read back only as the upper-triangle C of the polynomial product below
      g.d = gram; g.ldd = a; g.d_bs = aa;
      g.d16 = gram_b; g.ld16 = a; g.d16_bs = aa; g.d16_fmt = 1;
      rc = launch_gemm(g, stream);
      if (rc) return rc;
    }
    {  // B = b A + c A A, rounded to BF16 for the next product
      toner_gemm_desc g = {};
      g.a = op16(gram_b, a, a, 0);
      g.b = g.a;
      g.m = a; g.n = a; g.k = a; g.batch = batch; g.segs = 1; g.fmt = 1;
      g.tri = 1; g.mirror = 1; g.alpha = cc; g.beta = cb;
      g.c = gram; g.ldc = a; g.c_bs = aa;
      g.d16 = poly_b; g.ld16 = a; g.d16_bs = aa; g.d16_fmt = 1;
      rc = launch_gemm(g, stream);
      if (rc) return rc;
    }
    {  // x <- a x + B x  (wide)   or   x <- a x + x B  (tall)
      toner_gemm_desc g = {};
      if (wide) {
        g.a = op16(poly_b, a, a, 0);
        g.b = op16(cur, m, n, 1);  // B operand indexed [n_index][k]: x stored (k, n_index) is its transposed view
      } else {
        g.a = op16(cur, m, n, 0);
        g.b = op16(poly_b, a, a, 0);  // symmetric: B^T = B
      }
      g.m = m; g.n = n; g.k = a; g.batch = batch; g.segs = 1; g.fmt = 1;
      g.alpha = 1.f; g.beta = ca;
      g.c = x_out; g.ldc = n; g.c_bs = mn;
      g.d = x_out; g.ldd = n; g.d_bs = mn;
      if (!last) {
        g.d16 = nxt; g.ld16 = n; g.d16_bs = mn; g.d16_fmt = 1;
      } else if (maxabs_out) {
        TONER_CUDA(cudaMemsetAsync(maxabs_out, 0, sizeof(uint32_t) * batch, stream));
        g.maxabs = maxabs_out;
      }
      rc = launch_gemm(g, stream);
      if (rc) return rc;
    }
  }
  return 0;
}

int toner_sumsq(const float* x, int32_t batch, int32_t rows, int32_t cols, int64_t ld, int64_t bs, float* scratch,
                float* out, void* stream) {
  if (!context()) return kErrCuda;
  if (!x || !scratch || !out || batch <= 0 || rows <= 0 || cols <= 0) return fail(kErrArg, "sumsq: bad arguments");
  if (ld < cols) return fail(kErrArg, "sumsq: ld (elements between rows) must be at least cols");
  return sumsq_det(x, batch, rows, cols, ld, bs, scratch, out, static_cast<cudaStream_t>(stream));
}

size_t toner_sumsq_scratch_bytes(int32_t batch) { return batch > 0 ? sumsq_scratch_bytes(batch) : 0; }

static int check_stack(const char* what, long long per) {
  if (per <= 0 || per % 4 != 0) return fail(kErrArg, std::string(what) + ": matrix size must be a positive multiple of 4");
  return 0;
}

int toner_muont_momentum(const float* const* grad_ptrs, float* m, float* u, int32_t count, int64_t per, float mu,
                         int32_t nesterov, uint32_t* maxabs, void* stream_) {
  Context* ctx = context();
  if (!ctx) return kErrCuda;
  if (!grad_ptrs || !m || !u || count <= 0) return fail(kErrArg, "muont_momentum: bad arguments");
  if (int rc = check_stack("muont_momentum", per)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (maxabs) TONER_CUDA(cudaMemsetAsync(maxabs, 0, sizeof(uint32_t) * count, stream));
  muont_momentum_kernel<<<dim3(ew_grid(per / 4, ctx->num_sms), count), 256, 0, stream>>>(grad_ptrs, m, u, per, mu, nesterov, maxabs);
  count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

int toner_muont_coeffs(const float* fro2, int32_t first, int32_t step, int32_t count, int32_t n, float lr, float wd,
                       float scale, float* c1, float* c2, void* stream) {
  if (!context()) return kErrCuda;
  if (!fro2 || !c1 || !c2 || count <= 0) return fail(kErrArg, "muont_coeffs: bad arguments");
  muont_coeff_kernel<<<(count + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(fro2, first, step, count, n, lr, wd, scale, c1, c2);
  count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

int toner_scale_vec(float* a, const float* b, int32_t count, void* stream) {
  if (!context()) return kErrCuda;
  if (!a || !b || count <= 0) return fail(kErrArg, "scale_vec: bad arguments");
  mul_vec_kernel2<<<(count + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(a, b, count);
  count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

int toner_adamt_first_moment(const float* const* grad_ptrs, float* m, int32_t count, int64_t per, float beta1, void* stream) {
  Context* ctx = context();
  if (!ctx) return kErrCuda;
  if (!grad_ptrs || !m || count <= 0) return fail(kErrArg, "adamt_first_moment: bad arguments");
  if (int rc = check_stack("adamt_first_moment", per)) return rc;
  adamt_m_kernel<<<dim3(ew_grid(per / 4, ctx->num_sms), count), 256, 0, static_cast<cudaStream_t>(stream)>>>(grad_ptrs, m, per, beta1);
  count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

int toner_adamt_ratio(const float* t, float* v, float* num, int32_t count, int64_t per, float beta2, float bc2, float eps,
                      uint32_t* maxabs, void* stream_) {
  Context* ctx = context();
  if (!ctx) return kErrCuda;
  if (!t || !v || !num || count <= 0) return fail(kErrArg, "adamt_ratio: bad arguments");
  if (int rc = check_stack("adamt_ratio", per)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (maxabs) TONER_CUDA(cudaMemsetAsync(maxabs, 0, sizeof(uint32_t) * count, stream));
  adamt_ratio_kernel<<<dim3(ew_grid(per / 4, ctx->num_sms), count), 256, 0, stream>>>(t, v, num, per, beta2, bc2, eps, maxabs);
  count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

int toner_adamt_coeffs(const float* fro2, int32_t first, int32_t step, int32_t count, int32_t n, float lr, float wd,
                       const float* ss_before, const float* ss_after, float* c1, float* c2, void* stream) {
  if (!context()) return kErrCuda;
  if (!fro2 || !ss_before || !ss_after || !c1 || !c2 || count <= 0) return fail(kErrArg, "adamt_coeffs: bad arguments");
  adamt_coeff_kernel<<<(count + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(fro2, first, step, count, n, lr, wd, ss_before, ss_after, c1, c2);
  count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

int toner_apply_delta(float* const* weight_ptrs, const float* delta, int32_t count, int64_t per, void* stream) {
  Context* ctx = context();
  if (!ctx) return kErrCuda;
  if (!weight_ptrs || !delta || count <= 0) return fail(kErrArg, "apply_delta: bad arguments");
  if (int rc = check_stack("apply_delta", per)) return rc;
  apply_delta_kernel<<<dim3(ew_grid(per / 4, ctx->num_sms), count), 256, 0, static_cast<cudaStream_t>(stream)>>>(weight_ptrs, delta, per);
  count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

int toner_apply_scaled(float* const* weight_ptrs, const float* delta, int32_t count, int64_t per, float weight_scale,
                       float delta_scale, void* stream) {
  Context* ctx = context();
  if (!ctx) return kErrCuda;
  if (!weight_ptrs || !delta || count <= 0) return fail(kErrArg, "apply_scaled: bad arguments");
  if (int rc = check_stack("apply_scaled", per)) return rc;
  apply_scaled_kernel<<<dim3(ew_grid(per / 4, ctx->num_sms), count), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      weight_ptrs, delta, per, weight_scale, delta_scale);
  count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

}  // extern "C"

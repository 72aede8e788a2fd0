// Statistic path: upper-triangle SYRK (on the tcgen05 GEMM), packed-triangle EMA, FP16 hi/lo splitting.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "runtime.cuh"

namespace toner {

// ------------------------------------------------------------------ packed triangle -> full EMA
// One 32x32 tile pair per block: the upper tile is updated in place from the packed triangle, the lower
// tile is its transpose written through shared memory, so every global access is row-contiguous.  Only the
// tiles that meet the upper triangle are launched (blockIdx.x counts them row by row), and a thread's four
// elements are all loaded before the first is stored.
__global__ void __launch_bounds__(256) unpack_ema_kernel(const float* __restrict__ packed, float* __restrict__ ema, int n,
                                                         int tiles, float beta, float gamma) {
  // tile (ti, tj), ti <= tj, from the running index: row ti holds tiles - ti of them
  // (rows 0 .. ti-1 hold ti * tiles - ti (ti - 1) / 2 tiles: solve for ti, then correct the rounding)
  const int idx = blockIdx.x;
  const float w = 2.f * tiles + 1.f;
  int ti = (int)((w - sqrtf(fmaxf(w * w - 8.f * idx, 0.f))) * 0.5f);
  ti = min(max(ti, 0), tiles - 1);
  while (ti > 0 && ti * tiles - ti * (ti - 1) / 2 > idx) --ti;
  while ((ti + 1) * tiles - (ti + 1) * ti / 2 <= idx) ++ti;
  const int tj = ti + (idx - (ti * tiles - ti * (ti - 1) / 2));
  __shared__ float tile[32][33];
  const long long b = blockIdx.z;
  const float* P = packed + b * ((long long)n * (n + 1) / 2);
  float* C = ema + b * (long long)n * n;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = tj * 32 + tx;
  float s[4], old[4];
  bool on[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ti * 32 + ty + 8 * i;
    on[i] = r < n && c < n && r <= c;
    s[i] = on[i] ? P[packed_off(r, c, n)] : 0.f;
    old[i] = on[i] ? C[(long long)r * n + c] : 0.f;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int lr = ty + 8 * i;
    const int r = ti * 32 + lr;
    float v = 0.f;
    if (on[i]) {
      v = fmaf(beta, old[i], gamma * s[i]);
      C[(long long)r * n + c] = v;
    }
    tile[lr][tx] = v;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int lr = ty + 8 * i;
    const int r = tj * 32 + lr, cc = ti * 32 + tx;  // element of the lower triangle, value from (cc, r)
    if (r < n && cc < n && r > cc) C[(long long)r * n + cc] = tile[tx][lr];
  }
}

// ------------------------------------------------------------------ sampled-row capture
// dst[(b * count + j), :] = bf16(x[b, positions[j], :]): the rows of the sampled token positions of one microbatch,
// written straight into the statistic's row buffer.  One warp per row, 16-byte accesses.
template <typename T>
__global__ void __launch_bounds__(256) gather_rows_kernel(const T* __restrict__ x, long long batch_stride, long long row_stride,
                                                          const int* __restrict__ positions, int count, int n, int rows_total,
                                                          __nv_bfloat16* __restrict__ dst) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows_total) return;
  const int b = row / count, j = row - b * count;
  const T* src = x + (long long)b * batch_stride + (long long)positions[j] * row_stride;
  __nv_bfloat16* out = dst + (long long)row * n;
  for (int c = lane * 8; c < n; c += 256) {
    if constexpr (sizeof(T) == 2) {
      *reinterpret_cast<uint4*>(out + c) = *reinterpret_cast<const uint4*>(src + c);
    } else {
      const float4 lo = *reinterpret_cast<const float4*>(src + c), hi = *reinterpret_cast<const float4*>(src + c + 4);
      __nv_bfloat162 p0 = __floats2bfloat162_rn(lo.x, lo.y), p1 = __floats2bfloat162_rn(lo.z, lo.w);
      __nv_bfloat162 p2 = __floats2bfloat162_rn(hi.x, hi.y), p3 = __floats2bfloat162_rn(hi.z, hi.w);
      uint4 u;
      u.x = *reinterpret_cast<uint32_t*>(&p0); u.y = *reinterpret_cast<uint32_t*>(&p1);
      u.z = *reinterpret_cast<uint32_t*>(&p2); u.w = *reinterpret_cast<uint32_t*>(&p3);
      *reinterpret_cast<uint4*>(out + c) = u;
    }
  }
}

// ------------------------------------------------------------------ max |aff_a*I + aff_b*x| per matrix
__global__ void __launch_bounds__(256) maxabs_kernel(const float* __restrict__ x, const float* const* __restrict__ x_list,
                                                     int rows, int cols, long long ld, long long bs, float aff_a,
                                                     float aff_b, unsigned int* __restrict__ out) {
  const int b = blockIdx.y;
  const float* X = x_list ? x_list[b] : x + (long long)b * bs;
  float m = 0.f;
  const bool vec = (cols % 4 == 0) && (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(X) & 15u) == 0);
  if (vec) {
    const int c4 = cols / 4;
    const long long total4 = (long long)rows * c4;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total4; i += (long long)gridDim.x * blockDim.x) {
      const int r = (int)(i / c4), c = (int)(i - (long long)r * c4) * 4;
      const float4 q = *reinterpret_cast<const float4*>(X + (long long)r * ld + c);
      const float v[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) m = fmaxf(m, fabsf(fmaf(aff_b, v[e], (c + e) == r ? aff_a : 0.f)));
    }
  } else {
    const long long total = (long long)rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
      const int r = (int)(i / cols), c = (int)(i - (long long)r * cols);
      m = fmaxf(m, fabsf(fmaf(aff_b, X[(long long)r * ld + c], r == c ? aff_a : 0.f)));
    }
  }
  block_atomic_max(m, out + b);
}

// scale = 2^(13 - floor(log2 maxabs)); 1 when the matrix is all zero or its maximum is not finite
__device__ __forceinline__ float split_scale(unsigned int maxabs_bits) {
  const float a = __uint_as_float(maxabs_bits);
  if (!(a > 0.f) || !isfinite(a)) return 1.f;
  int e;
  frexpf(a, &e);  // a = f * 2^e, f in [0.5, 1)  =>  floor(log2 a) = e - 1
  return ldexpf(1.f, 13 - (e - 1));
}

__global__ void __launch_bounds__(256) split16_kernel(const float* __restrict__ x, const float* const* __restrict__ x_list,
                                                      int batch, int rows, int cols, long long ld, long long bs,
                                                      float aff_a, float aff_b, const unsigned int* __restrict__ maxabs,
                                                      __half* __restrict__ planes, float* __restrict__ inv_scale) {
  const int b = blockIdx.y;
  const float* X = x_list ? x_list[b] : x + (long long)b * bs;
  const float s = split_scale(maxabs[b]);
  if (blockIdx.x == 0 && threadIdx.x == 0 && inv_scale) inv_scale[b] = 1.f / s;
  const long long per = (long long)rows * cols;
  __half* hi = planes + (long long)b * per;
  __half* lo = planes + ((long long)batch + b) * per;
  const bool vec = (cols % 4 == 0) && (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(X) & 15u) == 0);
  if (vec) {
    const long long total4 = per / 4;
    const int c4 = cols / 4;
    auto split4 = [&](long long i, const float4 q) {
      const int r = (int)(i / c4), c = (int)(i - (long long)r * c4) * 4;
      const float v[4] = {q.x, q.y, q.z, q.w};
      __half h[4], l[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float w = (aff_b * v[e] + ((c + e) == r ? aff_a : 0.f)) * s;
        h[e] = __float2half_rn(w);
        l[e] = __float2half_rn(w - __half2float(h[e]));
      }
      *reinterpret_cast<uint2*>(hi + (long long)r * cols + c) = *reinterpret_cast<uint2*>(h);
      *reinterpret_cast<uint2*>(lo + (long long)r * cols + c) = *reinterpret_cast<uint2*>(l);
    };
    auto load4 = [&](long long i) {
      const int r = (int)(i / c4), c = (int)(i - (long long)r * c4) * 4;
      return *reinterpret_cast<const float4*>(X + (long long)r * ld + c);
    };
    // four independent 16-byte loads in flight per thread before the first store
    const long long step = (long long)gridDim.x * blockDim.x;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * step < total4; i += 4 * step) {
      const float4 q0 = load4(i), q1 = load4(i + step), q2 = load4(i + 2 * step), q3 = load4(i + 3 * step);
      split4(i, q0); split4(i + step, q1); split4(i + 2 * step, q2); split4(i + 3 * step, q3);
    }
    for (; i < total4; i += step) split4(i, load4(i));
  } else {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per; i += (long long)gridDim.x * blockDim.x) {
      const int r = (int)(i / cols), c = (int)(i - (long long)r * cols);
      const float w = (aff_b * X[(long long)r * ld + c] + (c == r ? aff_a : 0.f)) * s;
      const __half h = __float2half_rn(w);
      hi[i] = h;
      lo[i] = __float2half_rn(w - __half2float(h));
    }
  }
}

// ------------------------------------------------------------------ deterministic sum of squares
// Fixed grid, fixed reduction tree: the same input always gives the same bits (float atomics would not).
constexpr int kSumsqBlocks = 296;  // two per SM on a 148-SM part; fixed so that results do not depend on the device

__global__ void __launch_bounds__(256) sumsq_partial_kernel(const float* __restrict__ x, int rows, int cols, long long ld,
                                                            long long bs, float* __restrict__ partial) {
  const int b = blockIdx.y;
  const float* X = x + (long long)b * bs;
  const long long total = (long long)rows * cols;
  float s = 0.f;
  if (ld == cols && total % 4 == 0 && (reinterpret_cast<uintptr_t>(X) & 15u) == 0) {
    // contiguous matrix: 16-byte loads, four running sums per thread, combined in a fixed order
    const long long total4 = total / 4;
    const long long per = (total4 + gridDim.x - 1) / gridDim.x;
    const long long lo = per * blockIdx.x, hi = (lo + per < total4) ? lo + per : total4;
    const float4* X4 = reinterpret_cast<const float4*>(X);
    // four independent 16-byte loads in flight per thread; the order of the additions is fixed by the indices alone,
    // so the result stays bitwise reproducible
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    long long i = lo + threadIdx.x;
    const long long step = blockDim.x;
    for (; i + 3 * step < hi; i += 4 * step) {
      const float4 a = X4[i], b = X4[i + step], c = X4[i + 2 * step], d = X4[i + 3 * step];
      s0 = fmaf(a.x, a.x, s0); s1 = fmaf(a.y, a.y, s1); s2 = fmaf(a.z, a.z, s2); s3 = fmaf(a.w, a.w, s3);
      s0 = fmaf(b.x, b.x, s0); s1 = fmaf(b.y, b.y, s1); s2 = fmaf(b.z, b.z, s2); s3 = fmaf(b.w, b.w, s3);
      s0 = fmaf(c.x, c.x, s0); s1 = fmaf(c.y, c.y, s1); s2 = fmaf(c.z, c.z, s2); s3 = fmaf(c.w, c.w, s3);
      s0 = fmaf(d.x, d.x, s0); s1 = fmaf(d.y, d.y, s1); s2 = fmaf(d.z, d.z, s2); s3 = fmaf(d.w, d.w, s3);
    }
    for (; i < hi; i += step) {
      const float4 v = X4[i];
      s0 = fmaf(v.x, v.x, s0); s1 = fmaf(v.y, v.y, s1); s2 = fmaf(v.z, v.z, s2); s3 = fmaf(v.w, v.w, s3);
    }
    s = (s0 + s1) + (s2 + s3);
  } else {
    const long long per = (total + gridDim.x - 1) / gridDim.x;
    const long long lo = per * blockIdx.x, hi = (lo + per < total) ? lo + per : total;
    for (long long i = lo + threadIdx.x; i < hi; i += blockDim.x) {
      const long long r = i / cols, c = i - r * cols;
      const float v = X[r * ld + c];
      s = fmaf(v, v, s);
    }
  }
  __shared__ float red[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    partial[(long long)b * gridDim.x + blockIdx.x] = t;
  }
}

__global__ void sumsq_final_kernel(const float* __restrict__ partial, int blocks, int batch, float* __restrict__ out) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  float t = 0.f;
  for (int i = 0; i < blocks; ++i) t += partial[(long long)b * blocks + i];
  out[b] = t;
}

size_t sumsq_scratch_bytes(int batch) { return (size_t)batch * kSumsqBlocks * sizeof(float); }

int sumsq_det(const float* x, int batch, int rows, int cols, long long ld, long long bs, float* scratch, float* out,
              cudaStream_t stream) {
  sumsq_partial_kernel<<<dim3(kSumsqBlocks, batch), 256, 0, stream>>>(x, rows, cols, ld, bs, scratch);
  count_launch();
  sumsq_final_kernel<<<(batch + 127) / 128, 128, 0, stream>>>(scratch, kSumsqBlocks, batch, out);
  count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------ sum of squares without caller scratch
// Partial sums of toner_sumsq_static live here instead of in a caller-provided buffer.  The array belongs to
// the library image: every device that loads the library holds these 296 KB until the process exits.
constexpr int kStaticSumsqMaxBatch = 256;
static __device__ __align__(256) float g_sumsq_static_scratch[kStaticSumsqMaxBatch * kSumsqBlocks];

// In host code the array's name is only a handle for the runtime, not an address a kernel can use: the
// device address is looked up once per device (with that device current) and remembered.
static float* g_sumsq_static_ptr[64] = {};
static std::mutex g_sumsq_static_mutex;

static int sumsq_static_scratch(float** out) {
  int dev = -1;
  TONER_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(kErrCuda, "sumsq_static: unexpected device ordinal");
  std::lock_guard<std::mutex> lock(g_sumsq_static_mutex);
  if (!g_sumsq_static_ptr[dev]) {
    int major = 0;
    TONER_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) return fail(kErrUnsupported, "sumsq_static: the kernels are built for sm_100a only");
    void* ptr = nullptr;
    TONER_CUDA(cudaGetSymbolAddress(&ptr, g_sumsq_static_scratch));
    if (!ptr) return fail(kErrCuda, "sumsq_static: the scratch array has no device address");
    g_sumsq_static_ptr[dev] = static_cast<float*>(ptr);
  }
  *out = g_sumsq_static_ptr[dev];
  return 0;
}

static int blocks_for(long long work, int per_block, int cap) {
  long long b = (work + per_block - 1) / per_block;
  if (b < 1) b = 1;
  if (b > cap) b = cap;
  return (int)b;
}

int split16(const float* x, const float* const* x_list, int batch, int rows, int cols, long long ld, long long bs,
            float aff_a, float aff_b, const uint32_t* maxabs, void* scratch, void* planes, float* inv_scale,
            cudaStream_t stream) {
  Context* ctx = context();
  if (!ctx) return kErrCuda;
  if ((!x && !x_list) || !planes || batch <= 0 || rows <= 0 || cols <= 0) return fail(kErrArg, "split16: bad arguments");
  if (cols % 8 != 0) return fail(kErrArg, "split16: cols must be a multiple of 8 (TMA row pitch)");
  const long long per = (long long)rows * cols;
  const int bx = blocks_for(per / 4 + 1, 256 * 4, 8 * ctx->num_sms / (batch < 8 ? batch : 8) + 1);
  if (!maxabs) {
    if (!scratch) return fail(kErrArg, "split16: maxabs or scratch is required");
    unsigned int* m = static_cast<unsigned int*>(scratch);
    TONER_CUDA(cudaMemsetAsync(m, 0, sizeof(unsigned int) * batch, stream));
    maxabs_kernel<<<dim3(bx, batch), 256, 0, stream>>>(x, x_list, rows, cols, ld, bs, aff_a, aff_b, m);
    count_launch();
    TONER_CUDA(cudaGetLastError());
    maxabs = m;
  }
  split16_kernel<<<dim3(bx, batch), 256, 0, stream>>>(x, x_list, batch, rows, cols, ld, bs, aff_a, aff_b, maxabs,
                                                     static_cast<__half*>(planes), inv_scale);
  count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace toner

extern "C" {

int toner_syrk_upper(const void* const* x_list, const void* x_base, int64_t x_batch_stride, int32_t k, int32_t rows,
                     int32_t n, int64_t ld, float* out, int32_t mode, float beta, float gamma, void* stream) {
  using namespace toner;
  if ((!x_list && !x_base) || !out) return fail(kErrArg, "syrk: null pointer");
  if (k <= 0 || rows <= 0 || n <= 0) return fail(kErrArg, "syrk: sizes must be positive");
  if (n % 8 != 0 || ld % 8 != 0) return fail(kErrArg, "syrk: n and ld must be multiples of 8");
  if (mode < 0 || mode > 2) return fail(kErrArg, "syrk: mode must be 0 (PACKED), 1 (PACKED_ACC) or 2 (EMA_FULL)");
  toner_gemm_desc d = {};
  toner_operand op = {};
  op.base = x_base;
  op.list = x_list;
  op.rows = rows;
  op.cols = n;
  op.ld = ld;
  op.z_stride = x_batch_stride;
  op.nz = x_list ? 1 : k;
  op.z_step = 1;
  op.mn_major = 1;  // the buffer is (rows = k-index) x (n = m/n-index): X^T X reads it transposed on both sides
  d.a = op;
  d.b = op;
  d.m = n; d.n = n; d.k = rows; d.batch = k;
  d.segs = 1;
  d.fmt = 1;
  d.tri = 1;
  // The tensor core adds into its accumulator by truncation; over tens of thousands of rows the all-positive
  // sums of the diagonal would drift low by 1e-4.  Chains of 4096 rows, summed with rounding, bound it by 1.5e-5
  // (two such chains also outlast the epilogue of the previous tile, so the tensor core never waits for it).
  d.promote = rows > 4096 ? 64 : 0;
  const long long tri_elems = (long long)n * (n + 1) / 2;
  if (mode == 2) {
    d.mirror = 1;
    d.alpha = gamma; d.beta = beta;
    d.c = out; d.ldc = n; d.c_bs = (long long)n * n;
    d.d = out; d.ldd = n; d.d_bs = (long long)n * n;
  } else {
    d.packed = 1;
    d.alpha = 1.f;
    d.d = out; d.ldd = n; d.d_bs = tri_elems;
    if (mode == 1) {
      d.beta = 1.f;
      d.c = out; d.ldc = n; d.c_bs = tri_elems;
    }
  }
  return launch_gemm(d, static_cast<cudaStream_t>(stream));
}

int toner_gather_rows(const void* x, int32_t x_is_fp32, int32_t batch, int32_t seq, int32_t n, int64_t batch_stride,
                      int64_t row_stride, const int32_t* positions, int32_t count, void* dst, void* stream) {
  using namespace toner;
  if (!context()) return kErrCuda;
  if (!x || !positions || !dst || batch <= 0 || seq <= 0 || n <= 0 || count <= 0) return fail(kErrArg, "gather_rows: bad arguments");
  const int elt = x_is_fp32 ? 4 : 2;
  if (n % 8 != 0 || (row_stride * elt) % 16 != 0 || (batch_stride * elt) % 16 != 0 ||
      (reinterpret_cast<uintptr_t>(x) & 15u) != 0 || (reinterpret_cast<uintptr_t>(dst) & 15u) != 0)
    return fail(kErrArg, "gather_rows: rows must be 16-byte aligned and n a multiple of 8");
  const long long rows = (long long)batch * count;
  if (rows > 0x7fffffffLL) return fail(kErrArg, "gather_rows: too many rows");
  const int blocks = (int)((rows + 7) / 8);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (x_is_fp32)
    gather_rows_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const float*>(x), batch_stride, row_stride, positions, count, n,
                                                     (int)rows, static_cast<__nv_bfloat16*>(dst));
  else
    gather_rows_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), batch_stride, row_stride,
                                                             positions, count, n, (int)rows, static_cast<__nv_bfloat16*>(dst));
  count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

int toner_sumsq_static_max_batch(void) { return toner::kStaticSumsqMaxBatch; }

int toner_sumsq_static(const float* x, int32_t batch, int32_t rows, int32_t cols, int64_t ld, int64_t bs, float* out,
                       void* stream) {
  using namespace toner;
  if (!x || !out || batch <= 0 || rows <= 0 || cols <= 0) return fail(kErrArg, "sumsq_static: bad arguments");
  if (ld < cols) return fail(kErrArg, "sumsq_static: ld (elements between rows) must be at least cols");
  if (batch > kStaticSumsqMaxBatch)
    return fail(kErrArg, "sumsq_static: batch " + std::to_string(batch) + " exceeds the built-in scratch (" +
                             std::to_string(kStaticSumsqMaxBatch) + " matrices); use toner_sumsq with caller scratch");
  float* scratch = nullptr;
  if (int rc = sumsq_static_scratch(&scratch)) return rc;
  // Every partial sum the second kernel reads is written by the first one in this call, so nothing left in
  // the array by an earlier call needs clearing.
  return sumsq_det(x, batch, rows, cols, ld, bs, scratch, out, static_cast<cudaStream_t>(stream));
}

int toner_unpack_ema(const float* packed, float* ema, int32_t k, int32_t n, float beta, float gamma, void* stream) {
  using namespace toner;
  if (!context()) return kErrCuda;
  if (!packed || !ema || k <= 0 || n <= 0) return fail(kErrArg, "unpack_ema: bad arguments");
  const int t = (n + 31) / 32;
  if (k > 65535) return fail(kErrArg, "unpack_ema: k too large");
  unpack_ema_kernel<<<dim3(t * (t + 1) / 2, 1, k), 256, 0, static_cast<cudaStream_t>(stream)>>>(packed, ema, n, t, beta, gamma);
  count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

int toner_split16(const float* x, const float* const* x_list, int32_t batch, int32_t rows, int32_t cols, int64_t ld,
                  int64_t bs, float aff_a, float aff_b, const uint32_t* maxabs, void* scratch, void* planes,
                  float* inv_scale, void* stream) {
  return toner::split16(x, x_list, batch, rows, cols, ld, bs, aff_a, aff_b, maxabs, scratch, planes, inv_scale,
                        static_cast<cudaStream_t>(stream));
}

}  // extern "C"

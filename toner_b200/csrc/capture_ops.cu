// Row capture: the sampled rows of a micro-batch's activations written straight into the statistics' row buffers,
// either copied or recomputed from what the forward pass keeps anyway (the RMSNorm input and weight; the gate and up
// projections), so that the normalised / gated activations never have to be kept for the optimizer.
//
// One launch serves every layer and every kind of row: the host describes the work as a table of jobs (source
// pointers, destination buffer, width, strides, kind); job j, sampled row r = b * P + p reads position idx[p] of
// sequence b and writes row at[r] of the job's buffer.  Each row is handled by one warp with 16-byte accesses; the
// work is HBM-bound (2 B read + 2 B written per element, 4 B read for the gated kind).
//
// Arithmetic, chosen to reproduce what the model computes in its forward pass:
//   kind 0  copy
//   kind 1  out = bf16(x * rsqrt(mean(x^2) + eps));  row = bf16(float(bf16(w)) * float(out))      (x BF16, w FP32)
//   kind 2  row = bf16(g * (1 / (1 + exp(-g))) * u)   in FP32 with one rounding                    (g, u BF16)
//   kind 3  row = bf16(a)                              the source is FP32 (what autocast would round)
#include <cuda_bf16.h>

#include "runtime.cuh"

namespace toner {

struct alignas(16) Bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ Bf16x8 load8(const __nv_bfloat16* p) {
  Bf16x8 r;
  *reinterpret_cast<uint4*>(&r) = __ldg(reinterpret_cast<const uint4*>(p));
  return r;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const Bf16x8& r) {
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}

constexpr int kCaptureWarps = 8;  // rows per block

__global__ void __launch_bounds__(32 * kCaptureWarps) capture_rows_kernel(const toner_capture_job* __restrict__ jobs,
                                                                          const long long* __restrict__ at,
                                                                          const long long* __restrict__ idx, int rows, int P,
                                                                          float eps) {
  const int lane = threadIdx.x & 31;
  const int r = blockIdx.x * kCaptureWarps + (threadIdx.x >> 5);
  if (r >= rows) return;
  const toner_capture_job job = jobs[blockIdx.y];
  const int D = job.width;
  const long long off = (long long)(r / P) * job.batch_stride + __ldg(idx + r % P) * job.row_stride;
  const __nv_bfloat16* a = static_cast<const __nv_bfloat16*>(job.a) + off;
  __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(job.dst) + __ldg(at + r) * (long long)D;

  if (job.kind == TONER_CAPTURE_COPY_F32) {
    const float* af = static_cast<const float*>(job.a) + off;
    for (int c = 8 * lane; c < D; c += 256) {
      const float4 lo = __ldg(reinterpret_cast<const float4*>(af + c)), hi = __ldg(reinterpret_cast<const float4*>(af + c + 4));
      Bf16x8 y;
      y.v[0] = __floats2bfloat162_rn(lo.x, lo.y); y.v[1] = __floats2bfloat162_rn(lo.z, lo.w);
      y.v[2] = __floats2bfloat162_rn(hi.x, hi.y); y.v[3] = __floats2bfloat162_rn(hi.z, hi.w);
      store8(dst + c, y);
    }
  } else if (job.kind == TONER_CAPTURE_COPY) {
    int c = 8 * lane;
    for (; c + 768 < D; c += 1024) {  // four independent 16-byte loads in flight per lane
      const Bf16x8 x0 = load8(a + c), x1 = load8(a + c + 256), x2 = load8(a + c + 512), x3 = load8(a + c + 768);
      store8(dst + c, x0); store8(dst + c + 256, x1); store8(dst + c + 512, x2); store8(dst + c + 768, x3);
    }
    for (; c < D; c += 256) store8(dst + c, load8(a + c));
  } else if (job.kind == TONER_CAPTURE_RMSNORM) {
    // two passes over the row; the second finds it in L1 (a row is a few KB)
    float ss = 0.f;
    auto square8 = [&ss](const Bf16x8& x) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(x.v[i]);
        ss = fmaf(f.x, f.x, ss);
        ss = fmaf(f.y, f.y, ss);
      }
    };
    int c1 = 8 * lane;
    for (; c1 + 768 < D; c1 += 1024) {
      const Bf16x8 x0 = load8(a + c1), x1 = load8(a + c1 + 256), x2 = load8(a + c1 + 512), x3 = load8(a + c1 + 768);
      square8(x0); square8(x1); square8(x2); square8(x3);
    }
    for (; c1 < D; c1 += 256) square8(load8(a + c1));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float scale = 1.0f / sqrtf(ss / (float)D + eps);
    const float* w = static_cast<const float*>(job.b);
    for (int c = 8 * lane; c < D; c += 256) {
      const Bf16x8 x = load8(a + c);
      const float4 w0 = __ldg(reinterpret_cast<const float4*>(w + c));
      const float4 w1 = __ldg(reinterpret_cast<const float4*>(w + c + 4));
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      Bf16x8 y;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(x.v[i]);
        const float o0 = __bfloat162float(__float2bfloat16_rn(f.x * scale));
        const float o1 = __bfloat162float(__float2bfloat16_rn(f.y * scale));
        const float h0 = __bfloat162float(__float2bfloat16_rn(wv[2 * i])) * o0;
        const float h1 = __bfloat162float(__float2bfloat16_rn(wv[2 * i + 1])) * o1;
        y.v[i] = __halves2bfloat162(__float2bfloat16_rn(h0), __float2bfloat16_rn(h1));
      }
      store8(dst + c, y);
    }
  } else {  // TONER_CAPTURE_SILU_MUL
    const __nv_bfloat16* u = static_cast<const __nv_bfloat16*>(job.b) + off;
    auto gated8 = [](const Bf16x8& g, const Bf16x8& uu) {
      Bf16x8 y;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 gf = __bfloat1622float2(g.v[i]), uf = __bfloat1622float2(uu.v[i]);
        const float h0 = gf.x * (1.0f / (1.0f + expf(-gf.x))) * uf.x;
        const float h1 = gf.y * (1.0f / (1.0f + expf(-gf.y))) * uf.y;
        y.v[i] = __halves2bfloat162(__float2bfloat16_rn(h0), __float2bfloat16_rn(h1));
      }
      return y;
    };
    int c = 8 * lane;
    for (; c + 256 < D; c += 512) {  // four independent 16-byte loads in flight per lane
      const Bf16x8 g0 = load8(a + c), u0 = load8(u + c), g1 = load8(a + c + 256), u1 = load8(u + c + 256);
      store8(dst + c, gated8(g0, u0));
      store8(dst + c + 256, gated8(g1, u1));
    }
    for (; c < D; c += 256) store8(dst + c, gated8(load8(a + c), load8(u + c)));
  }
}

}  // namespace toner

extern "C" int toner_capture(const toner_capture_job* jobs_device, const toner_capture_job* jobs_host, int32_t n_jobs,
                             const int64_t* at, const int64_t* idx, int32_t batch, int32_t positions, float eps,
                             void* stream_) {
  using namespace toner;
  Context* ctx = context();
  if (!ctx) return kErrCuda;
  if (!jobs_device || !jobs_host || !at || !idx) return fail(kErrArg, "capture: null pointer");
  if (n_jobs <= 0 || n_jobs > 65535) return fail(kErrArg, "capture: between 1 and 65535 jobs per call");
  if (batch <= 0 || positions <= 0) return fail(kErrArg, "capture: sizes must be positive");
  const long long rows = (long long)batch * positions;
  if (rows > (1LL << 30)) return fail(kErrArg, "capture: too many rows");
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  for (int j = 0; j < n_jobs; ++j) {
    const toner_capture_job& q = jobs_host[j];
    if (q.kind < TONER_CAPTURE_COPY || q.kind > TONER_CAPTURE_COPY_F32) return fail(kErrArg, "capture: unknown kind");
    const bool copies = q.kind == TONER_CAPTURE_COPY || q.kind == TONER_CAPTURE_COPY_F32;
    if (!q.a || !q.dst || (!copies && !q.b)) return fail(kErrArg, "capture: null pointer in a job");
    if (q.width <= 0 || q.width % 8 || q.batch_stride % 8 || q.row_stride % 8)
      return fail(kErrUnsupported, "capture: width and strides must be multiples of 8 elements");
    if (!al16(q.a) || !al16(q.dst) || (q.b && !al16(q.b))) return fail(kErrUnsupported, "capture: pointers must be 16-byte aligned");
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const dim3 grid((unsigned)((rows + kCaptureWarps - 1) / kCaptureWarps), (unsigned)n_jobs);
  capture_rows_kernel<<<grid, 32 * kCaptureWarps, 0, stream>>>(jobs_device, reinterpret_cast<const long long*>(at),
                                                             reinterpret_cast<const long long*>(idx), (int)rows, positions, eps);
  count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

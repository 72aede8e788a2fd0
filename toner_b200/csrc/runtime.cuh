// Host runtime shared by the C-ABI entry points: per-device context, tensor-map cache, GEMM launcher.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/toner_b200.h"
#include "gemm_tcgen05.cuh"

namespace toner {

// Return codes of the C-ABI (0 = ok, > 0 = host-side argument / runtime error).
enum : int {
  kErrArg = 1,         // null / misaligned pointer, bad size
  kErrCuda = 2,        // a CUDA runtime call failed (see toner_last_error)
  kErrDriver = 3,      // cuTensorMapEncodeTiled unavailable or failed
  kErrWorkspace = 4,   // caller-provided workspace too small
  kErrUnsupported = 5  // shape or option outside what the kernels cover
};

void set_error(const std::string& msg);
int fail(int code, const std::string& msg);

#define TONER_CUDA(expr)                                                                         \
  do {                                                                                           \
    cudaError_t err__ = (expr);                                                                  \
    if (err__ != cudaSuccess)                                                                    \
      return ::toner::fail(::toner::kErrCuda, std::string(#expr) + ": " + cudaGetErrorString(err__)); \
  } while (0)

struct Context {
  int device = -1;
  int num_sms = 0;
  int gemm_sms = 0;  // CTAs the persistent GEMM may occupy (toner_set_gemm_sm_limit)
  int gemm_wide_k = 16384;  // accumulation depth (k x segments) from which 256 x 512 tiles are chosen; 0: never
  CUtensorMap* arena_dev = nullptr;   // tensor maps live here; slots are never rewritten between resets
  CUtensorMap* arena_host = nullptr;  // pinned mirror used as the copy source
  int arena_cap = 0, arena_used = 0;
  int* status_dev = nullptr;          // set by a kernel whose bounded wait ran out
  unsigned long long* prof_dev = nullptr;  // eight cycle counters, allocated when phase profiling is switched on
  void* map_cache = nullptr;          // operand description -> arena slot and upload event (runtime.cu)
};

// Number of kernels this library has launched (all devices, all streams).
void count_launch(int n = 1);

// Context of the current device (created on first use).  Returns nullptr and sets the error on failure.
Context* context();

// Device pointer to `count` consecutive tensor maps describing `op` (one per batch when op.list is
// given, else one).  box_rows is the outer box extent for K-major operands (tile rows); MN-major
// operands always use 64 x 64 boxes.
int get_maps(Context* ctx, const toner_operand& op, int batch, int box_rows, cudaStream_t stream, const CUtensorMap** out);

int launch_gemm(const toner_gemm_desc& d, cudaStream_t stream);

// FP16 hi/lo split of an FP32 stack (see toner_split16).
int split16(const float* x, const float* const* x_list, int batch, int rows, int cols, long long ld, long long bs,
            float aff_a, float aff_b, const uint32_t* maxabs, void* scratch, void* planes, float* inv_scale,
            cudaStream_t stream);

// out[b] = sum of squares of matrix b, bitwise reproducible.  scratch: sumsq_scratch_bytes(batch).
size_t sumsq_scratch_bytes(int batch);
int sumsq_det(const float* x, int batch, int rows, int cols, long long ld, long long bs, float* scratch, float* out,
              cudaStream_t stream);

// Block-wide max of non-negative values into one FP32-bits accumulator: one atomic per block, and none when the
// accumulator already holds as much (thousands of blocks share a few addresses; per-warp atomics serialise in L2).
// Every thread of a 256-thread block calls this.
__device__ __forceinline__ void block_atomic_max(float v, unsigned int* acc) {
  __shared__ float warp_max[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = warp_max[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) m = fmaxf(m, warp_max[w]);
    const unsigned int bits = __float_as_uint(m);
    if (bits > *reinterpret_cast<volatile unsigned int*>(acc)) atomicMax(acc, bits);
  }
}

// k-blocks per accumulation chain used for FP32-accurate (split-precision) products
constexpr int kPromoteAccurate = 2;
// chain length where a relative error of 1e-6 only propagates linearly (products applied to X, W, gradients)
constexpr int kPromoteLinear = 8;

}  // namespace toner

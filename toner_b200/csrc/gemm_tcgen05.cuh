// Batched 16-bit-operand GEMM with FP32 accumulation in tensor memory, for sm_100a.
//
//   D[b] = alpha_b * sum_seg A_seg[b] * B_seg[b]^T   (+ beta_b * C[b])
//
// One persistent CTA per SM (or one CTA pair per SM pair: cta_group::2, 256 x 256 or 256 x 512 tiles), warp-specialised:
//   warp 0      TMA producer: 128-byte-swizzled operand tiles into a shared-memory ring
//   warp 1      allocates tensor memory and issues tcgen05.mma (one thread), accumulating in TMEM
//   warps 4..11 epilogue: tcgen05.ld the accumulator (double-buffered, so it overlaps the next chain's
//               MMAs), sum chains in registers, apply the affine epilogue, store FP32 / 16-bit results
// The tensor core adds every 16-deep partial sum into its FP32 accumulator by truncation; over long K
// that bias reaches 1e-5 relative.  Where FP32 accuracy matters (`promote`), accumulation chains are
// kept short in TMEM and summed with round-to-nearest by the epilogue warps.
// Operands may be stored K-major (k contiguous) or MN-major (m or n contiguous: a transposed view, as
// in X^T X); symmetric results can be computed from the tiles that meet the upper triangle only and
// mirrored on store.  "Segments" concatenate several operand planes along K into one accumulator,
// which is how the FP32-accurate product  Ah*Bh + Ah*Bl + Al*Bh  of FP16 hi/lo splits is formed.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace toner {

constexpr int kBM = 128;          // tile rows (UMMA M)
constexpr int kBK = 64;           // 16-bit elements per k-block: one 128-byte swizzle row
constexpr int kUmmaK = 16;        // K per tcgen05.mma for 16-bit operands
constexpr int kMaxSegs = 3;
constexpr int kGemmThreads = 384;      // warpgroup 0: TMA warp, MMA warp, two idle; warpgroups 1-2: epilogue
constexpr long long kWaitCycles = 4000000000LL;  // about two seconds; a healthy wait is microseconds
constexpr long long kDrainCycles = 2000000LL;    // per stage, after an abort: about a millisecond for copies in flight
constexpr long long kSettleCycles = 200000LL;    // after an abort: a CTA of a pair lets copies it cannot observe land

enum GemmStatus : int { kOk = 0, kTimeoutProducer = 101, kTimeoutMma = 102, kTimeoutEpilogue = 103, kTimeoutSelftest = 199 };

struct GemmParams {
  // operands: arrays of 3-D tensor maps (inner, outer, z) in global memory
  const CUtensorMap* a_maps;
  const CUtensorMap* b_maps;
  int a_map_stride, b_map_stride;  // map index   = batch * map_stride
  int a_z_stride, b_z_stride;      // z coordinate = batch * z_stride + seg_z[seg]
  int a_mn, b_mn;                  // 1: stored MN-major (outer index is k), 0: K-major (outer index is m / n)
  int a_seg_z[kMaxSegs], b_seg_z[kMaxSegs];
  int segs;
  int M, N, K, batch;
  int fmt;  // operand format: 0 FP16, 1 BF16
  int tri;  // 1: M == N, only tiles meeting the upper triangle are computed
  int promote;  // > 0: k-blocks per tensor-core accumulation chain; chains are summed in FP32 registers
  int promote_all;  // 0: only the first segment is chained (split products); 1: every segment
  int raster;   // tile columns per rasterisation group (full schedules): keeps a group's B panels in L2
  // epilogue: d = alpha * acc + beta * C ; alpha, beta optionally scaled per batch from device arrays
  float alpha, beta;
  const float* alpha_a;
  const float* alpha_b;
  const float* beta_v;
  int alpha_b_step;
  const float* C;
  long long ldc, c_bs;
  float* D;
  long long ldd, d_bs;
  void* D16;
  long long ld16, d16_bs;
  int d16_fmt;  // 0 FP16, 1 BF16
  int packed;   // C and D are packed upper triangles (row r starts at r*N - r(r-1)/2 - r ... see packed_off)
  int mirror;   // tri: also store the transposed element
  int upper_d;  // tri + mirror: the FP32 result D is not mirrored (its lower triangle is never read)
  int vec_ok;   // leading dimensions and batch strides allow 16-byte vector access
  float* sumsq;           // per batch: sum of d^2 over the full (mirrored) result
  unsigned int* maxabs;   // per batch: max |d| as FP32 bits
  unsigned int* maxaff;   // per batch: max |aff_a * [r==c] + aff_b * d| as FP32 bits
  float aff_a, aff_b;
  unsigned int* maxres;   // per batch: max |[r==c] - d| as FP32 bits (distance of the result from the identity)
  // optional FP16 hi/lo operand planes of the result, ready to feed the next split-precision product:
  //   S0: planes of s0_scale * d            S1: planes of s1_scale * (s1_aff_a * [r==c] + s1_aff_b * d)
  // hi plane at S + b * s_bs + r * s_ld + c, lo plane s_plane elements further
  __half* S0;
  __half* S1;
  long long s_ld, s_bs, s_plane;
  float s0_scale, s1_scale, s1_aff_a, s1_aff_b;
  int* status;  // set non-zero if a bounded wait ran out
  unsigned long long* prof;  // optional: eight cycle counters summed over CTAs (see toner_gemm_phase_cycles)
};

__host__ __device__ inline long long packed_off(long long r, long long c, long long n) {
  return r * n - r * (r + 1) / 2 + c;
}

// Tiles are TM x BN (TM = 128, or 256 for CTA pairs).
__host__ __device__ inline int gemm_tiles_per_batch(int M, int N, int BN, int tri, int TM = kBM) {
  const int tm = (M + TM - 1) / TM, tn = (N + BN - 1) / BN;
  if (!tri) return tm * tn;
  int total = 0;
  for (int i = 0; i < tm; ++i) {
    const int first = (i * TM) / BN;
    if (first < tn) total += tn - first;
  }
  return total;
}

// kPair: two CTAs of a cluster work on one 256 x BN tile (cta_group::2); each holds 128 rows of A and BN/2
// rows of B per stage, so a stage is two thirds the size and the ring two stages deeper.
// BN = 512 (pairs only) is the wide tile: two 256-column MMAs per k-step share the A rows, which cuts the operand
// bytes fetched per flop by a quarter (48 KB per CTA and k-block for twice the work of 32 KB).  Its accumulator
// fills all 512 columns of tensor memory, so there is no second buffer: the epilogue of a tile overlaps the next
// tile's MMAs only half by half.  It pays where the accumulation is long (K in the thousands of k-blocks, as in
// the statistic X^T X, or three plane passes of a wide matrix).
template <int BN, bool kPair = false>
struct GemmSmem {
  static constexpr bool kWide = kPair && BN == 512;
  static constexpr int kABytes = kBM * kBK * 2;
  static constexpr int kBRows = kPair ? BN / 2 : BN;   // rows of B this CTA loads per stage
  static constexpr int kBBytes = kBRows * kBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (192 * 1024) / kStageBytes;
  static constexpr int kTileBytes = kStages * kStageBytes;
  static constexpr int kBarBytes = 256;
  static constexpr int kEpiBytes = 8 * 32 * 33 * 4;  // one padded 32 x 32 FP32 staging block per epilogue warp
  static constexpr int kTotal = kTileBytes + kBarBytes + kEpiBytes + 1024;  // 1024: alignment slack
  static constexpr int kTmemCols = kWide ? 512 : 2 * BN;
};

__device__ __forceinline__ void tile_coord(const GemmParams& p, int BN, int TM, int t, int tiles_per_batch, int tiles_n,
                                           int& b, int& tm, int& tn) {
  b = t / tiles_per_batch;
  int r = t - b * tiles_per_batch;
  if (!p.tri) {
    // Column groups of `raster` tiles, rows swept inside a group: the tiles in flight at any moment share
    // a few B panels (resident in L2 for the whole sweep) and stream A panels once per group.
    const int tiles_m = tiles_per_batch / tiles_n;
    const int g = p.raster > 0 ? p.raster : tiles_n;
    const int per_group = g * tiles_m;
    const int group = r / per_group;
    const int in_group = r - group * per_group;
    const int width = min(g, tiles_n - group * g);
    tm = in_group / width;
    tn = group * g + (in_group - tm * width);
    return;
  }
  tm = 0;
  for (;;) {
    const int first = (tm * TM) / BN;
    const int cnt = tiles_n - first;
    if (r < cnt) {
      tn = first + r;
      return;
    }
    r -= cnt;
    ++tm;
  }
}

__device__ __forceinline__ void report(int* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

// Per-tile epilogue state (uniform over the warp).
struct EpilogueTile {
  const float* Cb;
  float* Db;
  uint16_t* Hb;  // 16-bit copy of the result (FP16 or BF16 bits)
  __half* S0b;
  __half* S1b;
  float alpha, beta;
  bool use_c;
};

constexpr int kEpiStride = 33;                      // floats per staged row: 32 + 1 keeps both access patterns conflict-free
constexpr int kEpiWarpBytes = 32 * kEpiStride * 4;  // one 32 x 32 block per epilogue warp

__device__ __forceinline__ uint16_t to_bits16(float v, int bf16) {
  const __half h = __float2half_rn(v);
  const __nv_bfloat16 g = __float2bfloat16_rn(v);
  return bf16 ? *reinterpret_cast<const uint16_t*>(&g) : *reinterpret_cast<const uint16_t*>(&h);
}

__device__ __forceinline__ uint2 pack4_16(float a, float b, float c, float d, int bf16) {
  const __half2 h0 = __floats2half2_rn(a, b), h1 = __floats2half2_rn(c, d);
  const __nv_bfloat162 g0 = __floats2bfloat162_rn(a, b), g1 = __floats2bfloat162_rn(c, d);
  uint2 u;
  u.x = bf16 ? *reinterpret_cast<const uint32_t*>(&g0) : *reinterpret_cast<const uint32_t*>(&h0);
  u.y = bf16 ? *reinterpret_cast<const uint32_t*>(&g1) : *reinterpret_cast<const uint32_t*>(&h1);
  return u;
}

// FP16 hi/lo split of four consecutive values: hi = rn(x), lo = rn(x - hi).
__device__ __forceinline__ void store_split4(__half* hi, long long plane, float x0, float x1, float x2, float x3) {
  const __half2 h0 = __floats2half2_rn(x0, x1), h1 = __floats2half2_rn(x2, x3);
  const float2 f0 = __half22float2(h0), f1 = __half22float2(h1);
  const __half2 l0 = __floats2half2_rn(x0 - f0.x, x1 - f0.y), l1 = __floats2half2_rn(x2 - f1.x, x3 - f1.y);
  uint2 u, w;
  u.x = *reinterpret_cast<const uint32_t*>(&h0); u.y = *reinterpret_cast<const uint32_t*>(&h1);
  w.x = *reinterpret_cast<const uint32_t*>(&l0); w.y = *reinterpret_cast<const uint32_t*>(&l1);
  *reinterpret_cast<uint2*>(hi) = u;
  *reinterpret_cast<uint2*>(hi + plane) = w;
}
__device__ __forceinline__ void store_split1(__half* hi, long long plane, float x) {
  const __half h = __float2half_rn(x);
  hi[0] = h;
  hi[plane] = __float2half_rn(x - __half2float(h));
}

// The epilogue writes the result in 32 x 32 blocks staged in shared memory (thread t's row of the
// accumulator at stage[t * kEpiStride ...]), so that the loops below are rolled -- the code stays a few
// KB and resident in the instruction cache -- and every global access of a warp is made of contiguous runs.

// Interior block: wholly inside the matrix, 16-byte aligned rows, no element needing diagonal treatment
// (for a symmetric result the block lies strictly above the diagonal, so all of it is mirrored and counts
// twice in the sum of squares).  Lane = (row within a group of four, four consecutive columns): one warp
// access covers four rows x 128 bytes.  The mirrored half is written the same way with rows and columns
// exchanged.  The values read from C are fetched four row-groups at a time before any store, so that the
// loads overlap (C and D may be the same matrix; every element is read before it is written).
__device__ __forceinline__ void epilogue_block_vec(const GemmParams& p, const EpilogueTile& e, float* stage, int row_first,
                                                   int c0, int lane, float& ssq, float& mabs, float& maff, float& mres) {
  const int q = lane & 7, sub = lane >> 3;
  const int col = c0 + 4 * q;
  const bool mirror = p.tri && p.mirror;
  const float s0 = p.s0_scale, s1 = p.s1_scale * p.s1_aff_b;  // no diagonal element in an interior block
  float s = 0.f, m = 0.f;
#pragma unroll 1
  for (int half = 0; half < 2; ++half) {
    float4 cv[4];
    if (e.use_c) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int row = row_first + 16 * half + 4 * u + sub;
        cv[u] = *reinterpret_cast<const float4*>(e.Cb + (long long)row * p.ldc + col);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = 16 * half + 4 * u + sub;
      const int row = row_first + i;
      float* src = stage + i * kEpiStride + 4 * q;
      float v0 = e.alpha * src[0], v1 = e.alpha * src[1], v2 = e.alpha * src[2], v3 = e.alpha * src[3];
      if (e.use_c) {
        v0 = fmaf(e.beta, cv[u].x, v0); v1 = fmaf(e.beta, cv[u].y, v1);
        v2 = fmaf(e.beta, cv[u].z, v2); v3 = fmaf(e.beta, cv[u].w, v3);
      }
      if (e.Db) *reinterpret_cast<float4*>(e.Db + (long long)row * p.ldd + col) = make_float4(v0, v1, v2, v3);
      if (e.Hb) *reinterpret_cast<uint2*>(e.Hb + (long long)row * p.ld16 + col) = pack4_16(v0, v1, v2, v3, p.d16_fmt);
      if (e.S0b) store_split4(e.S0b + (long long)row * p.s_ld + col, p.s_plane, s0 * v0, s0 * v1, s0 * v2, s0 * v3);
      if (e.S1b) store_split4(e.S1b + (long long)row * p.s_ld + col, p.s_plane, s1 * v0, s1 * v1, s1 * v2, s1 * v3);
      if (mirror) {
        src[0] = v0; src[1] = v1; src[2] = v2; src[3] = v3;
      }
      s = fmaf(v0, v0, s); s = fmaf(v1, v1, s); s = fmaf(v2, v2, s); s = fmaf(v3, v3, s);
      m = fmaxf(fmaxf(fmaxf(m, fabsf(v0)), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
    }
  }
  ssq += p.tri ? 2.f * s : s;
  mabs = fmaxf(mabs, m);
  maff = fmaxf(maff, fabsf(p.aff_b) * m);  // off the diagonal the affine map is a plain scaling
  // and the distance from the identity is |d|; fmaxf drops NaN, the sum of squares does not
  mres = fmaxf(mres, isfinite(s) ? m : INFINITY);
  if (mirror) {
    __syncwarp();
    const int tcol = row_first + 4 * q;  // source rows 4q .. 4q+3 become four consecutive target columns
    const float* src = stage + (4 * q) * kEpiStride;
#pragma unroll 2
    for (int it = 0; it < 8; ++it) {
      const int j = 4 * it + sub;  // source column = target row
      const float v0 = src[j], v1 = src[kEpiStride + j], v2 = src[2 * kEpiStride + j], v3 = src[3 * kEpiStride + j];
      const long long trow = c0 + j;
      if (e.Db && !p.upper_d) *reinterpret_cast<float4*>(e.Db + trow * p.ldd + tcol) = make_float4(v0, v1, v2, v3);
      if (e.Hb) *reinterpret_cast<uint2*>(e.Hb + trow * p.ld16 + tcol) = pack4_16(v0, v1, v2, v3, p.d16_fmt);
      if (e.S0b) store_split4(e.S0b + trow * p.s_ld + tcol, p.s_plane, s0 * v0, s0 * v1, s0 * v2, s0 * v3);
      if (e.S1b) store_split4(e.S1b + trow * p.s_ld + tcol, p.s_plane, s1 * v0, s1 * v1, s1 * v2, s1 * v3);
    }
  }
  __syncwarp();
}

// Any other block (matrix edge, diagonal block of a symmetric result, packed or unaligned output): one
// element per lane with full masking, lane = column, so rows -- also rows of a packed triangle -- are
// still written as contiguous runs; the mirrored half with lane = source row.
__device__ __forceinline__ void epilogue_block_scalar(const GemmParams& p, const EpilogueTile& e, float* stage, int row_first,
                                                      int c0, int lane, float& ssq, float& mabs, float& maff, float& mres) {
  const int col = c0 + lane;
  const bool col_ok = col < p.N;
  const bool mirror = p.tri && p.mirror;
  const int rows = min(32, p.M - row_first);
#pragma unroll 1
  for (int i = 0; i < rows; ++i) {
    const int row = row_first + i;
    float v = 0.f;
    if (col_ok && !(p.tri && col < row)) {
      v = e.alpha * stage[i * kEpiStride + lane];
      const long long co = p.packed ? packed_off(row, col, p.N) : (long long)row * p.ldc + col;
      const long long dof = p.packed ? packed_off(row, col, p.N) : (long long)row * p.ldd + col;
      if (e.use_c) v = fmaf(e.beta, e.Cb[co], v);
      if (e.Db) e.Db[dof] = v;
      if (e.Hb) e.Hb[(long long)row * p.ld16 + col] = to_bits16(v, p.d16_fmt);
      const float dg = (col == row) ? 1.f : 0.f;
      if (e.S0b) store_split1(e.S0b + (long long)row * p.s_ld + col, p.s_plane, p.s0_scale * v);
      if (e.S1b) store_split1(e.S1b + (long long)row * p.s_ld + col, p.s_plane, p.s1_scale * fmaf(p.s1_aff_b, v, p.s1_aff_a * dg));
      mres = isfinite(v) ? fmaxf(mres, fabsf(dg - v)) : INFINITY;  // a non-finite result must not pass as converged
      const float w = (p.tri && col > row) ? 2.f : 1.f;
      ssq = fmaf(w * v, v, ssq);
      mabs = fmaxf(mabs, fabsf(v));
      maff = fmaxf(maff, fabsf(fmaf(p.aff_b, v, col == row ? p.aff_a : 0.f)));
    }
    if (mirror) stage[i * kEpiStride + lane] = v;  // final value; zero where masked
  }
  if (mirror) {
    __syncwarp();
    const int row = row_first + lane;  // this lane's source row becomes the target column
    const int cols = min(32, p.N - c0);
    if (row < p.M) {
#pragma unroll 1
      for (int j = 0; j < cols; ++j) {
        const int c = c0 + j;
        if (c > row) {
          const float v = stage[lane * kEpiStride + j];
          if (e.Db && !p.upper_d) e.Db[(long long)c * p.ldd + row] = v;
          if (e.Hb) e.Hb[(long long)c * p.ld16 + row] = to_bits16(v, p.d16_fmt);
          if (e.S0b) store_split1(e.S0b + (long long)c * p.s_ld + row, p.s_plane, p.s0_scale * v);
          if (e.S1b) store_split1(e.S1b + (long long)c * p.s_ld + row, p.s_plane, p.s1_scale * p.s1_aff_b * v);
        }
      }
    }
  }
  __syncwarp();
}

// kChained: the kernel sums several accumulation chains per tile in registers (p.promote > 0).
// kPair: launched as clusters of two CTAs that share each 256 x BN tile (BN = 256): both load their halves of
// the operands, the leader CTA's MMA thread issues cta_group::2 MMAs, each CTA's epilogue warps write the
// 128 rows that sit in its own tensor memory.  The pair halves the operand traffic per flop of B.
template <int BN, bool kChained, bool kPair = false>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_tcgen05_kernel(const __grid_constant__ GemmParams p) {
  using S = GemmSmem<BN, kPair>;
  static_assert(BN == 128 || BN == 256 || (BN == 512 && kPair && !kChained), "tile widths: 128, 256, or 512 on a pair");
  constexpr bool kWide = S::kWide;
  constexpr int BNI = kWide ? 256 : BN;                // columns of one MMA instruction
  constexpr int NJ = BN / BNI;                         // MMAs per k-step (column halves of a wide tile)
  constexpr int TM = kPair ? 2 * kBM : kBM;            // rows of one scheduled tile
  const uint32_t cta_rank = kPair ? ptx::cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;
  const int unit = kPair ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;     // which persistent worker this CTA (pair) is
  const int units = kPair ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* const smem = smem_raw + (base - raw);
  // barrier block after the tiles
  const uint32_t bars = base + S::kTileBytes;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (S::kStages + s); };
  auto tfull_bar = [&](int s) { return bars + 8u * (2 * S::kStages + s); };
  auto tempty_bar = [&](int s) { return bars + 8u * (2 * S::kStages + 2 + s); };
  volatile uint32_t* const tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + S::kTileBytes + 8 * (2 * S::kStages + 4));
  volatile int* const abort_flag = reinterpret_cast<volatile int*>(smem + S::kTileBytes + 8 * (2 * S::kStages + 4) + 8);
  // A role that gives up stops its own CTA and, in a pair, the peer as well: both CTAs' roles poll their CTA's flag
  // between waits, so neither keeps issuing copies or MMAs for two more seconds.  The peer's shared memory is valid
  // until the closing cluster barrier, which every thread of both CTAs reaches.
  auto raise_abort = [&]() {
    *abort_flag = 1;
    if constexpr (kPair)
      ptx::st_cluster_u32(ptx::mapa(ptx::smem_u32(const_cast<int*>(abort_flag)), cta_rank ^ 1u), 1u);
  };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int tiles_per_batch = gemm_tiles_per_batch(p.M, p.N, BN, p.tri, TM);
  const int total_tiles = tiles_per_batch * p.batch;
  const int kb_per_seg = (p.K + kBK - 1) / kBK;
  const int num_kb = kb_per_seg * p.segs;
  // Accumulation chains: with promote > 0 the MMA warp starts a fresh TMEM accumulator every `promote`
  // k-blocks of the FIRST segment and the epilogue warps sum the chains in registers.  Later segments
  // (the hi*lo cross terms of a split product, 2^-11 of the first) form one chain each: truncation
  // inside them is far below the result's last bit.  promote_all chains every segment the same way.
  const int chunks_seg0 = p.promote > 0 ? (kb_per_seg + p.promote - 1) / p.promote : 1;
  const int chunks_rest = (p.promote > 0 && p.promote_all) ? chunks_seg0 : 1;
  const int chunks_per_tile = p.promote > 0 ? chunks_seg0 + (p.segs - 1) * chunks_rest : 1;
  // Order of work inside a tile.  When only the first segment is chained, the later segments come FIRST, one
  // long chain each: while the epilogue warps are still writing the previous tile they cannot sum chains, and
  // two long chains give them that time; the short chains of the first segment follow.
  const bool rest_first = p.promote > 0 && !p.promote_all && p.segs > 1;
  auto chunk_range = [&](int ch, int& kb_begin, int& kb_end) {  // k-block indices in processing order
    if (p.promote <= 0) {
      kb_begin = 0;
      kb_end = num_kb;
      return;
    }
    if (rest_first) {
      const int rest = p.segs - 1;
      if (ch < rest) {
        kb_begin = ch * kb_per_seg;
        kb_end = kb_begin + kb_per_seg;
      } else {
        kb_begin = rest * kb_per_seg + (ch - rest) * p.promote;
        kb_end = min(kb_begin + p.promote, num_kb);
      }
      return;
    }
    int seg = 0, c = ch;
    if (ch >= chunks_seg0) {
      seg = 1 + (ch - chunks_seg0) / chunks_rest;
      c = (ch - chunks_seg0) - (seg - 1) * chunks_rest;
    }
    const bool chained = (seg == 0) || p.promote_all;
    kb_begin = seg * kb_per_seg + (chained ? c * p.promote : 0);
    kb_end = chained ? min(kb_begin + p.promote, (seg + 1) * kb_per_seg) : (seg + 1) * kb_per_seg;
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < S::kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(tfull_bar(s), 1);
      // one arrival per epilogue warp (of both CTAs of a pair); per half of a wide tile: the four warps that read it
      ptx::mbar_init(tempty_bar(s), kWide ? 8 : (kPair ? 16 : 8));
    }
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 1) {
    if constexpr (kPair) {
      ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), S::kTmemCols);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), S::kTmemCols);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before();
  if constexpr (kPair) ptx::cluster_sync();  // the peer's barriers exist before anything signals them
  else __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4) {
  ptx::reg_dec<48>();
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long prof_wait = 0;
      for (int t = unit; t < total_tiles && ok; t += units) {
        int b, tm, tn;
        tile_coord(p, BN, TM, t, tiles_per_batch, tiles_n, b, tm, tn);
        const CUtensorMap* amap = p.a_maps + (long long)b * p.a_map_stride;
        const CUtensorMap* bmap = p.b_maps + (long long)b * p.b_map_stride;
        ptx::fence_tensormap_acquire(amap);
        ptx::fence_tensormap_acquire(bmap);
        // a pair splits the tile's rows (A) and its columns (B) between its two CTAs
        // (of a wide tile each CTA holds 128 columns of either 256-column half: n0 is its share of the first half)
        const int m0 = tm * TM + (int)cta_rank * kBM, n0 = tn * BN + (int)cta_rank * (kWide ? BNI / 2 : S::kBRows);
        for (int si = 0; si < p.segs && ok; ++si) {
          const int seg = rest_first ? (si + 1 == p.segs ? 0 : si + 1) : si;
          const int za = b * p.a_z_stride + p.a_seg_z[seg];
          const int zb = b * p.b_z_stride + p.b_seg_z[seg];
          for (int k0 = 0; k0 < p.K; k0 += kBK) {
            const long long w0 = p.prof ? clock64() : 0;
            const bool got = ptx::mbar_wait(empty_bar(stage), phase ^ 1u, kWaitCycles);
            if (p.prof) prof_wait += clock64() - w0;
            if (!got || *abort_flag) {
              report(p.status, kTimeoutProducer);
              raise_abort();
              ok = false;
              break;
            }
            const uint32_t sa = base + stage * S::kStageBytes;
            const uint32_t sb = sa + S::kABytes;
            if constexpr (kPair) {
              // Both CTAs' copies report to the leader's barrier, which expects the bytes of the whole pair.
              const uint32_t lbar = ptx::mapa(full_bar(stage), 0);
              if (leader) ptx::mbar_expect_tx(full_bar(stage), 2 * S::kStageBytes);
              if (p.a_mn) {
#pragma unroll
                for (int s = 0; s < kBM / 64; ++s) ptx::tma_load_3d_pair(sa + s * 8192, amap, lbar, m0 + s * 64, k0, za);
              } else {
                ptx::tma_load_3d_pair(sa, amap, lbar, k0, m0, za);
              }
              if constexpr (kWide) {
                if (p.b_mn) {
#pragma unroll
                  for (int s = 0; s < 4; ++s)
                    ptx::tma_load_3d_pair(sb + s * 8192, bmap, lbar, n0 + (s >> 1) * BNI + (s & 1) * 64, k0, zb);
                } else {
#pragma unroll
                  for (int j = 0; j < 2; ++j) ptx::tma_load_3d_pair(sb + j * 16384, bmap, lbar, k0, n0 + j * BNI, zb);
                }
              } else if (p.b_mn) {
#pragma unroll
                for (int s = 0; s < S::kBRows / 64; ++s) ptx::tma_load_3d_pair(sb + s * 8192, bmap, lbar, n0 + s * 64, k0, zb);
              } else {
                ptx::tma_load_3d_pair(sb, bmap, lbar, k0, n0, zb);
              }
            } else {
              ptx::mbar_expect_tx(full_bar(stage), S::kStageBytes);
              if (p.a_mn) {
#pragma unroll
                for (int s = 0; s < kBM / 64; ++s) ptx::tma_load_3d(sa + s * 8192, amap, full_bar(stage), m0 + s * 64, k0, za);
              } else {
                ptx::tma_load_3d(sa, amap, full_bar(stage), k0, m0, za);
              }
              if (p.b_mn) {
#pragma unroll
                for (int s = 0; s < BN / 64; ++s) ptx::tma_load_3d(sb + s * 8192, bmap, full_bar(stage), n0 + s * 64, k0, zb);
              } else {
                ptx::tma_load_3d(sb, bmap, full_bar(stage), k0, n0, zb);
              }
            }
            if (++stage == S::kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
      if (p.prof && leader) atomicAdd(p.prof + 3, (unsigned long long)prof_wait);
      if (!ok || *abort_flag) {
        // Copies already issued must land before this CTA gives its shared memory back (the closing barrier waits
        // for threads, not for bulk copies).  Stage s was last filled in this round if s < stage, else in the round
        // before (a stage never filled is "complete" at once: its barrier has not left phase 0).  In a pair every
        // copy of both CTAs reports to the leader's barriers, so the leader waits for them; a barrier whose other
        // half was never issued cannot complete, hence the bound.  Copies the leader cannot account for (the peer
        // ran a few stages ahead of it) get a fixed settling time in both CTAs: a copy lands within microseconds.
        if (!kPair || leader) {
          for (int s = 0; s < S::kStages; ++s)
            ptx::mbar_wait(full_bar(s), (s < stage) ? phase : (phase ^ 1u), kDrainCycles);
        }
        if constexpr (kPair) {
          const long long t0 = clock64();
          while (clock64() - t0 < kSettleCycles) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (of a pair: the leader CTA only)
    if (lane == 0 && leader) {
      const uint32_t idesc = (1u << 4) | ((uint32_t)p.fmt << 7) | ((uint32_t)p.fmt << 10) | ((uint32_t)p.a_mn << 15) |
                             ((uint32_t)p.b_mn << 16) | ((uint32_t)(BNI >> 3) << 17) | ((uint32_t)(TM >> 4) << 24);
      // K-major: 8-row groups 1024 B apart, k advances 32 B inside the swizzled row.
      // MN-major: 64-element slabs 8192 B apart (LBO), 8-k-row groups 1024 B apart (SBO), k advances 16 rows = 2048 B.
      // The descriptor's upper word (8-row groups 1024 B apart, version, 128-byte swizzle) never changes; the lower
      // word is the address in 16-byte units plus the leading-dimension offset, so a k-step is an addition.
      const uint32_t desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
      const uint32_t a_lo_const = ((p.a_mn ? 8192u : 16u) >> 4) << 16, b_lo_const = ((p.b_mn ? 8192u : 16u) >> 4) << 16;
      const uint32_t a_step16 = (p.a_mn ? 2048u : 32u) >> 4, b_step16 = (p.b_mn ? 2048u : 32u) >> 4;
      int stage = 0;
      uint32_t phase = 0;
      uint32_t gchunk = 0;  // accumulator hand-offs so far; buffer = gchunk & 1
      bool ok = true;
      long long prof_acc = 0, prof_ops = 0;
      const long long prof_t0 = p.prof ? clock64() : 0;
      for (int t = unit; t < total_tiles && ok; t += units) {
        for (int ch = 0; ch < chunks_per_tile && ok; ++ch, ++gchunk) {
          int kb_begin, kb_end;
          chunk_range(ch, kb_begin, kb_end);
          // The wide tile has one accumulator of two halves, each with its own "drained" barrier (tempty 0 / 1): the
          // MMAs of the first k-block's first half start as soon as that half has been read out.
          const int buf = kWide ? 0 : (int)(gchunk & 1u);
          const uint32_t acc_parity = (kWide ? (gchunk & 1u) : ((gchunk >> 1) & 1u)) ^ 1u;
          auto wait_drained = [&](int bar) {
            const long long w0 = p.prof ? clock64() : 0;
            const bool got_acc = ptx::mbar_wait(tempty_bar(bar), acc_parity, kWaitCycles);
            if (p.prof) prof_acc += clock64() - w0;
            if (!got_acc || *abort_flag) {
              report(p.status, kTimeoutMma);
              raise_abort();
              ok = false;
              return false;
            }
            ptx::tc_fence_after();
            return true;
          };
          if (!wait_drained(buf)) break;
          const uint32_t d_tmem = tmem_base + (uint32_t)(kWide ? 0 : buf * BN);
          for (int kb = kb_begin; kb < kb_end; ++kb) {
            const long long w1 = p.prof ? clock64() : 0;
            const bool got_ops = ptx::mbar_wait(full_bar(stage), phase, kWaitCycles);
            if (p.prof) prof_ops += clock64() - w1;
            if (!got_ops || *abort_flag) {
              report(p.status, kTimeoutMma);
              raise_abort();
              ok = false;
              break;
            }
            ptx::tc_fence_after();
            const uint32_t sa = base + stage * S::kStageBytes;
            const uint32_t a_lo = ((sa & 0x3FFFFu) >> 4) | a_lo_const;
            const uint32_t b_lo = (((sa + S::kABytes) & 0x3FFFFu) >> 4) | b_lo_const;
            const uint32_t fresh = (kb != kb_begin) ? 1u : 0u;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
              if (kWide && j == 1 && kb == kb_begin && !wait_drained(1)) break;
#pragma unroll
              for (int k = 0; k < kBK / kUmmaK; ++k) {
                const uint64_t da = ((uint64_t)desc_hi << 32) | (a_lo + k * a_step16);
                const uint64_t db = ((uint64_t)desc_hi << 32) | (b_lo + j * ((BNI / 2) * kBK * 2 / 16) + k * b_step16);
                if constexpr (kPair) ptx::mma_f16_pair(d_tmem + j * BNI, da, db, idesc, k != 0 ? 1u : fresh);
                else ptx::mma_f16(d_tmem, da, db, idesc, k != 0 ? 1u : fresh);
              }
            }
            if (!ok) break;
            // frees the stage (in both CTAs of a pair) once these MMAs have read it
            if constexpr (kPair) {
              ptx::mma_commit_pair(empty_bar(stage));
              ptx::mma_commit_pair(ptx::mapa(empty_bar(stage), 1));
            } else {
              ptx::mma_commit(empty_bar(stage));
            }
            if (++stage == S::kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (ok) {  // this chain's partial sum is complete
            if constexpr (kPair) {
              ptx::mma_commit_pair(tfull_bar(buf));
              ptx::mma_commit_pair(ptx::mapa(tfull_bar(buf), 1));
            } else {
              ptx::mma_commit(tfull_bar(buf));
            }
          }
        }
      }
      if (p.prof) {
        atomicAdd(p.prof + 0, (unsigned long long)(clock64() - prof_t0));
        atomicAdd(p.prof + 1, (unsigned long long)prof_acc);
        atomicAdd(p.prof + 2, (unsigned long long)prof_ops);
        atomicAdd(p.prof + 7, 1ull);
      }
    }
  }
  } else {
    ptx::reg_inc<224>();
    // ------------------------------------------------------------ epilogue (warps 4..11)
    // Warp w may read TMEM lanes [32*(w&3), +32); two warps share a lane group and split the columns.
    constexpr int NCH = BN / 64;  // 32-column chunks per warp
    const int lane_group = warp & 3;
    const int half = (warp - 4) >> 2;
    float* const stage = reinterpret_cast<float*>(smem + S::kTileBytes + S::kBarBytes) + (warp - 4) * (32 * kEpiStride);
    constexpr bool chained = kChained;
    // Running sums of the accumulation chains (chained products only), added with round-to-nearest: the
    // tensor core itself adds into its accumulator by truncation.
    float racc[kChained ? NCH * 32 : 1];
    uint32_t gchunk = 0;
    bool alive = true;
    long long prof_wait = 0, prof_out = 0, prof_sum = 0;
    for (int t = unit; t < total_tiles && alive; t += units) {
      int b, tm, tn;
      tile_coord(p, BN, TM, t, tiles_per_batch, tiles_n, b, tm, tn);
      const int m0 = tm * TM + (int)cta_rank * kBM, n0 = tn * BN;  // this CTA's 128 rows of the tile
      const int row_first = m0 + lane_group * 32;
      const int col_first = n0 + half * (BN / 2);
      // 32-column blocks this warp never needs: beyond N, or wholly below the diagonal (warp-uniform)
      auto needed = [&](int c0) { return (c0 < p.N) && !(p.tri && c0 + 31 < row_first); };
      auto wait_chain = [&](int buf) {
        const long long w0 = p.prof ? clock64() : 0;
        // every lane observes the barrier itself, so each one is ordered after the MMAs' TMEM writes
        const uint32_t parity = kWide ? (gchunk & 1u) : ((gchunk >> 1) & 1u);
        const int waited = __all_sync(0xffffffffu, ptx::mbar_wait(tfull_bar(buf), parity, kWaitCycles) ? 1 : 0);
        if (!waited || *abort_flag) {
          if (lane == 0) {
            report(p.status, kTimeoutEpilogue);
            raise_abort();
          }
          return false;
        }
        ptx::tc_fence_after();
        if (p.prof) prof_wait += clock64() - w0;
        return true;
      };
      auto release = [&](int buf) {  // buffer drained: hand it back to the MMA warp
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kPair) ptx::mbar_arrive_cluster(ptx::mapa(tempty_bar(buf), 0));  // the leader's MMA thread waits
          else ptx::mbar_arrive(tempty_bar(buf));
        }
      };
      auto tmem_of = [&](int buf) {
        return tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)((kWide ? 0 : buf * BN) + half * (BN / 2));
      };

      if (chained) {
#pragma unroll
        for (int j = 0; j < NCH * 32; ++j) racc[j] = 0.f;
        for (int ch = 0; ch < chunks_per_tile; ++ch, ++gchunk) {
          const int buf = gchunk & 1u;
          if (!wait_chain(buf)) {
            alive = false;
            break;
          }
          const long long a0 = p.prof ? clock64() : 0;
          const uint32_t taddr = tmem_of(buf);
          // Software pipeline in steps of 16 columns: the next load is in flight while the current one is added.
          // (Blocks wholly below the diagonal are loaded and added too: their sums are simply never written.)
          uint32_t s0[16], s1[16];
          ptx::tmem_ld16(taddr, s0);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < NCH * 2; ++h) {
            uint32_t* cur = (h & 1) ? s1 : s0;
            uint32_t* nxt = (h & 1) ? s0 : s1;
            if (h + 1 < NCH * 2) ptx::tmem_ld16(taddr + (uint32_t)((h + 1) * 16), nxt);
#pragma unroll
            for (int j = 0; j < 16; ++j) racc[h * 16 + j] += __uint_as_float(cur[j]);
            if (h + 1 < NCH * 2) ptx::tmem_ld_wait();
          }
          release(buf);
          if (p.prof) prof_sum += clock64() - a0;
        }
        if (!alive) break;
      } else if (!wait_chain(kWide ? 0 : (int)(gchunk & 1u))) {
        alive = false;
        break;
      }

      // ---- write the tile: one rolled loop over the warp's 32 x 32 blocks, staged through shared memory
      const long long o0 = p.prof ? clock64() : 0;
      EpilogueTile e;
      e.alpha = p.alpha;
      e.beta = p.beta;
      if (p.alpha_a) e.alpha *= __ldg(p.alpha_a + b);
      if (p.alpha_b) e.alpha *= __ldg(p.alpha_b + (long long)b * p.alpha_b_step);
      if (p.beta_v) e.beta *= __ldg(p.beta_v + b);
      e.use_c = (p.C != nullptr) && (e.beta != 0.f);
      e.Cb = p.C ? p.C + (long long)b * p.c_bs : nullptr;
      e.Db = p.D ? p.D + (long long)b * p.d_bs : nullptr;
      e.Hb = p.D16 ? reinterpret_cast<uint16_t*>(p.D16) + (long long)b * p.d16_bs : nullptr;
      e.S0b = p.S0 ? p.S0 + (long long)b * p.s_bs : nullptr;
      e.S1b = p.S1 ? p.S1 + (long long)b * p.s_bs : nullptr;
      float ssq = 0.f, mabs = 0.f, maff = 0.f, mres = 0.f;
      const bool rows_inside = row_first + 32 <= p.M;
      const uint32_t taddr = tmem_of(kWide ? 0 : (int)(gchunk & 1u));
      float* const mine = stage + lane * kEpiStride;
#pragma unroll 1
      for (int cc = 0; cc < NCH; ++cc) {
        const int c0 = col_first + cc * 32;
        if (!needed(c0)) continue;
        if (chained) {
          switch (cc) {  // the running sums live in registers: static indices only
            case 0:
#pragma unroll
              for (int j = 0; j < 32; ++j) mine[j] = racc[j];
              break;
            case 1:
#pragma unroll
              for (int j = 0; j < 32; ++j) mine[j] = racc[32 + j];
              break;
            case 2:
              if (NCH > 2) {
#pragma unroll
                for (int j = 0; j < 32; ++j) mine[j] = racc[(NCH > 2 ? 64 : 0) + j];
              }
              break;
            default:
              if (NCH > 2) {
#pragma unroll
                for (int j = 0; j < 32; ++j) mine[j] = racc[(NCH > 2 ? 96 : 0) + j];
              }
              break;
          }
        } else {
          uint32_t raw[32];
          ptx::tmem_ld32(taddr + (uint32_t)(cc * 32), raw);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) mine[j] = __uint_as_float(raw[j]);
        }
        __syncwarp();
        // warp-uniform choice: interior blocks take the vector path
        const bool holds_diag = (c0 <= row_first + 31) && (c0 + 31 >= row_first);
        if (rows_inside && (c0 + 32 <= p.N) && p.vec_ok && !(holds_diag && (p.tri || p.maxaff || p.maxres || p.S1))) {
          epilogue_block_vec(p, e, stage, row_first, c0, lane, ssq, mabs, maff, mres);
        } else {
          epilogue_block_scalar(p, e, stage, row_first, c0, lane, ssq, mabs, maff, mres);
        }
      }
      if (!chained) {
        // wide tile: this warp read columns of half `half` only, and that half's barrier counts its four lane groups
        // of both CTAs
        release(kWide ? half : (int)(gchunk & 1u));
        ++gchunk;
      }
      if (p.prof) prof_out += clock64() - o0;

      if (p.sumsq || p.maxabs || p.maxaff || p.maxres) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
          mabs = fmaxf(mabs, __shfl_xor_sync(0xffffffffu, mabs, o));
          maff = fmaxf(maff, __shfl_xor_sync(0xffffffffu, maff, o));
          mres = fmaxf(mres, __shfl_xor_sync(0xffffffffu, mres, o));
        }
        if (lane == 0) {
          if (p.sumsq) atomicAdd(p.sumsq + b, ssq);  // order of these additions is not fixed
          if (p.maxabs) atomicMax(p.maxabs + b, __float_as_uint(mabs));
          if (p.maxaff) atomicMax(p.maxaff + b, __float_as_uint(maff));
          if (p.maxres) atomicMax(p.maxres + b, __float_as_uint(mres));
        }
      }
    }
    if (p.prof && leader && warp == 4 && lane == 0) {
      atomicAdd(p.prof + 4, (unsigned long long)prof_wait);
      atomicAdd(p.prof + 5, (unsigned long long)prof_out);
      atomicAdd(p.prof + 6, (unsigned long long)prof_sum);
    }
  }

  // ---------------------------------------------------------------- teardown
  ptx::tc_fence_before();
  if constexpr (kPair) ptx::cluster_sync();  // neither CTA leaves while the other may still signal or read it
  else __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    if constexpr (kPair) ptx::tmem_dealloc_pair(tmem_base, S::kTmemCols);
    else ptx::tmem_dealloc(tmem_base, S::kTmemCols);
  }
}

}  // namespace toner

// Per-device context, TMA tensor-map cache and the GEMM launcher.
#include "runtime.cuh"

#include <atomic>
#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

namespace toner {

static thread_local std::string g_error;
static std::mutex g_mutex;
static Context g_ctx[16];

// One cached operand description: where its tensor maps sit in the arena, and the upload that put them there.
struct MapEntry {
  int slot = 0;
  cudaStream_t stream = nullptr;  // stream the upload was enqueued on
  cudaEvent_t uploaded = nullptr; // recorded right after the upload
  bool settled = false;           // the upload is known to have finished: no ordering needed any more
};
using MapCache = std::unordered_map<std::string, MapEntry>;

static std::atomic<long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

void set_error(const std::string& msg) { g_error = msg; }
int fail(int code, const std::string& msg) {
  g_error = msg;
  return code;
}
const char* last_error() { return g_error.c_str(); }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode = nullptr;

static int load_encode() {
  if (g_encode) return 0;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  if (e != cudaSuccess || fn == nullptr || q != cudaDriverEntryPointSuccess)
    return fail(kErrDriver, "cuTensorMapEncodeTiled is not available from the CUDA driver");
  g_encode = reinterpret_cast<EncodeTiledFn>(fn);
  return 0;
}

Context* context() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) {
    set_error("no CUDA device is current: toner_b200 has no CPU path");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  Context& c = g_ctx[dev];
  if (c.device == dev) return &c;
  if (load_encode()) return nullptr;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) {
    set_error("cudaGetDeviceProperties failed");
    return nullptr;
  }
  if (prop.major != 10) {
    set_error("toner_b200 kernels are built for sm_100a only; device reports sm_" + std::to_string(prop.major) +
              std::to_string(prop.minor));
    return nullptr;
  }
  c.num_sms = prop.multiProcessorCount;
  c.gemm_sms = c.num_sms;
  c.arena_cap = 32768;
  if (cudaMalloc(&c.arena_dev, sizeof(CUtensorMap) * c.arena_cap) != cudaSuccess ||
      cudaMallocHost(&c.arena_host, sizeof(CUtensorMap) * c.arena_cap) != cudaSuccess ||
      cudaMalloc(&c.status_dev, sizeof(int)) != cudaSuccess || cudaMemset(c.status_dev, 0, sizeof(int)) != cudaSuccess) {
    set_error("could not allocate the tensor-map arena");
    return nullptr;
  }
  c.map_cache = new MapCache();
  cudaFuncSetAttribute(gemm_tcgen05_kernel<256, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<256>::kTotal);
  cudaFuncSetAttribute(gemm_tcgen05_kernel<256, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<256>::kTotal);
  cudaFuncSetAttribute(gemm_tcgen05_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<128>::kTotal);
  cudaFuncSetAttribute(gemm_tcgen05_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<128>::kTotal);
  cudaFuncSetAttribute(gemm_tcgen05_kernel<256, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<256, true>::kTotal);
  cudaFuncSetAttribute(gemm_tcgen05_kernel<256, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<256, true>::kTotal);
  cudaFuncSetAttribute(gemm_tcgen05_kernel<512, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<512, true>::kTotal);
  c.device = dev;
  return &c;
}

static int encode_one(CUtensorMap* out, const void* base, int rows, int cols, long long ld, long long z_stride, int nz,
                      int box_rows) {
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return fail(kErrArg, "operand base must be 16-byte aligned");
  if (ld % 8 != 0 || ld < cols) return fail(kErrArg, "operand leading dimension must be a multiple of 8 elements and >= cols");
  if (nz > 1 && z_stride % 8 != 0) return fail(kErrArg, "operand z stride must be a multiple of 8 elements");
  const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)(nz > 0 ? nz : 1)};
  const long long zs = (nz > 1) ? z_stride : (long long)rows * ld;
  const cuuint64_t strides[2] = {(cuuint64_t)ld * 2ull, (cuuint64_t)zs * 2ull};
  const cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, 1u};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(kErrDriver, "cuTensorMapEncodeTiled failed with code " + std::to_string((int)r));
  return 0;
}

int get_maps(Context* ctx, const toner_operand& op, int batch, int box_rows, cudaStream_t stream, const CUtensorMap** out) {
  const int count = op.list ? batch : 1;
  const int brows = op.mn_major ? 64 : box_rows;
  std::string key;
  key.reserve(64 + 8 * count);
  auto put = [&key](const void* p, size_t n) { key.append(reinterpret_cast<const char*>(p), n); };
  put(&op.rows, 4); put(&op.cols, 4); put(&op.ld, 8); put(&op.z_stride, 8); put(&op.nz, 4); put(&brows, 4);
  if (op.list) {
    for (int i = 0; i < batch; ++i) put(&op.list[i], sizeof(void*));
  } else {
    put(&op.base, sizeof(void*));
  }
  std::lock_guard<std::mutex> lock(g_mutex);
  auto* cache = static_cast<MapCache*>(ctx->map_cache);
  auto it = cache->find(key);
  if (it != cache->end()) {
    // The maps were uploaded by an asynchronous copy on the stream of the call that first used this operand.  A
    // launch on that stream is ordered after the copy by the stream itself; a launch on any other stream waits for
    // the copy's event (until the copy is known to be done, after which the entry needs no ordering at all).
    MapEntry& e = it->second;
    if (!e.settled) {
      if (cudaEventQuery(e.uploaded) == cudaSuccess) {
        e.settled = true;
      } else {
        (void)cudaGetLastError();  // cudaErrorNotReady is not an error here
        if (e.stream != stream) TONER_CUDA(cudaStreamWaitEvent(stream, e.uploaded, 0));
      }
    }
    *out = ctx->arena_dev + e.slot;
    return 0;
  }
  if (ctx->arena_used + count > ctx->arena_cap) {
    // Start over: wait for everything that may still read old maps, then reuse the arena from slot 0.
    TONER_CUDA(cudaDeviceSynchronize());
    for (auto& kv : *cache)
      if (kv.second.uploaded) cudaEventDestroy(kv.second.uploaded);
    cache->clear();
    ctx->arena_used = 0;
    if (count > ctx->arena_cap) return fail(kErrArg, "too many separately allocated operands in one call");
  }
  const int slot = ctx->arena_used;
  for (int i = 0; i < count; ++i) {
    const void* base = op.list ? op.list[i] : op.base;
    if (base == nullptr) return fail(kErrArg, "null operand pointer");
    int rc = encode_one(ctx->arena_host + slot + i, base, op.rows, op.cols, op.ld, op.z_stride, op.list ? 1 : op.nz, brows);
    if (rc) return rc;
  }
  MapEntry e;
  e.slot = slot;
  e.stream = stream;
  TONER_CUDA(cudaEventCreateWithFlags(&e.uploaded, cudaEventDisableTiming));
  TONER_CUDA(cudaMemcpyAsync(ctx->arena_dev + slot, ctx->arena_host + slot, sizeof(CUtensorMap) * count,
                             cudaMemcpyHostToDevice, stream));
  TONER_CUDA(cudaEventRecord(e.uploaded, stream));
  ctx->arena_used += count;
  (*cache)[key] = e;
  *out = ctx->arena_dev + slot;
  return 0;
}

int launch_gemm(const toner_gemm_desc& d, cudaStream_t stream) {
  Context* ctx = context();
  if (!ctx) return kErrCuda;
  if (d.m <= 0 || d.n <= 0 || d.k <= 0 || d.batch <= 0) return fail(kErrArg, "gemm: sizes must be positive");
  if (d.segs < 1 || d.segs > kMaxSegs) return fail(kErrArg, "gemm: segs must be 1..3");
  if (d.tri && d.m != d.n) return fail(kErrArg, "gemm: a symmetric result needs m == n");
  if (d.packed && (!d.tri || d.mirror || d.d16)) return fail(kErrArg, "gemm: packed output is upper-triangle FP32 only");
  if (!d.d && !d.d16 && !d.split0 && !d.split1) return fail(kErrArg, "gemm: no output");
  if (d.packed && (d.split0 || d.split1)) return fail(kErrArg, "gemm: operand planes cannot be packed");
  if (d.fmt != 0 && d.fmt != 1) return fail(kErrArg, "gemm: fmt must be 0 (FP16) or 1 (BF16)");

  // Tile choice: 256 x 256 tiles on CTA pairs when they fill the machine (fewest operand bytes per flop), else
  // 128 x 256, else 128 x 128 (most tiles for small problems).  tile_n forces one: 128, 256, or 512 for the pair.
  int bn = d.tile_n;
  bool pair = false;
  if (bn == 0) {
    const long long tpair = (long long)gemm_tiles_per_batch(d.m, d.n, 256, d.tri, 256) * d.batch;
    const long long t256 = (long long)gemm_tiles_per_batch(d.m, d.n, 256, d.tri) * d.batch;
    if (tpair >= ctx->gemm_sms / 2) {
      bn = 256;
      pair = true;
      // The wide tile: long accumulations only (its epilogue is not hidden behind the next tile), enough tiles for
      // several waves, and a width for which the 512-column steps do not overshoot the triangle by much.
      const long long twide = (long long)gemm_tiles_per_batch(d.m, d.n, 512, d.tri, 256) * d.batch;
      const long long depth = (long long)d.k * d.segs;
      if (ctx->gemm_wide_k > 0 && d.promote <= 0 && depth >= ctx->gemm_wide_k && twide >= 4LL * (ctx->gemm_sms / 2) &&
          2 * twide * 100 <= tpair * 106)
        bn = 512;
    } else {
      bn = (t256 >= ctx->gemm_sms) ? 256 : 128;
    }
  } else if (bn == 512) {
    bn = 256;
    pair = true;
  } else if (bn == 1024) {
    if (d.promote > 0) return fail(kErrArg, "gemm: the wide tile has no chained accumulation");
    bn = 512;
    pair = true;
  }
  if (bn != 128 && bn != 256 && !(bn == 512 && pair))
    return fail(kErrArg, "gemm: tile_n must be 0, 128, 256, 512 (256 x 256 on a CTA pair) or 1024 (256 x 512 on a pair)");

  GemmParams p;
  std::memset(&p, 0, sizeof(p));
  int rc = get_maps(ctx, d.a, d.batch, kBM, stream, &p.a_maps);
  if (rc) return rc;
  rc = get_maps(ctx, d.b, d.batch, pair ? 128 : bn, stream, &p.b_maps);  // a pair's CTA loads B in boxes of 128 rows
  if (rc) return rc;
  p.a_map_stride = d.a.list ? 1 : 0;
  p.b_map_stride = d.b.list ? 1 : 0;
  p.a_z_stride = d.a.list ? 0 : d.a.z_step;
  p.b_z_stride = d.b.list ? 0 : d.b.z_step;
  p.a_mn = d.a.mn_major ? 1 : 0;
  p.b_mn = d.b.mn_major ? 1 : 0;
  for (int s = 0; s < kMaxSegs; ++s) {
    p.a_seg_z[s] = d.a.list ? 0 : d.a.seg_z[s];
    p.b_seg_z[s] = d.b.list ? 0 : d.b.seg_z[s];
  }
  p.segs = d.segs;
  p.M = d.m; p.N = d.n; p.K = d.k; p.batch = d.batch;
  p.fmt = d.fmt;
  p.tri = d.tri ? 1 : 0;
  p.promote = d.promote > 0 ? d.promote : 0;
  p.promote_all = d.promote_all ? 1 : 0;
  p.raster = d.tri ? 0 : (d.raster > 0 ? d.raster : 8);
  p.alpha = d.alpha; p.beta = d.beta;
  p.alpha_a = d.alpha_a; p.alpha_b = d.alpha_b; p.beta_v = d.beta_v;
  p.alpha_b_step = d.alpha_b_step > 0 ? d.alpha_b_step : 1;
  p.C = d.c; p.ldc = d.ldc; p.c_bs = d.c_bs;
  p.D = d.d; p.ldd = d.ldd; p.d_bs = d.d_bs;
  p.D16 = d.d16; p.ld16 = d.ld16; p.d16_bs = d.d16_bs; p.d16_fmt = d.d16_fmt;
  p.packed = d.packed ? 1 : 0;
  p.mirror = d.mirror ? 1 : 0;
  p.upper_d = (d.upper_d && d.tri && d.mirror) ? 1 : 0;
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  p.vec_ok = !d.packed && (!d.c || (d.ldc % 4 == 0 && d.c_bs % 4 == 0 && al16(d.c))) &&
             (!d.d || (d.ldd % 4 == 0 && d.d_bs % 4 == 0 && al16(d.d))) &&
             (!d.d16 || (d.ld16 % 4 == 0 && d.d16_bs % 4 == 0 && (reinterpret_cast<uintptr_t>(d.d16) & 7u) == 0));
  if (d.split0 || d.split1) {
    const bool ok = d.split_ld % 4 == 0 && d.split_bs % 4 == 0 && d.split_plane % 4 == 0 &&
                    (!d.split0 || (reinterpret_cast<uintptr_t>(d.split0) & 7u) == 0) &&
                    (!d.split1 || (reinterpret_cast<uintptr_t>(d.split1) & 7u) == 0);
    p.vec_ok = p.vec_ok && ok;
  }
  p.S0 = static_cast<__half*>(d.split0); p.S1 = static_cast<__half*>(d.split1);
  p.s_ld = d.split_ld; p.s_bs = d.split_bs; p.s_plane = d.split_plane;
  p.s0_scale = d.split0_scale; p.s1_scale = d.split1_scale; p.s1_aff_a = d.split1_aff_a; p.s1_aff_b = d.split1_aff_b;
  p.maxres = d.maxres;
  p.sumsq = d.sumsq; p.maxabs = d.maxabs; p.maxaff = d.maxaff;
  p.aff_a = d.aff_a; p.aff_b = d.aff_b;
  p.status = ctx->status_dev;
  p.prof = ctx->prof_dev;

  const long long total = (long long)gemm_tiles_per_batch(d.m, d.n, bn, d.tri, pair ? 256 : kBM) * d.batch;
  if (total > 0x7fffffffLL) return fail(kErrArg, "gemm: too many tiles");
  const bool chained = p.promote > 0;
  if (pair) {
    const int pairs = (int)(total < ctx->gemm_sms / 2 ? total : ctx->gemm_sms / 2);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = bn == 512 ? GemmSmem<512, true>::kTotal : GemmSmem<256, true>::kTotal;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    if (bn == 512) TONER_CUDA(cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<512, false, true>, p));
    else if (chained) TONER_CUDA(cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<256, true, true>, p));
    else TONER_CUDA(cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<256, false, true>, p));
    count_launch();
    return 0;
  }
  const int grid = (int)(total < ctx->gemm_sms ? total : ctx->gemm_sms);
  if (bn == 256) {
    if (chained) gemm_tcgen05_kernel<256, true><<<grid, kGemmThreads, GemmSmem<256>::kTotal, stream>>>(p);
    else gemm_tcgen05_kernel<256, false><<<grid, kGemmThreads, GemmSmem<256>::kTotal, stream>>>(p);
  } else {
    if (chained) gemm_tcgen05_kernel<128, true><<<grid, kGemmThreads, GemmSmem<128>::kTotal, stream>>>(p);
    else gemm_tcgen05_kernel<128, false><<<grid, kGemmThreads, GemmSmem<128>::kTotal, stream>>>(p);
  }
  count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

// A wait that nothing will ever satisfy: the barrier expects one arrival and gets none.  The wait gives up after
// `limit_cycles`, reports through the status word like the GEMM's waits do, and the kernel returns normally.
__global__ void bounded_wait_selftest_kernel(long long limit_cycles, int* status) {
  __shared__ unsigned long long bar;
  const uint32_t b = ptx::smem_u32(&bar);
  if (threadIdx.x == 0) {
    ptx::mbar_init(b, 1);
    ptx::fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0 && !ptx::mbar_wait(b, 0, limit_cycles)) report(status, kTimeoutSelftest);
}

}  // namespace toner

// ------------------------------------------------------------------ C ABI: library + generic GEMM
extern "C" {

int toner_init(int device) {
  if (cudaSetDevice(device) != cudaSuccess) return toner::fail(toner::kErrCuda, "cudaSetDevice failed");
  return toner::context() ? 0 : toner::kErrCuda;
}

const char* toner_last_error(void) {
  return toner::g_error.c_str();
}

long long toner_launch_count(void) { return toner::g_launches.load(std::memory_order_relaxed); }

int toner_sm_count(void) {
  toner::Context* c = toner::context();
  return c ? c->num_sms : 0;
}

int toner_set_gemm_sm_limit(int32_t sms) {
  toner::Context* c = toner::context();
  if (!c) return toner::kErrCuda;
  if (sms < 0) return toner::fail(toner::kErrArg, "gemm sm limit: must be 0 (all) or a positive count");
  int n = sms == 0 || sms > c->num_sms ? c->num_sms : sms;
  n &= ~1;  // CTA pairs
  c->gemm_sms = n < 2 ? 2 : n;
  return 0;
}

int toner_device_status(void* stream, int* status_out) {
  toner::Context* c = toner::context();
  if (!c) return toner::kErrCuda;
  if (!status_out) return toner::fail(toner::kErrArg, "status_out is null");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int v = 0;
  TONER_CUDA(cudaMemcpyAsync(&v, c->status_dev, sizeof(int), cudaMemcpyDeviceToHost, s));
  TONER_CUDA(cudaStreamSynchronize(s));
  if (v != 0) TONER_CUDA(cudaMemsetAsync(c->status_dev, 0, sizeof(int), s));
  *status_out = v;
  return 0;
}

int toner_status_snapshot(int32_t* host_out, void* stream) {
  toner::Context* c = toner::context();
  if (!c) return toner::kErrCuda;
  if (!host_out) return toner::fail(toner::kErrArg, "status_snapshot: host_out is null");
  TONER_CUDA(cudaMemcpyAsync(host_out, c->status_dev, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)));
  return 0;
}

int toner_selftest_bounded_wait(long long limit_cycles, void* stream) {
  toner::Context* c = toner::context();
  if (!c) return toner::kErrCuda;
  if (limit_cycles <= 0 || limit_cycles > 2000000000LL)
    return toner::fail(toner::kErrArg, "selftest: the limit must be between 1 and 2e9 cycles");
  toner::bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_cycles, c->status_dev);
  toner::count_launch();
  TONER_CUDA(cudaGetLastError());
  return 0;
}

int toner_gemm_phase_cycles(int enable, void* stream, unsigned long long* out8) {
  toner::Context* c = toner::context();
  if (!c) return toner::kErrCuda;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (out8) {
    for (int i = 0; i < 8; ++i) out8[i] = 0;
    if (c->prof_dev) {
      TONER_CUDA(cudaMemcpyAsync(out8, c->prof_dev, 8 * sizeof(unsigned long long), cudaMemcpyDeviceToHost, s));
      TONER_CUDA(cudaStreamSynchronize(s));
      TONER_CUDA(cudaMemsetAsync(c->prof_dev, 0, 8 * sizeof(unsigned long long), s));
    }
  }
  if (enable && !c->prof_dev) {
    TONER_CUDA(cudaMalloc(&c->prof_dev, 8 * sizeof(unsigned long long)));
    TONER_CUDA(cudaMemset(c->prof_dev, 0, 8 * sizeof(unsigned long long)));
  } else if (!enable && c->prof_dev) {
    TONER_CUDA(cudaStreamSynchronize(s));
    TONER_CUDA(cudaFree(c->prof_dev));
    c->prof_dev = nullptr;
  }
  return 0;
}

int toner_gemm(const toner_gemm_desc* desc, void* stream) {
  if (!desc) return toner::fail(toner::kErrArg, "gemm: null descriptor");
  return toner::launch_gemm(*desc, static_cast<cudaStream_t>(stream));
}

}  // extern "C"

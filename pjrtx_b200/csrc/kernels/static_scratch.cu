// Streaming contraction for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need a contraction: a runtime that
// has already handed all device memory to its own arena, a callback running inside another framework's
// allocator lock, or a latency-critical serving loop that forbids allocator traffic after start-up. The
// split-K streaming kernel normally borrows scratch (f32 partial sums and per-tile arrival counters) from the
// executable that owns it; here the scratch lives in a fixed array inside the library image instead, so the
// entry point below touches no allocator at all. The price: the array has a fixed size (problems that need more
// are refused), every GPU that loads the library carries it until the process exits, and all calls share it.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>

#include "../common.h"
#include "kernels.h"
#include "stream_tma.cuh"

namespace pjrtx {

// 8 MiB of partial sums + 64 KiB of counters + one error word. Enough for m <= 8 against any rhs up to the
// 4096 x 128256 vocabulary projection (501 column tiles x 2 contributors x 8 rows x 1 KiB = 7.8 MiB).
constexpr size_t kStaticPartialBytes = 8u << 20;
constexpr size_t kStaticCounterBytes = 64u << 10;
constexpr size_t kStaticScratchBytes = kStaticPartialBytes + kStaticCounterBytes + 256;

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
unsigned char* g_scratch_address[kMaxDevices] = {nullptr};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Once per device, with that device current: resolve the array's device address and raise the kernels'
// dynamic shared-memory limit. Neither call allocates.
unsigned char* setup_device(int device) {
  std::lock_guard<std::mutex> lock(g_setup_mu);
  if (g_scratch_address[device]) return g_scratch_address[device];
  unsigned char* ptr = nullptr;
  cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
  if (e != cudaSuccess || !ptr) {
    set_last_error("cudaGetSymbolAddress(static scratch) on device %d: %s", device, cudaGetErrorString(e));
    return nullptr;
  }
#define RAISE(T, M)                                                                                                          \
  if ((e = cudaFuncSetAttribute(tma::stream_tma_kernel<T, M, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)) !=   \
      cudaSuccess) {                                                                                                         \
    set_last_error("cudaFuncSetAttribute: %s", cudaGetErrorString(e));                                                       \
    return nullptr;                                                                                                          \
  }
  RAISE(float, 1) RAISE(float, 2) RAISE(float, 4) RAISE(float, 8)
  RAISE(__half, 1) RAISE(__half, 2) RAISE(__half, 4) RAISE(__half, 8)
  RAISE(__nv_bfloat16, 1) RAISE(__nv_bfloat16, 2) RAISE(__nv_bfloat16, 4) RAISE(__nv_bfloat16, 8)
#undef RAISE
  g_scratch_address[device] = ptr;
  return ptr;
}

// Makes `device` current for the lifetime of the object and restores the caller's device afterwards.
struct CurrentDevice {
  int previous = -1;
  bool ok = false;
  explicit CurrentDevice(int device) {
    if (cudaGetDevice(&previous) != cudaSuccess) previous = -1;
    ok = cudaSetDevice(device) == cudaSuccess;
  }
  ~CurrentDevice() {
    if (previous >= 0) cudaSetDevice(previous);
  }
};

template <typename T>
int launch(const DotShape& s, const DotScratch& plan, const void* lhs, const void* rhs, void* out, unsigned char* scratch,
           cudaStream_t stream) {
  constexpr int V = 16 / sizeof(T);
  constexpr int COLS = 32 * V;
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) {
    set_last_error("cuTensorMapEncodeTiled is not available");
    return 0;
  }
  tma::Params p{};
  tma::Maps maps{};
  p.segments = 1;
  p.barrier = nullptr;
  tma::Segment& sg = p.seg[0];
  sg.lhs = lhs;
  sg.lhs2 = nullptr;
  sg.lhs_m = s.lhs_m;
  sg.lhs_k = s.lhs_k;
  sg.lhs_kind = tma::kLhsPlain;
  sg.m = (int)s.m;
  sg.k = (int)s.k;
  sg.count = 1;
  const int tiles = (int)((s.n + COLS - 1) / COLS);
  for (int g = 0; g <= tma::kGroupMax; g++) sg.tile_begin[g] = g == 0 ? 0 : tiles;
  sg.out[0] = out;
  sg.residual[0] = nullptr;
  sg.n[0] = s.n;
  const CUtensorMapDataType dt = sizeof(T) == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : s.dtype == kF16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  cuuint64_t gdim[2] = {(cuuint64_t)s.n, (cuuint64_t)s.k};
  cuuint64_t gstride[1] = {(cuuint64_t)s.rhs_k * sizeof(T)};
  cuuint32_t box[2] = {(cuuint32_t)COLS, (cuuint32_t)tma::kUnitRows};
  cuuint32_t estr[2] = {1, 1};
  if (((EncodeTiledFn)fn)(&maps.map[0][0], dt, 2, const_cast<void*>(rhs), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
    set_last_error("tensor map encoding failed (rhs must be 16-byte aligned with a row pitch that is a multiple of 16 bytes)");
    return 0;
  }
  for (int q = 0; q < tma::kSegmentMax; q++)
    for (int g = 0; g < tma::kGroupMax; g++) maps.map[q][g] = maps.map[0][0];
  sg.chunks = (int)((s.k + tma::kUnitRows - 1) / tma::kUnitRows);
  sg.units = (long long)tiles * sg.chunks;
  sg.max_contrib = plan.max_contrib;
  sg.partials = reinterpret_cast<float*>(scratch);
  sg.counters = reinterpret_cast<unsigned*>(scratch + kStaticPartialBytes);
  p.error_flag = reinterpret_cast<int*>(scratch + kStaticPartialBytes + kStaticCounterBytes);
  p.timeout_ns = tma::kDefaultTimeoutNs;
  p.stages = plan.stages;
  p.early_rhs = 0;
  p.evict_first = 1;
  // The array keeps whatever the previous call left: counters and the error word must start at zero.
  if (cudaMemsetAsync(scratch + kStaticPartialBytes, 0, kStaticCounterBytes + 256, stream) != cudaSuccess) {
    set_last_error("clearing the static scratch counters failed");
    return 0;
  }
  const int M = s.m <= 1 ? 1 : s.m <= 2 ? 2 : s.m <= 4 ? 4 : 8;
  cudaError_t e;
#define GO(MM) tma::stream_tma_kernel<T, MM, false><<<plan.grid, tma::kThreads, plan.smem, stream>>>(p, maps)
  if (M == 1) GO(1); else if (M == 2) GO(2); else if (M == 4) GO(4); else GO(8);
#undef GO
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_last_error("static-scratch contraction launch failed: %s", cudaGetErrorString(e));
    return 0;
  }
  return 1;
}

}  // namespace

int stream_dot_static_scratch(int device, int dtype, const void* lhs, const void* rhs, void* out, int64_t m, int64_t k, int64_t n,
                              cudaStream_t stream) {
  if (device < 0 || device >= kMaxDevices) {
    set_last_error("device ordinal %d is out of range", device);
    return 0;
  }
  const size_t esize = dtype_size(dtype);
  if (!dtype_is_float(dtype)) {
    set_last_error("static-scratch contraction supports f32, f16 and bf16");
    return 0;
  }
  const int V = (int)(16 / esize);
  if (!lhs || !rhs || !out || m < 1 || m > 8 || k < 1 || n < 1 || n % V != 0 || ((uintptr_t)rhs & 15) || ((uintptr_t)out & 15)) {
    set_last_error("static-scratch contraction needs 1 <= m <= 8, k >= 1, n a multiple of %d, and 16-byte aligned rhs/out", V);
    return 0;
  }
  CurrentDevice scope(device);  // the caller's current device is put back when the call returns
  if (!scope.ok) {
    set_last_error("cudaSetDevice(%d) failed", device);
    return 0;
  }
  unsigned char* scratch = setup_device(device);
  if (!scratch) return 0;
  int sm_count = 148;
  if (cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) sm_count = 148;
  DotShape s;
  s.dtype = dtype;
  s.m = m;
  s.k = k;
  s.n = n;
  s.lhs_m = k;
  s.lhs_k = 1;
  s.rhs_k = n;
  s.rhs_n = 1;
  s.out_m = n;
  const DotScratch plan = dot_group_plan(&s, 1, sm_count, /*allow_tensor=*/false);
  if (!plan.tma || plan.partial_bytes > kStaticPartialBytes || plan.counter_bytes > kStaticCounterBytes) {
    set_last_error("contraction m=%lld k=%lld n=%lld needs %llu bytes of partial sums and %llu bytes of counters; the static "
                   "scratch holds %zu and %zu",
                   (long long)m, (long long)k, (long long)n, (unsigned long long)plan.partial_bytes,
                   (unsigned long long)plan.counter_bytes, kStaticPartialBytes, kStaticCounterBytes);
    return 0;
  }
  switch (dtype) {
    case kF32: return launch<float>(s, plan, lhs, rhs, out, scratch, stream);
    case kF16: return launch<__half>(s, plan, lhs, rhs, out, scratch, stream);
    default: return launch<__nv_bfloat16>(s, plan, lhs, rhs, out, scratch, stream);
  }
}

// The kernel's bounded waits report through an error word inside the static array (the call clears it before the
// launch). Reading it back is one 4-byte copy into a stack variable followed by a wait on the caller's stream: no
// allocation here either.
int stream_dot_static_scratch_status(int device, cudaStream_t stream) {
  if (device < 0 || device >= kMaxDevices) {
    set_last_error("device ordinal %d is out of range", device);
    return 0;
  }
  CurrentDevice scope(device);
  if (!scope.ok) {
    set_last_error("cudaSetDevice(%d) failed", device);
    return 0;
  }
  unsigned char* scratch = setup_device(device);
  if (!scratch) return 0;
  int code = 0;
  cudaError_t e = cudaMemcpyAsync(&code, scratch + kStaticPartialBytes + kStaticCounterBytes, sizeof(int), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) {
    set_last_error("reading the static-scratch status failed: %s", cudaGetErrorString(e));
    return 0;
  }
  if (code != 0) {
    set_last_error("the last static-scratch contraction on device %d gave up a bounded wait (code %d); its output is not valid",
                   device, code);
    return 0;
  }
  return 1;
}

}  // namespace pjrtx

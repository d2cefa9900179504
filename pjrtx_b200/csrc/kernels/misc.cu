// dynamic_update_slice and split-KV attention kernels for sm_100a.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../common.h"
#include "kernels.h"

namespace pjrtx {

namespace {

__device__ __forceinline__ int64_t load_index(const void* p, int dtype) {
  switch (dtype) {
    case kS32: return *static_cast<const int32_t*>(p);
    case kU32: return *static_cast<const uint32_t*>(p);
    case kS64: return *static_cast<const int64_t*>(p);
    case kU64: return (int64_t)*static_cast<const uint64_t*>(p);
    case kS8: return *static_cast<const int8_t*>(p);
    case kU8: return *static_cast<const uint8_t*>(p);
    case kS16: return *static_cast<const int16_t*>(p);
    case kU16: return *static_cast<const uint16_t*>(p);
    default: return 0;
  }
}

struct DusArgs {
  int rank;
  int unit;             // bytes moved per thread step
  int64_t upd_units[8];  // update dims, innermost in units
  int64_t dst_units[8];
  int64_t dst_dims[8];   // element dims for clamping
  int64_t upd_dims[8];
  int start_dtype[8];
  const void* start[8];
  int64_t last_scale;    // units per index step along the innermost kept axis
  int64_t total_units;
};

// Start indices are clamped to [0, dst_dim - upd_dim] as StableHLO specifies
// (the reference passes them to MLX slice_update, src/backend/mlx_metal/api.cc:2552-2635).
template <typename U>
__global__ void dus_kernel(DusArgs a, U* __restrict__ dst, const U* __restrict__ upd) {
  PJRTX_PDL_PROLOGUE();
  __shared__ int64_t start[8];
  if (threadIdx.x < a.rank) {
    const int d = threadIdx.x;
    int64_t s = a.start[d] ? load_index(a.start[d], a.start_dtype[d]) : 0;
    const int64_t hi = a.dst_dims[d] - a.upd_dims[d];
    s = s < 0 ? 0 : (s > hi ? hi : s);
    start[d] = (d == a.rank - 1) ? s * a.last_scale : s;
  }
  __syncthreads();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < a.total_units; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t rem = i, off = 0, stride = 1;
    for (int d = a.rank - 1; d >= 0; d--) {
      const int64_t c = rem % a.upd_units[d];
      rem /= a.upd_units[d];
      off += (c + start[d]) * stride;
      stride *= a.dst_units[d];
    }
    dst[off] = upd[i];
  }
}

// ------------------------------------------------------------------ attention
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

struct AttnArgs {
  int64_t batch, q_len, heads, kv_len, kv_heads, head_dim;
  int token_dtype;
  float scale;
};

// One thread per (batch, query, head): two passes over the keys, scores held
// only as running max / sum. Correctness path for any head_dim and dtype
// (the reference's generated attention kernel has the same shape:
// src/backend/mlx_metal/executable_metal_graph_custom_call.zig:126-219).
template <typename T>
__global__ void sdpa_simple_kernel(AttnArgs a, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                   const void* __restrict__ token, T* __restrict__ out) {
  PJRTX_PDL_PROLOGUE();
  const int64_t total = a.batch * a.q_len * a.heads;
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  const int64_t h = t % a.heads, qi = (t / a.heads) % a.q_len, b = t / (a.heads * a.q_len);
  const int64_t g = h / (a.heads / a.kv_heads);
  int64_t limit = load_index(token, a.token_dtype) + qi;  // keys 0..limit are visible
  if (limit >= a.kv_len) limit = a.kv_len - 1;
  const T* qp = q + ((b * a.q_len + qi) * a.heads + h) * a.head_dim;
  T* op = out + ((b * a.q_len + qi) * a.heads + h) * a.head_dim;
  const T* kb = k + (b * a.kv_len * a.kv_heads + g) * a.head_dim;
  const T* vb = v + (b * a.kv_len * a.kv_heads + g) * a.head_dim;
  const int64_t row = a.kv_heads * a.head_dim;
  float m = -INFINITY;
  for (int64_t j = 0; j <= limit; j++) {
    float s = 0.f;
    for (int64_t d = 0; d < a.head_dim; d++) s = fmaf(to_f(qp[d]), to_f(kb[j * row + d]), s);
    m = fmaxf(m, s * a.scale);
  }
  float l = 0.f;
  for (int64_t j = 0; j <= limit; j++) {
    float s = 0.f;
    for (int64_t d = 0; d < a.head_dim; d++) s = fmaf(to_f(qp[d]), to_f(kb[j * row + d]), s);
    l += expf(s * a.scale - m);
  }
  for (int64_t d = 0; d < a.head_dim; d++) {
    float acc = 0.f;
    for (int64_t j = 0; j <= limit; j++) {
      float s = 0.f;
      for (int64_t e = 0; e < a.head_dim; e++) s = fmaf(to_f(qp[e]), to_f(kb[j * row + e]), s);
      acc = fmaf(expf(s * a.scale - m), to_f(vb[j * row + d]), acc);
    }
    op[d] = from_f<T>(limit < 0 ? 0.f : acc / l);
  }
}

}  // namespace

int dus_launch(const SliceUpdateShape& s, void* dst, const void* update, const void* const* start_ptrs, bool pdl,
               cudaStream_t stream) {
  if (s.rank < 0 || s.rank > 8 || s.elem_size <= 0) return 0;
  int64_t upd[8] = {1}, dstd[8] = {1};
  const int rank = s.rank == 0 ? 1 : s.rank;
  int64_t total = 1;
  for (int d = 0; d < s.rank; d++) {
    upd[d] = s.upd_dims[d];
    dstd[d] = s.dst_dims[d];
    total *= upd[d];
  }
  if (total == 0) return 1;
  // Trailing axes the update covers completely have start 0; fold them into
  // the last axis that can move so each thread copies one contiguous unit.
  int t = rank - 1;
  int64_t covered = 1;
  while (t > 0 && upd[t] == dstd[t]) {
    covered *= upd[t];
    t--;
  }
  int unit = s.elem_size;
  if ((covered * s.elem_size) % 16 == 0) unit = 16;
  else if (upd[t] == dstd[t] && (upd[t] * covered * s.elem_size) % 16 == 0) unit = 16;
  DusArgs k{};
  k.rank = t + 1;
  k.unit = unit;
  for (int d = 0; d <= t; d++) {
    k.upd_dims[d] = upd[d];
    k.dst_dims[d] = dstd[d];
    k.upd_units[d] = upd[d];
    k.dst_units[d] = dstd[d];
    k.start_dtype[d] = s.rank == 0 ? 0 : s.start_dtype[d];
    k.start[d] = s.rank == 0 ? nullptr : start_ptrs[d];
  }
  k.upd_units[t] = upd[t] * covered * s.elem_size / unit;
  k.dst_units[t] = dstd[t] * covered * s.elem_size / unit;
  // Units per step of the start index along axis t (0 when that axis is fully covered).
  k.last_scale = upd[t] == dstd[t] ? 0 : covered * s.elem_size / unit;
  k.total_units = 1;
  for (int d = 0; d <= t; d++) k.total_units *= k.upd_units[d];
  const unsigned blocks = (unsigned)std::min<int64_t>((k.total_units + 255) / 256, 148 * 16);
  switch (unit) {
    case 16: launch_kernel(dus_kernel<uint4>, dim3(blocks), dim3(256), 0, stream, pdl, k, (uint4*)dst, (const uint4*)update); break;
    case 8: launch_kernel(dus_kernel<uint2>, dim3(blocks), dim3(256), 0, stream, pdl, k, (uint2*)dst, (const uint2*)update); break;
    case 4: launch_kernel(dus_kernel<uint32_t>, dim3(blocks), dim3(256), 0, stream, pdl, k, (uint32_t*)dst, (const uint32_t*)update); break;
    case 2: launch_kernel(dus_kernel<uint16_t>, dim3(blocks), dim3(256), 0, stream, pdl, k, (uint16_t*)dst, (const uint16_t*)update); break;
    case 1: launch_kernel(dus_kernel<uint8_t>, dim3(blocks), dim3(256), 0, stream, pdl, k, (uint8_t*)dst, (const uint8_t*)update); break;
    default: return 0;
  }
  return 1;
}

int sdpa_launch(const SdpaShape& s, const void* q, const void* k, const void* v, const void* token_index, void* out,
                bool pdl, cudaStream_t stream) {
  AttnArgs a{s.batch, s.q_len, s.heads, s.kv_len, s.kv_heads, s.head_dim, s.token_dtype,
             1.0f / sqrtf((float)s.head_dim)};
  const int64_t total = s.batch * s.q_len * s.heads;
  if (total == 0) return 1;
  const unsigned blocks = (unsigned)((total + 63) / 64);
  switch (s.dtype) {
    case kF32: launch_kernel(sdpa_simple_kernel<float>, dim3(blocks), dim3(64), 0, stream, pdl, a, (const float*)q, (const float*)k, (const float*)v, token_index, (float*)out); break;
    case kF16: launch_kernel(sdpa_simple_kernel<__half>, dim3(blocks), dim3(64), 0, stream, pdl, a, (const __half*)q, (const __half*)k, (const __half*)v, token_index, (__half*)out); break;
    case kBF16: launch_kernel(sdpa_simple_kernel<__nv_bfloat16>, dim3(blocks), dim3(64), 0, stream, pdl, a, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, token_index, (__nv_bfloat16*)out); break;
    default: return 0;
  }
  return 1;
}

}  // namespace pjrtx

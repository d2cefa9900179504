// dot_general kernels for sm_100a.
//
// Four paths behind one canonical contraction out[b0,b1,m,n] = sum_k lhs*rhs
// (the reference reaches MLX matmul/tensordot for the same op,
// src/backend/mlx_metal/api.cc:3349-3498; its generated kernels are the
// one-thread-per-output and 256-thread tiled dots of
// src/backend/mlx_metal/metal_graph_dot.zig:46-64 and :199-256):
//   1  stream_kn : m <= 8, rhs[K,N] with N contiguous. Bandwidth-bound GEMV /
//                  skinny GEMM: 16-byte loads of rhs rows, f32 accumulators in
//                  registers, K split over warps and CTAs, deterministic
//                  last-CTA fold of the f32 partials.
//   2  stream_nk : m <= 8, rhs[N,K] with K contiguous (attention scores, tied
//                  heads): lane groups own output columns and shuffle-reduce.
//   3  tile      : shared-memory tiled FFMA contraction with f32 accumulate,
//                  any strides (f32 matmul at 1e-5 needs real FFMA, not TF32).
//   0  generic   : one thread per output element, any strides, any m.
// 16-bit floats without batch axes whose operands a TMA tensor map can describe run on the tensor cores instead
// (umma_gemm.cuh): rhs[K,N] as a variant of path 1 (so that q/k/v and gate/up still share one launch), rhs[N,K] as
// path 4. PJRTX_B200_UMMA=0 turns that off; PJRTX_B200_UMMA_MIN_M (default 3: measured on the
// 8B decode shapes the CUDA-core kernel is ahead for one and two rows only) keeps the CUDA-core streaming kernels below that m.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "../common.h"
#include "kernels.h"
#include "stream_tma.cuh"
#include "umma_gemm.cuh"

namespace pjrtx {

namespace {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Sixteen bytes of T held in registers; get(i) unpacks without taking an address
// so the value never leaves the register file.
__device__ __forceinline__ unsigned word_of(const uint4& r, int i) { return i == 0 ? r.x : i == 1 ? r.y : i == 2 ? r.z : r.w; }
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  uint4 raw;
  __device__ __forceinline__ float get(int i) const { return __uint_as_float(word_of(raw, i)); }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ float get(int i) const {
    const unsigned u = word_of(raw, i >> 1);
    return __uint_as_float((i & 1) ? (u & 0xffff0000u) : (u << 16));
  }
};
template <> struct Vec16<__half> {
  static constexpr int N = 8;
  uint4 raw;
  __device__ __forceinline__ float get(int i) const {
    const unsigned u = word_of(raw, i >> 1);
    return __half2float(__ushort_as_half((unsigned short)((i & 1) ? (u >> 16) : (u & 0xffffu))));
  }
};

// Streaming 16-byte load that does not pollute L1 (weights are read once).
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// ---------------------------------------------------------------- generic
template <typename T>
__global__ void dot_generic_kernel(DotShape s, const T* __restrict__ lhs, const T* __restrict__ rhs, T* __restrict__ out) {
  PJRTX_PDL_PROLOGUE();
  const int64_t total = s.b0 * s.b1 * s.m * s.n;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t n = i % s.n, m = (i / s.n) % s.m, b1 = (i / (s.n * s.m)) % s.b1, b0 = i / (s.n * s.m * s.b1);
    const T* a = lhs + b0 * s.lhs_b0 + b1 * s.lhs_b1 + m * s.lhs_m;
    const T* b = rhs + b0 * s.rhs_b0 + b1 * s.rhs_b1 + n * s.rhs_n;
    float acc = 0.f;
    for (int64_t k = 0; k < s.k; k++) acc = fmaf(to_f(a[k * s.lhs_k]), to_f(b[k * s.rhs_k]), acc);
    out[b0 * s.out_b0 + b1 * s.out_b1 + m * s.out_m + n] = from_f<T>(acc);
  }
}

// ---------------------------------------------------------------- stream_kn
constexpr int kKnUnroll = 8;
constexpr int kKnChunk = 512;  // lhs elements staged in shared memory per pass

// Up to four contractions that share lhs, m and k run as one launch: the column
// tiles of all of them form one grid (q/k/v or gate/up projections; the reference
// groups dots that share an lhs the same way, src/backend/mlx_metal/metal_graph_dot.zig:70-152).
struct KnGroup {
  int count;
  int tile_begin[kDotGroupMax + 1];
  const void* rhs[kDotGroupMax];
  void* out[kDotGroupMax];
  long long n[kDotGroupMax];
  long long rhs_k[kDotGroupMax];
  long long partial_offset[kDotGroupMax];  // in floats
};

template <typename T, int M, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
stream_kn_kernel(DotShape s, KnGroup grp, const T* __restrict__ lhs, float* __restrict__ partials,
                 unsigned* __restrict__ counters, int ksplit, int kslice) {
  PJRTX_PDL_PROLOGUE();
  constexpr int V = Vec16<T>::N;
  constexpr int TILE = 32 * V;
  constexpr int THREADS = WARPS * 32;
  __shared__ float red[WARPS - 1][M][TILE];
  __shared__ T xs[M][kKnChunk];
  __shared__ int is_last;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int g = 0;
#pragma unroll
  for (int q = 1; q < kDotGroupMax; q++)
    if (q < grp.count && (int)blockIdx.x >= grp.tile_begin[q]) g = q;
  const int64_t n_cols = grp.n[g], ldb = grp.rhs_k[g];
  const int64_t batch = blockIdx.z, b0 = batch / s.b1, b1 = batch % s.b1;
  const int64_t col = (int64_t)((int)blockIdx.x - grp.tile_begin[g]) * TILE + lane * V;
  const int64_t k_begin = (int64_t)blockIdx.y * kslice;
  const int64_t k_end = min(k_begin + (int64_t)kslice, s.k);
  const T* a = lhs + b0 * s.lhs_b0 + b1 * s.lhs_b1;
  const T* b = static_cast<const T*>(grp.rhs[g]) + b0 * s.rhs_b0 + b1 * s.rhs_b1;
  T* out = static_cast<T*>(grp.out[g]);
  const int rows = (int)min((int64_t)M, s.m);

  float acc[M][V];
#pragma unroll
  for (int m = 0; m < M; m++)
#pragma unroll
    for (int v = 0; v < V; v++) acc[m][v] = 0.f;

  const bool col_ok = col < n_cols;
  for (int64_t kc = k_begin; kc < k_end; kc += kKnChunk) {
    const int chunk = (int)min((int64_t)kKnChunk, k_end - kc);
    __syncthreads();
    for (int idx = threadIdx.x; idx < rows * chunk; idx += THREADS) {
      const int m = idx / chunk, kk = idx % chunk;
      xs[m][kk] = a[m * s.lhs_m + (kc + kk) * s.lhs_k];
    }
    __syncthreads();
    if (col_ok) {
      const T* bp = b + (kc + warp) * ldb + col;
      int kk = warp;
      for (; kk + (kKnUnroll - 1) * WARPS < chunk; kk += kKnUnroll * WARPS) {
        Vec16<T> w[kKnUnroll];
#pragma unroll
        for (int u = 0; u < kKnUnroll; u++) w[u].raw = ld_stream(bp + (int64_t)u * WARPS * ldb);
        bp += (int64_t)kKnUnroll * WARPS * ldb;
#pragma unroll
        for (int u = 0; u < kKnUnroll; u++)
#pragma unroll
          for (int m = 0; m < M; m++) {
            const float x = to_f(xs[m][kk + u * WARPS]);
#pragma unroll
            for (int v = 0; v < V; v++) acc[m][v] = fmaf(x, w[u].get(v), acc[m][v]);
          }
      }
      for (; kk < chunk; kk += WARPS) {
        Vec16<T> w;
        w.raw = ld_stream(bp);
        bp += (int64_t)WARPS * ldb;
#pragma unroll
        for (int m = 0; m < M; m++) {
          const float x = to_f(xs[m][kk]);
#pragma unroll
          for (int v = 0; v < V; v++) acc[m][v] = fmaf(x, w.get(v), acc[m][v]);
        }
      }
    }
  }
  // Fold the warps of this CTA in a fixed order.
  if (warp > 0) {
#pragma unroll
    for (int m = 0; m < M; m++)
#pragma unroll
      for (int v = 0; v < V; v++) red[warp - 1][m][lane * V + v] = acc[m][v];
  }
  __syncthreads();
  float* part = partials + grp.partial_offset[g];
  if (warp == 0 && col_ok) {
#pragma unroll
    for (int m = 0; m < M; m++)
#pragma unroll
      for (int v = 0; v < V; v++) {
        float t = acc[m][v];
#pragma unroll
        for (int w = 0; w < WARPS - 1; w++) t += red[w][m][lane * V + v];
        acc[m][v] = t;
      }
    if (ksplit == 1) {
#pragma unroll
      for (int m = 0; m < M; m++) {
        if (m < rows) {
          T* o = out + b0 * s.out_b0 + b1 * s.out_b1 + m * n_cols + col;
#pragma unroll
          for (int v = 0; v < V; v++) o[v] = from_f<T>(acc[m][v]);
        }
      }
    } else {
      float* p = part + ((batch * ksplit + blockIdx.y) * (int64_t)M) * n_cols + col;
#pragma unroll
      for (int m = 0; m < M; m++)
        if (m < rows) {
#pragma unroll
          for (int v = 0; v < V; v++) p[(int64_t)m * n_cols + v] = acc[m][v];
        }
    }
  }
  if (ksplit == 1) return;
  // The CTA that arrives last for this column tile folds the partials in slice order.
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(&counters[batch * gridDim.x + blockIdx.x], 1u);
    is_last = prev == (unsigned)ksplit - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  const int64_t slice_stride = (int64_t)M * n_cols;
  for (int idx = threadIdx.x; idx < rows * TILE; idx += THREADS) {
    const int m = idx / TILE;
    const int64_t c = (int64_t)((int)blockIdx.x - grp.tile_begin[g]) * TILE + idx % TILE;
    if (c >= n_cols) continue;
    const float* p = part + (batch * ksplit * (int64_t)M + m) * n_cols + c;
    float t = 0.f;
    int ks = 0;
    for (; ks + 8 <= ksplit; ks += 8) {  // loads first, then the adds in slice order
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; u++) v[u] = __ldcg(p + (int64_t)(ks + u) * slice_stride);
#pragma unroll
      for (int u = 0; u < 8; u++) t += v[u];
    }
    for (; ks < ksplit; ks++) t += __ldcg(p + (int64_t)ks * slice_stride);
    out[b0 * s.out_b0 + b1 * s.out_b1 + m * n_cols + c] = from_f<T>(t);
  }
  if (threadIdx.x == 0) counters[batch * gridDim.x + blockIdx.x] = 0;  // ready for the next launch
}

// ---------------------------------------------------------------- stream_nk
template <typename T, int M>
__global__ void __launch_bounds__(256)
stream_nk_kernel(DotShape s, const T* __restrict__ lhs, const T* __restrict__ rhs, T* __restrict__ out, int group) {
  PJRTX_PDL_PROLOGUE();
  constexpr int V = Vec16<T>::N;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rows_per_warp = 32 / group;
  const int64_t batch = blockIdx.y, b0 = batch / s.b1, b1 = batch % s.b1;
  const int64_t n = ((int64_t)blockIdx.x * 8 + warp) * rows_per_warp + lane / group;
  const int gl = lane % group;
  const T* a = lhs + b0 * s.lhs_b0 + b1 * s.lhs_b1;
  const T* b = rhs + b0 * s.rhs_b0 + b1 * s.rhs_b1 + n * s.rhs_n;
  const int rows = (int)min((int64_t)M, s.m);
  float acc[M];
#pragma unroll
  for (int m = 0; m < M; m++) acc[m] = 0.f;
  if (n < s.n) {
    for (int64_t k = (int64_t)gl * V; k < s.k; k += (int64_t)group * V) {
      Vec16<T> w;
      w.raw = ld_stream(b + k);
#pragma unroll
      for (int m = 0; m < M; m++) {
        if (m < rows) {
          Vec16<T> x;
          x.raw = __ldg(reinterpret_cast<const uint4*>(a + m * s.lhs_m + k));
#pragma unroll
          for (int v = 0; v < V; v++) acc[m] = fmaf(x.get(v), w.get(v), acc[m]);
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < M; m++)
    for (int o = group >> 1; o > 0; o >>= 1) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], o);
  if (n < s.n && gl == 0) {
#pragma unroll
    for (int m = 0; m < M; m++)
      if (m < rows) out[b0 * s.out_b0 + b1 * s.out_b1 + m * s.out_m + n] = from_f<T>(acc[m]);
  }
}

// ---------------------------------------------------------------- tile
constexpr int kTile = 64, kTileK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
tile_kernel(DotShape s, const T* __restrict__ lhs, const T* __restrict__ rhs, T* __restrict__ out) {
  PJRTX_PDL_PROLOGUE();
  __shared__ float As[kTileK][kTile + 4];
  __shared__ float Bs[kTileK][kTile + 4];
  const int64_t batch = blockIdx.z, b0 = batch / s.b1, b1 = batch % s.b1;
  const T* a = lhs + b0 * s.lhs_b0 + b1 * s.lhs_b1;
  const T* b = rhs + b0 * s.rhs_b0 + b1 * s.rhs_b1;
  const int64_t m0 = (int64_t)blockIdx.y * kTile, n0 = (int64_t)blockIdx.x * kTile;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  float acc[4][4] = {};
  for (int64_t k0 = 0; k0 < s.k; k0 += kTileK) {
    for (int idx = threadIdx.x; idx < kTile * kTileK; idx += 256) {
      // Walk the contiguous axis fastest for both operands.
      int mm, kk;
      if (s.lhs_k == 1) { kk = idx % kTileK; mm = idx / kTileK; } else { mm = idx % kTile; kk = idx / kTile; }
      const int64_t gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < s.m && gk < s.k) ? to_f(a[gm * s.lhs_m + gk * s.lhs_k]) : 0.f;
      int nn;
      if (s.rhs_n == 1) { nn = idx % kTile; kk = idx / kTile; } else { kk = idx % kTileK; nn = idx / kTileK; }
      const int64_t gn = n0 + nn, gk2 = k0 + kk;
      Bs[kk][nn] = (gn < s.n && gk2 < s.k) ? to_f(b[gk2 * s.rhs_k + gn * s.rhs_n]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTileK; kk++) {
      float av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int64_t gm = m0 + ty * 4 + i;
    if (gm >= s.m) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int64_t gn = n0 + tx * 4 + j;
      if (gn < s.n) out[b0 * s.out_b0 + b1 * s.out_b1 + gm * s.out_m + gn] = from_f<T>(acc[i][j]);
    }
  }
}

// ---------------------------------------------------------------- f32 tile, register-blocked
// out[m, n] = sum_k lhs[m, k] * rhs[k, n] in true f32 (the parity bar for f32 contractions is rel 1e-5, which TF32
// products miss at k = 1024), for dense operands: lhs k-contiguous, rhs n-contiguous, 16-byte aligned rows.
// 128 x 64 output tile per CTA of 256 threads, 8 x 4 outputs per thread, k in slabs of 16: the next slab travels
// global -> registers while the current one is multiplied out of shared memory (two buffers, one barrier per slab).
// Per k step a thread issues three 16-byte shared loads (two broadcast, one conflict-free) for 32 FFMAs, so the FMA pipe
// is the limit. A 1024^3 product is 128 tiles: one wave of one CTA per SM.
constexpr int kSgBM = 128, kSgBN = 64, kSgBK = 16;

__global__ void __launch_bounds__(256, 2)
sgemm_kernel(DotShape s, const float* __restrict__ lhs, const float* __restrict__ rhs, float* __restrict__ out) {
  PJRTX_PDL_PROLOGUE();
  __shared__ __align__(16) float As[2][kSgBK][kSgBM + 4];
  __shared__ __align__(16) float Bs[2][kSgBK][kSgBN + 4];
  const int tid = threadIdx.x;
  const int64_t batch = blockIdx.z, b0 = batch / s.b1, b1 = batch % s.b1;
  const float* a = lhs + b0 * s.lhs_b0 + b1 * s.lhs_b1;
  const float* b = rhs + b0 * s.rhs_b0 + b1 * s.rhs_b1;
  float* o = out + b0 * s.out_b0 + b1 * s.out_b1;
  const int64_t m0 = (int64_t)blockIdx.y * kSgBM, n0 = (int64_t)blockIdx.x * kSgBN;
  // Global -> register mapping: A slab = 128 rows x 4 chunks of 4 k (two chunks per thread), B slab = 16 rows x 16
  // chunks of 4 n (one per thread).
  const int a_row[2] = {tid >> 2, (tid + 256) >> 2}, a_kc = tid & 3;
  const int b_row = tid >> 4, b_nc = tid & 15;
  float4 ra[2], rb;
  auto gload = [&](int64_t k0) {
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const int64_t gm = m0 + a_row[i], gk = k0 + a_kc * 4;
      if (gm < s.m && gk + 3 < s.k) {
        ra[i] = *reinterpret_cast<const float4*>(a + gm * s.lhs_m + gk);
      } else {
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) v[j] = (gm < s.m && gk + j < s.k) ? a[gm * s.lhs_m + gk + j] : 0.f;
        ra[i] = make_float4(v[0], v[1], v[2], v[3]);
      }
    }
    const int64_t gk = k0 + b_row, gn = n0 + b_nc * 4;
    if (gk < s.k && gn + 3 < s.n) {
      rb = *reinterpret_cast<const float4*>(b + gk * s.rhs_k + gn);
    } else {
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; j++) v[j] = (gk < s.k && gn + j < s.n) ? b[gk * s.rhs_k + gn + j] : 0.f;
      rb = make_float4(v[0], v[1], v[2], v[3]);
    }
  };
  auto sstore = [&](int buf) {
#pragma unroll
    for (int i = 0; i < 2; i++) {
      As[buf][a_kc * 4 + 0][a_row[i]] = ra[i].x;
      As[buf][a_kc * 4 + 1][a_row[i]] = ra[i].y;
      As[buf][a_kc * 4 + 2][a_row[i]] = ra[i].z;
      As[buf][a_kc * 4 + 3][a_row[i]] = ra[i].w;
    }
    *reinterpret_cast<float4*>(&Bs[buf][b_row][b_nc * 4]) = rb;
  };
  const int tx = tid & 15, ty = tid >> 4;  // outputs: rows ty * 8 .. + 7, columns tx * 4 .. + 3
  float acc[8][4] = {};
  const int64_t slabs = (s.k + kSgBK - 1) / kSgBK;
  gload(0);
  sstore(0);
  __syncthreads();
  for (int64_t t = 0; t < slabs; t++) {
    const int buf = (int)(t & 1);
    if (t + 1 < slabs) gload((t + 1) * kSgBK);
#pragma unroll
    for (int kk = 0; kk < kSgBK; kk++) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 8]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][kk][ty * 8 + 4]);
      const float4 bv = *reinterpret_cast<const float4*>(&Bs[buf][kk][tx * 4]);
      const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bw[j], acc[i][j]);
    }
    if (t + 1 < slabs) sstore(buf ^ 1);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; i++) {
    const int64_t gm = m0 + ty * 8 + i, gn = n0 + tx * 4;
    if (gm >= s.m) continue;
    float* dst = o + gm * s.out_m + gn;
    if (gn + 3 < s.n && (s.out_m & 3) == 0) {
      *reinterpret_cast<float4*>(dst) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    } else {
#pragma unroll
      for (int j = 0; j < 4; j++)
        if (gn + j < s.n) dst[j] = acc[i][j];
    }
  }
}

// True when the register-blocked f32 kernel can take the contraction as it lies in memory.
inline bool sgemm_ok(const DotShape& s, const void* lhs, const void* rhs, const void* out) {
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return s.dtype == kF32 && s.lhs_k == 1 && s.rhs_n == 1 && (s.lhs_m & 3) == 0 && (s.rhs_k & 3) == 0 && (s.lhs_b0 & 3) == 0 &&
         (s.lhs_b1 & 3) == 0 && (s.rhs_b0 & 3) == 0 && (s.rhs_b1 & 3) == 0 && (s.out_b0 & 3) == 0 && (s.out_b1 & 3) == 0 &&
         al16(lhs) && al16(rhs) && al16(out) && (s.m + kSgBM - 1) / kSgBM <= 65535;
}

template <typename T>
int launch_group_typed(const DotShape* shapes, int count, const DotScratch& plan, const void* lhs, const void* const* rhs,
                       void* const* out, void* partials, void* counters, bool pdl, cudaStream_t stream) {
  constexpr int V = 16 / sizeof(T);
  const int tile = 32 * V;
  const DotShape& s = shapes[0];
  const int M = s.m <= 1 ? 1 : s.m <= 2 ? 2 : s.m <= 4 ? 4 : 8;
  KnGroup grp{};
  grp.count = count;
  int tiles = 0;
  long long poff = 0;
  for (int g = 0; g < count; g++) {
    grp.tile_begin[g] = tiles;
    tiles += (int)((shapes[g].n + tile - 1) / tile);
    grp.rhs[g] = rhs[g];
    grp.out[g] = out[g];
    grp.n[g] = shapes[g].n;
    grp.rhs_k[g] = shapes[g].rhs_k;
    grp.partial_offset[g] = poff;
    poff += (long long)s.b0 * s.b1 * plan.ksplit * M * shapes[g].n;
  }
  for (int g = count; g <= kDotGroupMax; g++) grp.tile_begin[g] = tiles;
  dim3 grid((unsigned)tiles, (unsigned)plan.ksplit, (unsigned)(s.b0 * s.b1));
  const int kslice = (int)((s.k + plan.ksplit - 1) / plan.ksplit);
  const T* a = static_cast<const T*>(lhs);
  float* p = static_cast<float*>(partials);
  unsigned* c = static_cast<unsigned*>(counters);
  cudaError_t e;
#define KN(MM, WW) e = launch_kernel(stream_kn_kernel<T, MM, WW>, grid, dim3(WW * 32), 0, stream, pdl, s, grp, a, p, c, plan.ksplit, kslice)
  if (M == 1) KN(1, 8); else if (M == 2) KN(2, 8); else if (M == 4) KN(4, 8); else KN(8, 4);
#undef KN
  return e == cudaSuccess ? 1 : 0;
}

template <typename T>
int launch_typed(const DotShape& s, const DotScratch& plan, const void* lhs, const void* rhs, void* out, void* partials,
                 void* counters, bool pdl, cudaStream_t stream) {
  const T* a = static_cast<const T*>(lhs);
  const T* b = static_cast<const T*>(rhs);
  T* o = static_cast<T*>(out);
  constexpr int V = 16 / sizeof(T);
  const int64_t batch = s.b0 * s.b1;
  if (plan.path == 1) {
    const DotShape* one = &s;
    const void* rhs_list[1] = {rhs};
    void* out_list[1] = {out};
    return launch_group_typed<T>(one, 1, plan, lhs, rhs_list, out_list, partials, counters, pdl, stream);
  }
  if (plan.path == 2) {
    int group = 32;
    while (group > 1 && (int64_t)group * V > s.k) group >>= 1;
    const int rows_per_cta = 8 * (32 / group);
    dim3 grid((unsigned)((s.n + rows_per_cta - 1) / rows_per_cta), (unsigned)batch);
    cudaError_t e;
#define NK(MM) e = launch_kernel(stream_nk_kernel<T, MM>, grid, dim3(256), 0, stream, pdl, s, a, b, o, group)
    if (s.m <= 1) NK(1); else if (s.m <= 2) NK(2); else if (s.m <= 4) NK(4); else NK(8);
#undef NK
    return e == cudaSuccess ? 1 : 0;
  }
  if (plan.path == 3) {
    if (sgemm_ok(s, lhs, rhs, out)) {
      dim3 grid((unsigned)((s.n + kSgBN - 1) / kSgBN), (unsigned)((s.m + kSgBM - 1) / kSgBM), (unsigned)batch);
      return launch_kernel(sgemm_kernel, grid, dim3(256), 0, stream, pdl, s, (const float*)lhs, (const float*)rhs, (float*)out) == cudaSuccess ? 1 : 0;
    }
    dim3 grid((unsigned)((s.n + kTile - 1) / kTile), (unsigned)((s.m + kTile - 1) / kTile), (unsigned)batch);
    return launch_kernel(tile_kernel<T>, grid, dim3(256), 0, stream, pdl, s, a, b, o) == cudaSuccess ? 1 : 0;
  }
  const int64_t total = batch * s.m * s.n;
  const unsigned blocks = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 32);
  return launch_kernel(dot_generic_kernel<T>, dim3(blocks ? blocks : 1), dim3(256), 0, stream, pdl, s, a, b, o) == cudaSuccess ? 1 : 0;
}

}  // namespace

namespace {
int umma_eligible(const DotShape& s);
DotScratch umma_plan(const DotShape* shapes, int count, int sm_count, bool k_major);
}  // namespace

namespace {
int tma_env_int(const char* name, int fallback) {
  const char* v = getenv(name);
  return v && *v ? atoi(v) : fallback;
}

// Budget of one launch for all of its device-side waits (PJRTX_B200_WAIT_TIMEOUT_MS, two seconds by default).
unsigned long long tma_timeout_ns() {
  static const unsigned long long ns = [] {
    const int ms = tma_env_int("PJRTX_B200_WAIT_TIMEOUT_MS", 2000);
    return (unsigned long long)(ms < 1 ? 1 : ms) * 1000000ull;
  }();
  return ns;
}

// Ring depth and CTAs per SM of the TMA streaming kernel: two CTAs per SM with three 32 KiB stages each while the
// cross-warp fold buffer is small (m <= 2 for 16-bit types), one CTA with a deeper ring otherwise.
void tma_ring(int M, int V, int* stages, int* per_sm) {
  const size_t red = (size_t)tma::kConsumerWarps * M * 32 * V * sizeof(float);
  const bool two = red <= 16 * 1024;
  *per_sm = two ? 2 : 1;
  *stages = two ? 3 : (M <= 4 ? 5 : 4);
  static const int env_stages = tma_env_int("PJRTX_B200_TMA_STAGES", 0);
  if (env_stages >= 2 && env_stages <= 6) *stages = env_stages;
}
}  // namespace

DotScratch dot_group_plan(const DotShape* shapes, int count, int sm_count, bool allow_tensor) {
  DotScratch p;
  p.path = 1;
  const DotShape& s = shapes[0];
  const int esize = (int)dtype_size(s.dtype);
  const int V = 16 / esize;
  const int64_t batch = s.b0 * s.b1;
  int64_t tiles = 0, n_total = 0;
  for (int g = 0; g < count; g++) {
    tiles += (shapes[g].n + 32 * V - 1) / (32 * V);
    n_total += shapes[g].n;
  }
  const int M = s.m <= 1 ? 1 : s.m <= 2 ? 2 : s.m <= 4 ? 4 : 8;
  if (batch == 1 && allow_tensor) {
    bool all_umma = true;
    for (int g = 0; g < count; g++) all_umma &= umma_eligible(shapes[g]) == 1;
    if (all_umma) return umma_plan(shapes, count, sm_count, false);
  }
  if (batch == 1) {
    // Persistent TMA kernel: equal shares of (column tile, row chunk) units per CTA, two CTAs per SM with a ring of
    // 32 KiB stages each. Measured on the 8B-shape decode step (ms per step): two CTAs x 3 stages 3.50; one CTA x 5
    // stages 3.67; two CTAs x 6 stages of 16 KiB 3.94; one CTA x 6 stages of 16 KiB 4.95.
    p.tma = 1;
    const int chunks = (int)((s.k + tma::kUnitRows - 1) / tma::kUnitRows);
    const int64_t units = tiles * chunks;
    int per_sm = 1;
    tma_ring(M, V, &p.stages, &per_sm);
    // A fixed grid of one (or two) CTAs per SM; units are dealt out evenly (shares differ by at most one unit).
    const int64_t ctas = std::max<int64_t>(1, std::min<int64_t>(units, (int64_t)sm_count * per_sm));
    p.grid = (int)ctas;
    p.per_cta = units / ctas;
    p.max_contrib = (int)((chunks + p.per_cta - 1) / p.per_cta) + 1;
    p.smem = tma::smem_bytes(p.stages, M, 32 * V);
    p.ksplit = p.max_contrib;
    p.partial_bytes = (uint64_t)tiles * p.max_contrib * M * 32 * V * sizeof(float);
    p.counter_bytes = (uint64_t)tiles * sizeof(unsigned);
    return p;
  }
  // About two CTAs per SM, every CTA streaming at least 256 rows of its tile.
  const int64_t want = ((int64_t)sm_count * 2 + tiles * batch - 1) / (tiles * batch);
  const int64_t max_split = std::max<int64_t>(1, s.k / 256);
  p.ksplit = (int)std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(want, max_split), 32));
  if (p.ksplit > 1) {
    p.partial_bytes = (uint64_t)batch * p.ksplit * M * n_total * sizeof(float);
    p.counter_bytes = (uint64_t)batch * tiles * sizeof(unsigned);
  }
  return p;
}

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
    return (EncodeTiledFn)p;
  }();
  return fn;
}

template <typename T, int M, bool EXTRAS>
int launch_tma_m(const tma::Params& prm, const tma::Maps& maps, int grid, size_t smem, bool pdl, cudaStream_t stream) {
  if (!raise_smem_limit((const void*)tma::stream_tma_kernel<T, M, EXTRAS>, 200 * 1024)) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(tma::kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  cfg.attrs = attr;
  cfg.numAttrs = fill_launch_attributes(attr, pdl);
  return cudaLaunchKernelEx(&cfg, tma::stream_tma_kernel<T, M, EXTRAS>, prm, maps) == cudaSuccess ? 1 : 0;
}

// Fills one segment of the kernel parameters (and its tensor maps) from a group of contractions sharing an lhs.
template <typename T>
bool fill_segment(const DotShape* shapes, int count, const DotLhs& lhs_desc, const void* lhs, const void* lhs2,
                  const void* const* rhs, void* const* out, const void* const* residual, int max_contrib, float* partials,
                  unsigned* counters, tma::Segment* sg, CUtensorMap* maps) {
  constexpr int V = 16 / sizeof(T);
  constexpr int COLS = 32 * V;
  const DotShape& s = shapes[0];
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return false;
  sg->lhs = lhs;
  sg->lhs2 = lhs2;
  sg->lhs_m = s.lhs_m;
  sg->lhs_k = s.lhs_k;
  sg->lhs_kind = lhs_desc.kind;
  sg->norm_scale = lhs_desc.norm_scale;
  sg->norm_eps = lhs_desc.norm_eps;
  sg->m = (int)s.m;
  sg->k = (int)s.k;
  sg->count = count;
  int tiles = 0;
  const CUtensorMapDataType dt = sizeof(T) == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  for (int g = 0; g < count; g++) {
    sg->tile_begin[g] = tiles;
    tiles += (int)((shapes[g].n + COLS - 1) / COLS);
    sg->out[g] = out[g];
    sg->residual[g] = residual ? residual[g] : nullptr;
    sg->n[g] = shapes[g].n;
    cuuint64_t gdim[2] = {(cuuint64_t)shapes[g].n, (cuuint64_t)s.k};
    cuuint64_t gstride[1] = {(cuuint64_t)shapes[g].rhs_k * sizeof(T)};
    cuuint32_t box[2] = {(cuuint32_t)COLS, (cuuint32_t)tma::kUnitRows};
    cuuint32_t estr[2] = {1, 1};
    if (enc(&maps[g], dt, 2, const_cast<void*>(rhs[g]), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return false;
  }
  for (int g = count; g <= tma::kGroupMax; g++) sg->tile_begin[g] = tiles;
  for (int g = count; g < tma::kGroupMax; g++) maps[g] = maps[0];
  sg->chunks = (int)((s.k + tma::kUnitRows - 1) / tma::kUnitRows);
  sg->units = (long long)tiles * sg->chunks;
  sg->max_contrib = max_contrib;
  sg->partials = partials;
  sg->counters = counters;
  sg->ssq_out = nullptr;
  sg->ssq_in = nullptr;
  sg->ssq_tiles = 0;
  return true;
}

template <typename T>
int launch_tma_params(tma::Params& p, const tma::Maps& maps, int m, int grid, int stages, size_t smem, int* error_flag,
                      bool early_rhs, bool pdl, cudaStream_t stream) {
  p.error_flag = error_flag;
  p.timeout_ns = tma_timeout_ns();
  p.stages = stages;
  p.early_rhs = early_rhs ? 1 : 0;
  static const int env_evict = tma_env_int("PJRTX_B200_TMA_EVICT_FIRST", 1);
  p.evict_first = env_evict;
  const int M = m <= 1 ? 1 : m <= 2 ? 2 : m <= 4 ? 4 : 8;
  // The plain contraction (one segment, untransformed lhs, no residual) runs the kernel without the segment machinery.
  bool extras = p.segments > 1 || p.seg[0].lhs_kind != tma::kLhsPlain;
  for (int g = 0; g < p.seg[0].count; g++) extras |= p.seg[0].residual[g] != nullptr;
#define GO(MM) (extras ? launch_tma_m<T, MM, true>(p, maps, grid, smem, pdl, stream) : launch_tma_m<T, MM, false>(p, maps, grid, smem, pdl, stream))
  switch (M) {
    case 1: return GO(1);
    case 2: return GO(2);
    case 4: return GO(4);
    default: return GO(8);
  }
#undef GO
}

template <typename T>
int launch_tma(const DotShape* shapes, int count, const DotScratch& plan, const void* lhs, const void* const* rhs, void* const* out,
               void* partials, void* counters, int* error_flag, bool early_rhs, bool pdl, cudaStream_t stream) {
  tma::Params p{};
  tma::Maps maps{};
  p.segments = 1;
  p.barrier = nullptr;
  if (!fill_segment<T>(shapes, count, DotLhs{}, lhs, nullptr, rhs, out, nullptr, plan.max_contrib, static_cast<float*>(partials),
                       static_cast<unsigned*>(counters), &p.seg[0], maps.map[0]))
    return 0;
  return launch_tma_params<T>(p, maps, (int)shapes[0].m, plan.grid, plan.stages, plan.smem, error_flag, early_rhs, pdl, stream);
}

template <typename T>
int launch_chain(const DotChainSegment* segs, const DotChainArgs* args, int n, const DotChainPlan& plan, void* partials,
                 void* counters, int* error_flag, bool early_rhs, bool pdl, cudaStream_t stream) {
  tma::Params p{};
  tma::Maps maps{};
  p.segments = n;
  unsigned* words = static_cast<unsigned*>(counters);
  p.barrier = words;  // the barrier words come first, then every segment's tile counters
  for (int s = 0; s < n; s++) {
    if (!fill_segment<T>(segs[s].shapes, segs[s].count, segs[s].lhs, args[s].lhs, args[s].lhs2, args[s].rhs, args[s].out,
                         args[s].residual, plan.max_contrib[s], static_cast<float*>(partials),
                         words + plan.counter_offset[s] / sizeof(unsigned), &p.seg[s], maps.map[s]))
      return 0;
  }
  for (int s = 0; s + 1 < n; s++)
    if (plan.ssq_offset[s]) {
      float* ssq = reinterpret_cast<float*>(static_cast<unsigned char*>(counters) + plan.ssq_offset[s]);
      p.seg[s].ssq_out = ssq;
      p.seg[s + 1].ssq_in = ssq;
      p.seg[s + 1].ssq_tiles = plan.tiles[s];
    }
  for (int s = n; s < tma::kSegmentMax; s++)
    for (int g = 0; g < tma::kGroupMax; g++) maps.map[s][g] = maps.map[0][0];
  return launch_tma_params<T>(p, maps, (int)segs[0].shapes[0].m, plan.grid, plan.stages, plan.smem, error_flag, early_rhs, pdl, stream);
}


// ---- tensor-core stream (umma_gemm.cuh) ---------------------------------------------------------------------------

int env_int(const char* name, int fallback) {
  const char* v = getenv(name);
  return v && *v ? atoi(v) : fallback;
}

// 0: not eligible, 1: rhs[K,N] with N contiguous, 2: rhs[N,K] with K contiguous. The tensor maps need 16-byte
// multiples for every row stride; lhs must be k-contiguous.
int umma_eligible(const DotShape& s) {
  static const int enabled = env_int("PJRTX_B200_UMMA", 1);
  static const int min_m = env_int("PJRTX_B200_UMMA_MIN_M", 3);
  if (!enabled || (s.dtype != kF16 && s.dtype != kBF16)) return 0;
  if (s.b0 * s.b1 != 1 || s.m < min_m || s.k < 1 || s.n < 1) return 0;
  if (s.lhs_k != 1 || (s.m > 1 && s.lhs_m % 8 != 0)) return 0;
  if (s.m > (1 << 20) || s.n > (1ll << 30) || s.k > (1ll << 30)) return 0;
  if (s.rhs_s8) return s.rhs_n == 1 && s.rhs_k % 16 == 0 && s.rhs_k >= s.n ? 1 : 0;  // byte rows: 16-byte pitch
  if (s.rhs_n == 1 && s.rhs_k % 8 == 0 && s.rhs_k >= s.n) return 1;
  if (s.rhs_k == 1 && s.rhs_n % 8 == 0 && s.rhs_n >= s.k) return 2;
  return 0;
}

DotScratch umma_plan(const DotShape* shapes, int count, int sm_count, bool k_major) {
  DotScratch p;
  const DotShape& s = shapes[0];
  p.path = k_major ? 4 : 1;
  p.umma = 1;
  p.m_tile = (int)std::min<int64_t>(256, (s.m + 15) / 16 * 16);
  const int64_t m_tiles = (s.m + p.m_tile - 1) / p.m_tile;
  // 256-column tiles (two accumulators per tile) are available behind PJRTX_B200_UMMA_WIDE=1; measured on B200 they
  // stream no faster than 128-column tiles and leave more partial sums to fold, so they are off by default.
  int64_t tiles128 = 0;
  for (int g = 0; g < count; g++) tiles128 += (shapes[g].n + 127) / 128 * m_tiles;
  static const int wide = env_int("PJRTX_B200_UMMA_WIDE", 0);
  p.nh = (wide && !s.rhs_s8 && p.m_tile <= 128 && tiles128 * ((s.k + 63) / 64) >= 16 * (int64_t)sm_count) ? 2 : 1;
  const int tw = umma::kTileN * p.nh;
  int64_t tiles = 0;
  for (int g = 0; g < count; g++) tiles += (shapes[g].n + tw - 1) / tw * m_tiles;
  // Short activation tiles leave room for two CTAs per SM (half the shared memory each; PJRTX_B200_UMMA_CTAS=2), so
  // that one CTA streams while the other folds a tile. Measured on B200 at m = 32 it is slower than one CTA per SM with
  // the whole ring (8B-width layers 1.665 against 1.640 ms per 8 layers; one eighth of the 70B-shape widths 3.00
  // against 2.79 ms per 20 layers): twice the partial sums to fold outweigh the overlap. Off by default.
  static const int ctas_wanted = env_int("PJRTX_B200_UMMA_CTAS", 1);
  const bool w8 = s.rhs_s8 != 0;
  const int per_sm = (ctas_wanted >= 2 && p.m_tile <= 64 && !w8 && p.nh == 1) ? 2 : 1;
  const int64_t slots = (int64_t)sm_count * per_sm;
  // PJRTX_B200_UMMA_SMEM_KB bounds the ring (experiments: a CTA that leaves half of the shared memory free lets the
  // first CTAs of the next kernel move in and start their weight copies while this one folds its last tile).
  static const int smem_kb = env_int("PJRTX_B200_UMMA_SMEM_KB", 0);
  const bool small_ring = smem_kb >= 48 && smem_kb <= 225 && !w8 && p.m_tile <= 64;
  const size_t smem_budget = small_ring ? (size_t)smem_kb * 1024 - 2048 : per_sm == 2 ? 112 * 1024 - 2048 : 227 * 1024 - 2048;
  const int64_t grid = std::max<int64_t>(1, std::min<int64_t>(tiles * ((s.k + 63) / 64), slots));
  // 128-deep stages once every CTA still gets a long run of them; 64-deep otherwise (finer split, better balance), and
  // whenever the ring would hold fewer than four of the deep ones.
  p.sub = (p.nh == 1 && tiles * ((s.k + 127) / 128) >= 32 * grid) ? 2 : 1;
  if (p.sub == 2 && smem_budget / umma::stage_bytes(p.m_tile, 2, p.nh, w8) < 4) p.sub = 1;
  // Int8 weights: 128-deep stages (PJRTX_B200_W8_SUB=1 gives 64-deep ones: a deeper ring of raw bytes, but twice the
  // hand-overs between copies, converters and the MMA lane; measured 1.54 against 1.25 ms for the contractions of eight
  // 8B-width layers and the LM head at 32 rows).
  static const int w8_sub = env_int("PJRTX_B200_W8_SUB", 2);
  if (w8) p.sub = w8_sub == 1 ? 1 : 2;
  const int64_t kblocks = (s.k + 64 * p.sub - 1) / (64 * p.sub);
  const int64_t units = tiles * kblocks;
  p.grid = (int)std::max<int64_t>(1, std::min<int64_t>(units, slots));
  // A split tile costs its f32 partial twice (written, read back): m_tile x 128 x 8 bytes per contributor, against
  // 128 x k x 2 bytes of weights per tile. Split only while the partials of a tile stay below about half its weights,
  // or when whole tiles would leave most of the machine idle.
  const int64_t split_ok = s.k / (8 * (int64_t)p.m_tile);
  p.whole_tiles = (split_ok < 2 || (p.m_tile >= 128 && 2 * tiles >= sm_count)) ? 1 : 0;
  if (p.whole_tiles) p.grid = (int)std::max<int64_t>(1, std::min<int64_t>(tiles, slots));
  p.per_cta = units / p.grid;
  p.max_contrib = p.whole_tiles ? 1 : (int)((kblocks + p.per_cta - 1) / p.per_cta) + 1;
  const size_t stage = umma::stage_bytes(p.m_tile, p.sub, p.nh, w8);
  const size_t ring_budget = smem_budget - (w8 ? umma::kOperandSlots * umma::operand_bytes(p.sub, p.nh) : 0);
  p.stages = (int)std::max<size_t>(w8 ? umma::kOperandSlots : 2, std::min<size_t>(w8 ? 16 : 12, ring_budget / stage));
  p.smem = umma::smem_bytes(p.stages, p.m_tile, p.sub, p.nh, w8);
  p.ksplit = p.max_contrib;
  p.partial_bytes = (uint64_t)tiles * p.max_contrib * p.m_tile * tw * sizeof(float);
  p.counter_bytes = (uint64_t)tiles * sizeof(unsigned);
  return p;
}

template <int SUB, int NH, bool W8 = false>
int launch_umma_sub(const umma::Params& prm, const umma::Maps& maps, const DotScratch& plan, bool pdl, cudaStream_t stream) {
  if (!raise_smem_limit((const void*)umma::umma_stream_kernel<SUB, NH, W8>, 227 * 1024)) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)plan.grid);
  cfg.blockDim = dim3(W8 ? umma::kThreadsW8 : umma::kThreads);
  cfg.dynamicSmemBytes = plan.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  cfg.attrs = attr;
  cfg.numAttrs = fill_launch_attributes(attr, pdl);
  return cudaLaunchKernelEx(&cfg, umma::umma_stream_kernel<SUB, NH, W8>, prm, maps) == cudaSuccess ? 1 : 0;
}

int launch_umma(const DotShape* shapes, int count, const DotScratch& plan, const void* lhs, const void* const* rhs, void* const* out,
                void* partials, void* counters, int* error_flag, bool early_rhs, bool pdl, cudaStream_t stream,
                const void* const* scales) {
  const DotShape& s = shapes[0];
  const bool w8 = s.rhs_s8 != 0;
  if (w8 && (!scales || plan.path == 4 || plan.nh != 1)) return 0;
  EncodeTiledFn enc = encode_tiled();
  if (!enc) return 0;
  const bool k_major = plan.path == 4;
  const int tw = umma::kTileN * plan.nh;
  umma::Params p{};
  umma::Maps maps{};
  p.m = (int)s.m;
  p.k = (int)s.k;
  p.m_tile = plan.m_tile;
  p.m_tiles = (int)((s.m + plan.m_tile - 1) / plan.m_tile);
  p.count = count;
  const CUtensorMapDataType dt = s.dtype == kF16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const cuuint32_t estr[2] = {1, 1};
  // One 3-d copy per stage when every rhs is made of whole 64-column blocks (a ragged last block would make the
  // view read past the end of the last row).
  static const int allow_3d = env_int("PJRTX_B200_UMMA_3D", 1);
  bool use_3d = allow_3d && !k_major && !w8;
  for (int g = 0; g < count; g++) use_3d &= shapes[g].n % 64 == 0;
  int tiles = 0;
  for (int g = 0; g < count; g++) {
    if ((reinterpret_cast<uintptr_t>(rhs[g]) & 15) != 0) return 0;
    p.tile_begin[g] = tiles;
    tiles += (int)((shapes[g].n + tw - 1) / tw) * p.m_tiles;
    p.out[g] = out[g];
    p.n[g] = shapes[g].n;
    p.ldo[g] = shapes[g].out_m;
    p.scale[g] = w8 ? scales[g] : nullptr;
  }
  auto encode_rhs = [&](bool three_d) {
    for (int g = 0; g < count; g++) {
      cuuint64_t gdim[3], gstride[2];
      cuuint32_t box[3];
      const cuuint32_t estr3[3] = {1, 1, 1};
      int rank = 2;
      if (w8) {
        // raw bytes: one box of 128 columns x 64 * SUB rows per stage, no swizzle (the converters place the values)
        gdim[0] = (cuuint64_t)shapes[g].n; gdim[1] = (cuuint64_t)s.k;
        gstride[0] = (cuuint64_t)shapes[g].rhs_k;
        box[0] = 128; box[1] = (cuuint32_t)(64 * plan.sub);
        // A row of the box is 128 bytes: with 256-byte promotion L2 would fetch the neighbouring tile's 128 bytes with
        // every row and usually lose them again before that tile's turn (measured on the 4096 x 128256 LM head:
        // 742 MB read for 525 MB of weights).
        if (enc(&maps.rhs[g], CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(rhs[g]), gdim, gstride, box, estr3,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
          return false;
        continue;
      }
      if (three_d) {
        rank = 3;
        gdim[0] = 64; gdim[1] = (cuuint64_t)s.k; gdim[2] = (cuuint64_t)shapes[g].n / 64;
        gstride[0] = (cuuint64_t)shapes[g].rhs_k * 2; gstride[1] = 128;
        box[0] = 64; box[1] = (cuuint32_t)(64 * plan.sub); box[2] = (cuuint32_t)(2 * plan.nh);
      } else if (k_major) {
        gdim[0] = (cuuint64_t)s.k; gdim[1] = (cuuint64_t)shapes[g].n;
        gstride[0] = (cuuint64_t)shapes[g].rhs_n * 2;
        box[0] = 64; box[1] = 128;
      } else {
        gdim[0] = (cuuint64_t)shapes[g].n; gdim[1] = (cuuint64_t)s.k;
        gstride[0] = (cuuint64_t)shapes[g].rhs_k * 2;
        box[0] = 64; box[1] = (cuuint32_t)(64 * plan.sub);
      }
      if (enc(&maps.rhs[g], dt, rank, const_cast<void*>(rhs[g]), gdim, gstride, box, estr3, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    }
    return true;
  };
  if (use_3d && !encode_rhs(true)) use_3d = false;  // the driver refused the view: fall back to two boxes per half
  if (!use_3d && !encode_rhs(false)) return 0;
  p.rhs_3d = use_3d ? 1 : 0;
  for (int g = count; g <= umma::kGroupMax; g++) p.tile_begin[g] = tiles;
  for (int g = count; g < umma::kGroupMax; g++) maps.rhs[g] = maps.rhs[0];
  {
    if ((reinterpret_cast<uintptr_t>(lhs) & 15) != 0) return 0;
    cuuint64_t gdim[2] = {(cuuint64_t)s.k, (cuuint64_t)s.m};
    // A single row has no stride to honour; any 16-byte multiple that covers the row will do.
    cuuint64_t gstride[1] = {(cuuint64_t)(s.m > 1 ? s.lhs_m : (s.k + 7) / 8 * 8) * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)plan.m_tile};
    if (enc(&maps.lhs, dt, 2, const_cast<void*>(lhs), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return 0;
  }
  p.kblocks = (int)((s.k + 64 * plan.sub - 1) / (64 * plan.sub));
  p.units = (long long)tiles * p.kblocks;
  p.max_contrib = plan.max_contrib;
  p.partials = static_cast<float*>(partials);
  p.counters = static_cast<unsigned*>(counters);
  p.error_flag = error_flag;
  p.stages = plan.stages;
  p.is_bf16 = s.dtype == kBF16;
  p.rhs_k_major = k_major ? 1 : 0;
  p.early_rhs = early_rhs ? 1 : 0;
  p.whole_tiles = plan.whole_tiles;
  if (w8)
    return plan.sub == 2 ? launch_umma_sub<2, 1, true>(p, maps, plan, pdl, stream) : launch_umma_sub<1, 1, true>(p, maps, plan, pdl, stream);
  if (plan.nh == 2)
    return plan.sub == 2 ? launch_umma_sub<2, 2>(p, maps, plan, pdl, stream) : launch_umma_sub<1, 2>(p, maps, plan, pdl, stream);
  return plan.sub == 2 ? launch_umma_sub<2, 1>(p, maps, plan, pdl, stream) : launch_umma_sub<1, 1>(p, maps, plan, pdl, stream);
}

}  // namespace

bool dot_chain_eligible(const DotShape& s, int sm_count) {
  if (s.b0 * s.b1 != 1) return false;
  const DotScratch p = dot_plan(s, sm_count);
  return p.path == 1 && p.tma == 1 && p.umma == 0;
}

DotChainPlan dot_chain_plan(const DotChainSegment* segs, int n, int sm_count) {
  DotChainPlan p;
  if (n < 1 || n > kDotChainMax) return p;
  const DotShape& first = segs[0].shapes[0];
  const int esize = (int)dtype_size(first.dtype);
  const int V = 16 / esize;
  const int M = first.m <= 1 ? 1 : first.m <= 2 ? 2 : first.m <= 4 ? 4 : 8;
  int per_sm = 1;
  tma_ring(M, V, &p.stages, &per_sm);
  const bool two_per_sm = per_sm == 2;
  p.smem = tma::smem_bytes(p.stages, M, 32 * V);
  // Every CTA takes part in the barriers between segments, so the grid must be wholly resident, and every CTA must own
  // at least one unit of every segment (the tile bookkeeping assumes consecutive, non-empty shares).
  int64_t grid = (int64_t)sm_count * (two_per_sm ? 2 : 1);
  int64_t tiles_all[kDotChainMax], chunks_all[kDotChainMax];
  for (int s = 0; s < n; s++) {
    int64_t tiles = 0;
    for (int g = 0; g < segs[s].count; g++) tiles += (segs[s].shapes[g].n + 32 * V - 1) / (32 * V);
    const int64_t chunks = (segs[s].shapes[0].k + tma::kUnitRows - 1) / tma::kUnitRows;
    tiles_all[s] = tiles;
    chunks_all[s] = chunks;
    grid = std::min(grid, std::max<int64_t>(1, tiles * chunks));
  }
  p.grid = (int)grid;
  p.segments = n;
  uint64_t counters = (uint64_t)2 * kDotChainMax * sizeof(unsigned);  // barrier words
  counters = (counters + 255) / 256 * 256;
  for (int s = 0; s < n; s++) {
    const int64_t per_cta = std::max<int64_t>(1, tiles_all[s] * chunks_all[s] / grid);
    p.max_contrib[s] = (int)std::min<int64_t>(chunks_all[s], (chunks_all[s] + per_cta - 1) / per_cta + 1);
    p.counter_offset[s] = counters;
    p.tiles[s] = (int)tiles_all[s];
    counters += ((uint64_t)tiles_all[s] * sizeof(unsigned) + 255) / 256 * 256;
    if (s + 1 < n && segs[s + 1].norm_of_previous && segs[s + 1].lhs.kind == kDotLhsRmsNorm && segs[s].count == 1) {
      p.ssq_offset[s] = counters;
      counters += ((uint64_t)tiles_all[s] * M * sizeof(float) + 255) / 256 * 256;
    }
    p.partial_bytes = std::max<uint64_t>(p.partial_bytes, (uint64_t)tiles_all[s] * p.max_contrib[s] * M * 32 * V * sizeof(float));
  }
  p.counter_bytes = counters;
  return p;
}

int dot_chain_launch(const DotChainSegment* segs, const DotChainArgs* args, int n, const DotChainPlan& plan, void* partials,
                     void* counters, int* error_flag, bool early_rhs, bool pdl, cudaStream_t stream) {
  if (n < 1 || n > kDotChainMax || plan.segments != n) return 0;
  switch (segs[0].shapes[0].dtype) {
    case kF32: return launch_chain<float>(segs, args, n, plan, partials, counters, error_flag, early_rhs, pdl, stream);
    case kF16: return launch_chain<__half>(segs, args, n, plan, partials, counters, error_flag, early_rhs, pdl, stream);
    case kBF16: return launch_chain<__nv_bfloat16>(segs, args, n, plan, partials, counters, error_flag, early_rhs, pdl, stream);
    default: return 0;
  }
}

namespace {
// One CTA waits, with the streaming kernel's own bounded wait, on an mbarrier that nothing ever completes.
__global__ void bounded_wait_probe_kernel(unsigned long long timeout_ns, int* error_flag) {
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  if (threadIdx.x == 0) {
    abort_word = 0;
    tma::mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const tma::WaitBudget budget{tma::global_timer_ns() + timeout_ns, &abort_word};
  if (!tma::mbar_wait(&bar, 0, budget) && threadIdx.x == 0) atomicExch(error_flag, 31);
}
}  // namespace

int bounded_wait_probe_launch(unsigned timeout_ms, int* error_flag, cudaStream_t stream) {
  if (!error_flag || timeout_ms < 1 || timeout_ms > 1000) return 0;
  bounded_wait_probe_kernel<<<1, 64, 0, stream>>>((unsigned long long)timeout_ms * 1000000ull, error_flag);
  return cudaGetLastError() == cudaSuccess ? 1 : 0;
}

bool dot_s8_supported(const DotShape& s) {
  DotShape probe = s;
  probe.rhs_s8 = 1;
  return umma_eligible(probe) == 1;
}

int dot_group_launch(const DotShape* shapes, int count, const DotScratch& plan, const void* lhs, const void* const* rhs,
                     void* const* out, void* partials, void* counters, int* error_flag, bool early_rhs, bool pdl,
                     cudaStream_t stream, const void* const* scales) {
  if (count < 1 || count > kDotGroupMax) return 0;
  if (plan.umma) return launch_umma(shapes, count, plan, lhs, rhs, out, partials, counters, error_flag, early_rhs, pdl, stream, scales);
  if (shapes[0].rhs_s8) return 0;  // int8 weights run on the tensor-core stream only
  if (plan.tma) {
    switch (shapes[0].dtype) {
      case kF32: return launch_tma<float>(shapes, count, plan, lhs, rhs, out, partials, counters, error_flag, early_rhs, pdl, stream);
      case kF16: return launch_tma<__half>(shapes, count, plan, lhs, rhs, out, partials, counters, error_flag, early_rhs, pdl, stream);
      case kBF16: return launch_tma<__nv_bfloat16>(shapes, count, plan, lhs, rhs, out, partials, counters, error_flag, early_rhs, pdl, stream);
      default: return 0;
    }
  }
  switch (shapes[0].dtype) {
    case kF32: return launch_group_typed<float>(shapes, count, plan, lhs, rhs, out, partials, counters, pdl, stream);
    case kF16: return launch_group_typed<__half>(shapes, count, plan, lhs, rhs, out, partials, counters, pdl, stream);
    case kBF16: return launch_group_typed<__nv_bfloat16>(shapes, count, plan, lhs, rhs, out, partials, counters, pdl, stream);
    default: return 0;
  }
}

DotScratch dot_plan(const DotShape& s, int sm_count) {
  DotScratch p;
  const int esize = (int)dtype_size(s.dtype);
  if (esize == 0 || !dtype_is_float(s.dtype)) return p;
  const int V = 16 / esize;
  const int64_t batch = s.b0 * s.b1;
  auto aligned = [&](int64_t stride) { return stride % V == 0; };
  const bool batches_fit = batch <= 65535;
  const int tensor = umma_eligible(s);
  if (tensor == 1) return umma_plan(&s, 1, sm_count, false);
  if (tensor == 2) return umma_plan(&s, 1, sm_count, true);
  if (s.m <= 8 && s.rhs_n == 1 && s.n % V == 0 && aligned(s.rhs_k) && aligned(s.rhs_b0) && aligned(s.rhs_b1) &&
      batches_fit && s.k >= 1) {
    p.path = 1;
    const DotShape one = s;
    return dot_group_plan(&one, 1, sm_count);
  }
  if (s.m <= 8 && s.rhs_k == 1 && s.lhs_k == 1 && s.k % V == 0 && aligned(s.rhs_n) && aligned(s.rhs_b0) &&
      aligned(s.rhs_b1) && aligned(s.lhs_m) && aligned(s.lhs_b0) && aligned(s.lhs_b1) && batches_fit) {
    p.path = 2;
    return p;
  }
  if (s.m > 8 && batches_fit && (s.m + kTile - 1) / kTile <= 65535) {
    p.path = 3;
    return p;
  }
  p.path = 0;
  return p;
}

int dot_launch(const DotShape& s, const DotScratch& plan, const void* lhs, const void* rhs, void* out, void* partials,
               void* counters, int* error_flag, bool early_rhs, bool pdl, cudaStream_t stream, const void* scale) {
  if (s.b0 * s.b1 * s.m * s.n == 0) return 1;
  if (plan.umma || (plan.path == 1 && plan.tma)) {
    const void* rhs_list[1] = {rhs};
    void* out_list[1] = {out};
    const void* scale_list[1] = {scale};
    return dot_group_launch(&s, 1, plan, lhs, rhs_list, out_list, partials, counters, error_flag, early_rhs, pdl, stream, scale_list);
  }
  if (s.rhs_s8) return 0;
  switch (s.dtype) {
    case kF32: return launch_typed<float>(s, plan, lhs, rhs, out, partials, counters, pdl, stream);
    case kF16: return launch_typed<__half>(s, plan, lhs, rhs, out, partials, counters, pdl, stream);
    case kBF16: return launch_typed<__nv_bfloat16>(s, plan, lhs, rhs, out, partials, counters, pdl, stream);
    default: return 0;
  }
}

}  // namespace pjrtx

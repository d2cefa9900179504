// Weight-streaming contraction for m <= 8: out[m, n] = sum_k lhs[m, k] * rhs[k, n], rhs row-major with n contiguous.
//
// The kernel is bandwidth-bound (every rhs element is read once and used m times), so it is built around keeping
// enough bytes in flight per SM with few threads: a persistent CTA per SM owns a ring of shared-memory stages that
// one producer warp fills with bulk asynchronous copies (cp.async.bulk, completion counted on an mbarrier), while
// eight consumer warps read finished stages and accumulate in registers. Each stage is one tiled TMA copy
// (cp.async.bulk.tensor.2d) of a 64-row x 512-byte box described by a tensor map of the rhs; rows and columns past
// the matrix edge arrive as zeros, so ragged k and n need no special case.
//
// Work decomposition (stream-K): the rhs is cut into units of kUnitRows rows x one 512-byte column tile, ordered
// tile-major; CTA b of G takes the b-th contiguous share of all units, so every SM streams the same number of bytes
// whatever the shape. A CTA that does not cover a tile's whole k range writes an f32 partial; the CTA that arrives
// last for a tile folds the partials in CTA order (fixed order: results are identical from run to run).
//
// Programmatic dependent launch: the kernel lets its successor start at once (griddepcontrol.launch_dependents) and
// itself waits for its predecessor (griddepcontrol.wait) only before the first access that can depend on it: the
// producer may already be copying rhs tiles (weights are never written by the stream's earlier work), the consumers
// wait before they read lhs or write anything.
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the kernel raises *error_flag and leaves.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pjrtx {
namespace tma {

constexpr int kGroupMax = 4;
constexpr int kUnitRows = 64;       // rows per unit
constexpr int kTileBytes = 512;     // bytes per row per unit (one warp x 16 B)
constexpr int kStageBytes = kUnitRows * kTileBytes;  // 32 KiB
constexpr int kConsumerWarps = 8;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr unsigned kSpinLimit = 1u << 22;  // about a quarter of a second of polling

struct Params {
  // Shared by all contractions of the launch.
  const void* lhs;
  long long lhs_m, lhs_k;            // element strides
  long long lhs_batch, rhs_batch;    // element strides of the (single, merged) batch axis; 0 when batch == 1
  int m, k, batch;
  int count;                          // contractions sharing lhs
  int tile_begin[kGroupMax + 1];      // column-tile prefix sums over the group
  const void* rhs[kGroupMax];
  void* out[kGroupMax];
  long long n[kGroupMax];
  long long ldb[kGroupMax];           // rhs row stride in elements
  long long out_batch[kGroupMax];     // out batch stride in elements (m * n)
  // Decomposition.
  int chunks;                         // ceil(k / kUnitRows)
  long long units;                    // batch * tiles * chunks
  long long per_cta;                  // floor(units / gridDim.x): CTA b owns units [b*units/grid, (b+1)*units/grid)
  int max_contrib;                    // partial slots per tile
  float* partials;                    // [batch * tiles][max_contrib][M][tile columns]
  unsigned* counters;                 // [batch * tiles], zero before the first launch, left zero by every launch
  int* error_flag;
  int stages;
  int early_rhs;                      // rhs copies may start before the preceding kernel of the stream has finished
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait; false when the limit was hit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
  for (unsigned spin = 0; spin < kSpinLimit; spin++)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// Arrival counter with release/acquire semantics at device scope: together with the CTA barriers around it, the
// partial sums every thread of this CTA wrote are visible to whichever CTA observes the final count.
__device__ __forceinline__ unsigned arrive_acq_rel(unsigned* counter) {
  unsigned old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
  return old;
}

// One box of the tensor map: x = first column (must be a multiple of 16 bytes), y = first row.
__device__ __forceinline__ void tensor_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
               : "memory");
}

template <typename T> struct Unpack;
template <> struct Unpack<float> {
  static constexpr int V = 4;
  static __device__ __forceinline__ void to_float(const uint4& r, float* f) {
    f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
  }
  static __device__ __forceinline__ float one(float v) { return v; }
  static __device__ __forceinline__ float store(float v) { return v; }
};
template <> struct Unpack<__nv_bfloat16> {
  static constexpr int V = 8;
  static __device__ __forceinline__ void to_float(const uint4& r, float* f) {
    f[0] = __uint_as_float(r.x << 16); f[1] = __uint_as_float(r.x & 0xffff0000u);
    f[2] = __uint_as_float(r.y << 16); f[3] = __uint_as_float(r.y & 0xffff0000u);
    f[4] = __uint_as_float(r.z << 16); f[5] = __uint_as_float(r.z & 0xffff0000u);
    f[6] = __uint_as_float(r.w << 16); f[7] = __uint_as_float(r.w & 0xffff0000u);
  }
  static __device__ __forceinline__ float one(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 store(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Unpack<__half> {
  static constexpr int V = 8;
  static __device__ __forceinline__ void to_float(const uint4& r, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float2 p = __half22float2(h[i]);
      f[2 * i] = p.x;
      f[2 * i + 1] = p.y;
    }
  }
  static __device__ __forceinline__ float one(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half store(float v) { return __float2half_rn(v); }
};

// Position of a unit: which column tile (over all contractions of the group) and which k chunk. Advancing is an
// increment; the divisions happen once per CTA and once per tile change.
struct Cursor {
  int tile;    // global tile index (over the group)
  int chunk;
  int group, tile_in_group;
};

__device__ __forceinline__ void locate_tile(const Params& p, Cursor* c) {
  int g = 0;
#pragma unroll
  for (int q = 1; q < kGroupMax; q++)
    if (q < p.count && c->tile >= p.tile_begin[q]) g = q;
  c->group = g;
  c->tile_in_group = c->tile - p.tile_begin[g];
}

__device__ __forceinline__ Cursor cursor_at(const Params& p, long long u) {
  Cursor c;
  c.tile = (int)(u / p.chunks);
  c.chunk = (int)(u - (long long)c.tile * p.chunks);
  locate_tile(p, &c);
  return c;
}

__device__ __forceinline__ void advance(const Params& p, Cursor* c) {
  if (++c->chunk == p.chunks) {
    c->chunk = 0;
    c->tile++;
    locate_tile(p, c);
  }
}

struct Maps {
  CUtensorMap map[kGroupMax];
};

template <typename T, int M>
__global__ void __launch_bounds__(kThreads, 1) stream_tma_kernel(const Params p, const __grid_constant__ Maps maps) {
  constexpr int V = Unpack<T>::V;
  constexpr int COLS = 32 * V;  // columns per tile
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* stage_base = smem_raw;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + (size_t)p.stages * kStageBytes);
  uint64_t* empty = full + p.stages;
  int* flags = reinterpret_cast<int*>(empty + p.stages);  // [0] is_last, [1] abort

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long u_begin = (long long)blockIdx.x * p.units / gridDim.x;
  const long long u_end = (long long)(blockIdx.x + 1) * p.units / gridDim.x;
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    flags[0] = 0;
    flags[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (u_begin >= u_end) return;

  if (warp == kConsumerWarps) {
    // ---- producer: one elected lane issues one tensor copy per stage -------------------------------------
    if (lane != 0) return;
    if (!p.early_rhs) asm volatile("griddepcontrol.wait;" ::: "memory");
    int stage = 0;
    unsigned phase = 0;
    Cursor cur = cursor_at(p, u_begin);
    const int count = (int)(u_end - u_begin);
    for (int i = 0; i < count; i++) {
      if (i >= p.stages) {
        if (!mbar_wait(&empty[stage], phase ^ 1)) {
          atomicExch(p.error_flag, 1);
          return;
        }
      }
      mbar_expect_tx(&full[stage], kStageBytes);
      tensor_load_2d(stage_base + (size_t)stage * kStageBytes, &maps.map[cur.group], cur.tile_in_group * COLS, cur.chunk * kUnitRows,
                     &full[stage]);
      advance(p, &cur);
      if (++stage == p.stages) {
        stage = 0;
        phase ^= 1;
      }
    }
    return;
  }

  // ---- consumer warps ---------------------------------------------------------------------------------------
  asm volatile("griddepcontrol.wait;" ::: "memory");
  float acc[M][V];
#pragma unroll
  for (int m = 0; m < M; m++)
#pragma unroll
    for (int v = 0; v < V; v++) acc[m][v] = 0.f;
  const T* lhs = static_cast<const T*>(p.lhs);
  float* red = reinterpret_cast<float*>(flags + 4);  // [kConsumerWarps][M][COLS] floats, after the barriers
  int stage = 0;
  unsigned phase = 0;
  long long cur_tile = -1;
  Cursor pos{};
  Cursor next = cursor_at(p, u_begin);
  const int count = (int)(u_end - u_begin);
  for (int i = 0; i <= count; i++) {
    const bool more = i < count;
    if (!more || next.tile != cur_tile) {
      if (cur_tile >= 0) {
        // Flush the finished tile segment: fold the eight warps through shared memory, then either write the
        // output (this CTA covered the whole k range) or publish a partial.
#pragma unroll
        for (int m = 0; m < M; m++)
#pragma unroll
          for (int v = 0; v < V; v++) red[(warp * M + m) * COLS + lane * V + v] = acc[m][v];
        asm volatile("bar.sync 1, %0;" ::"r"(kConsumerWarps * 32));
        // CTA that owns unit u: the largest b with b*units/grid <= u, i.e. ceil((u+1)*grid/units) - 1.
        const long long tile_units_begin = cur_tile * p.chunks;
        const long long first_cta = ((tile_units_begin + 1) * gridDim.x + p.units - 1) / p.units - 1;
        const long long last_cta = ((tile_units_begin + p.chunks) * gridDim.x + p.units - 1) / p.units - 1;
        const int contributors = (int)(last_cta - first_cta + 1);
        const long long n = p.n[pos.group];
        const long long col0 = (long long)pos.tile_in_group * COLS;
        T* out = static_cast<T*>(p.out[pos.group]);
        float* slot = p.partials + ((cur_tile * p.max_contrib + (blockIdx.x - first_cta)) * M) * COLS;
        for (int idx = threadIdx.x; idx < M * COLS; idx += kConsumerWarps * 32) {
          const int m = idx / COLS, c = idx % COLS;
          float t = 0.f;
#pragma unroll
          for (int w = 0; w < kConsumerWarps; w++) t += red[(w * M + m) * COLS + c];
          if (contributors == 1) {
            if (m < p.m && col0 + c < n) out[(long long)m * n + col0 + c] = Unpack<T>::store(t);
          } else {
            slot[idx] = t;
          }
        }
        if (contributors > 1) {
          asm volatile("bar.sync 1, %0;" ::"r"(kConsumerWarps * 32));
          if (threadIdx.x == 0) flags[0] = arrive_acq_rel(&p.counters[cur_tile]) == (unsigned)contributors - 1;
          asm volatile("bar.sync 1, %0;" ::"r"(kConsumerWarps * 32));
          if (flags[0]) {
            const float* base = p.partials + (cur_tile * p.max_contrib * (long long)M) * COLS;
            for (int idx = threadIdx.x; idx < M * COLS; idx += kConsumerWarps * 32) {
              const int m = idx / COLS, c = idx % COLS;
              float t = 0.f;
              int q = 0;
              for (; q + 8 <= contributors; q += 8) {  // loads first, then the adds in CTA order
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; e++) v[e] = __ldcg(base + (long long)(q + e) * M * COLS + idx);
#pragma unroll
                for (int e = 0; e < 8; e++) t += v[e];
              }
              for (; q < contributors; q++) t += __ldcg(base + (long long)q * M * COLS + idx);
              if (m < p.m && col0 + c < n) out[(long long)m * n + col0 + c] = Unpack<T>::store(t);
            }
            if (threadIdx.x == 0) p.counters[cur_tile] = 0;
          }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(kConsumerWarps * 32));
#pragma unroll
        for (int m = 0; m < M; m++)
#pragma unroll
          for (int v = 0; v < V; v++) acc[m][v] = 0.f;
      }
      if (!more) break;
      cur_tile = next.tile;
    }
    pos = next;
    advance(p, &next);
    // This chunk's lhs values: lane l holds x[k0 + l] (and x[k0 + 32 + l] for 64-row units) for every lhs row (loaded before the wait
    // so the latency hides behind it); rows are then broadcast with shuffles.
    const int k0 = pos.chunk * kUnitRows;
    float xa[M], xb[M];
#pragma unroll
    for (int m = 0; m < M; m++) {
      const T* xr = lhs + (long long)m * p.lhs_m + (long long)(k0 + lane) * p.lhs_k;
      xa[m] = (m < p.m && k0 + lane < p.k) ? Unpack<T>::one(*xr) : 0.f;
      xb[m] = (kUnitRows > 32 && m < p.m && k0 + 32 + lane < p.k) ? Unpack<T>::one(xr[32 * p.lhs_k]) : 0.f;
    }
    if (!mbar_wait(&full[stage], phase)) {
      if (lane == 0) atomicExch(p.error_flag, 2);
      return;
    }
    // Rows and columns past the matrix edge were zero-filled by the copy, so no bounds checks here.
    const unsigned char* src = stage_base + (size_t)stage * kStageBytes + lane * 16 + (size_t)warp * kTileBytes;
#pragma unroll
    for (int r8 = 0; r8 < kUnitRows / kConsumerWarps; r8++) {
      const int r = r8 * kConsumerWarps + warp;
      const uint4 raw = *reinterpret_cast<const uint4*>(src + (size_t)r8 * kConsumerWarps * kTileBytes);
      float w[V];
      Unpack<T>::to_float(raw, w);
#pragma unroll
      for (int m = 0; m < M; m++) {
        const float xv = __shfl_sync(0xffffffffu, r8 * kConsumerWarps < 32 ? xa[m] : xb[m], r & 31);
#pragma unroll
        for (int v = 0; v < V; v++) acc[m][v] = fmaf(xv, w[v], acc[m][v]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[stage]);
    if (++stage == p.stages) {
      stage = 0;
      phase ^= 1;
    }
  }
}

inline size_t smem_bytes(int stages, int M, int cols) {
  return (size_t)stages * kStageBytes + 2 * (size_t)stages * sizeof(uint64_t) + 16 + (size_t)kConsumerWarps * M * cols * sizeof(float);
}

}  // namespace tma
}  // namespace pjrtx

// Weight-streaming contraction for m <= 8: out[m, n] = sum_k lhs[m, k] * rhs[k, n], rhs row-major with n contiguous.
//
// The kernel is bandwidth-bound (every rhs element is read once and used m times), so it is built around keeping
// enough bytes in flight per SM with few threads: persistent CTAs (two per SM) each own a ring of shared-memory stages
// that one producer warp fills with bulk asynchronous copies (completion counted on an mbarrier), while eight consumer
// warps read finished stages and accumulate in registers. Each stage is one tiled TMA copy (cp.async.bulk.tensor.2d)
// of a 64-row x 512-byte box described by a tensor map of the rhs; rows and columns past the matrix edge arrive as
// zeros, so ragged k and n need no special case.
//
// Work decomposition (stream-K): the rhs is cut into units of kUnitRows rows x one 512-byte column tile, ordered
// tile-major; CTA b of G takes the b-th contiguous share of all units, so every SM streams the same number of bytes
// whatever the shape. A CTA that does not cover a tile's whole k range writes an f32 partial; the CTA that arrives
// last for a tile folds the partials in CTA order (fixed order: results are identical from run to run).
//
// Segments. One launch runs up to kSegmentMax *segments* one after the other; a segment is a group of up to kGroupMax
// contractions that share an lhs. Segment s + 1 reads what segment s wrote, so the consumers of all CTAs meet at a
// grid-wide barrier between segments (every CTA of the grid is resident: the grid never exceeds two CTAs per SM) -
// but the producer warp does not: the weights depend on nothing, so it keeps filling the ring with the next segment's
// first units while the consumers fold, wait and prepare, and HBM stays busy across what used to be four kernel
// boundaries (projection -> normalisation -> projection -> activation -> projection ...). What used to run in the
// small kernels between two contractions is done where the values are touched anyway:
//   * lhs transforms, applied by every CTA as it loads its lhs values:
//       kLhsRmsNorm   h[k] = round(round(x[k] * rsqrt(sum(x^2) * scale + eps)) * gain[k]); every CTA reduces the row
//                     itself (a few KB from L2), in the same order, so all CTAs use the same factor
//       kLhsSiluMul   h[k] = round(round(g[k] * round(logistic(g[k]))) * u[k])
//     with `round` = rounding to the element type, as the op-by-op program rounds;
//   * a residual epilogue, applied by the CTA that completes a tile: out = round(residual + round(sum)); the same CTA
//     leaves the tile's sum of squares for a normalising successor, which then needs 64 bytes per row, not the row.
//
// Programmatic dependent launch: the kernel lets its successor start at once (griddepcontrol.launch_dependents) and
// itself waits for its predecessor (griddepcontrol.wait) only before the first access that can depend on it: the
// producer may already be copying rhs tiles (weights are never written by the stream's earlier work), the consumers
// wait before they read lhs or write anything.
//
// Weight tiles are read once: their copies carry an evict-first L2 policy, so that a long stream does not push the
// small, reused operands of the neighbouring kernels out of L2 (measured on the 8B-shape decode step: 3.50 ms per step
// with the policy, 3.58 ms without). Requesting tiles into L2 ahead of the copies (cp.async.bulk.prefetch.tensor, 8 to
// 64 units in front, continuously or only at start) was measured too and made every configuration slower.
//
// Every wait (mbarrier or grid barrier) is bounded by time: a launch has `timeout_ns` from its start; the thread that
// sees the deadline pass raises *error_flag, sets the CTA's abort word, and every other wait of the CTA gives up at its
// next check, so a launch that cannot finish costs one timeout and returns.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pjrtx {
namespace tma {

constexpr int kGroupMax = 4;        // contractions sharing an lhs
constexpr int kSegmentMax = 4;      // dependent groups in one launch
constexpr int kUnitRows = 64;       // rows per unit
constexpr int kTileBytes = 512;     // bytes per row per unit (one warp x 16 B)
constexpr int kStageBytes = kUnitRows * kTileBytes;  // 32 KiB
constexpr int kConsumerWarps = 8;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = (kConsumerWarps + 1) * 32;
constexpr unsigned long long kDefaultTimeoutNs = 2000000000ull;  // budget of one launch for all of its waits

enum LhsKind { kLhsPlain = 0, kLhsRmsNorm = 1, kLhsSiluMul = 2 };

struct Segment {
  const void* lhs;                    // plain: the operand; rms_norm: x; silu_mul: the gate
  const void* lhs2;                   // rms_norm: gain[k] (contiguous); silu_mul: up (same strides as lhs)
  long long lhs_m, lhs_k;             // element strides
  float norm_scale, norm_eps;         // rms_norm: factor = rsqrt(sum(x^2) * norm_scale + norm_eps)
  int lhs_kind;
  int m, k;
  int count;                          // contractions sharing lhs
  int tile_begin[kGroupMax + 1];      // column-tile prefix sums over the group
  void* out[kGroupMax];
  const void* residual[kGroupMax];    // non-null: out = round(residual + round(sum)), same layout as out
  long long n[kGroupMax];
  int chunks;                         // ceil(k / kUnitRows)
  int max_contrib;                    // partial slots per tile
  long long units;                    // tiles * chunks; CTA b owns units [b*units/grid, (b+1)*units/grid)
  float* partials;                    // [tiles][max_contrib][M][tile columns]
  unsigned* counters;                 // [tiles], zero before the first launch, left zero by every launch
  // Sum of squares of the rows, by column tile. A segment with one contraction whose result the next segment
  // normalises writes, per completed tile, the sum of its (rounded) outputs' squares to ssq_out[tile * M + m]; the
  // normalising segment then adds `ssq_tiles` numbers per row (ssq_in) instead of reading the whole row again.
  float* ssq_out;
  const float* ssq_in;
  int ssq_tiles;
};

struct Params {
  Segment seg[kSegmentMax];
  int segments;
  // Grid barrier state: [0] launch epoch e (how many launches have passed their first barrier), [1 + b] arrivals at
  // barrier b since the memory was cleared (monotonic: a launch waits for (e + 1) * grid). Nothing is ever reset, so no
  // CTA waits for a second round trip; counts wrap consistently in 32 bits.
  unsigned* barrier;
  int* error_flag;
  unsigned long long timeout_ns;      // budget for all waits of the launch, counted from its start
  int stages;
  int early_rhs;                      // rhs copies may start before the preceding kernel of the stream has finished
  int evict_first;                    // rhs copies carry the evict-first L2 policy
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
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Deadline of the launch and the CTA's abort word (shared memory), passed to every wait.
struct WaitBudget {
  unsigned long long deadline;
  volatile int* abort;
};
// True when the wait must be given up: another thread of the CTA already did, or the deadline has passed.
__device__ __forceinline__ bool give_up(const WaitBudget& w) {
  if (*w.abort) return true;
  if (global_timer_ns() > w.deadline) {
    *w.abort = 1;
    return true;
  }
  return false;
}
// Bounded wait; false when it was given up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, const WaitBudget& w) {
  for (unsigned spin = 0;; spin++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 15) == 15 && give_up(w)) return false;
  }
}
// Arrival counter with release/acquire semantics at device scope: together with the CTA barriers around it, the
// partial sums every thread of this CTA wrote are visible to whichever CTA observes the final count.
__device__ __forceinline__ unsigned arrive_acq_rel(unsigned* counter) {
  unsigned old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
  return old;
}
__device__ __forceinline__ unsigned load_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One box of the tensor map: x = first column (must be a multiple of 16 bytes), y = first row.
__device__ __forceinline__ void tensor_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tensor_load_2d_hint(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar,
                                                    uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(
          smem_u32(smem_dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
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

__device__ __forceinline__ void locate_tile(const Segment& p, Cursor* c) {
  int g = 0;
#pragma unroll
  for (int q = 1; q < kGroupMax; q++)
    if (q < p.count && c->tile >= p.tile_begin[q]) g = q;
  c->group = g;
  c->tile_in_group = c->tile - p.tile_begin[g];
}

__device__ __forceinline__ Cursor cursor_at(const Segment& p, long long u) {
  Cursor c;
  c.tile = (int)(u / p.chunks);
  c.chunk = (int)(u - (long long)c.tile * p.chunks);
  locate_tile(p, &c);
  return c;
}

__device__ __forceinline__ void advance(const Segment& p, Cursor* c) {
  if (++c->chunk == p.chunks) {
    c->chunk = 0;
    c->tile++;
    locate_tile(p, c);
  }
}

struct Maps {
  CUtensorMap map[kSegmentMax][kGroupMax];
};

template <typename T> __device__ __forceinline__ float round_to(float v) { return Unpack<T>::one(Unpack<T>::store(v)); }

// One lhs value of a segment, transformed as the segment asks (KIND is a compile-time constant: the unit loop is
// instantiated per kind, the kernel is bound by instruction issue as much as by bytes). `factor` is the row's
// normalisation factor; `a` / `b` point at the row's first element of lhs / lhs2.
template <typename T, int KIND>
__device__ __forceinline__ float lhs_value(const T* a, const T* b, int stride, int kk, float factor) {
  const float x = Unpack<T>::one(a[kk * stride]);
  if (KIND == kLhsPlain) return x;
  if (KIND == kLhsRmsNorm) {
    const float w = Unpack<T>::one(b[kk]);
    return round_to<T>(round_to<T>(x * factor) * w);
  }
  const float u = Unpack<T>::one(b[kk * stride]);
  const float sg = round_to<T>(1.0f / (1.0f + expf(-x)));
  return round_to<T>(round_to<T>(x * sg) * u);
}

// Consumer-side state that lives across segments.
struct ConsumerState {
  int stage;
  unsigned phase;
};

// All units of one segment owned by this CTA: accumulate, flush at tile changes (partial or final), fold as the last
// arriver. Returns false when a bounded wait gave up.
template <typename T, int M, int KIND, bool EXTRAS>
__device__ __forceinline__ bool run_units(const Params& p, const Segment& sg, const float (&factor)[M], unsigned char* stage_base,
                                          uint64_t* full, uint64_t* empty, int* flags, float* red, ConsumerState* cs, long long u_begin,
                                          long long u_end, const WaitBudget& budget) {
  constexpr int V = Unpack<T>::V;
  constexpr int COLS = 32 * V;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float acc[M][V];
#pragma unroll
  for (int m = 0; m < M; m++)
#pragma unroll
    for (int v = 0; v < V; v++) acc[m][v] = 0.f;
  const T* lhs_row[M];
  const T* lhs2_row[M];
#pragma unroll
  for (int m = 0; m < M; m++) {
    const int mm = m < sg.m ? m : 0;
    lhs_row[m] = static_cast<const T*>(sg.lhs) + (long long)mm * sg.lhs_m;
    lhs2_row[m] = KIND == kLhsSiluMul ? static_cast<const T*>(sg.lhs2) + (long long)mm * sg.lhs_m : static_cast<const T*>(sg.lhs2);
  }
  const int lhs_stride = (int)sg.lhs_k;
  const int seg_m = sg.m, seg_k = sg.k, chunks = sg.chunks;
  long long cur_tile = -1;
  Cursor pos{};
  Cursor next = cursor_at(sg, u_begin);
  const int count = (int)(u_end - u_begin);
  int stage = cs->stage;
  unsigned phase = cs->phase;
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
        asm volatile("bar.sync 1, %0;" ::"r"(kConsumers));
        // CTA that owns unit u: the largest b with b*units/grid <= u, i.e. ceil((u+1)*grid/units) - 1.
        const long long tile_units_begin = cur_tile * chunks;
        const long long first_cta = ((tile_units_begin + 1) * gridDim.x + sg.units - 1) / sg.units - 1;
        const long long last_cta = ((tile_units_begin + chunks) * gridDim.x + sg.units - 1) / sg.units - 1;
        const int contributors = (int)(last_cta - first_cta + 1);
        const long long n = sg.n[pos.group];
        const long long col0 = (long long)pos.tile_in_group * COLS;
        T* out = static_cast<T*>(sg.out[pos.group]);
        const T* residual = EXTRAS ? static_cast<const T*>(sg.residual[pos.group]) : nullptr;
        float sq[M];  // this thread's share of the tile's sum of squares, by row
#pragma unroll
        for (int m = 0; m < M; m++) sq[m] = 0.f;
        auto emit = [&](int m, int c, float t) {
          if (m < seg_m && col0 + c < n) {
            const long long at = (long long)m * n + col0 + c;
            T r = Unpack<T>::store(t);
            if (residual) r = Unpack<T>::store(Unpack<T>::one(residual[at]) + Unpack<T>::one(r));
            out[at] = r;
            if (EXTRAS) {
              const float rv = Unpack<T>::one(r);
#pragma unroll
              for (int q = 0; q < M; q++)
                if (q == m) sq[q] = fmaf(rv, rv, sq[q]);
            }
          }
        };
        // Sum of squares of a completed tile, reduced in a fixed order; overwrites `red` (all reads of it are done).
        auto publish_ssq = [&]() {
          if (!EXTRAS || !sg.ssq_out) return;
          asm volatile("bar.sync 1, %0;" ::"r"(kConsumers));
#pragma unroll
          for (int m = 0; m < M; m++) {
            float v = sq[m];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            if (lane == 0) red[m * kConsumerWarps + warp] = v;
          }
          asm volatile("bar.sync 1, %0;" ::"r"(kConsumers));
          if (threadIdx.x < M) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; w++) v += red[threadIdx.x * kConsumerWarps + w];
            sg.ssq_out[cur_tile * M + threadIdx.x] = v;
          }
        };
        float* slot = sg.partials + ((cur_tile * sg.max_contrib + (blockIdx.x - first_cta)) * M) * COLS;
        for (int idx = threadIdx.x; idx < M * COLS; idx += kConsumers) {
          const int m = idx / COLS, c = idx % COLS;
          float t = 0.f;
#pragma unroll
          for (int w = 0; w < kConsumerWarps; w++) t += red[(w * M + m) * COLS + c];
          if (contributors == 1) emit(m, c, t);
          else slot[idx] = t;
        }
        if (contributors == 1) publish_ssq();
        if (contributors > 1) {
          asm volatile("bar.sync 1, %0;" ::"r"(kConsumers));
          if (threadIdx.x == 0) flags[0] = arrive_acq_rel(&sg.counters[cur_tile]) == (unsigned)contributors - 1;
          asm volatile("bar.sync 1, %0;" ::"r"(kConsumers));
          if (flags[0]) {
            const float* base = sg.partials + (cur_tile * sg.max_contrib * (long long)M) * COLS;
            for (int idx = threadIdx.x; idx < M * COLS; idx += kConsumers) {
              const int m = idx / COLS, c = idx % COLS;
              float t = 0.f;
              // All of a tile's partials (12 to 19 contributors at the decode shapes) are requested in one round of
              // loads, then added in CTA order: the fold sits in the kernel's tail, where a round trip is what it costs.
              // (Without the arrival counter - partials published as {value, launch stamp} pairs that the tile's first
              // contributor polls and folds, no fence and no atomic - the 8B-shape step measured 3.30 against 3.29 ms.)
              for (int q = 0; q < contributors; q += 24) {
                float v[24];
#pragma unroll
                for (int e = 0; e < 24; e++) v[e] = q + e < contributors ? __ldcg(base + (long long)(q + e) * M * COLS + idx) : 0.f;
#pragma unroll
                for (int e = 0; e < 24; e++) t += v[e];
              }
              emit(m, c, t);
            }
            if (threadIdx.x == 0) sg.counters[cur_tile] = 0;
            publish_ssq();
          }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(kConsumers));
#pragma unroll
        for (int m = 0; m < M; m++)
#pragma unroll
          for (int v = 0; v < V; v++) acc[m][v] = 0.f;
      }
      if (!more) break;
      cur_tile = next.tile;
    }
    pos = next;
    advance(sg, &next);
    // This chunk's lhs values: lane l holds x[k0 + l] and x[k0 + 32 + l] for every lhs row (loaded before the wait so
    // the latency hides behind it); rows are then broadcast with shuffles.
    static_assert(kUnitRows == 64, "two lhs values per lane and unit");
    const int k0 = pos.chunk * kUnitRows;
    float xa[M], xb[M];
#pragma unroll
    for (int m = 0; m < M; m++) {
      xa[m] = (m < seg_m && k0 + lane < seg_k) ? lhs_value<T, KIND>(lhs_row[m], lhs2_row[m], lhs_stride, k0 + lane, factor[m]) : 0.f;
      xb[m] = (m < seg_m && k0 + 32 + lane < seg_k) ? lhs_value<T, KIND>(lhs_row[m], lhs2_row[m], lhs_stride, k0 + 32 + lane, factor[m]) : 0.f;
    }
    if (!mbar_wait(&full[stage], phase, budget)) {
      if (lane == 0) atomicExch(p.error_flag, 2);
      return false;
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
  cs->stage = stage;
  cs->phase = phase;
  return true;
}

// Two CTAs share an SM while the cross-warp fold buffer is at most 16 KiB (the launch code sizes the grid on that), so
// the register budget must allow it: a chained launch needs its whole grid resident.
// EXTRAS = false is the plain contraction (one segment, untransformed lhs, no residual): the same code with the
// segment machinery compiled out, for the launches that use none of it.
template <typename T, int M, bool EXTRAS>
__global__ void __launch_bounds__(kThreads, (M * Unpack<T>::V <= 16 ? 2 : 1)) stream_tma_kernel(const __grid_constant__ Params p, const __grid_constant__ Maps maps) {
  constexpr int V = Unpack<T>::V;
  constexpr int COLS = 32 * V;  // columns per tile
  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* stage_base = smem_raw;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + (size_t)p.stages * kStageBytes);
  uint64_t* empty = full + p.stages;
  int* flags = reinterpret_cast<int*>(empty + p.stages);  // [0] is_last, [1] barrier ok, [2] abort
  const WaitBudget budget{global_timer_ns() + p.timeout_ns, flags + 2};

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    flags[0] = 0;
    flags[1] = 0;
    flags[2] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ---- producer: one elected lane issues one tensor copy per stage, segment after segment -----------------
    if (lane != 0) return;
    if (!p.early_rhs) asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint64_t policy = p.evict_first ? policy_evict_first() : 0;
    int stage = 0;
    unsigned phase = 0;
    long long issued = 0;
    const int segments = EXTRAS ? p.segments : 1;
    for (int si = 0; si < segments; si++) {
      const Segment& sg = p.seg[EXTRAS ? si : 0];
      const long long u_begin = (long long)blockIdx.x * sg.units / gridDim.x;
      const long long u_end = (long long)(blockIdx.x + 1) * sg.units / gridDim.x;
      if (u_begin >= u_end) continue;
      Cursor cur = cursor_at(sg, u_begin);
      const int count = (int)(u_end - u_begin);
      for (int i = 0; i < count; i++, issued++) {
        if (issued >= p.stages) {
          if (!mbar_wait(&empty[stage], phase ^ 1, budget)) {
            atomicExch(p.error_flag, 1);
            return;
          }
        }
        mbar_expect_tx(&full[stage], kStageBytes);
        if (p.evict_first)
          tensor_load_2d_hint(stage_base + (size_t)stage * kStageBytes, &maps.map[EXTRAS ? si : 0][cur.group],
                              cur.tile_in_group * COLS, cur.chunk * kUnitRows, &full[stage], policy);
        else
          tensor_load_2d(stage_base + (size_t)stage * kStageBytes, &maps.map[EXTRAS ? si : 0][cur.group], cur.tile_in_group * COLS,
                         cur.chunk * kUnitRows, &full[stage]);
        advance(sg, &cur);
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    return;
  }

  // ---- consumer warps ---------------------------------------------------------------------------------------
  asm volatile("griddepcontrol.wait;" ::: "memory");
  float* red = reinterpret_cast<float*>(flags + 4);  // [kConsumerWarps][M][COLS] floats, after the barriers
  ConsumerState cs{0, 0};
  if (!EXTRAS) {
    const Segment& sg = p.seg[0];
    const long long u_begin = (long long)blockIdx.x * sg.units / gridDim.x;
    const long long u_end = (long long)(blockIdx.x + 1) * sg.units / gridDim.x;
    if (u_begin >= u_end) return;
    const float unit_factor[M] = {};
    run_units<T, M, kLhsPlain, false>(p, sg, unit_factor, stage_base, full, empty, flags, red, &cs, u_begin, u_end, budget);
    return;
  }
  unsigned epoch = 0;
  if (p.segments > 1 && threadIdx.x == 0) epoch = *reinterpret_cast<volatile unsigned*>(p.barrier);
  for (int si = 0; si < p.segments; si++) {
    const Segment& sg = p.seg[si];
    if (si > 0) {
      // Grid-wide barrier: everything the previous segment wrote (by any CTA) is complete and visible afterwards.
      unsigned* arrivals = p.barrier + si;  // barrier si - 1 counts in word si
      asm volatile("bar.sync 1, %0;" ::"r"(kConsumers));
      if (threadIdx.x == 0) {
        const unsigned target = (epoch + 1) * gridDim.x;
        __threadfence();
        const unsigned before = arrive_acq_rel(arrivals);
        if (si == 1 && before + 1 == target) *reinterpret_cast<volatile unsigned*>(p.barrier) = epoch + 1;  // every CTA has read it
        bool ok = before + 1 == target;
        for (unsigned spin = 0; !ok; spin++) {
          ok = (int)(load_acquire(arrivals) - target) >= 0;
          if (!ok && (spin & 15) == 15 && give_up(budget)) break;
        }
        if (!ok) atomicExch(p.error_flag, 4);
        flags[1] = ok ? 1 : 0;
      }
      asm volatile("bar.sync 1, %0;" ::"r"(kConsumers));
      if (!flags[1]) return;
    }
    // Row factors of a normalising lhs: sum of squares over the whole row, reduced in a fixed order (the same in
    // every CTA, so all of them use the same factor).
    float factor[M];
#pragma unroll
    for (int m = 0; m < M; m++) factor[m] = 1.f;
    if (sg.lhs_kind == kLhsRmsNorm) {
      if (sg.ssq_in) {
#pragma unroll
        for (int m = 0; m < M; m++) {
          float ss = 0.f;
          for (int t = 0; t < sg.ssq_tiles; t++) ss += __ldcg(sg.ssq_in + t * M + m);
          factor[m] = 1.0f / sqrtf(ss * sg.norm_scale + sg.norm_eps);
        }
      } else {
        const T* x = static_cast<const T*>(sg.lhs);
#pragma unroll
        for (int m = 0; m < M; m++) {
          float ss = 0.f;
          if (m < sg.m)
            for (int kk = threadIdx.x; kk < sg.k; kk += kConsumers) {
              const float xv = Unpack<T>::one(x[(long long)m * sg.lhs_m + (long long)kk * sg.lhs_k]);
              ss = fmaf(xv, xv, ss);
            }
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
          if (lane == 0) red[m * kConsumerWarps + warp] = ss;
        }
        asm volatile("bar.sync 1, %0;" ::"r"(kConsumers));
#pragma unroll
        for (int m = 0; m < M; m++) {
          float ss = 0.f;
#pragma unroll
          for (int w = 0; w < kConsumerWarps; w++) ss += red[m * kConsumerWarps + w];
          factor[m] = 1.0f / sqrtf(ss * sg.norm_scale + sg.norm_eps);
        }
        asm volatile("bar.sync 1, %0;" ::"r"(kConsumers));
      }
    }
    const long long u_begin = (long long)blockIdx.x * sg.units / gridDim.x;
    const long long u_end = (long long)(blockIdx.x + 1) * sg.units / gridDim.x;
    if (u_begin >= u_end) continue;
    bool ok;
    if (sg.lhs_kind == kLhsPlain)
      ok = run_units<T, M, kLhsPlain, true>(p, sg, factor, stage_base, full, empty, flags, red, &cs, u_begin, u_end, budget);
    else if (sg.lhs_kind == kLhsRmsNorm)
      ok = run_units<T, M, kLhsRmsNorm, true>(p, sg, factor, stage_base, full, empty, flags, red, &cs, u_begin, u_end, budget);
    else
      ok = run_units<T, M, kLhsSiluMul, true>(p, sg, factor, stage_base, full, empty, flags, red, &cs, u_begin, u_end, budget);
    if (!ok) return;
  }
}

inline size_t smem_bytes(int stages, int M, int cols) {
  return (size_t)stages * kStageBytes + 2 * (size_t)stages * sizeof(uint64_t) + 16 + (size_t)kConsumerWarps * M * cols * sizeof(float);
}

}  // namespace tma
}  // namespace pjrtx

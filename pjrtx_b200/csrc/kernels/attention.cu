// Split-KV attention for decode: one query position per sequence, grouped-query heads.
//
// out[b, h, :] = softmax_j( q[b, h, :] . k[b, j, g, :] * scale  for j <= limit ) . v[b, j, g, :],   g = h / rep
//
// Semantics are those of the reference's attention custom call (src/backend/mlx_metal/api.cc:4929-5043, mask
// api.cc:937-950: key index <= token_index + query index, scale 1/sqrt(head_dim)) and of the explicit
// dot_general -> masked softmax -> dot_general form the planner recognises.
//
// The cache is the only large operand (2 * (limit+1) * kv_heads * head_dim elements per sequence), so the kernel is
// HBM-bound and organised around reading each K/V row exactly once with 16-byte loads: all `rep` query heads that
// share a KV head are processed by the same CTA; a group of head_dim*esize/16 lanes owns a key row, keeps its slice
// of every query head and of every output accumulator in registers and needs only log2(group) shuffles per key for
// the score. At batch 1 the kernel is bound by latency, not bytes, so the work per CTA is short and flat: a chunk of
// keys is loaded at once, one block-wide maximum per chunk replaces per-key rescaling, and partial sums of different
// threads are simply added. The key range is split across CTAs (grid.x); partial (max, sum, out) triples go to an f32
// workspace and the CTA that arrives last merges them in split order (deterministic).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <type_traits>

#include "../common.h"
#include "kernels.h"

namespace pjrtx {

namespace {

template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int V = 4;
  static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
    f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
  }
  static __device__ __forceinline__ float round(float v) { return v; }
  static __device__ __forceinline__ float store(float v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
  static constexpr int V = 8;
  static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
    f[0] = __uint_as_float(r.x << 16); f[1] = __uint_as_float(r.x & 0xffff0000u);
    f[2] = __uint_as_float(r.y << 16); f[3] = __uint_as_float(r.y & 0xffff0000u);
    f[4] = __uint_as_float(r.z << 16); f[5] = __uint_as_float(r.z & 0xffff0000u);
    f[6] = __uint_as_float(r.w << 16); f[7] = __uint_as_float(r.w & 0xffff0000u);
  }
  static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
  static __device__ __forceinline__ __nv_bfloat16 store(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<__half> {
  static constexpr int V = 8;
  static __device__ __forceinline__ void unpack(const uint4& r, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float2 p = __half22float2(h[i]);
      f[2 * i] = p.x;
      f[2 * i + 1] = p.y;
    }
  }
  static __device__ __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
  static __device__ __forceinline__ __half store(float v) { return __float2half_rn(v); }
};

__device__ __forceinline__ long long load_scalar(const void* p, int dtype) {
  switch (dtype) {
    case kS32: return *static_cast<const int*>(p);
    case kU32: return *static_cast<const unsigned*>(p);
    case kS64: return *static_cast<const long long*>(p);
    case kU64: return (long long)*static_cast<const unsigned long long*>(p);
    default: return 0;
  }
}

struct DecodeArgs {
  long long batch, heads, kv_heads, kv_len;
  long long q_batch_stride, q_head_stride;          // elements
  long long kv_batch_stride, kv_row_stride, kv_head_stride;
  int token_dtype;
  int round_scores;
  float scale;
  int splits;
  float* workspace;   // [batch * kv_heads][splits][REP][HD + 2]
  unsigned* counters;  // [batch * kv_heads]
  int* error_flag;     // receives a non-zero code when a bounded wait gives up (may be null)
  int early_kv;        // cache rows below the token index are not written by earlier work of the stream
  // Weights of the contraction that follows (never written by the stream): requested into L2 by this kernel's CTAs as
  // they start, so that HBM works through the attention step's latencies instead of idling.
  const unsigned char* prefetch;
  unsigned long long prefetch_bytes;
  // 1: the whole grid is resident at once, so the CTAs of a (sequence, KV head) wait for each other and each merges
  // its own slice of the outputs instead of leaving the whole merge to the CTA that arrives last.
  int coop_merge;
  unsigned long long timeout_ns;
};

constexpr int kMergeChunk = 24;  // splits whose (max, sum, value) a merging thread requests at once

// PJRTX_B200_ATTENTION_COOP_MERGE=0 makes the CTA that arrives last merge a tile's splits alone.
inline bool coop_merge_allowed() {
  static const bool allowed = [] {
    const char* e = getenv("PJRTX_B200_ATTENTION_COOP_MERGE");
    return !(e && *e && atoi(e) == 0);
  }();
  return allowed;
}

// Every CTA asks for its share of [prefetch, prefetch + prefetch_bytes) in 16 KiB bulk requests (no destination, no
// completion to wait for).
__device__ __forceinline__ void prefetch_next_weights(const DecodeArgs& a) {
  if (!a.prefetch_bytes) return;
  constexpr unsigned long long kPiece = 16384;
  const unsigned long long pieces = (a.prefetch_bytes + kPiece - 1) / kPiece;
  const unsigned long long cta = blockIdx.x + (unsigned long long)gridDim.x * (blockIdx.y + (unsigned long long)gridDim.y * blockIdx.z);
  const unsigned long long ctas = (unsigned long long)gridDim.x * gridDim.y * gridDim.z;
  for (unsigned long long i = cta * blockDim.x + threadIdx.x; i < pieces; i += ctas * blockDim.x) {
    const unsigned long long at = i * kPiece;
    const unsigned size = (unsigned)((a.prefetch_bytes - at < kPiece ? a.prefetch_bytes - at : kPiece) & ~15ull);
    if (size) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(a.prefetch + at), "r"(size) : "memory");
  }
}

// Second half of a split: after every thread has written its part of this split's (max, sum, out) triple to the
// workspace, the CTA that arrives last for the (sequence, KV head) merges all splits in split order and writes `out`.
// `scratch` is shared memory for 64 * REP * 2 floats that nothing else uses any more.
template <typename T, int REP, int HD, int THREADS>
__device__ __forceinline__ void merge_splits(const DecodeArgs& a, long long tile, int b, int g, float* scratch, int* is_last,
                                             T* __restrict__ out) {
  if (a.coop_merge) {
    // Cooperative merge. counters[2 * tile] counts arrivals, counters[2 * tile + 1] departures (the last one to leave
    // clears both). Every CTA of the launch is resident (the host checked), so the wait ends as soon as the slowest split
    // has published; it is bounded by time all the same.
    unsigned* arrive = a.counters + 2 * tile;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      atomicAdd(arrive, 1u);
      unsigned long long t0;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
      bool ok = false;
      for (unsigned spin = 0;; spin++) {
        unsigned seen;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(arrive) : "memory");
        if (seen >= (unsigned)a.splits) {
          ok = true;
          break;
        }
        if ((spin & 63) == 63) {
          unsigned long long t1;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
          if (t1 - t0 > a.timeout_ns) break;
        }
      }
      if (!ok && a.error_flag) atomicExch(a.error_flag, 5);
      *is_last = ok ? 1 : 0;
    }
    __syncthreads();
    if (!*is_last) return;
    const int split = blockIdx.x;
    const int per = (REP * HD + a.splits - 1) / a.splits;
    const int lo = split * per, hi = min(lo + per, REP * HD);
    const float* base = a.workspace + tile * a.splits * (long long)REP * (HD + 2);
    const long long split_stride = (long long)REP * (HD + 2);
    // All loads of a round are issued before the first is used (a dependent load per split would cost a round trip to
    // L2 each): up to kMergeChunk splits need one round, more need two passes of chunks.
    constexpr int CH = kMergeChunk;
    for (int idx = lo + threadIdx.x; idx < hi; idx += THREADS) {
      const int r = idx / HD, d = idx % HD;
      const float* row = base + r * (HD + 2);
      float mm = -INFINITY, acc = 0.f, lsum = 0.f;
      if (a.splits <= CH) {
        float ms[CH], lv[CH], ov[CH];
#pragma unroll
        for (int u = 0; u < CH; u++) {
          const bool in = u < a.splits;
          const float* src = row + (in ? u : 0) * split_stride;
          ms[u] = in ? __ldcg(src + HD) : -INFINITY;
          lv[u] = in ? __ldcg(src + HD + 1) : 0.f;
          ov[u] = in ? __ldcg(src + d) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < CH; u++) mm = fmaxf(mm, ms[u]);
#pragma unroll
        for (int u = 0; u < CH; u++) {  // split order, the same arithmetic as the single-CTA merge
          const float w = ms[u] == -INFINITY ? 0.f : __expf(ms[u] - mm);
          lsum = fmaf(lv[u], w, lsum);
          acc = fmaf(ov[u], w, acc);
        }
      } else {
        for (int sp0 = 0; sp0 < a.splits; sp0 += CH) {
          float ms[CH];
#pragma unroll
          for (int u = 0; u < CH; u++) ms[u] = sp0 + u < a.splits ? __ldcg(row + (sp0 + u) * split_stride + HD) : -INFINITY;
#pragma unroll
          for (int u = 0; u < CH; u++) mm = fmaxf(mm, ms[u]);
        }
        for (int sp0 = 0; sp0 < a.splits; sp0 += CH) {
          float ms[CH], lv[CH], ov[CH];
#pragma unroll
          for (int u = 0; u < CH; u++) {
            const bool in = sp0 + u < a.splits;
            const float* src = row + (in ? sp0 + u : 0) * split_stride;
            ms[u] = in ? __ldcg(src + HD) : -INFINITY;
            lv[u] = in ? __ldcg(src + HD + 1) : 0.f;
            ov[u] = in ? __ldcg(src + d) : 0.f;
          }
#pragma unroll
          for (int u = 0; u < CH; u++) {
            const float w = ms[u] == -INFINITY ? 0.f : __expf(ms[u] - mm);
            lsum = fmaf(lv[u], w, lsum);
            acc = fmaf(ov[u], w, acc);
          }
        }
      }
      out[b * a.q_batch_stride + (g * REP + r) * a.q_head_stride + d] = Elem<T>::store(lsum > 0.f ? acc / lsum : 0.f);
    }
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(arrive + 1, 1u) == (unsigned)a.splits - 1) {
      arrive[0] = 0;
      arrive[1] = 0;
    }
    return;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) *is_last = atomicAdd(&a.counters[tile], 1u) == (unsigned)a.splits - 1;
  __syncthreads();
  if (!*is_last) return;
  __threadfence();
  // Merge of the splits in two rounds of loads: (max, sum) of every split and head into shared memory, then all the
  // `out` values a thread needs at once; the weights exp(max_split - max) are applied in split order.
  const float* base = a.workspace + tile * a.splits * (long long)REP * (HD + 2);
  const long long split_stride = (long long)REP * (HD + 2);
  float* sm_ml = scratch;  // [splits][REP][2], splits <= 64
  for (int idx = threadIdx.x; idx < a.splits * REP * 2; idx += THREADS) {
    const int sp = idx / (REP * 2), r = (idx / 2) % REP, which = idx & 1;
    sm_ml[idx] = __ldcg(base + sp * split_stride + r * (HD + 2) + HD + which);
  }
  __syncthreads();
  constexpr int PER_THREAD = (REP * HD + THREADS - 1) / (THREADS);
  constexpr int BATCH = 16;
  float acc[PER_THREAD], lsum[PER_THREAD], mmax[PER_THREAD];
#pragma unroll
  for (int e = 0; e < PER_THREAD; e++) {
    const int idx = threadIdx.x + e * THREADS;
    const int r = idx < REP * HD ? idx / HD : 0;
    float mm = -INFINITY;
    for (int sp = 0; sp < a.splits; sp++) mm = fmaxf(mm, sm_ml[(sp * REP + r) * 2]);
    mmax[e] = mm;
    acc[e] = 0.f;
    lsum[e] = 0.f;
  }
  for (int sp0 = 0; sp0 < a.splits; sp0 += BATCH) {
    float ov[PER_THREAD][BATCH];
#pragma unroll
    for (int e = 0; e < PER_THREAD; e++) {
      const int idx = threadIdx.x + e * THREADS;
      const int r = idx < REP * HD ? idx / HD : 0, d = idx < REP * HD ? idx % HD : 0;
#pragma unroll
      for (int u = 0; u < BATCH; u++)
        ov[e][u] = sp0 + u < a.splits ? __ldcg(base + (sp0 + u) * split_stride + r * (HD + 2) + d) : 0.f;
    }
#pragma unroll
    for (int e = 0; e < PER_THREAD; e++) {
      const int idx = threadIdx.x + e * THREADS;
      const int r = idx < REP * HD ? idx / HD : 0;
#pragma unroll
      for (int u = 0; u < BATCH; u++) {
        if (sp0 + u < a.splits) {
          const float ms = sm_ml[((sp0 + u) * REP + r) * 2];
          const float w = ms == -INFINITY ? 0.f : __expf(ms - mmax[e]);
          lsum[e] = fmaf(sm_ml[((sp0 + u) * REP + r) * 2 + 1], w, lsum[e]);
          acc[e] = fmaf(ov[e][u], w, acc[e]);
        }
      }
    }
  }
#pragma unroll
  for (int e = 0; e < PER_THREAD; e++) {
    const int idx = threadIdx.x + e * THREADS;
    if (idx < REP * HD) {
      const int r = idx / HD, d = idx % HD;
      out[b * a.q_batch_stride + (g * REP + r) * a.q_head_stride + d] = Elem<T>::store(lsum[e] > 0.f ? acc[e] / lsum[e] : 0.f);
    }
  }
  if (threadIdx.x == 0) a.counters[tile] = 0;
}

// One CTA = one (sequence, KV head, key split). The split is walked in chunks of GROUPS * KPG keys; per chunk every
// lane group (HD * esize / 16 lanes, one 16-byte slice of a row per lane) takes KPG keys:
//   1. all K and V rows of the chunk are requested at once (2 * KPG 16-byte loads in flight per lane),
//   2. scores = q . k for the `REP` query heads that share the KV head (log2(lanes per group) shuffles per score),
//   3. one block-wide maximum per head (shuffles + one shared-memory round), so that
//   4. p = exp(score - max) needs no per-key rescaling and the per-thread (sum, out) accumulators of different
//      threads are plain partial sums; they are rescaled once per chunk when the running maximum moves.
// After the last chunk the partial sums are added across the CTA, and (max, sum, out) goes to the workspace; the CTA
// that arrives last for the (sequence, KV head) merges the splits in split order.
template <typename T, int REP, int HD, int KPG, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_kernel(DecodeArgs a, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                   const void* __restrict__ token, T* __restrict__ out) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  prefetch_next_weights(a);
  if (!a.early_kv) asm volatile("griddepcontrol.wait;" ::: "memory");
  constexpr int V = Elem<T>::V;
  constexpr int LPK = HD / V;                  // lanes per key row
  constexpr int GPW = 32 / LPK;                // lane groups per warp
  constexpr int GROUPS = WARPS * GPW;         // lane groups per CTA
  constexpr int CHUNK = GROUPS * KPG;          // keys per chunk
  static_assert(LPK >= 1 && LPK <= 32 && (LPK & (LPK - 1)) == 0, "head_dim must give a power-of-two lane group");
  __shared__ float sm_max[2][WARPS][REP];     // double-buffered: one barrier per chunk
  __shared__ float sm_l[WARPS][REP];
  __shared__ float sm_o[WARPS][REP][HD];
  __shared__ int is_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPK, gl = lane % LPK;  // lane group within the warp, slice of the row
  const int group = warp * GPW + sub;
  const int split = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  long long limit = load_scalar(token, a.token_dtype);  // keys 0..limit are visible
  if (limit >= a.kv_len) limit = a.kv_len - 1;
  const long long count = limit + 1;
  const long long per_split = (count + a.splits - 1) / a.splits;
  const long long j_begin = (long long)split * per_split;
  const long long j_end = min(j_begin + per_split, count);
  const T* kb = k + b * a.kv_batch_stride + g * a.kv_head_stride + gl * V;
  const T* vb = v + b * a.kv_batch_stride + g * a.kv_head_stride + gl * V;
  if (a.early_kv) {
    // Rows below the token index hold what earlier steps left: ask for the first chunk's rows now, so that they come
    // from L2 once the predecessor (which writes the row at the token index, and the query) has finished.
#pragma unroll
    for (int u = 0; u < KPG; u++) {
      const long long j = j_begin + group + (long long)u * GROUPS;
      if (j < j_end && j < limit) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(kb + j * a.kv_row_stride));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(vb + j * a.kv_row_stride));
      }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
  }

  // Query slices of the `rep` heads that share this KV head.
  float qf[REP][V];
#pragma unroll
  for (int r = 0; r < REP; r++) {
    const T* qp = q + b * a.q_batch_stride + (g * REP + r) * a.q_head_stride + gl * V;
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(qp));
    Elem<T>::unpack(raw, qf[r]);
  }
  float m_run[REP], l[REP], o[REP][V];
#pragma unroll
  for (int r = 0; r < REP; r++) {
    m_run[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < V; i++) o[r][i] = 0.f;
  }

  int parity = 0;
  for (long long c0 = j_begin; c0 < j_end; c0 += CHUNK, parity ^= 1) {  // same trip count for every thread of the CTA
    uint4 kr[KPG], vr[KPG];
    bool ok[KPG];
#pragma unroll
    for (int u = 0; u < KPG; u++) {
      const long long j = c0 + group + (long long)u * GROUPS;  // consecutive groups read consecutive rows
      ok[u] = j < j_end;
      const long long jj = ok[u] ? j : j_begin;  // a valid row; its contribution is masked below
      kr[u] = __ldg(reinterpret_cast<const uint4*>(kb + jj * a.kv_row_stride));
      vr[u] = __ldg(reinterpret_cast<const uint4*>(vb + jj * a.kv_row_stride));
    }
    float s[KPG][REP];
    float mx[REP];
#pragma unroll
    for (int r = 0; r < REP; r++) mx[r] = -INFINITY;
#pragma unroll
    for (int u = 0; u < KPG; u++) {
      float kf[V];
      Elem<T>::unpack(kr[u], kf);
#pragma unroll
      for (int r = 0; r < REP; r++) {
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < V; i++) d = fmaf(qf[r][i], kf[i], d);
#pragma unroll
        for (int off = LPK >> 1; off > 0; off >>= 1) d += __shfl_xor_sync(0xffffffffu, d, off);
        if (a.round_scores) d = Elem<T>::round(d);
        s[u][r] = ok[u] ? d * a.scale : -INFINITY;
        mx[r] = fmaxf(mx[r], s[u][r]);
      }
    }
    // Block-wide maximum per head.
#pragma unroll
    for (int r = 0; r < REP; r++) {
#pragma unroll
      for (int off = LPK; off < 32; off <<= 1) mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], off));
      if (lane == 0) sm_max[parity][warp][r] = mx[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < REP; r++) {
      float m_new = m_run[r];
#pragma unroll
      for (int w = 0; w < WARPS; w++) m_new = fmaxf(m_new, sm_max[parity][w][r]);
      if (m_new != m_run[r]) {  // uniform over the CTA
        const float corr = m_run[r] == -INFINITY ? 0.f : __expf(m_run[r] - m_new);
        l[r] *= corr;
#pragma unroll
        for (int i = 0; i < V; i++) o[r][i] *= corr;
        m_run[r] = m_new;
      }
    }
#pragma unroll
    for (int u = 0; u < KPG; u++) {
      float vf[V];
      Elem<T>::unpack(vr[u], vf);
#pragma unroll
      for (int r = 0; r < REP; r++) {
        const float p = s[u][r] == -INFINITY ? 0.f : __expf(s[u][r] - m_run[r]);
        l[r] += p;
#pragma unroll
        for (int i = 0; i < V; i++) o[r][i] = fmaf(p, vf[i], o[r][i]);
      }
    }
  }
  // Sum the partial (l, o) of the lane groups: inside the warp with shuffles, across warps through shared memory.
#pragma unroll
  for (int r = 0; r < REP; r++) {
#pragma unroll
    for (int off = LPK; off < 32; off <<= 1) {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], off);
#pragma unroll
      for (int i = 0; i < V; i++) o[r][i] += __shfl_xor_sync(0xffffffffu, o[r][i], off);
    }
    if (sub == 0) {
      if (gl == 0) sm_l[warp][r] = l[r];
#pragma unroll
      for (int i = 0; i < V; i++) sm_o[warp][r][gl * V + i] = o[r][i];
    }
  }
  __syncthreads();
  const long long tile = (long long)b * a.kv_heads + g;
  float* ws = a.workspace + (tile * a.splits + split) * (long long)REP * (HD + 2);
  for (int idx = threadIdx.x; idx < REP * HD; idx += WARPS * 32) {
    const int r = idx / HD, d = idx % HD;
    float oo = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; w++) {
      oo += sm_o[w][r][d];
      ll += sm_l[w][r];
    }
    if (a.splits == 1) {  // nothing to merge: this CTA saw every key
      out[b * a.q_batch_stride + (g * REP + r) * a.q_head_stride + d] = Elem<T>::store(ll > 0.f ? oo / ll : 0.f);
      continue;
    }
    ws[r * (HD + 2) + d] = oo;
    if (d == 0) {
      ws[r * (HD + 2) + HD] = m_run[r];
      ws[r * (HD + 2) + HD + 1] = ll;
    }
  }
  if (a.splits == 1) return;
  merge_splits<T, REP, HD, WARPS * 32>(a, tile, b, g, &sm_o[0][0][0], &is_last, out);
}

// ---------------------------------------------------------------------------------------------------------------
// Shared-memory staged variant for 16-bit caches and few (sequence, KV head) pairs: batch-1 decode.
//
// At batch 1 the whole cache of a step is a few megabytes and the kernel is a chain of latencies. The register-staged
// kernel above keeps every K/V row of its split in registers (about 54 K registers per CTA), which also keeps the CTAs
// of the following projection from becoming resident and requesting their weights while attention runs. Here the rows
// of a split (at most kStagedKeys) are brought into shared memory by bulk asynchronous copies, one 16-byte-aligned row
// slice per copy, all completing on one mbarrier; no register holds data in flight, the CTA needs about 10 K registers
// and 75 KiB, and one CTA of the next streaming contraction fits beside it on the SM.
//   phase 1  scores: a thread owns a key and REP / 2 query heads; K rows are read with 16-byte loads from rows padded
//            by 16 bytes (conflict-free), the query slices come as broadcasts from an f32 copy in shared memory
//   phase 2  softmax statistics: one warp per query head (max, exp, sum)
//   phase 3  context: a thread owns two adjacent output elements of one head and walks the keys
// Partial (max, sum, out) triples are merged across splits exactly as in the kernel above.
// With `early_kv` the rows below the token index (which no earlier kernel of the step writes) are requested before
// the kernel waits for its predecessor; only the row at the token index is requested after the wait.
constexpr int kStagedKeys = 128;
constexpr int kStagedThreads = 256;
constexpr unsigned kStagedSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t attn_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

template <int REP, int HD> struct StagedLayout {
  static constexpr int ROW = HD * 2 + 16;            // padded pitch of a K / V row in bytes
  static constexpr int QROW = HD + 4;                // padded pitch of a query row in floats
  static constexpr size_t k_off = 0;
  static constexpr size_t v_off = (size_t)kStagedKeys * ROW;
  static constexpr size_t q_off = 2 * (size_t)kStagedKeys * ROW;
  static constexpr size_t s_off = q_off + (size_t)REP * QROW * sizeof(float);
  static constexpr size_t s_floats = (size_t)REP * kStagedKeys > 64 * REP * 2 ? (size_t)REP * kStagedKeys : 64 * REP * 2;
  static constexpr size_t ml_off = s_off + s_floats * sizeof(float);
  static constexpr size_t bar_off = (ml_off + (size_t)REP * 2 * sizeof(float) + 15) / 16 * 16;
  static constexpr size_t bytes = bar_off + 16;
};

template <typename T, int REP, int HD>
__global__ void __launch_bounds__(kStagedThreads)
attn_decode_staged_kernel(DecodeArgs a, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                          const void* __restrict__ token, T* __restrict__ out) {
  static_assert(sizeof(T) == 2, "16-bit caches");
  using L = StagedLayout<REP, HD>;
  constexpr int ROW = L::ROW, QROW = L::QROW;
  constexpr int TPK = REP >= 2 ? 2 : 1;  // threads per key in the score phase
  constexpr int HPT = REP / TPK;         // query heads per thread
  extern __shared__ __align__(128) unsigned char smem_staged[];
  unsigned char* ks = smem_staged + L::k_off;
  unsigned char* vs = smem_staged + L::v_off;
  float* qs = reinterpret_cast<float*>(smem_staged + L::q_off);
  float* ss = reinterpret_cast<float*>(smem_staged + L::s_off);
  float* ml = reinterpret_cast<float*>(smem_staged + L::ml_off);
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem_staged + L::bar_off);
  int* is_last = reinterpret_cast<int*>(bar + 1);

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  prefetch_next_weights(a);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(attn_smem_u32(bar)), "r"(1));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (!a.early_kv) asm volatile("griddepcontrol.wait;" ::: "memory");
  long long limit = load_scalar(token, a.token_dtype);  // keys 0..limit are visible
  if (limit >= a.kv_len) limit = a.kv_len - 1;
  const long long count = limit + 1;
  const long long per_split = (count + a.splits - 1) / a.splits;
  const long long j_begin = (long long)split * per_split;
  const long long j_end = min(j_begin + per_split, count);
  const int n = (int)max(0ll, min(j_end - j_begin, (long long)kStagedKeys));
  if (tid == 0 && n > 0)
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(attn_smem_u32(bar)), "r"(2 * n * HD * 2) : "memory");
  __syncthreads();  // the barrier expects the bytes before any copy can complete on it
  const T* kb = k + b * a.kv_batch_stride + g * a.kv_head_stride;
  const T* vb = v + b * a.kv_batch_stride + g * a.kv_head_stride;
  auto copy_row = [&](int i) {
    const int row = i < n ? i : i - n;
    const T* src = (i < n ? kb : vb) + (j_begin + row) * a.kv_row_stride;
    unsigned char* dst = (i < n ? ks : vs) + (size_t)row * ROW;
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(attn_smem_u32(dst)),
                 "l"(src), "r"(HD * 2), "r"(attn_smem_u32(bar))
                 : "memory");
  };
  // Rows written by this step (the one at the token index) may only be read after the predecessor has finished.
  for (int i = tid; i < 2 * n; i += kStagedThreads) {
    const int row = i < n ? i : i - n;
    if (!a.early_kv || j_begin + row < limit) copy_row(i);
  }
  if (a.early_kv) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int i = tid; i < 2 * n; i += kStagedThreads) {
      const int row = i < n ? i : i - n;
      if (j_begin + row >= limit) copy_row(i);
    }
  }
  // Query slices of the heads that share this KV head, as f32.
  for (int idx = tid; idx < REP * HD; idx += kStagedThreads) {
    const int r = idx / HD, d = idx % HD;
    qs[r * QROW + d] = (float)q[b * a.q_batch_stride + (g * REP + r) * a.q_head_stride + d];
  }
  __syncthreads();
  if (n > 0) {
    bool arrived = false;
    for (unsigned spin = 0; spin < kStagedSpinLimit && !arrived; spin++) {
      unsigned ok;
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(ok)
          : "r"(attn_smem_u32(bar)), "r"(0)
          : "memory");
      arrived = ok != 0;
    }
    if (!arrived) {
      if (a.error_flag && lane == 0) atomicExch(a.error_flag, 3);
      return;
    }
  }
  // Phase 1: scores.
  {
    const int j = tid / TPK, hg = tid % TPK;
    if (j < n) {
      float acc[HPT];
#pragma unroll
      for (int h = 0; h < HPT; h++) acc[h] = 0.f;
      const unsigned char* krow = ks + (size_t)j * ROW;
#pragma unroll 4
      for (int c = 0; c < HD / 8; c++) {
        float kf[8];
        Elem<T>::unpack(*reinterpret_cast<const uint4*>(krow + c * 16), kf);
#pragma unroll
        for (int h = 0; h < HPT; h++) {
          const float4 q0 = *reinterpret_cast<const float4*>(qs + (hg * HPT + h) * QROW + c * 8);
          const float4 q1 = *reinterpret_cast<const float4*>(qs + (hg * HPT + h) * QROW + c * 8 + 4);
          acc[h] = fmaf(q0.x, kf[0], acc[h]); acc[h] = fmaf(q0.y, kf[1], acc[h]);
          acc[h] = fmaf(q0.z, kf[2], acc[h]); acc[h] = fmaf(q0.w, kf[3], acc[h]);
          acc[h] = fmaf(q1.x, kf[4], acc[h]); acc[h] = fmaf(q1.y, kf[5], acc[h]);
          acc[h] = fmaf(q1.z, kf[6], acc[h]); acc[h] = fmaf(q1.w, kf[7], acc[h]);
        }
      }
#pragma unroll
      for (int h = 0; h < HPT; h++) {
        float d = acc[h];
        if (a.round_scores) d = Elem<T>::round(d);
        ss[(hg * HPT + h) * kStagedKeys + j] = d * a.scale;
      }
    }
  }
  __syncthreads();
  // Phase 2: per head maximum, probabilities relative to it, and their sum.
  for (int r = warp; r < REP; r += kStagedThreads / 32) {
    float m = -INFINITY;
    for (int j = lane; j < n; j += 32) m = fmaxf(m, ss[r * kStagedKeys + j]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    float l = 0.f;
    for (int j = lane; j < n; j += 32) {
      const float p = __expf(ss[r * kStagedKeys + j] - m);
      ss[r * kStagedKeys + j] = p;
      l += p;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
    if (lane == 0) {
      ml[r * 2] = m;
      ml[r * 2 + 1] = l;
    }
  }
  __syncthreads();
  // Phase 3: context. A thread owns outputs (r, 2 * d2) and (r, 2 * d2 + 1).
  const long long tile = (long long)b * a.kv_heads + g;
  float* ws = a.workspace + (tile * a.splits + split) * (long long)REP * (HD + 2);
  for (int pi = tid; pi < REP * HD / 2; pi += kStagedThreads) {
    const int r = pi / (HD / 2), d2 = pi % (HD / 2);
    float o0 = 0.f, o1 = 0.f;
    const unsigned char* vcol = vs + d2 * 4;
    const float* pr = ss + r * kStagedKeys;
#pragma unroll 8
    for (int j = 0; j < n; j++) {
      const uint32_t raw = *reinterpret_cast<const uint32_t*>(vcol + (size_t)j * ROW);
      const T* pair = reinterpret_cast<const T*>(&raw);
      const float v0 = (float)pair[0], v1 = (float)pair[1];
      const float p = pr[j];
      o0 = fmaf(p, v0, o0);
      o1 = fmaf(p, v1, o1);
    }
    const float l = ml[r * 2 + 1];
    if (a.splits == 1) {
      T* dst = out + b * a.q_batch_stride + (g * REP + r) * a.q_head_stride + 2 * d2;
      dst[0] = Elem<T>::store(l > 0.f ? o0 / l : 0.f);
      dst[1] = Elem<T>::store(l > 0.f ? o1 / l : 0.f);
      continue;
    }
    ws[r * (HD + 2) + 2 * d2] = o0;
    ws[r * (HD + 2) + 2 * d2 + 1] = o1;
    if (d2 == 0) {
      ws[r * (HD + 2) + HD] = ml[r * 2];
      ws[r * (HD + 2) + HD + 1] = l;
    }
  }
  if (a.splits == 1) return;
  __syncthreads();  // the merge scratch overlaps the probabilities
  merge_splits<T, REP, HD, kStagedThreads>(a, tile, b, g, ss, is_last, out);
}

// ---------------------------------------------------------------------------------------------------------------
// Tensor-core variant for 16-bit caches with many query heads per KV head or many sequences: with eight heads per KV
// head the CUDA cores need ~4000 lane-instructions per K/V row pair and become the limit long before HBM does, while
// the same work is 32 warp-level MMAs per 16 keys.
//
// One CTA (4 warps) = one (sequence, KV head, key split). K and V rows stream through a ring of shared-memory stages
// of 64 keys (cp.async, 16 bytes per request, rows XOR-swizzled in 16-byte units so that ldmatrix reads are
// conflict-free); rows past the end of the split are zero-filled. Each warp owns 16 keys of a stage:
//   S[16 x 16 keys] = Q[16 x HD] . K^T      mma.m16n8k16, Q fragments held in registers (rows >= REP are zero),
//                                           K fragments by ldmatrix
//   online softmax on the accumulator fragments (row statistics are shared by the four lanes of a quad)
//   O[16 x HD]     += P[16 x 16 keys] . V   the S accumulators, rounded to the element type, are the A fragments;
//                                           V fragments by ldmatrix.trans
// After the last stage the four warps' (max, sum, out) are merged through shared memory and the split is published
// like in the CUDA-core kernel.
constexpr int kMmaWarps = 4;
constexpr int kMmaStageKeys = 16 * kMmaWarps;

template <typename T> struct MmaOps;
template <> struct MmaOps<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ unsigned pack(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
  }
};
template <> struct MmaOps<__half> {
  static __device__ __forceinline__ void mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
  static __device__ __forceinline__ unsigned pack(float lo, float hi) {
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const unsigned*>(&v);
  }
};

__device__ __forceinline__ void ldmatrix_x4(unsigned* r, unsigned smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned* r, unsigned smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr));
}
// STAGES = 3: two CTAs per SM, two stages in flight each. (A two-stage ring with three CTAs per SM and a third more
// splits was measured on thirty-two (sequence, KV head) pairs of 4K keys: no faster.)
template <typename T, int REP, int HD, int STAGES>
__global__ void __launch_bounds__(kMmaWarps * 32, STAGES == 2 ? 3 : 2)
attn_decode_mma_kernel(DecodeArgs a, const T* __restrict__ q, const __grid_constant__ CUtensorMap kmap,
                       const __grid_constant__ CUtensorMap vmap, const void* __restrict__ token, T* __restrict__ out) {
  static_assert(sizeof(T) == 2 && (HD == 64 || HD == 128) && REP <= 16, "16-bit elements, head_dim 64 or 128");
  constexpr int THREADS = kMmaWarps * 32;
  constexpr int HALVES = HD / 64;                     // 128-byte column blocks per row
  constexpr int TILE_BYTES = kMmaStageKeys * HD * 2;  // one of K or V for one stage
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  // The swizzle of a tiled copy follows the absolute shared-memory address: tiles start on 1024-byte boundaries.
  extern __shared__ unsigned char smem_attn_raw[];
  unsigned char* smem_attn = smem_attn_raw + ((1024u - (attn_smem_u32(smem_attn_raw) & 1023u)) & 1023u);
  __shared__ int is_last;
  __shared__ int gave_up;
  __shared__ __align__(8) uint64_t full[STAGES];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int st = 0; st < STAGES; st++)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(attn_smem_u32(&full[st])), "r"(1));
    gave_up = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // With `early_kv` the only row an earlier kernel of the step writes is the one at the token index (and the token is a
  // parameter): stages that do not hold that row are requested before the wait for the predecessor.
  if (!a.early_kv) asm volatile("griddepcontrol.wait;" ::: "memory");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  long long limit = load_scalar(token, a.token_dtype);  // keys 0..limit are visible
  if (limit >= a.kv_len) limit = a.kv_len - 1;
  const long long count = limit + 1;
  const long long per_split = (count + a.splits - 1) / a.splits;
  const long long j_begin = (long long)split * per_split;
  const long long j_end = min(j_begin + per_split, count);
  const int stages_total = j_end > j_begin ? (int)((j_end - j_begin + kMmaStageKeys - 1) / kMmaStageKeys) : 0;

  const unsigned smem_base = (unsigned)__cvta_generic_to_shared(smem_attn);

  // Row `row` (0..63) of a stage tile, 16-byte chunk `c` of the row: column block c / 8 holds [64 rows][128 bytes],
  // chunk position XORed with the row's low three bits - the layout a 128-byte swizzled tensor copy writes.
  auto tile_offset = [](int row, int c) { return (unsigned)((c >> 3) * (kMmaStageKeys * 128) + row * 128 + (((c & 7) ^ (row & 7)) << 4)); };
  // A stage is 64 K rows and 64 V rows: one tiled copy per 128-byte column block of each, issued by one thread and
  // completing on the stage's barrier. The maps are [head_dim][keys][KV heads][sequences]; rows past the end of the
  // cache arrive as zeros.
  auto issue_stage = [&](int st) {
    if (threadIdx.x != 0) return;
    const int slot = st % STAGES;
    const unsigned bar = attn_smem_u32(&full[slot]);
    const unsigned dst = smem_base + (unsigned)slot * STAGE_BYTES;
    const int j0 = (int)(j_begin + (long long)st * kMmaStageKeys);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(STAGE_BYTES) : "memory");
#pragma unroll
    for (int c = 0; c < HALVES; c++) {
      asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
                       dst + c * (kMmaStageKeys * 128)),
                   "l"(&kmap), "r"(c * 64), "r"(j0), "r"(g), "r"(b), "r"(bar)
                   : "memory");
      asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
                       dst + TILE_BYTES + c * (kMmaStageKeys * 128)),
                   "l"(&vmap), "r"(c * 64), "r"(j0), "r"(g), "r"(b), "r"(bar)
                   : "memory");
    }
  };
  {
    bool issued[STAGES - 1];
#pragma unroll
    for (int st = 0; st < STAGES - 1; st++) {
      const long long j0 = j_begin + (long long)st * kMmaStageKeys;
      const bool holds_token_row = j0 <= limit && limit < j0 + kMmaStageKeys;
      issued[st] = st < stages_total && !(a.early_kv && holds_token_row);
      if (issued[st]) issue_stage(st);
    }
    if (a.early_kv) {
      asm volatile("griddepcontrol.wait;" ::: "memory");
#pragma unroll
      for (int st = 0; st < STAGES - 1; st++)
        if (st < stages_total && !issued[st]) issue_stage(st);
    }
  }
  unsigned long long deadline;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(deadline));
  deadline += a.timeout_ns;

  // Q fragments: row r = lane / 4 (and r + 8), columns ks * 16 + (lane % 4) * 2 (+ 8).
  unsigned qa[HD / 16][4];
  {
    const int r0 = lane >> 2, c0 = (lane & 3) * 2;
    const T* qrow0 = q + b * a.q_batch_stride + (g * REP + r0) * a.q_head_stride;
    const T* qrow1 = q + b * a.q_batch_stride + (g * REP + r0 + 8) * a.q_head_stride;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) {
      qa[ks][0] = r0 < REP ? __ldg(reinterpret_cast<const unsigned*>(qrow0 + ks * 16 + c0)) : 0u;
      qa[ks][1] = r0 + 8 < REP ? __ldg(reinterpret_cast<const unsigned*>(qrow1 + ks * 16 + c0)) : 0u;
      qa[ks][2] = r0 < REP ? __ldg(reinterpret_cast<const unsigned*>(qrow0 + ks * 16 + c0 + 8)) : 0u;
      qa[ks][3] = r0 + 8 < REP ? __ldg(reinterpret_cast<const unsigned*>(qrow1 + ks * 16 + c0 + 8)) : 0u;
    }
  }
  float m_run[2] = {-INFINITY, -INFINITY}, l_part[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int nt = 0; nt < HD / 8; nt++)
#pragma unroll
    for (int e = 0; e < 4; e++) o[nt][e] = 0.f;

  bool arrived = true;
  for (int st = 0; st < stages_total; st++) {
    {  // every row of stage st has landed (bounded by time: a copy that never completes must not hang the GPU)
      const unsigned bar = attn_smem_u32(&full[st % STAGES]), parity = (unsigned)(st / STAGES) & 1u;
      for (unsigned spin = 0;; spin++) {
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) break;
        if ((spin & 255) == 255) {
          unsigned long long now;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
          if (now > deadline || *reinterpret_cast<volatile int*>(&gave_up)) {
            gave_up = 1;
            arrived = false;
            break;
          }
        }
      }
    }
    // V rows past the end of the split belong to other splits or to nobody: their probabilities are zero, but
    // 0 * whatever is stored there need not be, so they are cleared (K rows need nothing: their scores are replaced).
    if (arrived && j_begin + (long long)(st + 1) * kMmaStageKeys > j_end) {
      const int first = (int)(j_end - (j_begin + (long long)st * kMmaStageKeys));
      unsigned char* vt = smem_attn + (size_t)(st % STAGES) * STAGE_BYTES + TILE_BYTES;
      for (int idx = first * (HD / 8) + threadIdx.x; idx < kMmaStageKeys * (HD / 8); idx += THREADS) {
        const int row = idx / (HD / 8), c = idx % (HD / 8);
        *reinterpret_cast<uint4*>(vt + tile_offset(row, c)) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    // Everyone is done with stage st - 1 (its slot is refilled below); a thread that gave up tells the others here.
    arrived = __syncthreads_and(arrived ? 1 : 0) != 0;
    if (!arrived) break;
    if (st + STAGES - 1 < stages_total) issue_stage(st + STAGES - 1);

    const unsigned ktile = smem_base + (unsigned)(st % STAGES) * STAGE_BYTES;
    const unsigned vtile = ktile + TILE_BYTES;
    const int row0 = warp * 16;  // this warp's keys inside the stage
    // S = Q . K^T for 16 keys: two accumulator tiles of 8 keys.
    float sc[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
#pragma unroll
      for (int e = 0; e < 4; e++) sc[nt][e] = 0.f;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) {
      // Matrices: (keys 0-7, hd 0-7), (keys 0-7, hd 8-15), (keys 8-15, hd 0-7), (keys 8-15, hd 8-15) of this k step.
      unsigned bk[4];
      const int key = row0 + ((lane >> 4) << 3) + (lane & 7);
      const int chunk = ks * 2 + ((lane >> 3) & 1);
      ldmatrix_x4(bk, ktile + tile_offset(key, chunk));
      MmaOps<T>::mma(sc[0], qa[ks], bk[0], bk[1]);
      MmaOps<T>::mma(sc[1], qa[ks], bk[2], bk[3]);
    }
    // Scale, mask and online softmax. Accumulator element e of tile nt: row (lane / 4) + 8 * (e / 2),
    // key row0 + nt * 8 + (lane % 4) * 2 + (e % 2).
    const long long key_base = j_begin + (long long)st * kMmaStageKeys + row0 + (lane & 3) * 2;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; nt++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        float d = sc[nt][e];
        if (a.round_scores) d = Elem<T>::round(d);
        const bool ok = key_base + nt * 8 + (e & 1) < j_end;
        d = ok ? d * a.scale : -INFINITY;
        sc[nt][e] = d;
        mx[e >> 1] = fmaxf(mx[e >> 1], d);
      }
    unsigned pa[4];
#pragma unroll
    for (int h = 0; h < 2; h++) {  // row lane / 4 (h = 0) and row lane / 4 + 8 (h = 1)
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      const float corr = (m_run[h] == -INFINITY || m_new == m_run[h]) ? (m_run[h] == -INFINITY ? 0.f : 1.f) : __expf(m_run[h] - m_new);
      if (corr != 1.f) {
        l_part[h] *= corr;
#pragma unroll
        for (int nt = 0; nt < HD / 8; nt++) {
          o[nt][2 * h] *= corr;
          o[nt][2 * h + 1] *= corr;
        }
      }
      m_run[h] = m_new;
      float p[4];
#pragma unroll
      for (int nt = 0; nt < 2; nt++)
#pragma unroll
        for (int e = 0; e < 2; e++) {
          const float sv = sc[nt][2 * h + e];
          p[nt * 2 + e] = sv == -INFINITY ? 0.f : __expf(sv - m_new);
        }
      // The probabilities enter the second contraction in the element type; the row sum uses the same rounded values.
      pa[h] = MmaOps<T>::pack(p[0], p[1]);       // keys 0-7 block
      pa[2 + h] = MmaOps<T>::pack(p[2], p[3]);   // keys 8-15 block
      l_part[h] += Elem<T>::round(p[0]) + Elem<T>::round(p[1]) + Elem<T>::round(p[2]) + Elem<T>::round(p[3]);
    }
    // O += P . V: B fragments from V[key][hd] by transposing loads, two 8-column tiles per ldmatrix.
#pragma unroll
    for (int np = 0; np < HD / 16; np++) {
      // Matrices: (keys 0-7, hd tile 2np), (keys 8-15, hd tile 2np), (keys 0-7, hd tile 2np+1), (keys 8-15, hd tile 2np+1).
      unsigned bv[4];
      const int key = row0 + (((lane >> 3) & 1) << 3) + (lane & 7);
      const int chunk = np * 2 + (lane >> 4);
      ldmatrix_x4_trans(bv, vtile + tile_offset(key, chunk));
      MmaOps<T>::mma(o[2 * np], pa, bv[0], bv[1]);
      MmaOps<T>::mma(o[2 * np + 1], pa, bv[2], bv[3]);
    }
  }
  if (!arrived) {
    // Copies of later stages may still be in flight towards this CTA's shared memory: give them the same bounded time
    // before leaving (the barriers they complete on must outlive them), then report and go.
    for (int st = 0; st < stages_total; st++) {
      const unsigned bar = attn_smem_u32(&full[st % STAGES]), parity = (unsigned)(st / STAGES) & 1u;
      for (unsigned spin = 0; spin < (1u << 16); spin++) {
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) break;
      }
    }
    if (threadIdx.x == 0 && a.error_flag) atomicExch(a.error_flag, 6);
    return;
  }
  __syncthreads();  // the stage memory is free: reuse it for the merge of the four warps

  // Row sums over the quad, then per-warp (max, sum, out) to shared memory.
#pragma unroll
  for (int h = 0; h < 2; h++) {
    l_part[h] += __shfl_xor_sync(0xffffffffu, l_part[h], 1);
    l_part[h] += __shfl_xor_sync(0xffffffffu, l_part[h], 2);
  }
  float* sm_m = reinterpret_cast<float*>(smem_attn);                 // [warps][16]
  float* sm_l = sm_m + kMmaWarps * 16;                               // [warps][16]
  float* sm_o = sm_l + kMmaWarps * 16;                               // [warps][REP][HD]
  {
    const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const int r = r0 + 8 * h;
      if (r < REP) {
        if ((lane & 3) == 0) {
          sm_m[warp * 16 + r] = m_run[h];
          sm_l[warp * 16 + r] = l_part[h];
        }
#pragma unroll
        for (int nt = 0; nt < HD / 8; nt++) {
          sm_o[(warp * REP + r) * HD + nt * 8 + c0] = o[nt][2 * h];
          sm_o[(warp * REP + r) * HD + nt * 8 + c0 + 1] = o[nt][2 * h + 1];
        }
      }
    }
  }
  __syncthreads();
  const long long tile = (long long)b * a.kv_heads + g;
  float* ws = a.workspace + (tile * a.splits + split) * (long long)REP * (HD + 2);
  for (int idx = threadIdx.x; idx < REP * HD; idx += THREADS) {
    const int r = idx / HD, d = idx % HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kMmaWarps; w++) mm = fmaxf(mm, sm_m[w * 16 + r]);
    float oo = 0.f, ll = 0.f;
#pragma unroll
    for (int w = 0; w < kMmaWarps; w++) {
      const float mw = sm_m[w * 16 + r];
      const float wgt = mw == -INFINITY ? 0.f : __expf(mw - mm);
      oo = fmaf(sm_o[(w * REP + r) * HD + d], wgt, oo);
      ll = fmaf(sm_l[w * 16 + r], wgt, ll);
    }
    if (a.splits == 1) {
      out[b * a.q_batch_stride + (g * REP + r) * a.q_head_stride + d] = Elem<T>::store(ll > 0.f ? oo / ll : 0.f);
      continue;
    }
    ws[r * (HD + 2) + d] = oo;
    if (d == 0) {
      ws[r * (HD + 2) + HD] = mm;
      ws[r * (HD + 2) + HD + 1] = ll;
    }
  }
  if (a.splits == 1) return;
  __syncthreads();  // the merge scratch below overlaps sm_m / sm_l / sm_o
  merge_splits<T, REP, HD, THREADS>(a, tile, b, g, reinterpret_cast<float*>(smem_attn), &is_last, out);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A cache as the 4-d tensor [head_dim][keys][KV heads][sequences] (strides in elements come with the launch); the box
// is 64 elements x kMmaStageKeys keys of one head of one sequence.
bool encode_kv_map(CUtensorMap* map, const void* base, bool f16, const DecodeArgs& a, int head_dim) {
  static const EncodeTiledFn enc = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
    return (EncodeTiledFn)p;
  }();
  if (!enc) return false;
  // A dimension of extent 1 may come with any stride (0 included); the encoder wants multiples of 16 bytes that
  // are not smaller than the dimension below, so give those dimensions the stride of the whole cache.
  const cuuint64_t gdim[4] = {(cuuint64_t)head_dim, (cuuint64_t)a.kv_len, (cuuint64_t)a.kv_heads, (cuuint64_t)a.batch};
  cuuint64_t gstride[3] = {(cuuint64_t)a.kv_row_stride * 2, (cuuint64_t)a.kv_head_stride * 2, (cuuint64_t)a.kv_batch_stride * 2};
  for (int d = 0; d < 3; d++)
    if (gdim[d + 1] == 1 && gstride[d] == 0) gstride[d] = (cuuint64_t)head_dim * 2;
  const cuuint32_t box[4] = {64, (cuuint32_t)kMmaStageKeys, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), gdim, gstride,
             box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T, int REP, int HD, int STAGES>
int launch_decode_mma_stages(const DecodeArgs& args, dim3 grid, const void* q, const void* k, const void* v, const void* token, void* out,
                      bool pdl, cudaStream_t stream) {
  constexpr size_t stage_smem = (size_t)STAGES * 2 * kMmaStageKeys * HD * 2;
  constexpr size_t merge_smem = (size_t)(2 * kMmaWarps * 16 + kMmaWarps * REP * HD) * sizeof(float);
  constexpr size_t scratch_smem = (size_t)64 * REP * 2 * sizeof(float);
  constexpr size_t smem = 1024 + (stage_smem > merge_smem ? (stage_smem > scratch_smem ? stage_smem : scratch_smem)
                                                          : (merge_smem > scratch_smem ? merge_smem : scratch_smem));
  if (!raise_smem_limit((const void*)attn_decode_mma_kernel<T, REP, HD, STAGES>, (int)smem)) return 0;
  // The splits merge cooperatively (every CTA waits for its tile's other splits) only when the whole grid is resident.
  DecodeArgs a = args;
  int device = 0, sms = 0, per_sm = 0;
  if (coop_merge_allowed() && a.splits > 1 && cudaGetDevice(&device) == cudaSuccess &&
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) == cudaSuccess &&
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_decode_mma_kernel<T, REP, HD, STAGES>, kMmaWarps * 32, smem) == cudaSuccess)
    a.coop_merge = (long long)grid.x * grid.y * grid.z <= (long long)per_sm * sms ? 1 : 0;
  // K and V as [head_dim][keys][KV heads][sequences] for tiled copies of 64 keys x 128 bytes, 128-byte swizzled.
  CUtensorMap kmap, vmap;
  if (!encode_kv_map(&kmap, k, sizeof(T) == 2 && std::is_same<T, __half>::value, a, HD) ||
      !encode_kv_map(&vmap, v, sizeof(T) == 2 && std::is_same<T, __half>::value, a, HD))
    return 0;
  return launch_kernel(attn_decode_mma_kernel<T, REP, HD, STAGES>, grid, dim3(kMmaWarps * 32), smem, stream, pdl, a, (const T*)q, kmap,
                       vmap, token, (T*)out) == cudaSuccess
             ? 1
             : 0;
}

template <typename T, int REP, int HD>
int launch_decode_mma(const DecodeArgs& args, dim3 grid, const void* q, const void* k, const void* v, const void* token, void* out,
                      bool pdl, cudaStream_t stream) {
  return launch_decode_mma_stages<T, REP, HD, 3>(args, grid, q, k, v, token, out, pdl, stream);
}

template <typename T>
int dispatch_decode_mma(int rep, int hd, const DecodeArgs& a, dim3 grid, const void* q, const void* k, const void* v,
                        const void* token, void* out, bool pdl, cudaStream_t stream) {
#define CASE(R, H) \
  if (rep == R && hd == H) return launch_decode_mma<T, R, H>(a, grid, q, k, v, token, out, pdl, stream);
  CASE(4, 128) CASE(8, 128) CASE(4, 64) CASE(8, 64)
#undef CASE
  return 0;
}

template <typename T, int REP, int HD>
int launch_decode_staged(const DecodeArgs& a, dim3 grid, const void* q, const void* k, const void* v, const void* token, void* out,
                         bool pdl, cudaStream_t stream) {
  constexpr size_t smem = StagedLayout<REP, HD>::bytes;
  if (!raise_smem_limit((const void*)attn_decode_staged_kernel<T, REP, HD>, (int)smem)) return 0;
  return launch_kernel(attn_decode_staged_kernel<T, REP, HD>, grid, dim3(kStagedThreads), smem, stream, pdl, a, (const T*)q,
                       (const T*)k, (const T*)v, token, (T*)out) == cudaSuccess
             ? 1
             : 0;
}

template <typename T>
int dispatch_decode_staged(int rep, int hd, const DecodeArgs& a, dim3 grid, const void* q, const void* k, const void* v,
                           const void* token, void* out, bool pdl, cudaStream_t stream) {
#define CASE(R, H) \
  if (rep == R && hd == H) return launch_decode_staged<T, R, H>(a, grid, q, k, v, token, out, pdl, stream);
  CASE(1, 128) CASE(2, 128) CASE(4, 128) CASE(8, 128) CASE(1, 64) CASE(2, 64) CASE(4, 64) CASE(8, 64)
#undef CASE
  return 0;
}

// Shape of a CTA: eight warps; eight keys per lane group and chunk while the scores of all heads still fit in
// registers, four beyond. A chunk is WARPS * (32 / lanes per key) * KPG keys. Sixteen warps with four keys each
// (same chunk, half the instruction stream per thread) measured slower at batch 1: 0.77 instead of 0.68 ms for the 32
// launches of an 8B-shape step (the kernel then spills at 128 registers).
template <int REP> struct KeysPerGroup { static constexpr int value = REP <= 4 ? 8 : 4; };
template <int REP> struct WarpsPerCta { static constexpr int value = 8; };

template <typename T, int REP, int HD>
int launch_decode(const DecodeArgs& a, dim3 grid, const void* q, const void* k, const void* v, const void* token, void* out, bool pdl,
                  cudaStream_t stream) {
  return launch_kernel(attn_decode_kernel<T, REP, HD, KeysPerGroup<REP>::value, WarpsPerCta<REP>::value>, grid,
                       dim3(WarpsPerCta<REP>::value * 32), 0, stream, pdl, a, (const T*)q, (const T*)k,
                       (const T*)v, token, (T*)out) == cudaSuccess
             ? 1
             : 0;
}

template <typename T>
int dispatch_decode(int rep, int hd, const DecodeArgs& a, dim3 grid, const void* q, const void* k, const void* v, const void* token,
                    void* out, bool pdl, cudaStream_t stream) {
#define CASE(R, H) \
  if (rep == R && hd == H) return launch_decode<T, R, H>(a, grid, q, k, v, token, out, pdl, stream);
  CASE(1, 128) CASE(2, 128) CASE(4, 128) CASE(8, 128) CASE(1, 64) CASE(2, 64) CASE(4, 64) CASE(8, 64)
#undef CASE
  return 0;
}


// ---- Causal self-attention over whole sequences (prefill) ---------------------------------------------------------
//
// out[b, g, s, r, :] = softmax_j( q[b, g, s, r, :] . k[b, j, g, :] * scale  for j <= s ) . v[b, j, g, :]
//
// q and out are [batch, kv_heads, seq, rep, head_dim] (the operand and result layout of the recognised
// dot_general -> masked softmax -> dot_general form), so the `seq * rep` query rows that share one KV head are one
// contiguous row-major matrix; row `x` belongs to position x / rep. One CTA (4 warps) owns 64 consecutive rows and
// walks the keys 0..(its last position) in stages of 64 through the same ring of tiled tensor-map copies and swizzled
// layout as the decode kernel above; every warp owns 16 rows and multiplies them with all 64 keys of a stage:
//   S[16 x 64] = Q[16 x HD] . K^T (mma.m16n8k16, Q fragments in registers), mask key <= position, online softmax on
//   the fragments, O[16 x HD] += P[16 x 64] . V with the rounded probabilities as A fragments.
// Scores and probabilities never leave the SM (the explicit form writes and re-reads batch*heads*seq*seq elements
// twice per layer). Row tiles are scheduled longest first (the last rows see the most keys), and a warp skips the
// stages that lie wholly above its rows' diagonal.
struct PrefillArgs {
  long long seq = 0, rows = 0;  // rows = seq * rep per (sequence, KV head)
  int rep = 1, kv_heads = 1;
  long long kv_batch_stride = 0, kv_row_stride = 0, kv_head_stride = 0;
  float scale = 1.f;
  int* error_flag = nullptr;
};
constexpr int kPrefillRows = 16 * kMmaWarps;
constexpr int kPrefillStages = 2;  // 64 KiB per CTA at head_dim 128: three CTAs (twelve warps) per SM

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T, int HD>
__global__ void __launch_bounds__(kMmaWarps * 32, 3)
attn_prefill_mma_kernel(PrefillArgs a, const T* __restrict__ q, const __grid_constant__ CUtensorMap kmap,
                        const __grid_constant__ CUtensorMap vmap, T* __restrict__ out) {
  static_assert(sizeof(T) == 2 && (HD == 64 || HD == 128), "16-bit elements, head_dim 64 or 128");
  constexpr int HALVES = HD / 64;
  constexpr int TILE_BYTES = kMmaStageKeys * HD * 2;
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  // The swizzle of a tiled copy follows the absolute shared-memory address: tiles start on 1024-byte boundaries.
  extern __shared__ unsigned char smem_prefill_raw[];
  unsigned char* smem_attn = smem_prefill_raw + ((1024u - (attn_smem_u32(smem_prefill_raw) & 1023u)) & 1023u);
  __shared__ int gave_up;
  __shared__ __align__(8) uint64_t full[kPrefillStages];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int st = 0; st < kPrefillStages; st++)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(attn_smem_u32(&full[st])), "r"(1));
    gave_up = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  asm volatile("griddepcontrol.wait;" ::: "memory");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.y, b = blockIdx.z;
  const long long tile_row0 = (long long)(gridDim.x - 1 - blockIdx.x) * kPrefillRows;  // longest tiles first
  const long long last_row = min(tile_row0 + kPrefillRows, a.rows) - 1;
  const int j_end = (int)(last_row / a.rep) + 1;  // keys 0 .. last position of the tile
  const int stages_total = (j_end + kMmaStageKeys - 1) / kMmaStageKeys;

  const long long bg = ((long long)b * a.kv_heads + g) * a.rows;
  const unsigned smem_base = (unsigned)__cvta_generic_to_shared(smem_attn);
  auto tile_offset = [](int row, int c) { return (unsigned)((c >> 3) * (kMmaStageKeys * 128) + row * 128 + (((c & 7) ^ (row & 7)) << 4)); };
  // A stage is 64 K rows and 64 V rows, brought by one tiled copy per 128-byte column block of each (the decode
  // kernel's maps and layout); one thread issues them. Keys past the tile's last position are other positions' rows
  // (masked: their probabilities are zero and their values finite), keys past the sequence arrive as zeros.
  auto issue_stage = [&](int st) {
    if (threadIdx.x != 0) return;
    const int slot = st % kPrefillStages;
    const unsigned bar = attn_smem_u32(&full[slot]);
    const unsigned dst = smem_base + (unsigned)slot * STAGE_BYTES;
    const int j0 = st * kMmaStageKeys;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(STAGE_BYTES) : "memory");
#pragma unroll
    for (int c = 0; c < HALVES; c++) {
      asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
                       dst + c * (kMmaStageKeys * 128)),
                   "l"(&kmap), "r"(c * 64), "r"(j0), "r"(g), "r"(b), "r"(bar)
                   : "memory");
      asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
                       dst + TILE_BYTES + c * (kMmaStageKeys * 128)),
                   "l"(&vmap), "r"(c * 64), "r"(j0), "r"(g), "r"(b), "r"(bar)
                   : "memory");
    }
  };
  for (int st = 0; st < kPrefillStages - 1; st++)
    if (st < stages_total) issue_stage(st);
  unsigned long long deadline;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(deadline));
  deadline += 2000000000ull;

  // This thread's two rows (accumulator rows lane / 4 and lane / 4 + 8 of the warp's 16) and their positions;
  // rows past the matrix end get position -1: every key is masked and nothing is stored.
  const long long row_lo = tile_row0 + warp * 16 + (lane >> 2);
  const long long rows2[2] = {row_lo, row_lo + 8};
  int pos[2];
#pragma unroll
  for (int h = 0; h < 2; h++) pos[h] = rows2[h] < a.rows ? (int)(rows2[h] / a.rep) : -1;
  const int warp_first_pos = (int)((tile_row0 + warp * 16) / a.rep);
  const int warp_last_pos = (int)(min(tile_row0 + warp * 16 + 15, a.rows - 1) / a.rep);

  unsigned qa[HD / 16][4];
  {
    const int c0 = (lane & 3) * 2;
    const T* qrow0 = q + (bg + rows2[0]) * HD;
    const T* qrow1 = q + (bg + rows2[1]) * HD;
    const bool in0 = rows2[0] < a.rows, in1 = rows2[1] < a.rows;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ks++) {
      qa[ks][0] = in0 ? __ldg(reinterpret_cast<const unsigned*>(qrow0 + ks * 16 + c0)) : 0u;
      qa[ks][1] = in1 ? __ldg(reinterpret_cast<const unsigned*>(qrow1 + ks * 16 + c0)) : 0u;
      qa[ks][2] = in0 ? __ldg(reinterpret_cast<const unsigned*>(qrow0 + ks * 16 + c0 + 8)) : 0u;
      qa[ks][3] = in1 ? __ldg(reinterpret_cast<const unsigned*>(qrow1 + ks * 16 + c0 + 8)) : 0u;
    }
  }
  // Scores are kept in log2 units (score * scale * log2 e), so a probability is one ex2 of a difference. The row
  // sums are one more accumulator tile: P times a matrix of ones, in the tensor pipe instead of 32 adds per thread.
  const float c_log2 = a.scale * 1.4426950408889634f;
  const unsigned ones = MmaOps<T>::pack(1.f, 1.f);
  float m_run[2] = {-INFINITY, -INFINITY};
  float lacc[4] = {0.f, 0.f, 0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int nt = 0; nt < HD / 8; nt++)
#pragma unroll
    for (int e = 0; e < 4; e++) o[nt][e] = 0.f;

  bool arrived = true;
  for (int st = 0; st < stages_total; st++) {
    {  // stage st has landed (bounded by time)
      const unsigned bar = attn_smem_u32(&full[st % kPrefillStages]), parity = (unsigned)(st / kPrefillStages) & 1u;
      for (unsigned spin = 0;; spin++) {
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) break;
        if ((spin & 255) == 255) {
          unsigned long long now;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
          if (now > deadline || *reinterpret_cast<volatile int*>(&gave_up)) {
            gave_up = 1;
            arrived = false;
            break;
          }
        }
      }
    }
    // Everyone is done with stage st - 1 (its slot is refilled below); a thread that gave up tells the others here.
    arrived = __syncthreads_and(arrived ? 1 : 0) != 0;
    if (!arrived) break;
    if (st + kPrefillStages - 1 < stages_total) issue_stage(st + kPrefillStages - 1);
    const int key0 = st * kMmaStageKeys;
    if (key0 > warp_last_pos) continue;  // wholly above this warp's diagonal

    const unsigned ktile = smem_base + (unsigned)(st % kPrefillStages) * STAGE_BYTES;
    const unsigned vtile = ktile + TILE_BYTES;
    // S = Q . K^T for 64 keys: eight accumulator tiles of 8 keys.
    float sc[kMmaStageKeys / 8][4];
#pragma unroll
    for (int nt = 0; nt < kMmaStageKeys / 8; nt++)
#pragma unroll
      for (int e = 0; e < 4; e++) sc[nt][e] = 0.f;
#pragma unroll
    for (int kb16 = 0; kb16 < kMmaStageKeys / 16; kb16++) {
#pragma unroll
      for (int ks = 0; ks < HD / 16; ks++) {
        unsigned bk[4];
        const int key = kb16 * 16 + ((lane >> 4) << 3) + (lane & 7);
        const int chunk = ks * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(bk, ktile + tile_offset(key, chunk));
        MmaOps<T>::mma(sc[2 * kb16], qa[ks], bk[0], bk[1]);
        MmaOps<T>::mma(sc[2 * kb16 + 1], qa[ks], bk[2], bk[3]);
      }
    }
    // Accumulator element e of tile nt: row h = e / 2, key key0 + nt * 8 + (lane % 4) * 2 + (e % 2). The explicit
    // form rounds q.k to the element type before it scales; only stages that touch the diagonal need the mask.
    const bool diagonal = key0 + kMmaStageKeys - 1 > warp_first_pos;
    const int key_base = key0 + (lane & 3) * 2;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < kMmaStageKeys / 8; nt++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        float d = Elem<T>::round(sc[nt][e]) * c_log2;
        if (diagonal && key_base + nt * 8 + (e & 1) > pos[e >> 1]) d = -INFINITY;
        sc[nt][e] = d;
        mx[e >> 1] = fmaxf(mx[e >> 1], d);
      }
    unsigned pa[kMmaStageKeys / 16][4];
#pragma unroll
    for (int h = 0; h < 2; h++) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      // Rows with no visible key yet (only rows past the matrix end) keep everything at zero.
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float corr = ex2_approx(m_run[h] - m_use);
      if (m_new != m_run[h]) {
        lacc[2 * h] *= corr;
        lacc[2 * h + 1] *= corr;
#pragma unroll
        for (int nt = 0; nt < HD / 8; nt++) {
          o[nt][2 * h] *= corr;
          o[nt][2 * h + 1] *= corr;
        }
      }
      m_run[h] = m_new;
#pragma unroll
      for (int kb16 = 0; kb16 < kMmaStageKeys / 16; kb16++) {
        // The probabilities enter both products (values and row sum) rounded to the element type.
        pa[kb16][h] = MmaOps<T>::pack(ex2_approx(sc[2 * kb16][2 * h] - m_use), ex2_approx(sc[2 * kb16][2 * h + 1] - m_use));
        pa[kb16][2 + h] = MmaOps<T>::pack(ex2_approx(sc[2 * kb16 + 1][2 * h] - m_use), ex2_approx(sc[2 * kb16 + 1][2 * h + 1] - m_use));
      }
    }
    // O += P . V and l += P . 1
#pragma unroll
    for (int kb16 = 0; kb16 < kMmaStageKeys / 16; kb16++) {
      MmaOps<T>::mma(lacc, pa[kb16], ones, ones);
#pragma unroll
      for (int np = 0; np < HD / 16; np++) {
        unsigned bv[4];
        const int key = kb16 * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
        const int chunk = np * 2 + (lane >> 4);
        ldmatrix_x4_trans(bv, vtile + tile_offset(key, chunk));
        MmaOps<T>::mma(o[2 * np], pa[kb16], bv[0], bv[1]);
        MmaOps<T>::mma(o[2 * np + 1], pa[kb16], bv[2], bv[3]);
      }
    }
  }
  if (!arrived) {
    // Copies of the next stage may still be in flight towards this CTA's shared memory: give them a bounded time
    // before leaving, then report (nothing is stored).
    for (int st = 0; st < stages_total; st++) {
      const unsigned bar = attn_smem_u32(&full[st % kPrefillStages]), parity = (unsigned)(st / kPrefillStages) & 1u;
      for (unsigned spin = 0; spin < (1u << 16); spin++) {
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) break;
      }
    }
    if (threadIdx.x == 0 && a.error_flag) atomicExch(a.error_flag, 8);
    return;
  }

  const int c0 = (lane & 3) * 2;
#pragma unroll
  for (int h = 0; h < 2; h++) {
    if (rows2[h] >= a.rows) continue;
    const float l = lacc[2 * h];
    const float inv = l > 0.f ? 1.f / l : 0.f;
    T* orow = out + (bg + rows2[h]) * HD + c0;
#pragma unroll
    for (int nt = 0; nt < HD / 8; nt++)
      *reinterpret_cast<unsigned*>(orow + nt * 8) = MmaOps<T>::pack(o[nt][2 * h] * inv, o[nt][2 * h + 1] * inv);
  }
}

template <typename T, int HD>
int launch_prefill_mma(const PrefillArgs& a, dim3 grid, const void* q, const void* k, const void* v, void* out, bool pdl,
                       cudaStream_t stream) {
  constexpr size_t smem = 1024 + (size_t)kPrefillStages * 2 * kMmaStageKeys * HD * 2;
  if (!raise_smem_limit((const void*)attn_prefill_mma_kernel<T, HD>, (int)smem)) return 0;
  if (((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) != 0) return 0;
  // K and V as [head_dim][keys][KV heads][sequences], the decode kernel's maps.
  DecodeArgs view{};
  view.kv_len = a.seq;
  view.kv_heads = a.kv_heads;
  view.batch = grid.z;
  view.kv_batch_stride = a.kv_batch_stride;
  view.kv_row_stride = a.kv_row_stride;
  view.kv_head_stride = a.kv_head_stride;
  CUtensorMap kmap, vmap;
  const bool f16 = std::is_same<T, __half>::value;
  if (!encode_kv_map(&kmap, k, f16, view, HD) || !encode_kv_map(&vmap, v, f16, view, HD)) return 0;
  return launch_kernel(attn_prefill_mma_kernel<T, HD>, grid, dim3(kMmaWarps * 32), smem, stream, pdl, a, (const T*)q, kmap, vmap,
                       (T*)out) == cudaSuccess
             ? 1
             : 0;
}

}  // namespace

bool attn_decode_supported(const AttnDecodeShape& s) {
  if (!dtype_is_float(s.dtype)) return false;
  if (s.heads % s.kv_heads != 0) return false;
  const long long rep = s.heads / s.kv_heads;
  if (rep != 1 && rep != 2 && rep != 4 && rep != 8) return false;
  if (s.head_dim != 64 && s.head_dim != 128) return false;
  if (s.dtype == kF32 && s.head_dim * 4 / 16 > 32) return false;
  const int V = (int)(16 / dtype_size(s.dtype));
  auto al = [&](long long stride) { return stride % V == 0; };
  return al(s.q_batch_stride) && al(s.q_head_stride) && al(s.kv_batch_stride) && al(s.kv_row_stride) && al(s.kv_head_stride) &&
         s.batch <= 65535 && s.kv_heads <= 65535;
}

AttnDecodePlan attn_decode_plan(const AttnDecodeShape& s, int sm_count) {
  AttnDecodePlan p;
  const long long tiles = s.batch * s.kv_heads;
  const long long rep = s.heads / s.kv_heads;
  // Tensor-core kernel: 16-bit caches with four or eight query heads per KV head and 16-byte aligned rows; everything else
  // (f32, other head ratios) runs on the CUDA-core kernel. PJRTX_B200_ATTENTION_MMA=0 / 1 forces the choice wherever
  // the tensor-core kernel applies.
  const bool mma_ok = (s.dtype == kF16 || s.dtype == kBF16) && (rep == 4 || rep == 8) && (s.head_dim == 64 || s.head_dim == 128) &&
                      s.kv_len >= kMmaStageKeys &&  // the copies' box is a whole stage of keys
                      s.kv_row_stride % 8 == 0 && s.kv_head_stride % 8 == 0 && s.kv_batch_stride % 8 == 0;  // 16-byte pitches
  const char* force = getenv("PJRTX_B200_ATTENTION_MMA");
  const bool large = tiles * s.kv_len >= (long long)sm_count * 256;  // measured: ahead from batch 4 at 2K keys, 8 KV heads
  // Few (sequence, KV head) pairs of a 16-bit cache can run on the shared-memory staged kernel (one split per
  // kStagedKeys keys at least, about one CTA per SM) with PJRTX_B200_ATTENTION_STAGED=1. It is not a
  // default: on the 8B-shape decode step it gave 3.53 ms per step against 3.50 ms for the register-staged kernel.
  const char* staged_env = getenv("PJRTX_B200_ATTENTION_STAGED");
  const bool staged_on = staged_env && *staged_env && atoi(staged_env) != 0;
  if (staged_on && !(force && *force) && !large && (s.dtype == kF16 || s.dtype == kBF16)) {
    const long long need = (s.kv_len + kStagedKeys - 1) / kStagedKeys;
    long long want = std::max<long long>(need, sm_count / std::max<long long>(tiles, 1));
    if (const char* w = getenv("PJRTX_B200_ATTENTION_SPLITS")) want = std::max<long long>(need, atoi(w));  // experiments
    if (need <= 64 && tiles * need <= 2ll * sm_count) {
      p.mma = 2;
      p.splits = (int)std::max<long long>(1, std::min<long long>(std::min<long long>(want, s.kv_len), 64));
      p.workspace_bytes = (uint64_t)tiles * p.splits * rep * (s.head_dim + 2) * sizeof(float);
      p.counter_bytes = (uint64_t)tiles * 2 * sizeof(unsigned);
      return p;
    }
  }
  // The tensor-core kernel wherever it applies: since its rows come by tiled copies and its splits merge cooperatively it
  // is ahead at every size measured (8B shape, batch 1: 3.28 against 3.35 ms per step with 2.1 K keys, 3.36 against
  // 3.48 ms with 2.7 K; batch 2: 3.75 against 3.93 ms).
  p.mma = mma_ok && (force && *force ? atoi(force) != 0 : true) ? 1 : 0;
  if (p.mma) {
    // Two CTAs per SM are resident: one wave of them, no more (measured at 4K keys, batch 32: 32 / 64 / 128 / 256
    // (sequence, KV head) pairs run fastest with 9 / 4 / 2 / 1 splits — 25.5 / 36 / 57 / 84 us against 44 / 50 / 68 /
    // 103 us with twice as many CTAs), and no split shorter than two stages of keys.
    long long want = std::max<long long>(1, 2ll * sm_count / tiles);
    if (const char* w = getenv("PJRTX_B200_ATTENTION_SPLITS")) want = std::max(1, atoi(w));  // experiments
    // No split shorter than two stages (splits of one stage measured slower at 2.1 K keys and 8 KV heads: 3.30 ms per
    // 8B-shape step with 37, 3.31 with 30, 3.23 with 24 against 3.21 with 18).
    long long max_splits = std::max<long long>(1, s.kv_len / (2 * kMmaStageKeys));
    p.splits = (int)std::max<long long>(1, std::min<long long>(std::min(want, max_splits), 64));
    p.workspace_bytes = (uint64_t)tiles * p.splits * rep * (s.head_dim + 2) * sizeof(float);
    p.counter_bytes = (uint64_t)tiles * 2 * sizeof(unsigned);
    return p;
  }
  // Keys one CTA handles per chunk (see the kernel): no split should be shorter than that.
  const long long lanes_per_key = s.head_dim * (long long)dtype_size(s.dtype) / 16;
  const long long chunk = 8 * (32 / lanes_per_key) * (rep <= 4 ? 8 : 4);
  // Many pairs: about four CTAs per SM in total, so that the tail of the last wave is short next to the whole. Fewer
  // pairs than SMs (the latency regime: batch-1 decode): one wave of one CTA per SM - the 16-bit kernel with four heads
  // per KV head holds one CTA of 256 threads per SM, a second wave would start after the first, and only a grid that
  // is resident as a whole merges its splits cooperatively (with a 3744-key buffer the old rule asked for 29 splits
  // of the 8B shape's 8 KV heads: 232 CTAs, two waves, 0.82 instead of 0.53 ms for a step's 32 launches).
  long long want = tiles < sm_count ? std::max<long long>(1, sm_count / tiles) : (4ll * sm_count + tiles - 1) / tiles;
  long long max_splits = std::max<long long>(1, s.kv_len / chunk);
  p.splits = (int)std::max<long long>(1, std::min<long long>(std::min(want, max_splits), 64));
  p.workspace_bytes = (uint64_t)tiles * p.splits * rep * (s.head_dim + 2) * sizeof(float);
  p.counter_bytes = (uint64_t)tiles * 2 * sizeof(unsigned);
  return p;
}

int attn_decode_launch(const AttnDecodeShape& s, const AttnDecodePlan& plan, const void* q, const void* k, const void* v,
                       const void* token, void* out, void* workspace, void* counters, bool pdl, cudaStream_t stream,
                       bool early_kv, int* error_flag, const void* prefetch, uint64_t prefetch_bytes) {
  DecodeArgs a{};
  a.error_flag = error_flag;
  // Off unless PJRTX_B200_ATTENTION_PREFETCH=1: measured on the 8B-shape decode step, the 2048 bulk L2 requests for the
  // 33 MB of the next projection double the attention kernel's time (18 -> 36 us) and the projection gains 3 us.
  static const bool prefetch_allowed = [] {
    const char* e = getenv("PJRTX_B200_ATTENTION_PREFETCH");
    return e && *e && atoi(e) != 0;
  }();
  a.prefetch = prefetch_allowed && prefetch && (reinterpret_cast<uintptr_t>(prefetch) & 15) == 0 ? static_cast<const unsigned char*>(prefetch) : nullptr;
  a.prefetch_bytes = a.prefetch ? prefetch_bytes : 0;
  static const bool early_allowed = [] {
    const char* e = getenv("PJRTX_B200_ATTENTION_EARLY_KV");
    return !(e && *e && atoi(e) == 0);
  }();
  a.early_kv = early_kv && early_allowed ? 1 : 0;
  a.batch = s.batch;
  a.heads = s.heads;
  a.kv_heads = s.kv_heads;
  a.kv_len = s.kv_len;
  a.q_batch_stride = s.q_batch_stride;
  a.q_head_stride = s.q_head_stride;
  a.kv_batch_stride = s.kv_batch_stride;
  a.kv_row_stride = s.kv_row_stride;
  a.kv_head_stride = s.kv_head_stride;
  a.token_dtype = s.token_dtype;
  a.round_scores = s.round_scores;
  a.scale = s.scale;
  a.splits = plan.splits;
  a.workspace = static_cast<float*>(workspace);
  a.counters = static_cast<unsigned*>(counters);
  dim3 grid((unsigned)plan.splits, (unsigned)s.kv_heads, (unsigned)s.batch);
  const int rep = (int)(s.heads / s.kv_heads);
  {
    // Cooperative merge of the splits only where every CTA of the grid has an SM to itself (the CUDA-core and the
    // staged kernels, at most one CTA per SM counted), so that CTAs may wait for each other.
    int device = 0, sms = 0;
    if (coop_merge_allowed() && plan.mma != 1 && plan.splits > 1 && cudaGetDevice(&device) == cudaSuccess &&
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) == cudaSuccess)
      a.coop_merge = (long long)plan.splits * s.kv_heads * s.batch <= sms ? 1 : 0;
    a.timeout_ns = 2000000000ull;
  }
  if (plan.mma == 1 && ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15) != 0) return 0;  // bulk copies of rows
  if (plan.mma == 2) {
    if (s.dtype == kF16) return dispatch_decode_staged<__half>(rep, (int)s.head_dim, a, grid, q, k, v, token, out, pdl, stream);
    return dispatch_decode_staged<__nv_bfloat16>(rep, (int)s.head_dim, a, grid, q, k, v, token, out, pdl, stream);
  }
  if (plan.mma) {
    if (s.dtype == kF16) return dispatch_decode_mma<__half>(rep, (int)s.head_dim, a, grid, q, k, v, token, out, pdl, stream);
    return dispatch_decode_mma<__nv_bfloat16>(rep, (int)s.head_dim, a, grid, q, k, v, token, out, pdl, stream);
  }
  if (s.dtype == kF32) {
    // f32 rows are twice as wide: only head_dim 64 and 128 with 16 / 32 lanes per key.
    return dispatch_decode<float>(rep, (int)s.head_dim, a, grid, q, k, v, token, out, pdl, stream);
  }
  if (s.dtype == kF16) return dispatch_decode<__half>(rep, (int)s.head_dim, a, grid, q, k, v, token, out, pdl, stream);
  return dispatch_decode<__nv_bfloat16>(rep, (int)s.head_dim, a, grid, q, k, v, token, out, pdl, stream);
}

bool attn_prefill_supported(const AttnPrefillShape& s) {
  if (s.dtype != kF16 && s.dtype != kBF16) return false;
  if (s.head_dim != 64 && s.head_dim != 128) return false;
  if (s.batch < 1 || s.kv_heads < 1 || s.rep < 1 || s.seq < 1 || s.seq > (1LL << 30)) return false;
  if (s.batch > 65535 || s.kv_heads > 65535) return false;
  if ((s.seq * s.rep + kPrefillRows - 1) / kPrefillRows > 0x7fffffffLL) return false;
  // 16-byte key/value rows.
  if (s.kv_row_stride % 8 || s.kv_head_stride % 8 || s.kv_batch_stride % 8) return false;
  return true;
}

int attn_prefill_launch(const AttnPrefillShape& s, const void* q, const void* k, const void* v, void* out, bool pdl,
                        cudaStream_t stream, int* error_flag) {
  if (!attn_prefill_supported(s)) return 0;
  PrefillArgs a;
  a.error_flag = error_flag;
  a.seq = s.seq;
  a.rep = (int)s.rep;
  a.rows = s.seq * s.rep;
  a.kv_heads = (int)s.kv_heads;
  a.kv_batch_stride = s.kv_batch_stride;
  a.kv_row_stride = s.kv_row_stride;
  a.kv_head_stride = s.kv_head_stride;
  a.scale = s.scale;
  dim3 grid((unsigned)((a.rows + kPrefillRows - 1) / kPrefillRows), (unsigned)s.kv_heads, (unsigned)s.batch);
  if (s.dtype == kBF16)
    return s.head_dim == 128 ? launch_prefill_mma<__nv_bfloat16, 128>(a, grid, q, k, v, out, pdl, stream)
                             : launch_prefill_mma<__nv_bfloat16, 64>(a, grid, q, k, v, out, pdl, stream);
  return s.head_dim == 128 ? launch_prefill_mma<__half, 128>(a, grid, q, k, v, out, pdl, stream)
                           : launch_prefill_mma<__half, 64>(a, grid, q, k, v, out, pdl, stream);
}

}  // namespace pjrtx

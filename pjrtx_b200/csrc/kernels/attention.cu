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
// share a KV head are processed by the same CTA; a group of head_dim*esize/16 lanes owns one key row at a time, keeps
// its slice of every query head and of every output accumulator in registers and needs only log2(group) shuffles per
// key for the score. The key range is split across CTAs (grid.x) to fill the GPU at batch 1; partial (max, sum, out)
// triples go to an f32 workspace and the CTA that arrives last merges them in split order (deterministic).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

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

constexpr int kWarps = 8;
constexpr int kKeysPerStep = 4;  // keys a lane group handles per loop iteration (loads issued together)

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
};

// Merge (m2, l2, o2) into (m1, l1, o1); -inf maxima stand for "no keys seen".
template <int N>
__device__ __forceinline__ void merge_state(float& m1, float& l1, float* o1, float m2, float l2, const float* o2) {
  const float m = fmaxf(m1, m2);
  const float a = m1 == -INFINITY ? 0.f : __expf(m1 - m);
  const float b = m2 == -INFINITY ? 0.f : __expf(m2 - m);
  l1 = l1 * a + l2 * b;
#pragma unroll
  for (int i = 0; i < N; i++) o1[i] = o1[i] * a + o2[i] * b;
  m1 = m;
}

template <typename T, int REP, int HD>
__global__ void __launch_bounds__(kWarps * 32)
attn_decode_kernel(DecodeArgs a, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                   const void* __restrict__ token, T* __restrict__ out) {
  PJRTX_PDL_PROLOGUE();
  constexpr int V = Elem<T>::V;
  constexpr int LPK = HD / V;        // lanes per key row
  constexpr int KPW = 32 / LPK;      // key rows per warp per step
  static_assert(LPK >= 1 && LPK <= 32 && (LPK & (LPK - 1)) == 0, "head_dim must give a power-of-two lane group");
  __shared__ float sm_m[kWarps][REP], sm_l[kWarps][REP];
  __shared__ float sm_o[kWarps][REP][HD];
  __shared__ int is_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPK, gl = lane % LPK;  // which key of the step, which slice of the row
  const int split = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  long long limit = load_scalar(token, a.token_dtype);  // keys 0..limit are visible
  if (limit >= a.kv_len) limit = a.kv_len - 1;
  const long long count = limit + 1;
  const long long chunk = (count + a.splits - 1) / a.splits;
  const long long j_begin = (long long)split * chunk;
  const long long j_end = min(j_begin + chunk, count);

  // Query slices of the `rep` heads that share this KV head.
  float qf[REP][V];
#pragma unroll
  for (int r = 0; r < REP; r++) {
    const T* qp = q + b * a.q_batch_stride + (g * REP + r) * a.q_head_stride + gl * V;
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(qp));
    Elem<T>::unpack(raw, qf[r]);
  }
  float m[REP], l[REP], o[REP][V];
#pragma unroll
  for (int r = 0; r < REP; r++) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < V; i++) o[r][i] = 0.f;
  }
  const T* kb = k + b * a.kv_batch_stride + g * a.kv_head_stride + gl * V;
  const T* vb = v + b * a.kv_batch_stride + g * a.kv_head_stride + gl * V;

  // Each lane group walks keys j_begin + warp*KPW + sub + t*(kWarps*KPW). The loop bound is the same for every
  // lane of the warp (the shuffles below need all 32 lanes); keys past the end are masked per lane.
  constexpr int STRIDE = kWarps * KPW;
  for (long long base = j_begin + warp * KPW; base < j_end; base += (long long)STRIDE * kKeysPerStep) {
    uint4 kr[kKeysPerStep], vr[kKeysPerStep];
    bool ok[kKeysPerStep];
#pragma unroll
    for (int u = 0; u < kKeysPerStep; u++) {
      const long long j = base + sub + (long long)u * STRIDE;
      ok[u] = j < j_end;
      const long long jj = ok[u] ? j : j_begin;  // a valid row; its contribution is masked below
      kr[u] = __ldg(reinterpret_cast<const uint4*>(kb + jj * a.kv_row_stride));
      vr[u] = __ldg(reinterpret_cast<const uint4*>(vb + jj * a.kv_row_stride));
    }
    float s[kKeysPerStep][REP];
#pragma unroll
    for (int u = 0; u < kKeysPerStep; u++) {
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
      }
    }
#pragma unroll
    for (int r = 0; r < REP; r++) {
      float mx = m[r];
#pragma unroll
      for (int u = 0; u < kKeysPerStep; u++) mx = fmaxf(mx, s[u][r]);
      if (mx == -INFINITY) continue;
      const float corr = m[r] == -INFINITY ? 0.f : __expf(m[r] - mx);
      l[r] *= corr;
#pragma unroll
      for (int i = 0; i < V; i++) o[r][i] *= corr;
      m[r] = mx;
    }
#pragma unroll
    for (int u = 0; u < kKeysPerStep; u++) {
      float vf[V];
      Elem<T>::unpack(vr[u], vf);
#pragma unroll
      for (int r = 0; r < REP; r++) {
        const float p = s[u][r] == -INFINITY ? 0.f : __expf(s[u][r] - m[r]);
        l[r] += p;
#pragma unroll
        for (int i = 0; i < V; i++) o[r][i] = fmaf(p, vf[i], o[r][i]);
      }
    }
  }
  // Merge the KPW lane groups of the warp.
#pragma unroll
  for (int off = LPK; off < 32; off <<= 1) {
#pragma unroll
    for (int r = 0; r < REP; r++) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m[r], off);
      const float l2 = __shfl_xor_sync(0xffffffffu, l[r], off);
      float o2[V];
#pragma unroll
      for (int i = 0; i < V; i++) o2[i] = __shfl_xor_sync(0xffffffffu, o[r][i], off);
      merge_state<V>(m[r], l[r], o[r], m2, l2, o2);
    }
  }
  if (sub == 0) {
#pragma unroll
    for (int r = 0; r < REP; r++) {
      if (gl == 0) {
        sm_m[warp][r] = m[r];
        sm_l[warp][r] = l[r];
      }
#pragma unroll
      for (int i = 0; i < V; i++) sm_o[warp][r][gl * V + i] = o[r][i];
    }
  }
  __syncthreads();
  // Merge the warps (fixed order) and publish this split's partial.
  const long long tile = (long long)b * a.kv_heads + g;
  float* ws = a.workspace + (tile * a.splits + split) * (long long)REP * (HD + 2);
  for (int idx = threadIdx.x; idx < REP * HD; idx += kWarps * 32) {
    const int r = idx / HD, d = idx % HD;
    float mm = sm_m[0][r], ll = sm_l[0][r], oo = sm_o[0][r][d];
#pragma unroll
    for (int w = 1; w < kWarps; w++) {
      float o2 = sm_o[w][r][d];
      merge_state<1>(mm, ll, &oo, sm_m[w][r], sm_l[w][r], &o2);
    }
    ws[r * (HD + 2) + d] = oo;
    if (d == 0) {
      ws[r * (HD + 2) + HD] = mm;
      ws[r * (HD + 2) + HD + 1] = ll;
    }
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(&a.counters[tile], 1u) == (unsigned)a.splits - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // Two passes over the splits with independent loads (issued in batches) instead of one dependent chain: first the
  // overall maximum, then the weighted sums in split order.
  const float* base = a.workspace + tile * a.splits * (long long)REP * (HD + 2);
  const long long split_stride = (long long)REP * (HD + 2);
  for (int idx = threadIdx.x; idx < REP * HD; idx += kWarps * 32) {
    const int r = idx / HD, d = idx % HD;
    const float* p = base + r * (HD + 2);
    float mm = -INFINITY;
    for (int sp = 0; sp < a.splits; sp += 8) {
      float mv[8];
#pragma unroll
      for (int e = 0; e < 8; e++) mv[e] = sp + e < a.splits ? __ldcg(p + (sp + e) * split_stride + HD) : -INFINITY;
#pragma unroll
      for (int e = 0; e < 8; e++) mm = fmaxf(mm, mv[e]);
    }
    float ll = 0.f, oo = 0.f;
    for (int sp = 0; sp < a.splits; sp += 4) {
      float mv[4], lv[4], ov[4];
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const bool in = sp + e < a.splits;
        mv[e] = in ? __ldcg(p + (sp + e) * split_stride + HD) : -INFINITY;
        lv[e] = in ? __ldcg(p + (sp + e) * split_stride + HD + 1) : 0.f;
        ov[e] = in ? __ldcg(p + (sp + e) * split_stride + d) : 0.f;
      }
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const float w = mv[e] == -INFINITY ? 0.f : __expf(mv[e] - mm);
        ll = fmaf(lv[e], w, ll);
        oo = fmaf(ov[e], w, oo);
      }
    }
    out[b * a.q_batch_stride + (g * REP + r) * a.q_head_stride + d] = Elem<T>::store(ll > 0.f ? oo / ll : 0.f);
  }
  if (threadIdx.x == 0) a.counters[tile] = 0;
}

template <typename T, int REP, int HD>
int launch_decode(const DecodeArgs& a, dim3 grid, const void* q, const void* k, const void* v, const void* token, void* out, bool pdl,
                  cudaStream_t stream) {
  return launch_kernel(attn_decode_kernel<T, REP, HD>, grid, dim3(kWarps * 32), 0, stream, pdl, a, (const T*)q, (const T*)k,
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
  // About one CTA per SM; every split should still cover a few hundred keys' worth of rows.
  long long want = ((long long)sm_count + tiles - 1) / tiles;
  long long max_splits = std::max<long long>(1, s.kv_len / 64);
  p.splits = (int)std::max<long long>(1, std::min<long long>(std::min(want, max_splits), 64));
  const long long rep = s.heads / s.kv_heads;
  p.workspace_bytes = (uint64_t)tiles * p.splits * rep * (s.head_dim + 2) * sizeof(float);
  p.counter_bytes = (uint64_t)tiles * sizeof(unsigned);
  return p;
}

int attn_decode_launch(const AttnDecodeShape& s, const AttnDecodePlan& plan, const void* q, const void* k, const void* v,
                       const void* token, void* out, void* workspace, void* counters, bool pdl, cudaStream_t stream) {
  DecodeArgs a{};
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
  if (s.dtype == kF32) {
    // f32 rows are twice as wide: only head_dim 64 and 128 with 16 / 32 lanes per key.
    return dispatch_decode<float>(rep, (int)s.head_dim, a, grid, q, k, v, token, out, pdl, stream);
  }
  if (s.dtype == kF16) return dispatch_decode<__half>(rep, (int)s.head_dim, a, grid, q, k, v, token, out, pdl, stream);
  return dispatch_decode<__nv_bfloat16>(rep, (int)s.head_dim, a, grid, q, k, v, token, out, pdl, stream);
}

}  // namespace pjrtx

// Launch wrappers of the precompiled sm_100a kernels. Every wrapper enqueues on
// the given stream and returns the number of kernels it launched (0 = refused).
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <set>
#include <utility>

namespace pjrtx {

// A kernel's dynamic shared-memory limit is an attribute of the (kernel, device) pair: raise it once for each device
// the kernel is launched on (the current device of the calling thread).
inline bool raise_smem_limit(const void* kernel, int bytes) {
  static std::mutex mu;
  static std::set<std::pair<const void*, int>> done;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return false;
  std::lock_guard<std::mutex> lock(mu);
  if (done.count({kernel, device})) return true;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) return false;
  done.insert({kernel, device});
  return true;
}

// Attributes of every launch of the library: programmatic stream serialization when `pdl`, and - when
// PJRTX_B200_CARVEOUT is set (0..100) - that shared-memory carveout, the same for every kernel, so that consecutive
// kernels never ask the SMs for different splits between L1 and shared memory. Returns the number filled in (<= 2).
inline unsigned fill_launch_attributes(cudaLaunchAttribute* attr, bool pdl) {
  static const int carveout = [] {
    const char* v = getenv("PJRTX_B200_CARVEOUT");
    return v && *v ? atoi(v) : -1;
  }();
  unsigned n = 0;
  if (pdl) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    n++;
  }
  if (carveout >= 0 && carveout <= 100) {
    attr[n].id = cudaLaunchAttributePreferredSharedMemoryCarveout;
    attr[n].val.sharedMemCarveout = (unsigned)carveout;
    n++;
  }
  return n;
}

// Launch with (optionally) programmatic stream serialization: the kernel may begin while its predecessor in the stream
// is still running; kernels call griddepcontrol.wait before their first dependent access.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl,
                                 Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  cfg.attrs = attr;
  cfg.numAttrs = fill_launch_attributes(attr, pdl);
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#define PJRTX_PDL_PROLOGUE()                                              \
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");         \
  asm volatile("griddepcontrol.wait;" ::: "memory")

// Canonical contraction out[b0,b1,m,n] = sum_k lhs[b0,b1,m,k] * rhs[b0,b1,k,n]
// with arbitrary element strides, as produced by analysing a dot_general
// (src/backend/mlx_metal/api.cc:3349-3498 canonicalises the same way by
// transposing; here the strides are passed to the kernel instead).
struct DotShape {
  int dtype = 0;
  int64_t b0 = 1, b1 = 1, m = 1, n = 1, k = 1;
  int64_t lhs_b0 = 0, lhs_b1 = 0, lhs_m = 0, lhs_k = 1;
  int64_t rhs_b0 = 0, rhs_b1 = 0, rhs_k = 0, rhs_n = 1;
  int64_t out_b0 = 0, out_b1 = 0, out_m = 0;  // out n stride is 1
  // 1: the rhs holds signed bytes with one f16 scale per column n; the contraction uses
  // round_to_dtype(round_f16(f16(byte) * scale)) as rhs[k, n] (the program's convert * multiply [* convert]).
  int rhs_s8 = 0;
};

// Scratch a split-K streaming contraction needs: f32 partials + tile counters.
struct DotScratch {
  uint64_t partial_bytes = 0;
  uint64_t counter_bytes = 0;
  int ksplit = 1;
  // 0 generic, 1 streaming rhs[K,N] (N contiguous), 2 streaming rhs[N,K] (K contiguous), 3 f32 tile,
  // 4 tensor-core stream with rhs[N,K] (K contiguous)
  int path = 0;
  // Path 1 without batch axes runs the TMA-fed persistent kernel (stream-K decomposition).
  int tma = 0;
  // Paths 1 and 4 for 16-bit floats without batch axes can run on the tensor cores (tcgen05, accumulator in TMEM).
  int umma = 0, m_tile = 0, sub = 1, nh = 1, whole_tiles = 0;
  int grid = 0, stages = 0, max_contrib = 0;
  long long per_cta = 0;
  uint64_t smem = 0;
};

constexpr int kDotGroupMax = 4;

// Streaming contractions (path 1) that share lhs, m, k, dtype and have no batch axes can run as one launch.
// `allow_tensor` = false keeps the CUDA-core streaming kernel even where the tensor-core one would apply.
DotScratch dot_group_plan(const DotShape* shapes, int count, int sm_count, bool allow_tensor = true);
// `error_flag` (device-visible int) receives a non-zero code if a bounded device-side wait gives up.
// `early_rhs`: the rhs operands are never written by earlier work of the same stream, so their copies may start
// before the preceding kernel has finished (programmatic dependent launch).
// `scales` (one f16 pointer per contraction) is read only when the shapes have `rhs_s8`.
int dot_group_launch(const DotShape* shapes, int count, const DotScratch& plan, const void* lhs, const void* const* rhs,
                     void* const* out, void* partials, void* counters, int* error_flag, bool early_rhs, bool pdl,
                     cudaStream_t stream, const void* const* scales = nullptr);

// Chooses the kernel for a shape and sizes its scratch.
DotScratch dot_plan(const DotShape& s, int sm_count);

// ---- chained streaming contractions --------------------------------------------------------------------------------
// A chain is a sequence of up to kDotChainMax segments run by ONE launch of the CUDA-core streaming kernel; a segment
// is a group of up to kDotGroupMax contractions that share an lhs. A segment may read what earlier segments of the
// chain wrote (the kernel separates segments with a grid-wide barrier while its weight copies run on). The lhs of a
// segment can be transformed as it is loaded, and a contraction's result can take a residual:
//   kDotLhsRmsNorm  lhs[m, k] = round(round(x[m, k] * rsqrt(sum_k(x[m, k]^2) * norm_scale + norm_eps)) * gain[k])
//   kDotLhsSiluMul  lhs[m, k] = round(round(g[m, k] * round(logistic(g[m, k]))) * u[m, k])
//   residual        out[m, n] = round(residual[m, n] + round(sum))
// with `round` = rounding to the element type (what the op-by-op program does between instructions).
constexpr int kDotChainMax = 4;
enum DotLhsKind { kDotLhsPlain = 0, kDotLhsRmsNorm = 1, kDotLhsSiluMul = 2 };
struct DotLhs {
  int kind = kDotLhsPlain;
  float norm_scale = 0.f, norm_eps = 0.f;
};
struct DotChainSegment {
  DotShape shapes[kDotGroupMax];
  int count = 0;
  DotLhs lhs;
  // rms_norm only: x is the (single) result of the previous segment of the chain. That segment then leaves the sum of
  // squares of every column tile it completes, and this one adds those instead of reading the row again.
  bool norm_of_previous = false;
};
struct DotChainArgs {
  const void* lhs = nullptr;    // plain: operand; rms_norm: x; silu_mul: gate
  const void* lhs2 = nullptr;   // rms_norm: gain; silu_mul: up
  const void* rhs[kDotGroupMax] = {nullptr, nullptr, nullptr, nullptr};
  void* out[kDotGroupMax] = {nullptr, nullptr, nullptr, nullptr};
  const void* residual[kDotGroupMax] = {nullptr, nullptr, nullptr, nullptr};
};
struct DotChainPlan {
  int segments = 0, grid = 0, stages = 0;
  uint64_t smem = 0;
  int max_contrib[kDotChainMax] = {};
  uint64_t counter_offset[kDotChainMax] = {};  // byte offsets into the counter region (after the barrier words)
  uint64_t ssq_offset[kDotChainMax] = {};      // per segment: where it leaves its tiles' sums of squares (0 = it does not)
  int tiles[kDotChainMax] = {};
  uint64_t partial_bytes = 0;   // one region shared by the segments (a segment's partials are consumed inside it)
  uint64_t counter_bytes = 0;   // barrier words + every segment's tile counters; zero before the first launch
};
// True when the contraction runs on the CUDA-core streaming kernel (and can therefore join a chain).
bool dot_chain_eligible(const DotShape& s, int sm_count);
DotChainPlan dot_chain_plan(const DotChainSegment* segs, int n, int sm_count);
int dot_chain_launch(const DotChainSegment* segs, const DotChainArgs* args, int n, const DotChainPlan& plan, void* partials,
                     void* counters, int* error_flag, bool early_rhs, bool pdl, cudaStream_t stream);
int dot_launch(const DotShape& s, const DotScratch& plan, const void* lhs, const void* rhs, void* out,
               void* partials, void* counters, int* error_flag, bool early_rhs, bool pdl, cudaStream_t stream,
               const void* scale = nullptr);
// True when an int8-weight contraction of this shape has a kernel (the tensor-core stream with in-kernel dequantisation).
bool dot_s8_supported(const DotShape& s);

// out[m, n] = lhs[m, k] . rhs[k, n] (dense row-major device pointers) with split-K scratch taken from a fixed
// array in the library image instead of an allocation. 1 on success, 0 with last_error set.
int stream_dot_static_scratch(int device, int dtype, const void* lhs, const void* rhs, void* out, int64_t m, int64_t k,
                              int64_t n, cudaStream_t stream);
// Waits for `stream` and reports whether the most recent static-scratch contraction on the device ran to completion
// (1) or gave up a bounded device-side wait (0 with last_error set). Allocates nothing.
int stream_dot_static_scratch_status(int device, cudaStream_t stream);

// Self-test of the bounded device-side waits: one CTA waits (with the wait the streaming kernels use) for an mbarrier
// that nothing completes, gives up after `timeout_ms` (1..1000) and raises `error_flag` with code 31. The kernel
// returns normally; nothing faults or hangs.
int bounded_wait_probe_launch(unsigned timeout_ms, int* error_flag, cudaStream_t stream);

// dynamic_update_slice: writes `update` into `dst` (already holding the operand)
// at start indices read from device scalars, clamped as StableHLO requires.
struct SliceUpdateShape {
  int rank = 0;
  int elem_size = 1;
  int64_t dst_dims[8] = {0};
  int64_t upd_dims[8] = {0};
  int start_dtype[8] = {0};
};
int dus_launch(const SliceUpdateShape& s, void* dst, const void* update, const void* const* start_ptrs, bool pdl,
               cudaStream_t stream);

// Scaled dot-product attention custom call (src/backend/mlx_metal/custom_call.zig:120-152,
// src/backend/mlx_metal/api.cc:4929-5043): q [b,]q,h,hd ; k,v [b,]kv,g,hd ; scalar token index.
struct SdpaShape {
  int dtype = 0;
  int64_t batch = 1, q_len = 1, heads = 1, kv_len = 1, kv_heads = 1, head_dim = 1;
  int token_dtype = 0;
};
int sdpa_launch(const SdpaShape& s, const void* q, const void* k, const void* v, const void* token_index, void* out,
                bool pdl, cudaStream_t stream);

// Decode attention (one query position per sequence, grouped-query heads) as one split-KV kernel.
// q / out: [batch, heads, head_dim] through (q_batch_stride, q_head_stride); k / v: [batch, kv_len, kv_heads, head_dim]
// through (kv_batch_stride, kv_row_stride, kv_head_stride); keys 0..token are visible.
struct AttnDecodeShape {
  int dtype = 0;
  long long batch = 1, heads = 1, kv_heads = 1, kv_len = 1, head_dim = 1;
  long long q_batch_stride = 0, q_head_stride = 0;
  long long kv_batch_stride = 0, kv_row_stride = 0, kv_head_stride = 0;
  int token_dtype = 0;
  int round_scores = 0;  // round q.k to the element type before scaling (what an explicit dot_general does)
  float scale = 1.f;
};
struct AttnDecodePlan {
  int splits = 1;
  // 0: CUDA-core kernel (rows held in registers), 1: warp-level tensor-core kernel (16-bit caches, many rows),
  // 2: shared-memory staged kernel fed by bulk copies (16-bit caches, few (sequence, KV head) pairs)
  int mma = 0;
  uint64_t workspace_bytes = 0, counter_bytes = 0;
};
bool attn_decode_supported(const AttnDecodeShape& s);
AttnDecodePlan attn_decode_plan(const AttnDecodeShape& s, int sm_count);
// `early_kv`: no earlier kernel of the stream writes cache rows below the token index (a decode step appends the row
// at the token index in place), so those rows may be requested before the preceding kernel has finished.
// `error_flag` (device-visible int, may be null) receives a non-zero code if a bounded device-side wait gives up.
// `prefetch` / `prefetch_bytes`: a 16-byte aligned range that no work of the stream writes (the weights of the
// contraction that follows); the kernel's CTAs request it into L2 as they start.
int attn_decode_launch(const AttnDecodeShape& s, const AttnDecodePlan& plan, const void* q, const void* k, const void* v,
                       const void* token, void* out, void* workspace, void* counters, bool pdl, cudaStream_t stream,
                       bool early_kv = false, int* error_flag = nullptr, const void* prefetch = nullptr,
                       uint64_t prefetch_bytes = 0);

// Causal self-attention over whole sequences (prefill) as one tensor-core kernel. q / out: [batch, kv_heads, seq, rep,
// head_dim] contiguous (query head = kv head * rep + r); k / v: [batch, seq, kv_heads, head_dim] through the strides;
// position s sees keys 0..s. q.k is rounded to the element type before it is scaled, as the explicit dot_general does.
struct AttnPrefillShape {
  int dtype = 0;
  long long batch = 1, kv_heads = 1, rep = 1, seq = 1, head_dim = 1;
  long long kv_batch_stride = 0, kv_row_stride = 0, kv_head_stride = 0;
  float scale = 1.f;
};
bool attn_prefill_supported(const AttnPrefillShape& s);
int attn_prefill_launch(const AttnPrefillShape& s, const void* q, const void* k, const void* v, void* out, bool pdl,
                        cudaStream_t stream, int* error_flag = nullptr);

// All-reduce (sum) over peer-mapped regions, one launch per rank (kernels/peer_reduce.cu). `regions[r]` is rank r's
// region as mapped into this process (regions[rank] is the local one), `peer_region_bytes(slot_bytes)` long.
// Returns 0 when the call does not fit (more than 8 ranks, size not a multiple of 8 x ranks bytes, or a part of it
// larger than half a slot).
uint64_t peer_region_bytes(uint64_t slot_bytes);
int peer_all_reduce_launch(void* const* regions, int rank, int world, uint64_t slot_bytes, int dtype, const void* in, void* out,
                           uint64_t count, int* error_flag, bool pdl, cudaStream_t stream);

}  // namespace pjrtx

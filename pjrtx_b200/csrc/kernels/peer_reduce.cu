// All-reduce over peer memory (NVLink / NVSwitch) for the small row-parallel activations of tensor-parallel decode
// (e.g. [32, 8192] bf16 = 512 KiB per call, 160 calls per 70B-shape step), where a library collective is bound by its
// fixed latency.
//
// Every rank owns a region of plain device memory that all other ranks have mapped (CUDA IPC). Data travels as
// self-validating 16-byte vectors {data, step, data, step}: the receiver polls the vector itself until both step words
// match, so there are no fences, no separate flags and no second round trip; the cost is that 8 data bytes occupy 16.
// One launch per rank, two hops (reduce-scatter, then all-gather), any thread independent of the others:
//   A. the input is cut into `world` equal parts; the piece of part p goes to rank p's region, slot A[rank];
//   B. for its own part a rank polls slots A[0..world) of its OWN region, adds them in rank order in f32, rounds to
//      the element type and sends the result to every rank's slot B[rank];
//   C. it polls slots B[0..world) of its own region and writes the parts of its output.
// Every rank computes a part exactly once and everybody receives the same rounded values: results are bit-identical
// across ranks and runs. Two sets of slots alternate with the step number: a rank can reach step s + 2 only after it
// has received step s + 1 from everybody, which they send after finishing step s. The step number lives in the region
// (advanced by the CTA that arrives last), so a captured launch replays correctly. Polls are bounded by TIME: a launch
// gives its peers `timeout_ns` (two seconds unless PJRTX_B200_PEER_TIMEOUT_MS says otherwise) from the moment it starts;
// the first thread that sees the deadline pass raises the error word (code 21) and tells its CTA, every other poll of
// the launch then gives up at once, and the kernel finishes with whatever it has - an absent rank costs one timeout,
// not one per element, and nothing hangs. The budget is also the skew the ranks may have when they reach a collective
// (a rank still compiling or paused on the host for longer makes the others report the error). No kernel waits on
// another kernel of the same GPU.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>

#include "../common.h"
#include "kernels.h"

namespace pjrtx {

namespace {

constexpr int kPeerMax = 8;
constexpr unsigned kHeaderBytes = 4096;
struct PeerArgs {
  unsigned char* region[kPeerMax];
  int rank, world;
  unsigned long long slot_bytes;  // one slot: a part (1 / world of the data) in the 16-byte wire format
  unsigned long long timeout_ns;  // budget of one launch for all its polls
  int* error_flag;
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void st_wire(void* p, unsigned d0, unsigned d1, unsigned step) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d0), "r"(step), "r"(d1), "r"(step) : "memory");
}
// Polls until both halves of a vector carry `step`; false when the launch's deadline passed (seen by this thread, or
// by another thread of the CTA that has set *gave_up). One vector of each source in `mask` at once: all loads of a
// round are issued before the first is looked at, so that waiting for eight peers costs the slowest arrival plus one
// round trip to L2, not eight.
// Source q's vector is at first + q * stride (bytes).
__device__ __forceinline__ bool ld_wire_all(const unsigned char* first, unsigned long long stride, unsigned mask, unsigned step,
                                            unsigned (&d0)[kPeerMax], unsigned (&d1)[kPeerMax], unsigned long long deadline,
                                            volatile int* gave_up) {
  unsigned pending = mask;
  for (unsigned spin = 0; pending; spin++) {
    unsigned a[kPeerMax], fa[kPeerMax], b[kPeerMax], fb[kPeerMax];
#pragma unroll
    for (int q = 0; q < kPeerMax; q++)
      if (pending >> q & 1u)
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(a[q]), "=r"(fa[q]), "=r"(b[q]), "=r"(fb[q])
                     : "l"(first + q * stride)
                     : "memory");
#pragma unroll
    for (int q = 0; q < kPeerMax; q++)
      if ((pending >> q & 1u) && fa[q] == step && fb[q] == step) {
        d0[q] = a[q];
        d1[q] = b[q];
        pending &= ~(1u << q);
      }
    if (pending && (spin & 63) == 63) {
      if (*gave_up) return false;
      if (global_timer_ns() > deadline) {
        *gave_up = 1;
        return false;
      }
    }
  }
  return true;
}

template <typename T> struct Pair;  // 8 data bytes = two 32-bit words
template <> struct Pair<float> {
  static __device__ __forceinline__ void add(float* acc, unsigned d0, unsigned d1) {
    acc[0] += __uint_as_float(d0);
    acc[1] += __uint_as_float(d1);
  }
  static __device__ __forceinline__ void store(const float* acc, unsigned* d0, unsigned* d1) {
    *d0 = __float_as_uint(acc[0]);
    *d1 = __float_as_uint(acc[1]);
  }
  static constexpr int N = 2;
};
template <> struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ void add(float* acc, unsigned d0, unsigned d1) {
    acc[0] += __uint_as_float(d0 << 16);
    acc[1] += __uint_as_float(d0 & 0xffff0000u);
    acc[2] += __uint_as_float(d1 << 16);
    acc[3] += __uint_as_float(d1 & 0xffff0000u);
  }
  static __device__ __forceinline__ void store(const float* acc, unsigned* d0, unsigned* d1) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(acc[0], acc[1]), hi = __floats2bfloat162_rn(acc[2], acc[3]);
    *d0 = *reinterpret_cast<const unsigned*>(&lo);
    *d1 = *reinterpret_cast<const unsigned*>(&hi);
  }
  static constexpr int N = 4;
};
template <> struct Pair<__half> {
  static __device__ __forceinline__ void add(float* acc, unsigned d0, unsigned d1) {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&d0)), b = __half22float2(*reinterpret_cast<const __half2*>(&d1));
    acc[0] += a.x;
    acc[1] += a.y;
    acc[2] += b.x;
    acc[3] += b.y;
  }
  static __device__ __forceinline__ void store(const float* acc, unsigned* d0, unsigned* d1) {
    const __half2 lo = __floats2half2_rn(acc[0], acc[1]), hi = __floats2half2_rn(acc[2], acc[3]);
    *d0 = *reinterpret_cast<const unsigned*>(&lo);
    *d1 = *reinterpret_cast<const unsigned*>(&hi);
  }
  static constexpr int N = 4;
};

// `part_pairs` = 8-byte pairs per part; the data holds world * part_pairs pairs.
template <typename T>
__global__ void __launch_bounds__(256) peer_all_reduce_kernel(PeerArgs a, const uint2* __restrict__ in, uint2* __restrict__ out,
                                                              unsigned long long part_pairs) {
  PJRTX_PDL_PROLOGUE();
  __shared__ int gave_up;
  if (threadIdx.x == 0) gave_up = 0;
  const unsigned long long deadline = global_timer_ns() + a.timeout_ns;
  unsigned* header = reinterpret_cast<unsigned*>(a.region[a.rank]);
  unsigned* arrive = header + 64;  // CTAs of this launch that have read the step number
  unsigned* step_word = header + 65;
  const unsigned step = *reinterpret_cast<volatile unsigned*>(step_word) + 1;  // never 0: fresh memory is all zeros
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(arrive, 1u) == gridDim.x - 1) {  // everybody has read it: advance for the next launch
    *arrive = 0;
    *reinterpret_cast<volatile unsigned*>(step_word) = step;
  }
  // Slot [set][stage][source rank] of a region; stage 0 = A (contributions to a part), 1 = B (finished parts).
  const unsigned long long set_offset = kHeaderBytes + (unsigned long long)(step & 1) * 2 * kPeerMax * a.slot_bytes;
  auto slot = [&](int owner, int stage, int source) {
    return reinterpret_cast<uint4*>(a.region[owner] + set_offset + ((unsigned long long)stage * kPeerMax + source) * a.slot_bytes);
  };
  const unsigned long long stride = (unsigned long long)gridDim.x * blockDim.x;
  const unsigned long long first = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x;
  bool ok = true;
  // A: this rank's piece of every part goes to the part's owner.
  for (unsigned long long j = first; j < part_pairs; j += stride) {
#pragma unroll
    for (int p = 0; p < kPeerMax; p++)
      if (p < a.world) {
        const uint2 v = in[(unsigned long long)p * part_pairs + j];
        st_wire(slot(p, 0, a.rank) + j, v.x, v.y, step);
      }
  }
  // B: reduce the own part in rank order and send it to everybody.
  for (unsigned long long j = first; j < part_pairs; j += stride) {
    float acc[Pair<T>::N];
#pragma unroll
    for (int e = 0; e < Pair<T>::N; e++) acc[e] = 0.f;
    {
      unsigned d0[kPeerMax], d1[kPeerMax];
#pragma unroll
      for (int q = 0; q < kPeerMax; q++) d0[q] = d1[q] = 0;
      ok &= ld_wire_all(reinterpret_cast<const unsigned char*>(slot(a.rank, 0, 0) + j), a.slot_bytes, (1u << a.world) - 1u, step, d0, d1,
                        deadline, &gave_up);
#pragma unroll
      for (int q = 0; q < kPeerMax; q++)  // rank order, whoever arrived first
        if (q < a.world) Pair<T>::add(acc, d0[q], d1[q]);
    }
    unsigned r0, r1;
    Pair<T>::store(acc, &r0, &r1);
#pragma unroll
    for (int p = 0; p < kPeerMax; p++)
      if (p < a.world && p != a.rank) st_wire(slot(p, 1, a.rank) + j, r0, r1, step);
    out[(unsigned long long)a.rank * part_pairs + j] = make_uint2(r0, r1);
  }
  // C: collect the other parts.
  for (unsigned long long j = first; j < part_pairs; j += stride) {
    unsigned d0[kPeerMax], d1[kPeerMax];
#pragma unroll
    for (int p = 0; p < kPeerMax; p++) d0[p] = d1[p] = 0;
    ok &= ld_wire_all(reinterpret_cast<const unsigned char*>(slot(a.rank, 1, 0) + j), a.slot_bytes,
                      ((1u << a.world) - 1u) & ~(1u << a.rank), step, d0, d1, deadline, &gave_up);
#pragma unroll
    for (int p = 0; p < kPeerMax; p++)
      if (p < a.world && p != a.rank) out[(unsigned long long)p * part_pairs + j] = make_uint2(d0[p], d1[p]);
  }
  if (!ok) atomicExch(a.error_flag, 21);
}

}  // namespace

uint64_t peer_region_bytes(uint64_t slot_bytes) { return kHeaderBytes + 2ull * 2 * kPeerMax * slot_bytes; }

int peer_all_reduce_launch(void* const* regions, int rank, int world, uint64_t slot_bytes, int dtype, const void* in, void* out,
                           uint64_t count, int* error_flag, bool pdl, cudaStream_t stream) {
  const uint64_t bytes = count * dtype_size(dtype);
  // Whole 8-byte pairs per part, and a part in wire format (2 x) must fit a slot.
  if (world < 2 || world > kPeerMax || bytes == 0 || bytes % (8ull * world) != 0 || 2 * (bytes / world) > slot_bytes) return 0;
  if ((reinterpret_cast<uintptr_t>(in) & 7) || (reinterpret_cast<uintptr_t>(out) & 7)) return 0;
  PeerArgs a{};
  for (int p = 0; p < world; p++) a.region[p] = static_cast<unsigned char*>(regions[p]);
  a.rank = rank;
  a.world = world;
  a.slot_bytes = slot_bytes;
  a.error_flag = error_flag;
  static const unsigned long long timeout_ms = [] {
    const char* v = getenv("PJRTX_B200_PEER_TIMEOUT_MS");
    const long long n = v && *v ? atoll(v) : 2000;
    return (unsigned long long)(n < 1 ? 1 : n);
  }();
  a.timeout_ns = timeout_ms * 1000000ull;
  const unsigned long long part_pairs = bytes / world / 8;
  const unsigned grid = (unsigned)std::max<unsigned long long>(1, std::min<unsigned long long>(64, (part_pairs + 255) / 256));
  cudaError_t e;
  switch (dtype) {
    case kF32: e = launch_kernel(peer_all_reduce_kernel<float>, dim3(grid), dim3(256), 0, stream, pdl, a, (const uint2*)in, (uint2*)out, part_pairs); break;
    case kBF16: e = launch_kernel(peer_all_reduce_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, pdl, a, (const uint2*)in, (uint2*)out, part_pairs); break;
    case kF16: e = launch_kernel(peer_all_reduce_kernel<__half>, dim3(grid), dim3(256), 0, stream, pdl, a, (const uint2*)in, (uint2*)out, part_pairs); break;
    default: return 0;
  }
  return e == cudaSuccess ? 1 : 0;
}

}  // namespace pjrtx

// Contraction on the 5th-generation tensor cores (tcgen05) for 16-bit floats with f32 accumulation in tensor memory:
//   out[m, n] = sum_k lhs[m, k] * rhs[k, n]        lhs k-contiguous; rhs n-contiguous ([k, n]) or k-contiguous ([n, k])
//
// The product is computed transposed, D^T[n, m] = W^T[n, k] . x^T[k, m]: the 128-row side of the MMA is the weight's
// n axis and the cheap N side (16..256) is m. One decode row, a batch of 32 rows or a 256-row prefill tile all use
// the same kernel; a small m costs a narrow MMA instead of a padded 128-row one, and no CUDA-core FMA work is left on
// the SM, so for small m the kernel is a pure HBM stream: TMA in, tensor core, a tiny epilogue.
//
// One persistent CTA per SM, three roles:
//   producer lane   per unit (one [128 n x 64*SUB k] weight block + the matching [m_tile x 64*SUB] activation block),
//                   tiled TMA copies with the 128-byte swizzle into a ring of shared-memory stages; completion is
//                   counted on the stage's `full` mbarrier
//   MMA lane        4*SUB tcgen05.mma.cta_group::1.kind::f16 (M=128, N=m_tile, K=16) per stage, operands read through
//                   shared-memory descriptors, accumulator in TMEM (two accumulators, so the epilogue of one tile
//                   segment overlaps the MMAs of the next); tcgen05.commit releases the stage (`empty`) and, after a
//                   segment's last MMA, publishes the accumulator (`acc_full`)
//   epilogue warps  tcgen05.ld of the 128 x m_tile accumulator (TMEM lane = n, one per thread), then either the
//                   converted output or an f32 partial
// Work decomposition (stream-K): units are ordered tile-major and CTA b of G takes the b-th equal share, so every SM
// streams the same number of bytes whatever the shape. A CTA that covers only part of a tile's k range writes a
// partial; the CTA that arrives last for the tile folds the partials in CTA order (run-to-run identical results).
// For tall tiles (many rows of m) the f32 partials would outweigh the weights they save from idling, so the host
// then asks for whole tiles per CTA (`whole_tiles`) and nothing is folded.
//
// Programmatic dependent launch: weights are never written by earlier work of the stream (`early_rhs`), so their
// copies for the first ring of stages are issued before griddepcontrol.wait; activation copies and all stores wait.
//
// Int8 weights (W8): the rhs is [k, n] signed bytes with one f16 scale per column, the program's
// convert(s8 -> f16) * scale [-> bf16] feeding the contraction. The weights stay one byte wide in HBM: a stage receives
// the raw bytes, eight converter warps write the integers (exact in either 16-bit type) into the swizzled operand tile
// the tensor core reads, the MMA lane waits for `ready` (converted) instead of `full`, and the epilogue multiplies each
// accumulator by its column's scale in f32. That is the contraction the program wrote with the scale moved out of the
// sum: sum_k x[k] * (w[k,n] * s[n]) = s[n] * sum_k x[k] * w[k,n]. The op-by-op program rounds every w * s to the element
// type first; this form skips that rounding (one relative 2^-9 per weight at bf16), so the two agree to rounding, not
// bit for bit, and a product w * s that overflows f16 in the written program stays finite here.
// What bounds it: shared memory. A 128-deep stage moves about 110 KB through shared memory (16 KB of raw bytes written
// by the copy and read by the converters, 32 KB of 16-bit values written by them and read by the tensor core, the
// activation tile) against 80 KB on the 16-bit path, for half the HBM bytes: measured 1630 cycles per stage on the
// 4096 x 128256 LM head at 32 rows, where the 16-bit path takes 1510 (HBM-bound). Two groups of converter warps on
// alternate stages (to overlap one group's proxy fence with the other's work) measured the same to four digits.
//
// Every mbarrier wait is bounded by time (two seconds per launch; the thread that sees the deadline pass sets a CTA-wide
// abort word and every other wait gives up at its next check); the kernel then sets *error_flag, every role falls
// through to the common exit, the allocating warp frees its tensor memory, and the kernel returns.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace pjrtx {
namespace umma {

constexpr int kGroupMax = 4;
constexpr int kTileN = 128;          // weight columns per tile (MMA M)
constexpr int kSubK = 64;            // k elements per swizzle row (128 bytes of 16-bit data)
constexpr int kThreads = 192;        // warps 0-3 epilogue, warp 4 TMA producer, warp 5 MMA issuer
constexpr int kThreadsW8 = 448;      // ... plus warps 6-13: int8 -> 16-bit converters
constexpr unsigned long long kTimeoutNs = 2000000000ull;  // budget of one launch for all of its waits

struct Params {
  int m, k;
  int m_tile;            // MMA N: multiple of 16, 16..256
  int m_tiles;           // ceil(m / m_tile)
  int count;             // contractions sharing lhs
  int tile_begin[kGroupMax + 1];  // prefix sums of (n tiles * m tiles) over the group; an n tile is 128 * NH columns
  void* out[kGroupMax];
  long long n[kGroupMax];
  long long ldo[kGroupMax];       // out row stride in elements
  int kblocks;           // ceil(k / (64 * SUB))
  long long units;       // tiles * kblocks
  int max_contrib;       // partial slots per tile
  float* partials;       // [tiles][max_contrib][m_tile][128 * NH]
  unsigned* counters;    // [tiles], zero before the first launch, left zero by every launch
  int* error_flag;
  int stages;
  int is_bf16;
  int rhs_k_major;       // 1: rhs is [n, k] with k contiguous
  int rhs_3d;            // rhs [k, n] with n % 64 == 0: one copy per stage through a 3-d view {64 n, k, n / 64}
  int early_rhs;         // rhs copies may start before the preceding kernel of the stream has finished
  int whole_tiles;       // 1: CTA b owns tiles [b*T/G, (b+1)*T/G) completely instead of an equal share of units
  const void* scale[kGroupMax];  // W8: f16 scale per weight column
#ifdef PJRTX_UMMA_TIMESTAMPS
  unsigned long long* stamps;  // [grid][16] nanosecond timestamps of the phases (measurement builds only)
#endif
};

struct Maps {
  // [k, n]: dims {n, k}, box {64, 64*SUB}, or (rhs_3d) dims {64, k, n/64}, box {64, 64*SUB, 2*NH};
  // [n, k]: dims {k, n}, box {64, 128}
  CUtensorMap rhs[kGroupMax];
  CUtensorMap lhs;             // dims {k, m}, box {64, m_tile}
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
// Deadline of the launch (every thread reads the timer when it starts) and the CTA's abort word in shared memory.
struct WaitBudget {
  unsigned long long deadline;
  volatile int* abort;
};
// Bounded by time: gives up when the launch's deadline has passed or another thread of the CTA already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, const WaitBudget& w) {
  for (unsigned spin = 0;; spin++) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 15) == 15) {
      if (*w.abort) return false;
      if (global_timer_ns() > w.deadline) {
        *w.abort = 1;
        return false;
      }
    }
  }
}
// x = innermost coordinate (always a multiple of 64 elements here, i.e. 128 bytes), y = outer coordinate.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   smem_dst),
               "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_dst),
      "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ unsigned arrive_acq_rel(unsigned* counter) {
  unsigned old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(counter) : "memory");
  return old;
}
// AND of a predicate over the 128 epilogue threads (named barrier 1), so that all four warps take the same branch
// around the warp-collective TMEM loads and the named barriers that follow.
__device__ __forceinline__ bool epilogue_all(bool ok) {
  unsigned out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "bar.red.and.pred q, 1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(out)
      : "r"((unsigned)ok)
      : "memory");
  return out != 0;
}

// Shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets in 16-byte units,
// descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc(uint32_t smem_addr, uint32_t leading_bytes, uint32_t stride_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3fff);
  d |= (uint64_t)((leading_bytes >> 4) & 0x3fff) << 16;
  d |= (uint64_t)((stride_bytes >> 4) & 0x3fff) << 32;
  d |= (uint64_t)1 << 46;  // version
  d |= (uint64_t)2 << 61;  // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16: f32 accumulate, B (activations) K-major.
__host__ __device__ inline uint32_t instr_desc(int is_bf16, int mma_n, int a_mn_major) {
  uint32_t d = 0;
  d |= 1u << 4;                                // D format f32
  d |= (uint32_t)(is_bf16 ? 1 : 0) << 7;       // A format
  d |= (uint32_t)(is_bf16 ? 1 : 0) << 10;      // B format
  d |= (uint32_t)(a_mn_major ? 1 : 0) << 15;   // A major: MN (weights [k, n]) or K (weights [n, k])
  d |= (uint32_t)(mma_n >> 3) << 17;
  d |= (uint32_t)(kTileN >> 4) << 24;
  return d;
}

__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
      :
      : "r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// A stage of the ring: the weight operand tile (16-bit, swizzled) and the activation tile. With int8 weights a stage
// holds the activation tile and the raw bytes (half the size, so the ring is deeper and more bytes are in flight), and
// the 16-bit operand tiles the converters write live in kOperandSlots slots of their own in front of the ring.
constexpr int kOperandSlots = 3;
__host__ __device__ inline size_t operand_bytes(int sub, int nh) { return (size_t)sub * nh * 16384; }
__host__ __device__ inline size_t stage_bytes(int m_tile, int sub, int nh, bool w8 = false) {
  return (size_t)sub * ((size_t)m_tile * 128 + (size_t)nh * (w8 ? 8192 : 16384));
}
inline size_t smem_bytes(int stages, int m_tile, int sub, int nh, bool w8 = false) {
  // stages (every block 1024-byte aligned: m_tile is a multiple of 16, so m_tile * 128 is a multiple of 2048) +
  // barriers and flags + slack for aligning the dynamic segment to 1024 bytes
  return (size_t)stages * stage_bytes(m_tile, sub, nh, w8) + (w8 ? kOperandSlots * operand_bytes(sub, nh) : 0) + 1024 + 512;
}

struct Cursor {
  int tile, kb;
  int group, n_tile, m_idx;
};
__device__ __forceinline__ void locate_tile(const Params& p, Cursor* c) {
  int g = 0;
#pragma unroll
  for (int q = 1; q < kGroupMax; q++)
    if (q < p.count && c->tile >= p.tile_begin[q]) g = q;
  c->group = g;
  const int t = c->tile - p.tile_begin[g];
  c->n_tile = t / p.m_tiles;
  c->m_idx = t - c->n_tile * p.m_tiles;
}
__device__ __forceinline__ Cursor cursor_at(const Params& p, long long u) {
  Cursor c;
  c.tile = (int)(u / p.kblocks);
  c.kb = (int)(u - (long long)c.tile * p.kblocks);
  locate_tile(p, &c);
  return c;
}
__device__ __forceinline__ void advance(const Params& p, Cursor* c) {
  if (++c->kb == p.kblocks) {
    c->kb = 0;
    c->tile++;
    locate_tile(p, c);
  }
}

// SUB: 64-deep k sub-blocks per stage (1 or 2). NH: 128-column halves per tile (1 or 2); two halves make every weight
// row of a stage 512 contiguous bytes in memory and take two accumulators per tile (so m_tile <= 128).
#ifdef PJRTX_UMMA_TIMESTAMPS
#define PJRTX_STAMP(slot) (p.stamps[(size_t)blockIdx.x * 16 + (slot)] = global_timer_ns())
#else
#define PJRTX_STAMP(slot) ((void)0)
#endif

template <int SUB, int NH, bool W8 = false>
__global__ void __launch_bounds__(W8 ? kThreadsW8 : kThreads, 1) umma_stream_kernel(const Params p, const __grid_constant__ Maps maps) {
  extern __shared__ unsigned char smem_dyn[];
  // 128-byte swizzled tiles need 1024-byte aligned bases.
  const uint32_t base = (smem_u32(smem_dyn) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_dyn + (base - smem_u32(smem_dyn));
  const uint32_t per_stage = (uint32_t)stage_bytes(p.m_tile, SUB, NH, W8);
  constexpr uint32_t a_bytes = NH * SUB * 16384u;  // one 16-bit weight operand tile
  // Without int8 weights a stage is [operand tile][activation tile]. With them the operand slots come first, then the
  // ring of [activation tile][raw bytes] stages.
  const uint32_t ring = base + (W8 ? kOperandSlots * a_bytes : 0u);
  unsigned char* ring_ptr = base_ptr + (W8 ? kOperandSlots * a_bytes : 0u);
  const uint32_t lhs_offset = W8 ? 0u : a_bytes;
  const uint32_t raw_offset = (uint32_t)SUB * p.m_tile * 128u;  // W8: raw bytes behind the activation tile
  constexpr int TW = kTileN * NH;  // tile width in weight columns
  uint64_t* full = reinterpret_cast<uint64_t*>(ring_ptr + (size_t)p.stages * per_stage);
  uint64_t* empty = full + p.stages;
  uint64_t* acc_full = empty + p.stages;   // [2]
  uint64_t* acc_empty = acc_full + 2;      // [2]
  uint64_t* ready = acc_empty + 2;         // [kOperandSlots], W8: the converters have written the slot's operand tile
  uint64_t* slot_empty = ready + 4;        // [kOperandSlots], W8: the MMAs that read the slot have completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(slot_empty + 4);
  int* flags = reinterpret_cast<int*>(tmem_slot + 1);  // [0] is_last of a fold, [1] abort
  const WaitBudget budget{global_timer_ns() + kTimeoutNs, flags + 1};

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) PJRTX_STAMP(0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // Equal shares of units; with `whole_tiles` equal shares of tiles (no tile is split, nothing to fold).
  const long long tiles_total = p.units / p.kblocks;
  const long long u_begin = p.whole_tiles ? ((long long)blockIdx.x * tiles_total / gridDim.x) * p.kblocks
                                          : (long long)blockIdx.x * p.units / gridDim.x;
  const long long u_end = p.whole_tiles ? ((long long)(blockIdx.x + 1) * tiles_total / gridDim.x) * p.kblocks
                                        : (long long)(blockIdx.x + 1) * p.units / gridDim.x;
  const int count = (int)(u_end - u_begin);
  // Two accumulator sets of NH x m_tile f32 columns; the allocation is a power of two >= 32 columns.
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < 2 * NH * p.m_tile) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; s++) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < kOperandSlots; s++) {
      mbar_init(&ready[s], (kThreadsW8 - kThreads) / 32);
      mbar_init(&slot_empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);
    }
    flags[0] = 0;
    flags[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) PJRTX_STAMP(1);

  if (warp == 4) {
    // ---- TMA producer ------------------------------------------------------------------------------------------
    if (lane == 0 && count > 0) {
      // bytes the copies of one stage deliver: weight tile (16-bit, or raw bytes with int8 weights) + activation tile
      const unsigned tx = per_stage;
      auto load_rhs = [&](const Cursor& c, int stage) {
        const uint32_t st = ring + (uint32_t)stage * per_stage;
        const int k0 = c.kb * (kSubK * SUB), n0 = c.n_tile * TW;
        if (W8) {
          // Raw bytes [64 * SUB k rows][128 columns] per half, unswizzled.
#pragma unroll
          for (int h = 0; h < NH; h++) tma_load_2d(st + raw_offset + h * (SUB * 8192u), &maps.rhs[c.group], n0 + h * kTileN, k0, &full[stage]);
          return;
        }
        if (p.rhs_3d) {
          // Blocks of 64 columns are the outer coordinate: the box lands as [column block][k row][128 bytes], which
          // is the layout the two-box form produces, in one copy of 16 * SUB * NH KiB.
          tma_load_3d(st, &maps.rhs[c.group], 0, k0, n0 / 64, &full[stage]);
          return;
        }
#pragma unroll
        for (int h = 0; h < NH; h++) {
          const uint32_t sh = st + h * (SUB * 16384u);
          if (p.rhs_k_major) {
#pragma unroll
            for (int s = 0; s < SUB; s++)
              tma_load_2d(sh + s * 16384u, &maps.rhs[c.group], k0 + s * kSubK, n0 + h * kTileN, &full[stage]);
          } else {
            tma_load_2d(sh, &maps.rhs[c.group], n0 + h * kTileN, k0, &full[stage]);
            tma_load_2d(sh + SUB * 8192u, &maps.rhs[c.group], n0 + h * kTileN + 64, k0, &full[stage]);
          }
        }
      };
      auto load_lhs = [&](const Cursor& c, int stage) {
        const uint32_t st = ring + (uint32_t)stage * per_stage + lhs_offset;
        const int k0 = c.kb * (kSubK * SUB);
#pragma unroll
        for (int s = 0; s < SUB; s++)
          tma_load_2d(st + (uint32_t)s * p.m_tile * 128u, &maps.lhs, k0 + s * kSubK, c.m_idx * p.m_tile, &full[stage]);
      };
      Cursor cur = cursor_at(p, u_begin);
      int first = count < p.stages ? count : p.stages;
      if (p.early_rhs) {
        // Weights first for the whole first ring, then wait for the predecessor, then the activations.
        Cursor c2 = cur;
        for (int i = 0; i < first; i++) {
          mbar_expect_tx(&full[i], tx);
          load_rhs(c2, i);
          advance(p, &c2);
        }
        asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int i = 0; i < first; i++) {
          load_lhs(cur, i);
          advance(p, &cur);
        }
      } else {
        asm volatile("griddepcontrol.wait;" ::: "memory");
        first = 0;
      }
      PJRTX_STAMP(2);
      int stage = first % p.stages;
      unsigned phase = first == p.stages ? 1 : 0;
      for (int i = first; i < count; i++) {
        if (i >= p.stages && !mbar_wait(&empty[stage], phase ^ 1, budget)) {
          atomicExch(p.error_flag, 11);
          break;
        }
        mbar_expect_tx(&full[stage], tx);
        load_rhs(cur, stage);
        load_lhs(cur, stage);
        advance(p, &cur);
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp == 5) {
    // ---- MMA issuer ----------------------------------------------------------------------------------------------
    if (lane == 0 && count > 0) {
      const uint32_t idesc = instr_desc(p.is_bf16, p.m_tile, !p.rhs_k_major);
      int stage = 0;
      unsigned phase = 0;
      int slot = 0;            // W8: operand slot of this unit
      unsigned slot_phase = 0;
      int seg = 0;
      Cursor cur = cursor_at(p, u_begin);
      int cur_tile = -1;
      bool fresh = true;
      uint32_t acc = tmem_base;
      for (int i = 0; i < count; i++) {
        if (cur.tile != cur_tile) {
          // New tile segment: take the next accumulator once the epilogue has drained its previous use.
          cur_tile = cur.tile;
          const int buf = seg & 1;
          if (seg >= 2 && !mbar_wait(&acc_empty[buf], ((seg >> 1) & 1) ^ 1, budget)) {
            atomicExch(p.error_flag, 14);
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          acc = tmem_base + (uint32_t)(buf * NH * p.m_tile);
          fresh = true;
        }
        // The activation tile of the stage has landed; with int8 weights the converters have also filled the slot.
        if (!mbar_wait(&full[stage], phase, budget) || (W8 && !mbar_wait(&ready[slot], slot_phase, budget))) {
          atomicExch(p.error_flag, 12);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (i == 0) PJRTX_STAMP(3);
        const uint32_t st = ring + (uint32_t)stage * per_stage;
        const uint32_t weights = W8 ? base + (uint32_t)slot * a_bytes : st;
#pragma unroll
        for (int kk = 0; kk < 4 * SUB; kk++) {
          const uint64_t b_desc = smem_desc(st + lhs_offset + (uint32_t)(kk >> 2) * p.m_tile * 128u + (kk & 3) * 32u, 16, 1024);
#pragma unroll
          for (int h = 0; h < NH; h++) {
            const uint32_t sh = weights + h * (SUB * 16384u);
            uint64_t a_desc;
            if (p.rhs_k_major) {
              // A K-major like B: 64-k sub-blocks 16 KiB apart, 32 bytes per 16-k step inside the swizzled row.
              a_desc = smem_desc(sh + (kk >> 2) * 16384u + (kk & 3) * 32u, 16, 1024);
            } else {
              // A MN-major: 16 k rows = two 1024-byte swizzle atoms further down; the two 64-column boxes are
              // SUB * 8192 bytes apart (leading offset), 8-row groups 1024 bytes apart (stride offset).
              a_desc = smem_desc(sh + kk * 2048u, SUB * 8192u, 1024);
            }
            mma_f16(acc + (uint32_t)(h * p.m_tile), a_desc, b_desc, idesc, (fresh && kk == 0) ? 0u : 1u);
          }
        }
        fresh = false;
        mma_commit(&empty[stage]);  // the stage is free once these MMAs have read it
        if (W8) {
          mma_commit(&slot_empty[slot]);  // and so is the operand slot
          if (++slot == kOperandSlots) {
            slot = 0;
            slot_phase ^= 1;
          }
        }
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1;
        }
        advance(p, &cur);
        if (i + 1 == count || cur.tile != cur_tile) {
          mma_commit(&acc_full[seg & 1]);
          seg++;
          if (i + 1 == count) PJRTX_STAMP(4);
        }
      }
    }
  } else if (W8 && warp >= 6) {
    // ---- converters (warps 6-13): raw s8 tile -> swizzled 16-bit operand tile ----------------------------------------
    // Thread t owns the 16 columns nc * 16 .. + 15 (nc = t % 8) of rows t / 8, t / 8 + 32, ... : one 16-byte read of
    // raw bytes per row, two 16-byte writes of eight 16-bit values each at their swizzled places. The values written
    // are the integers themselves (exact in f16 and bf16); the column scales multiply the accumulators.
    if (count > 0) {
      const int t = threadIdx.x - kThreads;
      const int nc = t & 7, row0 = t >> 3;
      constexpr int ROWS = 2 * SUB;  // rows per thread and half: 64 * SUB rows over 32 row slots
      int stage = 0, slot = 0;
      unsigned phase = 0, slot_phase = 0;
      for (int i = 0; i < count; i++) {
        // The raw bytes have landed, and the MMAs that read this slot's previous tile have completed.
        if (!mbar_wait(&full[stage], phase, budget) || (i >= kOperandSlots && !mbar_wait(&slot_empty[slot], slot_phase ^ 1, budget))) {
          if (lane == 0) atomicExch(p.error_flag, 15);
          break;
        }
        const unsigned char* st = ring_ptr + (size_t)stage * per_stage;
        unsigned char* operand = base_ptr + (size_t)slot * a_bytes;
#pragma unroll
        for (int h = 0; h < NH; h++) {
          const unsigned char* raw = st + raw_offset + h * (SUB * 8192u) + row0 * 128 + nc * 16;
          unsigned char* dst = operand + h * (SUB * 16384u) + (nc >> 2) * (SUB * 8192u);
          uint4 q[ROWS];  // every row of this thread is requested before the first is converted
#pragma unroll
          for (int r = 0; r < ROWS; r++) q[r] = *reinterpret_cast<const uint4*>(raw + r * 32 * 128);
#pragma unroll
          for (int r = 0; r < ROWS; r++) {
            const int k = row0 + 32 * r;
            const uint32_t words[4] = {q[r].x, q[r].y, q[r].z, q[r].w};
            uint32_t packed[8];
#pragma unroll
            for (int w = 0; w < 4; w++) {
              if (p.is_bf16) {
                // b = low7 - 128 * sign. {0x43, low7} is the bf16 128 + low7 and {0x43, sign << 7} is 128 or 256:
                // their difference is b, exactly.
                const uint32_t low7 = words[w] & 0x7f7f7f7fu, sign = words[w] & 0x80808080u;
#pragma unroll
                for (int e = 0; e < 2; e++) {
                  const uint32_t sel = e ? 0x4342 : 0x4140;
                  const uint32_t x = __byte_perm(low7, 0x43434343u, sel), y = __byte_perm(sign, 0x43434343u, sel);
                  const __nv_bfloat162 v = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&x), *reinterpret_cast<const __nv_bfloat162*>(&y));
                  packed[w * 2 + e] = *reinterpret_cast<const uint32_t*>(&v);
                }
              } else {
                // {0x64, b + 128} is the f16 1024 + 128 + b.
                const uint32_t flipped = words[w] ^ 0x80808080u;
                const __half2 bias = __float2half2_rn(1152.0f);
#pragma unroll
                for (int e = 0; e < 2; e++) {
                  const uint32_t x = __byte_perm(flipped, 0x64646464u, e ? 0x4342 : 0x4140);
                  const __half2 v = __hsub2(*reinterpret_cast<const __half2*>(&x), bias);
                  packed[w * 2 + e] = *reinterpret_cast<const uint32_t*>(&v);
                }
              }
            }
            const int cc = (nc & 3) * 2;  // first of this thread's two 16-byte column chunks inside the 64-column box
            *reinterpret_cast<uint4*>(dst + k * 128 + (((cc) ^ (k & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            *reinterpret_cast<uint4*>(dst + k * 128 + (((cc + 1) ^ (k & 7)) << 4)) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
          }
        }
        // The tile was written through the generic proxy; the tensor core reads it through the async proxy.
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&ready[slot]);
        if (++slot == kOperandSlots) {
          slot = 0;
          slot_phase ^= 1;
        }
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else if (warp < 4) {
    // ---- epilogue warps 0..3: TMEM lane quarter = warp index ------------------------------------------------------
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (count > 0) {
      const int first_tile = (int)(u_begin / p.kblocks);
      const int last_tile = (int)((u_end - 1) / p.kblocks);
      const int n_local = warp * 32 + lane;
      int seg = 0;
      for (int tile = first_tile; tile <= last_tile; tile++, seg++) {
        Cursor c;
        c.tile = tile;
        c.kb = 0;
        locate_tile(p, &c);
        const int buf = seg & 1;
        // One decision for all four warps: tcgen05.ld is warp-collective and named barriers follow.
        const bool ok = epilogue_all(mbar_wait(&acc_full[buf], (seg >> 1) & 1, budget));
        if (!ok) {
          if (threadIdx.x == 0) atomicExch(p.error_flag, 13);
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (threadIdx.x == 0 && tile == last_tile) PJRTX_STAMP(5);
        // CTA that owns unit u: the largest b with b*units/grid <= u, i.e. ceil((u+1)*grid/units) - 1.
        const long long tile_units_begin = (long long)tile * p.kblocks;
        const long long first_cta = ((tile_units_begin + 1) * gridDim.x + p.units - 1) / p.units - 1;
        const long long last_cta = ((tile_units_begin + p.kblocks) * gridDim.x + p.units - 1) / p.units - 1;
        const int contributors = p.whole_tiles ? 1 : (int)(last_cta - first_cta + 1);
        const long long n_total = p.n[c.group];
        const long long n_first = (long long)c.n_tile * TW + n_local;  // this thread's column in half 0
        const int m0 = c.m_idx * p.m_tile;
        const long long ldo = p.ldo[c.group];
        float* slot = p.partials + (((long long)tile * p.max_contrib + (blockIdx.x - first_cta)) * p.m_tile) * TW;
        const int m_rows = min(p.m_tile, p.m - m0);  // rows of this tile that exist
#pragma unroll
        for (int h = 0; h < NH; h++) {
          const long long n = n_first + h * kTileN;
          // Int8 weights: the tensor core contracted the integers; this thread's column scale finishes the product.
          const float scale = W8 ? (n < n_total ? __half2float(static_cast<const __half*>(p.scale[c.group])[n]) : 0.f) : 1.f;
          const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)((buf * NH + h) * p.m_tile);
          for (int c0 = 0; c0 < m_rows; c0 += 16) {
            uint32_t r[16];
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                  "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                : "r"(taddr + (uint32_t)c0));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (W8) {
#pragma unroll
              for (int j = 0; j < 16; j++) r[j] = __float_as_uint(__uint_as_float(r[j]) * scale);
            }
            if (contributors > 1) {
#pragma unroll
              for (int j = 0; j < 16; j++)
                if (c0 + j < m_rows) slot[(c0 + j) * TW + h * kTileN + n_local] = __uint_as_float(r[j]);
            } else if (n < n_total) {
#pragma unroll
              for (int j = 0; j < 16; j++) {
                const int m = m0 + c0 + j;
                if (c0 + j < m_rows) {
                  const float v = __uint_as_float(r[j]);
                  if (p.is_bf16) static_cast<__nv_bfloat16*>(p.out[c.group])[(long long)m * ldo + n] = __float2bfloat16_rn(v);
                  else static_cast<__half*>(p.out[c.group])[(long long)m * ldo + n] = __float2half_rn(v);
                }
              }
            }
          }
        }
        // The accumulator is in registers / memory now: hand it back to the MMA lane.
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[buf]);
        if (contributors > 1) {
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (threadIdx.x == 0 && tile == last_tile) PJRTX_STAMP(6);
          if (threadIdx.x == 0) flags[0] = arrive_acq_rel(&p.counters[tile]) == (unsigned)contributors - 1;
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (threadIdx.x == 0 && tile == last_tile) PJRTX_STAMP(7);
          if (flags[0]) {
            if (threadIdx.x == 0) PJRTX_STAMP(10);
            const float* first_slot = p.partials + ((long long)tile * p.max_contrib * p.m_tile) * TW;
            const long long slot_stride = (long long)p.m_tile * TW;
            // (Thirty-two rows at a time - 128 loads in flight, 239 registers - measured the same within noise.)
            constexpr int kFoldRows = 16;
            // Sixteen rows at a time, all their loads issued before the adds; contributors are added in CTA order.
#pragma unroll
            for (int h = 0; h < NH; h++) {
              const long long n = n_first + h * kTileN;
              for (int r0 = 0; r0 < m_rows; r0 += kFoldRows) {
                float t[kFoldRows];
#pragma unroll
                for (int j = 0; j < kFoldRows; j++) t[j] = 0.f;
                // Four contributors' rows are requested at once (64 loads in flight per thread: the fold of a tile
                // with fifteen contributors is a quarter of a megabyte through one CTA, so its time is round trips),
                // then added in CTA order. (A fold shared by the contributors - every CTA waits until the tile's
                // partials are all published, then adds a slice of the rows with one round of loads - was measured
                // slower: 2.80 against 2.23 ms for the 81 contractions of twenty 70B-shape layers cut eight ways,
                // 1.57 against 1.31 ms for eight 8B-width layers at 32 rows.)
                int q = 0;
                for (; q + 4 <= contributors; q += 4) {
                  float v[4][kFoldRows];
#pragma unroll
                  for (int e = 0; e < 4; e++) {
                    const float* src = first_slot + (long long)(q + e) * slot_stride + r0 * TW + h * kTileN + n_local;
#pragma unroll
                    for (int j = 0; j < kFoldRows; j++) v[e][j] = (r0 + j < m_rows) ? __ldcg(src + j * TW) : 0.f;
                  }
#pragma unroll
                  for (int e = 0; e < 4; e++)
#pragma unroll
                    for (int j = 0; j < kFoldRows; j++) t[j] += v[e][j];
                }
                for (; q < contributors; q++) {
                  const float* src = first_slot + (long long)q * slot_stride + r0 * TW + h * kTileN + n_local;
                  float v[kFoldRows];
#pragma unroll
                  for (int j = 0; j < kFoldRows; j++) v[j] = (r0 + j < m_rows) ? __ldcg(src + j * TW) : 0.f;
#pragma unroll
                  for (int j = 0; j < kFoldRows; j++) t[j] += v[j];
                }
                if (n < n_total) {
#pragma unroll
                  for (int j = 0; j < kFoldRows; j++) {
                    if (r0 + j < m_rows) {
                      const long long at = (long long)(m0 + r0 + j) * ldo + n;
                      if (p.is_bf16) static_cast<__nv_bfloat16*>(p.out[c.group])[at] = __float2bfloat16_rn(t[j]);
                      else static_cast<__half*>(p.out[c.group])[at] = __float2half_rn(t[j]);
                    }
                  }
                }
              }
            }
            if (threadIdx.x == 0) p.counters[tile] = 0;
            if (threadIdx.x == 0) PJRTX_STAMP(12);
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if (threadIdx.x == 0) PJRTX_STAMP(8);
  }
  __syncthreads();
  if (threadIdx.x == 0) PJRTX_STAMP(9);
  if (warp == 5) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

}  // namespace umma
}  // namespace pjrtx

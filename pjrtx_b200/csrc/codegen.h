// Fusion-group code generator: turns a run of fusible plan instructions into
// one CUDA C++ kernel for sm_100a.
//
// The reference generates one Metal kernel per view+elementwise fusion group by
// writing every group output as a scalar expression of the group inputs with
// index substitution for broadcast/slice/reshape/transpose
// (src/backend/mlx_metal/executable_metal_graph_fusion_request_writer.zig:9-55,
//  executable_metal_graph_map_rules.zig:167-220,
//  executable_metal_graph_fusion_expression.zig:56-130), and separate kernels
// for reductions (executable_metal_graph_reduction.zig:12-323). This generator
// keeps the "expression per output element with index substitution" idea and
// extends it: suffix-axis reductions (sum/max/min/and/or and the two-operand
// max-with-index form) join the group as row stages, so RMSNorm, softmax and
// argmax each become a single kernel that reads its inputs with 128-bit loads,
// reduces with warp shuffles + shared memory and keeps every intermediate in
// registers. iota, concatenate, dynamic_slice, reverse and the embedding form
// of gather are expression operators too.
#pragma once

#include <set>
#include <string>
#include <vector>

#include "plan.h"

namespace pjrtx {

struct FusedKernel {
  std::string name;
  std::string source;             // complete translation unit
  std::vector<uint32_t> inputs;   // external values, kernel pointer params in this order
  std::vector<uint32_t> outputs;  // stored values, pointer params after the inputs
  std::vector<uint32_t> scatter_dst;  // results of in-place slice updates done by the kernel, pointer params after the outputs
  bool row = false;               // true: one CTA per row with reduce stages
  int64_t rows = 1, cols = 1;     // row kernel iteration space
  int64_t n = 0;                  // map kernel element count
  int vec = 1;
  int block = 256;
  int64_t grid = 1;
  int stages = 1;
  int reduce_count = 0;
};

// True when the kind can take part in a generated kernel.
bool codegen_fusible(const Plan& plan, const Instruction& ins);

// Generates the kernel for `nodes` (ascending instruction indices). `outputs`
// are the values that must be stored. `scatters` are dynamic_update_slice
// instructions among the nodes whose operand storage is updated in place: the
// kernel computes the update and stores it at the (clamped) start indices.
// Returns false with a reason when the run cannot be expressed as one kernel
// (the planner then shortens the run).
bool generate_fused_kernel(const Plan& plan, const std::vector<size_t>& nodes,
                           const std::vector<uint32_t>& outputs, const std::vector<size_t>& scatters, int sm_count,
                           FusedKernel* out, std::string* why);

}  // namespace pjrtx

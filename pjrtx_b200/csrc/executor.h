// Compiled executable: legalization, kernel planning and per-step execution.
//
// Mirrors the reference's compile → execute pair
//   src/backend/mlx_metal/executable_compile.zig:17-108   (legalize, build program, upload constants)
//   src/backend/mlx_metal/execution_call.zig:66-145        (argument checks, run schedule, wrap outputs)
//   src/backend/mlx_metal/executable_stats.zig:6-56        (counters)
// with a different execution strategy: the schedule is lowered once, at compile
// time, into a list of kernel steps (generated fusion kernels, streaming /
// tiled contractions, in-place slice updates, attention, collectives) whose
// intermediates live in one liveness-planned arena, and the whole step list is
// replayed as a CUDA graph.
#pragma once

#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "codegen.h"
#include "device.h"
#include "kernels/kernels.h"
#include "plan.h"
#include "program.h"

namespace pjrtx {

struct ExecutableStats {
  uint64_t resident_constant_count = 0, resident_constant_bytes = 0;
  uint64_t program_value_count = 0, program_node_count = 0, program_edge_count = 0;
  uint64_t program_schedule_item_count = 0, program_subprogram_count = 0, program_control_flow_count = 0;
  uint64_t program_fusion_group_count = 0, program_materialization_boundary_count = 0;
  uint64_t program_planned_release_count = 0, program_planned_release_bytes = 0;
  uint64_t program_peak_live_value_count = 0, program_peak_live_bytes = 0;
  uint64_t program_device_count = 0;
  uint64_t last_execute_device_index = UINT64_MAX;
  int32_t last_execute_local_hardware_id = -1;
  uint64_t execute_count = 0;
  uint64_t compiled_program_execute_count = 0, compiled_program_output_count = 0;
  uint64_t captured_program_execute_count = 0, captured_program_dynamic_input_count = 0;
  uint64_t captured_program_captured_input_count = 0;
  uint64_t donation_alias_output_count = 0, donation_alias_output_bytes = 0;
  uint64_t fusion_group_execute_count = 0;
  uint64_t execute_wall_us_total = 0, execute_wall_us_peak = 0;
  // Additions describing the kernel plan.
  uint64_t kernel_step_count = 0;        // launches per execute
  uint64_t generated_kernel_count = 0;   // fusion kernels compiled
  uint64_t arena_bytes = 0, scratch_bytes = 0;
  uint64_t graph_capture_count = 0, graph_launch_count = 0;
  uint64_t kernel_launch_total = 0;      // kernels enqueued since compile
  // Profiling: what two event records with nothing between them read in the latest profiled execution - the part of
  // every step time that is the measurement's, not the kernel's (0 before the first profiled execution).
  uint64_t profile_event_gap_ns = 0;
};

// One segment of a chained streaming contraction (kernels.h, DotChainSegment): a group of contractions sharing an
// lhs, with the lhs transform and the residuals the planner folded into it. Values are storage-class roots.
struct DotSeg {
  std::vector<DotShape> group;
  uint32_t lhs = UINT32_MAX, lhs2 = UINT32_MAX;
  DotLhs lhs_desc;
  std::vector<uint32_t> rhs, out, residual;  // per contraction; residual UINT32_MAX = none
};

struct Step {
  enum Type { kFused, kDot, kSliceUpdate, kSdpa, kAllReduce, kAllGather, kCopy, kAttnDecode, kAttnPrefill } type = kFused;
  std::vector<size_t> nodes;        // plan instructions this step covers
  std::vector<uint32_t> inputs;     // root values read
  std::vector<uint32_t> outputs;    // root values written
  FusedKernel fused;
  JitKernel* jit = nullptr;
  DotShape dot;
  std::vector<DotShape> dot_group;  // more than one entry: contractions sharing inputs[0], launched together
  std::vector<uint32_t> dot_scales; // int8 weights: the f16 column scales, one per contraction (parameters / constants)
  DotScratch dot_scratch;
  // Non-empty: the step runs as one launch of the chained streaming kernel (dot / dot_group describe its first segment).
  std::vector<DotSeg> segs;
  DotChainPlan chain_plan;
  uint64_t scratch_offset = 0, counter_offset = 0;
  SliceUpdateShape dus;
  bool in_place = false;
  bool early_rhs = false;  // every rhs of the contraction is a parameter or constant no step writes
  bool early_kv = false;   // decode attention: cache rows below the token index are not written earlier in the step
  SdpaShape sdpa;
  AttnDecodeShape attn;
  AttnDecodePlan attn_plan;
  AttnPrefillShape attn_prefill;
  uint64_t bytes = 0;  // kCopy / collectives
  uint64_t count = 0;
  int dtype = 0;
};

struct Storage {
  enum Kind { kNone, kParameter, kConstant, kArena, kFresh } kind = kNone;
  uint64_t offset = 0;      // arena
  uint32_t index = 0;       // parameter index / constant slot
};

struct Executable;

// Runs legalization only; "" when the plan can be compiled, otherwise one line
//   invalid executable plan: pass=b200-backend-legalization [instruction=N] [op=<kind>] ... detail="..." feature=<label>
// (format of src/backend/mlx_metal/lowering_diagnostic.zig:31-45).
std::string lowering_diagnostic(const Plan& plan, size_t device_count);

// Kernel plan without touching a device: used by the introspection entry point.
std::string describe_kernel_plan(const Plan& plan, std::string* error);

Executable* compile_executable(const Plan& plan, const std::vector<int>& device_ordinals, std::string* error);
bool execute_executable(Executable* exe, size_t device_index, Buffer* const* args, size_t nargs,
                        std::vector<Buffer*>* outputs, std::string* error);
ExecutableStats executable_stats(Executable* exe);
// Device ordinals the executable was compiled for, in device-index order.
std::vector<int> executable_device_ordinals(Executable* exe);
// Per-step device times: when enabled, the next executions run the step list directly (no graph replay) with a
// CUDA event pair around every step; step_times returns the durations of the latest such execution in
// milliseconds, in step order (the reference prints the same information as `backend_schedule_item` profile
// events, src/backend/mlx_metal/profiling_writer.zig:160).
void executable_set_profiling(Executable* exe, bool enabled);
std::vector<float> executable_step_times(Executable* exe);
std::string executable_describe(Executable* exe);
void destroy_executable(Executable* exe);

// Custom-call registry (src/backend/mlx_metal/custom_call.zig): named targets
// that lower to an elementwise kind or to identity.
bool register_custom_call(const std::string& target, const std::string& op_name, int arity);
void unregister_custom_call(const std::string& target);
uint64_t custom_call_registry_version();

}  // namespace pjrtx

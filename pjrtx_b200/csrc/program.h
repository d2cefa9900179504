// Backend program graph built from an executable plan: nodes, producer→consumer
// edges, greedy contiguous view+elementwise fusion groups, the schedule over
// {node, fusion_group, materialization_boundary} items, and liveness statistics.
//
// Restates (structure, not code) the reference's
//   src/backend/mlx_metal/program.zig:22-250         (vocabulary)
//   src/backend/mlx_metal/program_build.zig:10-263   (classification + grouping)
//   src/backend/mlx_metal/program_fusion.zig:8-70    (group boundary values)
//   src/backend/mlx_metal/program_schedule_build.zig:6-51
//   src/backend/mlx_metal/program_liveness.zig:10-150
// so that the counters the reference's tests assert come out identical.
#pragma once

#include <string>
#include <vector>

#include "plan.h"

namespace pjrtx {

enum class NodeKind : int {
  constant, parameter, structural, view, elementwise, reduction, matmul, control_flow,
  library_call, materialize, collective
};
const char* node_kind_name(NodeKind k);

struct Node {
  size_t instruction_index = 0;
  NodeKind kind = NodeKind::materialize;
  std::vector<uint32_t> inputs;
  std::vector<uint32_t> outputs;
  bool materializes = true;
  long fusion_group = -1;
};

struct FusionGroup {
  size_t id = 0;
  size_t first_node = 0, last_node = 0, node_count = 0;
  std::vector<size_t> node_indices;
  std::vector<uint32_t> input_values;   // enter from parameters or outside producers
  std::vector<uint32_t> output_values;  // leave to outside consumers or a boundary
};

struct ProgramValue {
  uint32_t value_id = 0;
  uint64_t byte_size = 0;
  long producer_node = -1;
  long last_use_node = -1;
  bool is_output = false;
  long materialization_boundary = -1;
};

struct Edge {
  uint32_t value_id;
  size_t from_node, to_node;
};

enum class ScheduleKind : int { node, fusion_group, materialization_boundary };
struct ScheduleItem {
  ScheduleKind kind;
  size_t index;
  size_t count;
};

struct LivenessStats {
  size_t planned_release_count = 0;
  uint64_t planned_release_bytes = 0;
  size_t peak_live_value_count = 0;
  uint64_t peak_live_bytes = 0;
};

struct Program {
  std::vector<ProgramValue> values;
  std::vector<Node> nodes;
  std::vector<Edge> edges;
  std::vector<ScheduleItem> schedule;
  std::vector<FusionGroup> fusion_groups;
  std::vector<uint32_t> materialization_boundaries;  // value ids, reason = pjrt_output
  LivenessStats liveness;
};

NodeKind program_node_kind(Kind k);
bool instruction_materializes(Kind k);
bool program_node_fusible(Kind k);

// Builds and validates the program; on failure returns false and fills `error`
// with a line tagged pass=backend-program-verify.
bool build_program(const Plan& plan, Program* out, std::string* error);
bool validate_program(const Plan& plan, const Program& program, std::string* error);
LivenessStats compute_liveness(const Program& program);

// JSON rendering used by the introspection entry points and the tests.
std::string describe_program(const Program& program);

}  // namespace pjrtx

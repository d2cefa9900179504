// Executable plan: the program contract handed from the compiler to a backend.
//
// C++ restatement of the reference's compiler IR vocabulary:
//   ExecutablePlan / PlanInstruction / Value    src/compiler/executable_plan.zig:9-139
//   PlanInstructionKind                          src/compiler/operation.zig:84-168
//   BufferDescriptor                             src/compiler/tensor.zig:40-49
//   CompileOptions / ShardingPlan                src/compiler/topology.zig:56-91
// The kind order below equals the reference enum order, so the numeric code of a
// kind is its position there; kinds after `unsupported` are additions that only
// the tensor-parallel planner emits (the reference has no collective kind).
#pragma once

#include <map>
#include <string>
#include <vector>

#include "common.h"

namespace pjrtx {

#define PJRTX_KINDS(X)                                                                      \
  X(constant) X(copy_arg0) X(add) X(subtract) X(multiply) X(divide) X(maximum) X(minimum)   \
  X(power) X(atan2) X(remainder) X(and_) X(or_) X(xor_) X(shift_left)                       \
  X(shift_right_arithmetic) X(shift_right_logical) X(negate) X(exp) X(expm1) X(tanh)        \
  X(sqrt) X(rsqrt) X(abs) X(cbrt) X(ceil) X(floor) X(log) X(log1p) X(logistic) X(sine)      \
  X(cosine) X(not_) X(sign) X(is_finite) X(round_nearest_afz) X(round_nearest_even)         \
  X(popcnt) X(count_leading_zeros) X(convert) X(bitcast_convert) X(reshape) X(transpose)    \
  X(broadcast_in_dim) X(slice) X(dynamic_slice) X(dynamic_update_slice) X(pad) X(reverse)   \
  X(concatenate) X(iota) X(gather) X(sort) X(top_k) X(dot_general) X(reduce_sum)            \
  X(reduce_max) X(reduce_min) X(reduce_and) X(reduce_or) X(reduce_window_sum)               \
  X(reduce_window_max) X(compare) X(select) X(clamp) X(cholesky) X(complex) X(convolution)  \
  X(custom_call) X(fft) X(get_tuple_element) X(imag) X(optimization_barrier)                \
  X(partition_id) X(real) X(reduce_precision) X(rng) X(rng_bit_generator) X(scatter)        \
  X(triangular_solve) X(tuple) X(while_) X(unsupported) X(all_reduce) X(all_gather)

enum class Kind : int {
#define X(n) n,
  PJRTX_KINDS(X)
#undef X
      kCount
};

const char* kind_name(Kind k);
Kind kind_from_name(const std::string& name);  // Kind::unsupported when unknown

enum class ValueRole : int { parameter = 0, constant = 1, instruction_result = 2, output = 3 };
enum class ShardingKind : int { replicated = 0, partitioned = 1, manual = 2 };
enum class CompareOp : int { eq = 0, ne = 1, ge = 2, gt = 3, le = 4, lt = 5 };

struct Value {
  uint32_t id = 0;
  ValueRole role = ValueRole::instruction_result;
  int dtype = kInvalid;
  std::vector<int64_t> dims;
  uint64_t bytes() const { return dense_byte_size(dtype, dims); }
  int64_t count() const { return element_count(dims); }
};

// One instruction. Integer-list attributes are stored by the reference's field
// name ("dims", "permutation", "broadcast_dimensions", "start_indices",
// "limit_indices", "strides", "slice_sizes", "dimension", "iota_dimension",
// "reduce_dimensions", "lhs_batch_dimensions", ..., "compare_direction",
// "index_vector_dim", "offset_dims", "collapsed_slice_dims", "start_index_map",
// "edge_padding_low", ...); scalars are one-element lists.
struct Instruction {
  Kind kind = Kind::unsupported;
  std::vector<uint32_t> inputs;
  std::vector<uint32_t> outputs;
  std::map<std::string, std::vector<int64_t>> attrs;
  std::vector<uint8_t> literal;     // constant payload, dense row-major
  std::string custom_call_target;

  bool has(const char* name) const { return attrs.count(name) != 0; }
  const std::vector<int64_t>& list(const char* name) const;
  int64_t scalar(const char* name, int64_t fallback) const;
};

struct Sharding {
  ShardingKind kind = ShardingKind::replicated;
  std::string mesh_name;
  std::vector<int32_t> device_assignment;
  // Extension consumed by the tensor-parallel planner: which tensor dimension
  // is split across partitions (-1 = none). The reference records only `kind`.
  int64_t split_dim = -1;
};

struct OutputAlias {
  uint32_t output_index = 0;
  uint32_t parameter_index = 0;
  int kind = 1;  // 0 identity, 1 donation (src/compiler/executable_plan.zig:40-53)
};

struct Plan {
  int32_t num_replicas = 1;
  int32_t num_partitions = 1;
  bool use_shardy = true;
  std::vector<int32_t> device_assignment;
  std::vector<Value> values;
  std::vector<Instruction> instructions;
  std::vector<Sharding> parameter_shardings;
  std::vector<Sharding> output_shardings;
  std::vector<uint32_t> output_ids;
  std::vector<uint32_t> donated_parameter_indices;
  std::vector<OutputAlias> output_aliases;

  std::vector<uint32_t> parameter_ids() const;
};

// Checks the invariants of src/compiler/executable_plan_verify.zig:328-449.
// Returns "" when the plan is well formed, otherwise one line of the form
//   invalid executable plan: pass=pjrtx-plan-verify [instruction=N] [value=N] detail="..." feature=<label>
std::string verify_plan(const Plan& plan);

// The whole plan as JSON (values, instructions with attributes, constant payloads as hex, shardings, outputs).
std::string describe_plan(const Plan& plan);

// Stable cache key of a plan for a backend state: "pjrtx-<16 hex digits>" over a version tag, the backend name, the
// custom-call registry version, the ordinals of the devices the executable is compiled for, the compile options,
// shardings, donation and every value and instruction (kinds, operands, attributes, constant payloads, call targets).
// Same fields as the reference's executable-cache fingerprint (src/runtime/executable_fingerprint.zig:9-140; target
// devices :38-56); the hash function differs (64-bit FNV-1a), so keys are not interchangeable with the reference's.
std::string plan_fingerprint(const Plan& plan, const char* backend_name, uint64_t custom_call_registry_version,
                             const std::vector<int32_t>& target_devices = {});

}  // namespace pjrtx

// Tensor-parallel planner.
//
// The reference records, per parameter and output, only a sharding kind and a
// mesh name (src/compiler/stablehlo_sharding.zig:40-93, src/compiler/topology.zig:69-91)
// and emits no partitioned program or collective. This planner takes the same
// metadata plus the split dimension of each partitioned parameter, propagates
// "replicated / split(dim) / partial sum" states forward through the plan
// (Megatron-style column- and row-parallel contractions) and writes the plan of
// one partition: local shapes, static slices where a replicated value meets a
// split one, all_reduce after a contraction over a split dimension, all_gather
// where a split value has to become replicated.
#pragma once

#include <string>

#include "plan.h"

namespace pjrtx {

bool partition_plan(const Plan& full, int partition, int num_partitions, Plan* out, std::string* error);

}  // namespace pjrtx

#include "program.h"

#include <algorithm>

namespace pjrtx {

const char* node_kind_name(NodeKind k) {
  static const char* names[] = {"constant", "parameter", "structural", "view", "elementwise",
                                "reduction", "matmul", "control_flow", "library_call",
                                "materialize", "collective"};
  return names[(int)k];
}

NodeKind program_node_kind(Kind k) {
  switch (k) {
    case Kind::constant: return NodeKind::constant;
    case Kind::copy_arg0: return NodeKind::parameter;
    case Kind::tuple: case Kind::get_tuple_element: return NodeKind::structural;
    case Kind::reshape: case Kind::transpose: case Kind::broadcast_in_dim: case Kind::slice:
      return NodeKind::view;
    case Kind::add: case Kind::subtract: case Kind::multiply: case Kind::divide:
    case Kind::maximum: case Kind::minimum: case Kind::power: case Kind::atan2:
    case Kind::remainder: case Kind::and_: case Kind::or_: case Kind::xor_:
    case Kind::shift_left: case Kind::shift_right_arithmetic: case Kind::shift_right_logical:
    case Kind::negate: case Kind::exp: case Kind::expm1: case Kind::tanh: case Kind::sqrt:
    case Kind::rsqrt: case Kind::abs: case Kind::cbrt: case Kind::ceil: case Kind::floor:
    case Kind::log: case Kind::log1p: case Kind::logistic: case Kind::sine: case Kind::cosine:
    case Kind::not_: case Kind::sign: case Kind::is_finite: case Kind::round_nearest_afz:
    case Kind::round_nearest_even: case Kind::popcnt: case Kind::count_leading_zeros:
    case Kind::real: case Kind::imag: case Kind::compare: case Kind::select: case Kind::clamp:
      return NodeKind::elementwise;
    case Kind::reduce_sum: case Kind::reduce_max: case Kind::reduce_min: case Kind::reduce_and:
    case Kind::reduce_or: case Kind::reduce_window_sum: case Kind::reduce_window_max:
      return NodeKind::reduction;
    case Kind::dot_general: return NodeKind::matmul;
    case Kind::while_: return NodeKind::control_flow;
    case Kind::sort: case Kind::top_k: case Kind::gather: case Kind::scatter:
    case Kind::dynamic_slice: case Kind::dynamic_update_slice: case Kind::pad:
    case Kind::reverse: case Kind::concatenate: case Kind::iota: case Kind::partition_id:
    case Kind::convert: case Kind::bitcast_convert: case Kind::reduce_precision: case Kind::rng:
    case Kind::rng_bit_generator: case Kind::custom_call: case Kind::optimization_barrier:
      return NodeKind::materialize;
    case Kind::all_reduce: case Kind::all_gather: return NodeKind::collective;
    default: return NodeKind::library_call;
  }
}

bool instruction_materializes(Kind k) {
  switch (k) {
    case Kind::tuple: case Kind::get_tuple_element: case Kind::reshape: case Kind::transpose:
    case Kind::broadcast_in_dim: case Kind::slice:
      return false;
    default:
      return true;
  }
}

bool program_node_fusible(Kind k) {
  NodeKind nk = program_node_kind(k);
  if (nk == NodeKind::view || nk == NodeKind::elementwise) return true;
  if (nk == NodeKind::structural) return !instruction_materializes(k);
  return k == Kind::copy_arg0 || k == Kind::convert || k == Kind::bitcast_convert ||
         k == Kind::reduce_precision;
}

LivenessStats compute_liveness(const Program& p) {
  std::vector<char> live(p.values.size(), 0);
  size_t live_count = 0;
  uint64_t live_bytes = 0;
  for (size_t i = 0; i < p.values.size(); i++) {
    const ProgramValue& v = p.values[i];
    if (v.producer_node >= 0) continue;
    if (v.last_use_node < 0 && !v.is_output) continue;
    live[i] = 1;
    live_count++;
    live_bytes += v.byte_size;
  }
  LivenessStats s;
  s.peak_live_value_count = live_count;
  s.peak_live_bytes = live_bytes;
  auto mark_outputs = [&](const Node& n) {
    for (uint32_t o : n.outputs) {
      if (live[o]) continue;
      live[o] = 1;
      live_count++;
      live_bytes += p.values[o].byte_size;
      s.peak_live_value_count = std::max(s.peak_live_value_count, live_count);
      s.peak_live_bytes = std::max(s.peak_live_bytes, live_bytes);
    }
  };
  auto release = [&](uint32_t id) {
    const ProgramValue& v = p.values[id];
    if (v.is_output || v.producer_node < 0) return;
    if (p.nodes[v.producer_node].kind == NodeKind::constant) return;
    if (!live[id]) return;
    live[id] = 0;
    live_count--;
    live_bytes -= v.byte_size;
    s.planned_release_count++;
    s.planned_release_bytes += v.byte_size;
  };
  for (const ScheduleItem& item : p.schedule) {
    if (item.kind == ScheduleKind::node) {
      const Node& n = p.nodes[item.index];
      mark_outputs(n);
      for (uint32_t in : n.inputs)
        if (p.values[in].last_use_node == (long)item.index) release(in);
    } else if (item.kind == ScheduleKind::fusion_group) {
      const FusionGroup& g = p.fusion_groups[item.index];
      for (size_t ni : g.node_indices) mark_outputs(p.nodes[ni]);
      for (size_t ni : g.node_indices)
        for (uint32_t in : p.nodes[ni].inputs) {
          long lu = p.values[in].last_use_node;
          if (lu < 0 || lu > (long)g.last_node) continue;
          release(in);
        }
    }
  }
  return s;
}

static void group_boundaries(const Program& p, FusionGroup* g) {
  // Inputs: values read by a member whose producer is absent or outside the
  // group. Outputs: member results that are program outputs or feed a node
  // outside the group. Both in ascending value-id order.
  std::vector<char> in_mark(p.values.size(), 0), out_mark(p.values.size(), 0);
  auto in_group = [&](long node) { return node >= 0 && p.nodes[node].fusion_group == (long)g->id; };
  for (size_t ni : g->node_indices) {
    const Node& n = p.nodes[ni];
    for (uint32_t in : n.inputs)
      if (!in_group(p.values[in].producer_node)) in_mark[in] = 1;
    for (uint32_t o : n.outputs)
      if (p.values[o].materialization_boundary >= 0) out_mark[o] = 1;
  }
  for (const Edge& e : p.edges)
    if (in_group((long)e.from_node) && !in_group((long)e.to_node)) out_mark[e.value_id] = 1;
  g->input_values.clear();
  g->output_values.clear();
  for (size_t i = 0; i < p.values.size(); i++) {
    if (in_mark[i]) g->input_values.push_back((uint32_t)i);
    if (out_mark[i]) g->output_values.push_back((uint32_t)i);
  }
}

bool build_program(const Plan& plan, Program* out, std::string* error) {
  Program p;
  const size_t nv = plan.values.size();
  std::vector<long> last_use(nv, -1), producer(nv, -1);
  std::vector<char> is_output(nv, 0);
  for (uint32_t id : plan.output_ids)
    if (id < nv) is_output[id] = 1;

  long current_group = -1;
  p.nodes.resize(plan.instructions.size());
  for (size_t i = 0; i < plan.instructions.size(); i++) {
    const Instruction& ins = plan.instructions[i];
    for (uint32_t in : ins.inputs)
      if (in < nv) last_use[in] = (long)i;
    for (uint32_t o : ins.outputs)
      if (o < nv) producer[o] = (long)i;
    Node& n = p.nodes[i];
    n.instruction_index = i;
    n.kind = program_node_kind(ins.kind);
    n.materializes = instruction_materializes(ins.kind);
    n.inputs = ins.inputs;
    n.outputs = ins.outputs;
    if (program_node_fusible(ins.kind)) {
      if (current_group < 0) {
        FusionGroup g;
        g.id = p.fusion_groups.size();
        g.first_node = g.last_node = i;
        p.fusion_groups.push_back(g);
        current_group = (long)g.id;
      }
      FusionGroup& g = p.fusion_groups[current_group];
      g.last_node = i;
      g.node_count++;
      g.node_indices.push_back(i);
      n.fusion_group = current_group;
    } else {
      current_group = -1;
    }
  }

  p.materialization_boundaries.assign(plan.output_ids.begin(), plan.output_ids.end());
  p.values.resize(nv);
  for (size_t i = 0; i < nv; i++) {
    ProgramValue& v = p.values[i];
    v.value_id = (uint32_t)i;
    v.byte_size = plan.values[i].bytes();
    v.producer_node = producer[i];
    v.last_use_node = last_use[i];
    v.is_output = is_output[i];
  }
  for (size_t b = 0; b < p.materialization_boundaries.size(); b++) {
    uint32_t id = p.materialization_boundaries[b];
    if (id < nv && p.values[id].materialization_boundary < 0) p.values[id].materialization_boundary = (long)b;
  }
  for (size_t to = 0; to < p.nodes.size(); to++)
    for (uint32_t in : p.nodes[to].inputs) {
      if (in >= nv || p.values[in].producer_node < 0) continue;
      p.edges.push_back({in, (size_t)p.values[in].producer_node, to});
    }
  for (FusionGroup& g : p.fusion_groups) group_boundaries(p, &g);

  for (size_t i = 0; i < p.nodes.size();) {
    long gid = p.nodes[i].fusion_group;
    if (gid >= 0 && p.fusion_groups[gid].first_node == i) {
      p.schedule.push_back({ScheduleKind::fusion_group, (size_t)gid, p.fusion_groups[gid].node_indices.size()});
      i = p.fusion_groups[gid].last_node + 1;
      continue;
    }
    p.schedule.push_back({ScheduleKind::node, i, 1});
    i++;
  }
  if (!p.materialization_boundaries.empty())
    p.schedule.push_back({ScheduleKind::materialization_boundary, 0, p.materialization_boundaries.size()});

  if (!validate_program(plan, p, error)) return false;
  p.liveness = compute_liveness(p);
  *out = std::move(p);
  return true;
}

static bool vfail(std::string* error, const std::string& detail) {
  if (error) *error = "invalid backend program: pass=backend-program-verify detail=\"" + detail + "\"";
  return false;
}

bool validate_program(const Plan& plan, const Program& p, std::string* error) {
  if (p.values.size() != plan.values.size()) return vfail(error, "value table size differs from plan");
  if (p.nodes.size() != plan.instructions.size()) return vfail(error, "node table size differs from plan");
  for (size_t i = 0; i < p.nodes.size(); i++) {
    const Node& n = p.nodes[i];
    if (n.instruction_index != i) return vfail(error, "node index does not match instruction index");
    for (uint32_t in : n.inputs)
      if (in >= p.values.size()) return vfail(error, "node input outside value table");
    for (uint32_t o : n.outputs) {
      if (o >= p.values.size()) return vfail(error, "node output outside value table");
      if (p.values[o].producer_node != (long)i) return vfail(error, "value producer does not match node");
    }
  }
  for (const Edge& e : p.edges) {
    if (e.from_node >= e.to_node) return vfail(error, "edge is not in dependency order");
    if (p.values[e.value_id].producer_node != (long)e.from_node) return vfail(error, "edge producer mismatch");
  }
  // Groups: contiguous, members agree, boundaries recompute to the same lists.
  for (const FusionGroup& g : p.fusion_groups) {
    if (g.node_count == 0 || g.last_node - g.first_node + 1 != g.node_count ||
        g.node_indices.size() != g.node_count)
      return vfail(error, "fusion group is not contiguous");
    for (size_t k = 0; k < g.node_indices.size(); k++) {
      if (g.node_indices[k] != g.first_node + k) return vfail(error, "fusion group node order");
      if (p.nodes[g.node_indices[k]].fusion_group != (long)g.id) return vfail(error, "fusion group membership");
    }
    FusionGroup check = g;
    group_boundaries(p, &check);
    if (check.input_values != g.input_values || check.output_values != g.output_values)
      return vfail(error, "fusion group boundary values are stale");
  }
  // Schedule: every node exactly once, ascending; every output has a boundary.
  std::vector<char> seen(p.nodes.size(), 0);
  size_t next = 0;
  for (const ScheduleItem& it : p.schedule) {
    if (it.kind == ScheduleKind::node) {
      if (it.index != next || it.index >= p.nodes.size()) return vfail(error, "schedule order");
      seen[it.index] = 1;
      next++;
    } else if (it.kind == ScheduleKind::fusion_group) {
      if (it.index >= p.fusion_groups.size()) return vfail(error, "schedule group index");
      const FusionGroup& g = p.fusion_groups[it.index];
      if (g.first_node != next || it.count != g.node_indices.size()) return vfail(error, "schedule group order");
      for (size_t ni : g.node_indices) seen[ni] = 1;
      next = g.last_node + 1;
    }
  }
  for (char s : seen)
    if (!s) return vfail(error, "node is not scheduled");
  for (uint32_t id : plan.output_ids)
    if (id >= p.values.size() || p.values[id].materialization_boundary < 0)
      return vfail(error, "program output has no materialization boundary");
  return true;
}

std::string describe_program(const Program& p) {
  std::string s = "{";
  s += strfmt("\"value_count\":%zu,\"node_count\":%zu,\"edge_count\":%zu,\"schedule_item_count\":%zu,",
              p.values.size(), p.nodes.size(), p.edges.size(), p.schedule.size());
  s += strfmt("\"fusion_group_count\":%zu,\"materialization_boundary_count\":%zu,",
              p.fusion_groups.size(), p.materialization_boundaries.size());
  s += strfmt("\"planned_release_count\":%zu,\"planned_release_bytes\":%llu,\"peak_live_value_count\":%zu,"
              "\"peak_live_bytes\":%llu,",
              p.liveness.planned_release_count, (unsigned long long)p.liveness.planned_release_bytes,
              p.liveness.peak_live_value_count, (unsigned long long)p.liveness.peak_live_bytes);
  auto list_u32 = [](const std::vector<uint32_t>& v) {
    std::string r = "[";
    for (size_t i = 0; i < v.size(); i++) r += strfmt(i ? ",%u" : "%u", v[i]);
    return r + "]";
  };
  s += "\"nodes\":[";
  for (size_t i = 0; i < p.nodes.size(); i++) {
    const Node& n = p.nodes[i];
    s += strfmt("%s{\"kind\":\"%s\",\"materializes\":%s,\"fusion_group\":%ld,\"inputs\":%s,\"outputs\":%s}",
                i ? "," : "", node_kind_name(n.kind), n.materializes ? "true" : "false", n.fusion_group,
                list_u32(n.inputs).c_str(), list_u32(n.outputs).c_str());
  }
  s += "],\"values\":[";
  for (size_t i = 0; i < p.values.size(); i++) {
    const ProgramValue& v = p.values[i];
    s += strfmt("%s{\"byte_size\":%llu,\"producer_node\":%ld,\"last_use_node\":%ld,\"is_output\":%s,"
                "\"materialization_boundary\":%ld}",
                i ? "," : "", (unsigned long long)v.byte_size, v.producer_node, v.last_use_node,
                v.is_output ? "true" : "false", v.materialization_boundary);
  }
  s += "],\"edges\":[";
  for (size_t i = 0; i < p.edges.size(); i++)
    s += strfmt("%s[%u,%zu,%zu]", i ? "," : "", p.edges[i].value_id, p.edges[i].from_node, p.edges[i].to_node);
  s += "],\"schedule\":[";
  static const char* sk[] = {"node", "fusion_group", "materialization_boundary"};
  for (size_t i = 0; i < p.schedule.size(); i++)
    s += strfmt("%s{\"kind\":\"%s\",\"index\":%zu,\"count\":%zu}", i ? "," : "", sk[(int)p.schedule[i].kind],
                p.schedule[i].index, p.schedule[i].count);
  s += "],\"fusion_groups\":[";
  for (size_t i = 0; i < p.fusion_groups.size(); i++) {
    const FusionGroup& g = p.fusion_groups[i];
    s += strfmt("%s{\"id\":%zu,\"kind\":\"view_elementwise\",\"first_node\":%zu,\"last_node\":%zu,"
                "\"node_count\":%zu,\"input_values\":%s,\"output_values\":%s}",
                i ? "," : "", g.id, g.first_node, g.last_node, g.node_count, list_u32(g.input_values).c_str(),
                list_u32(g.output_values).c_str());
  }
  s += "],\"materialization_boundaries\":" + list_u32(p.materialization_boundaries) + "}";
  return s;
}

}  // namespace pjrtx

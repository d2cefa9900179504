#include "sharding.h"

#include <algorithm>
#include <map>

#include "program.h"

namespace pjrtx {

namespace {

struct State {
  enum Kind { kReplicated, kSplit, kPartial } kind = kReplicated;
  int64_t dim = -1;
};

struct Fail {
  std::string why;
};

class Partitioner {
 public:
  Partitioner(const Plan& full, int partition, int parts) : full_(full), part_(partition), parts_(parts) {}

  Plan run() {
    out_.num_replicas = full_.num_replicas;
    out_.num_partitions = parts_;
    out_.use_shardy = full_.use_shardy;
    out_.device_assignment = full_.device_assignment;
    while ((int)out_.device_assignment.size() < full_.num_replicas * parts_)
      out_.device_assignment.push_back((int32_t)out_.device_assignment.size());
    map_.assign(full_.values.size(), UINT32_MAX);
    state_.assign(full_.values.size(), State{});
    producer_.assign(full_.values.size(), -1);
    for (size_t i = 0; i < full_.instructions.size(); i++)
      for (uint32_t o : full_.instructions[i].outputs) producer_[o] = (long)i;
    // Parameters first, in order, so parameter indices are unchanged.
    size_t p = 0;
    for (const Value& v : full_.values) {
      if (v.role != ValueRole::parameter) continue;
      const Sharding& sh = full_.parameter_shardings[p++];
      State st;
      std::vector<int64_t> dims = v.dims;
      if (sh.kind == ShardingKind::partitioned && sh.split_dim >= 0) {
        if (sh.split_dim >= (int64_t)dims.size() || dims[sh.split_dim] % parts_ != 0)
          fail(strfmt("parameter %u cannot be split %d ways along dimension %lld", v.id, parts_, (long long)sh.split_dim));
        dims[sh.split_dim] /= parts_;
        st = State{State::kSplit, sh.split_dim};
      }
      uint32_t id = add_value(ValueRole::parameter, v.dtype, dims);
      out_.parameter_shardings.push_back(sh);
      map_[v.id] = id;
      state_[v.id] = st;
    }
    for (size_t i = 0; i < full_.instructions.size(); i++) lower(i);
    // Outputs.
    for (size_t o = 0; o < full_.output_ids.size(); o++) {
      uint32_t v = full_.output_ids[o];
      const Sharding& want = full_.output_shardings[o];
      uint32_t id = map_[v];
      if (state_[v].kind == State::kPartial) id = reduce_partial(v);
      if (state_[v].kind == State::kSplit && !(want.kind == ShardingKind::partitioned)) id = gather_split(v);
      out_.output_ids.push_back(id);
      out_.output_shardings.push_back(want);
    }
    out_.donated_parameter_indices = full_.donated_parameter_indices;
    out_.output_aliases = full_.output_aliases;
    return out_;
  }

 private:
  const Plan& full_;
  int part_, parts_;
  Plan out_;
  std::vector<uint32_t> map_;   // full value -> local value
  std::vector<State> state_;    // of the local value
  std::vector<long> producer_;  // full value -> full instruction that defines it
  std::map<std::pair<uint32_t, int64_t>, uint32_t> localized_;

  [[noreturn]] void fail(const std::string& why) { throw Fail{why}; }

  uint32_t add_value(ValueRole role, int dtype, const std::vector<int64_t>& dims) {
    Value v;
    v.id = (uint32_t)out_.values.size();
    v.role = role;
    v.dtype = dtype;
    v.dims = dims;
    out_.values.push_back(v);
    return v.id;
  }

  std::vector<int64_t> local_dims(uint32_t full_value, const State& st) {
    std::vector<int64_t> dims = full_.values[full_value].dims;
    if (st.kind == State::kSplit) {
      if (dims[st.dim] % parts_ != 0) fail(strfmt("value %u: dimension %lld is not divisible by %d", full_value, (long long)st.dim, parts_));
      dims[st.dim] /= parts_;
    }
    return dims;
  }

  uint32_t emit(Kind kind, const std::vector<uint32_t>& inputs, int dtype, const std::vector<int64_t>& dims,
                const std::map<std::string, std::vector<int64_t>>& attrs = {}) {
    Instruction ins;
    ins.kind = kind;
    ins.inputs = inputs;
    ins.attrs = attrs;
    uint32_t id = add_value(ValueRole::instruction_result, dtype, dims);
    ins.outputs = {id};
    out_.instructions.push_back(ins);
    return id;
  }

  // Sum of per-partition partials -> replicated.
  uint32_t reduce_partial(uint32_t v) {
    const Value& lv = out_.values[map_[v]];
    uint32_t id = emit(Kind::all_reduce, {map_[v]}, lv.dtype, lv.dims);
    map_[v] = id;
    state_[v] = State{};
    return id;
  }

  // Split value -> replicated: all_gather places partition blocks along a new
  // leading axis; a transpose + reshape (both free views) restore the layout.
  uint32_t gather_split(uint32_t v) {
    const Value lv = out_.values[map_[v]];
    const int64_t d = state_[v].dim;
    std::vector<int64_t> gdims = lv.dims;
    gdims.insert(gdims.begin(), parts_);
    uint32_t g = emit(Kind::all_gather, {map_[v]}, lv.dtype, gdims);
    uint32_t id = g;
    if (d != 0) {
      // [P, d0, .., dd, ..] -> [d0, .., P, dd, ..]
      std::vector<int64_t> perm, tdims;
      for (int64_t k = 0; k < (int64_t)lv.dims.size(); k++) {
        if (k == d) {
          perm.push_back(0);
          tdims.push_back(parts_);
        }
        perm.push_back(k + 1);
        tdims.push_back(lv.dims[k]);
      }
      id = emit(Kind::transpose, {g}, lv.dtype, tdims, {{"permutation", perm}});
    }
    id = emit(Kind::reshape, {id}, lv.dtype, full_.values[v].dims, {{"dims", full_.values[v].dims}});
    map_[v] = id;
    state_[v] = State{};
    return id;
  }

  // Local block of a replicated value along `dim`.
  uint32_t slice_replicated(uint32_t v, int64_t dim) {
    const Value lv = out_.values[map_[v]];
    if (lv.dims[dim] % parts_ != 0) fail(strfmt("value %u cannot be sliced %d ways", v, parts_));
    std::vector<int64_t> start(lv.dims.size(), 0), limit = lv.dims, strides(lv.dims.size(), 1), dims = lv.dims;
    dims[dim] /= parts_;
    start[dim] = part_ * dims[dim];
    limit[dim] = start[dim] + dims[dim];
    return emit(Kind::slice, {map_[v]}, lv.dtype, dims, {{"start_indices", start}, {"limit_indices", limit}, {"strides", strides}});
  }

  // Local block of a replicated value along `dim`, rebuilt from its definition where that costs nothing: a broadcast
  // that is constant along `dim`, an iota along another axis, or elementwise work over such values is emitted at the
  // local shape (so a causal mask or a splatted scale stays a recognisable splat instead of becoming a slice of a
  // full-size tensor); everything else is sliced. The full-size definition is left for dead-code elimination.
  uint32_t localize(uint32_t v, int64_t dim, int depth = 0) {
    const auto key = std::make_pair(v, dim);
    auto hit = localized_.find(key);
    if (hit != localized_.end()) return hit->second;
    uint32_t result = UINT32_MAX;
    const long p = producer_[v];
    const Value& fv = full_.values[v];
    if (p >= 0 && depth < 12 && fv.dims[dim] % parts_ == 0) {
      const Instruction& ins = full_.instructions[p];
      std::vector<int64_t> dims = fv.dims;
      dims[dim] /= parts_;
      auto rebuild = [&](const std::vector<uint32_t>& inputs) {
        Instruction n = ins;
        n.inputs = inputs;
        n.outputs = {add_value(ValueRole::instruction_result, fv.dtype, dims)};
        if (n.has("dims")) n.attrs["dims"] = dims;
        out_.instructions.push_back(n);
        return n.outputs[0];
      };
      const NodeKind nk = program_node_kind(ins.kind);
      if (ins.kind == Kind::broadcast_in_dim && state_[ins.inputs[0]].kind == State::kReplicated) {
        const std::vector<int64_t>& bd = ins.list("broadcast_dimensions");
        long source = -1;
        for (size_t k = 0; k < bd.size(); k++)
          if (bd[k] == dim) source = (long)k;
        const Value& operand = full_.values[ins.inputs[0]];
        if (source < 0 || operand.dims[source] == 1) result = rebuild({map_[ins.inputs[0]]});
        else result = rebuild({localize(ins.inputs[0], source, depth + 1)});
      } else if (ins.kind == Kind::iota && ins.scalar("iota_dimension", -1) != dim) {
        result = rebuild({});
      } else if ((nk == NodeKind::elementwise || ins.kind == Kind::convert) && ins.outputs.size() == 1) {
        bool ok = true;
        for (uint32_t in : ins.inputs)
          ok &= state_[in].kind == State::kReplicated && (full_.values[in].count() == 1 || full_.values[in].dims == fv.dims);
        if (ok) {
          std::vector<uint32_t> inputs;
          for (uint32_t in : ins.inputs) inputs.push_back(full_.values[in].count() == 1 ? map_[in] : localize(in, dim, depth + 1));
          result = rebuild(inputs);
        }
      }
    }
    if (result == UINT32_MAX) result = slice_replicated(v, dim);
    localized_[key] = result;
    return result;
  }

  void copy_instruction(const Instruction& ins, const std::vector<uint32_t>& inputs, const State& st,
                        const std::map<std::string, std::vector<int64_t>>* attrs = nullptr) {
    Instruction n = ins;
    n.inputs = inputs;
    if (attrs) n.attrs = *attrs;
    n.outputs.clear();
    for (uint32_t o : ins.outputs) {
      std::vector<int64_t> dims = local_dims(o, st);
      uint32_t id = add_value(full_.values[o].role == ValueRole::constant ? ValueRole::constant : ValueRole::instruction_result,
                              full_.values[o].dtype, dims);
      n.outputs.push_back(id);
      map_[o] = id;
      state_[o] = st;
    }
    if (n.has("dims")) n.attrs["dims"] = out_.values[n.outputs[0]].dims;
    out_.instructions.push_back(n);
  }

  std::vector<uint32_t> mapped(const Instruction& ins) {
    std::vector<uint32_t> r;
    for (uint32_t v : ins.inputs) r.push_back(map_[v]);
    return r;
  }

  void lower(size_t index) {
    const Instruction& ins = full_.instructions[index];
    // Partial sums are resolved before any use except the all_reduce itself.
    for (uint32_t v : ins.inputs)
      if (state_[v].kind == State::kPartial) reduce_partial(v);
    const NodeKind nk = program_node_kind(ins.kind);
    if (ins.kind == Kind::constant) {
      copy_instruction(ins, {}, State{});
      return;
    }
    if (nk == NodeKind::elementwise || ins.kind == Kind::convert || ins.kind == Kind::bitcast_convert ||
        ins.kind == Kind::copy_arg0 || ins.kind == Kind::optimization_barrier) {
      State st;
      for (uint32_t v : ins.inputs)
        if (state_[v].kind == State::kSplit) {
          if (st.kind == State::kSplit && st.dim != state_[v].dim) fail("elementwise operands are split along different dimensions");
          st = state_[v];
        }
      std::vector<uint32_t> in = mapped(ins);
      if (st.kind == State::kSplit)
        for (size_t k = 0; k < ins.inputs.size(); k++)
          if (state_[ins.inputs[k]].kind == State::kReplicated && full_.values[ins.inputs[k]].count() != 1)
            in[k] = localize(ins.inputs[k], st.dim);
      copy_instruction(ins, in, st);
      return;
    }
    switch (ins.kind) {
      case Kind::iota:
        copy_instruction(ins, {}, State{});
        return;
      case Kind::broadcast_in_dim: {
        State st;
        const State& s = state_[ins.inputs[0]];
        if (s.kind == State::kSplit) st = State{State::kSplit, ins.list("broadcast_dimensions")[s.dim]};
        copy_instruction(ins, mapped(ins), st);
        return;
      }
      case Kind::reshape: {
        State st;
        const State& s = state_[ins.inputs[0]];
        if (s.kind == State::kSplit) {
          const auto& id = full_.values[ins.inputs[0]].dims;
          const auto& od = full_.values[ins.outputs[0]].dims;
          int64_t prefix = 1;
          for (int64_t k = 0; k < s.dim; k++) prefix *= id[k];
          int64_t acc = 1, found = -1;
          for (size_t k = 0; k < od.size(); k++) {
            if (acc == prefix && od[k] != 1 && od[k] % parts_ == 0) {
              found = (int64_t)k;
              break;
            }
            acc *= od[k];
          }
          if (found < 0) fail(strfmt("reshape at instruction %zu moves a split dimension", index));
          st = State{State::kSplit, found};
        }
        copy_instruction(ins, mapped(ins), st);
        return;
      }
      case Kind::transpose: {
        State st;
        const State& s = state_[ins.inputs[0]];
        const auto& perm = ins.list("permutation");
        if (s.kind == State::kSplit)
          for (size_t k = 0; k < perm.size(); k++)
            if (perm[k] == s.dim) st = State{State::kSplit, (int64_t)k};
        copy_instruction(ins, mapped(ins), st);
        return;
      }
      case Kind::slice: {
        const State& s = state_[ins.inputs[0]];
        auto attrs = ins.attrs;
        if (s.kind == State::kSplit) {
          const auto& id = full_.values[ins.inputs[0]].dims;
          if (ins.list("start_indices")[s.dim] != 0 || ins.list("limit_indices")[s.dim] != id[s.dim])
            fail("slice cuts through a split dimension");
          attrs["limit_indices"][s.dim] = id[s.dim] / parts_;
        }
        copy_instruction(ins, mapped(ins), s, &attrs);
        return;
      }
      case Kind::reverse: case Kind::concatenate: {
        State st;
        for (uint32_t v : ins.inputs)
          if (state_[v].kind == State::kSplit) st = state_[v];
        std::vector<uint32_t> in = mapped(ins);
        if (st.kind == State::kSplit) {
          int64_t along = ins.kind == Kind::concatenate ? ins.scalar("dimension", 0) : -1;
          if (along == st.dim) fail("concatenate along a split dimension");
          for (size_t k = 0; k < ins.inputs.size(); k++) {
            const State& s = state_[ins.inputs[k]];
            if (s.kind == State::kReplicated) in[k] = localize(ins.inputs[k], st.dim);
            else if (s.dim != st.dim) fail("operands are split along different dimensions");
          }
        }
        copy_instruction(ins, in, st);
        return;
      }
      case Kind::dynamic_slice: case Kind::dynamic_update_slice: {
        State st = state_[ins.inputs[0]];
        std::vector<uint32_t> in = mapped(ins);
        auto attrs = ins.attrs;
        if (ins.kind == Kind::dynamic_update_slice) {
          const State& us = state_[ins.inputs[1]];
          if (st.kind == State::kSplit && us.kind == State::kReplicated) in[1] = localize(ins.inputs[1], st.dim);
          else if (st.kind != us.kind || st.dim != us.dim) fail("dynamic_update_slice operand and update are sharded differently");
        } else if (st.kind == State::kSplit) {
          const auto& id = full_.values[ins.inputs[0]].dims;
          if (ins.list("slice_sizes")[st.dim] != id[st.dim]) fail("dynamic_slice cuts through a split dimension");
          attrs["slice_sizes"][st.dim] = id[st.dim] / parts_;
        }
        copy_instruction(ins, in, st, &attrs);
        return;
      }
      case Kind::gather: {
        if (state_[ins.inputs[0]].kind != State::kReplicated || state_[ins.inputs[1]].kind != State::kReplicated)
          fail("gather operands must be replicated");
        copy_instruction(ins, mapped(ins), State{});
        return;
      }
      case Kind::reduce_sum: case Kind::reduce_max: case Kind::reduce_min: case Kind::reduce_and: case Kind::reduce_or: {
        const size_t operands = ins.outputs.size() == 2 ? 2 : 1;
        State s = state_[ins.inputs[0]];
        const auto& rd = ins.list("reduce_dimensions");
        std::vector<uint32_t> in = mapped(ins);
        if (s.kind == State::kSplit && std::find(rd.begin(), rd.end(), s.dim) != rd.end()) {
          // Reducing over the split dimension: make the operands replicated first.
          for (size_t k = 0; k < operands; k++)
            if (state_[ins.inputs[k]].kind == State::kSplit) in[k] = gather_split(ins.inputs[k]);
          s = State{};
        }
        for (size_t k = 0; k < operands; k++) {
          const State& o = state_[ins.inputs[k]];
          if (s.kind == State::kSplit && o.kind == State::kReplicated) in[k] = slice_replicated(ins.inputs[k], s.dim);
        }
        State st;
        if (s.kind == State::kSplit) {
          int64_t removed = 0;
          for (int64_t d : rd) removed += d < s.dim;
          st = State{State::kSplit, s.dim - removed};
        }
        copy_instruction(ins, in, st);
        return;
      }
      case Kind::dot_general: {
        const State& ls = state_[ins.inputs[0]];
        const State& rs = state_[ins.inputs[1]];
        const auto& lb = ins.list("lhs_batch_dimensions");
        const auto& rb = ins.list("rhs_batch_dimensions");
        const int64_t lc = ins.list("lhs_contracting_dimensions")[0], rc = ins.list("rhs_contracting_dimensions")[0];
        const auto& ld = full_.values[ins.inputs[0]].dims;
        const auto& rd = full_.values[ins.inputs[1]].dims;
        auto pos = [](const std::vector<int64_t>& l, int64_t d) {
          auto it = std::find(l.begin(), l.end(), d);
          return it == l.end() ? (int64_t)-1 : (int64_t)(it - l.begin());
        };
        // Output layout: batch..., lhs free..., rhs free...
        auto lhs_free_pos = [&](int64_t d) {
          int64_t p = (int64_t)lb.size();
          for (int64_t k = 0; k < d; k++)
            if (pos(lb, k) < 0 && k != lc) p++;
          return p;
        };
        auto rhs_free_pos = [&](int64_t d) {
          int64_t p = (int64_t)lb.size();
          for (int64_t k = 0; k < (int64_t)ld.size(); k++)
            if (pos(lb, k) < 0 && k != lc) p++;
          for (int64_t k = 0; k < d; k++)
            if (pos(rb, k) < 0 && k != rc) p++;
          return p;
        };
        (void)rd;
        std::vector<uint32_t> in = mapped(ins);
        State st;
        const bool l_split = ls.kind == State::kSplit, r_split = rs.kind == State::kSplit;
        if (!l_split && !r_split) {
          st = State{};
        } else if (l_split && r_split && ls.dim == lc && rs.dim == rc) {
          st = State{State::kPartial, -1};  // row-parallel
        } else if (l_split && r_split && pos(lb, ls.dim) >= 0 && pos(lb, ls.dim) == pos(rb, rs.dim)) {
          st = State{State::kSplit, pos(lb, ls.dim)};
        } else if (!l_split && r_split && rs.dim != rc && pos(rb, rs.dim) < 0) {
          st = State{State::kSplit, rhs_free_pos(rs.dim)};  // column-parallel
        } else if (l_split && !r_split && ls.dim != lc && pos(lb, ls.dim) < 0) {
          st = State{State::kSplit, lhs_free_pos(ls.dim)};
        } else if (l_split && !r_split && ls.dim == lc) {
          in[1] = slice_replicated(ins.inputs[1], rc);
          st = State{State::kPartial, -1};
        } else if (!l_split && r_split && rs.dim == rc) {
          in[0] = slice_replicated(ins.inputs[0], lc);
          st = State{State::kPartial, -1};
        } else if (l_split && !r_split && pos(lb, ls.dim) >= 0) {
          in[1] = slice_replicated(ins.inputs[1], rb[pos(lb, ls.dim)]);
          st = State{State::kSplit, pos(lb, ls.dim)};
        } else if (!l_split && r_split && pos(rb, rs.dim) >= 0) {
          in[0] = slice_replicated(ins.inputs[0], lb[pos(rb, rs.dim)]);
          st = State{State::kSplit, pos(rb, rs.dim)};
        } else {
          fail(strfmt("dot_general at instruction %zu has an unsupported sharding combination", index));
        }
        if (st.kind == State::kPartial) {
          // The local result has the full shape; mark it partial, the all_reduce follows on first use.
          copy_instruction(ins, in, State{});
          state_[ins.outputs[0]] = st;
        } else {
          copy_instruction(ins, in, st);
        }
        return;
      }
      case Kind::custom_call: {
        // Attention: heads split on q and on k/v together.
        State st;
        std::vector<uint32_t> in = mapped(ins);
        if (ins.inputs.size() == 4) {
          const State& q = state_[ins.inputs[0]];
          const State& k = state_[ins.inputs[1]];
          const State& v = state_[ins.inputs[2]];
          const int64_t head_axis = (int64_t)full_.values[ins.inputs[0]].dims.size() - 2;
          if (q.kind == State::kSplit || k.kind == State::kSplit || v.kind == State::kSplit) {
            if (q.kind != State::kSplit || k.kind != State::kSplit || v.kind != State::kSplit || q.dim != head_axis ||
                k.dim != head_axis || v.dim != head_axis)
              fail("attention operands must all be split along the head axis");
            st = q;
          }
        }
        copy_instruction(ins, in, st);
        return;
      }
      case Kind::all_reduce: case Kind::all_gather:
        copy_instruction(ins, mapped(ins), State{});
        return;
      default:
        for (uint32_t v : ins.inputs)
          if (state_[v].kind != State::kReplicated) fail(strfmt("%s has no sharding rule", kind_name(ins.kind)));
        copy_instruction(ins, mapped(ins), State{});
    }
  }
};

}  // namespace

bool partition_plan(const Plan& full, int partition, int num_partitions, Plan* out, std::string* error) {
  if (num_partitions < 1 || partition < 0 || partition >= num_partitions) {
    *error = "partition index is outside the partition count";
    return false;
  }
  std::string v = verify_plan(full);
  if (!v.empty()) {
    *error = v;
    return false;
  }
  try {
    Partitioner p(full, partition, num_partitions);
    *out = p.run();
  } catch (const Fail& f) {
    *error = "invalid executable plan: pass=b200-sharding-planner detail=\"" + f.why + "\" feature=sharding";
    return false;
  }
  std::string check = verify_plan(*out);
  if (!check.empty()) {
    *error = check;
    return false;
  }
  return true;
}

}  // namespace pjrtx

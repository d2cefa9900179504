#include "executor.h"

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cmath>
#include <cstring>
#include <map>
#include <set>

namespace pjrtx {

// ---------------------------------------------------------------------------
// Custom-call registry.

namespace {

struct CustomCallEntry {
  std::string op_name;  // "identity" or a plan kind name
  int arity;
};
std::mutex g_registry_mu;
std::map<std::string, CustomCallEntry> g_registry;
uint64_t g_registry_version = 0;

const char* kSdpaTargets[] = {"pjrtx.mlx_metal.scaled_dot_product_attention", "pjrtx.b200.scaled_dot_product_attention"};
const char* kBinaryAddTargets[] = {"pjrtx.mlx_metal.custom_binary_add_f32", "pjrtx.b200.custom_binary_add_f32"};

bool is_sdpa_target(const std::string& t) {
  for (const char* n : kSdpaTargets)
    if (t == n) return true;
  return false;
}

}  // namespace

bool register_custom_call(const std::string& target, const std::string& op_name, int arity) {
  if (target.empty()) return false;
  if (op_name != "identity") {
    Kind k = kind_from_name(op_name);
    NodeKind nk = program_node_kind(k);
    if (k == Kind::unsupported || nk != NodeKind::elementwise) return false;
  }
  std::lock_guard<std::mutex> lock(g_registry_mu);
  g_registry[target] = CustomCallEntry{op_name, arity};
  g_registry_version++;
  return true;
}

void unregister_custom_call(const std::string& target) {
  std::lock_guard<std::mutex> lock(g_registry_mu);
  if (g_registry.erase(target)) g_registry_version++;
}

uint64_t custom_call_registry_version() {
  std::lock_guard<std::mutex> lock(g_registry_mu);
  return g_registry_version;
}

// ---------------------------------------------------------------------------
// Plan rewriting and legalization.

namespace {

// Resolves registered custom calls into ordinary kinds so they fuse.
Plan rewrite_plan(const Plan& plan) {
  Plan p = plan;
  std::lock_guard<std::mutex> lock(g_registry_mu);
  for (Instruction& ins : p.instructions) {
    if (ins.kind != Kind::custom_call) continue;
    const std::string& t = ins.custom_call_target;
    if (t == "annotate_device_placement" && ins.inputs.size() == 1 && ins.outputs.size() == 1) {
      ins.kind = Kind::copy_arg0;
      continue;
    }
    for (const char* n : kBinaryAddTargets)
      if (t == n && ins.inputs.size() == 2) ins.kind = Kind::add;
    auto it = g_registry.find(t);
    if (it == g_registry.end() || ins.kind != Kind::custom_call) continue;
    if (it->second.op_name == "identity") {
      if (ins.inputs.size() == 1 && ins.outputs.size() == 1) ins.kind = Kind::copy_arg0;
    } else if ((int)ins.inputs.size() == it->second.arity) {
      ins.kind = kind_from_name(it->second.op_name);
    }
  }
  return p;
}

bool mergeable(const std::vector<int64_t>& sizes, const std::vector<int64_t>& strides, int64_t* size, int64_t* stride) {
  int64_t total = 1, last_stride = 0;
  bool any = false;
  for (size_t i = 0; i < sizes.size(); i++) {
    if (sizes[i] == 1) continue;
    if (any && last_stride != strides[i] * sizes[i]) return false;
    any = true;
    last_stride = strides[i];
    total *= sizes[i];
  }
  *size = total;
  *stride = any ? last_stride : 0;
  return true;
}

std::vector<int64_t> dense_strides(const std::vector<int64_t>& dims) {
  std::vector<int64_t> s(dims.size());
  int64_t st = 1;
  for (size_t d = dims.size(); d-- > 0;) {
    s[d] = st;
    st *= dims[d];
  }
  return s;
}

// Canonical contraction of a dot_general, or a reason why it has none.
bool analyze_dot(const Plan& plan, const Instruction& ins, DotShape* out, std::string* why) {
  const Value& lhs = plan.values[ins.inputs[0]];
  const Value& rhs = plan.values[ins.inputs[1]];
  const Value& res = plan.values[ins.outputs[0]];
  const bool rhs_s8 = ins.scalar("rhs_s8", 0) != 0;  // set by the planner: the rhs holds bytes, the third operand column scales
  if ((!rhs_s8 && lhs.dtype != rhs.dtype) || (rhs_s8 && rhs.dtype != kS8) || lhs.dtype != res.dtype || !dtype_is_float(lhs.dtype)) {
    *why = "dot_general operands and result must share one of f32, f16, bf16";
    return false;
  }
  const auto& lb = ins.list("lhs_batch_dimensions");
  const auto& rb = ins.list("rhs_batch_dimensions");
  const auto& lc = ins.list("lhs_contracting_dimensions");
  const auto& rc = ins.list("rhs_contracting_dimensions");
  if (lb.size() != rb.size() || lc.size() != 1 || rc.size() != 1) {
    *why = "dot_general needs equal batch ranks and exactly one contracting dimension";
    return false;
  }
  auto valid = [](const std::vector<int64_t>& l, size_t rank) {
    for (int64_t d : l)
      if (d < 0 || d >= (int64_t)rank) return false;
    return true;
  };
  if (!valid(lb, lhs.dims.size()) || !valid(lc, lhs.dims.size()) || !valid(rb, rhs.dims.size()) || !valid(rc, rhs.dims.size())) {
    *why = "dot_general dimension number is out of range";
    return false;
  }
  if (lhs.dims[lc[0]] != rhs.dims[rc[0]]) {
    *why = "dot_general contracting sizes differ";
    return false;
  }
  std::vector<int64_t> ls = dense_strides(lhs.dims), rs = dense_strides(rhs.dims);
  auto is_in = [](const std::vector<int64_t>& l, int64_t d) { return std::find(l.begin(), l.end(), d) != l.end(); };
  std::vector<int64_t> bsz, lbs, rbs, msz, mst, nsz, nst;
  for (size_t i = 0; i < lb.size(); i++) {
    if (lhs.dims[lb[i]] != rhs.dims[rb[i]]) {
      *why = "dot_general batch sizes differ";
      return false;
    }
    bsz.push_back(lhs.dims[lb[i]]);
    lbs.push_back(ls[lb[i]]);
    rbs.push_back(rs[rb[i]]);
  }
  for (size_t d = 0; d < lhs.dims.size(); d++)
    if (!is_in(lb, (int64_t)d) && (int64_t)d != lc[0]) {
      msz.push_back(lhs.dims[d]);
      mst.push_back(ls[d]);
    }
  for (size_t d = 0; d < rhs.dims.size(); d++)
    if (!is_in(rb, (int64_t)d) && (int64_t)d != rc[0]) {
      nsz.push_back(rhs.dims[d]);
      nst.push_back(rs[d]);
    }
  DotShape s;
  s.dtype = lhs.dtype;
  s.k = lhs.dims[lc[0]];
  s.lhs_k = ls[lc[0]];
  s.rhs_k = rs[rc[0]];
  if (!mergeable(msz, mst, &s.m, &s.lhs_m) || !mergeable(nsz, nst, &s.n, &s.rhs_n)) {
    *why = "dot_general free dimensions are not contiguous in their operand";
    return false;
  }
  // Batch axes: drop size-1 axes, then merge into at most two strided axes.
  std::vector<int64_t> b, bl, br;
  for (size_t i = 0; i < bsz.size(); i++)
    if (bsz[i] != 1) {
      b.push_back(bsz[i]);
      bl.push_back(lbs[i]);
      br.push_back(rbs[i]);
    }
  for (size_t i = 0; i + 1 < b.size();) {
    if (bl[i] == bl[i + 1] * b[i + 1] && br[i] == br[i + 1] * b[i + 1]) {
      b[i] *= b[i + 1];
      bl[i] = bl[i + 1];
      br[i] = br[i + 1];
      b.erase(b.begin() + i + 1);
      bl.erase(bl.begin() + i + 1);
      br.erase(br.begin() + i + 1);
    } else {
      i++;
    }
  }
  if (b.size() > 2) {
    *why = "dot_general has more than two independent batch strides";
    return false;
  }
  if (b.size() == 2) {
    s.b0 = b[0]; s.lhs_b0 = bl[0]; s.rhs_b0 = br[0];
    s.b1 = b[1]; s.lhs_b1 = bl[1]; s.rhs_b1 = br[1];
  } else if (b.size() == 1) {
    s.b1 = b[0]; s.lhs_b1 = bl[0]; s.rhs_b1 = br[0];
  }
  s.out_m = s.n;
  s.out_b1 = s.m * s.n;
  s.out_b0 = s.b1 * s.m * s.n;
  if (res.count() != s.b0 * s.b1 * s.m * s.n) {
    *why = "dot_general result shape does not match its operands";
    return false;
  }
  s.rhs_s8 = rhs_s8 ? 1 : 0;
  *out = s;
  return true;
}

bool analyze_sdpa(const Plan& plan, const Instruction& ins, SdpaShape* out, std::string* why) {
  if (ins.inputs.size() != 4 || ins.outputs.size() != 1) {
    *why = "scaled_dot_product_attention takes q, k, v, token_index";
    return false;
  }
  const Value& q = plan.values[ins.inputs[0]];
  const Value& k = plan.values[ins.inputs[1]];
  const Value& v = plan.values[ins.inputs[2]];
  const Value& t = plan.values[ins.inputs[3]];
  const Value& o = plan.values[ins.outputs[0]];
  if (q.dtype != k.dtype || q.dtype != v.dtype || !dtype_is_float(q.dtype) || o.dtype != q.dtype || o.dims != q.dims ||
      (q.dims.size() != 3 && q.dims.size() != 4) || k.dims.size() != q.dims.size() || k.dims != v.dims ||
      t.count() != 1 || !dtype_is_int(t.dtype)) {
    *why = "scaled_dot_product_attention operand types or ranks are not supported";
    return false;
  }
  const bool hb = q.dims.size() == 4;
  SdpaShape s;
  s.dtype = q.dtype;
  s.batch = hb ? q.dims[0] : 1;
  s.q_len = q.dims[hb ? 1 : 0];
  s.heads = q.dims[hb ? 2 : 1];
  s.head_dim = q.dims[hb ? 3 : 2];
  s.kv_len = k.dims[hb ? 1 : 0];
  s.kv_heads = k.dims[hb ? 2 : 1];
  s.token_dtype = t.dtype;
  if (s.batch <= 0 || s.q_len <= 0 || s.heads <= 0 || s.kv_len <= 0 || s.kv_heads <= 0 || s.head_dim <= 0 ||
      k.dims[hb ? 3 : 2] != s.head_dim || s.heads % s.kv_heads != 0 || (hb && k.dims[0] != s.batch)) {
    *why = "scaled_dot_product_attention shapes are inconsistent";
    return false;
  }
  *out = s;
  return true;
}

struct Issue {
  long instruction = -1;
  long value = -1;
  std::string detail;
  std::string feature = "b200-backend-executable";
};

std::string format_issue(const Plan& plan, const Issue& is) {
  std::string s = "invalid executable plan: pass=b200-backend-legalization";
  if (is.instruction >= 0) {
    s += strfmt(" instruction=%ld", is.instruction);
    const char* n = kind_name(plan.instructions[is.instruction].kind);
    std::string op = n;
    while (!op.empty() && op.back() == '_') op.pop_back();
    s += " op=" + op;
  }
  if (is.value >= 0 && is.value < (long)plan.values.size()) {
    const Value& v = plan.values[is.value];
    s += strfmt(" value=%ld dtype=%s rank=%zu shape=[", is.value, dtype_name(v.dtype), v.dims.size());
    for (size_t d = 0; d < v.dims.size(); d++) s += strfmt(d ? ",%lld" : "%lld", (long long)v.dims[d]);
    s += "] sharding=";
    const char* sharding = "internal";
    std::vector<uint32_t> params = plan.parameter_ids();
    for (size_t p = 0; p < params.size() && p < plan.parameter_shardings.size(); p++)
      if (params[p] == v.id) {
        static const char* names[] = {"replicated", "partitioned", "manual"};
        sharding = names[(int)plan.parameter_shardings[p].kind];
      }
    s += sharding;
  }
  s += " detail=\"" + is.detail + "\" feature=" + is.feature;
  return s;
}

bool dtype_supported(int dt) {
  switch (dt) {
    case kPred: case kS8: case kU8: case kS16: case kU16: case kS32: case kU32: case kS64: case kU64:
    case kF16: case kBF16: case kF32:
      return true;
    default:
      return false;
  }
}

// First reason the rewritten plan cannot run on this backend.
bool lowering_issue(const Plan& plan, size_t device_count, Issue* out) {
  if (device_count == 0) {
    *out = Issue{-1, -1, "backend executable requires at least one device", "b200-device-assignment"};
    return true;
  }
  for (uint32_t id : plan.output_ids)
    if (id >= plan.values.size()) {
      *out = Issue{-1, (long)id, "plan output value is outside the executable value table", "b200-executable-values"};
      return true;
    }
  for (size_t i = 0; i < plan.instructions.size(); i++) {
    const Instruction& ins = plan.instructions[i];
    for (uint32_t v : ins.outputs)
      if (!dtype_supported(plan.values[v].dtype)) {
        *out = Issue{(long)i, (long)v, "element type is not supported by the B200 backend", "b200-element-type"};
        return true;
      }
    for (uint32_t v : ins.inputs)
      if (!dtype_supported(plan.values[v].dtype)) {
        *out = Issue{(long)i, (long)v, "element type is not supported by the B200 backend", "b200-element-type"};
        return true;
      }
    std::string why;
    switch (ins.kind) {
      case Kind::constant:
        break;
      case Kind::dot_general: {
        DotShape s;
        if (ins.inputs.size() != 2 || ins.outputs.size() != 1 || !analyze_dot(plan, ins, &s, &why)) {
          *out = Issue{(long)i, (long)ins.outputs[0], why.empty() ? "malformed dot_general" : why, "b200-dot-general"};
          return true;
        }
        break;
      }
      case Kind::dynamic_update_slice: {
        if (ins.inputs.size() < 2 || ins.outputs.size() != 1) {
          *out = Issue{(long)i, -1, "dynamic_update_slice needs operand, update and start indices", "b200-dynamic-update-slice"};
          return true;
        }
        const Value& op = plan.values[ins.inputs[0]];
        const Value& up = plan.values[ins.inputs[1]];
        bool ok = op.dims.size() == up.dims.size() && op.dtype == up.dtype && ins.inputs.size() == 2 + op.dims.size() &&
                  op.dims.size() <= 8 && plan.values[ins.outputs[0]].dims == op.dims;
        for (size_t d = 0; ok && d < op.dims.size(); d++) {
          ok = up.dims[d] <= op.dims[d] && plan.values[ins.inputs[2 + d]].count() == 1 &&
               dtype_is_int(plan.values[ins.inputs[2 + d]].dtype);
        }
        if (!ok) {
          *out = Issue{(long)i, (long)ins.outputs[0], "dynamic_update_slice operands are inconsistent", "b200-dynamic-update-slice"};
          return true;
        }
        break;
      }
      case Kind::custom_call: {
        SdpaShape s;
        if (ins.custom_call_target == "pjrtx.b200.internal.attention_decode" ||
            ins.custom_call_target == "pjrtx.b200.internal.attention_prefill")
          break;
        if (is_sdpa_target(ins.custom_call_target)) {
          if (!analyze_sdpa(plan, ins, &s, &why)) {
            *out = Issue{(long)i, -1, why, ins.custom_call_target};
            return true;
          }
          break;
        }
        *out = Issue{(long)i, ins.outputs.empty() ? -1 : (long)ins.outputs[0], "custom call target is not registered",
                     ins.custom_call_target.empty() ? "custom-call" : ins.custom_call_target};
        return true;
      }
      case Kind::all_reduce: case Kind::all_gather:
        if (ins.inputs.size() != 1 || ins.outputs.size() != 1) {
          *out = Issue{(long)i, -1, "collective takes one operand", "b200-collective"};
          return true;
        }
        break;
      case Kind::gather:
        if (!codegen_fusible(plan, ins)) {
          *out = Issue{(long)i, (long)ins.outputs[0], "only row-lookup gathers (embedding form) are supported", "gather-form"};
          return true;
        }
        break;
      default:
        if (!codegen_fusible(plan, ins)) {
          *out = Issue{(long)i, ins.outputs.empty() ? -1 : (long)ins.outputs[0],
                       "operation is not supported by the B200 backend executable", "b200-op"};
          return true;
        }
    }
  }
  return false;
}

// ---------------------------------------------------------------------------
// Kernel planning.

// ---------------------------------------------------------------------------
// Decode-attention recognition: dot_general(q, K) -> [convert] -> * scale -> select(key <= pos, ., -inf) -> max ->
// exp(. - max) -> sum -> / sum -> [convert] -> dot_general(., V) becomes one internal attention call, so the split-KV
// kernel reads the cache once instead of three kernels round-tripping scores and probabilities through memory.
// Anything that deviates from this exact dataflow is left alone and runs as separate steps.
//
// The same chain one rank higher is causal self-attention over whole sequences (prefill): q [B, G, S, rep, hd],
// K / V [B, S, G, hd], scores [B, G, S, rep, S'], mask = iota(key axis) <= iota(position axis). It becomes the
// prefill attention call, which keeps scores and probabilities on the SM.

const char* kAttnDecodeTarget = "pjrtx.b200.internal.attention_decode";
const char* kAttnPrefillTarget = "pjrtx.b200.internal.attention_prefill";

struct AttnMatch {
  size_t d1 = 0, d2 = 0;
  std::vector<size_t> consumed;
  uint32_t q = 0, k = 0, v = 0, pos = 0, out = 0;
  float scale = 1.f;
  bool prefill = false;
};

AttnPrefillShape prefill_shape(const Value& q, const Value& k, float scale) {
  AttnPrefillShape s;
  s.dtype = q.dtype;
  s.batch = q.dims[0];
  s.kv_heads = q.dims[1];
  s.seq = q.dims[2];
  s.rep = q.dims[3];
  s.head_dim = q.dims[4];
  s.kv_batch_stride = k.dims[1] * k.dims[2] * k.dims[3];
  s.kv_row_stride = k.dims[2] * k.dims[3];
  s.kv_head_stride = k.dims[3];
  s.scale = scale;
  return s;
}

void fuse_decode_attention(Plan* plan) {
  const char* prefill_env = getenv("PJRTX_B200_ATTENTION_PREFILL");
  const bool prefill_enabled = !(prefill_env && prefill_env[0] == '0');
  const size_t nv = plan->values.size();
  std::vector<long> producer(nv, -1);
  std::vector<std::vector<size_t>> users(nv);
  std::vector<char> is_output(nv, 0);
  for (uint32_t id : plan->output_ids) is_output[id] = 1;
  for (size_t i = 0; i < plan->instructions.size(); i++) {
    for (uint32_t v : plan->instructions[i].inputs) users[v].push_back(i);
    for (uint32_t v : plan->instructions[i].outputs) producer[v] = (long)i;
  }
  auto ins_of = [&](uint32_t v) -> const Instruction* { return producer[v] < 0 ? nullptr : &plan->instructions[producer[v]]; };
  auto sole_user = [&](uint32_t v) -> long {
    if (is_output[v] || users[v].size() != 1) return -1;
    return (long)users[v][0];
  };
  // broadcast_in_dim (or nothing, for rank 0) of a one-element constant: its value as float.
  auto splat_constant = [&](uint32_t v, float* value) {
    const Instruction* b = ins_of(v);
    if (!b) return false;
    if (b->kind == Kind::broadcast_in_dim) {
      if (plan->values[b->inputs[0]].count() != 1) return false;
      b = ins_of(b->inputs[0]);
      if (!b) return false;
    }
    if (b->kind != Kind::constant || plan->values[b->outputs[0]].count() != 1) return false;
    const Value& cv = plan->values[b->outputs[0]];
    if (cv.dtype == kF32 && b->literal.size() == 4) {
      memcpy(value, b->literal.data(), 4);
      return true;
    }
    return false;
  };
  auto is_list = [](const std::vector<int64_t>& l, std::initializer_list<int64_t> want) { return l == std::vector<int64_t>(want); };

  std::vector<AttnMatch> matches;
  std::vector<char> taken(plan->instructions.size(), 0);
  for (size_t i = 0; i < plan->instructions.size(); i++) {
    const Instruction& d1 = plan->instructions[i];
    if (d1.kind != Kind::dot_general || d1.inputs.size() != 2) continue;
    const Value& q = plan->values[d1.inputs[0]];
    const Value& k = plan->values[d1.inputs[1]];
    if ((q.dims.size() != 4 && q.dims.size() != 5) || k.dims.size() != 4 || !dtype_is_float(q.dtype)) continue;
    const bool prefill = q.dims.size() == 5;
    if (prefill && !prefill_enabled) continue;
    const int64_t key_axis = prefill ? 4 : 3;  // of the scores
    const std::vector<int64_t> lead = prefill ? std::vector<int64_t>{0, 1, 2, 3} : std::vector<int64_t>{0, 1, 2};
    if (!is_list(d1.list("lhs_batch_dimensions"), {0, 1}) || !is_list(d1.list("rhs_batch_dimensions"), {0, 2}) ||
        !is_list(d1.list("lhs_contracting_dimensions"), {key_axis}) || !is_list(d1.list("rhs_contracting_dimensions"), {3}))
      continue;
    AttnMatch m;
    m.prefill = prefill;
    m.d1 = i;
    m.q = d1.inputs[0];
    m.k = d1.inputs[1];
    m.consumed.push_back(i);
    uint32_t x = d1.outputs[0];
    long u = sole_user(x);
    if (u < 0) continue;
    const Instruction* n = &plan->instructions[u];
    if (n->kind == Kind::convert && plan->values[n->outputs[0]].dtype == kF32) {
      m.consumed.push_back(u);
      x = n->outputs[0];
      if ((u = sole_user(x)) < 0) continue;
      n = &plan->instructions[u];
    }
    if (n->kind == Kind::multiply) {
      uint32_t other = n->inputs[0] == x ? n->inputs[1] : n->inputs[0];
      if (!splat_constant(other, &m.scale)) continue;
      m.consumed.push_back(u);
      x = n->outputs[0];
      if ((u = sole_user(x)) < 0) continue;
      n = &plan->instructions[u];
    }
    // select(key_index <= pos, x, -inf)
    if (n->kind != Kind::select || n->inputs[1] != x) continue;
    {
      float neg = 0.f;
      if (!splat_constant(n->inputs[2], &neg) || !(neg == -INFINITY)) continue;
      const Instruction* cmp = ins_of(n->inputs[0]);
      if (!cmp || cmp->kind != Kind::compare || cmp->scalar("compare_direction", -1) != (int64_t)CompareOp::le) continue;
      const Instruction* io = ins_of(cmp->inputs[0]);
      const Instruction* pb = ins_of(cmp->inputs[1]);
      if (!io || io->kind != Kind::iota || io->scalar("iota_dimension", -1) != key_axis) continue;
      if (prefill) {  // key index <= position index
        if (!pb || pb->kind != Kind::iota || pb->scalar("iota_dimension", -1) != 2) continue;
        if (plan->values[io->outputs[0]].dims != plan->values[x].dims || plan->values[pb->outputs[0]].dims != plan->values[x].dims ||
            !dtype_is_int(plan->values[io->outputs[0]].dtype) || plan->values[io->outputs[0]].dtype != plan->values[pb->outputs[0]].dtype)
          continue;
      } else {
        if (!pb || pb->kind != Kind::broadcast_in_dim || plan->values[pb->inputs[0]].count() != 1 ||
            !plan->values[pb->inputs[0]].dims.empty() || !dtype_is_int(plan->values[pb->inputs[0]].dtype))
          continue;
        m.pos = pb->inputs[0];
      }
    }
    m.consumed.push_back(u);
    x = n->outputs[0];
    if (is_output[x] || users[x].size() != 2) continue;
    // max over the key axis, subtract, exp
    long rmax = -1, sub = -1;
    for (size_t w : users[x]) {
      const Instruction& c = plan->instructions[w];
      if (c.kind == Kind::reduce_max && c.outputs.size() == 1 && is_list(c.list("reduce_dimensions"), {key_axis})) rmax = (long)w;
      if (c.kind == Kind::subtract && c.inputs[0] == x) sub = (long)w;
    }
    if (rmax < 0 || sub < 0) continue;
    {
      const Instruction* bm = ins_of(plan->instructions[sub].inputs[1]);
      if (!bm || bm->kind != Kind::broadcast_in_dim || bm->inputs[0] != plan->instructions[rmax].outputs[0] ||
          bm->list("broadcast_dimensions") != lead || sole_user(plan->instructions[rmax].outputs[0]) != producer[bm->outputs[0]] ||
          sole_user(bm->outputs[0]) != sub)
        continue;
      m.consumed.push_back(rmax);
      m.consumed.push_back(producer[bm->outputs[0]]);
      m.consumed.push_back(sub);
    }
    x = plan->instructions[sub].outputs[0];
    if ((u = sole_user(x)) < 0 || plan->instructions[u].kind != Kind::exp) continue;
    m.consumed.push_back(u);
    x = plan->instructions[u].outputs[0];
    if (is_output[x] || users[x].size() != 2) continue;
    long rsum = -1, div = -1;
    for (size_t w : users[x]) {
      const Instruction& c = plan->instructions[w];
      if (c.kind == Kind::reduce_sum && is_list(c.list("reduce_dimensions"), {key_axis})) rsum = (long)w;
      if (c.kind == Kind::divide && c.inputs[0] == x) div = (long)w;
    }
    if (rsum < 0 || div < 0) continue;
    {
      const Instruction* bz = ins_of(plan->instructions[div].inputs[1]);
      if (!bz || bz->kind != Kind::broadcast_in_dim || bz->inputs[0] != plan->instructions[rsum].outputs[0] ||
          bz->list("broadcast_dimensions") != lead || sole_user(plan->instructions[rsum].outputs[0]) != producer[bz->outputs[0]] ||
          sole_user(bz->outputs[0]) != div)
        continue;
      m.consumed.push_back(rsum);
      m.consumed.push_back(producer[bz->outputs[0]]);
      m.consumed.push_back(div);
    }
    x = plan->instructions[div].outputs[0];
    if ((u = sole_user(x)) < 0) continue;
    n = &plan->instructions[u];
    if (n->kind == Kind::convert && plan->values[n->outputs[0]].dtype == q.dtype) {
      m.consumed.push_back(u);
      x = n->outputs[0];
      if ((u = sole_user(x)) < 0) continue;
      n = &plan->instructions[u];
    }
    if (n->kind != Kind::dot_general || n->inputs[0] != x) continue;
    if (!is_list(n->list("lhs_batch_dimensions"), {0, 1}) || !is_list(n->list("rhs_batch_dimensions"), {0, 2}) ||
        !is_list(n->list("lhs_contracting_dimensions"), {key_axis}) || !is_list(n->list("rhs_contracting_dimensions"), {1}))
      continue;
    const Value& vv = plan->values[n->inputs[1]];
    if (vv.dims != k.dims || vv.dtype != q.dtype || k.dtype != q.dtype || plan->values[x].dtype != q.dtype) continue;
    if (producer[n->inputs[1]] > (long)i || (!prefill && producer[m.pos] > (long)i)) continue;  // every input exists before the first dot
    m.d2 = (size_t)u;
    m.v = n->inputs[1];
    m.out = n->outputs[0];
    m.consumed.push_back(u);
    if (prefill) {
      // q [B, G, S, rep, hd], k / v [B, S, G, hd]; the kernel must support the shape.
      if (k.dims[0] != q.dims[0] || k.dims[2] != q.dims[1] || k.dims[1] != q.dims[2] || k.dims[3] != q.dims[4] ||
          !attn_prefill_supported(prefill_shape(q, k, 1.f)))
        continue;
      bool clash = false;
      for (size_t c : m.consumed) clash |= taken[c] != 0;
      if (clash) continue;
      for (size_t c : m.consumed) taken[c] = 1;
      matches.push_back(m);
      continue;
    }
    // The split-KV kernel must support the shape.
    AttnDecodeShape shape;
    shape.dtype = q.dtype;
    shape.batch = q.dims[0];
    shape.kv_heads = q.dims[1];
    shape.heads = q.dims[1] * q.dims[2];
    shape.head_dim = q.dims[3];
    shape.kv_len = k.dims[1];
    shape.q_batch_stride = shape.heads * shape.head_dim;
    shape.q_head_stride = shape.head_dim;
    shape.kv_batch_stride = k.dims[1] * k.dims[2] * k.dims[3];
    shape.kv_row_stride = k.dims[2] * k.dims[3];
    shape.kv_head_stride = k.dims[3];
    if (k.dims[0] != q.dims[0] || k.dims[2] != q.dims[1] || k.dims[3] != q.dims[3] || !attn_decode_supported(shape)) continue;
    bool clash = false;
    for (size_t c : m.consumed) clash |= taken[c] != 0;
    if (clash) continue;
    for (size_t c : m.consumed) taken[c] = 1;
    matches.push_back(m);
  }
  if (matches.empty()) return;
  std::vector<char> erase(plan->instructions.size(), 0);
  for (const AttnMatch& m : matches) {
    for (size_t c : m.consumed) erase[c] = 1;
    erase[m.d1] = 0;
    Instruction call;
    call.kind = Kind::custom_call;
    call.custom_call_target = m.prefill ? kAttnPrefillTarget : kAttnDecodeTarget;
    call.inputs = {m.q, m.k, m.v, m.pos};
    if (m.prefill) call.inputs.pop_back();
    call.outputs = {m.out};
    uint32_t bits;
    memcpy(&bits, &m.scale, 4);
    call.attrs["scale_bits"] = {(int64_t)bits};
    call.attrs["dims"] = plan->values[m.out].dims;
    plan->instructions[m.d1] = call;
  }
  std::vector<Instruction> kept;
  for (size_t i = 0; i < plan->instructions.size(); i++)
    if (!erase[i]) kept.push_back(std::move(plan->instructions[i]));
  plan->instructions = std::move(kept);
}

// Weight-only int8: dot_general(x, W) with W = [convert ->] multiply(convert(w : s8 -> f16), broadcast(scale : f16[n]))
// over a [k, n] weight (the only quantised form the reference accepts: its mixed-type dot is rejected,
// src/backend/mlx_metal/lowering_linalg.zig:14-53, and convert is api.cc:907-935). When the dequantised weight has no
// other reader and the tensor-core stream can take the shape, the dot_general reads the bytes itself: its rhs becomes
// w, the scale its third operand, and the dequantising instructions die. The kernel rebuilds, per element, exactly the
// value the written program would have stored (f16 product rounded to nearest, then the conversion), so results are
// those of the op-by-op program while the weights stay one byte wide in HBM.
void fuse_dequant_dots(Plan* plan) {
  const size_t ni = plan->instructions.size(), nv = plan->values.size();
  std::vector<long> producer(nv, -1);
  std::vector<int> readers(nv, 0);
  for (size_t i = 0; i < ni; i++) {
    for (uint32_t v : plan->instructions[i].outputs) producer[v] = (long)i;
    for (uint32_t v : plan->instructions[i].inputs) readers[v]++;
  }
  for (uint32_t o : plan->output_ids) readers[o]++;
  auto made_by = [&](uint32_t v, Kind kind) -> const Instruction* {
    return producer[v] >= 0 && plan->instructions[producer[v]].kind == kind ? &plan->instructions[producer[v]] : nullptr;
  };
  for (size_t i = 0; i < ni; i++) {
    Instruction& dot = plan->instructions[i];
    if (dot.kind != Kind::dot_general || dot.inputs.size() != 2) continue;
    const Value& x = plan->values[dot.inputs[0]];
    uint32_t w = dot.inputs[1];
    const Value& wv = plan->values[w];
    if ((x.dtype != kBF16 && x.dtype != kF16) || wv.dtype != x.dtype || wv.dims.size() != 2 || readers[w] != 1) continue;
    if (!dot.list("lhs_batch_dimensions").empty() || dot.list("rhs_contracting_dimensions") != std::vector<int64_t>{0} ||
        dot.list("lhs_contracting_dimensions") != std::vector<int64_t>{(int64_t)x.dims.size() - 1})
      continue;
    if (x.dtype == kBF16) {  // f16 product converted to the element type
      const Instruction* cv = made_by(w, Kind::convert);
      if (!cv || plan->values[cv->inputs[0]].dtype != kF16 || readers[cv->inputs[0]] != 1) continue;
      w = cv->inputs[0];
    }
    const Instruction* mul = made_by(w, Kind::multiply);
    if (!mul || plan->values[w].dtype != kF16) continue;
    const Instruction* widen = nullptr;
    const Instruction* spread = nullptr;
    for (int sw = 0; sw < 2; sw++) {
      const Instruction* a = made_by(mul->inputs[sw], Kind::convert);
      const Instruction* b = made_by(mul->inputs[1 - sw], Kind::broadcast_in_dim);
      if (a && b && readers[mul->inputs[0]] == 1 && readers[mul->inputs[1]] == 1) {
        widen = a;
        spread = b;
      }
    }
    if (!widen || !spread) continue;
    const uint32_t bytes = widen->inputs[0], scale = spread->inputs[0];
    const Value& bv = plan->values[bytes];
    const Value& sv = plan->values[scale];
    if (bv.dtype != kS8 || bv.dims != wv.dims || sv.dtype != kF16 || sv.dims != std::vector<int64_t>{wv.dims[1]} ||
        spread->list("broadcast_dimensions") != std::vector<int64_t>{1})
      continue;
    // Bytes and scales must be values no instruction writes (parameters or constants): the kernel may read them early.
    if ((producer[bytes] >= 0 && plan->instructions[producer[bytes]].kind != Kind::constant) ||
        (producer[scale] >= 0 && plan->instructions[producer[scale]].kind != Kind::constant))
      continue;
    DotShape shape;
    shape.dtype = x.dtype;
    shape.m = x.count() / std::max<int64_t>(x.dims.back(), 1);
    shape.k = wv.dims[0];
    shape.n = wv.dims[1];
    shape.lhs_m = shape.k;
    shape.lhs_k = 1;
    shape.rhs_k = shape.n;
    shape.rhs_n = 1;
    shape.out_m = shape.n;
    if (!dot_s8_supported(shape)) continue;
    dot.inputs = {dot.inputs[0], bytes, scale};
    dot.attrs["rhs_s8"] = {1};
  }
}

struct KernelPlan {
  Plan plan;  // rewritten
  Program program;
  std::vector<uint32_t> root;      // storage class representative per value
  std::vector<Step> steps;
  std::vector<Storage> storage;    // per value (meaningful for roots)
  std::vector<uint32_t> params;    // parameter value ids in order
  std::vector<size_t> constants;   // constant instruction indices in slot order
  std::vector<uint64_t> param_slot;  // arena offset of the staging slot of a small parameter, or UINT64_MAX
  std::vector<char> param_donated;
  uint64_t arena_bytes = 0, scratch_bytes = 0;
};

bool env_flag_local(const char* name, bool fallback) {
  const char* v = getenv(name);
  if (!v || !*v) return fallback;
  return !(v[0] == '0' || v[0] == 'f' || v[0] == 'F' || v[0] == 'n' || v[0] == 'N');
}

constexpr uint64_t kAlign = 256;
uint64_t align_up(uint64_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

bool is_alias_kind(const Instruction& ins) {
  return (ins.kind == Kind::reshape || ins.kind == Kind::copy_arg0 ||
          (ins.kind == Kind::optimization_barrier && ins.inputs.size() == 1)) &&
         ins.inputs.size() == 1 && ins.outputs.size() == 1;
}

bool plan_kernels(const Plan& original, int sm_count, KernelPlan* kp, std::string* error) {
  kp->plan = rewrite_plan(original);
  const Plan& plan = kp->plan;
  std::string verr = verify_plan(plan);
  if (!verr.empty()) {
    *error = verr;
    return false;
  }
  Issue issue;
  if (lowering_issue(plan, 1, &issue)) {
    *error = format_issue(plan, issue);
    return false;
  }
  if (!build_program(plan, &kp->program, error)) return false;
  if (env_flag_local("PJRTX_B200_FUSE_ATTENTION", true)) fuse_decode_attention(&kp->plan);
  if (env_flag_local("PJRTX_B200_FUSE_DEQUANT", true)) fuse_dequant_dots(&kp->plan);

  const size_t nv = plan.values.size(), ni = plan.instructions.size();
  kp->params = plan.parameter_ids();
  kp->param_donated.assign(kp->params.size(), 0);
  for (uint32_t p : plan.donated_parameter_indices)
    if (p < kp->params.size()) kp->param_donated[p] = 1;
  std::map<uint32_t, uint32_t> param_index;
  for (size_t p = 0; p < kp->params.size(); p++) param_index[kp->params[p]] = (uint32_t)p;

  std::vector<long> producer(nv, -1), last_read(nv, -1);
  std::vector<std::vector<size_t>> users(nv);
  std::vector<char> is_output(nv, 0);
  for (uint32_t id : plan.output_ids) is_output[id] = 1;
  for (size_t i = 0; i < ni; i++) {
    for (uint32_t v : plan.instructions[i].inputs) {
      users[v].push_back(i);
      last_read[v] = (long)i;
    }
    for (uint32_t v : plan.instructions[i].outputs) producer[v] = (long)i;
  }
  // Dead instructions (left behind by rewrites, or simply unused) are skipped: nothing reads what they produce.
  std::vector<char> dead(ni, 0);
  {
    std::vector<char> value_live(nv, 0);
    for (uint32_t id : plan.output_ids) value_live[id] = 1;
    for (size_t i = ni; i-- > 0;) {
      bool live = false;
      for (uint32_t v : plan.instructions[i].outputs) live |= value_live[v] != 0;
      if (!live) {
        dead[i] = 1;
        continue;
      }
      for (uint32_t v : plan.instructions[i].inputs) value_live[v] = 1;
    }
    for (size_t v = 0; v < nv; v++) {
      users[v].erase(std::remove_if(users[v].begin(), users[v].end(), [&](size_t u) { return dead[u] != 0; }), users[v].end());
      last_read[v] = users[v].empty() ? -1 : (long)users[v].back();
    }
  }

  // Storage classes: pure aliases and in-place slice updates share their operand's storage.
  kp->root.resize(nv);
  std::vector<long> class_last(nv, -1);
  std::vector<char> class_output(nv, 0);
  for (size_t v = 0; v < nv; v++) {
    kp->root[v] = (uint32_t)v;
    if (producer[v] < 0) {  // parameters
      class_last[v] = last_read[v];
      class_output[v] = is_output[v];
    }
  }
  std::vector<char> dus_in_place(ni, 0);
  for (size_t i = 0; i < ni; i++) {
    const Instruction& ins = plan.instructions[i];
    if (dead[i]) continue;
    auto join = [&](uint32_t out, uint32_t r) {
      kp->root[out] = r;
      class_last[r] = std::max(class_last[r], last_read[out]);
      class_output[r] |= is_output[out];
    };
    if (is_alias_kind(ins)) {
      join(ins.outputs[0], kp->root[ins.inputs[0]]);
      continue;
    }
    if (ins.kind == Kind::dynamic_update_slice) {
      uint32_t r = kp->root[ins.inputs[0]];
      bool storage_ok = producer[r] >= 0 ? plan.instructions[producer[r]].kind != Kind::constant
                                         : (param_index.count(r) && kp->param_donated[param_index[r]]);
      // The update and the start indices must not live in the operand's storage.
      bool disjoint = true;
      for (size_t k = 1; k < ins.inputs.size(); k++) disjoint &= kp->root[ins.inputs[k]] != r;
      if (storage_ok && disjoint && class_last[r] <= (long)i && !class_output[r]) {
        dus_in_place[i] = 1;
        join(ins.outputs[0], r);
        continue;
      }
    }
    for (uint32_t o : ins.outputs) {
      class_last[o] = last_read[o];
      class_output[o] = is_output[o];
    }
  }

  // Steps. Runs of fusible nodes become generated kernels (longest prefix that
  // one kernel can express), everything else is one step per node.
  std::vector<char> in_set(ni, 0);
  auto stored_roots = [&](size_t a, size_t b) {  // instruction range [a, b)
    std::vector<uint32_t> stored;
    for (size_t i = a; i < b; i++) {
      if (plan.instructions[i].kind == Kind::constant || dead[i]) continue;
      for (uint32_t v : plan.instructions[i].outputs) {
        bool needed = is_output[v];
        for (size_t u : users[v]) needed |= (u < a || u >= b);
        if (!needed) continue;
        uint32_t r = kp->root[v];
        if (producer[r] < (long)a || producer[r] >= (long)b) continue;  // storage owned elsewhere
        if (std::find(stored.begin(), stored.end(), r) == stored.end()) stored.push_back(r);
      }
    }
    return stored;
  };
  auto skipped = [&](size_t i) { return plan.instructions[i].kind == Kind::constant || dead[i] != 0; };
  // An in-place slice update can be the tail of a generated kernel: the kernel computes the update and stores it at
  // the start indices (a KV-cache row written by the kernel that rotated it).
  const bool fuse_dus = env_flag_local("PJRTX_B200_FUSE_SLICE_UPDATE", true);
  auto scatter_at = [&](size_t i) {
    return fuse_dus && plan.instructions[i].kind == Kind::dynamic_update_slice && dus_in_place[i] != 0 && !dead[i];
  };
  auto fusible_at = [&](size_t i) {
    const Instruction& ins = plan.instructions[i];
    return skipped(i) || scatter_at(i) || codegen_fusible(plan, ins);
  };
  // The slice updates of [a, b) can run inside one kernel when nothing else in the range touches their storage
  // (another thread of the same kernel could read a row before or after it is overwritten) and no two of them share it.
  auto scatters_of = [&](size_t a, size_t b, std::vector<size_t>* out) {
    out->clear();
    for (size_t n = a; n < b; n++)
      if (scatter_at(n)) out->push_back(n);
    for (size_t q = 0; q < out->size(); q++) {
      const Instruction& d = plan.instructions[(*out)[q]];
      const uint32_t r = kp->root[d.outputs[0]];
      for (size_t q2 = q + 1; q2 < out->size(); q2++)
        if (kp->root[plan.instructions[(*out)[q2]].outputs[0]] == r) return false;
      for (size_t n = a; n < b; n++) {
        if (n == (*out)[q] || skipped(n)) continue;
        for (uint32_t v : plan.instructions[n].inputs)
          if (kp->root[v] == r) return false;
      }
      for (size_t k = 1; k < d.inputs.size(); k++)
        if (kp->root[d.inputs[k]] == r) return false;
    }
    return true;
  };

  const bool fusion_debug = env_flag_local("PJRTX_B200_FUSION_DEBUG", false);
  size_t i = 0;
  while (i < ni) {
    const Instruction& ins = plan.instructions[i];
    if (skipped(i)) {
      i++;
      continue;
    }
    if (fusible_at(i)) {
      size_t end = i;
      while (end < ni && fusible_at(end)) end++;
      size_t a = i;
      while (a < end) {
        size_t b = end;
        bool placed = false;
        std::string why;
        for (; b > a; b--) {
          if (skipped(b - 1) && b - 1 > a) continue;  // never end a kernel on a skipped instruction
          std::vector<uint32_t> stored = stored_roots(a, b);
          // Values without elements need no kernel (their storage has no bytes either).
          stored.erase(std::remove_if(stored.begin(), stored.end(), [&](uint32_t r) { return plan.values[r].count() == 0; }),
                       stored.end());
          std::vector<size_t> scatters;
          if (!scatters_of(a, b, &scatters)) {
            why = "a slice update's storage is used elsewhere in the run";
            if (fusion_debug) fprintf(stderr, "pjrtx_b200 fusion: nodes [%zu, %zu) not one kernel: %s\n", a, b, why.c_str());
            continue;
          }
          if (stored.empty() && scatters.empty()) {
            placed = true;  // pure aliases: nothing to launch
            break;
          }
          std::vector<size_t> nodes;
          for (size_t n = a; n < b; n++)
            if (!skipped(n)) nodes.push_back(n);
          Step st;
          st.type = Step::kFused;
          if (generate_fused_kernel(plan, nodes, stored, scatters, sm_count, &st.fused, &why)) {
            st.nodes = nodes;
            for (uint32_t v : st.fused.inputs) {
              uint32_t r = kp->root[v];
              if (std::find(st.inputs.begin(), st.inputs.end(), r) == st.inputs.end()) st.inputs.push_back(r);
            }
            st.outputs = stored;
            for (uint32_t v : st.fused.scatter_dst) st.outputs.push_back(kp->root[v]);
            kp->steps.push_back(std::move(st));
            placed = true;
            break;
          }
          if (fusion_debug) fprintf(stderr, "pjrtx_b200 fusion: nodes [%zu, %zu) not one kernel: %s\n", a, b, why.c_str());
        }
        if (!placed) {
          Issue is{(long)a, plan.instructions[a].outputs.empty() ? -1 : (long)plan.instructions[a].outputs[0],
                   "no kernel can be generated: " + why, "b200-fusion"};
          *error = format_issue(plan, is);
          return false;
        }
        a = b;
      }
      i = end;
      continue;
    }
    Step st;
    st.nodes = {i};
    std::string why;
    switch (ins.kind) {
      case Kind::dot_general:
        st.type = Step::kDot;
        analyze_dot(plan, ins, &st.dot, &why);
        st.dot_scratch = dot_plan(st.dot, sm_count);
        st.inputs = {kp->root[ins.inputs[0]], kp->root[ins.inputs[1]]};
        if (st.dot.rhs_s8) st.dot_scales = {kp->root[ins.inputs[2]]};
        st.outputs = {ins.outputs[0]};
        break;
      case Kind::dynamic_update_slice: {
        st.type = Step::kSliceUpdate;
        const Value& op = plan.values[ins.inputs[0]];
        const Value& up = plan.values[ins.inputs[1]];
        st.dus.rank = (int)op.dims.size();
        st.dus.elem_size = (int)dtype_size(op.dtype);
        for (size_t d = 0; d < op.dims.size(); d++) {
          st.dus.dst_dims[d] = op.dims[d];
          st.dus.upd_dims[d] = up.dims[d];
          st.dus.start_dtype[d] = plan.values[ins.inputs[2 + d]].dtype;
        }
        st.in_place = dus_in_place[i];
        st.bytes = op.bytes();
        for (uint32_t v : ins.inputs) st.inputs.push_back(kp->root[v]);
        st.outputs = {kp->root[ins.outputs[0]]};
        break;
      }
      case Kind::custom_call: {
        for (uint32_t v : ins.inputs) st.inputs.push_back(kp->root[v]);
        st.outputs = {ins.outputs[0]};
        AttnDecodeShape& ad = st.attn;
        if (ins.custom_call_target == kAttnPrefillTarget) {
          float scale;
          uint32_t bits = (uint32_t)ins.scalar("scale_bits", 0);
          memcpy(&scale, &bits, 4);
          st.attn_prefill = prefill_shape(plan.values[ins.inputs[0]], plan.values[ins.inputs[1]], scale);
          if (!attn_prefill_supported(st.attn_prefill)) {
            *error = format_issue(plan, Issue{(long)i, -1, "internal attention call has an unsupported shape", "b200-attention"});
            return false;
          }
          st.type = Step::kAttnPrefill;
        } else if (ins.custom_call_target == kAttnDecodeTarget) {
          const Value& q = plan.values[ins.inputs[0]];
          const Value& k = plan.values[ins.inputs[1]];
          ad.dtype = q.dtype;
          ad.batch = q.dims[0];
          ad.kv_heads = q.dims[1];
          ad.heads = q.dims[1] * q.dims[2];
          ad.head_dim = q.dims[3];
          ad.kv_len = k.dims[1];
          ad.round_scores = 1;
          uint32_t bits = (uint32_t)ins.scalar("scale_bits", 0);
          memcpy(&ad.scale, &bits, 4);
          ad.token_dtype = plan.values[ins.inputs[3]].dtype;
          st.type = Step::kAttnDecode;
        } else {
          st.type = Step::kSdpa;
          analyze_sdpa(plan, ins, &st.sdpa, &why);
          if (st.sdpa.q_len == 1) {  // decode-shaped call: the split-KV kernel
            ad.dtype = st.sdpa.dtype;
            ad.batch = st.sdpa.batch;
            ad.heads = st.sdpa.heads;
            ad.kv_heads = st.sdpa.kv_heads;
            ad.head_dim = st.sdpa.head_dim;
            ad.kv_len = st.sdpa.kv_len;
            ad.round_scores = 0;
            ad.scale = 1.0f / sqrtf((float)st.sdpa.head_dim);
            ad.token_dtype = st.sdpa.token_dtype;
            st.type = Step::kAttnDecode;
          }
        }
        if (st.type == Step::kAttnDecode) {
          ad.q_batch_stride = ad.heads * ad.head_dim;
          ad.q_head_stride = ad.head_dim;
          ad.kv_batch_stride = ad.kv_len * ad.kv_heads * ad.head_dim;
          ad.kv_row_stride = ad.kv_heads * ad.head_dim;
          ad.kv_head_stride = ad.head_dim;
          if (!attn_decode_supported(ad)) {
            if (ins.custom_call_target == kAttnDecodeTarget) {
              *error = format_issue(plan, Issue{(long)i, -1, "internal attention call has an unsupported shape", "b200-attention"});
              return false;
            }
            st.type = Step::kSdpa;
          } else {
            st.attn_plan = attn_decode_plan(ad, sm_count);
          }
        }
        break;
      }
      case Kind::all_reduce: case Kind::all_gather:
        st.type = ins.kind == Kind::all_reduce ? Step::kAllReduce : Step::kAllGather;
        st.inputs = {kp->root[ins.inputs[0]]};
        st.outputs = {ins.outputs[0]};
        st.count = (uint64_t)plan.values[ins.inputs[0]].count();
        st.dtype = plan.values[ins.inputs[0]].dtype;
        break;
      default:
        *error = format_issue(plan, Issue{(long)i, -1, "operation has no kernel", "b200-op"});
        return false;
    }
    kp->steps.push_back(std::move(st));
    i++;
  }

  // Adjacent streaming contractions that read the same lhs become one launch
  // (q/k/v and gate/up projections).
  {
    std::vector<Step> merged;
    for (Step& st : kp->steps) {
      Step* prev = merged.empty() ? nullptr : &merged.back();
      bool can = prev && prev->type == Step::kDot && st.type == Step::kDot && prev->dot_scratch.path == 1 &&
                 st.dot_scratch.path == 1 && prev->dot_scratch.umma == st.dot_scratch.umma && prev->inputs[0] == st.inputs[0] && prev->dot.b0 * prev->dot.b1 == 1 &&
                 st.dot.b0 * st.dot.b1 == 1 && prev->dot.m == st.dot.m && prev->dot.k == st.dot.k &&
                 prev->dot.dtype == st.dot.dtype && prev->dot.rhs_s8 == st.dot.rhs_s8 && prev->dot.lhs_m == st.dot.lhs_m &&
                 prev->dot.lhs_k == st.dot.lhs_k &&
                 std::max<size_t>(prev->dot_group.size(), 1) < (size_t)kDotGroupMax;
      if (can)
        for (uint32_t o : prev->outputs) can &= (o != st.inputs[1]);
      if (!can) {
        merged.push_back(std::move(st));
        continue;
      }
      if (prev->dot_group.empty()) prev->dot_group.push_back(prev->dot);
      prev->dot_group.push_back(st.dot);
      prev->nodes.push_back(st.nodes[0]);
      prev->inputs.push_back(st.inputs[1]);
      for (uint32_t sc : st.dot_scales) prev->dot_scales.push_back(sc);
      prev->outputs.push_back(st.outputs[0]);
      prev->dot_scratch = dot_group_plan(prev->dot_group.data(), (int)prev->dot_group.size(), sm_count);
    }
    kp->steps = std::move(merged);
  }

  // Streaming contractions on the CUDA-core kernel take over what the small kernels around them did, and consecutive
  // ones run as one launch (kernels/stream_tma.cuh):
  //   * a generated kernel that only computes silu(gate) * up for the next contraction's lhs becomes that
  //     contraction's lhs transform;
  //   * a generated row kernel that only computes RMSNorm(x) * gain (optionally of x = a + b, where one addend is the
  //     previous contraction's result) for the next contraction's lhs becomes an lhs transform, and the addition becomes
  //     the previous contraction's residual epilogue;
  //   * adjacent streaming contractions are chained (up to kDotChainMax segments per launch).
  // The dataflow is matched exactly; anything else keeps its generated kernel.
  // Both are off unless PJRTX_B200_DOT_FUSE=1 (and PJRTX_B200_DOT_CHAIN=1): measured on the 8B-shape decode step, ms per
  // step with programmatic dependent launch between kernels: separate launches 3.50; transforms and residuals folded in
  // 3.58 (every CTA repeats the row reduction after it has waited for its predecessor, where the one-CTA norm kernel ran
  // concurrently with the next contraction's ramp); chained 4.16 (a segment boundary - fold, grid barrier, factors,
  // first lhs values - is 7 to 8 us of dependent round trips against the 4 us of weights the rings hold).
  // PJRTX_B200_DOT_FUSE=silu folds in only the silu(gate) * up transform (no row reduction involved): 3.47 against
  // 3.40 ms per step - the generated kernel costs 2.6 us inside the step, the transform costs the contraction more.
  const char* fuse_env = getenv("PJRTX_B200_DOT_FUSE");
  const bool fuse_silu_only = fuse_env && std::string(fuse_env) == "silu";  // only the silu(gate) * up transform
  if (fuse_silu_only || env_flag_local("PJRTX_B200_DOT_FUSE", false)) {
    auto chainable = [&](const Step& st) {
      return st.type == Step::kDot && st.dot_scratch.path == 1 && st.dot_scratch.tma == 1 && st.dot_scratch.umma == 0 &&
             st.dot.b0 * st.dot.b1 == 1;
    };
    for (Step& st : kp->steps) {
      if (!chainable(st)) continue;
      DotSeg seg;
      if (st.dot_group.size() > 1) seg.group = st.dot_group;
      else seg.group = {st.dot};
      seg.lhs = st.inputs[0];
      for (size_t g = 1; g < st.inputs.size(); g++) seg.rhs.push_back(st.inputs[g]);
      seg.out = st.outputs;
      seg.residual.assign(seg.out.size(), UINT32_MAX);
      st.segs.push_back(std::move(seg));
    }
    // Readers of a storage class: every live instruction that reads a value of the class.
    auto class_users = [&](uint32_t r) {
      std::vector<size_t> out;
      for (size_t v = 0; v < nv; v++)
        if (kp->root[v] == r)
          for (size_t u : users[v])
            if (!is_alias_kind(plan.instructions[u])) out.push_back(u);
      return out;
    };
    auto subset_of = [&](const std::vector<size_t>& a, const std::vector<size_t>& nodes) {
      for (size_t x : a)
        if (std::find(nodes.begin(), nodes.end(), x) == nodes.end()) return false;
      return true;
    };
    auto in_step = [&](const Step& f, uint32_t v) -> const Instruction* {
      const long pi = producer[v];
      if (pi < 0 || std::find(f.nodes.begin(), f.nodes.end(), (size_t)pi) == f.nodes.end()) return nullptr;
      return &plan.instructions[pi];
    };
    auto scalar_f32 = [&](uint32_t v, float* out) {
      long pi = producer[v];
      if (pi >= 0 && plan.instructions[pi].kind == Kind::broadcast_in_dim) {
        v = plan.instructions[pi].inputs[0];
        pi = producer[v];
      }
      if (pi < 0 || plan.instructions[pi].kind != Kind::constant) return false;
      const Instruction& c = plan.instructions[pi];
      if (plan.values[v].dtype != kF32 || c.literal.size() != 4) return false;
      memcpy(out, c.literal.data(), 4);
      return true;
    };
    auto non_alias_nodes = [&](const Step& f) {
      size_t n = 0;
      for (size_t i : f.nodes) n += is_alias_kind(plan.instructions[i]) ? 0 : 1;
      return n;
    };
    auto replace_value = [](std::vector<uint32_t>& list, uint32_t from, uint32_t to) {
      for (uint32_t& v : list)
        if (v == from) v = to;
    };
    auto add_unique = [](std::vector<uint32_t>& list, uint32_t v) {
      if (std::find(list.begin(), list.end(), v) == list.end()) list.push_back(v);
    };

    // silu(gate) * up feeding the lhs of D.
    auto match_silu = [&](const Step& f, Step& d) {
      if (f.type != Step::kFused || f.fused.row || f.outputs.size() != 1 || !f.fused.scatter_dst.empty()) return false;
      DotSeg& seg = d.segs[0];
      const uint32_t act = f.outputs[0];
      if (fusion_debug)
        fprintf(stderr, "pjrtx_b200 fusion: silu candidate lhs=%u act=%u nodes=%zu users_ok=%d\n", seg.lhs, act, non_alias_nodes(f),
                (int)subset_of(class_users(act), d.nodes));
      if (seg.lhs != act || is_output[act] || non_alias_nodes(f) != 3) return false;
      if (!subset_of(class_users(act), d.nodes)) return false;
      const Instruction* top = nullptr;
      for (size_t i : f.nodes)
        if (plan.instructions[i].kind == Kind::multiply && kp->root[plan.instructions[i].outputs[0]] == act) top = &plan.instructions[i];
      if (!top) return false;
      for (int swap_top = 0; swap_top < 2; swap_top++) {
        const uint32_t t2 = top->inputs[swap_top], u = top->inputs[1 - swap_top];
        const Instruction* inner = in_step(f, t2);
        if (!inner || inner->kind != Kind::multiply || in_step(f, u)) continue;
        for (int swap_in = 0; swap_in < 2; swap_in++) {
          const uint32_t g = inner->inputs[swap_in], sg = inner->inputs[1 - swap_in];
          const Instruction* lg = in_step(f, sg);
          if (!lg || lg->kind != Kind::logistic || lg->inputs[0] != g || in_step(f, g)) continue;
          const Value& gv = plan.values[g];
          const Value& uv = plan.values[u];
          if (gv.dtype != seg.group[0].dtype || uv.dtype != gv.dtype || gv.dims != uv.dims) continue;
          if ((int64_t)gv.count() != seg.group[0].m * seg.group[0].k || seg.group[0].lhs_k != 1 ||
              (seg.group[0].m > 1 && seg.group[0].lhs_m != seg.group[0].k))
            continue;
          seg.lhs = kp->root[g];
          seg.lhs2 = kp->root[u];
          seg.lhs_desc.kind = kDotLhsSiluMul;
          replace_value(d.inputs, act, seg.lhs);
          add_unique(d.inputs, seg.lhs2);
          return true;
        }
      }
      return false;
    };

    // RMSNorm(x) * gain feeding the lhs of D, x optionally the sum of two values one of which P produced.
    auto match_norm = [&](const Step& f, Step& d, Step* p) {
      if (f.type != Step::kFused || !f.fused.row || !f.fused.scatter_dst.empty() || f.outputs.empty() || f.outputs.size() > 2) return false;
      DotSeg& seg = d.segs[0];
      const uint32_t h = seg.lhs;
      if (std::find(f.outputs.begin(), f.outputs.end(), h) == f.outputs.end() || is_output[h]) return false;
      if (!subset_of(class_users(h), d.nodes)) return false;
      const int dt = seg.group[0].dtype;
      if (dt != kBF16 && dt != kF16) return false;
      const Instruction* top = nullptr;
      for (size_t i : f.nodes)
        if (plan.instructions[i].kind == Kind::multiply && kp->root[plan.instructions[i].outputs[0]] == h) top = &plan.instructions[i];
      if (!top) return false;
      std::set<const Instruction*> seen;
      auto pick = [&](const Instruction* ins, Kind first_kind, uint32_t* a, uint32_t* b) {
        // Orders the two operands of a commutative instruction so that *a is produced inside the step by `first_kind`.
        for (int sw = 0; sw < 2; sw++) {
          const Instruction* q = in_step(f, ins->inputs[sw]);
          if (q && q->kind == first_kind) {
            *a = ins->inputs[sw];
            *b = ins->inputs[1 - sw];
            return true;
          }
        }
        return false;
      };
      uint32_t xn, wb;
      if (!pick(top, Kind::convert, &xn, &wb)) return false;
      const Instruction* wbi = in_step(f, wb);
      if (!wbi || wbi->kind != Kind::broadcast_in_dim) return false;
      const uint32_t w = wbi->inputs[0];
      const Value& hv = plan.values[top->outputs[0]];
      const size_t rank = hv.dims.size();
      if (rank != 2 || in_step(f, w) || plan.values[w].dims.size() != 1 || plan.values[w].dims[0] != hv.dims[1] ||
          plan.values[w].dtype != dt || wbi->list("broadcast_dimensions") != std::vector<int64_t>{1})
        return false;
      const Instruction* xni = in_step(f, xn);
      const Instruction* mul32 = in_step(f, xni->inputs[0]);
      if (!mul32 || mul32->kind != Kind::multiply || plan.values[mul32->outputs[0]].dtype != kF32 || hv.dtype != dt) return false;
      uint32_t xf, rb;
      if (!pick(mul32, Kind::convert, &xf, &rb)) return false;
      const Instruction* xfi = in_step(f, xf);
      const Instruction* rbi = in_step(f, rb);
      if (!rbi || rbi->kind != Kind::broadcast_in_dim || rbi->list("broadcast_dimensions") != std::vector<int64_t>{0}) return false;
      const Instruction* rs = in_step(f, rbi->inputs[0]);
      if (!rs || rs->kind != Kind::rsqrt) return false;
      const Instruction* addi = in_step(f, rs->inputs[0]);
      if (!addi || addi->kind != Kind::add) return false;
      uint32_t mean, ceps;
      if (!pick(addi, Kind::multiply, &mean, &ceps)) return false;
      const Instruction* meani = in_step(f, mean);
      uint32_t ssum, cscale;
      if (!pick(meani, Kind::reduce_sum, &ssum, &cscale)) return false;
      const Instruction* sumi = in_step(f, ssum);
      if (sumi->outputs.size() != 1 || sumi->list("reduce_dimensions") != std::vector<int64_t>{1}) return false;
      const Instruction* sq = in_step(f, sumi->inputs[0]);
      if (!sq || sq->kind != Kind::multiply || sq->inputs[0] != xf || sq->inputs[1] != xf) return false;
      float scale = 0.f, eps = 0.f;
      if (!scalar_f32(cscale, &scale) || !scalar_f32(ceps, &eps)) return false;
      const uint32_t xs = xfi->inputs[0];
      if (plan.values[xs].dtype != dt || plan.values[xs].dims != hv.dims) return false;
      if ((int64_t)hv.dims[0] != seg.group[0].m || (int64_t)hv.dims[1] != seg.group[0].k || seg.group[0].lhs_k != 1 ||
          (seg.group[0].m > 1 && seg.group[0].lhs_m != seg.group[0].k))
        return false;
      size_t matched = 11;  // top, wb, xn, mul32, xf, rb, rsqrt, add, mean, sum, square (+ broadcasts of the scalars)
      for (uint32_t c : {cscale, ceps})
        if (const Instruction* q = in_step(f, c)) matched += q->kind == Kind::broadcast_in_dim ? 1 : 100;
      const Instruction* addx = in_step(f, xs);
      uint32_t lhs_root;
      if (!addx) {
        if (f.outputs.size() != 1 || non_alias_nodes(f) != matched) return false;
        lhs_root = kp->root[xs];
      } else {
        // x = a + b: one addend is the result of the previous contraction (read by nothing else), the other the residual.
        if (addx->kind != Kind::add || non_alias_nodes(f) != matched + 1 || !p || p->segs.empty()) return false;
        if (f.outputs.size() == 2 && std::find(f.outputs.begin(), f.outputs.end(), kp->root[xs]) == f.outputs.end()) return false;
        if (f.outputs.size() == 1 && !class_users(kp->root[xs]).empty() && !subset_of(class_users(kp->root[xs]), f.nodes)) return false;
        DotSeg& ps = p->segs.back();
        int slot = -1;
        uint32_t res = UINT32_MAX;
        for (int sw = 0; sw < 2 && slot < 0; sw++) {
          const uint32_t y = kp->root[addx->inputs[sw]], other = kp->root[addx->inputs[1 - sw]];
          for (size_t j = 0; j < ps.out.size(); j++)
            if (ps.out[j] == y && ps.residual[j] == UINT32_MAX && !is_output[y] &&
                std::find(ps.out.begin(), ps.out.end(), other) == ps.out.end() && in_step(f, addx->inputs[1 - sw]) == nullptr &&
                class_users(y) == std::vector<size_t>{(size_t)(addx - plan.instructions.data())}) {
              slot = (int)j;
              res = other;
            }
        }
        if (slot < 0 || plan.values[res].dims != hv.dims || plan.values[res].dtype != dt) return false;
        const DotShape& pd = ps.group[slot];
        if (pd.m != (int64_t)hv.dims[0] || pd.n != (int64_t)hv.dims[1] || pd.out_m != pd.n) return false;
        const uint32_t y = ps.out[slot];
        lhs_root = kp->root[xs];
        ps.residual[slot] = res;
        ps.out[slot] = lhs_root;
        replace_value(p->outputs, y, lhs_root);
        add_unique(p->inputs, res);
      }
      seg.lhs = lhs_root;
      seg.lhs2 = kp->root[w];
      seg.lhs_desc.kind = kDotLhsRmsNorm;
      seg.lhs_desc.norm_scale = scale;
      seg.lhs_desc.norm_eps = eps;
      replace_value(d.inputs, h, lhs_root);
      add_unique(d.inputs, seg.lhs2);
      return true;
    };

    std::vector<Step> fused;
    for (size_t i = 0; i < kp->steps.size(); i++) {
      Step& d = kp->steps[i];
      if (!d.segs.empty() && !fused.empty() && fused.back().type == Step::kFused) {
        Step* prev_dot = fused.size() >= 2 && !fused[fused.size() - 2].segs.empty() ? &fused[fused.size() - 2] : nullptr;
        if (match_silu(fused.back(), d) || (!fuse_silu_only && match_norm(fused.back(), d, prev_dot))) {
          for (size_t n : fused.back().nodes) d.nodes.push_back(n);
          fused.pop_back();
        }
      }
      fused.push_back(std::move(d));
    }
    kp->steps = std::move(fused);

    if (env_flag_local("PJRTX_B200_DOT_CHAIN", false)) {
      std::vector<Step> chained;
      for (Step& st : kp->steps) {
        Step* prev = chained.empty() ? nullptr : &chained.back();
        const bool can = prev && !prev->segs.empty() && !st.segs.empty() &&
                         prev->segs.size() + st.segs.size() <= (size_t)kDotChainMax &&
                         prev->segs[0].group[0].dtype == st.segs[0].group[0].dtype &&
                         prev->segs[0].group[0].m == st.segs[0].group[0].m;
        if (!can) {
          chained.push_back(std::move(st));
          continue;
        }
        for (DotSeg& sg : st.segs) prev->segs.push_back(std::move(sg));
        for (size_t n : st.nodes) prev->nodes.push_back(n);
        for (uint32_t v : st.inputs) add_unique(prev->inputs, v);
        for (uint32_t v : st.outputs) add_unique(prev->outputs, v);
      }
      kp->steps = std::move(chained);
    }
    for (Step& st : kp->steps) {
      if (st.segs.empty()) continue;
      if (st.segs.size() == 1 && st.segs[0].lhs_desc.kind == kDotLhsPlain &&
          std::all_of(st.segs[0].residual.begin(), st.segs[0].residual.end(), [](uint32_t r) { return r == UINT32_MAX; })) {
        st.segs.clear();  // nothing folded in: the plain launch
        continue;
      }
      std::vector<DotChainSegment> desc(st.segs.size());
      for (size_t q = 0; q < st.segs.size(); q++) {
        desc[q].count = (int)st.segs[q].group.size();
        for (int g = 0; g < desc[q].count; g++) desc[q].shapes[g] = st.segs[q].group[g];
        desc[q].lhs = st.segs[q].lhs_desc;
        desc[q].norm_of_previous = q > 0 && st.segs[q - 1].out.size() == 1 && st.segs[q - 1].out[0] == st.segs[q].lhs;
      }
      st.chain_plan = dot_chain_plan(desc.data(), (int)desc.size(), sm_count);
      st.dot_scratch.partial_bytes = st.chain_plan.partial_bytes;
      st.dot_scratch.counter_bytes = st.chain_plan.counter_bytes;
      st.dot_scratch.grid = st.chain_plan.grid;
    }
  }

  // Storage: parameters, constants, arena intervals for everything produced by a step.
  kp->storage.assign(nv, Storage{});
  for (size_t p = 0; p < kp->params.size(); p++) kp->storage[kp->params[p]] = Storage{Storage::kParameter, 0, (uint32_t)p};
  for (size_t n = 0; n < ni; n++)
    if (plan.instructions[n].kind == Kind::constant) {
      kp->storage[plan.instructions[n].outputs[0]] = Storage{Storage::kConstant, 0, (uint32_t)kp->constants.size()};
      kp->constants.push_back(n);
    }
  const size_t ns = kp->steps.size();
  std::vector<long> first_write(nv, -1), last_touch(nv, -1);
  for (size_t s = 0; s < ns; s++) {
    for (uint32_t r : kp->steps[s].outputs) {
      if (first_write[r] < 0) first_write[r] = (long)s;
      last_touch[r] = (long)s;
    }
    for (uint32_t r : kp->steps[s].inputs) last_touch[r] = std::max(last_touch[r], (long)s);
  }
  for (size_t v = 0; v < nv; v++)
    if (is_output[v]) last_touch[kp->root[v]] = (long)ns;  // lives to the end
  // Small non-donated parameters get a staging slot so a captured graph reads a fixed address.
  uint64_t top = 0;
  kp->param_slot.assign(kp->params.size(), UINT64_MAX);
  for (size_t p = 0; p < kp->params.size(); p++) {
    const Value& v = plan.values[kp->params[p]];
    if (!kp->param_donated[p] && v.bytes() <= 4096) {
      kp->param_slot[p] = top;
      top += align_up(std::max<uint64_t>(v.bytes(), 1));
    }
  }
  const uint64_t slots_end = top;
  struct Block { uint64_t offset, size; long free_after; };
  std::vector<Block> live;
  uint64_t high = slots_end;
  for (size_t s = 0; s < ns; s++) {
    for (uint32_t r : kp->steps[s].outputs) {
      if (kp->storage[r].kind != Storage::kNone) continue;  // parameter storage (in-place update) or already placed
      uint64_t size = align_up(std::max<uint64_t>(plan.values[r].bytes(), 1));
      // Drop blocks whose last reader ran before this step, then first-fit.
      live.erase(std::remove_if(live.begin(), live.end(), [&](const Block& b) { return b.free_after < (long)s; }), live.end());
      std::sort(live.begin(), live.end(), [](const Block& a, const Block& b) { return a.offset < b.offset; });
      uint64_t at = slots_end;
      for (const Block& b : live) {
        if (at + size <= b.offset) break;
        at = std::max(at, b.offset + b.size);
      }
      live.push_back(Block{at, size, last_touch[r]});
      high = std::max(high, at + size);
      kp->storage[r] = Storage{Storage::kArena, at, 0};
    }
  }
  kp->arena_bytes = high;
  // Contractions whose rhs no step ever writes may start copying it before their predecessor finishes.
  {
    std::set<uint32_t> written;
    for (const Step& st : kp->steps)
      for (uint32_t r : st.outputs) written.insert(r);
    for (Step& st : kp->steps) {
      if (st.type != Step::kDot) continue;
      bool ok = true;
      std::vector<uint32_t> weights;
      if (st.segs.empty()) weights.assign(st.inputs.begin() + 1, st.inputs.end());
      for (const DotSeg& sg : st.segs) weights.insert(weights.end(), sg.rhs.begin(), sg.rhs.end());
      for (uint32_t wv : weights) {
        const Storage& sg = kp->storage[wv];
        ok &= (sg.kind == Storage::kParameter || sg.kind == Storage::kConstant) && !written.count(wv);
      }
      st.early_rhs = ok;
    }
  }
  // Decode attention whose caches are only touched, earlier in the step, by the in-place write of the row at its own
  // token index: the rows below that index hold what previous steps left, so the kernel may request them before its
  // predecessor has finished. The token itself must be a parameter no step writes.
  {
    std::set<uint32_t> written;
    for (const Step& st : kp->steps)
      for (uint32_t r : st.outputs) written.insert(r);
    for (size_t si = 0; si < kp->steps.size(); si++) {
      Step& st = kp->steps[si];
      if (st.type != Step::kAttnDecode || st.inputs.size() < 4) continue;
      const uint32_t tok = st.inputs[3];
      if (kp->storage[tok].kind != Storage::kParameter || written.count(tok)) continue;
      bool ok = true;
      for (int which = 1; which <= 2 && ok; which++) {
        const uint32_t cache = st.inputs[which];
        if (plan.values[cache].dims.size() != 4) ok = false;
        for (size_t e = 0; e < si && ok; e++) {
          const Step& w = kp->steps[e];
          if (std::find(w.outputs.begin(), w.outputs.end(), cache) == w.outputs.end()) continue;
          if (w.type != Step::kFused) ok = false;
          for (size_t n : w.nodes) {
            const Instruction& wi = plan.instructions[n];
            bool touches = false;
            for (uint32_t o : wi.outputs) touches |= kp->root[o] == cache;
            if (!touches || !ok) continue;
            if (wi.kind != Kind::dynamic_update_slice || wi.inputs.size() != 6) {
              ok = false;
              continue;
            }
            const Value& up = plan.values[wi.inputs[1]];
            if (up.dims.size() != 4 || up.dims[1] != 1 || kp->root[wi.inputs[3]] != tok) ok = false;
          }
        }
      }
      st.early_kv = ok;
    }
  }
  // Scratch for split-K partials and their counters (counters first: they must start at zero).
  uint64_t scratch = 0;
  for (Step& st : kp->steps)
    if (st.type == Step::kDot && st.dot_scratch.counter_bytes) {
      st.counter_offset = scratch;
      scratch += align_up(st.dot_scratch.counter_bytes);
    } else if (st.type == Step::kAttnDecode) {
      st.counter_offset = scratch;
      scratch += align_up(st.attn_plan.counter_bytes);
    }
  uint64_t counters_end = scratch;
  uint64_t partial_max = 0;
  for (Step& st : kp->steps)
    if (st.type == Step::kDot && st.dot_scratch.partial_bytes) {
      st.scratch_offset = counters_end;  // partials are consumed inside the launch that wrote them: one shared region
      partial_max = std::max(partial_max, align_up(st.dot_scratch.partial_bytes));
    } else if (st.type == Step::kAttnDecode) {
      st.scratch_offset = counters_end;
      partial_max = std::max(partial_max, align_up(st.attn_plan.workspace_bytes));
    }
  kp->scratch_bytes = counters_end + partial_max;
  return true;
}

std::string step_type_name(Step::Type t) {
  static const char* names[] = {"fused", "dot", "slice_update", "sdpa", "all_reduce", "all_gather", "copy", "attention_decode",
                                "attention_prefill"};
  return names[(int)t];
}

std::string describe_steps(const KernelPlan& kp, bool with_source) {
  std::string s = strfmt("{\"arena_bytes\":%llu,\"scratch_bytes\":%llu,\"steps\":[", (unsigned long long)kp.arena_bytes,
                         (unsigned long long)kp.scratch_bytes);
  for (size_t i = 0; i < kp.steps.size(); i++) {
    const Step& st = kp.steps[i];
    s += strfmt("%s{\"type\":\"%s\",\"nodes\":[", i ? "," : "", step_type_name(st.type).c_str());
    for (size_t n = 0; n < st.nodes.size(); n++) s += strfmt(n ? ",%zu" : "%zu", st.nodes[n]);
    s += "]";
    if (st.type == Step::kFused) {
      s += strfmt(",\"row\":%s,\"rows\":%lld,\"cols\":%lld,\"n\":%lld,\"vec\":%d,\"block\":%d,\"grid\":%lld,\"stages\":%d,"
                  "\"reduces\":%d,\"inputs\":%zu,\"outputs\":%zu",
                  st.fused.row ? "true" : "false", (long long)st.fused.rows, (long long)st.fused.cols, (long long)st.fused.n,
                  st.fused.vec, st.fused.block, (long long)st.fused.grid, st.fused.stages, st.fused.reduce_count,
                  st.fused.inputs.size(), st.fused.outputs.size());
      if (with_source) {
        std::string esc;
        for (char c : st.fused.source) {
          if (c == '"' || c == '\\') { esc += '\\'; esc += c; }
          else if (c == '\n') esc += "\\n";
          else if (c == '\t') esc += "\\t";
          else esc += c;
        }
        s += ",\"source\":\"" + esc + "\"";
      }
    } else if (st.type == Step::kDot) {
      long long n_total = st.dot.n;
      if (st.dot_group.size() > 1) {
        n_total = 0;
        for (const DotShape& d : st.dot_group) n_total += d.n;
      }
      s += strfmt(",\"path\":%d,\"tma\":%d,\"umma\":%d,\"grid\":%d,\"ksplit\":%d,\"b0\":%lld,\"b1\":%lld,\"m\":%lld,\"n\":%lld,\"k\":%lld,\"group\":%zu",
                  st.dot_scratch.path, st.dot_scratch.tma, st.dot_scratch.umma, st.dot_scratch.grid, st.dot_scratch.ksplit, (long long)st.dot.b0, (long long)st.dot.b1, (long long)st.dot.m,
                  n_total, (long long)st.dot.k, std::max<size_t>(st.dot_group.size(), 1));
      long long weight_elems = 0;
      if (st.segs.empty()) {
        weight_elems = n_total * (long long)st.dot.k * st.dot.b0 * st.dot.b1;
      } else {
        s += strfmt(",\"segments\":%zu,\"lhs_kinds\":[", st.segs.size());
        for (size_t q = 0; q < st.segs.size(); q++) {
          s += strfmt(q ? ",%d" : "%d", st.segs[q].lhs_desc.kind);
          for (const DotShape& d : st.segs[q].group) weight_elems += (long long)d.k * d.n;
        }
        s += "],\"residuals\":";
        size_t residuals = 0;
        for (const DotSeg& sg : st.segs)
          for (uint32_t r : sg.residual) residuals += r != UINT32_MAX;
        s += strfmt("%zu", residuals);
      }
      s += strfmt(",\"weight_elems\":%lld,\"rhs_s8\":%d", weight_elems, st.dot.rhs_s8);
    } else if (st.type == Step::kSliceUpdate) {
      s += strfmt(",\"in_place\":%s", st.in_place ? "true" : "false");
    } else if (st.type == Step::kAttnDecode) {
      s += strfmt(",\"mma\":%d,\"early_kv\":%d,\"splits\":%d,\"batch\":%lld,\"heads\":%lld,\"kv_heads\":%lld,\"kv_len\":%lld,\"head_dim\":%lld",
                  st.attn_plan.mma, st.early_kv ? 1 : 0, st.attn_plan.splits, st.attn.batch, st.attn.heads, st.attn.kv_heads, st.attn.kv_len, st.attn.head_dim);
    } else if (st.type == Step::kAttnPrefill) {
      s += strfmt(",\"batch\":%lld,\"kv_heads\":%lld,\"rep\":%lld,\"seq\":%lld,\"head_dim\":%lld", st.attn_prefill.batch,
                  st.attn_prefill.kv_heads, st.attn_prefill.rep, st.attn_prefill.seq, st.attn_prefill.head_dim);
    }
    s += "}";
  }
  return s + "]}";
}

}  // namespace

std::string lowering_diagnostic(const Plan& plan, size_t device_count) {
  Plan p = rewrite_plan(plan);
  Issue issue;
  if (!lowering_issue(p, device_count, &issue)) return "";
  return format_issue(p, issue);
}

std::string describe_kernel_plan(const Plan& plan, std::string* error) {
  KernelPlan kp;
  if (!plan_kernels(plan, 148, &kp, error)) return "";
  return describe_steps(kp, true);
}

// ---------------------------------------------------------------------------
// Executable.

struct DeviceState {
  Device* dev = nullptr;
  std::vector<void*> constants;
  void* arena = nullptr;
  void* scratch = nullptr;
  cudaGraphExec_t graph = nullptr;
  std::vector<void*> graph_param_ptrs;  // pointers the graph was captured with
};

struct Executable {
  KernelPlan kp;
  std::vector<int> device_ordinals;
  std::vector<DeviceState> devices;
  ExecutableStats stats;
  bool use_graph = false;
  bool pdl = false;  // programmatic dependent launch between consecutive kernels
  bool profiling = false;
  std::vector<float> step_ms;
  std::vector<cudaEvent_t> step_events;
  std::mutex mu;
};

namespace {

bool env_flag(const char* name, bool fallback) {
  const char* v = getenv(name);
  if (!v || !*v) return fallback;
  return !(v[0] == '0' || v[0] == 'f' || v[0] == 'F' || v[0] == 'n' || v[0] == 'N');
}

bool profile_enabled() {
  static int on = -1;
  if (on < 0) on = env_flag("PJRTX_PROFILE", false) ? 1 : 0;
  return on == 1;
}

struct Pointers {
  const KernelPlan* kp;
  const DeviceState* ds;
  const std::vector<void*>* param_ptrs;
  std::vector<void*> fresh;  // per value, outputs allocated outside the arena (direct mode)
  void* of(uint32_t value) const {
    uint32_t r = kp->root[value];
    const Storage& st = kp->storage[r];
    switch (st.kind) {
      case Storage::kParameter: return (*param_ptrs)[st.index];
      case Storage::kConstant: return ds->constants[st.index];
      case Storage::kArena:
        if (!fresh.empty() && fresh[r]) return fresh[r];
        return (char*)ds->arena + st.offset;
      default: return nullptr;
    }
  }
};

// Inside a stream capture an ordinary event record only marks a dependency; the external flag makes it a graph node
// that takes a timestamp every time the graph runs.
void record_step_event(cudaEvent_t event, cudaStream_t stream, bool capturing) {
  if (capturing) cudaEventRecordWithFlags(event, stream, cudaEventRecordExternal);
  else cudaEventRecord(event, stream);
}

// Waits for the last step event and fills step_ms from consecutive event pairs.
void collect_step_times(Executable* exe) {
  const size_t n = exe->kp.steps.size();
  cudaEventSynchronize(exe->step_events[n + 1]);
  exe->step_ms.assign(n, 0.f);
  for (size_t k = 0; k < n; k++) cudaEventElapsedTime(&exe->step_ms[k], exe->step_events[k], exe->step_events[k + 1]);
  // The last two records have nothing between them: their distance is what the records themselves cost.
  float gap_ms = 0.f;
  if (cudaEventElapsedTime(&gap_ms, exe->step_events[n], exe->step_events[n + 1]) == cudaSuccess && gap_ms > 0.f)
    exe->stats.profile_event_gap_ns = (uint64_t)(gap_ms * 1e6f);
}

// `timed`: an event is recorded before every step and after the last one. Outside a stream capture the call then
// waits and fills step_ms; inside a capture (`capturing`) the records become graph nodes and the caller reads the
// times after it has launched the graph (collect_step_times).
//
// `ordered_first`: the first kernel of the call is launched without the programmatic-launch attribute. Outside a graph
// the stream predecessor of that kernel belongs to other work (another executable that may still be writing a buffer
// this one treats as a never-written weight, or this executable's previous run); a fully ordered first kernel makes
// every later kernel of the call, which waits on its predecessor, ordered after that work too. A graph launch is
// ordered as a whole, so captures do not need it.
bool run_steps(Executable* exe, DeviceState& ds, const Pointers& ptr, uint64_t* launches, std::string* error,
               bool timed = false, bool capturing = false, bool ordered_first = false) {
  Device* dev = ds.dev;
  const KernelPlan& kp = exe->kp;
  const bool pdl_setting = exe->pdl;
  struct RestorePdl {
    Executable* exe;
    bool value;
    ~RestorePdl() { exe->pdl = value; }
  } restore{exe, pdl_setting};
  const uint64_t launches_at_entry = *launches;
  if (timed) {
    while (exe->step_events.size() < kp.steps.size() + 2) {
      cudaEvent_t e;
      cudaEventCreate(&e);
      exe->step_events.push_back(e);
    }
    record_step_event(exe->step_events[0], dev->stream, capturing);
  }
  size_t step_index = 0;
  for (const Step& st : kp.steps) {
    if (timed && step_index > 0) record_step_event(exe->step_events[step_index], dev->stream, capturing);
    step_index++;
    exe->pdl = pdl_setting && !(ordered_first && *launches == launches_at_entry);
#ifdef PJRTX_DEBUG_SKIP
    {
      // Timing diagnostic of a special build only: leave out every step of the named types (results are then wrong).
      static const char* skip = getenv("PJRTX_DEBUG_SKIP");
      if (skip && strstr(skip, ("," + step_type_name(st.type) + ",").c_str())) continue;
    }
#endif
    switch (st.type) {
      case Step::kFused: {
        std::vector<void*> addr;
        for (uint32_t v : st.fused.inputs) addr.push_back(ptr.of(v));
        for (uint32_t v : st.fused.outputs) addr.push_back(ptr.of(v));
        for (uint32_t v : st.fused.scatter_dst) addr.push_back(ptr.of(v));
        std::vector<void*> args(addr.size());
        for (size_t k = 0; k < addr.size(); k++) args[k] = &addr[k];
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)st.fused.grid);
        cfg.blockDim = dim3((unsigned)st.fused.block);
        cfg.stream = dev->stream;
        cudaLaunchAttribute attr[2];
        cfg.attrs = attr;
        cfg.numAttrs = fill_launch_attributes(attr, exe->pdl);
        cudaError_t e = cudaLaunchKernelExC(&cfg, (const void*)st.jit->kernel, args.data());
        if (e != cudaSuccess) {
          *error = std::string("fused kernel launch failed: ") + cudaGetErrorString(e);
          return false;
        }
        (*launches)++;
        break;
      }
      case Step::kDot: {
        void* partials = st.dot_scratch.partial_bytes ? (char*)ds.scratch + st.scratch_offset : nullptr;
        void* counters = st.dot_scratch.counter_bytes ? (char*)ds.scratch + st.counter_offset : nullptr;
        int n;
        if (!st.segs.empty()) {
          DotChainSegment desc[kDotChainMax];
          DotChainArgs cargs[kDotChainMax];
          for (size_t q = 0; q < st.segs.size(); q++) {
            const DotSeg& sg = st.segs[q];
            desc[q].count = (int)sg.group.size();
            desc[q].lhs = sg.lhs_desc;
            desc[q].norm_of_previous = q > 0 && st.segs[q - 1].out.size() == 1 && st.segs[q - 1].out[0] == sg.lhs;
            cargs[q].lhs = ptr.of(sg.lhs);
            cargs[q].lhs2 = sg.lhs2 == UINT32_MAX ? nullptr : ptr.of(sg.lhs2);
            for (size_t g = 0; g < sg.group.size(); g++) {
              desc[q].shapes[g] = sg.group[g];
              cargs[q].rhs[g] = ptr.of(sg.rhs[g]);
              cargs[q].out[g] = ptr.of(sg.out[g]);
              cargs[q].residual[g] = sg.residual[g] == UINT32_MAX ? nullptr : ptr.of(sg.residual[g]);
            }
          }
          n = dot_chain_launch(desc, cargs, (int)st.segs.size(), st.chain_plan, partials, counters, dev->error_flag_dev,
                               st.early_rhs, exe->pdl, dev->stream);
        } else if (st.dot_group.size() > 1) {
          const void* rhs[kDotGroupMax];
          const void* scales[kDotGroupMax] = {nullptr, nullptr, nullptr, nullptr};
          void* out[kDotGroupMax];
          for (size_t g = 0; g < st.dot_group.size(); g++) {
            rhs[g] = ptr.of(st.inputs[1 + g]);
            out[g] = ptr.of(st.outputs[g]);
            if (g < st.dot_scales.size()) scales[g] = ptr.of(st.dot_scales[g]);
          }
          n = dot_group_launch(st.dot_group.data(), (int)st.dot_group.size(), st.dot_scratch, ptr.of(st.inputs[0]), rhs, out,
                               partials, counters, dev->error_flag_dev, st.early_rhs, exe->pdl, dev->stream, scales);
        } else {
          n = dot_launch(st.dot, st.dot_scratch, ptr.of(st.inputs[0]), ptr.of(st.inputs[1]), ptr.of(st.outputs[0]), partials,
                         counters, dev->error_flag_dev, st.early_rhs, exe->pdl, dev->stream,
                         st.dot_scales.empty() ? nullptr : ptr.of(st.dot_scales[0]));
        }
        if (n == 0) {
          *error = "dot_general kernel refused the shape";
          return false;
        }
        *launches += n;
        break;
      }
      case Step::kSliceUpdate: {
        void* dst = ptr.of(st.outputs[0]);
        if (!st.in_place) {
          if (cudaMemcpyAsync(dst, ptr.of(st.inputs[0]), st.bytes, cudaMemcpyDeviceToDevice, dev->stream) != cudaSuccess) {
            *error = "dynamic_update_slice operand copy failed";
            return false;
          }
          (*launches)++;
        }
        const void* starts[8] = {nullptr};
        for (int d = 0; d < st.dus.rank; d++) starts[d] = ptr.of(st.inputs[2 + d]);
        if (!dus_launch(st.dus, dst, ptr.of(st.inputs[1]), starts, exe->pdl, dev->stream)) {
          *error = "dynamic_update_slice kernel refused the shape";
          return false;
        }
        (*launches)++;
        break;
      }
      case Step::kAttnDecode: {
        // The contraction that follows streams weights nothing writes: let the attention CTAs ask for them.
        const void* next_weights = nullptr;
        uint64_t next_bytes = 0;
        if (step_index < kp.steps.size()) {
          const Step& nx = kp.steps[step_index];  // step_index already points past this step
          if (nx.type == Step::kDot && nx.early_rhs && nx.dot.b0 * nx.dot.b1 == 1) {
            const DotShape& d = nx.segs.empty() ? nx.dot : nx.segs[0].group[0];
            const uint32_t w = nx.segs.empty() ? nx.inputs[1] : nx.segs[0].rhs[0];
            if (d.rhs_n == 1 && d.rhs_k == d.n) {
              next_weights = ptr.of(w);
              next_bytes = std::min<uint64_t>((uint64_t)d.k * d.n * dtype_size(d.dtype), 48ull << 20);
            }
          }
        }
        if (!attn_decode_launch(st.attn, st.attn_plan, ptr.of(st.inputs[0]), ptr.of(st.inputs[1]), ptr.of(st.inputs[2]),
                                ptr.of(st.inputs[3]), ptr.of(st.outputs[0]), (char*)ds.scratch + st.scratch_offset,
                                (char*)ds.scratch + st.counter_offset, exe->pdl, dev->stream, st.early_kv, dev->error_flag_dev,
                                next_weights, next_bytes)) {
          *error = "attention kernel refused the shape";
          return false;
        }
        (*launches)++;
        break;
      }
      case Step::kAttnPrefill:
        if (!attn_prefill_launch(st.attn_prefill, ptr.of(st.inputs[0]), ptr.of(st.inputs[1]), ptr.of(st.inputs[2]),
                                 ptr.of(st.outputs[0]), exe->pdl, dev->stream, dev->error_flag_dev)) {
          *error = "attention kernel refused the shape";
          return false;
        }
        (*launches)++;
        break;
      case Step::kSdpa:
        if (!sdpa_launch(st.sdpa, ptr.of(st.inputs[0]), ptr.of(st.inputs[1]), ptr.of(st.inputs[2]), ptr.of(st.inputs[3]),
                         ptr.of(st.outputs[0]), exe->pdl, dev->stream)) {
          *error = "attention kernel refused the shape";
          return false;
        }
        (*launches)++;
        break;
      case Step::kAllReduce:
        if (!comm_all_reduce_sum(dev, ptr.of(st.inputs[0]), ptr.of(st.outputs[0]), st.count, st.dtype, exe->pdl)) {
          *error = last_error();
          return false;
        }
        (*launches)++;
        break;
      case Step::kAllGather:
        if (!comm_all_gather(dev, ptr.of(st.inputs[0]), ptr.of(st.outputs[0]), st.count, st.dtype)) {
          *error = last_error();
          return false;
        }
        (*launches)++;
        break;
      case Step::kCopy:
        break;
    }
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    *error = std::string("kernel launch failed: ") + cudaGetErrorString(e);
    return false;
  }
  if (timed) {
    record_step_event(exe->step_events[kp.steps.size()], dev->stream, capturing);
    record_step_event(exe->step_events[kp.steps.size() + 1], dev->stream, capturing);  // an empty interval: calibration
    if (!capturing) collect_step_times(exe);
  }
  return true;
}

}  // namespace

void executable_set_profiling(Executable* exe, bool enabled) {
  std::lock_guard<std::mutex> lock(exe->mu);
  exe->profiling = enabled;
}

std::vector<float> executable_step_times(Executable* exe) {
  std::lock_guard<std::mutex> lock(exe->mu);
  return exe->step_ms;
}

Executable* compile_executable(const Plan& plan, const std::vector<int>& device_ordinals, std::string* error) {
  if (device_ordinals.empty()) {
    *error = "invalid executable plan: pass=b200-backend-legalization detail=\"backend executable requires at least one device\" "
             "feature=b200-device-assignment";
    return nullptr;
  }
  auto exe = std::make_unique<Executable>();
  std::vector<Device*> devs;
  for (int ord : device_ordinals) {
    Device* d = get_device(ord);
    if (!d) {
      *error = last_error();
      return nullptr;
    }
    devs.push_back(d);
  }
  if (!plan_kernels(plan, devs[0]->sm_count, &exe->kp, error)) return nullptr;
  KernelPlan& kp = exe->kp;
  exe->device_ordinals = device_ordinals;
  // Generated kernels: compile once per distinct source.
  uint64_t generated = 0;
  for (Step& st : kp.steps) {
    if (st.type != Step::kFused) continue;
    std::string log;
    st.jit = jit_get_kernel(st.fused.source, st.fused.name.c_str(), &log);
    if (!st.jit) {
      *error = "generated fusion kernel failed to compile: " + log;
      return nullptr;
    }
    generated++;
  }
  // Resident constants, arena and scratch per device.
  uint64_t const_bytes = 0;
  for (Device* d : devs) {
    DeviceState ds;
    ds.dev = d;
    cudaSetDevice(d->ordinal);
    const_bytes = 0;
    for (size_t n : kp.constants) {
      const Instruction& ins = kp.plan.instructions[n];
      void* p = device_malloc(d, ins.literal.size());
      if (!p) {
        *error = last_error();
        return nullptr;
      }
      if (!ins.literal.empty() &&
          !check_cuda(cudaMemcpyAsync(p, ins.literal.data(), ins.literal.size(), cudaMemcpyHostToDevice, d->stream), "constant upload")) {
        *error = last_error();
        return nullptr;
      }
      ds.constants.push_back(p);
      const_bytes += ins.literal.size();
    }
    ds.arena = device_malloc(d, kp.arena_bytes);
    ds.scratch = device_malloc(d, kp.scratch_bytes);
    if (!ds.arena || !ds.scratch) {
      *error = last_error();
      return nullptr;
    }
    cudaMemsetAsync(ds.scratch, 0, std::max<uint64_t>(kp.scratch_bytes, 1), d->stream);
    if (!check_cuda(cudaStreamSynchronize(d->stream), "compile synchronize")) {
      *error = last_error();
      return nullptr;
    }
    exe->devices.push_back(std::move(ds));
  }
  exe->use_graph = env_flag("PJRTX_B200_GRAPH", true) && kp.steps.size() >= 4;
  exe->pdl = env_flag("PJRTX_B200_PDL", true);
  ExecutableStats& s = exe->stats;
  s.resident_constant_count = kp.constants.size();
  s.resident_constant_bytes = const_bytes;
  s.program_value_count = kp.program.values.size();
  s.program_node_count = kp.program.nodes.size();
  s.program_edge_count = kp.program.edges.size();
  s.program_schedule_item_count = kp.program.schedule.size();
  s.program_fusion_group_count = kp.program.fusion_groups.size();
  s.program_materialization_boundary_count = kp.program.materialization_boundaries.size();
  s.program_planned_release_count = kp.program.liveness.planned_release_count;
  s.program_planned_release_bytes = kp.program.liveness.planned_release_bytes;
  s.program_peak_live_value_count = kp.program.liveness.peak_live_value_count;
  s.program_peak_live_bytes = kp.program.liveness.peak_live_bytes;
  s.program_device_count = device_ordinals.size();
  s.kernel_step_count = kp.steps.size();
  s.generated_kernel_count = generated;
  s.arena_bytes = kp.arena_bytes;
  s.scratch_bytes = kp.scratch_bytes;
  return exe.release();
}

bool execute_executable(Executable* exe, size_t device_index, Buffer* const* args, size_t nargs,
                        std::vector<Buffer*>* outputs, std::string* error) {
  auto t0 = std::chrono::steady_clock::now();
  if (!exe) {
    *error = "null executable";
    return false;
  }
  const KernelPlan& kp = exe->kp;
  const Plan& plan = kp.plan;
  if (device_index >= exe->devices.size()) {
    *error = strfmt("device index %zu is outside the executable's %zu devices", device_index, exe->devices.size());
    return false;
  }
  if (nargs != kp.params.size()) {
    *error = strfmt("executable takes %zu arguments, got %zu", kp.params.size(), nargs);
    return false;
  }
  DeviceState& ds = exe->devices[device_index];
  Device* dev = ds.dev;
  for (size_t p = 0; p < nargs; p++) {
    const Value& v = plan.values[kp.params[p]];
    Buffer* b = args[p];
    if (!b || b->donated || !b->ptr) {
      *error = strfmt("argument %zu is null, deleted or donated", p);
      return false;
    }
    if (b->device != dev->ordinal) {
      *error = strfmt("argument %zu lives on device %d, executable runs on device %d", p, b->device, dev->ordinal);
      return false;
    }
    if (b->dtype != v.dtype || b->dims != v.dims) {
      *error = strfmt("argument %zu does not match the parameter descriptor (%s)", p, dtype_name(v.dtype));
      return false;
    }
    for (size_t q = 0; q < p; q++)
      if (args[q] == b && (kp.param_donated[p] || kp.param_donated[q])) {
        *error = strfmt("donated argument %zu is passed twice", p);
        return false;
      }
  }
  std::lock_guard<std::mutex> lock(exe->mu);
  cudaSetDevice(dev->ordinal);
  std::vector<void*> param_ptrs(nargs);
  for (size_t p = 0; p < nargs; p++) param_ptrs[p] = args[p]->ptr;

  uint64_t launches = 0;
  Pointers ptr{&kp, &ds, &param_ptrs, {}};
  std::vector<Buffer*> outs(plan.output_ids.size(), nullptr);
  auto cleanup = [&]() {
    for (Buffer* b : outs)
      if (b) buffer_free(b);
  };

  if (exe->use_graph) {
    // Small parameters are staged into fixed slots; the graph reads the slots.
    std::vector<void*> graph_ptrs = param_ptrs;
    uint64_t dynamic_inputs = 0;
    for (size_t p = 0; p < nargs; p++)
      if (kp.param_slot[p] != UINT64_MAX) {
        void* slot = (char*)ds.arena + kp.param_slot[p];
        if (args[p]->bytes &&
            !check_cuda(cudaMemcpyAsync(slot, args[p]->ptr, args[p]->bytes, cudaMemcpyDeviceToDevice, dev->stream), "stage argument")) {
          *error = last_error();
          return false;
        }
        graph_ptrs[p] = slot;
        dynamic_inputs++;
      }
    if (exe->profiling) {
      // Profiled replay: the same steps captured with an event record between them, so the step times are those of
      // graph nodes (no host launch gap) running one after the other; instantiated for this call only.
      Pointers gp{&kp, &ds, &graph_ptrs, {}};
      cudaGraph_t graph = nullptr;
      cudaGraphExec_t timed_exec = nullptr;
      if (!check_cuda(cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeThreadLocal), "begin capture")) {
        *error = last_error();
        return false;
      }
      uint64_t captured = 0;
      std::string run_error;
      // An event record between two kernels leaves no kernel-to-kernel edge to make programmatic, and the launch
      // attribute is refused there: the timed capture launches without it.
      const bool pdl = exe->pdl;
      exe->pdl = false;
      bool ok = run_steps(exe, ds, gp, &captured, &run_error, true, true);
      exe->pdl = pdl;
      cudaError_t ce = cudaStreamEndCapture(dev->stream, &graph);
      if (ok && ce == cudaSuccess && graph) ce = cudaGraphInstantiate(&timed_exec, graph, 0);
      if (graph) cudaGraphDestroy(graph);
      if (!ok || ce != cudaSuccess || !timed_exec) {
        *error = ok ? std::string("profiled graph capture failed: ") + cudaGetErrorString(ce) : run_error;
        cudaGetLastError();
        return false;
      }
      ce = cudaGraphLaunch(timed_exec, dev->stream);
      if (ce == cudaSuccess) collect_step_times(exe);
      cudaGraphExecDestroy(timed_exec);
      if (ce != cudaSuccess) {
        *error = std::string("profiled graph launch failed: ") + cudaGetErrorString(ce);
        return false;
      }
    } else {
    if (!ds.graph || ds.graph_param_ptrs != graph_ptrs) {
      if (ds.graph) {
        cudaGraphExecDestroy(ds.graph);
        ds.graph = nullptr;
      }
      Pointers gp{&kp, &ds, &graph_ptrs, {}};
      cudaGraph_t graph = nullptr;
      if (!check_cuda(cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeThreadLocal), "begin capture")) {
        *error = last_error();
        return false;
      }
      uint64_t captured = 0;
      std::string run_error;
      bool ok = run_steps(exe, ds, gp, &captured, &run_error);
      cudaError_t ce = cudaStreamEndCapture(dev->stream, &graph);
      if (!ok || ce != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        *error = ok ? std::string("graph capture failed: ") + cudaGetErrorString(ce) : run_error;
        cudaGetLastError();
        return false;
      }
      ce = cudaGraphInstantiate(&ds.graph, graph, 0);
      cudaGraphDestroy(graph);
      if (ce != cudaSuccess) {
        *error = std::string("graph instantiate failed: ") + cudaGetErrorString(ce);
        ds.graph = nullptr;
        return false;
      }
      ds.graph_param_ptrs = graph_ptrs;
      exe->stats.graph_capture_count++;
    }
    if (!check_cuda(cudaGraphLaunch(ds.graph, dev->stream), "graph launch")) {
      *error = last_error();
      return false;
    }
    }
    launches = kp.steps.size();
    exe->stats.graph_launch_count++;
    exe->stats.captured_program_execute_count++;
    exe->stats.captured_program_dynamic_input_count = dynamic_inputs;
    exe->stats.captured_program_captured_input_count = nargs - dynamic_inputs;
    ptr.param_ptrs = &param_ptrs;
  } else {
    // Direct mode: program outputs are written straight into fresh buffers.
    ptr.fresh.assign(plan.values.size(), nullptr);
    for (size_t o = 0; o < plan.output_ids.size(); o++) {
      uint32_t r = kp.root[plan.output_ids[o]];
      if (kp.storage[r].kind != Storage::kArena || ptr.fresh[r]) continue;
      const Value& rv = plan.values[r];
      Buffer* b = buffer_alloc(dev, rv.dtype, rv.dims, false);
      if (!b) {
        *error = last_error();
        cleanup();
        return false;
      }
      ptr.fresh[r] = b->ptr;
      outs[o] = b;
    }
    if (!run_steps(exe, ds, ptr, &launches, error, exe->profiling, false, /*ordered_first=*/true)) {
      cleanup();
      return false;
    }
  }

  // Wrap outputs.
  std::vector<char> param_taken(nargs, 0);
  for (size_t o = 0; o < plan.output_ids.size(); o++) {
    const Value& ov = plan.values[plan.output_ids[o]];
    uint32_t r = kp.root[ov.id];
    const Storage& st = kp.storage[r];
    if (outs[o]) {  // direct mode fresh buffer; give it the output's own dims
      outs[o]->dims = ov.dims;
      outs[o]->dtype = ov.dtype;
      continue;
    }
    if (st.kind == Storage::kParameter && kp.param_donated[st.index] && !param_taken[st.index]) {
      // Donation: the output takes over the argument's storage (src/backend/mlx_metal/api.cc:5474-5478).
      Buffer* in = args[st.index];
      Buffer* b = new Buffer();
      b->device = in->device;
      b->dtype = ov.dtype;
      b->dims = ov.dims;
      b->ptr = in->ptr;
      b->bytes = in->bytes;
      b->owns = in->owns;
      in->donated = true;
      in->ptr = nullptr;
      param_taken[st.index] = 1;
      outs[o] = b;
      exe->stats.donation_alias_output_count++;
      exe->stats.donation_alias_output_bytes += b->bytes;
      continue;
    }
    Buffer* b = buffer_alloc(dev, ov.dtype, ov.dims, false);
    if (!b) {
      *error = last_error();
      cleanup();
      return false;
    }
    const void* src = st.kind == Storage::kParameter && param_taken[st.index] ? nullptr : ptr.of(ov.id);
    if (st.kind == Storage::kParameter && param_taken[st.index]) {
      // A second output aliasing an already transferred argument: copy from the first one.
      for (size_t q = 0; q < o; q++)
        if (kp.root[plan.output_ids[q]] == r) src = outs[q]->ptr;
    }
    if (b->bytes && src &&
        !check_cuda(cudaMemcpyAsync(b->ptr, src, b->bytes, cudaMemcpyDeviceToDevice, dev->stream), "output copy")) {
      *error = last_error();
      buffer_free(b);
      cleanup();
      return false;
    }
    outs[o] = b;
  }
  *outputs = outs;

  ExecutableStats& s = exe->stats;
  s.execute_count++;
  s.last_execute_device_index = device_index;
  s.last_execute_local_hardware_id = dev->ordinal;
  s.compiled_program_execute_count++;
  s.compiled_program_output_count += outs.size();
  s.kernel_launch_total += launches;
  for (const Step& st : kp.steps)
    if (st.type == Step::kFused) s.fusion_group_execute_count++;
  uint64_t us = (uint64_t)std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
  s.execute_wall_us_total += us;
  s.execute_wall_us_peak = std::max(s.execute_wall_us_peak, us);
  if (profile_enabled())
    fprintf(stderr,
            "pjrtx_profile event=backend_execute device_index=%zu local_hardware_id=%d inputs=%zu outputs=%zu kernel_steps=%zu "
            "graph=%d host_enqueue_us=%llu\n",
            device_index, dev->ordinal, nargs, outs.size(), kp.steps.size(), exe->use_graph ? 1 : 0, (unsigned long long)us);
  return true;
}

ExecutableStats executable_stats(Executable* exe) {
  std::lock_guard<std::mutex> lock(exe->mu);
  return exe->stats;
}

std::vector<int> executable_device_ordinals(Executable* exe) { return exe->device_ordinals; }

std::string executable_describe(Executable* exe) {
  return "{\"program\":" + describe_program(exe->kp.program) + ",\"kernel_plan\":" + describe_steps(exe->kp, false) + "}";
}

void destroy_executable(Executable* exe) {
  if (!exe) return;
  for (DeviceState& ds : exe->devices) {
    cudaSetDevice(ds.dev->ordinal);
    if (ds.graph) cudaGraphExecDestroy(ds.graph);
    for (cudaEvent_t e : exe->step_events) cudaEventDestroy(e);
    exe->step_events.clear();
    for (size_t k = 0; k < ds.constants.size(); k++)
      device_free(ds.dev, ds.constants[k], exe->kp.plan.instructions[exe->kp.constants[k]].literal.size());
    device_free(ds.dev, ds.arena, exe->kp.arena_bytes);
    device_free(ds.dev, ds.scratch, exe->kp.scratch_bytes);
  }
  delete exe;
}

}  // namespace pjrtx

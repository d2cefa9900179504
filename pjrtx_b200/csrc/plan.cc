#include "plan.h"

#include <cstring>

namespace pjrtx {

static thread_local std::string g_last_error;

void set_last_error(const char* fmt, ...) {
  char buf[2048];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_last_error = buf;
}

const char* last_error() { return g_last_error.c_str(); }

std::string strfmt(const char* fmt, ...) {
  char buf[4096];
  va_list ap;
  va_start(ap, fmt);
  int n = vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (n < 0) return "";
  if ((size_t)n < sizeof buf) return std::string(buf, n);
  std::string big(n + 1, '\0');
  va_start(ap, fmt);
  vsnprintf(&big[0], big.size(), fmt, ap);
  va_end(ap);
  big.resize(n);
  return big;
}

static const char* kKindNames[] = {
#define X(n) #n,
    PJRTX_KINDS(X)
#undef X
};

const char* kind_name(Kind k) {
  int i = (int)k;
  if (i < 0 || i >= (int)Kind::kCount) return "unsupported";
  return kKindNames[i];
}

Kind kind_from_name(const std::string& name) {
  for (int i = 0; i < (int)Kind::kCount; i++)
    if (name == kKindNames[i]) return (Kind)i;
  // The reference spells these without the trailing underscore in diagnostics.
  if (name == "and") return Kind::and_;
  if (name == "or") return Kind::or_;
  if (name == "xor") return Kind::xor_;
  if (name == "not") return Kind::not_;
  if (name == "while") return Kind::while_;
  return Kind::unsupported;
}

static const std::vector<int64_t> kEmptyList;

const std::vector<int64_t>& Instruction::list(const char* name) const {
  auto it = attrs.find(name);
  return it == attrs.end() ? kEmptyList : it->second;
}

int64_t Instruction::scalar(const char* name, int64_t fallback) const {
  auto it = attrs.find(name);
  if (it == attrs.end() || it->second.empty()) return fallback;
  return it->second[0];
}

std::vector<uint32_t> Plan::parameter_ids() const {
  std::vector<uint32_t> ids;
  for (const Value& v : values)
    if (v.role == ValueRole::parameter) ids.push_back(v.id);
  return ids;
}

namespace {

bool is_unary_kind(Kind k) {
  switch (k) {
    case Kind::copy_arg0: case Kind::negate: case Kind::exp: case Kind::expm1: case Kind::tanh:
    case Kind::sqrt: case Kind::rsqrt: case Kind::abs: case Kind::cbrt: case Kind::ceil:
    case Kind::floor: case Kind::log: case Kind::log1p: case Kind::logistic: case Kind::sine:
    case Kind::cosine: case Kind::not_: case Kind::sign: case Kind::is_finite:
    case Kind::round_nearest_afz: case Kind::round_nearest_even: case Kind::popcnt:
    case Kind::count_leading_zeros: case Kind::convert: case Kind::bitcast_convert:
    case Kind::reshape: case Kind::transpose: case Kind::broadcast_in_dim: case Kind::slice:
    case Kind::top_k: case Kind::reverse: case Kind::cholesky: case Kind::fft:
    case Kind::get_tuple_element: case Kind::imag: case Kind::real: case Kind::reduce_precision:
    case Kind::all_reduce: case Kind::all_gather:
      return true;
    default:
      return false;
  }
}

bool is_binary_kind(Kind k) {
  switch (k) {
    case Kind::add: case Kind::subtract: case Kind::multiply: case Kind::divide:
    case Kind::maximum: case Kind::minimum: case Kind::power: case Kind::atan2:
    case Kind::remainder: case Kind::and_: case Kind::or_: case Kind::xor_:
    case Kind::shift_left: case Kind::shift_right_arithmetic: case Kind::shift_right_logical:
    case Kind::dot_general: case Kind::compare: case Kind::gather: case Kind::pad:
    case Kind::complex: case Kind::convolution: case Kind::triangular_solve:
      return true;
    default:
      return false;
  }
}

// Fixed operand count of a kind, or -1 when it varies
// (src/compiler/executable_plan_verify.zig:19-30).
int expected_arity(Kind k) {
  switch (k) {
    case Kind::constant: case Kind::iota: case Kind::partition_id: return 0;
    case Kind::select: case Kind::clamp: return 3;
    case Kind::dynamic_slice: case Kind::dynamic_update_slice: case Kind::concatenate:
    case Kind::custom_call: case Kind::optimization_barrier: case Kind::rng_bit_generator:
    case Kind::scatter: case Kind::sort: case Kind::tuple: case Kind::while_:
    case Kind::reduce_sum: case Kind::reduce_max: case Kind::reduce_min: case Kind::reduce_and:
    case Kind::reduce_or: case Kind::rng: case Kind::unsupported:
      return -1;
    default:
      if (is_unary_kind(k)) return 1;
      if (is_binary_kind(k)) return 2;
      return -1;
  }
}

std::string fail(long instruction, long value, const std::string& detail, const char* feature) {
  std::string s = "invalid executable plan: pass=pjrtx-plan-verify";
  if (instruction >= 0) s += strfmt(" instruction=%ld", instruction);
  if (value >= 0) s += strfmt(" value=%ld", value);
  s += " detail=\"" + detail + "\" feature=" + feature;
  return s;
}

bool elementwise_same_shape_kind(Kind k) {
  switch (k) {
    case Kind::add: case Kind::subtract: case Kind::multiply: case Kind::divide:
    case Kind::maximum: case Kind::minimum: case Kind::power: case Kind::atan2:
    case Kind::remainder: case Kind::and_: case Kind::or_: case Kind::xor_:
    case Kind::shift_left: case Kind::shift_right_arithmetic: case Kind::shift_right_logical:
    case Kind::negate: case Kind::exp: case Kind::expm1: case Kind::tanh: case Kind::sqrt:
    case Kind::rsqrt: case Kind::abs: case Kind::cbrt: case Kind::ceil: case Kind::floor:
    case Kind::log: case Kind::log1p: case Kind::logistic: case Kind::sine: case Kind::cosine:
    case Kind::not_: case Kind::sign: case Kind::round_nearest_afz:
    case Kind::round_nearest_even: case Kind::popcnt: case Kind::count_leading_zeros:
      return true;
    default:
      return false;
  }
}

}  // namespace

std::string verify_plan(const Plan& plan) {
  if (plan.num_replicas < 1 || plan.num_partitions < 1)
    return fail(-1, -1, "replica and partition counts must be positive", "topology");
  size_t slots = (size_t)plan.num_replicas * (size_t)plan.num_partitions;
  if (plan.device_assignment.size() < slots)
    return fail(-1, -1, "device assignment is shorter than replicas*partitions", "topology");
  if (plan.values.empty())
    return fail(-1, -1, "executable plan has no values", "value-graph");

  std::vector<char> defined(plan.values.size(), 0);
  size_t parameter_count = 0;
  for (size_t i = 0; i < plan.values.size(); i++) {
    const Value& v = plan.values[i];
    if (v.id != i) return fail(-1, (long)i, "value id does not match its table index", "value-graph");
    for (int64_t d : v.dims)
      if (d < 0) return fail(-1, (long)i, "value has a negative dimension", "value-storage");
    if (v.role == ValueRole::parameter) {
      defined[i] = 1;
      parameter_count++;
    }
  }
  if (plan.parameter_shardings.size() != parameter_count)
    return strfmt(
        "invalid executable plan: pass=pjrtx-plan-verify detail=\"parameter sharding count must match "
        "parameter value count: shardings=%zu parameters=%zu\" feature=sharding",
        plan.parameter_shardings.size(), parameter_count);
  if (plan.output_ids.size() != plan.output_shardings.size())
    return fail(-1, -1, "output sharding count must match output count", "sharding");

  for (size_t n = 0; n < plan.instructions.size(); n++) {
    const Instruction& ins = plan.instructions[n];
    if (ins.kind == Kind::unsupported || ins.kind == Kind::kCount)
      return fail((long)n, -1, "unsupported instruction kind entered the plan", "instruction-kind");
    int arity = expected_arity(ins.kind);
    if (arity >= 0 && (int)ins.inputs.size() != arity)
      return fail((long)n, -1,
                  strfmt("%s expects %d operands, got %zu", kind_name(ins.kind), arity, ins.inputs.size()),
                  "instruction-arity");
    for (uint32_t in : ins.inputs) {
      if (in >= plan.values.size())
        return fail((long)n, (long)in, "instruction input is outside the value table", "value-graph");
      if (!defined[in])
        return fail((long)n, (long)in, "instruction input is used before it is defined", "value-graph");
    }
    if (ins.outputs.empty())
      return fail((long)n, -1, "instruction defines no value", "value-graph");
    for (uint32_t out : ins.outputs) {
      if (out >= plan.values.size())
        return fail((long)n, (long)out, "instruction output is outside the value table", "value-graph");
      if (defined[out])
        return fail((long)n, (long)out, "value is defined more than once", "value-graph");
      ValueRole role = plan.values[out].role;
      if (role == ValueRole::parameter)
        return fail((long)n, (long)out, "instruction result has parameter role", "value-role");
      defined[out] = 1;
    }
    const Value& out0 = plan.values[ins.outputs[0]];
    if (ins.kind == Kind::constant) {
      if (ins.literal.size() != out0.bytes())
        return fail((long)n, (long)out0.id, "constant literal size does not match its descriptor", "value-storage");
    }
    if (elementwise_same_shape_kind(ins.kind)) {
      for (uint32_t in : ins.inputs) {
        const Value& v = plan.values[in];
        if (v.dims != out0.dims)
          return fail((long)n, (long)in, "elementwise operand shape differs from result shape", "value-storage");
        if (v.dtype != out0.dtype)
          return fail((long)n, (long)in, "elementwise operand type differs from result type", "value-storage");
      }
    }
    if (ins.kind == Kind::compare || ins.kind == Kind::select || ins.kind == Kind::clamp) {
      for (uint32_t in : ins.inputs) {
        const Value& v = plan.values[in];
        // select/clamp accept rank-0 predicate / bounds.
        if (v.dims != out0.dims && !v.dims.empty())
          return fail((long)n, (long)in, "operand shape differs from result shape", "value-storage");
      }
      if (ins.kind == Kind::compare && out0.dtype != kPred)
        return fail((long)n, (long)out0.id, "compare result must be a predicate", "value-storage");
    }
    if (ins.kind == Kind::reshape) {
      if (plan.values[ins.inputs[0]].count() != out0.count())
        return fail((long)n, (long)out0.id, "reshape changes the element count", "value-storage");
    }
    if (ins.kind == Kind::transpose) {
      const auto& perm = ins.list("permutation");
      const Value& src = plan.values[ins.inputs[0]];
      if (perm.size() != src.dims.size() || out0.dims.size() != src.dims.size())
        return fail((long)n, -1, "transpose permutation rank mismatch", "value-storage");
      for (size_t d = 0; d < perm.size(); d++)
        if (perm[d] < 0 || perm[d] >= (int64_t)src.dims.size() || out0.dims[d] != src.dims[perm[d]])
          return fail((long)n, -1, "transpose permutation does not produce the result shape", "value-storage");
    }
  }
  for (size_t i = 0; i < plan.values.size(); i++)
    if (!defined[i] && plan.values[i].role != ValueRole::parameter)
      return fail(-1, (long)i, "value is never defined", "value-graph");

  for (uint32_t id : plan.output_ids)
    if (id >= plan.values.size())
      return fail(-1, (long)id, "output id is outside the value table", "value-graph");
  for (uint32_t p : plan.donated_parameter_indices)
    if (p >= parameter_count) return fail(-1, -1, "donated parameter index is out of range", "donation-alias");
  for (const OutputAlias& a : plan.output_aliases) {
    if (a.output_index >= plan.output_ids.size())
      return fail(-1, -1, "output alias names an unknown output", "donation-alias");
    if (a.parameter_index >= parameter_count)
      return fail(-1, -1, "output alias names an unknown parameter", "donation-alias");
    bool donated = false;
    for (uint32_t p : plan.donated_parameter_indices) donated |= (p == a.parameter_index);
    if (!donated) return fail(-1, -1, "output alias parameter is not donated", "donation-alias");
  }
  return "";
}

std::string describe_plan(const Plan& plan) {
  auto ints = [](const std::vector<int64_t>& v) {
    std::string r = "[";
    for (size_t i = 0; i < v.size(); i++) r += strfmt(i ? ",%lld" : "%lld", (long long)v[i]);
    return r + "]";
  };
  auto ids = [](const std::vector<uint32_t>& v) {
    std::string r = "[";
    for (size_t i = 0; i < v.size(); i++) r += strfmt(i ? ",%u" : "%u", v[i]);
    return r + "]";
  };
  auto sharding = [](const Sharding& sh) {
    return strfmt("{\"kind\":%d,\"mesh\":\"%s\",\"split_dim\":%lld}", (int)sh.kind, sh.mesh_name.c_str(), (long long)sh.split_dim);
  };
  std::string s = strfmt("{\"num_replicas\":%d,\"num_partitions\":%d,\"values\":[", plan.num_replicas, plan.num_partitions);
  for (size_t i = 0; i < plan.values.size(); i++) {
    const Value& v = plan.values[i];
    s += strfmt("%s{\"role\":%d,\"dtype\":%d,\"dims\":%s}", i ? "," : "", (int)v.role, v.dtype, ints(v.dims).c_str());
  }
  s += "],\"instructions\":[";
  for (size_t i = 0; i < plan.instructions.size(); i++) {
    const Instruction& ins = plan.instructions[i];
    s += strfmt("%s{\"kind\":\"%s\",\"inputs\":%s,\"outputs\":%s,\"attrs\":{", i ? "," : "", kind_name(ins.kind),
                ids(ins.inputs).c_str(), ids(ins.outputs).c_str());
    bool first = true;
    for (const auto& kv : ins.attrs) {
      s += strfmt("%s\"%s\":%s", first ? "" : ",", kv.first.c_str(), ints(kv.second).c_str());
      first = false;
    }
    s += "}";
    if (!ins.literal.empty()) {
      static const char* hex = "0123456789abcdef";
      std::string h(ins.literal.size() * 2, '0');
      for (size_t b = 0; b < ins.literal.size(); b++) {
        h[2 * b] = hex[ins.literal[b] >> 4];
        h[2 * b + 1] = hex[ins.literal[b] & 15];
      }
      s += ",\"literal\":\"" + h + "\"";
    }
    if (!ins.custom_call_target.empty()) s += ",\"target\":\"" + ins.custom_call_target + "\"";
    s += "}";
  }
  s += "],\"outputs\":" + ids(plan.output_ids) + ",\"parameter_shardings\":[";
  for (size_t i = 0; i < plan.parameter_shardings.size(); i++) s += (i ? "," : "") + sharding(plan.parameter_shardings[i]);
  s += "],\"output_shardings\":[";
  for (size_t i = 0; i < plan.output_shardings.size(); i++) s += (i ? "," : "") + sharding(plan.output_shardings[i]);
  std::vector<int64_t> donated(plan.donated_parameter_indices.begin(), plan.donated_parameter_indices.end());
  s += "],\"donated\":" + ints(donated) + ",\"aliases\":[";
  for (size_t i = 0; i < plan.output_aliases.size(); i++)
    s += strfmt("%s[%u,%u]", i ? "," : "", plan.output_aliases[i].output_index, plan.output_aliases[i].parameter_index);
  return s + "]}";
}

namespace {
struct Fnv {
  uint64_t h = 1469598103934665603ull;
  void bytes(const void* p, size_t n) {
    const uint8_t* b = static_cast<const uint8_t*>(p);
    for (size_t i = 0; i < n; i++) {
      h ^= b[i];
      h *= 1099511628211ull;
    }
  }
  template <typename T> void pod(const T& v) { bytes(&v, sizeof(T)); }
  void str(const std::string& s) {
    pod((uint64_t)s.size());
    bytes(s.data(), s.size());
  }
  template <typename T> void list(const std::vector<T>& v) {
    pod((uint64_t)v.size());
    if (!v.empty()) bytes(v.data(), v.size() * sizeof(T));
  }
};
}  // namespace

std::string plan_fingerprint(const Plan& plan, const char* backend_name, uint64_t custom_call_registry_version,
                             const std::vector<int32_t>& target_devices) {
  Fnv f;
  f.str("pjrtx-b200-executable-cache-v2");
  f.str(backend_name ? backend_name : "");
  f.pod(custom_call_registry_version);
  // Target devices (src/runtime/executable_fingerprint.zig:38-56 hashes the resolved device ids and their local
  // hardware ids even when the plan carries no assignment): the same plan compiled for another GPU is another entry.
  f.list(target_devices);
  f.pod(plan.num_replicas);
  f.pod(plan.num_partitions);
  f.pod(plan.use_shardy);
  f.list(plan.device_assignment);
  auto shardings = [&](const std::vector<Sharding>& v) {
    f.pod((uint64_t)v.size());
    for (const Sharding& s : v) {
      f.pod((int)s.kind);
      f.str(s.mesh_name);
      f.list(s.device_assignment);
      f.pod(s.split_dim);
    }
  };
  shardings(plan.parameter_shardings);
  shardings(plan.output_shardings);
  f.list(plan.output_ids);
  f.list(plan.donated_parameter_indices);
  f.pod((uint64_t)plan.output_aliases.size());
  for (const OutputAlias& a : plan.output_aliases) {
    f.pod(a.output_index);
    f.pod(a.parameter_index);
    f.pod(a.kind);
  }
  f.pod((uint64_t)plan.values.size());
  for (const Value& v : plan.values) {
    f.pod((int)v.role);
    f.pod(v.dtype);
    f.list(v.dims);
  }
  f.pod((uint64_t)plan.instructions.size());
  for (const Instruction& ins : plan.instructions) {
    f.pod((int)ins.kind);
    f.list(ins.inputs);
    f.list(ins.outputs);
    f.pod((uint64_t)ins.attrs.size());
    for (const auto& kv : ins.attrs) {
      f.str(kv.first);
      f.list(kv.second);
    }
    f.list(ins.literal);
    f.str(ins.custom_call_target);
  }
  return strfmt("pjrtx-%016llx", (unsigned long long)f.h);
}

}  // namespace pjrtx

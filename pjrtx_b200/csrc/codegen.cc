#include "codegen.h"
#include "program.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <functional>
#include <map>

namespace pjrtx {

namespace {

const char* kPreamble = R"CUDA(
#include <cuda_fp16.h>
#include <cuda_bf16.h>
typedef unsigned char u8_t;
typedef signed char s8_t;
typedef unsigned short u16_t;
typedef short s16_t;
typedef unsigned int u32_t;
typedef int s32_t;
typedef unsigned long long u64_t;
typedef long long s64_t;

__device__ __forceinline__ float rnd_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float rnd_f16(float x) { return __half2float(__float2half_rn(x)); }
__device__ __forceinline__ float lit_f(unsigned bits) { return __uint_as_float(bits); }

// 128-bit (or narrower) read-only vector load of V consecutive elements.
template <typename T, int V>
__device__ __forceinline__ void ldvec(T* dst, const T* __restrict__ src) {
  constexpr int B = sizeof(T) * V;
  if constexpr (B == 16) { *reinterpret_cast<uint4*>(dst) = __ldg(reinterpret_cast<const uint4*>(src)); }
  else if constexpr (B == 8) { *reinterpret_cast<uint2*>(dst) = __ldg(reinterpret_cast<const uint2*>(src)); }
  else if constexpr (B == 4) { *reinterpret_cast<unsigned*>(dst) = __ldg(reinterpret_cast<const unsigned*>(src)); }
  else if constexpr (B == 2) { *reinterpret_cast<unsigned short*>(dst) = __ldg(reinterpret_cast<const unsigned short*>(src)); }
  else if constexpr (B == 32) {
    reinterpret_cast<uint4*>(dst)[0] = __ldg(reinterpret_cast<const uint4*>(src));
    reinterpret_cast<uint4*>(dst)[1] = __ldg(reinterpret_cast<const uint4*>(src) + 1);
  } else {
#pragma unroll
    for (int k = 0; k < V; k++) dst[k] = src[k];
  }
}
template <typename T, int V>
__device__ __forceinline__ void stvec(T* __restrict__ dst, const T* src) {
  constexpr int B = sizeof(T) * V;
  if constexpr (B == 16) { *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src); }
  else if constexpr (B == 8) { *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(src); }
  else if constexpr (B == 4) { *reinterpret_cast<unsigned*>(dst) = *reinterpret_cast<const unsigned*>(src); }
  else if constexpr (B == 2) { *reinterpret_cast<unsigned short*>(dst) = *reinterpret_cast<const unsigned short*>(src); }
  else if constexpr (B == 32) {
    reinterpret_cast<uint4*>(dst)[0] = reinterpret_cast<const uint4*>(src)[0];
    reinterpret_cast<uint4*>(dst)[1] = reinterpret_cast<const uint4*>(src)[1];
  } else {
#pragma unroll
    for (int k = 0; k < V; k++) dst[k] = src[k];
  }
}

template <typename T>
__device__ __forceinline__ T shfl_x(T v, int o) {
  constexpr int W = (sizeof(T) + 3) / 4;
  unsigned w[W];
  memcpy(w, &v, sizeof(T));
#pragma unroll
  for (int k = 0; k < W; k++) w[k] = __shfl_xor_sync(0xffffffffu, w[k], o);
  memcpy(&v, w, sizeof(T));
  return v;
}

// Butterfly inside each warp, then a fixed-order fold of the per-warp partials
// by every thread: the result is identical in all threads and from run to run.
template <typename T, typename F>
__device__ __forceinline__ T block_reduce(T v, F f, void* smem_raw) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = f(v, shfl_x(v, o));
  const int nw = (blockDim.x + 31) >> 5;
  if (nw == 1) return v;
  T* smem = reinterpret_cast<T*>(smem_raw);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
  __syncthreads();
  T t = smem[0];
  for (int k = 1; k < nw; k++) t = f(t, smem[k]);
  return t;
}

template <typename V, typename I> struct ArgPair { V v; I i; };
// a is kept when it is "better": NaN counts as the maximum, ties keep the smaller index.
template <typename V, typename I>
__device__ __forceinline__ ArgPair<V, I> arg_better(ArgPair<V, I> a, ArgPair<V, I> b) {
  const bool an = a.v != a.v, bn = b.v != b.v;
  const bool keep_a = (an && !bn) || (!bn && a.v > b.v) || ((a.v == b.v || (an && bn)) && a.i < b.i);
  return keep_a ? a : b;
}
__device__ __forceinline__ float xla_max(float a, float b) { return (a >= b || a != a) ? a : b; }
__device__ __forceinline__ float xla_min(float a, float b) { return (a <= b || a != a) ? a : b; }
template <typename T> __device__ __forceinline__ T int_max(T a, T b) { return a > b ? a : b; }
template <typename T> __device__ __forceinline__ T int_min(T a, T b) { return a < b ? a : b; }
template <typename T> __device__ __forceinline__ T int_div(T a, T b) {
  if (b == 0) return (T)-1;
  if (T(-1) < T(0) && b == (T)-1) return (T)(0 - a);
  return a / b;
}
template <typename T> __device__ __forceinline__ T int_rem(T a, T b) {
  if (b == 0) return a;
  if (T(-1) < T(0) && b == (T)-1) return 0;
  return a % b;
}
template <typename T> __device__ __forceinline__ T int_pow(T a, T b) {
  if (T(-1) < T(0) && b < 0) return a == 1 ? 1 : (a == (T)-1 ? ((b & 1) ? (T)-1 : 1) : 0);
  T r = 1;
  while (b) { if (b & 1) r *= a; a *= a; b >>= 1; }
  return r;
}
template <typename T> __device__ __forceinline__ T f2i(float x) {
  if (x != x) return 0;
  constexpr bool is_signed = T(-1) < T(0);
  constexpr int bits = sizeof(T) * 8;
  const float hi = is_signed ? ldexpf(1.0f, bits - 1) : ldexpf(1.0f, bits);
  const float lo = is_signed ? -ldexpf(1.0f, bits - 1) : 0.0f;
  if (x >= hi) return is_signed ? (T)((~(unsigned long long)0) >> (65 - bits)) : (T)~(T)0;
  if (x <= lo) return is_signed ? (T)((unsigned long long)1 << (bits - 1)) : (T)0;
  return (T)x;
}
__device__ __forceinline__ float f_sign(float x) { return x != x ? x : (x > 0.f ? 1.f : (x < 0.f ? -1.f : x)); }
__device__ __forceinline__ float f_logistic(float x) { return 1.0f / (1.0f + expf(-x)); }
// For results stored in a 16-bit type: the approximate exponential and division are off by about 2^-21, the rounding
// to f16 / bf16 that follows by 2^-12 / 2^-9.
__device__ __forceinline__ float f_logistic16(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
__device__ __forceinline__ float f_rsqrt(float x) { return 1.0f / sqrtf(x); }
)CUDA";

const char* ctype(int dt) {
  switch (dt) {
    case kU8: return "u8_t";
    case kPred: return "u8_t";
    case kS8: return "s8_t";
    case kU16: return "u16_t";
    case kS16: return "s16_t";
    case kU32: return "u32_t";
    case kS32: return "s32_t";
    case kU64: return "u64_t";
    case kS64: return "s64_t";
    case kF32: return "float";
    case kF16: return "__half";
    case kBF16: return "__nv_bfloat16";
    default: return nullptr;
  }
}

// Type a value is held in while computing.
const char* comp_type(int dt) {
  if (dtype_is_float(dt)) return "float";
  if (dt == kPred) return "bool";
  return ctype(dt);
}

std::string load_conv(int dt, const std::string& raw) {
  if (dt == kF16) return "__half2float(" + raw + ")";
  if (dt == kBF16) return "__bfloat162float(" + raw + ")";
  if (dt == kPred) return "(" + raw + " != 0)";
  return raw;
}

std::string store_conv(int dt, const std::string& v) {
  if (dt == kF16) return "__float2half_rn(" + v + ")";
  if (dt == kBF16) return "__float2bfloat16_rn(" + v + ")";
  if (dt == kPred) return "(u8_t)(" + v + " ? 1 : 0)";
  return v;
}

std::string round_to(int dt, const std::string& v) {
  if (dt == kBF16) return "rnd_bf16(" + v + ")";
  if (dt == kF16) return "rnd_f16(" + v + ")";
  return v;
}

float half_bits_to_float(uint16_t h) {
  uint32_t sign = (h >> 15) & 1, exp = (h >> 10) & 0x1f, man = h & 0x3ff;
  float v;
  if (exp == 0) v = std::ldexp((float)man, -24);
  else if (exp == 31) v = man ? NAN : INFINITY;
  else v = std::ldexp((float)(man | 0x400), (int)exp - 25);
  return sign ? -v : v;
}

enum class IdxClass { LIN, ROW, COL, GEN };
struct Idx {
  std::string var;
  IdxClass cls;
};

struct Fail {
  std::string why;
};

struct Scope {
  std::map<std::pair<uint32_t, std::string>, std::string> memo;  // (value, index var) -> variable
  std::map<std::string, std::string> index_memo;                 // expression -> variable
  std::string code;
  int indent = 2;
};

struct VecAccess {
  uint32_t value;
  IdxClass cls;  // LIN or COL
  std::string array;
};

class Gen {
 public:
  Gen(const Plan& plan, const std::vector<size_t>& nodes, const std::vector<uint32_t>& outputs,
      const std::vector<size_t>& scatters, int sm_count)
      : plan_(plan), nodes_(nodes), outputs_(outputs), scatters_(scatters), sm_count_(sm_count > 0 ? sm_count : 148) {
    for (size_t n : nodes)
      for (uint32_t o : plan.instructions[n].outputs) producer_[o] = n;
    for (size_t i = 0; i < plan.instructions.size(); i++)
      if (plan.instructions[i].kind == Kind::constant) constant_of_[plan.instructions[i].outputs[0]] = i;
  }

  FusedKernel run(bool allow_serial_reduce) {
    allow_serial_ = allow_serial_reduce;
    analyze();
    FusedKernel k;
    k.row = row_;
    k.rows = R_;
    k.cols = C_;
    k.n = N_;
    k.vec = vec_;
    std::string body = row_ ? emit_row_kernel(&k) : emit_map_kernel(&k);
    // Signature is known only after the body has discovered its inputs.
    std::string sig;
    for (size_t s = 0; s < inputs_.size(); s++)
      sig += strfmt("%sconst %s* __restrict__ in%zu", s ? ", " : "", ctype(plan_.values[inputs_[s]].dtype), s);
    for (size_t s = 0; s < outputs_.size(); s++)
      sig += strfmt("%s%s* __restrict__ out%zu", (s || !inputs_.empty()) ? ", " : "",
                    ctype(plan_.values[outputs_[s]].dtype), s);
    for (size_t q = 0; q < scatters_.size(); q++) {
      const uint32_t dst = plan_.instructions[scatters_[q]].outputs[0];
      sig += strfmt("%s%s* __restrict__ dst%zu", (q || !outputs_.empty() || !inputs_.empty()) ? ", " : "",
                    ctype(plan_.values[dst].dtype), q);
      k.scatter_dst.push_back(dst);
    }
    k.name = "pjrtx_fused";
    k.source = std::string(kPreamble) + strfmt("typedef %s idx_t;\n", wide_index_ ? "long long" : "int") +
               strfmt("extern \"C\" __global__ void __launch_bounds__(%d) pjrtx_fused(%s) {\n", k.block,
                      sig.c_str()) +
               // Programmatic dependent launch: let the next kernel of the stream start its prologue now, and wait
               // for the previous one before the first global access.
               "  asm volatile(\"griddepcontrol.launch_dependents;\" ::: \"memory\");\n"
               "  asm volatile(\"griddepcontrol.wait;\" ::: \"memory\");\n" +
               body + "}\n";
    k.inputs = inputs_;
    k.outputs = outputs_;
    return k;
  }

 private:
  const Plan& plan_;
  std::vector<size_t> nodes_;
  std::vector<uint32_t> outputs_;
  std::vector<size_t> scatters_;  // in-place dynamic_update_slice instructions performed as offset stores
  int sm_count_;
  std::map<uint32_t, size_t> producer_;     // value -> in-group instruction
  std::map<uint32_t, size_t> constant_of_;  // value -> constant instruction
  std::vector<uint32_t> inputs_;
  std::map<uint32_t, int> input_slot_;
  bool row_ = false, allow_serial_ = false, wide_index_ = false;
  int64_t R_ = 1, C_ = 1, N_ = 0;
  int vec_ = 1;
  int tmp_ = 0;
  std::map<uint32_t, int> depth_;
  std::map<uint32_t, std::string> reduce_var_;  // reduce result value -> row-scope variable
  std::vector<Scope*> scopes_;
  std::vector<VecAccess> vec_loads_;  // of the loop body being emitted
  bool in_vec_loop_ = false;

  [[noreturn]] void fail(const std::string& why) { throw Fail{why}; }
  const Value& val(uint32_t id) const { return plan_.values[id]; }
  bool in_group(uint32_t v) const { return producer_.count(v) != 0; }
  const Instruction& prod(uint32_t v) const { return plan_.instructions[producer_.at(v)]; }
  static bool is_reduce(Kind k) {
    return k == Kind::reduce_sum || k == Kind::reduce_max || k == Kind::reduce_min || k == Kind::reduce_and ||
           k == Kind::reduce_or;
  }

  Scope& scope() { return *scopes_.back(); }
  void line(const std::string& s) { scope().code += std::string(scope().indent, ' ') + s + "\n"; }
  std::string tmp(const char* p) { return strfmt("%s%d", p, tmp_++); }

  // ---- analysis ---------------------------------------------------------
  int depth_of(uint32_t v) {
    auto it = depth_.find(v);
    if (it != depth_.end()) return it->second;
    int d = 0;
    if (in_group(v)) {
      const Instruction& ins = prod(v);
      size_t operands = is_reduce(ins.kind) ? (ins.outputs.size() == 2 ? 2 : 1) : ins.inputs.size();
      for (size_t k = 0; k < operands && k < ins.inputs.size(); k++) d = std::max(d, depth_of(ins.inputs[k]));
      if (is_reduce(ins.kind)) d += 1;
    }
    depth_[v] = d;
    return d;
  }

  static bool suffix_reduce(const std::vector<int64_t>& dims, std::vector<int64_t> rd, int64_t* rows, int64_t* cols) {
    // True when the reduced axes are the trailing ones once size-1 axes are ignored.
    std::sort(rd.begin(), rd.end());
    std::vector<char> red(dims.size(), 0);
    for (int64_t d : rd) {
      if (d < 0 || d >= (int64_t)dims.size()) return false;
      red[d] = 1;
    }
    int64_t r = 1, c = 1;
    bool seen_reduced = false;
    for (size_t d = 0; d < dims.size(); d++) {
      if (dims[d] == 1) continue;
      if (red[d]) {
        seen_reduced = true;
        c *= dims[d];
      } else {
        if (seen_reduced) return false;
        r *= dims[d];
      }
    }
    *rows = r;
    *cols = c;
    return true;
  }

  void analyze() {
    int64_t max_count = 1;
    bool any_reduce = false, all_suffix = true;
    int64_t R = -1, C = -1;
    for (size_t n : nodes_) {
      const Instruction& ins = plan_.instructions[n];
      for (uint32_t v : ins.inputs) max_count = std::max<int64_t>(max_count, val(v).count());
      for (uint32_t v : ins.outputs) max_count = std::max<int64_t>(max_count, val(v).count());
      if (!is_reduce(ins.kind)) continue;
      any_reduce = true;
      int64_t r, c;
      if (!suffix_reduce(val(ins.inputs[0]).dims, ins.list("reduce_dimensions"), &r, &c) || c <= 1) {
        all_suffix = false;
        continue;
      }
      if (R < 0) {
        R = r;
        C = c;
      } else if (R != r || C != c) {
        all_suffix = false;
      }
    }
    wide_index_ = max_count >= (int64_t)1 << 30;
    if (any_reduce && all_suffix) {
      row_ = true;
      R_ = R;
      C_ = C;
      N_ = R * C;
    } else if (any_reduce) {
      if (!allow_serial_) fail("reduction is not a uniform suffix-axis reduction");
      row_ = false;
    }
    if (outputs_.empty() && scatters_.empty()) fail("group has no stored value");
    if (row_ && !scatters_.empty()) fail("slice update inside a row kernel");
    std::vector<int64_t> counts;  // element counts of everything a map kernel stores (one loop per distinct count)
    for (uint32_t o : outputs_) {
      if (!in_group(o)) fail("stored value is not produced in the group");
      if (!ctype(val(o).dtype)) fail("unsupported element type");
      int64_t n = val(o).count();
      if (row_) {
        if (n != N_ && n != R_) fail("stored value does not span the row space");
      } else {
        N_ = std::max(N_, n);
        counts.push_back(n);
      }
      depth_of(o);
    }
    for (size_t n : scatters_) {
      const Instruction& ins = plan_.instructions[n];
      if (ins.kind != Kind::dynamic_update_slice || ins.inputs.size() != 2 + val(ins.inputs[0]).dims.size())
        fail("malformed slice update");
      const Value& update = val(ins.inputs[1]);
      if (!ctype(update.dtype) || update.dims.size() != val(ins.inputs[0]).dims.size()) fail("unsupported slice update");
      N_ = std::max(N_, update.count());
      counts.push_back(update.count());
      depth_of(ins.inputs[1]);
    }
    if (N_ == 0) fail("empty iteration space");
    // Vector width: 16 bytes of the widest element that is read or written
    // contiguously, shrunk until it divides the contiguous extent.
    size_t widest = 1;
    for (uint32_t o : outputs_) widest = std::max(widest, dtype_size(val(o).dtype));
    for (size_t n : nodes_)
      for (uint32_t v : plan_.instructions[n].inputs)
        if (!in_group(v) && val(v).count() > 1) widest = std::max(widest, dtype_size(val(v).dtype));
    for (size_t n : scatters_) widest = std::max(widest, dtype_size(val(plan_.instructions[n].inputs[1]).dtype));
    vec_ = (int)(16 / widest);
    if (row_) counts = {C_};
    for (int64_t extent : counts)
      while (vec_ > 1 && extent % vec_ != 0) vec_ /= 2;
  }

  // ---- index helpers ----------------------------------------------------
  std::string index_var(const std::string& expr) {
    auto it = scope().index_memo.find(expr);
    if (it != scope().index_memo.end()) return it->second;
    // Look through enclosing scopes so loop-invariant indices are reused.
    for (size_t s = scopes_.size(); s-- > 0;) {
      auto f = scopes_[s]->index_memo.find(expr);
      if (f != scopes_[s]->index_memo.end()) return f->second;
    }
    std::string v = tmp("j");
    line("const idx_t " + v + " = " + expr + ";");
    scope().index_memo[expr] = v;
    return v;
  }

  std::vector<std::string> coords(const std::string& lin, const std::vector<int64_t>& dims) {
    std::vector<std::string> out(dims.size());
    int64_t stride = 1;
    std::vector<int64_t> strides(dims.size());
    for (size_t d = dims.size(); d-- > 0;) {
      strides[d] = stride;
      stride *= dims[d];
    }
    bool first_nontrivial = true;
    for (size_t d = 0; d < dims.size(); d++) {
      if (dims[d] == 1) {
        out[d] = "0";
        continue;
      }
      std::string e = lin;
      if (strides[d] != 1) e = "(" + e + " / " + std::to_string(strides[d]) + ")";
      if (!first_nontrivial) e = "(" + e + " % " + std::to_string(dims[d]) + ")";
      first_nontrivial = false;
      out[d] = index_var(e);
    }
    return out;
  }

  static std::vector<int64_t> strides_of(const std::vector<int64_t>& dims) {
    std::vector<int64_t> s(dims.size());
    int64_t st = 1;
    for (size_t d = dims.size(); d-- > 0;) {
      s[d] = st;
      st *= dims[d];
    }
    return s;
  }

  std::string linearize(const std::vector<std::string>& c, const std::vector<int64_t>& dims) {
    std::vector<int64_t> st = strides_of(dims);
    std::string e;
    for (size_t d = 0; d < dims.size(); d++) {
      if (dims[d] == 1 || c[d] == "0") continue;
      std::string t = st[d] == 1 ? c[d] : "(idx_t)" + c[d] + " * " + std::to_string(st[d]);
      e += e.empty() ? t : " + " + t;
    }
    return e.empty() ? "0" : e;
  }

  Idx scalar_index() { return Idx{"0", IdxClass::GEN}; }

  // Index of the broadcast operand for an output index (broadcast_in_dim).
  Idx broadcast_index(const Idx& out_idx, const std::vector<int64_t>& od, const std::vector<int64_t>& odims,
                      const std::vector<int64_t>& bd) {
    int64_t ocount = element_count(od);
    if (ocount == 1) return (row_ && R_ == 1) ? Idx{"r", IdxClass::ROW} : scalar_index();  // one row: the scalar is the row's value
    // Significant operand axes (size > 1) and the output axes they map to.
    std::vector<size_t> sig;
    for (size_t k = 0; k < od.size(); k++)
      if (od[k] != 1) sig.push_back(k);
    for (size_t k : sig)
      if (bd[k] < 0 || bd[k] >= (int64_t)odims.size() || odims[bd[k]] != od[k]) fail("malformed broadcast_in_dim");
    // Non-trivial output axes.
    std::vector<size_t> nt;
    for (size_t d = 0; d < odims.size(); d++)
      if (odims[d] != 1) nt.push_back(d);
    auto maps_run = [&](size_t start) {  // operand axes == nt[start .. start+sig.size())
      if (start + sig.size() > nt.size()) return false;
      for (size_t k = 0; k < sig.size(); k++)
        if ((size_t)bd[sig[k]] != nt[start + k]) return false;
      return true;
    };
    if (out_idx.cls == IdxClass::LIN) {
      if (sig.size() == nt.size() && maps_run(0)) return out_idx;  // pure reshape-like broadcast
      if (row_) {
        if (ocount == R_ && maps_run(0)) return Idx{"r", IdxClass::ROW};
        if (ocount == C_ && maps_run(nt.size() - sig.size())) return Idx{"c", IdxClass::COL};
      } else if (maps_run(nt.size() - sig.size())) {
        // Trailing-axes broadcast in a map kernel: period = operand count.
        return Idx{index_var("(" + out_idx.var + " % " + std::to_string(ocount) + ")"), IdxClass::GEN};
      }
    }
    if (out_idx.cls == IdxClass::ROW) {
      // The output ranges over the rows; an operand that covers the same axes keeps the class.
      if (sig.size() == nt.size() && maps_run(0)) return out_idx;
    }
    std::vector<std::string> oc = coords(out_idx.var, odims);
    std::vector<std::string> sc(od.size(), "0");
    for (size_t k : sig) sc[k] = oc[bd[k]];
    return Idx{index_var(linearize(sc, od)), IdxClass::GEN};
  }

  // ---- value emission ---------------------------------------------------
  std::string literal(int dt, const uint8_t* p) {
    switch (dt) {
      case kF32: { uint32_t b; memcpy(&b, p, 4); return strfmt("lit_f(0x%08xu)", b); }
      case kBF16: { uint16_t h; memcpy(&h, p, 2); return strfmt("lit_f(0x%08xu)", (uint32_t)h << 16); }
      case kF16: {
        uint16_t h; memcpy(&h, p, 2);
        float f = half_bits_to_float(h);
        uint32_t b; memcpy(&b, &f, 4);
        return strfmt("lit_f(0x%08xu)", b);
      }
      case kPred: return *p ? "true" : "false";
      case kU8: return strfmt("(u8_t)%u", (unsigned)*p);
      case kS8: return strfmt("(s8_t)%d", (int)*(const int8_t*)p);
      case kU16: { uint16_t v; memcpy(&v, p, 2); return strfmt("(u16_t)%u", (unsigned)v); }
      case kS16: { int16_t v; memcpy(&v, p, 2); return strfmt("(s16_t)%d", (int)v); }
      case kU32: { uint32_t v; memcpy(&v, p, 4); return strfmt("%uu", v); }
      case kS32: { int32_t v; memcpy(&v, p, 4); return v == INT32_MIN ? "(-2147483647 - 1)" : strfmt("%d", v); }
      case kU64: { uint64_t v; memcpy(&v, p, 8); return strfmt("%lluull", (unsigned long long)v); }
      case kS64: {
        int64_t v; memcpy(&v, p, 8);
        return v == INT64_MIN ? "(-9223372036854775807ll - 1)" : strfmt("%lldll", (long long)v);
      }
      default: fail("unsupported literal type");
    }
  }

  int slot_of(uint32_t v) {
    auto it = input_slot_.find(v);
    if (it != input_slot_.end()) return it->second;
    if (!ctype(val(v).dtype)) fail("unsupported element type");
    int s = (int)inputs_.size();
    inputs_.push_back(v);
    input_slot_[v] = s;
    return s;
  }

  std::string load_external(uint32_t v, const Idx& idx) {
    const Value& value = val(v);
    auto c = constant_of_.find(v);
    if (c != constant_of_.end() && value.count() == 1)
      return literal(value.dtype, plan_.instructions[c->second].literal.data());
    int s = slot_of(v);
    if (value.count() == 1) return load_conv(value.dtype, strfmt("__ldg(in%d)", s));
    bool contiguous = (idx.cls == IdxClass::LIN && value.count() == N_) ||
                      (idx.cls == IdxClass::COL && row_ && value.count() == C_);
    if (in_vec_loop_ && vec_ > 1 && contiguous) {
      for (const VecAccess& a : vec_loads_)
        if (a.value == v && a.cls == idx.cls) return load_conv(value.dtype, a.array + "[v]");
      VecAccess a{v, idx.cls, strfmt("L%d%s", s, idx.cls == IdxClass::LIN ? "i" : "c")};
      vec_loads_.push_back(a);
      return load_conv(value.dtype, a.array + "[v]");
    }
    return load_conv(value.dtype, strfmt("__ldg(in%d + %s)", s, idx.var.c_str()));
  }

  std::string define(uint32_t v, const Idx& idx, const std::string& expr) {
    std::string name = tmp("t");
    line(std::string("const ") + comp_type(val(v).dtype) + " " + name + " = " + expr + ";");
    scope().memo[{v, idx.var}] = name;
    return name;
  }

  std::string emit(uint32_t v, const Idx& idx) {
    for (size_t s = scopes_.size(); s-- > 0;) {
      auto it = scopes_[s]->memo.find({v, idx.var});
      if (it != scopes_[s]->memo.end()) return it->second;
    }
    if (!in_group(v)) return define(v, idx, load_external(v, idx));
    const Instruction& ins = prod(v);
    const Value& out = val(v);
    const int dt = out.dtype;
    if (!ctype(dt)) fail("unsupported element type");
    auto in = [&](size_t k) { return ins.inputs[k]; };
    auto same = [&](size_t k) {  // operand evaluated at the same index (rank-0 operands broadcast)
      if (val(in(k)).count() == 1 && out.count() != 1) return emit(in(k), scalar_index());
      return emit(in(k), idx);
    };
    auto fbin = [&](const char* op) { return define(v, idx, round_to(dt, "(" + same(0) + " " + op + " " + same(1) + ")")); };
    auto ffun = [&](const char* fn) { return define(v, idx, round_to(dt, std::string(fn) + "(" + same(0) + ")")); };
    const bool isf = dtype_is_float(dt);
    const int in_dt = ins.inputs.empty() ? dt : val(in(0)).dtype;
    switch (ins.kind) {
      case Kind::copy_arg0: case Kind::optimization_barrier:
        return same(0);
      case Kind::add:
        if (dt == kPred) return define(v, idx, "(" + same(0) + " || " + same(1) + ")");
        return fbin("+");
      case Kind::subtract: return fbin("-");
      case Kind::multiply:
        if (dt == kPred) return define(v, idx, "(" + same(0) + " && " + same(1) + ")");
        return fbin("*");
      case Kind::divide:
        if (isf) return fbin("/");
        return define(v, idx, strfmt("int_div<%s>(%s, %s)", ctype(dt), same(0).c_str(), same(1).c_str()));
      case Kind::remainder:
        if (isf) return define(v, idx, round_to(dt, "fmodf(" + same(0) + ", " + same(1) + ")"));
        return define(v, idx, strfmt("int_rem<%s>(%s, %s)", ctype(dt), same(0).c_str(), same(1).c_str()));
      case Kind::power:
        if (isf) return define(v, idx, round_to(dt, "powf(" + same(0) + ", " + same(1) + ")"));
        return define(v, idx, strfmt("int_pow<%s>(%s, %s)", ctype(dt), same(0).c_str(), same(1).c_str()));
      case Kind::atan2: return define(v, idx, round_to(dt, "atan2f(" + same(0) + ", " + same(1) + ")"));
      case Kind::maximum:
        if (isf) return define(v, idx, "xla_max(" + same(0) + ", " + same(1) + ")");
        if (dt == kPred) return define(v, idx, "(" + same(0) + " || " + same(1) + ")");
        return define(v, idx, strfmt("int_max<%s>(%s, %s)", ctype(dt), same(0).c_str(), same(1).c_str()));
      case Kind::minimum:
        if (isf) return define(v, idx, "xla_min(" + same(0) + ", " + same(1) + ")");
        if (dt == kPred) return define(v, idx, "(" + same(0) + " && " + same(1) + ")");
        return define(v, idx, strfmt("int_min<%s>(%s, %s)", ctype(dt), same(0).c_str(), same(1).c_str()));
      case Kind::and_:
        return define(v, idx, dt == kPred ? "(" + same(0) + " && " + same(1) + ")"
                                          : strfmt("(%s)(%s & %s)", ctype(dt), same(0).c_str(), same(1).c_str()));
      case Kind::or_:
        return define(v, idx, dt == kPred ? "(" + same(0) + " || " + same(1) + ")"
                                          : strfmt("(%s)(%s | %s)", ctype(dt), same(0).c_str(), same(1).c_str()));
      case Kind::xor_:
        return define(v, idx, dt == kPred ? "(" + same(0) + " != " + same(1) + ")"
                                          : strfmt("(%s)(%s ^ %s)", ctype(dt), same(0).c_str(), same(1).c_str()));
      case Kind::not_:
        return define(v, idx, dt == kPred ? "(!" + same(0) + ")" : strfmt("(%s)(~%s)", ctype(dt), same(0).c_str()));
      case Kind::shift_left: case Kind::shift_right_logical: case Kind::shift_right_arithmetic: {
        if (!dtype_is_int(dt)) fail("shift of a non-integer type");
        int bits = (int)dtype_size(dt) * 8;
        std::string a = same(0), b = same(1);
        std::string big = strfmt("((u64_t)%s >= %du)", b.c_str(), bits);
        if (ins.kind == Kind::shift_left)
          return define(v, idx, strfmt("%s ? (%s)0 : (%s)(%s << %s)", big.c_str(), ctype(dt), ctype(dt), a.c_str(), b.c_str()));
        if (ins.kind == Kind::shift_right_logical) {
          const char* ut = bits == 8 ? "u8_t" : bits == 16 ? "u16_t" : bits == 32 ? "u32_t" : "u64_t";
          return define(v, idx, strfmt("%s ? (%s)0 : (%s)((%s)%s >> %s)", big.c_str(), ctype(dt), ctype(dt), ut, a.c_str(), b.c_str()));
        }
        const char* st = bits == 8 ? "s8_t" : bits == 16 ? "s16_t" : bits == 32 ? "s32_t" : "s64_t";
        return define(v, idx, strfmt("(%s)(%s ? ((%s)%s < 0 ? (%s)-1 : (%s)0) : ((%s)%s >> %s))", ctype(dt), big.c_str(), st,
                                     a.c_str(), st, st, st, a.c_str(), b.c_str()));
      }
      case Kind::negate:
        if (isf) return define(v, idx, "(-" + same(0) + ")");
        return define(v, idx, strfmt("(%s)(0 - %s)", ctype(dt), same(0).c_str()));
      case Kind::abs:
        if (isf) return define(v, idx, "fabsf(" + same(0) + ")");
        if (dtype_is_unsigned_int(dt)) return same(0);
        return define(v, idx, strfmt("(%s)(%s < 0 ? 0 - %s : %s)", ctype(dt), same(0).c_str(), same(0).c_str(), same(0).c_str()));
      case Kind::exp: return ffun("expf");
      case Kind::expm1: return ffun("expm1f");
      case Kind::tanh: return ffun("tanhf");
      case Kind::sqrt: return ffun("sqrtf");
      case Kind::rsqrt: return ffun("f_rsqrt");
      case Kind::cbrt: return ffun("cbrtf");
      case Kind::ceil: return ffun("ceilf");
      case Kind::floor: return ffun("floorf");
      case Kind::log: return ffun("logf");
      case Kind::log1p: return ffun("log1pf");
      case Kind::logistic: return ffun(dt == kF16 || dt == kBF16 ? "f_logistic16" : "f_logistic");
      case Kind::sine: return ffun("sinf");
      case Kind::cosine: return ffun("cosf");
      case Kind::round_nearest_afz: return ffun("roundf");
      case Kind::round_nearest_even: return ffun("rintf");
      case Kind::sign:
        if (isf) return define(v, idx, "f_sign(" + same(0) + ")");
        if (dtype_is_unsigned_int(dt)) return define(v, idx, strfmt("(%s)(%s != 0)", ctype(dt), same(0).c_str()));
        return define(v, idx, strfmt("(%s)((%s > 0) - (%s < 0))", ctype(dt), same(0).c_str(), same(0).c_str()));
      case Kind::is_finite: return define(v, idx, "isfinite(" + same(0) + ")");
      case Kind::popcnt:
        return define(v, idx, dtype_size(dt) == 8 ? strfmt("(%s)__popcll((u64_t)%s)", ctype(dt), same(0).c_str())
                                                  : strfmt("(%s)__popc((u32_t)(%s)%s)", ctype(dt),
                                                           dtype_size(dt) == 1 ? "u8_t" : dtype_size(dt) == 2 ? "u16_t" : "u32_t",
                                                           same(0).c_str()));
      case Kind::count_leading_zeros: {
        int bits = (int)dtype_size(dt) * 8;
        if (bits == 64) return define(v, idx, strfmt("(%s)__clzll((s64_t)%s)", ctype(dt), same(0).c_str()));
        const char* ut = bits == 8 ? "u8_t" : bits == 16 ? "u16_t" : "u32_t";
        return define(v, idx, strfmt("(%s)(__clz((int)(u32_t)(%s)%s) - %d)", ctype(dt), ut, same(0).c_str(), 32 - bits));
      }
      case Kind::convert: {
        std::string a = same(0);
        if (in_dt == dt) return a;
        if (isf) {
          if (dtype_is_float(in_dt)) return define(v, idx, round_to(dt, a));
          if (in_dt == kPred) return define(v, idx, "(" + a + " ? 1.0f : 0.0f)");
          return define(v, idx, round_to(dt, "(float)" + a));
        }
        if (dt == kPred) return define(v, idx, "(" + a + " != 0)");
        if (dtype_is_float(in_dt)) return define(v, idx, strfmt("f2i<%s>(%s)", ctype(dt), a.c_str()));
        return define(v, idx, strfmt("(%s)%s", ctype(dt), a.c_str()));
      }
      case Kind::bitcast_convert: {
        std::string a = same(0);
        if (dtype_size(in_dt) != dtype_size(dt)) fail("bitcast_convert between different widths");
        if (in_dt == dt) return a;
        if (dt == kF32) return define(v, idx, "__uint_as_float((u32_t)" + a + ")");
        if (in_dt == kF32) return define(v, idx, strfmt("(%s)__float_as_uint(%s)", ctype(dt), a.c_str()));
        if (dt == kBF16) return define(v, idx, "__bfloat162float(__ushort_as_bfloat16((u16_t)" + a + "))");
        if (dt == kF16) return define(v, idx, "__half2float(__ushort_as_half((u16_t)" + a + "))");
        if (in_dt == kBF16) return define(v, idx, strfmt("(%s)__bfloat16_as_ushort(__float2bfloat16_rn(%s))", ctype(dt), a.c_str()));
        if (in_dt == kF16) return define(v, idx, strfmt("(%s)__half_as_ushort(__float2half_rn(%s))", ctype(dt), a.c_str()));
        return define(v, idx, strfmt("(%s)%s", ctype(dt), a.c_str()));
      }
      case Kind::compare: {
        static const char* ops[] = {"==", "!=", ">=", ">", "<=", "<"};
        int64_t dir = ins.scalar("compare_direction", 0);
        if (dir < 0 || dir > 5) fail("bad compare direction");
        return define(v, idx, "(" + same(0) + " " + ops[dir] + " " + same(1) + ")");
      }
      case Kind::select: return define(v, idx, "(" + same(0) + " ? " + same(1) + " : " + same(2) + ")");
      case Kind::clamp: {
        std::string lo = same(0), x = same(1), hi = same(2);
        if (isf) return define(v, idx, "xla_min(xla_max(" + x + ", " + lo + "), " + hi + ")");
        return define(v, idx, strfmt("int_min<%s>(int_max<%s>(%s, %s), %s)", ctype(dt), ctype(dt), x.c_str(), lo.c_str(), hi.c_str()));
      }
      case Kind::reshape: return emit(in(0), idx);
      case Kind::broadcast_in_dim:
        return emit(in(0), broadcast_index(idx, val(in(0)).dims, out.dims, ins.list("broadcast_dimensions")));
      case Kind::transpose: {
        const auto& perm = ins.list("permutation");
        const auto& sd = val(in(0)).dims;
        bool identity = true;
        for (size_t d = 0; d < perm.size(); d++) identity &= perm[d] == (int64_t)d;
        if (identity) return emit(in(0), idx);
        std::vector<std::string> oc = coords(idx.var, out.dims), sc(sd.size(), "0");
        for (size_t d = 0; d < perm.size(); d++) sc[perm[d]] = oc[d];
        return emit(in(0), Idx{index_var(linearize(sc, sd)), IdxClass::GEN});
      }
      case Kind::slice: {
        const auto& st = ins.list("start_indices");
        const auto& sr = ins.list("strides");
        const auto& sd = val(in(0)).dims;
        if (sd == out.dims) return emit(in(0), idx);
        std::vector<std::string> oc = coords(idx.var, out.dims), sc(sd.size());
        for (size_t d = 0; d < sd.size(); d++) {
          int64_t stride = d < sr.size() ? sr[d] : 1, start = d < st.size() ? st[d] : 0;
          std::string e = oc[d];
          if (stride != 1) e = "(" + e + " * " + std::to_string(stride) + ")";
          if (start != 0) e = "(" + e + " + " + std::to_string(start) + ")";
          sc[d] = e;
        }
        return emit(in(0), Idx{index_var(linearize(sc, sd)), IdxClass::GEN});
      }
      case Kind::reverse: {
        const auto& rd = ins.list("dimensions");
        std::vector<std::string> oc = coords(idx.var, out.dims);
        for (int64_t d : rd) oc[d] = "(" + std::to_string(out.dims[d] - 1) + " - " + oc[d] + ")";
        return emit(in(0), Idx{index_var(linearize(oc, out.dims)), IdxClass::GEN});
      }
      case Kind::iota: {
        int64_t d = ins.scalar("iota_dimension", 0);
        if (d < 0 || d >= (int64_t)out.dims.size()) fail("bad iota dimension");
        std::vector<std::string> oc = coords(idx.var, out.dims);
        if (isf) return define(v, idx, round_to(dt, "(float)" + oc[d]));
        return define(v, idx, strfmt("(%s)%s", ctype(dt), oc[d].c_str()));
      }
      case Kind::dynamic_slice: {
        const auto& sd = val(in(0)).dims;
        if (ins.inputs.size() != 1 + sd.size()) fail("dynamic_slice needs one start index per axis");
        std::vector<std::string> oc = coords(idx.var, out.dims), sc(sd.size());
        for (size_t d = 0; d < sd.size(); d++) {
          if (sd[d] == out.dims[d]) {  // start is clamped to 0
            sc[d] = oc[d];
            continue;
          }
          std::string s = emit(in(1 + d), scalar_index());
          std::string cl = index_var(strfmt("min(max((idx_t)%s, (idx_t)0), (idx_t)%lld)", s.c_str(),
                                            (long long)(sd[d] - out.dims[d])));
          sc[d] = "(" + cl + " + " + oc[d] + ")";
        }
        return emit(in(0), Idx{index_var(linearize(sc, sd)), IdxClass::GEN});
      }
      case Kind::pad: {
        // out[o] = operand[(o - low) / (interior + 1)] where every axis lands on an operand element, else the padding
        // scalar. Negative edge padding crops (src/backend/mlx_metal/api.cc:2637 pads with non-negative widths only;
        // StableHLO allows both).
        const auto& sd = val(in(0)).dims;
        const auto& lo = ins.list("edge_padding_low");
        const auto& interior = ins.list("interior_padding");
        if (lo.size() != sd.size() || (!interior.empty() && interior.size() != sd.size())) fail("pad attributes do not match the operand rank");
        std::vector<std::string> oc = coords(idx.var, out.dims), sc(sd.size());
        std::string cond;
        for (size_t d = 0; d < sd.size(); d++) {
          const int64_t step = (interior.empty() ? 0 : interior[d]) + 1;
          if (step < 1) fail("negative interior padding");
          std::string t = index_var("((idx_t)" + oc[d] + " - (idx_t)" + std::to_string(lo[d]) + ")");
          std::string inside = "(" + t + " >= 0 && " + t + " < (idx_t)" + std::to_string((sd[d] - 1) * step + 1);
          if (step > 1) inside += " && " + t + " % " + std::to_string(step) + " == 0";
          inside += ")";
          cond += (cond.empty() ? "" : " && ") + inside;
          sc[d] = step > 1 ? "(" + t + " / " + std::to_string(step) + ")" : t;
        }
        if (cond.empty()) cond = "true";
        std::string name = tmp("t");
        line(std::string(comp_type(dt)) + " " + name + ";");
        line("if (" + cond + ") {");
        {
          Scope inner;
          inner.indent = scope().indent + 2;
          scopes_.push_back(&inner);
          std::string e = emit(in(0), Idx{index_var(linearize(sc, sd)), IdxClass::GEN});
          line(name + " = " + e + ";");
          scopes_.pop_back();
          scope().code += inner.code;
        }
        line("} else {");
        {
          Scope inner;
          inner.indent = scope().indent + 2;
          scopes_.push_back(&inner);
          std::string e = emit(in(1), scalar_index());
          line(name + " = " + e + ";");
          scopes_.pop_back();
          scope().code += inner.code;
        }
        line("}");
        scope().memo[{v, idx.var}] = name;
        return name;
      }
      case Kind::concatenate: {
        int64_t dim = ins.scalar("dimension", 0);
        std::vector<std::string> oc = coords(idx.var, out.dims);
        std::string name = tmp("t");
        line(std::string(comp_type(dt)) + " " + name + ";");
        int64_t offset = 0;
        for (size_t k = 0; k < ins.inputs.size(); k++) {
          const auto& sd = val(in(k)).dims;
          bool last = k + 1 == ins.inputs.size();
          std::string cond = last ? "" : strfmt("if (%s < %lld) ", oc[dim].c_str(), (long long)(offset + sd[dim]));
          line(std::string(k ? "else " : "") + cond + "{");
          Scope inner;
          inner.indent = scope().indent + 2;
          scopes_.push_back(&inner);
          std::vector<std::string> sc = oc;
          if (offset != 0) sc[dim] = "(" + oc[dim] + " - " + std::to_string(offset) + ")";
          std::string e = emit(in(k), Idx{index_var(linearize(sc, sd)), IdxClass::GEN});
          line(name + " = " + e + ";");
          scopes_.pop_back();
          scope().code += inner.code;
          line("}");
          offset += sd[dim];
        }
        scope().memo[{v, idx.var}] = name;
        return name;
      }
      case Kind::gather: {
        // Embedding form only: rows of operand[V, D...] selected by integer ids.
        const auto& od = val(in(0)).dims;
        int64_t row_elems = 1;
        for (size_t d = 1; d < od.size(); d++) row_elems *= od[d];
        int64_t ids = val(in(1)).count();
        if (out.count() != ids * row_elems) fail("gather is not a row lookup");
        std::string b = index_var("(" + idx.var + " / " + std::to_string(row_elems) + ")");
        std::string d = index_var("(" + idx.var + " % " + std::to_string(row_elems) + ")");
        std::string id = emit(in(1), Idx{b, IdxClass::GEN});
        std::string rowv = index_var(strfmt("min(max((idx_t)%s, (idx_t)0), (idx_t)%lld)", id.c_str(), (long long)(od[0] - 1)));
        return emit(in(0), Idx{index_var("(idx_t)" + rowv + " * " + std::to_string(row_elems) + " + " + d), IdxClass::GEN});
      }
      case Kind::reduce_sum: case Kind::reduce_max: case Kind::reduce_min: case Kind::reduce_and: case Kind::reduce_or: {
        auto rv = reduce_var_.find(v);
        if (row_) {
          if (idx.cls != IdxClass::ROW && R_ != 1) fail("reduction result is read at a non-row index");
          if (rv == reduce_var_.end()) fail("reduction result is read before its stage");
          return rv->second;
        }
        if (!allow_serial_) fail("reduction outside a row kernel");
        return emit_serial_reduce(v, idx);
      }
      default:
        fail(std::string("operation cannot be fused: ") + kind_name(ins.kind));
    }
  }

  // ---- reductions -------------------------------------------------------
  struct RedInfo {
    const Instruction* ins;
    bool pair;
    std::string acc, acc_type, init, combine_fn;  // combine_fn(a, b) expression builder name
  };

  std::string reduce_identity(Kind k, int dt) {
    const bool isf = dtype_is_float(dt);
    switch (k) {
      case Kind::reduce_sum: return isf ? "0.0f" : (dt == kPred ? "false" : strfmt("(%s)0", ctype(dt)));
      case Kind::reduce_max:
        if (isf) return "lit_f(0xff800000u)";
        if (dt == kPred) return "false";
        if (dtype_is_unsigned_int(dt)) return strfmt("(%s)0", ctype(dt));
        return strfmt("(%s)((u64_t)1 << %d)", ctype(dt), (int)dtype_size(dt) * 8 - 1);
      case Kind::reduce_min:
        if (isf) return "lit_f(0x7f800000u)";
        if (dt == kPred) return "true";
        if (dtype_is_unsigned_int(dt)) return strfmt("(%s)~(%s)0", ctype(dt), ctype(dt));
        return strfmt("(%s)(((u64_t)1 << %d) - 1)", ctype(dt), (int)dtype_size(dt) * 8 - 1);
      case Kind::reduce_and: return dt == kPred ? "true" : strfmt("(%s)~(%s)0", ctype(dt), ctype(dt));
      case Kind::reduce_or: return dt == kPred ? "false" : strfmt("(%s)0", ctype(dt));
      default: fail("not a reduction");
    }
  }

  std::string reduce_combine(Kind k, int dt, const std::string& a, const std::string& b) {
    const bool isf = dtype_is_float(dt);
    switch (k) {
      case Kind::reduce_sum: return dt == kPred ? "(" + a + " || " + b + ")" : strfmt("(%s)(%s + %s)", comp_type(dt), a.c_str(), b.c_str());
      case Kind::reduce_max:
        return isf ? "xla_max(" + a + ", " + b + ")" : dt == kPred ? "(" + a + " || " + b + ")" : strfmt("int_max<%s>(%s, %s)", ctype(dt), a.c_str(), b.c_str());
      case Kind::reduce_min:
        return isf ? "xla_min(" + a + ", " + b + ")" : dt == kPred ? "(" + a + " && " + b + ")" : strfmt("int_min<%s>(%s, %s)", ctype(dt), a.c_str(), b.c_str());
      case Kind::reduce_and: return dt == kPred ? "(" + a + " && " + b + ")" : strfmt("(%s)(%s & %s)", ctype(dt), a.c_str(), b.c_str());
      case Kind::reduce_or: return dt == kPred ? "(" + a + " || " + b + ")" : strfmt("(%s)(%s | %s)", ctype(dt), a.c_str(), b.c_str());
      default: fail("not a reduction");
    }
  }

  // One thread folds the whole reduced extent of one output element. Used only
  // when the reduced axes are not the trailing ones.
  std::string emit_serial_reduce(uint32_t v, const Idx& idx) {
    const Instruction& ins = prod(v);
    const bool pair = ins.outputs.size() == 2;
    const Value& src = val(ins.inputs[0]);
    const Value& out = val(ins.outputs[0]);
    std::vector<char> red(src.dims.size(), 0);
    for (int64_t d : ins.list("reduce_dimensions")) red[d] = 1;
    std::vector<std::string> oc = coords(idx.var, out.dims), sc(src.dims.size());
    size_t o = 0;
    for (size_t d = 0; d < src.dims.size(); d++)
      if (!red[d]) sc[d] = o < oc.size() ? oc[o++] : "0";
    const int dt = src.dtype;
    std::string acc = tmp("a"), acci;
    if (pair) {
      acci = tmp("a");
      line(strfmt("ArgPair<%s, %s> %s = {%s, 0};", comp_type(dt), comp_type(val(ins.inputs[1]).dtype), acc.c_str(),
                  reduce_identity(Kind::reduce_max, dt).c_str()));
      line("bool " + acci + " = false;");
    } else {
      line(std::string(comp_type(dt)) + " " + acc + " = " + reduce_identity(ins.kind, dt) + ";");
    }
    int opened = 0;
    for (size_t d = 0; d < src.dims.size(); d++) {
      if (!red[d]) continue;
      std::string lv = tmp("k");
      line(strfmt("for (idx_t %s = 0; %s < %lld; %s++) {", lv.c_str(), lv.c_str(), (long long)src.dims[d], lv.c_str()));
      scope().indent += 2;
      sc[d] = lv;
      opened++;
    }
    Scope inner;
    inner.indent = scope().indent;
    scopes_.push_back(&inner);
    Idx sidx{index_var(linearize(sc, src.dims)), IdxClass::GEN};
    std::string e = emit(ins.inputs[0], sidx);
    if (pair) {
      std::string ei = emit(ins.inputs[1], sidx);
      line(strfmt("{ ArgPair<%s, %s> cand = {%s, %s}; %s = %s ? arg_better(%s, cand) : cand; %s = true; }",
                  comp_type(dt), comp_type(val(ins.inputs[1]).dtype), e.c_str(), ei.c_str(), acc.c_str(), acci.c_str(),
                  acc.c_str(), acci.c_str()));
    } else {
      line(acc + " = " + reduce_combine(ins.kind, dt, acc, e) + ";");
    }
    scopes_.pop_back();
    scope().code += inner.code;
    for (int k = 0; k < opened; k++) {
      scope().indent -= 2;
      line("}");
    }
    if (pair) {
      std::string rv = define(ins.outputs[0], idx, round_to(out.dtype, acc + ".v"));
      std::string ri = define(ins.outputs[1], idx, acc + ".i");
      return v == ins.outputs[0] ? rv : ri;
    }
    return define(v, idx, round_to(out.dtype, acc));
  }

  // ---- kernels ----------------------------------------------------------
  // Index into the destination of an in-place slice update for element `i` of the update: update coordinates plus
  // the start indices, each clamped so that the update stays inside the destination (StableHLO semantics).
  std::string scatter_index(const Instruction& ins, const std::string& i) {
    const auto& dd = val(ins.inputs[0]).dims;
    const auto& ud = val(ins.inputs[1]).dims;
    std::vector<std::string> uc = coords(i, ud), dc(dd.size());
    for (size_t d = 0; d < dd.size(); d++) {
      if (ud[d] > dd[d]) fail("slice update larger than its destination");
      if (ud[d] == dd[d]) {  // the clamp leaves 0
        dc[d] = uc[d];
        continue;
      }
      std::string start = emit(ins.inputs[2 + d], scalar_index());
      std::string clamped = index_var(strfmt("min(max((idx_t)%s, (idx_t)0), (idx_t)%lld)", start.c_str(), (long long)(dd[d] - ud[d])));
      dc[d] = uc[d] == "0" ? clamped : "(" + uc[d] + " + " + clamped + ")";
    }
    return index_var(linearize(dc, dd));
  }

  // Map kernel: one grid-stride loop per distinct element count among the stored values and slice updates.
  std::string emit_map_kernel(FusedKernel* k) {
    k->block = 256;
    const int64_t n_max = N_;
    int64_t items = (n_max + vec_ - 1) / vec_;
    k->grid = std::max<int64_t>(1, std::min<int64_t>((items + k->block - 1) / k->block, (int64_t)sm_count_ * 16));
    k->stages = 1;
    struct Item { bool scatter; size_t index; int64_t count; };
    std::vector<Item> all;
    for (size_t s = 0; s < outputs_.size(); s++) all.push_back(Item{false, s, val(outputs_[s]).count()});
    for (size_t q = 0; q < scatters_.size(); q++)
      all.push_back(Item{true, q, val(plan_.instructions[scatters_[q]].inputs[1]).count()});
    std::vector<int64_t> distinct;
    for (const Item& it : all)
      if (std::find(distinct.begin(), distinct.end(), it.count) == distinct.end()) distinct.push_back(it.count);
    Scope top;
    scopes_.push_back(&top);
    std::string loops;
    for (size_t g = 0; g < distinct.size(); g++) {
      N_ = distinct[g];  // contiguity of loads is judged against this loop's extent
      Scope body;
      body.indent = vec_ > 1 ? 6 : 4;
      scopes_.push_back(&body);
      in_vec_loop_ = true;
      vec_loads_.clear();
      Idx lin{"i", IdxClass::LIN};
      std::vector<std::string> decl, after;
      for (const Item& it : all) {
        if (it.count != N_) continue;
        if (!it.scatter) {
          const size_t s = it.index;
          const char* t = ctype(val(outputs_[s]).dtype);
          std::string sv = store_conv(val(outputs_[s]).dtype, emit(outputs_[s], lin));
          line(vec_ > 1 ? strfmt("S%zu[v] = %s;", s, sv.c_str()) : strfmt("out%zu[i] = %s;", s, sv.c_str()));
          if (vec_ > 1) {
            decl.push_back(strfmt("    __align__(16) %s S%zu[%d];\n", t, s, vec_));
            after.push_back(strfmt("    stvec<%s, %d>(out%zu + i0, S%zu);\n", t, vec_, s, s));
          }
        } else {
          const size_t q = it.index;
          const Instruction& ins = plan_.instructions[scatters_[q]];
          const int dt = val(ins.inputs[1]).dtype;
          const char* t = ctype(dt);
          // Vector stores need the trailing full-extent axes of the update to hold whole vectors.
          const auto& dd = val(ins.inputs[0]).dims;
          const auto& ud = val(ins.inputs[1]).dims;
          // (a window inside an axis starts at a run-time offset, so only full axes guarantee alignment)
          int64_t run = 1;
          for (size_t d = ud.size(); d-- > 0 && ud[d] == dd[d];) run *= ud[d];
          std::string sv = store_conv(dt, emit(ins.inputs[1], lin));
          if (vec_ > 1 && run % vec_ == 0) {
            line(strfmt("D%zu[v] = %s;", q, sv.c_str()));
            line(strfmt("if (v == 0) D%zu_at = %s;", q, scatter_index(ins, "i").c_str()));
            decl.push_back(strfmt("    __align__(16) %s D%zu[%d]; idx_t D%zu_at = 0;\n", t, q, vec_, q));
            after.push_back(strfmt("    stvec<%s, %d>(dst%zu + D%zu_at, D%zu);\n", t, vec_, q, q, q));
          } else {
            line(strfmt("dst%zu[%s] = %s;", q, scatter_index(ins, "i").c_str(), sv.c_str()));
          }
        }
      }
      scopes_.pop_back();
      in_vec_loop_ = false;
      // Later loops start at a rotated block so that small loops do not all land on block 0.
      std::string bx = g == 0 ? "blockIdx.x" : strfmt("((blockIdx.x + %zuu) %% gridDim.x)", g);
      if (vec_ > 1) {
        // (Unrolling this loop two or four times, so that more loads are in flight per thread, measured no change on the
        // 705 MB SiLU x up kernel of an 8B-shape prefill: 170 us either way.)
        loops += strfmt("  for (idx_t i0 = ((idx_t)%s * %d + threadIdx.x) * %d; i0 < %lld; i0 += (idx_t)gridDim.x * %d) {\n",
                        bx.c_str(), k->block, vec_, (long long)N_, k->block * vec_);
        for (const VecAccess& a : vec_loads_) {
          const char* t = ctype(val(a.value).dtype);
          loops += strfmt("    __align__(16) %s %s[%d]; ldvec<%s, %d>(%s, in%d + i0);\n", t, a.array.c_str(), vec_, t, vec_,
                          a.array.c_str(), input_slot_[a.value]);
        }
        for (const std::string& d : decl) loops += d;
        loops += strfmt("#pragma unroll\n    for (int v = 0; v < %d; v++) {\n      const idx_t i = i0 + v;\n", vec_);
        loops += body.code;
        loops += "    }\n";
        for (const std::string& d : after) loops += d;
        loops += "  }\n";
      } else {
        loops += strfmt("  for (idx_t i = (idx_t)%s * %d + threadIdx.x; i < %lld; i += (idx_t)gridDim.x * %d) {\n", bx.c_str(),
                        k->block, (long long)N_, k->block);
        loops += body.code;
        loops += "  }\n";
      }
    }
    N_ = n_max;
    std::string code = top.code + loops;
    scopes_.pop_back();
    return code;
  }

  std::string emit_row_kernel(FusedKernel* k) {
    int64_t items = C_ / vec_;
    int block = 32;
    // Many rows: a few items per thread keep the SMs full with small CTAs. Fewer rows than SMs: latency is what
    // counts, so one item per thread (every loop over the row is then a single round of loads).
    static const int few_rows_max = [] {
      const char* v = getenv("PJRTX_B200_ROW_BLOCK_MAX");
      const int n = v && *v ? atoi(v) : 1024;
      return n < 32 ? 32 : n > 1024 ? 1024 : n;
    }();
    if (R_ >= sm_count_) {
      while (block < 512 && block * 4 < items) block *= 2;
    } else {
      while (block < few_rows_max && block < items) block *= 2;
    }
    k->block = block;
    k->grid = std::max<int64_t>(1, std::min<int64_t>(R_, (int64_t)sm_count_ * std::max(1, 2048 / block)));
    // Reductions by stage (a reduction of depth d runs in stage d-1).
    std::vector<const Instruction*> reduces;
    int max_depth = 0;
    for (size_t n : nodes_) {
      const Instruction& ins = plan_.instructions[n];
      if (!is_reduce(ins.kind)) continue;
      // Only reductions that something stored depends on were given a depth.
      if (!depth_.count(ins.outputs[0]) && !(ins.outputs.size() == 2 && depth_.count(ins.outputs[1]))) continue;
      reduces.push_back(&ins);
      max_depth = std::max(max_depth, depth_of(ins.outputs[0]));
    }
    for (uint32_t o : outputs_) max_depth = std::max(max_depth, depth_of(o));
    k->stages = max_depth + 1;
    k->reduce_count = (int)reduces.size();

    Scope kernel_scope;
    scopes_.push_back(&kernel_scope);
    line("__shared__ __align__(16) unsigned long long red_smem[64];");
    line(strfmt("for (idx_t r = blockIdx.x; r < %lld; r += gridDim.x) {", (long long)R_));
    Scope row_scope;
    row_scope.indent = 4;
    scopes_.push_back(&row_scope);
    Idx row_idx{"r", IdxClass::ROW};

    for (int stage = 0; stage <= max_depth; stage++) {
      std::vector<const Instruction*> stage_reduces;
      for (const Instruction* ins : reduces)
        if (depth_of(ins->outputs[0]) == stage + 1) stage_reduces.push_back(ins);
      std::vector<size_t> lin_outputs, row_outputs;
      for (size_t s = 0; s < outputs_.size(); s++) {
        uint32_t o = outputs_[s];
        if (depth_of(o) != stage) continue;
        if (is_reduce(prod(o).kind)) continue;  // stored right after its own stage
        if (val(o).count() == N_ && N_ != R_) lin_outputs.push_back(s);
        else row_outputs.push_back(s);
      }
      // Row-uniform stored values of this depth (functions of earlier reductions only).
      for (size_t s : row_outputs) {
        std::string e = emit(outputs_[s], row_idx);
        line(strfmt("if (threadIdx.x == 0) out%zu[r] = %s;", s, store_conv(val(outputs_[s]).dtype, e).c_str()));
      }
      if (stage_reduces.empty() && lin_outputs.empty()) continue;

      // Accumulators.
      std::vector<std::string> accs;
      for (const Instruction* ins : stage_reduces) {
        const int dt = val(ins->inputs[0]).dtype;
        std::string acc = tmp("acc");
        accs.push_back(acc);
        if (ins->outputs.size() == 2) {
          line(strfmt("ArgPair<%s, %s> %s = {%s, 0}; bool %s_set = false;", comp_type(dt),
                      comp_type(val(ins->inputs[1]).dtype), acc.c_str(), reduce_identity(Kind::reduce_max, dt).c_str(),
                      acc.c_str()));
        } else {
          line(std::string(comp_type(dt)) + " " + acc + " = " + reduce_identity(ins->kind, dt) + ";");
        }
      }
      // Column loop body.
      Scope body;
      body.indent = vec_ > 1 ? 8 : 6;
      scopes_.push_back(&body);
      in_vec_loop_ = true;
      vec_loads_.clear();
      Idx lin{"i", IdxClass::LIN};
      for (size_t q = 0; q < stage_reduces.size(); q++) {
        const Instruction* ins = stage_reduces[q];
        const int dt = val(ins->inputs[0]).dtype;
        std::string e = emit(ins->inputs[0], lin);
        if (ins->outputs.size() == 2) {
          std::string ei = emit(ins->inputs[1], lin);
          line(strfmt("{ ArgPair<%s, %s> cand = {%s, %s}; %s = %s_set ? arg_better(%s, cand) : cand; %s_set = true; }",
                      comp_type(dt), comp_type(val(ins->inputs[1]).dtype), e.c_str(), ei.c_str(), accs[q].c_str(),
                      accs[q].c_str(), accs[q].c_str(), accs[q].c_str()));
        } else {
          line(accs[q] + " = " + reduce_combine(ins->kind, dt, accs[q], e) + ";");
        }
      }
      for (size_t s : lin_outputs) {
        std::string e = emit(outputs_[s], lin);
        std::string sv = store_conv(val(outputs_[s]).dtype, e);
        line(vec_ > 1 ? strfmt("S%zu[v] = %s;", s, sv.c_str()) : strfmt("out%zu[i] = %s;", s, sv.c_str()));
      }
      scopes_.pop_back();
      in_vec_loop_ = false;
      // Assemble the loop in the row scope.
      std::string& code = scope().code;
      if (vec_ > 1) {
        code += strfmt("    for (idx_t c0 = (idx_t)threadIdx.x * %d; c0 < %lld; c0 += %d) {\n", vec_, (long long)C_,
                       block * vec_);
        code += strfmt("      const idx_t i0 = r * (idx_t)%lld + c0;\n", (long long)C_);
        for (const VecAccess& a : vec_loads_) {
          const char* t = ctype(val(a.value).dtype);
          code += strfmt("      __align__(16) %s %s[%d]; ldvec<%s, %d>(%s, in%d + %s);\n", t, a.array.c_str(), vec_, t, vec_,
                         a.array.c_str(), input_slot_[a.value], a.cls == IdxClass::LIN ? "i0" : "c0");
        }
        for (size_t s : lin_outputs) code += strfmt("      __align__(16) %s S%zu[%d];\n", ctype(val(outputs_[s]).dtype), s, vec_);
        code += strfmt("#pragma unroll\n      for (int v = 0; v < %d; v++) {\n        const idx_t c = c0 + v; const idx_t i = i0 + v;\n", vec_);
        code += body.code;
        code += "      }\n";
        for (size_t s : lin_outputs)
          code += strfmt("      stvec<%s, %d>(out%zu + i0, S%zu);\n", ctype(val(outputs_[s]).dtype), vec_, s, s);
        code += "    }\n";
      } else {
        code += strfmt("    for (idx_t c = threadIdx.x; c < %lld; c += %d) {\n      const idx_t i = r * (idx_t)%lld + c;\n",
                       (long long)C_, block, (long long)C_);
        code += body.code;
        code += "    }\n";
      }
      // Finish the stage's reductions.
      for (size_t q = 0; q < stage_reduces.size(); q++) {
        const Instruction* ins = stage_reduces[q];
        const int dt = val(ins->inputs[0]).dtype;
        if (ins->outputs.size() == 2) {
          const char* vt = comp_type(dt);
          const char* it = comp_type(val(ins->inputs[1]).dtype);
          // Threads that saw no element hold the identity with index 0; give them the
          // largest index so they lose every tie.
          line(strfmt("if (!%s_set) %s.i = (%s)(((u64_t)1 << %d) - 1);", accs[q].c_str(), accs[q].c_str(), it,
                      (int)dtype_size(val(ins->inputs[1]).dtype) * 8 - 1));
          std::string res = tmp("red");
          line(strfmt("const ArgPair<%s, %s> %s = block_reduce(%s, [](ArgPair<%s, %s> a, ArgPair<%s, %s> b) { return arg_better(a, b); }, red_smem);",
                      vt, it, res.c_str(), accs[q].c_str(), vt, it, vt, it));
          std::string rv = tmp("red"), ri = tmp("red");
          line(strfmt("const %s %s = %s;", vt, rv.c_str(), round_to(val(ins->outputs[0]).dtype, res + ".v").c_str()));
          line(strfmt("const %s %s = %s.i;", it, ri.c_str(), res.c_str()));
          reduce_var_[ins->outputs[0]] = rv;
          reduce_var_[ins->outputs[1]] = ri;
        } else {
          const char* ct = comp_type(dt);
          std::string res = tmp("red");
          line(strfmt("const %s %s = %s;", ct, res.c_str(),
                      round_to(val(ins->outputs[0]).dtype,
                               strfmt("block_reduce(%s, [](%s a, %s b) { return %s; }, red_smem)", accs[q].c_str(), ct, ct,
                                      reduce_combine(ins->kind, dt, "a", "b").c_str()))
                          .c_str()));
          reduce_var_[ins->outputs[0]] = res;
        }
        for (size_t s = 0; s < outputs_.size(); s++)
          for (uint32_t o : ins->outputs)
            if (outputs_[s] == o)
              line(strfmt("if (threadIdx.x == 0) out%zu[r] = %s;", s, store_conv(val(o).dtype, reduce_var_[o]).c_str()));
      }
    }
    scopes_.pop_back();
    kernel_scope.code += row_scope.code;
    line("}");
    scopes_.pop_back();
    return kernel_scope.code;
  }
};

}  // namespace

bool codegen_fusible(const Plan& plan, const Instruction& ins) {
  if (ins.outputs.empty()) return false;
  for (uint32_t o : ins.outputs)
    if (!ctype(plan.values[o].dtype)) return false;
  for (uint32_t i : ins.inputs)
    if (!ctype(plan.values[i].dtype)) return false;
  switch (ins.kind) {
    case Kind::reduce_sum: case Kind::reduce_max: case Kind::reduce_min: case Kind::reduce_and:
    case Kind::reduce_or:
      return ins.outputs.size() == 1 || (ins.kind == Kind::reduce_max && ins.outputs.size() == 2 && ins.inputs.size() >= 2);
    case Kind::iota: case Kind::concatenate: case Kind::dynamic_slice: case Kind::reverse:
      return true;
    case Kind::pad: {
      if (ins.inputs.size() != 2 || plan.values[ins.inputs[1]].count() != 1) return false;
      const Value& operand = plan.values[ins.inputs[0]];
      const Value& result = plan.values[ins.outputs[0]];
      const auto& lo = ins.list("edge_padding_low");
      const auto& hi = ins.list("edge_padding_high");
      const auto& interior = ins.list("interior_padding");
      if (lo.size() != operand.dims.size() || hi.size() != operand.dims.size() || result.dims.size() != operand.dims.size()) return false;
      if (!interior.empty() && interior.size() != operand.dims.size()) return false;
      for (size_t d = 0; d < operand.dims.size(); d++) {
        const int64_t gap = interior.empty() ? 0 : interior[d];
        if (gap < 0) return false;
        const int64_t span = operand.dims[d] == 0 ? 0 : (operand.dims[d] - 1) * (gap + 1) + 1;
        if (result.dims[d] != std::max<int64_t>(0, lo[d] + span + hi[d])) return false;
      }
      return operand.dtype == result.dtype && plan.values[ins.inputs[1]].dtype == operand.dtype;
    }
    case Kind::optimization_barrier:
      return ins.inputs.size() == 1 && ins.outputs.size() == 1;
    case Kind::gather: {
      // Embedding lookup: operand[V, D...] rows picked by integer ids
      // (the axis-0 `take` fast path of src/backend/mlx_metal/api.cc:2813-2859).
      if (ins.inputs.size() != 2) return false;
      const Value& operand = plan.values[ins.inputs[0]];
      const Value& ids = plan.values[ins.inputs[1]];
      if (operand.dims.empty() || !dtype_is_int(ids.dtype)) return false;
      if (ins.list("collapsed_slice_dims") != std::vector<int64_t>{0}) return false;
      if (ins.list("start_index_map") != std::vector<int64_t>{0}) return false;
      if (!ins.list("operand_batching_dims").empty() || !ins.list("start_indices_batching_dims").empty()) return false;
      const auto& ss = ins.list("slice_sizes");
      if (ss.size() != operand.dims.size() || ss[0] != 1) return false;
      for (size_t d = 1; d < ss.size(); d++)
        if (ss[d] != operand.dims[d]) return false;
      int64_t ivd = ins.scalar("index_vector_dim", (int64_t)ids.dims.size());
      size_t batch_rank = ids.dims.size();
      if (ivd < (int64_t)ids.dims.size()) {
        if (ivd != (int64_t)ids.dims.size() - 1 || ids.dims.back() != 1) return false;
        batch_rank -= 1;
      }
      const auto& od = ins.list("offset_dims");
      if (od.size() != operand.dims.size() - 1) return false;
      for (size_t d = 0; d < od.size(); d++)
        if (od[d] != (int64_t)(batch_rank + d)) return false;
      return true;
    }
    default:
      return program_node_fusible(ins.kind) && ins.kind != Kind::tuple && ins.kind != Kind::get_tuple_element &&
             ins.kind != Kind::reduce_precision && ins.kind != Kind::real && ins.kind != Kind::imag;
  }
}

bool generate_fused_kernel(const Plan& plan, const std::vector<size_t>& nodes, const std::vector<uint32_t>& outputs,
                           const std::vector<size_t>& scatters, int sm_count, FusedKernel* out, std::string* why) {
  for (int serial = 0; serial < 2; serial++) {
    // The one-thread-per-output reduction form is tried only for a lone reduction.
    if (serial == 1 && nodes.size() != 1) break;
    try {
      Gen gen(plan, nodes, outputs, scatters, sm_count);
      *out = gen.run(serial == 1);
      return true;
    } catch (const Fail& f) {
      if (why) *why = f.why;
    }
  }
  return false;
}

}  // namespace pjrtx

// Shared vocabulary of the B200 backend: element types, error reporting.
//
// Element-type codes follow the reference backend's C ABI
// (src/backend/mlx_metal/api.h:107-120) so a runtime that already speaks those
// codes needs no translation table; codes 12+ are additions.
#pragma once

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

namespace pjrtx {

enum DType : int {
  kInvalid = 0,
  kU8 = 1,
  kF32 = 2,
  kPred = 3,
  kS32 = 4,
  kU32 = 5,
  kS8 = 6,
  kF16 = 7,
  kBF16 = 8,
  kC64 = 9,  // declared for code parity; every executable containing it is rejected
  kU16 = 10,
  kU64 = 11,
  kS64 = 12,
  kS16 = 13,
  kF64 = 14,  // declared for code parity; rejected by legalization
};

inline size_t dtype_size(int dt) {
  switch (dt) {
    case kU8: case kPred: case kS8: return 1;
    case kF16: case kBF16: case kU16: case kS16: return 2;
    case kF32: case kS32: case kU32: return 4;
    case kU64: case kS64: case kC64: case kF64: return 8;
    default: return 0;
  }
}

inline const char* dtype_name(int dt) {
  switch (dt) {
    case kU8: return "u8";
    case kF32: return "f32";
    case kPred: return "pred";
    case kS32: return "s32";
    case kU32: return "u32";
    case kS8: return "s8";
    case kF16: return "f16";
    case kBF16: return "bf16";
    case kC64: return "c64";
    case kU16: return "u16";
    case kU64: return "u64";
    case kS64: return "s64";
    case kS16: return "s16";
    case kF64: return "f64";
    default: return "invalid";
  }
}

inline bool dtype_is_float(int dt) { return dt == kF32 || dt == kF16 || dt == kBF16; }
inline bool dtype_is_signed_int(int dt) { return dt == kS8 || dt == kS16 || dt == kS32 || dt == kS64; }
inline bool dtype_is_unsigned_int(int dt) { return dt == kU8 || dt == kU16 || dt == kU32 || dt == kU64; }
inline bool dtype_is_int(int dt) { return dtype_is_signed_int(dt) || dtype_is_unsigned_int(dt); }

// Dense byte size; 0 for invalid types, negative dims or overflow
// (src/compiler/tensor.zig:52-61).
inline uint64_t dense_byte_size(int dt, const std::vector<int64_t>& dims) {
  uint64_t n = dtype_size(dt);
  if (n == 0) return 0;
  for (int64_t d : dims) {
    if (d < 0) return 0;
    if (d != 0 && n > UINT64_MAX / (uint64_t)d) return 0;
    n *= (uint64_t)d;
  }
  return n;
}

inline int64_t element_count(const std::vector<int64_t>& dims) {
  int64_t n = 1;
  for (int64_t d : dims) n *= d;
  return n;
}

// Thread-local message behind pjrtx_b200_last_error().
void set_last_error(const char* fmt, ...);
const char* last_error();

std::string strfmt(const char* fmt, ...);

}  // namespace pjrtx

// StableHLO text reader for the subset of operations the backend executes (see stablehlo_text.cc).
#pragma once

#include <string>

#include "plan.h"

namespace pjrtx {

// Fills `plan` from the module's `func.func @main`. On failure returns false with one diagnostic line in `error`:
//   unsupported op: op=<name> loc=L:C dtype=<t> rank=<r|unknown> sharding=<...> feature=stablehlo-op
//   invalid module: loc=L:C detail="..." feature=stablehlo-text
bool import_stablehlo_text(const std::string& text, Plan* plan, std::string* error);

}  // namespace pjrtx

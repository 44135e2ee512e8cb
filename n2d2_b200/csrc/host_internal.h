// Host-side helpers shared between translation units of the library (internal).
#pragma once
#include <stdint.h>
#include <vector>
#include "../../include/n2d2b.h"

namespace n2d2b {

// Records the calling thread's error message (what n2d2b_last_error returns) and returns `code`.
int set_error(int code, const char* fmt, ...);

// Validates `quant` for `channels` outputs and, when its arithmetic fits the 32-bit epilogue, fills
// consts with [5][cpad] words (lo, hi, mult, add, shift).  acc_bound bounds |accumulator|.
// Returns 0, a negative status on an invalid quant, or 1 when the quant is valid but outside the
// 32-bit form.
int prepare_fast_constants(const n2d2b_quant* quant, int channels, const int32_t* bias, long long acc_bound,
                           std::vector<int32_t>& consts, int* cpad, int* out_unsigned, bool* need_clamp);

}  // namespace n2d2b

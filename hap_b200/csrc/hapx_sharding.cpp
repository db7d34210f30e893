// Ratio -> integer extent rounding, restated from the planner.
//
// Follows fn sharding_round (hap.rs:3536-3559 in the reference): truncate
// ratio * full_length in f64, then hand the remainder out one element at a time to
// the rank whose ratio exceeds its share the most; among equal candidates the
// highest index wins (Rust's max_by_key keeps the last maximum).  full_length == 1
// yields all ones (hap.rs:3538-3540).
#include <string>
#include <vector>

#include "hapx.h"

namespace hapx { int fail(int code, const std::string& msg); }

extern "C" int hapx_sharding_round(int64_t full_length, const double* ratios, int world, int64_t* out_lengths) {
  if (!ratios || !out_lengths || world < 1 || full_length < 0)
    return hapx::fail(HAPX_ERR_ARGUMENT, "sharding_round: bad argument");
  if (full_length == 1) {
    for (int i = 0; i < world; ++i) out_lengths[i] = 1;
    return HAPX_OK;
  }
  const double full = static_cast<double>(full_length);
  int64_t sum = 0;
  for (int i = 0; i < world; ++i) {
    double v = ratios[i] * full;
    int64_t t = (v > 0.0) ? static_cast<int64_t>(v) : 0;  // Rust `as usize`: truncate, saturate at 0
    out_lengths[i] = t;
    sum += t;
  }
  if (sum > full_length) return hapx::fail(HAPX_ERR_EXTENT, "sharding_round: ratios sum to more than 1");
  while (sum < full_length) {
    int best = 0;
    double best_key = 0.0;
    for (int i = 0; i < world; ++i) {
      double key = ratios[i] - static_cast<double>(out_lengths[i]) / full;
      if (i == 0 || key >= best_key) { best = i; best_key = key; }
    }
    out_lengths[best] += 1;
    sum += 1;
  }
  return HAPX_OK;
}

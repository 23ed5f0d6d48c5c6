// Result of KNOperator::profile (reference: include/mirage/profile_result.h:22-28).
#pragma once
#include <limits>
namespace mirage {
struct ProfileResult {
  static constexpr int NUM_WARPUP_ITERATIONS = 1024; // spelling kept from the reference
  static constexpr int NUM_ITERATIONS = 1024;
  float run_time; // milliseconds per launch
  static ProfileResult infinity() { return ProfileResult{std::numeric_limits<float>::max()}; }
};
} // namespace mirage

// Integer helpers usable on host and device (reference: `common/math.hpp:9-38`).
#pragma once

#include "compiled.hpp"

namespace deep_ep::math {

template <typename T>
EP_HOST_DEVICE constexpr T ceil_div(T a, T b) { return (a + b - 1) / b; }

template <typename T>
EP_HOST_DEVICE constexpr T align(T a, T b) { return ceil_div(a, b) * b; }

template <typename T>
EP_HOST_DEVICE constexpr bool is_pow2(T a) { return a > 0 and (a & (a - 1)) == 0; }

}  // namespace deep_ep::math

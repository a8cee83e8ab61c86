// Stand-in for <openvino/genai/generation_config.hpp> used ONLY to compile the reference's
// sampling/logit_transformers.hpp unmodified for the oracle (oracle/ref_sampler_bridge.cpp).
// That header needs nothing from the real file except the standard containers and the
// OPENVINO_ASSERT macro; this shim provides exactly those.  TEST INFRASTRUCTURE.
#pragma once

#include <cstddef>
#include <cstdint>
#include <limits>
#include <map>
#include <memory>
#include <set>
#include <stdexcept>
#include <string>
#include <vector>

namespace ov {
class Exception : public std::runtime_error {
public:
    using std::runtime_error::runtime_error;
};
}  // namespace ov

#define OPENVINO_ASSERT(cond, ...) \
    do {                           \
        if (!(cond)) throw ::ov::Exception(#cond); \
    } while (0)

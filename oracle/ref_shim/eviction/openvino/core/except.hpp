// TEST INFRASTRUCTURE.  Assertion macros of the stand-in OpenVINO headers.
#pragma once

#include <sstream>
#include <stdexcept>
#include <string>

namespace ov {
class Exception : public std::runtime_error {
public:
    explicit Exception(const std::string& what) : std::runtime_error(what) {}
};
namespace shim_detail {
inline void stream_all(std::ostringstream&) {}
template <class T, class... Rest> void stream_all(std::ostringstream& os, const T& first, const Rest&... rest) {
    os << first;
    stream_all(os, rest...);
}
template <class... Args> [[noreturn]] void fail(const char* expr, const Args&... args) {
    std::ostringstream os;
    os << "Check '" << expr << "' failed. ";
    stream_all(os, args...);
    throw Exception(os.str());
}
}  // namespace shim_detail
}  // namespace ov

#define OPENVINO_ASSERT(cond, ...)                                 \
    do {                                                           \
        if (!(cond)) ::ov::shim_detail::fail(#cond, ##__VA_ARGS__); \
    } while (0)
#define OPENVINO_THROW(...) ::ov::shim_detail::fail("throw", ##__VA_ARGS__)
#define OPENVINO_ENUM_DEPRECATED(msg)
#define OPENVINO_DEPRECATED(msg)
#define OPENVINO_GENAI_EXPORTS

// TEST INFRASTRUCTURE.  A stand-in for the OpenVINO runtime header with just the surface that the
// reference's cache_eviction.cpp and kvcrush.cpp touch, so that those two files compile
// unmodified from where they lie: a 1-D f32 tensor with a region-of-interest view, shapes,
// coordinates and the assertion macros.  Nothing here is product code.
#pragma once

#include <algorithm>
#include <cmath>
#include <cstddef>
#include <deque>
#include <functional>
#include <iostream>
#include <limits>
#include <numeric>
#include <queue>
#include <random>
#include <set>
#include <unordered_map>
#include <unordered_set>
#include <list>
#include <optional>
#include <iomanip>
#include <cstring>
#include <map>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#include "openvino/core/except.hpp"

namespace ov {

using Shape = std::vector<size_t>;
using Coordinate = std::vector<size_t>;

namespace element {
enum Type { f32 };
}

class Tensor {
public:
    Tensor() = default;
    Tensor(element::Type, const Shape& shape) : m_shape(shape), m_store(std::make_shared<std::vector<float>>(count(shape))), m_offset(0) {}
    Tensor(element::Type, const Shape& shape, void* host) : m_shape(shape), m_external((float*)host), m_offset(0) {}
    // region of interest [begin, end) of a 1-D tensor; shares the owner's memory
    Tensor(const Tensor& owner, const Coordinate& begin, const Coordinate& end)
        : m_shape{end.at(0) - begin.at(0)}, m_store(owner.m_store), m_external(owner.m_external), m_offset(owner.m_offset + begin.at(0)) {}
    const Shape& get_shape() const { return m_shape; }
    size_t get_size() const { return count(m_shape); }
    element::Type get_element_type() const { return element::f32; }
    template <class T> T* data() const { return reinterpret_cast<T*>(base() + m_offset); }
    void copy_to(Tensor& dst) const { std::memcpy(dst.data<float>(), data<float>(), get_size() * sizeof(float)); }
    explicit operator bool() const { return m_store || m_external; }

private:
    static size_t count(const Shape& s) { size_t n = 1; for (size_t d : s) n *= d; return n; }
    float* base() const { return m_external ? m_external : m_store->data(); }
    Shape m_shape;
    std::shared_ptr<std::vector<float>> m_store;
    float* m_external = nullptr;
    size_t m_offset = 0;
};

}  // namespace ov

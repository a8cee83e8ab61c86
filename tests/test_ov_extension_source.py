"""The OpenVINO extension shim (integration/pa_b200_extension.cpp) cannot be built here (no OpenVINO headers), but
it must at least stay in step with the C ABI: every pa_forward_args member and entry point it names exists in
include/pa_b200.h, and it compiles against a minimal stand-in of the OpenVINO interfaces it uses."""
import re
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

STAND_IN = r'''
#pragma once
#include <cstdint>
#include <cstddef>
#include <memory>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>
namespace ov {
namespace element { enum Type_t { f32, f16, bf16, i32 }; struct Type { Type_t t; Type(Type_t x = f32) : t(x) {} bool operator==(Type_t o) const { return t == o; } }; }
struct Dimension { static Dimension dynamic() { return {}; } };
struct PartialShape { PartialShape() = default; PartialShape(std::initializer_list<Dimension>) {} };
using Shape = std::vector<size_t>;
class Tensor {
public:
    void* data() const { return nullptr; }
    template <class T> T* data() const { return nullptr; }
    Shape get_shape() const { return {1, 1}; }
    size_t get_size() const { return 0; }
    void set_shape(const Shape&) {}
    element::Type get_element_type() const { return element::f32; }
};
using TensorVector = std::vector<Tensor>;
class Node; template <class T> struct Output {}; using OutputVector = std::vector<Output<Node>>;
struct AttributeVisitor { template <class T> void on_attribute(const std::string&, T&) {} };
class Node { public: virtual ~Node() = default; };
namespace op { class Op : public Node { public: Op() = default; explicit Op(const OutputVector&) {}
    virtual void validate_and_infer_types() {} virtual std::shared_ptr<Node> clone_with_new_inputs(const OutputVector&) const = 0;
    virtual bool visit_attributes(AttributeVisitor&) { return true; } virtual bool evaluate(TensorVector&, const TensorVector&) const { return false; }
    virtual bool has_evaluate() const { return false; }
    void constructor_validate_and_infer_types() {} void set_output_type(size_t, element::Type, PartialShape) {}
    element::Type get_input_element_type(size_t) const { return element::f32; } PartialShape get_input_partial_shape(size_t) const { return {}; } }; }
struct Extension { using Ptr = std::shared_ptr<Extension>; virtual ~Extension() = default; };
template <class T> struct OpExtension : Extension {};
template <class... A> inline void assert_fail(A&&... a) { std::ostringstream s; (s << ... << a); throw std::runtime_error(s.str()); }
}
#define OPENVINO_OP(name) static const char* type_name() { return name; }
#define OPENVINO_ASSERT(cond, ...) do { if (!(cond)) ::ov::assert_fail(__VA_ARGS__); } while (0)
#define OPENVINO_CREATE_EXTENSIONS(x) std::vector<ov::Extension::Ptr> create_extensions() { return x; }
'''


def test_shim_names_only_what_the_header_declares():
    src = (ROOT / "integration" / "pa_b200_extension.cpp").read_text()
    header = (ROOT / "include" / "pa_b200.h").read_text()
    for member in set(re.findall(r"\ba\.(\w+)\s*=", src)):
        assert re.search(r"\b%s\s*;" % member, header), f"pa_forward_args has no member {member}"
    for fn in set(re.findall(r"\b(pa_b200_\w+)\s*\(", src)):
        assert re.search(r"\b%s\s*\(" % fn, header), f"{fn} is not declared in pa_b200.h"


def test_shim_compiles_against_a_stand_in_of_the_openvino_interfaces(tmp_path):
    inc = tmp_path / "openvino"
    for sub in ("core", "op"):
        (inc / sub).mkdir(parents=True)
    (inc / "stand_in.hpp").write_text(STAND_IN)
    for rel in ("core/extension.hpp", "core/op_extension.hpp", "op/op.hpp"):
        (inc / rel).write_text('#include "../stand_in.hpp"\n')
    cmd = ["g++", "-std=c++17", "-fsyntax-only", "-I", str(tmp_path), "-I", str(ROOT / "include"), str(ROOT / "integration" / "pa_b200_extension.cpp")]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr

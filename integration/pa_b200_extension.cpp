// OpenVINO extension operator whose evaluate() runs the PagedAttention step through the C ABI of
// libgenai_b200.so (include/pa_b200.h).
//
// This is the reference's own route for foreign operators: an extension library that exports
// OPENVINO_CREATE_EXTENSIONS with an ov::OpExtension<T>, T : ov::op::Op implementing
// validate_and_infer_types / clone_with_new_inputs / visit_attributes / evaluate / has_evaluate
// (tests/cpp/custom_op/custom_add.hpp:10-23, custom_add.cpp:49-84, ov_extension.cpp:12-16), loaded with
// ov::genai::extensions(path) (src/cpp/include/openvino/genai/extensions.hpp:19-56) and registered through
// ov::Core::add_extension (src/cpp/src/utils.cpp:996-1015).  Continuous batching runs such an operator end to
// end in tests/python_tests/test_continuous_batching.py:984-1023.
//
// Built only where OpenVINO's developer package is installed (integration/CMakeLists.txt, option
// GENAI_B200_BUILD_OV_EXTENSION); the rest of the repository does not depend on it.
//
// Inputs, by the tensor names ModelRunner fills (src/cpp/src/continuous_batching/model_runner.hpp:505-522,
// 802-853, 1420-1509); input 3 / 4 are the cache tensors KVCacheManager owns (cache/kv_cache_manager.hpp:74-113):
//    0 query  1 key  2 value  3 key_cache  4 value_cache  5 past_lens  6 subsequence_begins  7 block_indices
//    8 block_indices_begins  9 scale  10 max_context_len  11 score_aggregation_window
//    12 rotated_block_indices  13 rotation_deltas  14 rotation_trig_lut
// Outputs: 0 attention output [tokens, Hq * D]; 1 scores [sum of past + new tokens] (f32) when input 11 is not empty.
#include <memory>
#include <mutex>
#include <vector>

#include <openvino/core/extension.hpp>
#include <openvino/core/op_extension.hpp>
#include <openvino/op/op.hpp>

#include "pa_b200.h"

namespace genai_b200_ov {

class PagedAttentionB200 : public ov::op::Op {
public:
    OPENVINO_OP("PagedAttentionB200");

    PagedAttentionB200() = default;
    PagedAttentionB200(const ov::OutputVector& args, int64_t num_q_heads, int64_t num_kv_heads, int64_t head_size, int64_t block_size,
                       int64_t cache_dtype, int64_t device)
        : Op(args), m_hq(num_q_heads), m_hkv(num_kv_heads), m_d(head_size), m_bs(block_size), m_cache(cache_dtype), m_device(device) {
        constructor_validate_and_infer_types();
    }

    void validate_and_infer_types() override {
        // output 0 has the query's type and shape; output 1 is a dynamic f32 vector
        set_output_type(0, get_input_element_type(0), get_input_partial_shape(0));
        set_output_type(1, ov::element::f32, ov::PartialShape{ov::Dimension::dynamic()});
    }

    std::shared_ptr<ov::Node> clone_with_new_inputs(const ov::OutputVector& new_args) const override {
        return std::make_shared<PagedAttentionB200>(new_args, m_hq, m_hkv, m_d, m_bs, m_cache, m_device);
    }

    bool visit_attributes(ov::AttributeVisitor& visitor) override {
        visitor.on_attribute("num_q_heads", m_hq);
        visitor.on_attribute("num_kv_heads", m_hkv);
        visitor.on_attribute("head_size", m_d);
        visitor.on_attribute("block_size", m_bs);
        visitor.on_attribute("cache_dtype", m_cache);   // pa_dtype: PA_DTYPE_F16 / BF16 / U8
        visitor.on_attribute("device", m_device);
        return true;
    }

    bool has_evaluate() const override { return true; }

    bool evaluate(ov::TensorVector& out, const ov::TensorVector& in) const override {
        OPENVINO_ASSERT(in.size() >= 11, "PagedAttentionB200 expects at least 11 inputs, got ", in.size());
        pa_handle* handle = ensure_handle(in[0].get_element_type());
        pa_forward_args a{};
        a.struct_size = sizeof(a);
        a.query = in[0].data();
        a.key = in[1].data();
        a.value = in[2].data();
        out[0].set_shape(in[0].get_shape());
        a.output = out[0].data();
        a.num_tokens = static_cast<int32_t>(in[0].get_shape()[0]);
        a.key_cache = in[3].data();     // device memory owned by KVCacheManager, layout of pa_b200_query_cache_layout
        a.value_cache = in[4].data();
        a.num_blocks = static_cast<int32_t>(in[3].get_shape()[0]);
        a.past_lens = in[5].data<int32_t>();
        a.num_sequences = static_cast<int32_t>(in[5].get_size());
        a.subsequence_begins = in[6].data<int32_t>();
        a.block_indices = in[7].data<int32_t>();
        a.num_block_indices = static_cast<int32_t>(in[7].get_size());
        a.block_indices_begins = in[8].data<int32_t>();
        a.scale = in[9].get_size() ? *in[9].data<float>() : 0.0f;
        a.max_context_len = *in[10].data<int32_t>();
        if (in.size() > 11 && in[11].get_size()) {
            // one slot of past_len + new tokens floats per sequence, in scheduled order (model_runner.hpp:1529-1537)
            size_t total = 0;
            const int32_t* past = in[5].data<int32_t>();
            const int32_t* begins = in[6].data<int32_t>();
            for (int32_t s = 0; s < a.num_sequences; ++s) total += static_cast<size_t>(past[s]) + static_cast<size_t>(begins[s + 1] - begins[s]);
            out[1].set_shape({total});
            a.score_aggregation_window = in[11].data<int32_t>();
            a.scores = out[1].data<float>();
            a.scores_len = static_cast<int64_t>(total);
        } else {
            out[1].set_shape({0});
        }
        if (in.size() > 14 && in[12].get_size()) {
            a.rotated_block_indices = in[12].data<int32_t>();
            a.rotation_deltas = in[13].data<int32_t>();
            a.num_rotated_blocks = static_cast<int32_t>(in[12].get_size());
            a.rotation_trig_lut = in[14].data<float>();
            a.rotation_lut_rows = static_cast<int32_t>(in[14].get_shape()[0]);
        }
        const int rc = pa_b200_forward_host(handle, &a);   // host tensors in and out, the cache stays on the device
        OPENVINO_ASSERT(rc == PA_OK, "pa_b200_forward_host: ", pa_b200_last_error());   // errors become ov::Exception, as elsewhere in genai
        return true;
    }

    ~PagedAttentionB200() override {
        if (m_handle) pa_b200_destroy(m_handle);
    }

private:
    pa_handle* ensure_handle(const ov::element::Type& act) const {
        std::lock_guard<std::mutex> lock(m_mutex);
        if (!m_handle) {
            pa_model_desc desc{};
            desc.struct_size = sizeof(desc);
            desc.num_q_heads = static_cast<int32_t>(m_hq);
            desc.num_kv_heads = static_cast<int32_t>(m_hkv);
            desc.head_size = static_cast<int32_t>(m_d);
            desc.block_size = static_cast<int32_t>(m_bs);
            desc.act_dtype = act == ov::element::f32 ? PA_DTYPE_F32 : act == ov::element::bf16 ? PA_DTYPE_BF16 : PA_DTYPE_F16;
            desc.cache_dtype = static_cast<int32_t>(m_cache);
            const int rc = pa_b200_create(&desc, static_cast<int>(m_device), &m_handle);
            OPENVINO_ASSERT(rc == PA_OK, "pa_b200_create: ", pa_b200_last_error());
        }
        return m_handle;
    }

    int64_t m_hq = 0, m_hkv = 0, m_d = 0, m_bs = 0, m_cache = PA_DTYPE_U8, m_device = 0;
    mutable std::mutex m_mutex;
    mutable pa_handle* m_handle = nullptr;
};

}  // namespace genai_b200_ov

OPENVINO_CREATE_EXTENSIONS(std::vector<ov::Extension::Ptr>({std::make_shared<ov::OpExtension<genai_b200_ov::PagedAttentionB200>>()}));

// The plugin's quantisation fusion: see quant_fusion.hpp for the list of rewrites and where nGraph's CPU backend
// keeps its own version of each.  Every rule below is a hand-written test on the nodes around a candidate root (no
// pattern matcher), and every rule states when the rewritten graph computes the same numbers as the original:
// "exact" rules never change a result; the convolution rules change WHERE the value is rounded (the integer output of
// the fused op has the range of u8 after the relu instead of i8 before it), which is the purpose of the fusion.
#include "quant_fusion.hpp"

#include <cstring>
#include <vector>

#include "ngraph/function.hpp"
#include "ngraph/graph_util.hpp"
#include "ngraph/op/add.hpp"
#include "ngraph/op/broadcast.hpp"
#include "ngraph/op/concat.hpp"
#include "ngraph/op/constant.hpp"
#include "ngraph/op/convert.hpp"
#include "ngraph/op/dequantize.hpp"
#include "ngraph/op/divide.hpp"
#include "ngraph/op/experimental/quantized_conv_bias.hpp"
#include "ngraph/op/experimental/quantized_conv_relu.hpp"
#include "ngraph/op/max_pool.hpp"
#include "ngraph/op/multiply.hpp"
#include "ngraph/op/quantize.hpp"
#include "ngraph/op/quantized_convolution.hpp"
#include "ngraph/op/relu.hpp"
#include "ngraph/op/reshape.hpp"
#include "ngraph/pass/pass_config.hpp"

using namespace ngraph;

namespace
{
    using NodePtr = std::shared_ptr<Node>;

    std::shared_ptr<op::v0::Constant> constant_of(const Output<Node>& v)
    {
        return as_type_ptr<op::v0::Constant>(v.get_node_shared_ptr());
    }

    // a Constant all of whose bytes are zero (integer 0 and +0.0f alike)
    bool is_zero_constant(const Output<Node>& v)
    {
        auto c = constant_of(v);
        if (!c)
            return false;
        const size_t bytes = shape_size(c->get_output_shape(0)) * c->get_output_element_type(0).size();
        const char* p = static_cast<const char*>(c->get_data_ptr());
        for (size_t i = 0; i < bytes; ++i)
            if (p[i])
                return false;
        return true;
    }

    // the same value: one node, or two Constants of equal type and element count holding equal bytes
    bool same_constant(const Output<Node>& a, const Output<Node>& b)
    {
        if (a == b)
            return true;
        auto ca = constant_of(a), cb = constant_of(b);
        if (!ca || !cb || ca->get_output_element_type(0) != cb->get_output_element_type(0) ||
            shape_size(ca->get_output_shape(0)) != shape_size(cb->get_output_shape(0)))
            return false;
        const size_t bytes = shape_size(ca->get_output_shape(0)) * ca->get_output_element_type(0).size();
        return memcmp(ca->get_data_ptr(), cb->get_data_ptr(), bytes) == 0;
    }

    // an f32 Constant whose every element is > 0 and far from both ends of the float range: a quantisation scale that keeps
    // the order of values, and for which code * scale (|code| <= 255) neither overflows nor goes subnormal, so that
    // (code * scale) / scale gives the code back and dequantised values compare like their codes
    bool is_positive_scale(const Output<Node>& v)
    {
        auto c = constant_of(v);
        if (!c || c->get_output_element_type(0) != element::f32)
            return false;
        const float* p = static_cast<const float*>(c->get_data_ptr());
        for (size_t i = 0, n = shape_size(c->get_output_shape(0)); i < n; ++i)
            if (!(p[i] >= 1.0e-30f) || p[i] > 1.0e30f)
                return false;
        return true;
    }

    size_t user_count(const Output<Node>& v) { return v.get_target_inputs().size(); }

    // Relu commutes with a Dequantize only for a positive scale.  A run-time scale cannot be inspected (quantisation
    // scales are positive by construction and the CPU backend fuses without looking); a Constant that is not positive
    // rules the rewrite out.
    bool may_be_positive_scale(const Output<Node>& v) { return !constant_of(v) || is_positive_scale(v); }

    // Steps back over Reshape / Broadcast nodes that change nothing (same shape in and out, no transposition): frameworks
    // leave such nodes between a Dequantize and the Add that consumes it.
    Output<Node> skip_identity_layout(Output<Node> v)
    {
        for (int guard = 0; guard < 8; ++guard)
        {
            Node* n = v.get_node();
            const bool reshape = is_type<op::v0::Reshape>(n) && !static_cast<op::v0::Reshape*>(n)->get_is_transpose();
            const bool broadcast = is_type<op::v0::Broadcast>(n) && static_cast<op::v0::Broadcast*>(n)->get_broadcast_axes().empty();
            if (!(reshape || broadcast) || n->get_input_shape(0) != n->get_output_shape(0))
                break;
            v = n->input_value(0);
        }
        return v;
    }

    // Dequantize to f32 with one scale for the whole tensor and zero point 0
    std::shared_ptr<op::v0::Dequantize> plain_dequantize(const Output<Node>& v)
    {
        auto dq = as_type_ptr<op::v0::Dequantize>(v.get_node_shared_ptr());
        if (!dq || !dq->get_axes().empty() || dq->get_output_element_type(0) != element::f32 || !is_zero_constant(dq->input_value(2)))
            return nullptr;
        return dq;
    }

    NodePtr zero_like(const element::Type& et, const Shape& shape)
    {
        std::vector<char> zeros(shape_size(shape) * et.size(), 0);
        return std::make_shared<op::v0::Constant>(et, shape, zeros.data());
    }

    using Counts = runtime::b200::pass::QuantFusion::Counts;

    // ---- Relu(Dequantize(conv)) ----------------------------------------------------------------------------
    // cpu_fusion.cpp:2025-2157.  The fused op applies the relu before it rounds and saturates to u8, so an output that
    // the un-fused graph would clip at 127 keeps its value up to 255; everything below 127 is the same number.
    bool fuse_conv_relu(const NodePtr& relu, Counts& counts)
    {
        auto dq = plain_dequantize(relu->input_value(0));
        if (!dq || user_count(dq->input_value(0)) != 1 || !may_be_positive_scale(dq->input_value(1)))
            return false;
        NodePtr conv = dq->input_value(0).get_node_shared_ptr();
        NodePtr fused;
        if (auto cb = as_type_ptr<op::v0::QuantizedConvolutionBias>(conv))
        {
            if (cb->with_relu())
                return false;
            fused = std::make_shared<op::v0::QuantizedConvolutionBias>(
                cb->input_value(0), cb->input_value(1), cb->input_value(2), cb->get_window_movement_strides(),
                cb->get_window_dilation_strides(), cb->get_padding_below(), cb->get_padding_above(),
                cb->get_data_dilation_strides(), cb->input_value(3), true);
            ++counts.conv_bias_relu;
        }
        else if (auto c = as_type_ptr<op::v0::QuantizedConvolution>(conv))
        {
            // inputs: data, filters, input scale, input zp, filter scale, filter zp, output scale, output zp
            const bool scalars = shape_size(c->get_input_shape(2)) == 1 && shape_size(c->get_input_shape(4)) == 1 &&
                                 shape_size(c->get_input_shape(6)) == 1;
            if (c->get_input_element_type(0) != element::u8 || c->get_input_element_type(1) != element::i8 ||
                c->get_output_element_type(0) != element::i8 || !scalars || !is_zero_constant(c->input_value(3)) ||
                !is_zero_constant(c->input_value(5)) || !is_zero_constant(c->input_value(7)) || !c->get_input_axes().empty() ||
                !c->get_filter_axes().empty() || !c->get_output_axes().empty())
                return false;
            auto product = std::make_shared<op::v1::Multiply>(c->input_value(2), c->input_value(4));
            auto requantize = std::make_shared<op::v1::Divide>(product, c->input_value(6));
            fused = std::make_shared<op::v0::QuantizedConvolutionRelu>(
                c->input_value(0), c->input_value(1), c->get_window_movement_strides(), c->get_window_dilation_strides(),
                c->get_padding_below(), c->get_padding_above(), c->get_data_dilation_strides(), requantize);
            ++counts.conv_relu;
        }
        else
            return false;
        auto out = std::make_shared<op::v0::Dequantize>(fused, dq->input_value(1),
                                                        zero_like(element::u8, dq->get_input_shape(2)), element::f32, dq->get_axes());
        relu->output(0).replace(out->output(0));
        return true;
    }

    // ---- Relu(Add(Dequantize(QuantizedConvolutionBias), Dequantize(summand))) ------------------------------------
    // cpu_fusion.cpp:2357-2540.  The CPU backend also demands that the summand can be overwritten in place (not a
    // Parameter, no later reader); the device kernel reads the summand and writes a separate output, so those two
    // conditions do not apply here.
    struct AddBranch
    {
        std::shared_ptr<op::v0::Dequantize> dq;
        std::shared_ptr<op::v0::QuantizedConvolutionBias> conv; // null for a branch that can only be the summand
    };

    AddBranch add_branch(const Output<Node>& v)
    {
        AddBranch b;
        b.dq = plain_dequantize(skip_identity_layout(v));
        if (b.dq)
        {
            auto cb = as_type_ptr<op::v0::QuantizedConvolutionBias>(b.dq->input_value(0).get_node_shared_ptr());
            if (cb && !cb->with_relu() && user_count(cb->output(0)) == 1)
                b.conv = cb;
        }
        return b;
    }

    bool fuse_conv_bias_add(const NodePtr& relu, Counts& counts)
    {
        auto add = as_type_ptr<op::v1::Add>(relu->input_value(0).get_node_shared_ptr());
        if (!add)
            return false;
        AddBranch left = add_branch(add->input_value(0)), right = add_branch(add->input_value(1));
        if (!left.dq || !right.dq || !may_be_positive_scale(left.dq->input_value(1)) || !may_be_positive_scale(right.dq->input_value(1)))
            return false;
        if (left.conv && right.conv)
        {
            // both sides are convolutions: the one whose scale the following Quantize uses becomes the fused op
            for (auto& in : relu->output(0).get_target_inputs())
                if (auto q = as_type<op::v0::Quantize>(in.get_node()))
                {
                    if (!same_constant(q->input_value(1), left.dq->input_value(1)) &&
                        same_constant(q->input_value(1), right.dq->input_value(1)))
                        std::swap(left, right);
                    break;
                }
        }
        else if (!left.conv)
            std::swap(left, right);
        if (!left.conv)
            return false;
        Output<Node> summand = right.dq->input_value(0);
        const element::Type& st = summand.get_element_type();
        if ((st != element::i8 && st != element::u8) || summand.get_shape() != left.conv->get_output_shape(0) ||
            relu->get_output_shape(0) != left.conv->get_output_shape(0))
            return false;
        auto& cb = left.conv;
        auto sum_scale = std::make_shared<op::v1::Divide>(right.dq->input_value(1), left.dq->input_value(1));
        NodePtr fused;
        if (st == element::i8)
            fused = std::make_shared<op::v0::Convert>(
                std::make_shared<op::v0::QuantizedConvolutionBiasSignedAdd>(
                    cb->input_value(0), cb->input_value(1), cb->input_value(2), summand, cb->get_window_movement_strides(),
                    cb->get_window_dilation_strides(), cb->get_padding_below(), cb->get_padding_above(),
                    cb->get_data_dilation_strides(), cb->input_value(3), sum_scale, true),
                element::u8);
        else
            fused = std::make_shared<op::v0::QuantizedConvolutionBiasAdd>(
                cb->input_value(0), cb->input_value(1), cb->input_value(2), summand, cb->get_window_movement_strides(),
                cb->get_window_dilation_strides(), cb->get_padding_below(), cb->get_padding_above(),
                cb->get_data_dilation_strides(), cb->input_value(3), sum_scale, true);
        auto out = std::make_shared<op::v0::Dequantize>(fused, left.dq->input_value(1), zero_like(element::u8, Shape{}),
                                                        element::f32, AxisSet{});
        relu->output(0).replace(out->output(0));
        ++counts.conv_bias_add;
        return true;
    }

    // ---- MaxPool(Dequantize(x)) -> Dequantize(MaxPool(x)) ----------------------------------------------------------
    // cpu_fusion.cpp:2219-2261.  Exact when one positive scale covers the tensor: x -> (x - zp) * scale then keeps the
    // order of values, so the largest integer of a window dequantises to the largest float.  (The CPU backend does
    // not look at the scale; a negative or per-axis scale is left alone here.)
    bool swap_max_pool(const NodePtr& node, Counts& counts)
    {
        auto pool = as_type_ptr<op::v0::MaxPool>(node);
        auto dq = pool ? as_type_ptr<op::v0::Dequantize>(pool->input_value(0).get_node_shared_ptr()) : nullptr;
        if (!dq || !dq->get_axes().empty() || !is_positive_scale(dq->input_value(1)) || !constant_of(dq->input_value(2)))
            return false;
        const element::Type& et = dq->get_input_element_type(0);
        if (et != element::u8 && et != element::i8)
            return false;
        auto moved = std::make_shared<op::v0::MaxPool>(dq->input_value(0), pool->get_window_shape(), pool->get_window_movement_strides(),
                                                       pool->get_padding_below(), pool->get_padding_above(), pool->get_pad_type(),
                                                       pool->get_ceil_mode());
        auto out = std::make_shared<op::v0::Dequantize>(moved, dq->input_value(1), dq->input_value(2), dq->get_output_element_type(0),
                                                        dq->get_axes());
        pool->output(0).replace(out->output(0));
        ++counts.max_pool;
        return true;
    }

    // ---- Concat(Dequantize(x_i)...) -> Dequantize(Concat(x_i...)) --------------------------------------------------
    // cpu_fusion.cpp:2263-2326.  Exact: every element goes through the same (x - zp) * scale either way.  The CPU
    // backend compares the scales only; the zero points and element types have to agree as well for that to hold.
    bool hoist_concat(const NodePtr& node, Counts& counts)
    {
        auto concat = as_type_ptr<op::v0::Concat>(node);
        if (!concat || concat->get_input_size() < 2)
            return false;
        std::shared_ptr<op::v0::Dequantize> first;
        OutputVector sources;
        for (size_t i = 0; i < concat->get_input_size(); ++i)
        {
            auto dq = as_type_ptr<op::v0::Dequantize>(concat->input_value(i).get_node_shared_ptr());
            if (!dq || !dq->get_axes().empty())
                return false;
            if (!first)
                first = dq;
            else if (!same_constant(dq->input_value(1), first->input_value(1)) || !same_constant(dq->input_value(2), first->input_value(2)) ||
                     dq->get_input_element_type(0) != first->get_input_element_type(0) ||
                     dq->get_output_element_type(0) != first->get_output_element_type(0))
                return false;
            sources.push_back(dq->input_value(0));
        }
        if (!constant_of(first->input_value(1)) || !constant_of(first->input_value(2)))
            return false;
        auto joined = std::make_shared<op::v0::Concat>(sources, concat->get_concatenation_axis());
        auto out = std::make_shared<op::v0::Dequantize>(joined, first->input_value(1), first->input_value(2),
                                                        first->get_output_element_type(0), first->get_axes());
        concat->output(0).replace(out->output(0));
        ++counts.concat;
        return true;
    }

    // ---- Quantize(Dequantize(x)) -> x ------------------------------------------------------------------------------
    // cpu_fusion.cpp:2328-2355.  With equal scales, zero points 0 and the same integer type, (x * s) / s is within a few
    // ulps of the integer x, so any round-to-nearest mode returns x: exact.  The directed modes (toward zero, up, down,
    // toward infinity) could land one below or above and are left alone.
    bool drop_dequantize_quantize(const NodePtr& node, Counts& counts)
    {
        auto q = as_type_ptr<op::v0::Quantize>(node);
        auto dq = q ? as_type_ptr<op::v0::Dequantize>(q->input_value(0).get_node_shared_ptr()) : nullptr;
        if (!dq || !q->get_axes().empty() || !dq->get_axes().empty())
            return false;
        using RM = op::v0::Quantize::RoundMode;
        const RM rm = q->get_round_mode();
        const bool nearest = rm == RM::ROUND_NEAREST_TOWARD_EVEN || rm == RM::ROUND_NEAREST_TOWARD_INFINITY ||
                             rm == RM::ROUND_NEAREST_TOWARD_ZERO || rm == RM::ROUND_NEAREST_UPWARD || rm == RM::ROUND_NEAREST_DOWNWARD;
        const element::Type& et = dq->get_input_element_type(0);
        if (!nearest || q->get_output_element_type(0) != et || (et != element::u8 && et != element::i8) ||
            !is_zero_constant(q->input_value(2)) || !is_zero_constant(dq->input_value(2)) || !is_positive_scale(q->input_value(1)) ||
            !same_constant(q->input_value(1), dq->input_value(1)))
            return false;
        q->output(0).replace(dq->input_value(0));
        ++counts.dq_q;
        return true;
    }
}

bool runtime::b200::pass::quant_fusion_enabled()
{
    ngraph::pass::PassConfig config; // reads NGRAPH_PASS_ENABLES
    auto& knobs = config.get_enables();
    auto it = knobs.find("B200QuantFusion");
    return it == knobs.end() || it->second;
}

bool runtime::b200::pass::QuantFusion::run_on_function(std::shared_ptr<Function> function)
{
    m_counts = Counts();
    // One rewrite changes the users of nodes later in the order, so the walk restarts after each one.  Every rewrite
    // removes at least one f32 op from the path it touched, which bounds the number of rounds by the size of the graph.
    const size_t limit = function->get_ordered_ops().size() + 1;
    for (size_t round = 0; round < limit; ++round)
    {
        bool changed = false;
        for (auto& node : function->get_ordered_ops())
        {
            if (is_type<op::v0::Relu>(node))
                changed = fuse_conv_bias_add(node, m_counts) || fuse_conv_relu(node, m_counts);
            else
                changed = swap_max_pool(node, m_counts) || hoist_concat(node, m_counts) || drop_dequantize_quantize(node, m_counts);
            if (changed)
                break;
        }
        if (!changed)
            break;
    }
    return m_counts.total() > 0;
}

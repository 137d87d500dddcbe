// Batch split of a lowered Function (see batch_split.hpp).
//
// The graph is rebuilt node by node in topological order.  Every value is either REPLICATED (it does not depend on the
// batch: constants, scales, weights, anything computed from them) or CARRIED: its leading extent is a multiple of the
// batch, its memory is batch-major (the rows of sample i are contiguous and come before those of sample i + 1), and the
// rows of sample i depend on sample i of the inputs only.  A carried value of the split graph has the same shape with the
// leading extent scaled by rows / batch.  Each op type has a rule that says when its output is carried; anything not
// covered by a rule fails the split, so a graph is only ever split when every node has been vouched for.
#include "batch_split.hpp"

#include <cstring>
#include <map>

#include "ngraph/ngraph.hpp"
#include "ngraph/op/experimental/batch_mat_mul.hpp"
#include "ngraph/op/experimental/quantized_conv_bias.hpp"
#include "ngraph/op/experimental/quantized_conv_relu.hpp"
#include "ngraph/op/experimental/quantized_dot_bias.hpp"
#include "ngraph/op/gelu.hpp"
#include "ngraph/op/layer_norm.hpp"
#include "ngraph/op/stop_gradient.hpp"

using namespace ngraph;

namespace
{
    struct Failure
    {
        std::string why;
    };

    [[noreturn]] void fail(const Node& n, const std::string& why)
    {
        throw Failure{std::string(n.get_type_name()) + " " + n.get_name() + ": " + why};
    }

    struct Splitter
    {
        size_t batch, rows;
        std::map<const Node*, std::shared_ptr<Node>> made; // original node -> its counterpart in the split graph
        std::map<const Node*, bool> carried;               // by original node (all ops of the path have one output)

        bool is_carried(const Output<Node>& v) const { return carried.at(v.get_node()); }
        Output<Node> in(const Node& n, size_t i) const
        {
            const Output<Node> src = n.input_value(i);
            return made.at(src.get_node())->output(src.get_index());
        }
        OutputVector inputs(const Node& n) const
        {
            OutputVector v;
            for (size_t i = 0; i < n.get_input_size(); ++i)
                v.push_back(in(n, i));
            return v;
        }
        size_t scaled(const Node& n, size_t extent) const
        {
            if (extent % batch != 0)
                fail(n, "leading extent " + std::to_string(extent) + " is not a multiple of the batch");
            return extent / batch * rows;
        }
        Shape scaled_shape(const Node& n, Shape s) const
        {
            if (s.empty())
                fail(n, "a scalar cannot carry the batch");
            s[0] = scaled(n, s[0]);
            return s;
        }
        // inputs `which` must be carried, every other one replicated
        void expect(const Node& n, std::initializer_list<size_t> which) const
        {
            for (size_t i = 0; i < n.get_input_size(); ++i)
            {
                bool want = false;
                for (size_t w : which)
                    want = want || w == i;
                if (is_carried(n.input_value(i)) != want)
                    fail(n, "input " + std::to_string(i) + (want ? " does not carry the batch" : " carries the batch"));
            }
        }
        bool any_carried(const Node& n) const
        {
            for (size_t i = 0; i < n.get_input_size(); ++i)
                if (is_carried(n.input_value(i)))
                    return true;
            return false;
        }
        bool all_carried(const Node& n) const
        {
            for (size_t i = 0; i < n.get_input_size(); ++i)
                if (!is_carried(n.input_value(i)))
                    return false;
            return n.get_input_size() > 0;
        }

        // Input i of `n` is replicated but has the full batch-carrying shape: acceptable when it is a Constant made of `batch`
        // identical blocks; the split graph then uses a Constant of the first rows.
        Output<Node> periodic_constant_rows(const Node& n, size_t i)
        {
            auto c = as_type_ptr<op::v0::Constant>(n.input_value(i).get_node_shared_ptr());
            if (!c)
                fail(n, "an operand spans the batch without carrying it");
            const Shape shape = c->get_output_shape(0);
            if (shape.empty() || shape[0] % batch != 0)
                fail(n, "a constant operand spans the batch without carrying it");
            const size_t bytes = shape_size(shape) * c->get_output_element_type(0).size(), block = bytes / batch;
            const char* data = static_cast<const char*>(c->get_data_ptr());
            for (size_t b = 1; b < batch; ++b)
                if (std::memcmp(data, data + b * block, block) != 0)
                    fail(n, "a constant operand spans the batch and differs between samples");
            return std::make_shared<op::v0::Constant>(c->get_output_element_type(0), scaled_shape(n, shape), data)->output(0);
        }

        // the op with its inputs replaced; shapes follow from the op's own shape inference
        void copy(const std::shared_ptr<Node>& n, bool is_carried_now)
        {
            made[n.get()] = n->copy_with_new_inputs(inputs(*n));
            carried[n.get()] = is_carried_now;
        }

        void visit(const std::shared_ptr<Node>& n)
        {
            const Node& node = *n;
            if (node.get_output_size() != 1)
                fail(node, "more than one output");
            if (auto p = as_type_ptr<op::v0::Parameter>(n))
            {
                const Shape s = p->get_output_shape(0);
                const bool c = !s.empty() && s[0] == batch;
                made[n.get()] = std::make_shared<op::v0::Parameter>(p->get_element_type(), c ? scaled_shape(node, s) : s);
                carried[n.get()] = c;
                return;
            }
            if (is_type<op::v0::Constant>(n))
            {
                made[n.get()] = n; // shared with the original graph: constants are immutable
                carried[n.get()] = false;
                return;
            }
            if (!any_carried(node))
            {
                copy(n, false); // computed from replicated values only (scale arithmetic and the like)
                return;
            }
            if (is_type<op::v0::Result>(n))
            {
                copy(n, true);
                return;
            }
            // ---- one batch-carrying input, the rest parameters of the op
            if (is_type<op::v0::Quantize>(n) || is_type<op::v0::Dequantize>(n))
            {
                expect(node, {0});
                const AxisSet axes = is_type<op::v0::Quantize>(n) ? as_type_ptr<op::v0::Quantize>(n)->get_axes()
                                                                  : as_type_ptr<op::v0::Dequantize>(n)->get_axes();
                if (axes.count(0))
                    fail(node, "scales along the batch axis");
                return copy(n, true);
            }
            if (is_type<op::v0::QuantizedConvolution>(n) || is_type<op::v0::QuantizedConvolutionBias>(n) ||
                is_type<op::v0::QuantizedConvolutionRelu>(n))
            {
                expect(node, {0});
                return copy(n, true);
            }
            if (is_type<op::v0::QuantizedConvolutionBiasAdd>(n) || is_type<op::v0::QuantizedConvolutionBiasSignedAdd>(n))
            {
                expect(node, {0, 3}); // data and the summand
                return copy(n, true);
            }
            if (is_type<op::v0::QuantizedDot>(n) || is_type<op::v0::QuantizedDotBias>(n))
            {
                expect(node, {0});
                if (node.get_input_shape(0).size() != 2)
                    fail(node, "rank");
                return copy(n, true);
            }
            if (auto d = as_type_ptr<op::v0::Dot>(n))
            {
                expect(node, {0});
                if (node.get_input_shape(0).size() < 2 || d->get_reduction_axes_count() >= node.get_input_shape(0).size())
                    fail(node, "the reduction reaches the batch axis");
                return copy(n, true);
            }
            if (is_type<op::v0::MaxPool>(n) || is_type<op::v0::AvgPool>(n))
                return copy(n, true);
            if (auto ln = as_type_ptr<op::v0::LayerNorm>(n))
            {
                expect(node, {0});
                const int64_t rank = int64_t(node.get_input_shape(0).size());
                const int64_t axis = ln->get_begin_norm_axis() >= 0 ? ln->get_begin_norm_axis() : rank + ln->get_begin_norm_axis();
                if (axis < 1 || ln->get_keep_stats())
                    fail(node, "normalises over the batch axis");
                return copy(n, true);
            }
            if (auto g = as_type_ptr<op::v0::Gather>(n))
            {
                expect(node, {1}); // rows of a replicated table picked by batch-carrying indices
                if (g->get_axis() != 0)
                    fail(node, "axis");
                return copy(n, true);
            }
            // ---- elementwise
            if (is_type<op::v0::Abs>(n) || is_type<op::v0::Negative>(n) || is_type<op::v0::Sqrt>(n) || is_type<op::v0::Exp>(n) ||
                is_type<op::v0::Erf>(n) || is_type<op::v0::Relu>(n) || is_type<op::v0::Convert>(n) || is_type<op::v0::Gelu>(n) ||
                is_type<op::v0::StopGradient>(n))
                return copy(n, true);
            if (is_type<op::v1::Add>(n) || is_type<op::v1::Subtract>(n) || is_type<op::v1::Multiply>(n) || is_type<op::v1::Divide>(n) ||
                is_type<op::v1::Maximum>(n) || is_type<op::v1::Minimum>(n))
            {
                // equal shapes (broadcasts are explicit nodes by now).  A replicated operand of the full shape can only be a
                // Constant whose samples are all alike (a broadcast bias row that ConstantFolding expanded): its first rows serve
                if (node.get_input_shape(0) != node.get_input_shape(1))
                    fail(node, "operand shapes differ");
                OutputVector operands;
                for (size_t i = 0; i < 2; ++i)
                    operands.push_back(is_carried(node.input_value(i)) ? in(node, i) : periodic_constant_rows(node, i));
                made[n.get()] = n->copy_with_new_inputs(operands);
                carried[n.get()] = true;
                return;
            }
            // ---- reductions and Softmax: never across the batch axis
            if (is_type<op::v0::Sum>(n) || is_type<op::v0::Max>(n) || is_type<op::v0::Min>(n))
            {
                expect(node, {0});
                const AxisSet axes = std::dynamic_pointer_cast<op::util::ArithmeticReduction>(n)->get_reduction_axes();
                if (axes.count(0))
                    fail(node, "reduces over the batch axis");
                return copy(n, true);
            }
            if (auto sm = as_type_ptr<op::v0::Softmax>(n))
            {
                expect(node, {0});
                if (sm->get_axes().count(0))
                    fail(node, "normalises over the batch axis");
                return copy(n, true);
            }
            if (is_type<op::v0::BatchMatMul>(n))
            {
                if (!all_carried(node))
                    fail(node, "one operand does not carry the batch");
                return copy(n, true);
            }
            if (auto c = as_type_ptr<op::v0::Concat>(n))
            {
                if (!all_carried(node) || c->get_concatenation_axis() == 0)
                    fail(node, "concatenates along the batch axis or mixes carried and replicated operands");
                return copy(n, true);
            }
            // ---- ops with a shape attribute: rebuilt with the scaled shape
            if (auto r = as_type_ptr<op::v0::Reshape>(n))
            {
                const AxisVector order = r->get_input_order();
                const Shape out = r->get_reshape_output_shape();
                if (out.empty())
                    fail(node, "to a scalar");
                if (r->get_is_transpose())
                {
                    // the batch axis stays in front and whole
                    if (order.empty() || order[0] != 0 || out[0] != node.get_input_shape(0)[0])
                        fail(node, "moves the batch axis");
                }
                made[n.get()] = std::make_shared<op::v0::Reshape>(in(node, 0), order, scaled_shape(node, out));
                carried[n.get()] = true;
                return;
            }
            fail(node, "no rule for this op");
        }

        // A Broadcast of a replicated value that gains a leading extent which is a multiple of the batch: every row is the
        // same, so the split graph simply broadcasts to fewer rows and the result counts as carried.
        bool visit_broadcast(const std::shared_ptr<Node>& n)
        {
            auto b = as_type_ptr<op::v0::Broadcast>(n);
            if (!b)
                return false;
            const Shape out = b->get_broadcast_shape();
            const AxisSet axes = b->get_broadcast_axes();
            const bool src_carried = is_carried(n->input_value(0));
            if (src_carried)
            {
                if (axes.count(0))
                    fail(*n, "adds an axis in front of the batch axis");
                made[n.get()] = std::make_shared<op::v0::Broadcast>(in(*n, 0), scaled_shape(*n, out), axes);
                carried[n.get()] = true;
            }
            else if (!out.empty() && axes.count(0) && out[0] % batch == 0 && out[0] >= batch)
            {
                made[n.get()] = std::make_shared<op::v0::Broadcast>(in(*n, 0), scaled_shape(*n, out), axes);
                carried[n.get()] = true;
            }
            else
            {
                made[n.get()] = n->copy_with_new_inputs(inputs(*n));
                carried[n.get()] = false;
            }
            return true;
        }
    };
}

size_t ngraph::runtime::b200::batch_of(const Function& function)
{
    const auto& params = function.get_parameters();
    if (params.empty() || !params[0]->get_partial_shape().is_static() || params[0]->get_output_shape(0).empty())
        return 0;
    return params[0]->get_output_shape(0)[0];
}

bool ngraph::runtime::b200::split_batch(const Function& function, size_t rows, BatchSplit& out, std::string& why)
{
    Splitter s;
    s.batch = batch_of(function);
    s.rows = rows;
    if (s.batch == 0 || rows == 0 || rows > s.batch)
    {
        why = "no batch axis, or more shards than rows";
        return false;
    }
    try
    {
        for (const auto& n : const_cast<Function&>(function).get_ordered_ops())
        {
            if (!s.visit_broadcast(n))
                s.visit(n);
            // the rebuilt node's own shape inference must agree with the rule
            if (s.carried.at(n.get()) && !is_type<op::v0::Result>(n))
            {
                Shape expect = n->get_output_shape(0);
                if (expect.empty() || expect[0] % s.batch != 0)
                    fail(*n, "result does not have a batch-major leading extent");
                expect[0] = expect[0] / s.batch * rows;
                if (s.made.at(n.get())->get_output_shape(0) != expect)
                    fail(*n, "shape inference of the split graph disagrees");
            }
        }
        ParameterVector params;
        ResultVector results;
        out.parameter_split.clear();
        out.result_split.clear();
        for (const auto& p : function.get_parameters())
        {
            params.push_back(as_type_ptr<op::v0::Parameter>(s.made.at(p.get())));
            out.parameter_split.push_back(s.carried.at(p.get()));
        }
        for (const auto& r : function.get_results())
        {
            if (!s.carried.at(r.get()))
                fail(*r, "a result that does not carry the batch");
            results.push_back(as_type_ptr<op::v0::Result>(s.made.at(r.get())));
            out.result_split.push_back(true);
        }
        out.function = std::make_shared<Function>(results, params);
    }
    catch (const Failure& f)
    {
        why = f.why;
        return false;
    }
    catch (const std::exception& e) // a rebuilt node that fails its own validation
    {
        why = e.what();
        return false;
    }
    return true;
}

// Binary Function (de)serialisation for the plugin's op set (see function_io.hpp).
#include "function_io.hpp"

#include <cstring>
#include <functional>
#include <map>
#include <stdexcept>
#include <unordered_map>

#include "ngraph/except.hpp"
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
    const char MAGIC[8] = {'B', '2', 'F', 'N', '0', '0', '0', '1'};

    struct Writer
    {
        std::string s;
        void raw(const void* p, size_t n) { s.append(static_cast<const char*>(p), n); }
        void u64(uint64_t v) { raw(&v, 8); }
        void i64(int64_t v) { raw(&v, 8); }
        void f64(double v) { raw(&v, 8); }
        void str(const std::string& v)
        {
            u64(v.size());
            raw(v.data(), v.size());
        }
        template <typename V>
        void sizes(const V& v)
        {
            u64(v.size());
            for (auto x : v)
                i64(int64_t(x));
        }
        void type(const element::Type& t) { str(t.get_type_name()); }
        void autob(const op::AutoBroadcastSpec& b)
        {
            u64(uint64_t(b.m_type));
            i64(b.m_axis);
        }
    };

    struct Reader
    {
        const char* p;
        const char* end;
        void raw(void* out, size_t n)
        {
            if (size_t(end - p) < n)
                throw std::runtime_error("B200 saved model: truncated");
            memcpy(out, p, n);
            p += n;
        }
        uint64_t u64()
        {
            uint64_t v;
            raw(&v, 8);
            return v;
        }
        int64_t i64()
        {
            int64_t v;
            raw(&v, 8);
            return v;
        }
        double f64()
        {
            double v;
            raw(&v, 8);
            return v;
        }
        std::string str()
        {
            uint64_t n = u64();
            if (size_t(end - p) < n)
                throw std::runtime_error("B200 saved model: truncated");
            std::string v(p, size_t(n));
            p += n;
            return v;
        }
        template <typename V>
        V sizes()
        {
            uint64_t n = u64();
            if (n > (1u << 20))
                throw std::runtime_error("B200 saved model: implausible vector length");
            V v;
            for (uint64_t i = 0; i < n; ++i)
                v.push_back(typename V::value_type(i64()));
            return v;
        }
        AxisSet axis_set()
        {
            AxisSet a;
            for (size_t x : sizes<std::vector<size_t>>())
                a.insert(x);
            return a;
        }
        element::Type type()
        {
            static const std::vector<element::Type> all = {element::boolean, element::bf16, element::f16, element::f32, element::f64,
                                                           element::i8,      element::i16,  element::i32, element::i64, element::u1,
                                                           element::u8,      element::u16,  element::u32, element::u64};
            const std::string name = str();
            for (const auto& t : all)
                if (t.get_type_name() == name)
                    return t;
            throw std::runtime_error("B200 saved model: unknown element type " + name);
        }
        op::AutoBroadcastSpec autob()
        {
            const auto t = static_cast<op::AutoBroadcastType>(u64());
            const int64_t axis = i64();
            return op::AutoBroadcastSpec(t, axis);
        }
    };

    std::vector<size_t> axes_vector(const AxisSet& a) { return std::vector<size_t>(a.begin(), a.end()); }

    // type key: name and opset version ("Add:1")
    std::string key_of(const Node& n) { return std::string(n.get_type_info().name) + ":" + std::to_string(n.get_type_info().version); }

    template <typename OP>
    void write_conv_geometry(Writer& w, const OP& c)
    {
        w.sizes(c.get_window_movement_strides());
        w.sizes(c.get_window_dilation_strides());
        w.sizes(c.get_padding_below());
        w.sizes(c.get_padding_above());
        w.sizes(c.get_data_dilation_strides());
    }
    struct ConvGeometry
    {
        Strides strides, dilation, data_dilation;
        CoordinateDiff below, above;
    };
    ConvGeometry read_conv_geometry(Reader& r)
    {
        ConvGeometry g;
        g.strides = r.sizes<Strides>();
        g.dilation = r.sizes<Strides>();
        g.below = r.sizes<CoordinateDiff>();
        g.above = r.sizes<CoordinateDiff>();
        g.data_dilation = r.sizes<Strides>();
        return g;
    }

    using Maker = std::function<std::shared_ptr<Node>(Reader&, const OutputVector&)>;

    // ---- attribute writers, one per op type with attributes; ops without attributes write nothing ----------------------
    bool write_attributes(Writer& w, const Node& n)
    {
        if (auto p = as_type<const op::v0::Parameter>(&n))
        {
            w.type(p->get_output_element_type(0));
            w.sizes(p->get_output_shape(0));
            return true;
        }
        if (auto c = as_type<const op::v0::Constant>(&n))
        {
            w.type(c->get_output_element_type(0));
            w.sizes(c->get_output_shape(0));
            const size_t bytes = shape_size(c->get_output_shape(0)) * c->get_output_element_type(0).size();
            w.u64(bytes);
            w.raw(c->get_data_ptr(), bytes);
            return true;
        }
        if (auto q = as_type<const op::v0::Quantize>(&n))
        {
            w.type(q->get_output_element_type(0));
            w.sizes(axes_vector(q->get_axes()));
            w.u64(uint64_t(q->get_round_mode()));
            return true;
        }
        if (auto d = as_type<const op::v0::Dequantize>(&n))
        {
            w.type(d->get_output_element_type(0));
            w.sizes(axes_vector(d->get_axes()));
            return true;
        }
        if (auto d = as_type<const op::v0::QuantizedDot>(&n))
        {
            w.u64(d->get_reduction_axes_count());
            w.type(d->get_output_type());
            w.sizes(axes_vector(d->get_input0_axes()));
            w.sizes(axes_vector(d->get_input1_axes()));
            w.sizes(axes_vector(d->get_output_axes()));
            return true;
        }
        if (auto d = as_type<const op::v0::QuantizedDotBias>(&n))
        {
            w.u64(d->requantize());
            w.u64(d->with_relu());
            return true;
        }
        if (auto c = as_type<const op::v0::QuantizedConvolution>(&n))
        {
            write_conv_geometry(w, *c);
            w.type(c->get_output_type());
            w.sizes(axes_vector(c->get_input_axes()));
            w.sizes(axes_vector(c->get_filter_axes()));
            w.sizes(axes_vector(c->get_output_axes()));
            return true;
        }
        if (auto c = as_type<const op::v0::QuantizedConvolutionBias>(&n))
        {
            write_conv_geometry(w, *c);
            w.u64(c->with_relu());
            return true;
        }
        if (auto c = as_type<const op::v0::QuantizedConvolutionBiasAdd>(&n))
        {
            write_conv_geometry(w, *c);
            w.u64(c->with_relu());
            return true;
        }
        if (auto c = as_type<const op::v0::QuantizedConvolutionBiasSignedAdd>(&n))
        {
            write_conv_geometry(w, *c);
            w.u64(c->with_relu());
            return true;
        }
        if (auto c = as_type<const op::v0::QuantizedConvolutionRelu>(&n))
        {
            write_conv_geometry(w, *c);
            return true;
        }
        if (auto c = as_type<const op::v0::Convolution>(&n))
        {
            write_conv_geometry(w, *c);
            return true;
        }
        if (auto m = as_type<const op::v0::MaxPool>(&n))
        {
            w.sizes(m->get_window_shape());
            w.sizes(m->get_window_movement_strides());
            w.sizes(m->get_padding_below());
            w.sizes(m->get_padding_above());
            w.u64(uint64_t(m->get_pad_type()));
            w.u64(m->get_ceil_mode());
            return true;
        }
        if (auto a = as_type<const op::v0::AvgPool>(&n))
        {
            w.sizes(a->get_window_shape());
            w.sizes(a->get_window_movement_strides());
            w.sizes(a->get_padding_below());
            w.sizes(a->get_padding_above());
            w.u64(a->get_include_padding_in_avg_computation());
            w.u64(uint64_t(a->get_pad_type()));
            w.u64(a->get_ceil_mode());
            return true;
        }
        if (auto r = as_type<const op::v0::Reshape>(&n))
        {
            w.sizes(r->get_input_order());
            w.sizes(r->get_reshape_output_shape());
            return true;
        }
        if (auto c = as_type<const op::v0::Convert>(&n))
        {
            w.type(c->get_destination_type());
            return true;
        }
        if (auto c = as_type<const op::v0::Concat>(&n))
        {
            w.i64(c->get_concatenation_axis());
            return true;
        }
        if (auto b = as_type<const op::v0::Broadcast>(&n))
        {
            w.sizes(b->get_broadcast_shape());
            w.sizes(axes_vector(b->get_broadcast_axes()));
            return true;
        }
        if (auto b = dynamic_cast<const op::util::BinaryElementwiseArithmetic*>(&n))
        {
            w.autob(b->get_autob());
            if (auto d = as_type<const op::v1::Divide>(&n))
                w.u64(d->is_pythondiv());
            return true;
        }
        if (auto d = as_type<const op::v0::Dot>(&n))
        {
            w.u64(d->get_reduction_axes_count());
            w.u64(d->get_has_reduction_axes_count());
            return true;
        }
        if (auto g = as_type<const op::v0::Gather>(&n))
        {
            w.u64(g->get_axis());
            return true;
        }
        if (auto l = as_type<const op::v0::LayerNorm>(&n))
        {
            w.u64(l->get_keep_stats());
            w.i64(l->get_begin_norm_axis());
            w.f64(l->get_epsilon());
            return true;
        }
        return false;
    }

    const std::unordered_map<std::string, Maker>& makers()
    {
        static std::unordered_map<std::string, Maker> m;
        if (!m.empty())
            return m;
        auto add = [&](const Node& proto, Maker f) { m[key_of(proto)] = std::move(f); };
#define B200_UNARY(OP) add(OP(), [](Reader&, const OutputVector& in) -> std::shared_ptr<Node> { return std::make_shared<OP>(in.at(0)); })
#define B200_TWO_INPUTS(OP) add(OP(), [](Reader&, const OutputVector& in) -> std::shared_ptr<Node> { return std::make_shared<OP>(in.at(0), in.at(1)); })
        // ops whose whole state is their inputs (the reduction axes of Sum / Max / Min / Softmax are their second input)
        B200_UNARY(op::v0::Result);
        B200_UNARY(op::v0::Abs);
        B200_UNARY(op::v0::Negative);
        B200_UNARY(op::v0::Sqrt);
        B200_UNARY(op::v0::Exp);
        B200_UNARY(op::v0::Erf);
        B200_UNARY(op::v0::Relu);
        B200_UNARY(op::v0::Gelu);
        B200_UNARY(op::v0::StopGradient);
        B200_TWO_INPUTS(op::v0::BatchMatMul);
        B200_TWO_INPUTS(op::v0::Sum);
        B200_TWO_INPUTS(op::v0::Max);
        B200_TWO_INPUTS(op::v0::Min);
        B200_TWO_INPUTS(op::v0::Softmax);
#undef B200_UNARY
#undef B200_TWO_INPUTS
        add(op::v0::Parameter(), [](Reader& r, const OutputVector&) -> std::shared_ptr<Node> {
            const element::Type t = r.type();
            return std::make_shared<op::v0::Parameter>(t, r.sizes<Shape>());
        });
        add(op::v0::Constant(), [](Reader& r, const OutputVector&) -> std::shared_ptr<Node> {
            const element::Type t = r.type();
            const Shape s = r.sizes<Shape>();
            const uint64_t bytes = r.u64();
            if (bytes != shape_size(s) * t.size() || size_t(r.end - r.p) < bytes)
                throw std::runtime_error("B200 saved model: constant size mismatch");
            auto c = std::make_shared<op::v0::Constant>(t, s, static_cast<const void*>(r.p));
            r.p += bytes;
            return c;
        });
        add(op::v0::Quantize(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const element::Type t = r.type();
            const AxisSet axes = r.axis_set();
            const auto mode = static_cast<op::v0::Quantize::RoundMode>(r.u64());
            return std::make_shared<op::v0::Quantize>(in.at(0), in.at(1), in.at(2), t, axes, mode);
        });
        add(op::v0::Dequantize(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const element::Type t = r.type();
            return std::make_shared<op::v0::Dequantize>(in.at(0), in.at(1), in.at(2), t, r.axis_set());
        });
        add(op::v0::QuantizedDot(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const size_t count = size_t(r.u64());
            const element::Type t = r.type();
            const AxisSet a0 = r.axis_set(), a1 = r.axis_set(), ao = r.axis_set();
            return std::make_shared<op::v0::QuantizedDot>(in.at(0), in.at(1), count, in.at(2), in.at(3), in.at(4), in.at(5), in.at(6),
                                                          in.at(7), t, a0, a1, ao);
        });
        add(op::v0::QuantizedDotBias(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const bool requantize = r.u64() != 0, relu = r.u64() != 0;
            return std::make_shared<op::v0::QuantizedDotBias>(in.at(0), in.at(1), in.at(2), in.at(3), requantize, relu);
        });
        add(op::v0::QuantizedConvolution(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const ConvGeometry g = read_conv_geometry(r);
            const element::Type t = r.type();
            const AxisSet ai = r.axis_set(), af = r.axis_set(), ao = r.axis_set();
            return std::make_shared<op::v0::QuantizedConvolution>(in.at(0), in.at(1), g.strides, g.dilation, g.below, g.above,
                                                                  g.data_dilation, in.at(2), in.at(3), in.at(4), in.at(5), in.at(6),
                                                                  in.at(7), t, ai, af, ao);
        });
        add(op::v0::QuantizedConvolutionBias(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const ConvGeometry g = read_conv_geometry(r);
            const bool relu = r.u64() != 0;
            return std::make_shared<op::v0::QuantizedConvolutionBias>(in.at(0), in.at(1), in.at(2), g.strides, g.dilation, g.below,
                                                                      g.above, g.data_dilation, in.at(3), relu);
        });
        add(op::v0::QuantizedConvolutionBiasAdd(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const ConvGeometry g = read_conv_geometry(r);
            const bool relu = r.u64() != 0;
            return std::make_shared<op::v0::QuantizedConvolutionBiasAdd>(in.at(0), in.at(1), in.at(2), in.at(3), g.strides, g.dilation,
                                                                         g.below, g.above, g.data_dilation, in.at(4), in.at(5), relu);
        });
        add(op::v0::QuantizedConvolutionBiasSignedAdd(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const ConvGeometry g = read_conv_geometry(r);
            const bool relu = r.u64() != 0;
            return std::make_shared<op::v0::QuantizedConvolutionBiasSignedAdd>(in.at(0), in.at(1), in.at(2), in.at(3), g.strides,
                                                                               g.dilation, g.below, g.above, g.data_dilation,
                                                                               in.at(4), in.at(5), relu);
        });
        add(op::v0::QuantizedConvolutionRelu(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const ConvGeometry g = read_conv_geometry(r);
            return std::make_shared<op::v0::QuantizedConvolutionRelu>(in.at(0), in.at(1), g.strides, g.dilation, g.below, g.above,
                                                                      g.data_dilation, in.at(2));
        });
        add(op::v0::Convolution(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const ConvGeometry g = read_conv_geometry(r);
            return std::make_shared<op::v0::Convolution>(in.at(0), in.at(1), g.strides, g.dilation, g.below, g.above, g.data_dilation);
        });
        add(op::v0::MaxPool(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const Shape win = r.sizes<Shape>();
            const Strides st = r.sizes<Strides>();
            const Shape below = r.sizes<Shape>(), above = r.sizes<Shape>();
            const auto pad = static_cast<op::PadType>(r.u64());
            const bool ceil = r.u64() != 0;
            return std::make_shared<op::v0::MaxPool>(in.at(0), win, st, below, above, pad, ceil);
        });
        add(op::v0::AvgPool(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const Shape win = r.sizes<Shape>();
            const Strides st = r.sizes<Strides>();
            const Shape below = r.sizes<Shape>(), above = r.sizes<Shape>();
            const bool include = r.u64() != 0;
            const auto pad = static_cast<op::PadType>(r.u64());
            const bool ceil = r.u64() != 0;
            return std::make_shared<op::v0::AvgPool>(in.at(0), win, st, below, above, include, pad, ceil);
        });
        add(op::v0::Reshape(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const AxisVector order = r.sizes<AxisVector>();
            return std::make_shared<op::v0::Reshape>(in.at(0), order, r.sizes<Shape>());
        });
        add(op::v0::Convert(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            return std::make_shared<op::v0::Convert>(in.at(0), r.type());
        });
        add(op::v0::Concat(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            return std::make_shared<op::v0::Concat>(in, r.i64());
        });
        add(op::v0::Broadcast(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const Shape s = r.sizes<Shape>();
            return std::make_shared<op::v0::Broadcast>(in.at(0), s, r.axis_set());
        });
#define B200_BINARY(OP) add(OP(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> { return std::make_shared<OP>(in.at(0), in.at(1), r.autob()); })
        B200_BINARY(op::v1::Add);
        B200_BINARY(op::v1::Subtract);
        B200_BINARY(op::v1::Multiply);
        B200_BINARY(op::v1::Maximum);
        B200_BINARY(op::v1::Minimum);
#undef B200_BINARY
        add(op::v1::Divide(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const op::AutoBroadcastSpec b = r.autob();
            return std::make_shared<op::v1::Divide>(in.at(0), in.at(1), r.u64() != 0, b);
        });
        add(op::v0::Dot(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const size_t count = size_t(r.u64());
            const bool has = r.u64() != 0;
            return std::make_shared<op::v0::Dot>(in.at(0), in.at(1), count, has);
        });
        add(op::v0::Gather(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            return std::make_shared<op::v0::Gather>(in.at(0), in.at(1), size_t(r.u64()));
        });
        add(op::v0::LayerNorm(), [](Reader& r, const OutputVector& in) -> std::shared_ptr<Node> {
            const bool keep = r.u64() != 0;
            const int64_t axis = r.i64();
            const double eps = r.f64();
            if (in.size() == 3)
                return std::make_shared<op::v0::LayerNorm>(in.at(0), in.at(1), in.at(2), keep, axis, eps);
            return std::make_shared<op::v0::LayerNorm>(in.at(0), keep, axis, eps);
        });
        return m;
    }
}

uint64_t runtime::b200::fnv1a(const void* data, size_t bytes)
{
    uint64_t h = 1469598103934665603ull;
    const unsigned char* p = static_cast<const unsigned char*>(data);
    for (size_t i = 0; i < bytes; ++i)
        h = (h ^ p[i]) * 1099511628211ull;
    return h;
}

std::string runtime::b200::write_function(const Function& function)
{
    Writer w;
    w.raw(MAGIC, sizeof(MAGIC));
    const auto nodes = const_cast<Function&>(function).get_ordered_ops();
    std::map<const Node*, uint64_t> id;
    w.u64(nodes.size());
    for (const auto& node : nodes)
    {
        const std::string key = key_of(*node);
        if (makers().find(key) == makers().end())
            throw unsupported_op("B200 backend: cannot save a Function that holds a " + key + " node (" + node->get_name() + ")");
        w.str(key);
        w.str(node->get_friendly_name());
        w.u64(node->get_input_size());
        for (size_t i = 0; i < node->get_input_size(); ++i)
        {
            const Output<Node> src = node->input_value(i);
            w.u64(id.at(src.get_node()));
            w.u64(src.get_index());
        }
        write_attributes(w, *node);
        const uint64_t position = id.size();
        id[node.get()] = position;
    }
    // parameters and results in the Function's own order
    w.u64(function.get_parameters().size());
    for (const auto& p : function.get_parameters())
        w.u64(id.at(p.get()));
    w.u64(function.get_results().size());
    for (const auto& r : function.get_results())
        w.u64(id.at(r.get()));
    return w.s;
}

std::shared_ptr<Function> runtime::b200::read_function(const std::string& bytes, std::vector<std::shared_ptr<Node>>* nodes_in_saved_order)
{
    Reader r{bytes.data(), bytes.data() + bytes.size()};
    char magic[8];
    r.raw(magic, 8);
    if (memcmp(magic, MAGIC, 8) != 0)
        throw std::runtime_error("B200 saved model: not a model written by this plugin version");
    const uint64_t count = r.u64();
    if (count > (1u << 24))
        throw std::runtime_error("B200 saved model: implausible node count");
    std::vector<std::shared_ptr<Node>> nodes;
    nodes.reserve(size_t(count));
    for (uint64_t n = 0; n < count; ++n)
    {
        const std::string key = r.str();
        const std::string friendly = r.str();
        const uint64_t inputs = r.u64();
        OutputVector in;
        for (uint64_t i = 0; i < inputs; ++i)
        {
            const uint64_t src = r.u64(), index = r.u64();
            if (src >= nodes.size() || index >= nodes[size_t(src)]->get_output_size())
                throw std::runtime_error("B200 saved model: input refers to a node that does not exist");
            in.push_back(nodes[size_t(src)]->output(size_t(index)));
        }
        auto it = makers().find(key);
        if (it == makers().end())
            throw std::runtime_error("B200 saved model: unknown op " + key);
        auto node = it->second(r, in);
        node->set_friendly_name(friendly);
        nodes.push_back(node);
    }
    ParameterVector params;
    for (uint64_t i = 0, n = r.u64(); i < n; ++i)
    {
        auto p = std::dynamic_pointer_cast<op::v0::Parameter>(nodes.at(size_t(r.u64())));
        if (!p)
            throw std::runtime_error("B200 saved model: parameter list names another op");
        params.push_back(p);
    }
    ResultVector results;
    for (uint64_t i = 0, n = r.u64(); i < n; ++i)
    {
        auto res = std::dynamic_pointer_cast<op::v0::Result>(nodes.at(size_t(r.u64())));
        if (!res)
            throw std::runtime_error("B200 saved model: result list names another op");
        results.push_back(res);
    }
    if (nodes_in_saved_order)
        *nodes_in_saved_order = nodes;
    return std::make_shared<Function>(results, params);
}

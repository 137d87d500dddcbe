// ng_capi: a small C facade over nGraph's C++ API so that the tests and the benchmark (Python,
// ctypes) can build nGraph Functions, create backends by name ("B200", "INTERPRETER") and run them
// exactly the way any nGraph client does: Backend::create -> compile -> create_tensor -> write ->
// call_with_validate -> read.  It contains no arithmetic of its own.
#include <dlfcn.h>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "ngraph/ngraph.hpp"
#include "ngraph/builder/quantized_concat_builder.hpp"
#include "ngraph/op/experimental/batch_mat_mul.hpp"
#include "ngraph/op/experimental/quantized_conv_bias.hpp"
#include "ngraph/op/gelu.hpp"
#include "ngraph/op/layer_norm.hpp"
#include "ngraph/op/experimental/quantized_conv_relu.hpp"
#include "ngraph/op/experimental/quantized_dot_bias.hpp"
#include "ngraph/runtime/backend.hpp"
#include "ngraph/runtime/backend_manager.hpp"
#include "../backend/function_io.hpp"
#include "../backend/batch_split.hpp"
#include "../backend/graph_passes.hpp"
#include <fstream>

using namespace ngraph;

#define NGC_API extern "C" __attribute__((visibility("default")))

namespace
{
    thread_local std::string g_error;

    const element::Type& et_of(int t)
    {
        switch (t)
        {
        case 0: return element::u8;
        case 1: return element::i8;
        case 2: return element::i32;
        case 3: return element::f32;
        case 4: return element::i64;
        default: throw std::runtime_error("ng_capi: bad element type code");
        }
    }

    Shape shape_of(const int64_t* s, int rank) { return Shape(s, s + rank); }

    using Val = Output<Node>;
    Val& val(void* p) { return *static_cast<Val*>(p); }
    void* box(const std::shared_ptr<Node>& n) { return new Val(n->output(0)); }

    struct Geom
    {
        Strides strides, dilation;
        CoordinateDiff below, above;
        Strides data_dilation;
    };
    Geom geom_of(const int64_t* g) // stride h,w, dilation h,w, below h,w, above h,w, data dilation h,w
    {
        return Geom{Strides{size_t(g[0]), size_t(g[1])}, Strides{size_t(g[2]), size_t(g[3])},
                    CoordinateDiff{g[4], g[5]}, CoordinateDiff{g[6], g[7]}, Strides{size_t(g[8]), size_t(g[9])}};
    }

    template <typename F>
    auto guarded(F f, decltype(f()) on_error) -> decltype(f())
    {
        try
        {
            return f();
        }
        catch (const std::exception& e)
        {
            g_error = e.what();
            return on_error;
        }
    }
}

NGC_API const char* ngc_last_error() { return g_error.c_str(); }

// dlopen a backend library and run its registration function (what BackendManager does for a
// library that sits next to libngraph.so; used here because the plugin lives in its own directory)
NGC_API int ngc_load_backend(const char* path, const char* register_symbol)
{
    return guarded([&]() -> int {
        void* h = dlopen(path, RTLD_NOW | RTLD_GLOBAL);
        if (!h) throw std::runtime_error(std::string("dlopen failed: ") + dlerror());
        auto fn = reinterpret_cast<void (*)()>(dlsym(h, register_symbol));
        if (!fn) throw std::runtime_error(std::string("symbol not found: ") + register_symbol);
        fn();
        return 0;
    }, -1);
}

NGC_API void* ngc_backend_create(const char* name)
{
    return guarded([&]() -> void* { return new std::shared_ptr<runtime::Backend>(runtime::Backend::create(name)); }, nullptr);
}
NGC_API void ngc_backend_free(void* b) { delete static_cast<std::shared_ptr<runtime::Backend>*>(b); }

NGC_API int ngc_registered_backends(char* buf, int n)
{
    std::string s;
    for (auto& d : runtime::BackendManager::get_registered_backends()) s += d + " ";
    strncpy(buf, s.c_str(), n - 1);
    buf[n - 1] = 0;
    return int(s.size());
}

// ------------------------------------------------------------------------------------ graph building
NGC_API void ngc_value_free(void* v) { delete static_cast<Val*>(v); }

NGC_API void* ngc_parameter(int et, const int64_t* shape, int rank)
{
    return guarded([&]() -> void* { return box(std::make_shared<op::v0::Parameter>(et_of(et), shape_of(shape, rank))); }, nullptr);
}

NGC_API void* ngc_constant(int et, const int64_t* shape, int rank, const void* data)
{
    return guarded([&]() -> void* { return box(std::make_shared<op::v0::Constant>(et_of(et), shape_of(shape, rank), data)); }, nullptr);
}

NGC_API void* ngc_quantize(void* x, void* scale, void* zp, int et, const int64_t* axes, int n_axes, int round_mode)
{
    return guarded([&]() -> void* {
        AxisSet ax;
        for (int i = 0; i < n_axes; ++i) ax.insert(size_t(axes[i]));
        return box(std::make_shared<op::v0::Quantize>(val(x), val(scale), val(zp), et_of(et), ax,
                                                      static_cast<op::v0::Quantize::RoundMode>(round_mode)));
    }, nullptr);
}

NGC_API void* ngc_dequantize(void* x, void* scale, void* zp, int et, const int64_t* axes, int n_axes)
{
    return guarded([&]() -> void* {
        AxisSet ax;
        for (int i = 0; i < n_axes; ++i) ax.insert(size_t(axes[i]));
        return box(std::make_shared<op::v0::Dequantize>(val(x), val(scale), val(zp), et_of(et), ax));
    }, nullptr);
}

NGC_API void* ngc_quantized_dot(void* a, void* b, void* sa, void* za, void* sb, void* zb, void* so, void* zo, int out_et)
{
    return guarded([&]() -> void* {
        return box(std::make_shared<op::v0::QuantizedDot>(val(a), val(b), 1, val(sa), val(za), val(sb), val(zb), val(so),
                                                          val(zo), et_of(out_et)));
    }, nullptr);
}

NGC_API void* ngc_quantized_dot_bias(void* x, void* w, void* bias, void* scale, int requantize, int relu)
{
    return guarded([&]() -> void* {
        return box(std::make_shared<op::v0::QuantizedDotBias>(val(x), val(w), val(bias), val(scale), requantize != 0, relu != 0));
    }, nullptr);
}

NGC_API void* ngc_quantized_conv(void* data, void* filt, const int64_t* g, void* si, void* zi, void* sf, void* zf, void* so,
                                 void* zo, int out_et)
{
    return guarded([&]() -> void* {
        Geom gg = geom_of(g);
        return box(std::make_shared<op::v0::QuantizedConvolution>(val(data), val(filt), gg.strides, gg.dilation, gg.below,
                                                                  gg.above, gg.data_dilation, val(si), val(zi), val(sf), val(zf),
                                                                  val(so), val(zo), et_of(out_et)));
    }, nullptr);
}

NGC_API void* ngc_quantized_conv_bias(void* data, void* filt, void* bias, const int64_t* g, void* scale, int relu)
{
    return guarded([&]() -> void* {
        Geom gg = geom_of(g);
        return box(std::make_shared<op::v0::QuantizedConvolutionBias>(val(data), val(filt), val(bias), gg.strides, gg.dilation,
                                                                      gg.below, gg.above, gg.data_dilation, val(scale), relu != 0));
    }, nullptr);
}

NGC_API void* ngc_quantized_conv_bias_add(void* data, void* filt, void* bias, void* sum, const int64_t* g, void* scale,
                                          void* sum_scale, int relu, int signed_add)
{
    return guarded([&]() -> void* {
        Geom gg = geom_of(g);
        if (signed_add)
            return box(std::make_shared<op::v0::QuantizedConvolutionBiasSignedAdd>(
                val(data), val(filt), val(bias), val(sum), gg.strides, gg.dilation, gg.below, gg.above, gg.data_dilation,
                val(scale), val(sum_scale), relu != 0));
        return box(std::make_shared<op::v0::QuantizedConvolutionBiasAdd>(val(data), val(filt), val(bias), val(sum), gg.strides,
                                                                         gg.dilation, gg.below, gg.above, gg.data_dilation,
                                                                         val(scale), val(sum_scale), relu != 0));
    }, nullptr);
}

NGC_API void* ngc_quantized_conv_relu(void* data, void* filt, const int64_t* g, void* scale)
{
    return guarded([&]() -> void* {
        Geom gg = geom_of(g);
        return box(std::make_shared<op::v0::QuantizedConvolutionRelu>(val(data), val(filt), gg.strides, gg.dilation, gg.below,
                                                                      gg.above, gg.data_dilation, val(scale)));
    }, nullptr);
}

NGC_API void* ngc_convolution(void* data, void* filt, const int64_t* g)
{
    return guarded([&]() -> void* {
        Geom gg = geom_of(g);
        return box(std::make_shared<op::v0::Convolution>(val(data), val(filt), gg.strides, gg.dilation, gg.below, gg.above,
                                                         gg.data_dilation));
    }, nullptr);
}

NGC_API void* ngc_max_pool(void* x, const int64_t* win, const int64_t* stride, const int64_t* below, const int64_t* above)
{
    return guarded([&]() -> void* {
        return box(std::make_shared<op::v0::MaxPool>(val(x), Shape{size_t(win[0]), size_t(win[1])},
                                                     Strides{size_t(stride[0]), size_t(stride[1])},
                                                     Shape{size_t(below[0]), size_t(below[1])},
                                                     Shape{size_t(above[0]), size_t(above[1])}));
    }, nullptr);
}

NGC_API void* ngc_avg_pool(void* x, const int64_t* win, const int64_t* stride)
{
    return guarded([&]() -> void* {
        return box(std::make_shared<op::v0::AvgPool>(val(x), Shape{size_t(win[0]), size_t(win[1])},
                                                     Strides{size_t(stride[0]), size_t(stride[1])}));
    }, nullptr);
}

// pooling with every attribute: padding below / above, ceil mode, and (AvgPool) whether padding counts in the divisor
NGC_API void* ngc_max_pool_ex(void* x, const int64_t* win, const int64_t* stride, const int64_t* below, const int64_t* above,
                              int ceil_mode)
{
    return guarded([&]() -> void* {
        return box(std::make_shared<op::v0::MaxPool>(val(x), Shape{size_t(win[0]), size_t(win[1])},
                                                     Strides{size_t(stride[0]), size_t(stride[1])},
                                                     Shape{size_t(below[0]), size_t(below[1])},
                                                     Shape{size_t(above[0]), size_t(above[1])}, op::PadType::EXPLICIT,
                                                     ceil_mode != 0));
    }, nullptr);
}

NGC_API void* ngc_avg_pool_ex(void* x, const int64_t* win, const int64_t* stride, const int64_t* below, const int64_t* above,
                              int include_padding, int ceil_mode)
{
    return guarded([&]() -> void* {
        return box(std::make_shared<op::v0::AvgPool>(val(x), Shape{size_t(win[0]), size_t(win[1])},
                                                     Strides{size_t(stride[0]), size_t(stride[1])},
                                                     Shape{size_t(below[0]), size_t(below[1])},
                                                     Shape{size_t(above[0]), size_t(above[1])}, include_padding != 0,
                                                     op::PadType::EXPLICIT, ceil_mode != 0));
    }, nullptr);
}

NGC_API void* ngc_concat(void** values, int n, int64_t axis)
{
    return guarded([&]() -> void* {
        OutputVector parts;
        for (int i = 0; i < n; ++i) parts.push_back(val(values[i]));
        return box(std::make_shared<op::v0::Concat>(parts, axis));
    }, nullptr);
}

// builder::QuantizedConcatBuilder (src/ngraph/builder/quantized_concat_builder.cpp): every operand is brought to the
// scale of the widest [min, max] range by a Dequantize / Quantize pair, then concatenated
NGC_API void* ngc_quantized_concat(void** values, void** mins, void** maxs, int n, int64_t axis)
{
    return guarded([&]() -> void* {
        OutputVector parts, lo, hi;
        for (int i = 0; i < n; ++i)
        {
            parts.push_back(val(values[i]));
            lo.push_back(val(mins[i]));
            hi.push_back(val(maxs[i]));
        }
        return box(builder::QuantizedConcatBuilder(parts, size_t(axis), lo, hi));
    }, nullptr);
}

// the float ops of quantized graphs' f32 islands (for the oracle pins; the encoder graph itself is built in bert_int8.cpp)
NGC_API void* ngc_sum(void* x, const int64_t* axes, int n_axes)
{
    return guarded([&]() -> void* {
        AxisSet ax;
        for (int i = 0; i < n_axes; ++i) ax.insert(size_t(axes[i]));
        return box(std::make_shared<op::v0::Sum>(val(x), ax));
    }, nullptr);
}

NGC_API void* ngc_softmax(void* x, const int64_t* axes, int n_axes)
{
    return guarded([&]() -> void* {
        AxisSet ax;
        for (int i = 0; i < n_axes; ++i) ax.insert(size_t(axes[i]));
        return box(std::make_shared<op::v0::Softmax>(val(x), ax));
    }, nullptr);
}

NGC_API void* ngc_layer_norm(void* x, void* scale, void* bias, int64_t begin_norm_axis, double epsilon)
{
    return guarded([&]() -> void* {
        return box(std::make_shared<op::v0::LayerNorm>(val(x), val(scale), val(bias), false, begin_norm_axis, epsilon));
    }, nullptr);
}

NGC_API void* ngc_gelu(void* x)
{
    return guarded([&]() -> void* { return box(std::make_shared<op::v0::Gelu>(val(x))); }, nullptr);
}

NGC_API void* ngc_batch_mat_mul(void* a, void* b)
{
    return guarded([&]() -> void* { return box(std::make_shared<op::v0::BatchMatMul>(val(a), val(b))); }, nullptr);
}

NGC_API void* ngc_convert(void* x, int et)
{
    return guarded([&]() -> void* { return box(std::make_shared<op::v0::Convert>(val(x), et_of(et))); }, nullptr);
}

NGC_API void* ngc_reshape(void* x, const int64_t* order, int n_order, const int64_t* shape, int rank)
{
    return guarded([&]() -> void* {
        AxisVector av(order, order + n_order);
        return box(std::make_shared<op::v0::Reshape>(val(x), av, shape_of(shape, rank)));
    }, nullptr);
}

// an op outside the quantized path (tests: it must be refused, not mis-handled)
NGC_API void* ngc_tanh(void* x)
{
    return guarded([&]() -> void* { return box(std::make_shared<op::v0::Tanh>(val(x))); }, nullptr);
}

NGC_API void* ngc_relu(void* x)
{
    return guarded([&]() -> void* { return box(std::make_shared<op::v0::Relu>(val(x))); }, nullptr);
}
NGC_API void* ngc_add(void* a, void* b)
{
    return guarded([&]() -> void* { return box(std::make_shared<op::v1::Add>(val(a), val(b))); }, nullptr);
}
NGC_API void* ngc_multiply(void* a, void* b)
{
    return guarded([&]() -> void* { return box(std::make_shared<op::v1::Multiply>(val(a), val(b))); }, nullptr);
}
NGC_API void* ngc_dot(void* a, void* b, int64_t reduction_axes)
{
    return guarded([&]() -> void* { return box(std::make_shared<op::v0::Dot>(val(a), val(b), size_t(reduction_axes))); }, nullptr);
}
NGC_API void* ngc_broadcast(void* x, const int64_t* shape, int rank, const int64_t* axes, int n_axes)
{
    return guarded([&]() -> void* {
        AxisSet ax;
        for (int i = 0; i < n_axes; ++i) ax.insert(size_t(axes[i]));
        return box(std::make_shared<op::v0::Broadcast>(val(x), shape_of(shape, rank), ax));
    }, nullptr);
}

NGC_API int ngc_value_shape(void* v, int64_t* shape, int max_rank, int* et)
{
    return guarded([&]() -> int {
        const Shape& s = val(v).get_shape();
        if (int(s.size()) > max_rank) throw std::runtime_error("rank too large");
        for (size_t i = 0; i < s.size(); ++i) shape[i] = int64_t(s[i]);
        const element::Type& t = val(v).get_element_type();
        *et = t == element::u8 ? 0 : t == element::i8 ? 1 : t == element::i32 ? 2 : t == element::f32 ? 3 : t == element::i64 ? 4 : -1;
        return int(s.size());
    }, -1);
}

NGC_API void* ngc_function(void** results, int n_results, void** params, int n_params)
{
    return guarded([&]() -> void* {
        OutputVector rs;
        for (int i = 0; i < n_results; ++i) rs.push_back(val(results[i]));
        ParameterVector ps;
        for (int i = 0; i < n_params; ++i)
        {
            auto p = as_type_ptr<op::v0::Parameter>(val(params[i]).get_node_shared_ptr());
            if (!p) throw std::runtime_error("ngc_function: not a Parameter");
            ps.push_back(p);
        }
        return new std::shared_ptr<Function>(std::make_shared<Function>(rs, ps));
    }, nullptr);
}
// A copy of the Function after the graph passes the B200 plugin runs in compile() (ngraph_b200/backend/graph_passes.cpp is
// compiled into this library as well: the plugin itself exports nothing but its registration symbol).
NGC_API void* ngc_function_after_b200_passes(void* function, int decompose_all)
{
    return guarded([&]() -> void* {
        auto copy = new std::shared_ptr<Function>(clone_function(**static_cast<std::shared_ptr<Function>*>(function)));
        try
        {
            runtime::b200::run_graph_passes(*copy, decompose_all != 0);
        }
        catch (...)
        {
            delete copy;
            throw;
        }
        return copy;
    }, nullptr);
}

// The batch split of the multi-device backend option (ngraph_b200/backend/batch_split.cpp, compiled into this library as well):
// a new Function for `rows` of the batch, from a copy of `function` after the plugin's passes; nullptr when the graph
// cannot be split (ngc_last_error() then says why).  split_flags receives one byte per Parameter, then one per Result.
// shapes_out receives rank + extents (8 slots) per Parameter, then per Result, of the split Function.
NGC_API void* ngc_function_split_batch(void* function, int64_t rows, unsigned char* split_flags, int64_t* shapes_out)
{
    return guarded([&]() -> void* {
        std::shared_ptr<Function> lowered = clone_function(**static_cast<std::shared_ptr<Function>*>(function));
        runtime::b200::run_graph_passes(lowered);
        runtime::b200::BatchSplit split;
        std::string why;
        if (!runtime::b200::split_batch(*lowered, size_t(rows), split, why))
            throw std::runtime_error("not split: " + why);
        size_t k = 0, slot = 0;
        auto put_shape = [&](const Shape& sh) {
            shapes_out[9 * slot] = int64_t(sh.size());
            for (size_t i = 0; i < sh.size() && i < 8; ++i)
                shapes_out[9 * slot + 1 + i] = int64_t(sh[i]);
            ++slot;
        };
        for (size_t i = 0; i < split.parameter_split.size(); ++i)
        {
            split_flags[k++] = split.parameter_split[i];
            put_shape(split.function->get_parameters()[i]->get_output_shape(0));
        }
        for (size_t i = 0; i < split.result_split.size(); ++i)
        {
            split_flags[k++] = split.result_split[i];
            put_shape(split.function->get_results()[i]->get_output_shape(0));
        }
        return new std::shared_ptr<Function>(split.function);
    }, nullptr);
}

NGC_API void ngc_function_free(void* f) { delete static_cast<std::shared_ptr<Function>*>(f); }

NGC_API int ngc_function_op_count(void* f)
{
    return guarded([&]() -> int { return int((*static_cast<std::shared_ptr<Function>*>(f))->get_ordered_ops().size()); }, -1);
}

// ------------------------------------------------------------------------------------ running
NGC_API void* ngc_compile(void* backend, void* function, int enable_performance_data)
{
    return guarded([&]() -> void* {
        auto& b = *static_cast<std::shared_ptr<runtime::Backend>*>(backend);
        auto& f = *static_cast<std::shared_ptr<Function>*>(function);
        return new std::shared_ptr<runtime::Executable>(b->compile(f, enable_performance_data != 0));
    }, nullptr);
}
// Executable::save to a file / Backend::load from a file (executable.hpp:76-78, backend.hpp:122-125)
NGC_API int ngc_executable_save(void* executable, const char* path)
{
    return guarded([&]() -> int {
        std::ofstream out(path, std::ios::binary);
        if (!out) throw std::runtime_error(std::string("cannot open ") + path);
        (*static_cast<std::shared_ptr<runtime::Executable>*>(executable))->save(out);
        out.flush();
        if (!out) throw std::runtime_error(std::string("write failed: ") + path);
        return 0;
    }, -1);
}
NGC_API void* ngc_backend_load(void* backend, const char* path)
{
    return guarded([&]() -> void* {
        std::ifstream in(path, std::ios::binary);
        if (!in) throw std::runtime_error(std::string("cannot open ") + path);
        auto exe = (*static_cast<std::shared_ptr<runtime::Backend>*>(backend))->load(in);
        if (!exe) throw std::runtime_error("Backend::load returned no executable");
        return new std::shared_ptr<runtime::Executable>(exe);
    }, nullptr);
}
// The plugin's binary Function form (ngraph_b200/backend/function_io.cpp, compiled into this library too): a copy of the
// Function after a write / read round trip, and the number of bytes written; no device needed.
NGC_API void* ngc_function_roundtrip(void* function, int64_t* bytes_out)
{
    return guarded([&]() -> void* {
        const std::string bytes = runtime::b200::write_function(**static_cast<std::shared_ptr<Function>*>(function));
        if (bytes_out) *bytes_out = int64_t(bytes.size());
        return new std::shared_ptr<Function>(runtime::b200::read_function(bytes));
    }, nullptr);
}

NGC_API void ngc_executable_free(void* e) { delete static_cast<std::shared_ptr<runtime::Executable>*>(e); }

NGC_API void* ngc_tensor_create(void* backend, int et, const int64_t* shape, int rank)
{
    return guarded([&]() -> void* {
        auto& b = *static_cast<std::shared_ptr<runtime::Backend>*>(backend);
        return new std::shared_ptr<runtime::Tensor>(b->create_tensor(et_of(et), shape_of(shape, rank)));
    }, nullptr);
}
NGC_API void* ngc_tensor_wrap(void* backend, int et, const int64_t* shape, int rank, void* memory)
{
    return guarded([&]() -> void* {
        auto& b = *static_cast<std::shared_ptr<runtime::Backend>*>(backend);
        return new std::shared_ptr<runtime::Tensor>(b->create_tensor(et_of(et), shape_of(shape, rank), memory));
    }, nullptr);
}
NGC_API void ngc_tensor_free(void* t) { delete static_cast<std::shared_ptr<runtime::Tensor>*>(t); }

NGC_API int ngc_tensor_write(void* t, const void* data, int64_t bytes)
{
    return guarded([&]() -> int { (*static_cast<std::shared_ptr<runtime::Tensor>*>(t))->write(data, size_t(bytes)); return 0; }, -1);
}
NGC_API int ngc_tensor_read(void* t, void* data, int64_t bytes)
{
    return guarded([&]() -> int { (*static_cast<std::shared_ptr<runtime::Tensor>*>(t))->read(data, size_t(bytes)); return 0; }, -1);
}

// Executable::create_input_tensor / create_output_tensor with a pipeline depth (src/ngraph/runtime/executable.hpp):
// `depth` tensors for parameter / result `index`, the double-buffering hook nbench's --double_buffer mode uses
NGC_API int ngc_executable_create_tensors(void* exe, int is_input, int index, int depth, void** out)
{
    return guarded([&]() -> int {
        auto& e = *static_cast<std::shared_ptr<runtime::Executable>*>(exe);
        auto v = is_input ? e->create_input_tensor(size_t(index), size_t(depth)) : e->create_output_tensor(size_t(index), size_t(depth));
        if (int(v.size()) != depth) throw std::runtime_error("create_*_tensor returned another pipeline depth");
        for (int i = 0; i < depth; ++i) out[i] = new std::shared_ptr<runtime::Tensor>(v[i]);
        return 0;
    }, -1);
}

NGC_API int ngc_call(void* exe, void** outs, int n_out, void** ins, int n_in, int validate)
{
    return guarded([&]() -> int {
        std::vector<std::shared_ptr<runtime::Tensor>> o, i;
        for (int k = 0; k < n_out; ++k) o.push_back(*static_cast<std::shared_ptr<runtime::Tensor>*>(outs[k]));
        for (int k = 0; k < n_in; ++k) i.push_back(*static_cast<std::shared_ptr<runtime::Tensor>*>(ins[k]));
        auto& e = *static_cast<std::shared_ptr<runtime::Executable>*>(exe);
        bool ok = validate ? e->call_with_validate(o, i) : e->call(o, i);
        return ok ? 0 : 1;
    }, -1);
}

// per-node performance counters: fills names (newline separated) and microseconds (total per node)
NGC_API int ngc_performance_data(void* exe, char* names, int names_bytes, int64_t* total_us, int64_t* calls, int max_nodes)
{
    return guarded([&]() -> int {
        auto& e = *static_cast<std::shared_ptr<runtime::Executable>*>(exe);
        auto data = e->get_performance_data();
        std::string s;
        int n = 0;
        for (auto& pc : data)
        {
            if (n >= max_nodes) break;
            s += pc.get_node()->description() + ":" + pc.get_node()->get_name() + "\n";
            total_us[n] = int64_t(pc.total_microseconds());
            calls[n] = int64_t(pc.call_count());
            ++n;
        }
        strncpy(names, s.c_str(), names_bytes - 1);
        names[names_bytes - 1] = 0;
        return n;
    }, -1);
}

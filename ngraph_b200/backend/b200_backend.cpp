// nGraph runtime backend "B200": see b200_backend.hpp.
//
// compile() turns the Function into a straight-line list of kernel launches ("steps") over device
// buffers ("slots"); call() binds the Parameter / Result tensors and enqueues the steps on the
// backend's stream.  There is no host fallback: an op the kernels cannot run makes compile() throw
// ngraph::unsupported_op, exactly like the other backends do for ops they lack.
//
// Data layout.  nGraph tensors are row-major (images NCHW, filters KCRS).  The int8 convolution
// kernels are channels-last, so every 4-D one-byte tensor may exist in two materialisations:
// canonical (what Parameters, Results and non-convolution ops see) and NHWC.  Convolutions, u8
// MaxPool and the pooling head consume and produce NHWC directly; a conversion kernel is emitted
// only where a consumer needs the other form, so activations stay channels-last between
// quantized layers and NCHW appears only at graph edges.  Constant filters are packed to KRSC
// once at compile time.
#include "b200_backend.hpp"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <sstream>

#include "b200_kernels.h"
#include "function_io.hpp"
#include "graph_passes.hpp"
#include "quant_fusion.hpp"
#include "ngraph/op/concat.hpp"
#include "ngraph/descriptor/layout/dense_tensor_layout.hpp"
#include "ngraph/except.hpp"
#include "ngraph/graph_util.hpp"
#include "ngraph/op/abs.hpp"
#include "ngraph/op/add.hpp"
#include "ngraph/op/avg_pool.hpp"
#include "ngraph/op/broadcast.hpp"
#include "ngraph/op/divide.hpp"
#include "ngraph/op/dot.hpp"
#include "ngraph/op/erf.hpp"
#include "ngraph/op/exp.hpp"
#include "ngraph/op/experimental/batch_mat_mul.hpp"
#include "ngraph/op/gather.hpp"
#include "ngraph/op/gelu.hpp"
#include "ngraph/op/layer_norm.hpp"
#include "ngraph/op/max.hpp"
#include "ngraph/op/min.hpp"
#include "ngraph/op/maximum.hpp"
#include "ngraph/op/minimum.hpp"
#include "ngraph/op/multiply.hpp"
#include "ngraph/op/negative.hpp"
#include "ngraph/op/relu.hpp"
#include "ngraph/op/softmax.hpp"
#include "ngraph/op/sqrt.hpp"
#include "ngraph/op/stop_gradient.hpp"
#include "ngraph/op/subtract.hpp"
#include "ngraph/op/sum.hpp"
#include "ngraph/op/constant.hpp"
#include "ngraph/op/convert.hpp"
#include "ngraph/op/dequantize.hpp"
#include "ngraph/op/experimental/quantized_conv_bias.hpp"
#include "ngraph/op/experimental/quantized_conv_relu.hpp"
#include "ngraph/op/experimental/quantized_dot_bias.hpp"
#include "ngraph/op/max_pool.hpp"
#include "ngraph/op/parameter.hpp"
#include "ngraph/op/quantize.hpp"
#include "ngraph/op/quantized_convolution.hpp"
#include "ngraph/op/quantized_dot.hpp"
#include "ngraph/op/reshape.hpp"
#include "ngraph/op/result.hpp"
#include "ngraph/pass/constant_folding.hpp"
#include "ngraph/pass/implicit_broadcast_elimination.hpp"
#include "ngraph/pass/fused_op_decomposition.hpp"
#include "ngraph/pass/like_replacement.hpp"
#include "ngraph/pass/manager.hpp"
#include "ngraph/runtime/backend_manager.hpp"
#include "ngraph/util.hpp"
#include "multi_device.hpp"
#include "ngraph/chrome_trace.hpp"
#include "ngraph/cpio.hpp"

using namespace ngraph;
using namespace ngraph::runtime::b200;

// ------------------------------------------------------------------------------------ helpers
namespace
{
    void cuda_check(cudaError_t e, const char* what)
    {
        if (e != cudaSuccess)
        {
            std::stringstream ss;
            ss << "B200 backend: " << what << ": " << cudaGetErrorString(e);
            throw std::runtime_error(ss.str());
        }
    }

    void kernel_check(int status, const std::string& what)
    {
        if (status != B200_OK)
        {
            std::stringstream ss;
            ss << "B200 backend: " << what << ": " << b200_status_string(status);
            if (status > 0)
                ss << " (" << b200_last_cuda_error() << ")";
            throw std::runtime_error(ss.str());
        }
    }

    [[noreturn]] void unsupported(const Node& node, const std::string& why)
    {
        std::stringstream ss;
        ss << "B200 backend: unsupported op " << node.description() << " (" << node.get_name() << "): " << why;
        throw unsupported_op(ss.str());
    }

    int dtype_of(const element::Type& et)
    {
        if (et == element::u8) return B200_U8;
        if (et == element::i8) return B200_I8;
        if (et == element::i32) return B200_I32;
        if (et == element::f32) return B200_F32;
        if (et == element::i64) return B200_I64;
        return -1;
    }

    size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

    std::shared_ptr<const op::v0::Constant> as_constant(const Output<Node>& out)
    {
        return as_type_ptr<op::v0::Constant>(out.get_node_shared_ptr());
    }

    template <typename N>
    size_t single_user_count(const Output<N>& out)
    {
        return out.get_target_inputs().size();
    }

    template <typename N>
    const Node* only_user(const Output<N>& out)
    {
        auto t = out.get_target_inputs();
        return t.size() == 1 ? t.begin()->get_node() : nullptr;
    }

    // Dequantize(u8, per-tensor, zero point 0) -> AvgPool(f32, window == whole image, no padding)
    // -> Quantize(u8, per-tensor, zero point 0, ROUND_NEAREST_TOWARD_EVEN): the pooling head of a
    // quantized network (src/ngraph/runtime/cpu/pass/cpu_fusion.cpp:2160-2200 starts from the same shape).
    struct AvgPoolHead
    {
        const op::v0::Dequantize* dq = nullptr;
        const op::v0::AvgPool* pool = nullptr;
        const op::v0::Quantize* q = nullptr;
    };

    bool constant_zero(const Output<Node>& out)
    {
        auto c = as_constant(out);
        if (!c)
            return false;
        size_t n = shape_size(c->get_output_shape(0)) * c->get_output_element_type(0).size();
        const char* p = static_cast<const char*>(c->get_data_ptr());
        for (size_t i = 0; i < n; ++i)
            if (p[i] != 0)
                return false;
        return true;
    }

    bool match_head(const Node* qn, AvgPoolHead& h)
    {
        auto q = as_type<const op::v0::Quantize>(qn);
        const auto one_byte = [](const element::Type& t) { return t == element::u8 || t == element::i8; };
        if (!q || !one_byte(q->get_output_element_type(0)) || !q->get_axes().empty() ||
            q->get_round_mode() != op::v0::Quantize::RoundMode::ROUND_NEAREST_TOWARD_EVEN ||
            !constant_zero(q->input_value(2)))
            return false;
        auto pool = as_type<const op::v0::AvgPool>(q->input_value(0).get_node());
        if (!pool || single_user_count(q->input_value(0)) != 1 || pool->get_output_element_type(0) != element::f32)
            return false;
        if (pool->get_input_shape(0).size() != 4)
            return false;
        auto dq = as_type<const op::v0::Dequantize>(pool->input_value(0).get_node());
        if (!dq || single_user_count(pool->input_value(0)) != 1 || !one_byte(dq->get_input_element_type(0)) ||
            !dq->get_axes().empty() || !constant_zero(dq->input_value(2)))
            return false;
        h.dq = dq;
        h.pool = pool;
        h.q = q;
        return true;
    }

    // the op's attributes and shapes as the kernels take them
    b200_pool_params pool_params_of(const op::v0::AvgPool& pool)
    {
        const Shape& in = pool.get_input_shape(0);
        const Shape& out = pool.get_output_shape(0);
        b200_pool_params g;
        g.N = int64_t(in[0]); g.C = int64_t(in[1]); g.H = int64_t(in[2]); g.W = int64_t(in[3]);
        g.P = int64_t(out[2]); g.Q = int64_t(out[3]);
        g.win_h = int64_t(pool.get_window_shape()[0]); g.win_w = int64_t(pool.get_window_shape()[1]);
        g.stride_h = int64_t(pool.get_window_movement_strides()[0]); g.stride_w = int64_t(pool.get_window_movement_strides()[1]);
        g.pad_h = int64_t(pool.get_padding_below()[0]); g.pad_w = int64_t(pool.get_padding_below()[1]);
        g.pad_h_above = int64_t(pool.get_padding_above()[0]); g.pad_w_above = int64_t(pool.get_padding_above()[1]);
        g.include_padding = pool.get_include_padding_in_avg_computation() ? 1 : 0;
        return g;
    }

    bool is_global_unpadded(const b200_pool_params& g)
    {
        return g.win_h == g.H && g.win_w == g.W && g.P == 1 && g.Q == 1 && g.pad_h == 0 && g.pad_w == 0 && g.pad_h_above == 0 &&
               g.pad_w_above == 0;
    }
}

// ------------------------------------------------------------------------------------ device context
DeviceContext::DeviceContext(int dev)
    : device(dev)
{
    int count = 0;
    cuda_check(cudaGetDeviceCount(&count), "cudaGetDeviceCount");
    if (dev < 0 || dev >= count)
        throw std::runtime_error("B200 backend: no CUDA device " + std::to_string(dev));
    cuda_check(cudaSetDevice(dev), "cudaSetDevice");
    cuda_check(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "cudaStreamCreate");
    cuda_check(cudaStreamCreateWithFlags(&copy_stream, cudaStreamNonBlocking), "cudaStreamCreate");
}

DeviceContext::DeviceContext(int dev, cudaStream_t external)
    : device(dev)
    , stream(external)
    , owns_stream(false)
{
    int count = 0;
    cuda_check(cudaGetDeviceCount(&count), "cudaGetDeviceCount");
    if (dev < 0 || dev >= count)
        throw std::runtime_error("B200 backend: no CUDA device " + std::to_string(dev));
    cuda_check(cudaSetDevice(dev), "cudaSetDevice");
    cuda_check(cudaStreamCreateWithFlags(&copy_stream, cudaStreamNonBlocking), "cudaStreamCreate");
}

DeviceContext::~DeviceContext()
{
    cudaSetDevice(device);
    if (copy_stream)
        cudaStreamDestroy(copy_stream);
    if (stream && owns_stream)
        cudaStreamDestroy(stream);
}

void DeviceContext::make_current() const
{
    cuda_check(cudaSetDevice(device), "cudaSetDevice");
}

void DeviceContext::synchronize() const
{
    cuda_check(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
}

// ------------------------------------------------------------------------------------ tensor
B200Tensor::B200Tensor(const std::shared_ptr<DeviceContext>& ctx,
                       const element::Type& type,
                       const Shape& shape,
                       void* device_pointer)
    : runtime::Tensor(std::make_shared<descriptor::Tensor>(type, shape, "external"))
    , m_ctx(ctx)
{
    m_descriptor->set_tensor_layout(std::make_shared<descriptor::layout::DenseTensorLayout>(*m_descriptor));
    m_bytes = shape_size(shape) * type.size();
    m_ctx->make_current();
    if (device_pointer)
    {
        cudaPointerAttributes attr;
        if (cudaPointerGetAttributes(&attr, device_pointer) != cudaSuccess ||
            (attr.type != cudaMemoryTypeDevice && attr.type != cudaMemoryTypeManaged))
        {
            cudaGetLastError();
            throw ngraph_error("The pointer passed to B200Tensor is not a device pointer.");
        }
        m_ptr = device_pointer;
    }
    else
    {
        cuda_check(cudaMalloc(&m_ptr, m_bytes ? m_bytes : 16), "cudaMalloc(tensor)");
        m_owned = true;
    }
}

B200Tensor::~B200Tensor()
{
    cudaSetDevice(m_ctx->device);
    if (m_last_use)
    {
        cudaEventSynchronize(m_last_use); // no kernel may still be using the memory when it is released
        cudaEventDestroy(m_last_use);
    }
    if (m_owned && m_ptr)
        cudaFree(m_ptr);
}

void B200Tensor::mark_used(cudaStream_t compute_stream)
{
    if (!m_last_use)
        cuda_check(cudaEventCreateWithFlags(&m_last_use, cudaEventDisableTiming), "cudaEventCreate");
    cuda_check(cudaEventRecord(m_last_use, compute_stream), "cudaEventRecord");
}

void B200Tensor::order_copy_after_use() const
{
    // A tensor no call() has used yet may still be the target of work the client enqueued on an external compute
    // stream (a device pointer wrapped with create_tensor): order after everything on that stream, once.
    if (m_last_use)
        cuda_check(cudaStreamWaitEvent(m_ctx->copy_stream, m_last_use, 0), "cudaStreamWaitEvent");
    else
        cuda_check(cudaStreamSynchronize(m_ctx->stream), "cudaStreamSynchronize");
}

void B200Tensor::write(const void* p, size_t n)
{
    if (n > m_bytes)
        throw std::out_of_range("B200Tensor::write: access past the end of the tensor");
    m_ctx->make_current();
    order_copy_after_use();
    cuda_check(cudaMemcpyAsync(m_ptr, p, n, cudaMemcpyHostToDevice, m_ctx->copy_stream), "cudaMemcpy H2D");
    // the caller may release p as soon as write() returns, and a later call() sees the data
    cuda_check(cudaStreamSynchronize(m_ctx->copy_stream), "cudaStreamSynchronize");
}

void B200Tensor::read(void* p, size_t n) const
{
    if (n > m_bytes)
        throw std::out_of_range("B200Tensor::read: access past the end of the tensor");
    m_ctx->make_current();
    order_copy_after_use(); // the call() that produced this tensor has completed when the copy starts
    cuda_check(cudaMemcpyAsync(p, m_ptr, n, cudaMemcpyDeviceToHost, m_ctx->copy_stream), "cudaMemcpy D2H");
    cuda_check(cudaStreamSynchronize(m_ctx->copy_stream), "cudaStreamSynchronize");
    int code = 0;
    if (b200_device_status(&code) != B200_OK)
        throw std::runtime_error("B200 backend: a kernel gave up on a bounded wait (device status " +
                                 std::to_string(code) + ")");
}

void B200Tensor::write_async(const void* p, size_t offset, size_t n)
{
    if (offset > m_bytes || n > m_bytes - offset)
        throw std::out_of_range("B200Tensor::write: access past the end of the tensor");
    m_ctx->make_current();
    order_copy_after_use();
    cuda_check(cudaMemcpyAsync(static_cast<char*>(m_ptr) + offset, p, n, cudaMemcpyHostToDevice, m_ctx->copy_stream), "cudaMemcpy H2D");
}

void B200Tensor::read_async(void* p, size_t offset, size_t n) const
{
    if (offset > m_bytes || n > m_bytes - offset)
        throw std::out_of_range("B200Tensor::read: access past the end of the tensor");
    m_ctx->make_current();
    order_copy_after_use();
    cuda_check(cudaMemcpyAsync(p, static_cast<const char*>(m_ptr) + offset, n, cudaMemcpyDeviceToHost, m_ctx->copy_stream), "cudaMemcpy D2H");
}

void B200Tensor::finish_copies() const
{
    m_ctx->make_current();
    cuda_check(cudaStreamSynchronize(m_ctx->copy_stream), "cudaStreamSynchronize");
    int code = 0;
    if (b200_device_status(&code) != B200_OK)
        throw std::runtime_error("B200 backend: a kernel gave up on a bounded wait (device status " + std::to_string(code) + ")");
}

void B200Tensor::order_copies_after(cudaEvent_t event) const
{
    m_ctx->make_current();
    cuda_check(cudaStreamWaitEvent(m_ctx->copy_stream, event, 0), "cudaStreamWaitEvent");
}

void B200Tensor::copy_from(const runtime::Tensor& source)
{
    auto src = dynamic_cast<const B200Tensor*>(&source);
    if (!src || src->m_ctx->device != m_ctx->device)
    {
        std::vector<char> tmp(source.get_size_in_bytes());
        source.read(tmp.data(), tmp.size());
        write(tmp.data(), tmp.size());
        return;
    }
    if (src->m_bytes != m_bytes)
        throw std::runtime_error("B200Tensor::copy_from: size mismatch");
    m_ctx->make_current();
    cuda_check(cudaMemcpyAsync(m_ptr, src->m_ptr, m_bytes, cudaMemcpyDeviceToDevice, m_ctx->stream), "cudaMemcpy D2D");
    mark_used(m_ctx->stream);
}

// ------------------------------------------------------------------------------------ backend
B200Backend::B200Backend(const std::string& options)
{
    // "<device ordinal>[,stream=<cudaStream_t as an integer>]": with stream= the backend enqueues on the
    // caller's stream (and never destroys it) instead of creating its own
    int dev = 0;
    unsigned long long stream = 0;
    bool have_stream = false;
    std::stringstream ss(options);
    std::string item;
    bool first = true;
    while (std::getline(ss, item, ','))
    {
        try
        {
            if (item.rfind("stream=", 0) == 0)
            {
                stream = std::stoull(item.substr(7), nullptr, 0);
                have_stream = true;
            }
            else if (first && !item.empty())
                dev = std::stoi(item);
            else if (!item.empty())
                throw std::invalid_argument(item);
        }
        catch (...)
        {
            throw std::runtime_error("B200 backend: bad option '" + item + "' (expected '<device>[,stream=<handle>]')");
        }
        first = false;
    }
    m_ctx = have_stream ? std::make_shared<DeviceContext>(dev, reinterpret_cast<cudaStream_t>(stream))
                        : std::make_shared<DeviceContext>(dev);
}

std::shared_ptr<runtime::Tensor> B200Backend::create_tensor()
{
    throw std::runtime_error("B200 backend does not support dynamic tensors");
}

std::shared_ptr<runtime::Tensor> B200Backend::create_tensor(const element::Type& type, const Shape& shape)
{
    return std::make_shared<B200Tensor>(m_ctx, type, shape);
}

std::shared_ptr<runtime::Tensor>
    B200Backend::create_tensor(const element::Type& type, const Shape& shape, void* memory_pointer)
{
    return std::make_shared<B200Tensor>(m_ctx, type, shape, memory_pointer);
}

std::shared_ptr<runtime::Executable> B200Backend::compile(std::shared_ptr<Function> func, bool enable_performance_data)
{
    std::lock_guard<std::mutex> lock(m_mutex);
    const auto key = std::make_pair(func, enable_performance_data);
    auto it = m_cache.find(key);
    if (it != m_cache.end())
        return it->second;
    auto exec = std::make_shared<B200Executable>(m_ctx, func, enable_performance_data);
    m_cache.insert({key, exec});
    return exec;
}

void B200Backend::remove_compiled_function(std::shared_ptr<runtime::Executable> exec)
{
    std::lock_guard<std::mutex> lock(m_mutex);
    for (auto it = m_cache.begin(); it != m_cache.end(); ++it)
        if (it->second == exec)
        {
            m_cache.erase(it);
            break;
        }
}

bool B200Backend::is_device_memory(void* ptr)
{
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess)
    {
        cudaGetLastError();
        return false;
    }
    return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}


bool B200Backend::is_supported(const Node& node) const
{
    // the op set of the quantized-inference path; shapes/types are checked at compile()
    return is_type<op::v0::Parameter>(&node) || is_type<op::v0::Constant>(&node) || is_type<op::v0::Result>(&node) ||
           is_type<op::v0::Quantize>(&node) || is_type<op::v0::Dequantize>(&node) ||
           is_type<op::v0::QuantizedDot>(&node) || is_type<op::v0::QuantizedDotBias>(&node) ||
           is_type<op::v0::QuantizedConvolution>(&node) || is_type<op::v0::QuantizedConvolutionBias>(&node) ||
           is_type<op::v0::QuantizedConvolutionBiasAdd>(&node) ||
           is_type<op::v0::QuantizedConvolutionBiasSignedAdd>(&node) ||
           is_type<op::v0::QuantizedConvolutionRelu>(&node) || is_type<op::v0::MaxPool>(&node) ||
           is_type<op::v0::AvgPool>(&node) || is_type<op::v0::Reshape>(&node) || is_type<op::v0::Convert>(&node) ||
           // f32 glue
           is_type<op::v1::Add>(&node) || is_type<op::v1::Subtract>(&node) || is_type<op::v1::Multiply>(&node) ||
           is_type<op::v1::Divide>(&node) || is_type<op::v1::Maximum>(&node) || is_type<op::v1::Minimum>(&node) ||
           is_type<op::v0::Abs>(&node) || is_type<op::v0::Negative>(&node) || is_type<op::v0::Sqrt>(&node) ||
           is_type<op::v0::Exp>(&node) || is_type<op::v0::Erf>(&node) || is_type<op::v0::Relu>(&node) ||
           is_type<op::v0::Broadcast>(&node) || is_type<op::v0::Sum>(&node) || is_type<op::v0::Max>(&node) || is_type<op::v0::Min>(&node) ||
           is_type<op::v0::Softmax>(&node) || is_type<op::v0::BatchMatMul>(&node) || is_type<op::v0::Dot>(&node) ||
           is_type<op::v0::Gather>(&node) || is_type<op::v0::Concat>(&node) || runs_undecomposed(node);
}

extern "C" B200_BACKEND_API void ngraph_register_b200_backend()
{
    // "B200" / "B200:<device>[,stream=...]": one device; "B200:all" / "B200:0+1+...": several devices behind one Backend
    runtime::BackendManager::register_backend("B200", [](const std::string& config) -> std::shared_ptr<runtime::Backend> {
        if (ShardedBackend::wants(config))
            return std::make_shared<ShardedBackend>(config);
        return std::make_shared<B200Backend>(config);
    });
}

// ------------------------------------------------------------------------------------ executable: compile
int B200Executable::new_slot(Slot::Kind kind, size_t bytes, size_t index)
{
    Slot s;
    s.kind = kind;
    s.bytes = bytes;
    s.index = index;
    if (kind == Slot::ARENA)
    {
        // provisional: one region per slot; plan_arena() overlays slots whose lifetimes do not meet
        s.offset = m_arena_bytes;
        m_arena_bytes += align_up(bytes ? bytes : 16, 256);
    }
    m_slots.push_back(s);
    const int id = int(m_slots.size()) - 1;
    m_birth.push_back(m_steps.size()); // the next step to be emitted is the first that can write it
    m_last.push_back(m_steps.size());
    m_touched.push_back(id);
    return id;
}

// `key` names the constant inside the image: what it is and the position, in the Function's node order, of the Constant(s)
// it was made from.  A saved executable's image is looked up by the same keys, so the loading side does not depend on
// the order in which the lowering asks for its constants.
std::string B200Executable::constant_key(const char* purpose, std::initializer_list<const Node*> sources) const
{
    std::string key = purpose;
    for (const Node* n : sources)
    {
        auto it = m_node_index.find(n);
        key += ":" + (it == m_node_index.end() ? std::string("?") : std::to_string(it->second));
    }
    return key;
}

bool B200Executable::have_saved_constant(const std::string& key) const { return m_use_preloaded && m_constant_index.count(key) != 0; }

int B200Executable::upload_constant(const std::string& key, const void* data, size_t bytes)
{
    Slot s;
    s.kind = Slot::CONSTANT;
    s.bytes = bytes;
    if (m_use_preloaded)
    {
        // the image of a saved executable already holds this constant
        auto it = m_constant_index.find(key);
        if (it == m_constant_index.end() || it->second.second != bytes || it->second.first + bytes > m_preloaded.size())
            throw std::runtime_error("B200 backend: the saved constant image does not belong to the saved model (" + key + ")");
        s.offset = it->second.first;
    }
    else
    {
        s.offset = align_up(m_constant_host.size(), 256);
        m_constant_host.resize(s.offset + align_up(bytes ? bytes : 16, 256), 0);
        if (bytes)
            memcpy(m_constant_host.data() + s.offset, data, bytes);
        m_constant_index.emplace(key, std::make_pair(s.offset, bytes)); // a repeated key keeps its first (identical) copy
    }
    m_slots.push_back(s);
    m_birth.push_back(0); // lifetimes are kept per slot index; constants live forever
    m_last.push_back(size_t(-1));
    return int(m_slots.size()) - 1;
}

B200Executable::Value& B200Executable::value_of(const Output<Node>& out)
{
    auto it = m_values.find(&out.get_tensor());
    if (it == m_values.end())
        throw std::runtime_error("B200 backend: value used before it was produced: " + out.get_node()->get_name());
    return it->second;
}

void B200Executable::emit(const std::shared_ptr<const Node>& node, const std::string& what,
                          std::function<int(const Ptrs&, cudaStream_t)> run)
{
    m_steps.push_back(Step{node, what, std::move(run)});
}

int B200Executable::canonical_slot(const Output<Node>& out)
{
    Value& v = value_of(out);
    if (v.skipped)
        throw std::runtime_error("B200 backend: internal error, fused value requested: " + out.get_node()->get_name());
    if (v.canonical >= 0)
    {
        m_touched.push_back(v.canonical);
        return v.canonical;
    }
    if (v.nhwc < 0)
        throw std::runtime_error("B200 backend: internal error, value has no materialisation");
    m_touched.push_back(v.nhwc);
    // channels-last -> NCHW
    const Shape sh = v.shape;
    if (sh.size() == 4 && (sh[1] == 1 || sh[2] * sh[3] == 1))
    {
        v.canonical = v.nhwc; // one channel or one pixel per image: both orders are the same bytes
        return v.canonical;
    }
    int dst = new_slot(Slot::ARENA, shape_size(sh) * v.et.size());
    int src = v.nhwc;
    emit(out.get_node_shared_ptr(), "nhwc_to_nchw", [=](const Ptrs& p, cudaStream_t st) {
        return b200_nhwc_to_nchw_u8(p[src], p[dst], sh[0], sh[1], sh[2], sh[3], sh[1], st);
    });
    v.canonical = dst;
    return dst;
}

int B200Executable::nhwc_slot(const Output<Node>& out)
{
    Value& v = value_of(out);
    if (v.nhwc >= 0)
    {
        m_touched.push_back(v.nhwc);
        return v.nhwc;
    }
    if (v.shape.size() != 4 || v.et.size() != 1)
        throw std::runtime_error("B200 backend: channels-last form exists for 4-D one-byte tensors only");
    const Shape sh = v.shape;
    int src = canonical_slot(out);
    if (sh[1] == 1 || sh[2] * sh[3] == 1)
    {
        value_of(out).nhwc = src; // the same bytes in both orders
        return src;
    }
    int dst = new_slot(Slot::ARENA, shape_size(sh));
    emit(out.get_node_shared_ptr(), "nchw_to_nhwc", [=](const Ptrs& p, cudaStream_t st) {
        return b200_nchw_to_nhwc_u8(p[src], p[dst], sh[0], sh[1], sh[2], sh[3], sh[1], st);
    });
    value_of(out).nhwc = dst;
    return dst;
}

// KCRS i8 filters -> KRSC (channels padded to c_pad) in device memory
int B200Executable::packed_filters(const Output<Node>& filters, size_t c_pad, bool* is_image)
{
    const Shape& fs = filters.get_shape();
    auto c = as_constant(filters);
    const std::string key = c ? constant_key(("filter_image/" + std::to_string(c_pad)).c_str(), {c.get()}) : std::string();
    if (c && have_saved_constant(key))
    {
        const int64_t kg = int64_t(fs[2] * fs[3] * c_pad), bk = b200_qconv_weight_block(int64_t(c_pad));
        if (is_image)
            *is_image = true;
        return upload_constant(key, nullptr, size_t(b200_packed_weights_bytes(int64_t(fs[0]), kg, bk)));
    }
    if (c)
    {
        const int8_t* src = static_cast<const int8_t*>(c->get_data_ptr());
        size_t K = fs[0], C = fs[1], R = fs[2], S = fs[3];
        std::vector<int8_t> packed(K * R * S * c_pad, 0);
        for (size_t k = 0; k < K; ++k)
            for (size_t ch = 0; ch < C; ++ch)
                for (size_t r = 0; r < R; ++r)
                    for (size_t s = 0; s < S; ++s)
                        packed[((k * R + r) * S + s) * c_pad + ch] = src[((k * C + ch) * R + r) * S + s];
        // constant filters go to the device in the tensor cores' shared-memory image (one bulk copy per tile and k-block)
        const int64_t kg = int64_t(R * S * c_pad), bk = b200_qconv_weight_block(int64_t(c_pad));
        std::vector<int8_t> image(size_t(b200_packed_weights_bytes(int64_t(K), kg, bk)));
        kernel_check(b200_pack_weights_host(packed.data(), image.data(), int64_t(K), kg, bk), "b200_pack_weights_host");
        if (is_image)
            *is_image = true;
        return upload_constant(key, image.data(), image.size());
    }
    if (is_image)
        *is_image = false;
    if (c_pad != fs[1])
        throw std::runtime_error("B200 backend: run-time filters need a channel count the kernels take directly");
    return nhwc_slot(filters);
}

// scale = a * b / c in fp32, left to right (runtime/reference/dot.hpp:154)
int B200Executable::scalar_product_scale(const Output<Node>& a, const Output<Node>& b, const Output<Node>& c)
{
    auto ca = as_constant(a), cb = as_constant(b), cc = as_constant(c);
    if (ca && cb && cc)
    {
        volatile float s = *static_cast<const float*>(ca->get_data_ptr()) * *static_cast<const float*>(cb->get_data_ptr());
        volatile float r = s / *static_cast<const float*>(cc->get_data_ptr());
        float v = r;
        return upload_constant(constant_key("requant_scale", {ca.get(), cb.get(), cc.get()}), &v, sizeof(float));
    }
    int sa = canonical_slot(a), sb = canonical_slot(b), sc = canonical_slot(c);
    int dst = new_slot(Slot::ARENA, sizeof(float));
    emit(a.get_node_shared_ptr(), "requant_scale", [=](const Ptrs& p, cudaStream_t st) {
        return b200_requant_scale(static_cast<const float*>(p[sa]), static_cast<const float*>(p[sb]),
                                  static_cast<const float*>(p[sc]), static_cast<float*>(p[dst]), st);
    });
    return dst;
}

bool B200Executable::avgpool_head_member(const Node* node)
{
    AvgPoolHead h;
    if (auto dq = as_type<const op::v0::Dequantize>(node))
    {
        const Node* pool = only_user(dq->output(0));
        const Node* q = pool ? only_user(pool->output(0)) : nullptr;
        return q && match_head(q, h) && h.dq == dq;
    }
    if (auto pool = as_type<const op::v0::AvgPool>(node))
    {
        const Node* q = only_user(pool->output(0));
        return q && match_head(q, h) && h.pool == pool;
    }
    return false;
}

B200Executable::B200Executable(const std::shared_ptr<DeviceContext>& ctx,
                               const std::shared_ptr<Function>& func,
                               bool enable_performance_data,
                               std::vector<char>* saved_constants,
                               const std::map<std::string, std::pair<size_t, size_t>>* saved_index,
                               const std::vector<std::shared_ptr<Node>>* saved_order)
    : m_ctx(ctx)
    , m_perf(enable_performance_data)
{
    m_ctx->make_current();
    if (saved_constants)
    {
        // Backend::load: `func` is the graph a previous compile() arrived at after its passes, and the constant image is the
        // one that compile() built (filters reordered and packed, weights transposed, scales folded): neither is redone
        m_function = func;
        m_preloaded.swap(*saved_constants);
        m_use_preloaded = true;
        if (saved_index)
            m_constant_index = *saved_index;
    }
    else
    {
        m_function = clone_function(*func); // never mutate the caller's graph
        run_graph_passes(m_function);
    }

    if (saved_order)
    {
        // Backend::load: the positions the saved constant keys count in are those of the saved node order
        for (size_t position = 0; position < saved_order->size(); ++position)
            m_node_index[(*saved_order)[position].get()] = position;
    }
    else
    {
        size_t position = 0;
        for (auto& node : m_function->get_ordered_ops())
            m_node_index[node.get()] = position++;
    }
    size_t pi = 0;
    for (auto& param : m_function->get_parameters())
    {
        Value v;
        v.et = param->get_output_element_type(0);
        v.shape = param->get_output_shape(0);
        v.canonical = new_slot(Slot::PARAMETER, shape_size(v.shape) * v.et.size(), pi++);
        m_values[&param->output(0).get_tensor()] = v;
    }
    for (auto& node : m_function->get_ordered_ops())
        compile_node(node);

    // results: produce the canonical form, then copy into the caller's tensor
    size_t ri = 0;
    for (auto& result : m_function->get_results())
    {
        Output<Node> src = result->input_value(0);
        int from = canonical_slot(src);
        Value& v = value_of(src);
        int to = new_slot(Slot::RESULT, shape_size(v.shape) * v.et.size(), ri++);
        m_result_copies.push_back({from, to});
        m_last[from] = size_t(-1); // read by the copy into the caller's tensor after the last step
    }
    // conversions emitted for the results read their sources at those (late) steps
    {
        const size_t last = m_steps.empty() ? 0 : m_steps.size() - 1;
        for (int slot : m_touched)
            m_last[slot] = std::max(m_last[slot], last);
        m_touched.clear();
    }
    plan_arena();

    if (m_arena_bytes)
        cuda_check(cudaMalloc(&m_arena, m_arena_bytes), "cudaMalloc(arena)");
    if (m_use_preloaded)
        m_constant_host.swap(m_preloaded);
    m_constant_bytes = m_constant_host.size();
    if (!m_constant_host.empty())
    {
        cuda_check(cudaMalloc(&m_constants, m_constant_host.size()), "cudaMalloc(constants)");
        cuda_check(cudaMemcpy(m_constants, m_constant_host.data(), m_constant_host.size(), cudaMemcpyHostToDevice),
                   "cudaMemcpy(constants)");
        std::vector<char>().swap(m_constant_host);
    }
    if (m_perf)
    {
        m_events.resize(2 * m_steps.size());
        for (auto& e : m_events)
            cuda_check(cudaEventCreate(&e), "cudaEventCreate");
        m_step_us.assign(m_steps.size(), 0.0);
    }
    set_parameters_and_results(*func);
}

B200Executable::~B200Executable()
{
    cudaSetDevice(m_ctx->device);
    cudaStreamSynchronize(m_ctx->stream);
    for (auto& e : m_events)
        cudaEventDestroy(e);
    if (m_arena) cudaFree(m_arena);
    if (m_constants) cudaFree(m_constants);
}

// Every slot a node's lowering asked for (or created) stays alive at least until the last step emitted for that node.
void B200Executable::compile_node(const std::shared_ptr<Node>& node)
{
    m_touched.clear();
    lower_node(node);
    const size_t last = m_steps.empty() ? 0 : m_steps.size() - 1;
    if (m_last.size() != m_slots.size() || m_birth.size() != m_slots.size())
        throw std::runtime_error("B200 backend: internal error, slot lifetimes out of step with the slot table");
    for (int slot : m_touched)
        m_last.at(size_t(slot)) = std::max(m_last.at(size_t(slot)), last);
    m_touched.clear();
}

// Arena layout from the lifetimes: slots in order of first write; a slot takes the lowest gap that fits among the slots
// still alive (first fit).  A slot is released only by a step AFTER its last reader, never by that step itself, so no
// kernel ever reads and writes the same region; kernels run in stream order (a programmatic dependent launch touches
// global memory only after the previous kernel has completed).
void B200Executable::plan_arena()
{
    struct Live { size_t offset, bytes, last; };
    std::vector<Live> live;
    size_t peak = 0;
    for (size_t i = 0; i < m_slots.size(); ++i)
    {
        Slot& s = m_slots[i];
        if (s.kind != Slot::ARENA)
            continue;
        const size_t bytes = align_up(s.bytes ? s.bytes : 16, 256);
        std::vector<Live> keep;
        for (auto& l : live)
            if (l.last >= m_birth[i])
                keep.push_back(l);
        live.swap(keep);
        std::sort(live.begin(), live.end(), [](const Live& a, const Live& b) { return a.offset < b.offset; });
        size_t at = 0;
        for (auto& l : live)
        {
            if (at + bytes <= l.offset)
                break;
            at = std::max(at, l.offset + l.bytes);
        }
        s.offset = at;
        live.push_back(Live{at, bytes, m_last[i]});
        peak = std::max(peak, at + bytes);
    }
    m_arena_bytes = peak;
}

void B200Executable::lower_node(const std::shared_ptr<Node>& node)
{
    if (is_type<op::v0::Parameter>(node) || is_type<op::v0::Result>(node))
        return;
    if (auto c = as_type_ptr<op::v0::Constant>(node))
    {
        Value v;
        v.et = c->get_output_element_type(0);
        v.shape = c->get_output_shape(0);
        v.constant = c;
        if (dtype_of(v.et) >= 0) // other element types can only feed ConstantFolding, never a kernel
            v.canonical = upload_constant(constant_key("plain", {c.get()}), c->get_data_ptr(), shape_size(v.shape) * v.et.size());
        m_values[&node->output(0).get_tensor()] = v;
        return;
    }
    Value out;
    out.et = node->get_output_element_type(0);
    out.shape = node->get_output_shape(0);
    if (node->get_output_size() != 1)
        unsupported(*node, "multiple outputs");
    m_values[&node->output(0).get_tensor()] = out;

    if (is_type<op::v0::Quantize>(node)) return compile_quantize(node);
    if (is_type<op::v0::Dequantize>(node)) return compile_dequantize(node);
    if (is_type<op::v0::QuantizedConvolutionBias>(node) || is_type<op::v0::QuantizedConvolutionBiasAdd>(node) ||
        is_type<op::v0::QuantizedConvolutionBiasSignedAdd>(node) || is_type<op::v0::QuantizedConvolutionRelu>(node))
        return compile_fused_conv(node);
    if (is_type<op::v0::QuantizedConvolution>(node)) return compile_core_conv(node);
    if (is_type<op::v0::QuantizedDotBias>(node)) return compile_dot_bias(node);
    if (is_type<op::v0::QuantizedDot>(node)) return compile_core_dot(node);
    if (is_type<op::v0::MaxPool>(node)) return compile_max_pool(node);
    if (is_type<op::v0::AvgPool>(node))
    {
        if (avgpool_head_member(node.get()))
        {
            value_of(node->output(0)).skipped = true;
            return;
        }
        return compile_avg_pool(node);
    }
    if (auto rs = as_type_ptr<op::v0::Reshape>(node))
    {
        Value& in = value_of(node->input_value(0));
        Value& o = value_of(node->output(0));
        if (!rs->get_is_transpose())
        {
            o.canonical = canonical_slot(node->input_value(0)); // same bytes, new shape
            return;
        }
        if (in.shape.size() == 2 && in.et.size() == 1)
        {
            int src = canonical_slot(node->input_value(0));
            int dst = new_slot(Slot::ARENA, shape_size(in.shape));
            int64_t r = in.shape[0], c = in.shape[1];
            emit(node, "transpose", [=](const Ptrs& p, cudaStream_t st) { return b200_transpose_u8(p[src], p[dst], r, c, st); });
            o.canonical = dst;
            return;
        }
        if (in.et.size() == 4 && in.shape.size() <= 8)
        {
            int src = canonical_slot(node->input_value(0));
            int dst = new_slot(Slot::ARENA, shape_size(in.shape) * 4);
            std::vector<int64_t> shape(in.shape.begin(), in.shape.end());
            std::vector<int64_t> order(rs->get_input_order().begin(), rs->get_input_order().end());
            emit(node, "permute", [=](const Ptrs& p, cudaStream_t st) {
                return b200_permute_b32(p[src], p[dst], shape.data(), int(shape.size()), order.data(), st);
            });
            o.canonical = dst;
            return;
        }
        unsupported(*node, "transposing Reshape other than a 2-D one-byte matrix or a 4-byte tensor");
    }
    if (auto cv = as_type_ptr<op::v0::Convert>(node))
    {
        const element::Type& from = node->get_input_element_type(0);
        const element::Type& to = node->get_output_element_type(0);
        if (from.size() == 1 && to.size() == 1 && from.is_integral() && to.is_integral())
        {
            // i8 <-> u8 static_cast keeps the byte: alias both materialisations
            Value in = value_of(node->input_value(0));
            Value& o = value_of(node->output(0));
            o.canonical = in.canonical;
            o.nhwc = in.nhwc;
            if (o.canonical < 0 && o.nhwc < 0)
                o.canonical = canonical_slot(node->input_value(0));
            return;
        }
        unsupported(*node, "Convert other than between i8 and u8");
    }
    if (auto cc = as_type_ptr<op::v0::Concat>(node))
    {
        // runtime/reference/concat.hpp on the row-major forms: each operand is a band of every output row
        const Shape& os = node->get_output_shape(0);
        const size_t axis = size_t(cc->get_concatenation_axis()), esz = node->get_output_element_type(0).size();
        int64_t rows = 1, tail = 1;
        for (size_t i = 0; i < axis; ++i) rows *= int64_t(os[i]);
        for (size_t i = axis + 1; i < os.size(); ++i) tail *= int64_t(os[i]);
        const int64_t pitch = int64_t(os[axis]) * tail * int64_t(esz);
        std::vector<int> sources;
        for (size_t i = 0; i < node->get_input_size(); ++i)
            sources.push_back(canonical_slot(node->input_value(i)));
        const int y = new_slot(Slot::ARENA, shape_size(os) * esz);
        int64_t offset = 0;
        for (size_t i = 0; i < sources.size(); ++i)
        {
            const int64_t band = int64_t(node->get_input_shape(i)[axis]) * tail * int64_t(esz);
            const int x = sources[i];
            emit(node, "concat", [=](const Ptrs& p, cudaStream_t st) {
                return b200_copy_rows(p[x], static_cast<char*>(p[y]) + offset, rows, band, pitch, st);
            });
            offset += band;
        }
        value_of(node->output(0)).canonical = y;
        return;
    }
    if (compile_f32_glue(node))
        return;
    unsupported(*node, "not part of the quantized-inference op set");
}

// The float islands of a quantized graph (dynamic activation scales, softmax, LayerNorm / GELU after
// FusedOpDecomposition, residual adds, attention matrix products, embedding lookups): one kernel per op, each with
// the arithmetic of the reference kernel (include/b200_kernels.h).  Returns false if `node` is not one of them.
bool B200Executable::compile_f32_glue(const std::shared_ptr<Node>& node)
{
    const element::Type& ot = node->get_output_element_type(0);
    const Shape os = node->get_output_shape(0);
    const int64_t n_out = int64_t(shape_size(os));
    auto all_f32 = [&]() {
        for (size_t i = 0; i < node->get_input_size(); ++i)
            if (node->get_input_element_type(i) != element::f32)
                return false;
        return ot == element::f32;
    };

    int bop = -1;
    if (is_type<op::v1::Add>(node)) bop = B200_F32_ADD;
    else if (is_type<op::v1::Subtract>(node)) bop = B200_F32_SUB;
    else if (is_type<op::v1::Multiply>(node)) bop = B200_F32_MUL;
    else if (is_type<op::v1::Divide>(node)) bop = B200_F32_DIV;
    else if (is_type<op::v1::Maximum>(node)) bop = B200_F32_MAX;
    else if (is_type<op::v1::Minimum>(node)) bop = B200_F32_MIN;
    if (bop >= 0)
    {
        if (!all_f32())
            unsupported(*node, "elementwise arithmetic on element types other than f32");
        if (node->get_input_shape(0) != os || node->get_input_shape(1) != os)
            unsupported(*node, "implicit broadcasting (use an explicit Broadcast)");
        // Producer ops folded into the row kernels that read them (b200_softmax_rows_scaled_f32 /
        // b200_layer_norm_rows_sum_f32): a Multiply by a broadcast scalar whose one reader is a last-axis Softmax, and an
        // Add of two tensors whose one reader is a LayerNorm that runs as one kernel.
        if (const Node* user = only_user(node->output(0)))
        {
            if (bop == B200_F32_MUL && is_type<op::v0::Softmax>(user) && !os.empty() && os.back() <= 1535 &&
                static_cast<const op::v0::Softmax*>(user)->get_axes() == AxisSet{os.size() - 1})
                for (int side = 0; side < 2; ++side)
                {
                    Output<Node> bc = node->input_value(side);
                    if (value_of(bc).skipped && is_type<op::v0::Broadcast>(bc.get_node()) &&
                        shape_size(bc.get_node()->get_input_shape(0)) == 1 && !value_of(node->input_value(1 - side)).skipped)
                    {
                        value_of(node->output(0)).skipped = true;
                        return true;
                    }
                }
            if (bop == B200_F32_ADD && is_type<op::v0::LayerNorm>(user) && runs_undecomposed(*user) &&
                user->input_value(0).get_node() == node.get() && !value_of(node->input_value(0)).skipped &&
                !value_of(node->input_value(1)).skipped)
            {
                value_of(node->output(0)).skipped = true;
                return true;
            }
        }
        // an operand that is a Broadcast along new leading axes, left unmaterialised for this op (see below)
        for (int side = 0; side < 2; ++side)
        {
            Output<Node> bc = node->input_value(side);
            if (!value_of(bc).skipped || !is_type<op::v0::Broadcast>(bc.get_node()))
                continue;
            const int64_t period = int64_t(shape_size(bc.get_node()->get_input_shape(0)));
            int v = canonical_slot(bc.get_node()->input_value(0)), a = canonical_slot(node->input_value(1 - side));
            int y = new_slot(Slot::ARENA, size_t(n_out) * 4);
            emit(node, "f32_binary_periodic", [=](const Ptrs& p, cudaStream_t st) {
                return b200_f32_binary_periodic(bop, static_cast<const float*>(p[a]), static_cast<const float*>(p[v]),
                                                static_cast<float*>(p[y]), n_out, period, side == 0, st);
            });
            value_of(node->output(0)).canonical = y;
            return true;
        }
        int a = canonical_slot(node->input_value(0)), b = canonical_slot(node->input_value(1));
        int y = new_slot(Slot::ARENA, size_t(n_out) * 4);
        emit(node, "f32_binary", [=](const Ptrs& p, cudaStream_t st) {
            return b200_f32_binary(bop, static_cast<const float*>(p[a]), static_cast<const float*>(p[b]), static_cast<float*>(p[y]),
                                   n_out, st);
        });
        value_of(node->output(0)).canonical = y;
        return true;
    }

    // Abs whose only reader is a Max (max |x| of a dynamic activation scale): the Max reads x itself
    if (is_type<op::v0::Abs>(node) && all_f32() && only_user(node->output(0)) && is_type<op::v0::Max>(only_user(node->output(0))))
    {
        value_of(node->output(0)).skipped = true;
        return true;
    }
    int uop = -1;
    if (is_type<op::v0::Abs>(node)) uop = B200_F32_ABS;
    else if (is_type<op::v0::Negative>(node)) uop = B200_F32_NEG;
    else if (is_type<op::v0::Sqrt>(node)) uop = B200_F32_SQRT;
    else if (is_type<op::v0::Exp>(node)) uop = B200_F32_EXP;
    else if (is_type<op::v0::Erf>(node)) uop = B200_F32_ERF;
    else if (is_type<op::v0::Relu>(node)) uop = B200_F32_RELU;
    if (uop >= 0)
    {
        if (!all_f32())
            unsupported(*node, "elementwise arithmetic on element types other than f32");
        int x = canonical_slot(node->input_value(0));
        int y = new_slot(Slot::ARENA, size_t(n_out) * 4);
        emit(node, "f32_unary", [=](const Ptrs& p, cudaStream_t st) {
            return b200_f32_unary(uop, static_cast<const float*>(p[x]), static_cast<float*>(p[y]), n_out, st);
        });
        value_of(node->output(0)).canonical = y;
        return true;
    }

    if (auto bc = as_type_ptr<op::v0::Broadcast>(node))
    {
        if (ot.size() != 4 || os.size() > 8)
            unsupported(*node, "Broadcast of element types that are not 4 bytes wide");
        // A Broadcast that only adds LEADING axes repeats its input every shape_size(input) elements.  When its one
        // reader is an f32 elementwise op whose other operand is a real tensor, that op indexes the small input itself and
        // the copy (as large as the op's output) is never written.
        {
            const AxisSet& added = bc->get_broadcast_axes();
            bool leading = ot == element::f32 && !added.empty();
            for (size_t i = 0; i < added.size() && leading; ++i)
                leading = added.count(i) == 1;
            const Node* user = only_user(node->output(0));
            const bool elementwise = user && (is_type<op::v1::Add>(user) || is_type<op::v1::Subtract>(user) || is_type<op::v1::Multiply>(user) ||
                                              is_type<op::v1::Divide>(user) || is_type<op::v1::Maximum>(user) || is_type<op::v1::Minimum>(user));
            if (leading && elementwise && user->get_input_size() == 2 && user->get_output_element_type(0) == element::f32 &&
                user->get_input_shape(0) == os && user->get_input_shape(1) == os)
            {
                const Node* other = user->input_value(0).get_node() == node.get() ? user->input_value(1).get_node()
                                                                                   : user->input_value(0).get_node();
                if (other != node.get() && !is_type<op::v0::Broadcast>(other))
                {
                    value_of(node->output(0)).skipped = true;
                    return true;
                }
            }
        }
        int x = canonical_slot(node->input_value(0));
        int y = new_slot(Slot::ARENA, size_t(n_out) * 4);
        std::vector<int64_t> shape(os.begin(), os.end());
        std::vector<int64_t> axes(bc->get_broadcast_axes().begin(), bc->get_broadcast_axes().end());
        emit(node, "broadcast", [=](const Ptrs& p, cudaStream_t st) {
            return b200_broadcast_b32(p[x], p[y], shape.data(), int(shape.size()), axes.data(), int(axes.size()), st);
        });
        value_of(node->output(0)).canonical = y;
        return true;
    }

    // one reduction: emitted into a given slot so that Softmax can reuse it
    auto emit_reduce = [&](int rop, int x, const Shape& in_shape, const AxisSet& axes_set, int y) {
        std::vector<int64_t> shape(in_shape.begin(), in_shape.end());
        std::vector<int64_t> axes(axes_set.begin(), axes_set.end());
        emit(node, rop == B200_REDUCE_SUM ? "reduce_sum" : rop == B200_REDUCE_MIN ? "reduce_min" : "reduce_max", [=](const Ptrs& p, cudaStream_t st) {
            return b200_reduce_f32(rop, static_cast<const float*>(p[x]), static_cast<float*>(p[y]), shape.data(), int(shape.size()),
                                   axes.data(), int(axes.size()), st);
        });
    };
    const bool is_sum = is_type<op::v0::Sum>(node), is_max = is_type<op::v0::Max>(node), is_min = is_type<op::v0::Min>(node);
    if (is_sum || is_max || is_min)
    {
        if (node->get_input_element_type(0) != element::f32 || node->get_input_shape(0).size() > 8)
            unsupported(*node, "reductions on element types other than f32");
        AxisSet axes = is_sum ? as_type_ptr<op::v0::Sum>(node)->get_reduction_axes()
                              : is_max ? as_type_ptr<op::v0::Max>(node)->get_reduction_axes()
                                       : as_type_ptr<op::v0::Min>(node)->get_reduction_axes();
        int rop = is_sum ? B200_REDUCE_SUM : is_max ? B200_REDUCE_MAX : B200_REDUCE_MIN;
        Output<Node> source = node->input_value(0);
        if (is_max && value_of(source).skipped && is_type<op::v0::Abs>(source.get_node()))
        {
            source = source.get_node()->input_value(0);
            rop = B200_REDUCE_MAX_ABS;
        }
        int x = canonical_slot(source);
        int y = new_slot(Slot::ARENA, size_t(n_out) * 4);
        emit_reduce(rop, x, node->get_input_shape(0), axes, y);
        value_of(node->output(0)).canonical = y;
        return true;
    }

    if (auto ln = as_type_ptr<op::v0::LayerNorm>(node))
    {
        if (!runs_undecomposed(*node))
            unsupported(*node, "LayerNorm other than f32, last axis, with scale and bias");
        const int64_t row = int64_t(os.back()), rows = n_out / row;
        const float eps = static_cast<float>(ln->get_epsilon()); // builder::make_constant(f32, ..., double epsilon)
        Output<Node> source = node->input_value(0);
        int addend = -1;
        if (value_of(source).skipped && is_type<op::v1::Add>(source.get_node())) // the residual Add in front: summed while loading
        {
            addend = canonical_slot(source.get_node()->input_value(1));
            source = source.get_node()->input_value(0);
        }
        int x = canonical_slot(source), g = canonical_slot(node->input_value(1)), b = canonical_slot(node->input_value(2));
        int y = new_slot(Slot::ARENA, size_t(n_out) * 4);
        emit(node, "layer_norm_rows", [=](const Ptrs& p, cudaStream_t st) {
            return b200_layer_norm_rows_sum_f32(static_cast<const float*>(p[x]), addend >= 0 ? static_cast<const float*>(p[addend]) : nullptr,
                                                static_cast<const float*>(p[g]), static_cast<const float*>(p[b]),
                                                static_cast<float*>(p[y]), rows, row, eps, st);
        });
        value_of(node->output(0)).canonical = y;
        return true;
    }
    if (is_type<op::v0::Gelu>(node))
    {
        if (!all_f32())
            unsupported(*node, "Gelu on element types other than f32");
        int x = canonical_slot(node->input_value(0));
        int y = new_slot(Slot::ARENA, size_t(n_out) * 4);
        emit(node, "gelu", [=](const Ptrs& p, cudaStream_t st) {
            return b200_gelu_f32(static_cast<const float*>(p[x]), static_cast<float*>(p[y]), n_out, st);
        });
        value_of(node->output(0)).canonical = y;
        return true;
    }
    if (auto sm = as_type_ptr<op::v0::Softmax>(node))
    {
        // runtime/reference/softmax.hpp: max over the axes, exp(x - max), Kahan sum, divide: the same five steps
        if (!all_f32() && node->get_input_element_type(0) != element::f32)
            unsupported(*node, "Softmax on element types other than f32");
        const AxisSet axes = sm->get_axes();
        Shape red;
        for (size_t i = 0; i < os.size(); ++i)
            if (!axes.count(i))
                red.push_back(os[i]);
        const int64_t n_red = int64_t(shape_size(red));
        Output<Node> source = node->input_value(0);
        int factor = -1;
        if (value_of(source).skipped && is_type<op::v1::Multiply>(source.get_node()))
        {
            // Multiply by a broadcast scalar in front (see the elementwise ops above): applied while the rows are loaded
            const Node* mul = source.get_node();
            const int side = value_of(mul->input_value(0)).skipped ? 0 : 1;
            factor = canonical_slot(mul->input_value(side).get_node()->input_value(0));
            source = mul->input_value(1 - side);
        }
        int x = canonical_slot(source);
        if (axes.size() == 1 && *axes.begin() == os.size() - 1 && os.back() >= 1 && os.back() <= 1535)
        {
            // the last axis of a matrix of rows: one kernel that keeps the rows in shared memory between the steps
            const int64_t row = int64_t(os.back()), rows = n_out / row;
            int y = new_slot(Slot::ARENA, size_t(n_out) * 4);
            emit(node, "softmax_rows", [=](const Ptrs& p, cudaStream_t st) {
                return b200_softmax_rows_scaled_f32(static_cast<const float*>(p[x]), factor >= 0 ? static_cast<const float*>(p[factor]) : nullptr,
                                                    static_cast<float*>(p[y]), rows, row, st);
            });
            value_of(node->output(0)).canonical = y;
            return true;
        }
        int small = new_slot(Slot::ARENA, size_t(n_red) * 4), wide = new_slot(Slot::ARENA, size_t(n_out) * 4),
            e = new_slot(Slot::ARENA, size_t(n_out) * 4), y = new_slot(Slot::ARENA, size_t(n_out) * 4);
        std::vector<int64_t> shape(os.begin(), os.end());
        std::vector<int64_t> ax(axes.begin(), axes.end());
        auto emit_wide = [&]() {
            emit(node, "softmax_broadcast", [=](const Ptrs& p, cudaStream_t st) {
                return b200_broadcast_b32(p[small], p[wide], shape.data(), int(shape.size()), ax.data(), int(ax.size()), st);
            });
        };
        emit_reduce(B200_REDUCE_MAX, x, os, axes, small);
        emit_wide();
        emit(node, "softmax_sub", [=](const Ptrs& p, cudaStream_t st) {
            return b200_f32_binary(B200_F32_SUB, static_cast<const float*>(p[x]), static_cast<const float*>(p[wide]),
                                   static_cast<float*>(p[e]), n_out, st);
        });
        emit(node, "softmax_exp", [=](const Ptrs& p, cudaStream_t st) {
            return b200_f32_unary(B200_F32_EXP, static_cast<const float*>(p[e]), static_cast<float*>(p[e]), n_out, st);
        });
        emit_reduce(B200_REDUCE_SUM, e, os, axes, small);
        emit_wide();
        emit(node, "softmax_div", [=](const Ptrs& p, cudaStream_t st) {
            return b200_f32_binary(B200_F32_DIV, static_cast<const float*>(p[e]), static_cast<const float*>(p[wide]),
                                   static_cast<float*>(p[y]), n_out, st);
        });
        value_of(node->output(0)).canonical = y;
        return true;
    }

    const bool is_bmm = is_type<op::v0::BatchMatMul>(node);
    auto dot = as_type_ptr<op::v0::Dot>(node);
    if (is_bmm || dot)
    {
        const Shape as = node->get_input_shape(0), bs = node->get_input_shape(1);
        if (!all_f32())
            unsupported(*node, "matrix products on element types other than f32 (int8 goes through QuantizedDot)");
        int64_t batch = 1, M, K, N;
        if (is_bmm)
        {
            batch = int64_t(as[0]); M = int64_t(as[1]); K = int64_t(as[2]); N = int64_t(bs[2]);
        }
        else
        {
            if (as.size() != 2 || bs.size() != 2 || dot->get_reduction_axes_count() != 1)
                unsupported(*node, "Dot other than matrix x matrix");
            M = int64_t(as[0]); K = int64_t(as[1]); N = int64_t(bs[1]);
        }
        int a = canonical_slot(node->input_value(0)), b = canonical_slot(node->input_value(1));
        int y = new_slot(Slot::ARENA, size_t(n_out) * 4);
        emit(node, "bmm_f32", [=](const Ptrs& p, cudaStream_t st) {
            return b200_bmm_f32(static_cast<const float*>(p[a]), static_cast<const float*>(p[b]), static_cast<float*>(p[y]), batch, M,
                                K, N, st);
        });
        value_of(node->output(0)).canonical = y;
        return true;
    }

    if (auto g = as_type_ptr<op::v0::Gather>(node))
    {
        const Shape ps = node->get_input_shape(0), is = node->get_input_shape(1);
        const element::Type& it = node->get_input_element_type(1);
        if (ot.size() != 4 || ps.size() != 2 || is.size() != 1 || g->get_axis() != 0 || (it != element::i32 && it != element::i64))
            unsupported(*node, "Gather other than rows of a 2-D 4-byte table by an i32 / i64 index vector");
        int t = canonical_slot(node->input_value(0)), idx = canonical_slot(node->input_value(1));
        int y = new_slot(Slot::ARENA, size_t(n_out) * 4);
        const int64_t rows = int64_t(ps[0]), width = int64_t(ps[1]), count = int64_t(is[0]);
        const int itype = dtype_of(it);
        emit(node, "gather_rows", [=](const Ptrs& p, cudaStream_t st) {
            return b200_gather_rows_b32(p[t], rows, width, p[idx], itype, count, p[y], st);
        });
        value_of(node->output(0)).canonical = y;
        return true;
    }
    return false;
}

static std::vector<int64_t> to_i64(const Shape& s)
{
    return std::vector<int64_t>(s.begin(), s.end());
}

namespace
{
    // A stride-2 convolution over <= 4 channels with constant filters (a network stem): the cell-grid path applies.
    bool stem_geometry_of(const Node* conv, b200_conv_params& c, int64_t geo[5])
    {
        Strides strides, dilation, data_dilation;
        CoordinateDiff below, above;
        if (auto o = as_type<const op::v0::QuantizedConvolutionBias>(conv))
        {
            strides = o->get_window_movement_strides(); dilation = o->get_window_dilation_strides();
            data_dilation = o->get_data_dilation_strides(); below = o->get_padding_below(); above = o->get_padding_above();
        }
        else if (auto o2 = as_type<const op::v0::QuantizedConvolutionRelu>(conv))
        {
            strides = o2->get_window_movement_strides(); dilation = o2->get_window_dilation_strides();
            data_dilation = o2->get_data_dilation_strides(); below = o2->get_padding_below(); above = o2->get_padding_above();
        }
        else
            return false;
        const Shape& ds = conv->get_input_shape(0);
        const Shape& fs = conv->get_input_shape(1);
        if (ds.size() != 4 || fs.size() != 4 || ds[1] > 4 || strides != Strides{2, 2} || dilation != Strides{1, 1} ||
            data_dilation != Strides{1, 1} || !as_constant(conv->input_value(1)))
            return false;
        for (auto v : below) if (v < 0) return false;
        for (auto v : above) if (v < 0) return false;
        c.N = ds[0]; c.H = ds[2]; c.W = ds[3]; c.C = 4;
        c.K = fs[0]; c.R = fs[2]; c.S = fs[3];
        c.stride_h = c.stride_w = 2;
        c.pad_h = below[0]; c.pad_w = below[1]; c.pad_h_above = above[0]; c.pad_w_above = above[1];
        c.dilation_h = c.dilation_w = 1;
        return b200_stem_geometry(c.H, c.W, c.R, c.S, c.pad_h, c.pad_w, c.pad_h_above, c.pad_w_above, &geo[0], &geo[1], &geo[2],
                                  &geo[3], &geo[4]) == B200_OK;
    }

    // Quantize(f32 -> u8/i8, per-tensor) whose only consumer is the data input of such a stem convolution: the
    // quantisation is done by the kernel that packs the stem's cell grid and the one-byte image is never written.
    bool quantize_feeds_stem(const Node* qn)
    {
        auto q = as_type<const op::v0::Quantize>(qn);
        if (!q || !q->get_axes().empty() || q->get_input_element_type(0) != element::f32)
            return false;
        const element::Type& ot = q->get_output_element_type(0);
        if (ot != element::u8 && ot != element::i8)
            return false;
        auto users = q->output(0).get_target_inputs();
        if (users.size() != 1 || users.begin()->get_index() != 0)
            return false;
        b200_conv_params c;
        int64_t geo[5];
        return stem_geometry_of(users.begin()->get_node(), c, geo);
    }
}

void B200Executable::compile_quantize(const std::shared_ptr<Node>& node)
{
    auto q = as_type_ptr<op::v0::Quantize>(node);
    AvgPoolHead head;
    if (match_head(node.get(), head))
    {
        if (try_compile_avgpool_head(node))
            return;
    }
    if (quantize_feeds_stem(node.get()))
    {
        value_of(node->output(0)).skipped = true; // emitted together with the convolution
        return;
    }
    if (node->get_input_element_type(0) != element::f32)
        unsupported(*node, "input element type " + node->get_input_element_type(0).get_type_name());
    int qt = dtype_of(q->get_output_element_type(0));
    if (qt != B200_U8 && qt != B200_I8 && qt != B200_I32)
        unsupported(*node, "output element type");
    int x = canonical_slot(node->input_value(0)), s = canonical_slot(node->input_value(1)),
        z = canonical_slot(node->input_value(2));
    std::vector<int64_t> shape = to_i64(node->get_input_shape(0));
    std::vector<int64_t> axes(q->get_axes().begin(), q->get_axes().end());
    int mode = static_cast<int>(q->get_round_mode());
    int y = new_slot(Slot::ARENA, shape_size(node->get_output_shape(0)) * q->get_output_element_type(0).size());
    emit(node, "quantize", [=](const Ptrs& p, cudaStream_t st) {
        return b200_quantize(static_cast<const float*>(p[x]), static_cast<const float*>(p[s]), p[z], p[y], qt,
                             shape.data(), int(shape.size()), axes.data(), int(axes.size()), mode, st);
    });
    value_of(node->output(0)).canonical = y;
}

bool B200Executable::try_compile_avgpool_head(const std::shared_ptr<Node>& node)
{
    AvgPoolHead h;
    if (!match_head(node.get(), h))
        return false;
    Output<Node> data = h.dq->input_value(0);
    const b200_pool_params g = pool_params_of(*h.pool);
    const int in_type = dtype_of(data.get_element_type()), out_type = dtype_of(h.q->get_output_element_type(0));
    int x = nhwc_slot(data);
    int s_in = canonical_slot(h.dq->input_value(1)), s_out = canonical_slot(h.q->input_value(1));
    int y = new_slot(Slot::ARENA, shape_size(h.q->get_output_shape(0)));
    if (is_global_unpadded(g) && in_type == B200_U8 && out_type == B200_U8)
    {
        int64_t N = g.N, C = g.C, H = g.H, W = g.W;
        emit(node, "global_avgpool_q", [=](const Ptrs& p, cudaStream_t st) {
            return b200_global_avgpool_q_nhwc_u8(p[x], p[y], static_cast<const float*>(p[s_in]),
                                                 static_cast<const float*>(p[s_out]), N, H, W, C, st);
        });
    }
    else
    {
        emit(node, "avgpool_q", [=](const Ptrs& p, cudaStream_t st) {
            return b200_avgpool_q_nhwc(p[x], in_type, p[y], out_type, static_cast<const float*>(p[s_in]),
                                       static_cast<const float*>(p[s_out]), &g, st);
        });
    }
    Value& o = value_of(node->output(0));
    o.nhwc = y;
    if (g.P * g.Q == 1)
        o.canonical = y; // [N,C,1,1]: channels-last and NCHW coincide
    return true;
}

// op::v0::AvgPool outside that pattern: f32 on NCHW, or the op applied to u8 / i8 directly (channels-last), both with the
// arithmetic of runtime::reference::avg_pool.
void B200Executable::compile_avg_pool(const std::shared_ptr<Node>& node)
{
    auto pool = as_type_ptr<op::v0::AvgPool>(node);
    const element::Type& et = node->get_input_element_type(0);
    if (node->get_input_shape(0).size() != 4)
        unsupported(*node, "pooling over other than two spatial dimensions");
    const b200_pool_params g = pool_params_of(*pool);
    if (et == element::f32)
    {
        int x = canonical_slot(node->input_value(0));
        int y = new_slot(Slot::ARENA, shape_size(node->get_output_shape(0)) * sizeof(float));
        emit(node, "avgpool_f32", [=](const Ptrs& p, cudaStream_t st) {
            return b200_avgpool_f32_nchw(static_cast<const float*>(p[x]), static_cast<float*>(p[y]), &g, st);
        });
        value_of(node->output(0)).canonical = y;
        return;
    }
    if (et != element::u8 && et != element::i8)
        unsupported(*node, "element type " + et.get_type_name());
    const int type = dtype_of(et);
    int x = nhwc_slot(node->input_value(0));
    int y = new_slot(Slot::ARENA, shape_size(node->get_output_shape(0)));
    emit(node, "avgpool_bytes", [=](const Ptrs& p, cudaStream_t st) { return b200_avgpool_nhwc_bytes(p[x], p[y], type, &g, st); });
    Value& o = value_of(node->output(0));
    o.nhwc = y;
    if (g.P * g.Q == 1)
        o.canonical = y;
}

void B200Executable::compile_dequantize(const std::shared_ptr<Node>& node)
{
    auto dq = as_type_ptr<op::v0::Dequantize>(node);
    if (avgpool_head_member(node.get()))
    {
        value_of(node->output(0)).skipped = true;
        return;
    }
    if (node->get_output_element_type(0) != element::f32)
        unsupported(*node, "output element type");
    int qt = dtype_of(node->get_input_element_type(0));
    if (qt != B200_U8 && qt != B200_I8 && qt != B200_I32)
        unsupported(*node, "input element type");
    int x = canonical_slot(node->input_value(0)), s = canonical_slot(node->input_value(1)),
        z = canonical_slot(node->input_value(2));
    std::vector<int64_t> shape = to_i64(node->get_input_shape(0));
    std::vector<int64_t> axes(dq->get_axes().begin(), dq->get_axes().end());
    int y = new_slot(Slot::ARENA, shape_size(node->get_output_shape(0)) * sizeof(float));
    emit(node, "dequantize", [=](const Ptrs& p, cudaStream_t st) {
        return b200_dequantize(p[x], static_cast<const float*>(p[s]), p[z], static_cast<float*>(p[y]), qt, shape.data(),
                               int(shape.size()), axes.data(), int(axes.size()), st);
    });
    value_of(node->output(0)).canonical = y;
}

namespace
{
    struct ConvAttrs
    {
        Strides strides, dilation, data_dilation;
        CoordinateDiff below, above;
    };

    template <typename T>
    ConvAttrs attrs_of(const std::shared_ptr<T>& op)
    {
        return ConvAttrs{op->get_window_movement_strides(), op->get_window_dilation_strides(),
                         op->get_data_dilation_strides(), op->get_padding_below(), op->get_padding_above()};
    }
}

// Shared by the fused and the core convolution: emits the layout work and the kernel launch.
static b200_conv_params make_conv_params(const Node& node, const ConvAttrs& a, const Shape& ds, const Shape& fs, size_t c_dev)
{
    if (ds.size() != 4 || fs.size() != 4)
        unsupported(node, "only 2-D convolutions");
    for (size_t v : a.data_dilation)
        if (v != 1)
            unsupported(node, "data dilation on this path");
    for (auto v : a.below)
        if (v < 0) unsupported(node, "negative padding on this path");
    for (auto v : a.above)
        if (v < 0) unsupported(node, "negative padding on this path");
    b200_conv_params c;
    c.N = ds[0]; c.H = ds[2]; c.W = ds[3]; c.C = c_dev;
    c.K = fs[0]; c.R = fs[2]; c.S = fs[3];
    c.stride_h = a.strides[0]; c.stride_w = a.strides[1];
    c.pad_h = a.below[0]; c.pad_w = a.below[1];
    c.pad_h_above = a.above[0]; c.pad_w_above = a.above[1];
    c.dilation_h = a.dilation[0]; c.dilation_w = a.dilation[1];
    return c;
}

// Data dilation and negative padding (legal in every convolution op, runtime/reference/convolution.hpp:59-265) are taken out
// of the convolution itself: the channels-last input `x` [N, H, W, c_dev] is dilated with zero pixels and cropped into a new
// buffer (b200_dilate_crop_nhwc_u8), `ds` then describes that buffer and `below` / `above` keep their non-negative part.
// Returns the slot to convolve.
int B200Executable::dilate_and_crop_input(const std::shared_ptr<Node>& node, int x, Shape& ds, Strides& data_dilation,
                                          CoordinateDiff& below, CoordinateDiff& above, size_t c_dev)
{
    const bool dilated = data_dilation[0] != 1 || data_dilation[1] != 1;
    const bool cropped = below[0] < 0 || below[1] < 0 || above[0] < 0 || above[1] < 0;
    if (!dilated && !cropped)
        return x;
    const int64_t N = ds[0], H = ds[2], W = ds[3], Cd = int64_t(c_dev);
    const int64_t dh = int64_t(data_dilation[0]), dw = int64_t(data_dilation[1]);
    const int64_t cb0 = std::max<int64_t>(-below[0], 0), cb1 = std::max<int64_t>(-below[1], 0);
    const int64_t ca0 = std::max<int64_t>(-above[0], 0), ca1 = std::max<int64_t>(-above[1], 0);
    const int64_t Ho = (H - 1) * dh + 1 - cb0 - ca0, Wo = (W - 1) * dw + 1 - cb1 - ca1;
    if (Ho <= 0 || Wo <= 0)
        unsupported(*node, "negative padding that leaves no input");
    int xd = new_slot(Slot::ARENA, size_t(N * Ho * Wo * Cd));
    emit(node, "dilate_crop", [=](const Ptrs& p, cudaStream_t st) {
        return b200_dilate_crop_nhwc_u8(p[x], p[xd], N, H, W, Cd, dh, dw, cb0, cb1, ca0, ca1, st);
    });
    ds[2] = size_t(Ho);
    ds[3] = size_t(Wo);
    data_dilation = Strides{1, 1};
    below = CoordinateDiff{std::max<std::ptrdiff_t>(below[0], 0), std::max<std::ptrdiff_t>(below[1], 0)};
    above = CoordinateDiff{std::max<std::ptrdiff_t>(above[0], 0), std::max<std::ptrdiff_t>(above[1], 0)};
    return xd;
}

void B200Executable::compile_fused_conv(const std::shared_ptr<Node>& node)
{
    ConvAttrs a;
    bool relu = false;
    int bias_in = -1, scale_in = -1, sum_in = -1, sum_scale_in = -1;
    if (auto op = as_type_ptr<op::v0::QuantizedConvolutionBias>(node))
    {
        a = attrs_of(op); relu = op->with_relu(); bias_in = 2; scale_in = 3;
    }
    else if (auto op = as_type_ptr<op::v0::QuantizedConvolutionBiasAdd>(node))
    {
        a = attrs_of(op); relu = op->with_relu(); bias_in = 2; sum_in = 3; scale_in = 4; sum_scale_in = 5;
    }
    else if (auto op = as_type_ptr<op::v0::QuantizedConvolutionBiasSignedAdd>(node))
    {
        a = attrs_of(op); relu = op->with_relu(); bias_in = 2; sum_in = 3; scale_in = 4; sum_scale_in = 5;
    }
    else
    {
        auto op2 = as_type_ptr<op::v0::QuantizedConvolutionRelu>(node);
        a = attrs_of(op2); relu = true; scale_in = 2;
    }
    Shape ds = node->get_input_shape(0);
    const Shape fs = node->get_input_shape(1), os = node->get_output_shape(0);
    if (ds.size() != 4 || fs.size() != 4)
        unsupported(*node, "only 2-D convolutions");
    const bool plain_geometry = a.data_dilation == Strides{1, 1} && a.below[0] >= 0 && a.below[1] >= 0 && a.above[0] >= 0 && a.above[1] >= 0;
    int dt = dtype_of(node->get_input_element_type(0));
    if ((dt != B200_U8 && dt != B200_I8) || node->get_input_element_type(1) != element::i8)
        unsupported(*node, "data must be u8/i8 and filters i8");
    if (bias_in >= 0 && node->get_input_element_type(bias_in) != element::i32)
        unsupported(*node, "bias must be i32 (the builders quantise f32 bias to i32)");
    if (node->get_input_element_type(scale_in) != element::f32)
        unsupported(*node, "scale must be f32");
    size_t n_scale = shape_size(node->get_input_shape(scale_in));
    if (n_scale != 1 && n_scale != fs[0])
        unsupported(*node, "scale must have 1 or K elements");
    int out_t = dtype_of(node->get_output_element_type(0));

    b200_epilogue e;
    memset(&e, 0, sizeof(e));
    e.relu = relu;
    e.scale_count = int64_t(n_scale);
    e.out_type = out_t;
    int bias = bias_in >= 0 ? canonical_slot(node->input_value(bias_in)) : -1;
    int scale = canonical_slot(node->input_value(scale_in));
    int sum = -1, sum_scale = -1;
    if (sum_in >= 0)
    {
        sum = nhwc_slot(node->input_value(sum_in));
        sum_scale = canonical_slot(node->input_value(sum_scale_in));
        e.sum_type = dtype_of(node->get_input_element_type(sum_in));
    }
    int y = new_slot(Slot::ARENA, shape_size(os));
    const size_t C = ds[1];

    if (plain_geometry && C <= 4 && a.strides[0] == 2 && a.strides[1] == 2 && a.dilation[0] == 1 && a.dilation[1] == 1 &&
        as_constant(node->input_value(1)))
    {
        // stride-2 small-channel stem: 2x2x4 cells, then an implicit GEMM over overlapping 64-byte windows
        b200_conv_params c = make_conv_params(*node, a, ds, fs, 4);
        int64_t P, Q, Hc, Wc, Rc;
        if (b200_stem_geometry(c.H, c.W, c.R, c.S, c.pad_h, c.pad_w, c.pad_h_above, c.pad_w_above, &P, &Q, &Hc, &Wc, &Rc) ==
            B200_OK)
        {
            auto cf = as_constant(node->input_value(1));
            std::vector<int8_t> w(size_t(c.K) * size_t(Rc) * 64);
            kernel_check(b200_stem_pack_filter_host(static_cast<const int8_t*>(cf->get_data_ptr()), w.data(), c.K, int64_t(C), c.R,
                                             c.S, c.pad_h, c.pad_w),
                  "b200_stem_pack_filter_host");
            int wslot = upload_constant(constant_key("stem_filter", {cf.get()}), w.data(), w.size());
            int cells = new_slot(Slot::ARENA, size_t(b200_stem_cells_bytes(c.N, c.H, c.W, c.R, c.S, c.pad_h, c.pad_w, c.pad_h_above,
                                                                           c.pad_w_above)));
            int64_t Ci = C;
            if (value_of(node->input_value(0)).skipped)
            {
                // the producing Quantize was held back (quantize_feeds_stem): quantise while packing
                auto qn = as_type_ptr<op::v0::Quantize>(node->input_value(0).get_node_shared_ptr());
                int xf = canonical_slot(qn->input_value(0)), qs = canonical_slot(qn->input_value(1)),
                    qz = canonical_slot(qn->input_value(2));
                int mode = static_cast<int>(qn->get_round_mode());
                emit(qn, "stem_cells_quantize", [=](const Ptrs& p, cudaStream_t st) {
                    return b200_stem_pack_input_f32(static_cast<const float*>(p[xf]), static_cast<const float*>(p[qs]), p[qz], dt,
                                                    mode, p[cells], c.N, Ci, c.H, c.W, c.R, c.S, c.pad_h, c.pad_w,
                                                    c.pad_h_above, c.pad_w_above, st);
                });
            }
            else
            {
                int xc = canonical_slot(node->input_value(0));
                emit(node, "stem_cells", [=](const Ptrs& p, cudaStream_t st) {
                    return b200_stem_pack_input(p[xc], p[cells], c.N, Ci, c.H, c.W, c.R, c.S, c.pad_h, c.pad_w, c.pad_h_above,
                                                c.pad_w_above, st);
                });
            }
            emit(node, "stem_qconv", [=](const Ptrs& p, cudaStream_t st) {
                b200_epilogue ee = e;
                ee.bias = bias >= 0 ? static_cast<const int32_t*>(p[bias]) : nullptr;
                ee.scale = static_cast<const float*>(p[scale]);
                ee.sum_in = sum >= 0 ? p[sum] : nullptr;
                ee.sum_scale = sum_scale >= 0 ? static_cast<const float*>(p[sum_scale]) : nullptr;
                return b200_qconv_stem(p[cells], dt, static_cast<const int8_t*>(p[wslot]), p[y], c.N, c.H, c.W, c.K, c.R, c.S,
                                       c.pad_h, c.pad_w, c.pad_h_above, c.pad_w_above, &ee, st);
            });
            value_of(node->output(0)).nhwc = y;
            return;
        }
    }

    if (plain_geometry && C <= 4 && fs[3] <= 8 && a.dilation[0] == 1 && a.dilation[1] == 1)
    {
        // small-channel stem: 4-channel pixels -> patch matrix -> matrix product
        b200_conv_params c = make_conv_params(*node, a, ds, fs, 4);
        int64_t P = 0, Q = 0;
        b200_qconv_out_shape(&c, &P, &Q);
        auto cf = as_constant(node->input_value(1));
        if (!cf)
            unsupported(*node, "the small-channel path needs constant filters");
        const int8_t* src = static_cast<const int8_t*>(cf->get_data_ptr());
        size_t K = fs[0], R = fs[2], S = fs[3];
        std::vector<int8_t> w(K * R * 32, 0);
        for (size_t k = 0; k < K; ++k)
            for (size_t ch = 0; ch < C; ++ch)
                for (size_t r = 0; r < R; ++r)
                    for (size_t s = 0; s < S; ++s)
                        w[(k * R + r) * 32 + s * 4 + ch] = src[((k * C + ch) * R + r) * S + s];
        int wslot = upload_constant(constant_key("c4_filter", {cf.get()}), w.data(), w.size());
        int xc = canonical_slot(node->input_value(0));
        int x4 = new_slot(Slot::ARENA, ds[0] * ds[2] * ds[3] * 4);
        int64_t M = int64_t(ds[0]) * P * Q, KK = int64_t(R) * 32;
        int patches = new_slot(Slot::ARENA, size_t(M) * size_t(KK));
        int64_t N = ds[0], H = ds[2], W = ds[3], Ci = C;
        emit(node, "nchw_to_nhwc4", [=](const Ptrs& p, cudaStream_t st) {
            return b200_nchw_to_nhwc_u8(p[xc], p[x4], N, Ci, H, W, 4, st);
        });
        emit(node, "im2col_c4", [=](const Ptrs& p, cudaStream_t st) {
            return b200_im2col_c4_u8(p[x4], p[patches], c.N, c.H, c.W, c.R, c.S, c.stride_h, c.stride_w, c.pad_h, c.pad_w,
                                     c.pad_h_above, c.pad_w_above, st);
        });
        int64_t Kout = fs[0];
        emit(node, "stem_qgemm", [=](const Ptrs& p, cudaStream_t st) {
            b200_epilogue ee = e;
            ee.bias = bias >= 0 ? static_cast<const int32_t*>(p[bias]) : nullptr;
            ee.scale = static_cast<const float*>(p[scale]);
            ee.sum_in = sum >= 0 ? p[sum] : nullptr;
            ee.sum_scale = sum_scale >= 0 ? static_cast<const float*>(p[sum_scale]) : nullptr;
            return b200_qgemm(p[patches], dt, static_cast<const int8_t*>(p[wslot]), p[y], M, Kout, KK, &ee, st);
        });
        value_of(node->output(0)).nhwc = y;
        return;
    }

    const size_t c_dev = align_up(C, 64);
    int x;
    if (c_dev == C)
        x = nhwc_slot(node->input_value(0));
    else
    {
        // channel counts the tensor-core path cannot take directly are zero-padded to a multiple of 64
        int xc = canonical_slot(node->input_value(0));
        x = new_slot(Slot::ARENA, ds[0] * ds[2] * ds[3] * c_dev);
        int64_t N = ds[0], H = ds[2], W = ds[3], Ci = C, Cp = c_dev;
        emit(node, "nchw_to_nhwc_pad", [=](const Ptrs& p, cudaStream_t st) {
            return b200_nchw_to_nhwc_u8(p[xc], p[x], N, Ci, H, W, Cp, st);
        });
    }
    x = dilate_and_crop_input(node, x, ds, a.data_dilation, a.below, a.above, c_dev);
    bool image = false;
    int w = packed_filters(node->input_value(1), c_dev, &image);
    b200_conv_params c = make_conv_params(*node, a, ds, fs, c_dev);
    emit(node, "qconv", [=](const Ptrs& p, cudaStream_t st) {
        b200_epilogue ee = e;
        ee.bias = bias >= 0 ? static_cast<const int32_t*>(p[bias]) : nullptr;
        ee.scale = static_cast<const float*>(p[scale]);
        ee.sum_in = sum >= 0 ? p[sum] : nullptr;
        ee.sum_scale = sum_scale >= 0 ? static_cast<const float*>(p[sum_scale]) : nullptr;
        return image ? b200_qconv_packed(p[x], dt, static_cast<const int8_t*>(p[w]), p[y], &c, &ee, st)
                     : b200_qconv(p[x], dt, static_cast<const int8_t*>(p[w]), p[y], &c, &ee, st);
    });
    value_of(node->output(0)).nhwc = y;
}

// The value of a one-element u8 / i8 Constant (a per-tensor zero point); false for anything else.
static bool scalar_zero_point(const Output<Node>& v, int32_t& value)
{
    auto c = as_type_ptr<op::v0::Constant>(v.get_node_shared_ptr());
    if (!c || shape_size(c->get_output_shape(0)) != 1)
        return false;
    if (c->get_output_element_type(0) == element::u8)
        value = *static_cast<const uint8_t*>(c->get_data_ptr());
    else if (c->get_output_element_type(0) == element::i8)
        value = *static_cast<const int8_t*>(c->get_data_ptr());
    else
        return false;
    return true;
}

void B200Executable::compile_core_conv(const std::shared_ptr<Node>& node)
{
    auto op = as_type_ptr<op::v0::QuantizedConvolution>(node);
    ConvAttrs a = attrs_of(op);
    Shape ds = node->get_input_shape(0);
    const Shape fs = node->get_input_shape(1), os = node->get_output_shape(0);
    if (ds.size() != 4 || fs.size() != 4)
        unsupported(*node, "only 2-D convolutions");
    int dt = dtype_of(node->get_input_element_type(0));
    const element::Type& ft = node->get_input_element_type(1);
    if (dt != B200_U8 || (ft != element::i8 && ft != element::u8))
        unsupported(*node, "data must be u8 and filters i8 or u8");
    if (ft == element::u8)
        dt |= B200_WEIGHTS_U8; // kind::i8 takes unsigned B operands as well
    int32_t za = 0, zf = 0;
    if (!scalar_zero_point(node->input_value(3), za) || !scalar_zero_point(node->input_value(5), zf))
        unsupported(*node, "input / filter zero points that are not per-tensor constants");
    auto zo = as_constant(node->input_value(7));
    if (!zo)
        unsupported(*node, "output zero point must be a constant");
    int out_t = dtype_of(node->get_output_element_type(0));
    int32_t out_zp = 0;
    if (out_t == B200_U8) out_zp = *static_cast<const uint8_t*>(zo->get_data_ptr());
    else if (out_t == B200_I8) out_zp = *static_cast<const int8_t*>(zo->get_data_ptr());
    else if (out_t == B200_I32) out_zp = *static_cast<const int32_t*>(zo->get_data_ptr());
    else unsupported(*node, "output element type");
    int scale = scalar_product_scale(node->input_value(2), node->input_value(4), node->input_value(6));
    const size_t C = ds[1];
    const size_t c_dev = align_up(C, 64);
    int x;
    if (c_dev == C)
        x = nhwc_slot(node->input_value(0));
    else
    {
        int xc = canonical_slot(node->input_value(0));
        x = new_slot(Slot::ARENA, ds[0] * ds[2] * ds[3] * c_dev);
        int64_t N = ds[0], H = ds[2], W = ds[3], Ci = C, Cp = c_dev;
        emit(node, "nchw_to_nhwc_pad", [=](const Ptrs& p, cudaStream_t st) {
            return b200_nchw_to_nhwc_u8(p[xc], p[x], N, Ci, H, W, Cp, st);
        });
    }
    // with non-zero zero points the correction terms count the taps inside the image from the op's own geometry: there the
    // dilated / cropped form is not offered
    if (za == 0 && zf == 0)
        x = dilate_and_crop_input(node, x, ds, a.data_dilation, a.below, a.above, c_dev);
    bool image = false;
    int w = packed_filters(node->input_value(1), c_dev, &image);
    b200_conv_params c = make_conv_params(*node, a, ds, fs, c_dev);
    const size_t esz = node->get_output_element_type(0).size();
    int y = new_slot(Slot::ARENA, shape_size(os) * esz);
    if (za != 0 || zf != 0)
    {
        // (a - za) * (w - zf) over the taps inside the image: the contraction on the stored bytes with exact int32
        // output, then one pass that subtracts the rank-one terms and requantises (zero_points.cu)
        b200_zero_point_params z;
        memset(&z, 0, sizeof(z));
        z.N = int64_t(os[0]); z.K = int64_t(os[1]); z.P = int64_t(os[2]); z.Q = int64_t(os[3]);
        z.H = int64_t(ds[2]); z.W = int64_t(ds[3]); z.C = int64_t(C); z.R = int64_t(fs[2]); z.S = int64_t(fs[3]);
        z.stride_h = c.stride_h; z.stride_w = c.stride_w; z.dilation_h = c.dilation_h; z.dilation_w = c.dilation_w;
        z.pad_h = c.pad_h; z.pad_w = c.pad_w;
        z.input_zero_point = za; z.filter_zero_point = zf;
        const int acc = new_slot(Slot::ARENA, shape_size(os) * 4);
        emit(node, "qconv_raw", [=](const Ptrs& p, cudaStream_t st) {
            b200_epilogue e;
            memset(&e, 0, sizeof(e));
            e.round_half_away = 2;
            e.out_type = B200_I32;
            return image ? b200_qconv_packed(p[x], dt, static_cast<const int8_t*>(p[w]), p[acc], &c, &e, st)
                         : b200_qconv(p[x], dt, static_cast<const int8_t*>(p[w]), p[acc], &c, &e, st);
        });
        int taps = -1, windows = -1;
        if (za != 0)
        {
            const int f = canonical_slot(node->input_value(1));
            const int ft_code = ft == element::u8 ? B200_U8 : B200_I8;
            taps = new_slot(Slot::ARENA, fs[0] * fs[2] * fs[3] * 4);
            const int64_t K = fs[0], RS = fs[2] * fs[3], Cf = fs[1];
            emit(node, "filter_tap_sums", [=](const Ptrs& p, cudaStream_t st) {
                return b200_strided_sums(p[f], ft_code, static_cast<int32_t*>(p[taps]), K, RS, Cf, Cf * RS, 1, RS, st);
            });
        }
        if (zf != 0)
        {
            const int xc = canonical_slot(node->input_value(0));
            const int pixels = new_slot(Slot::ARENA, ds[0] * ds[2] * ds[3] * 4);
            windows = new_slot(Slot::ARENA, os[0] * os[2] * os[3] * 4);
            const int64_t N = ds[0], HW = ds[2] * ds[3], Ci = C;
            emit(node, "pixel_sums", [=](const Ptrs& p, cudaStream_t st) {
                return b200_strided_sums(p[xc], B200_U8, static_cast<int32_t*>(p[pixels]), N, HW, Ci, Ci * HW, 1, HW, st);
            });
            emit(node, "window_sums", [=](const Ptrs& p, cudaStream_t st) {
                return b200_window_sums(static_cast<const int32_t*>(p[pixels]), static_cast<int32_t*>(p[windows]), &z, st);
            });
        }
        emit(node, "requant_zero_points", [=](const Ptrs& p, cudaStream_t st) {
            b200_epilogue e;
            memset(&e, 0, sizeof(e));
            e.scale = static_cast<const float*>(p[scale]);
            e.scale_count = 1;
            e.round_half_away = 1;
            e.out_zero_point = out_zp;
            e.out_type = out_t;
            return b200_requant_zero_points(static_cast<const int32_t*>(p[acc]), taps >= 0 ? static_cast<const int32_t*>(p[taps]) : nullptr,
                                            windows >= 0 ? static_cast<const int32_t*>(p[windows]) : nullptr, &z, &e, p[y], st);
        });
    }
    else
    emit(node, "qconv_core", [=](const Ptrs& p, cudaStream_t st) {
        b200_epilogue e;
        memset(&e, 0, sizeof(e));
        e.scale = static_cast<const float*>(p[scale]);
        e.scale_count = 1;
        e.round_half_away = 1;
        e.out_zero_point = out_zp;
        e.out_type = out_t;
        return image ? b200_qconv_packed(p[x], dt, static_cast<const int8_t*>(p[w]), p[y], &c, &e, st)
                     : b200_qconv(p[x], dt, static_cast<const int8_t*>(p[w]), p[y], &c, &e, st);
    });
    Value& o = value_of(node->output(0));
    if (esz == 1)
        o.nhwc = y;
    else
    {
        // 4-byte outputs: bring [N,P,Q,K] back to NCHW with the byte transposer (4 bytes per element)
        int yc = new_slot(Slot::ARENA, shape_size(os) * esz);
        int64_t N = os[0], K = os[1], PQ = os[2] * os[3];
        emit(node, "nhwc_to_nchw_i32", [=](const Ptrs& p, cudaStream_t st) {
            return b200_nhwc_to_nchw_b32(p[y], p[yc], N, K, PQ, st);
        });
        o.canonical = yc;
    }
}

void B200Executable::compile_dot_bias(const std::shared_ptr<Node>& node)
{
    auto op = as_type_ptr<op::v0::QuantizedDotBias>(node);
    const Shape as = node->get_input_shape(0), ws = node->get_input_shape(1);
    int dt = dtype_of(node->get_input_element_type(0));
    if ((dt != B200_U8 && dt != B200_I8) || node->get_input_element_type(1) != element::i8)
        unsupported(*node, "data must be u8/i8 and weights i8");
    if (node->get_input_element_type(2) != element::i32)
        unsupported(*node, "bias must be i32");
    if (as.size() != 2 || ws.size() != 2 || as[1] % 16 != 0)
        unsupported(*node, "2-D operands with a reduction length that is a multiple of 16");
    size_t n_scale = shape_size(node->get_input_shape(3));
    if (n_scale != 1 && n_scale != ws[0])
        unsupported(*node, "scale must have 1 or N elements");
    int a = canonical_slot(node->input_value(0)), bias = canonical_slot(node->input_value(2)),
        scale = canonical_slot(node->input_value(3));
    // constant weights [N,K] go to the device in the packed image
    int w;
    bool w_image = false;
    const std::string wkey = constant_key("weight_image", {node->input_value(1).get_node()});
    if (as_constant(node->input_value(1)) && have_saved_constant(wkey))
    {
        w = upload_constant(wkey, nullptr, size_t(b200_packed_weights_bytes(int64_t(ws[0]), int64_t(ws[1]), 128)));
        w_image = true;
    }
    else if (auto cw = as_constant(node->input_value(1)))
    {
        std::vector<int8_t> image(size_t(b200_packed_weights_bytes(int64_t(ws[0]), int64_t(ws[1]), 128)));
        kernel_check(b200_pack_weights_host(static_cast<const int8_t*>(cw->get_data_ptr()), image.data(), int64_t(ws[0]),
                                            int64_t(ws[1]), 128),
                     "b200_pack_weights_host");
        w = upload_constant(wkey, image.data(), image.size());
        w_image = true;
    }
    else
        w = canonical_slot(node->input_value(1));
    int out_t = dtype_of(node->get_output_element_type(0));
    int y = new_slot(Slot::ARENA, shape_size(node->get_output_shape(0)) * node->get_output_element_type(0).size());
    int64_t M = as[0], K = as[1], N = ws[0];
    bool relu = op->with_relu();
    emit(node, "qgemm", [=](const Ptrs& p, cudaStream_t st) {
        b200_epilogue e;
        memset(&e, 0, sizeof(e));
        e.bias = static_cast<const int32_t*>(p[bias]);
        e.scale = static_cast<const float*>(p[scale]);
        e.scale_count = int64_t(n_scale);
        e.relu = relu;
        e.out_type = out_t;
        return w_image ? b200_qgemm_packed(p[a], dt, static_cast<const int8_t*>(p[w]), p[y], M, N, K, &e, st)
                       : b200_qgemm(p[a], dt, static_cast<const int8_t*>(p[w]), p[y], M, N, K, &e, st);
    });
    value_of(node->output(0)).canonical = y;
}

void B200Executable::compile_core_dot(const std::shared_ptr<Node>& node)
{
    auto op = as_type_ptr<op::v0::QuantizedDot>(node);
    const Shape as = node->get_input_shape(0), bs = node->get_input_shape(1);
    const element::Type& bt = node->get_input_element_type(1);
    if (node->get_input_element_type(0) != element::u8 || (bt != element::i8 && bt != element::u8))
        unsupported(*node, "input0 must be u8 and input1 i8 or u8");
    const int operands = B200_U8 | (bt == element::u8 ? B200_WEIGHTS_U8 : 0);
    if (as.size() != 2 || bs.size() != 2 || op->get_reduction_axes_count() != 1 || as[1] % 16 != 0)
        unsupported(*node, "2-D operands with a reduction length that is a multiple of 16");
    int32_t za = 0, zb = 0;
    if (!scalar_zero_point(node->input_value(3), za) || !scalar_zero_point(node->input_value(5), zb))
        unsupported(*node, "input zero points that are not per-tensor constants");
    auto zo = as_constant(node->input_value(7));
    if (!zo)
        unsupported(*node, "output zero point must be a constant");
    int out_t = dtype_of(node->get_output_element_type(0));
    int32_t out_zp = 0;
    if (out_t == B200_U8) out_zp = *static_cast<const uint8_t*>(zo->get_data_ptr());
    else if (out_t == B200_I8) out_zp = *static_cast<const int8_t*>(zo->get_data_ptr());
    else if (out_t == B200_I32) out_zp = *static_cast<const int32_t*>(zo->get_data_ptr());
    else unsupported(*node, "output element type");
    int scale = scalar_product_scale(node->input_value(2), node->input_value(4), node->input_value(6));
    int a = canonical_slot(node->input_value(0));
    int64_t M = as[0], K = as[1], N = bs[1];
    // B [K,N] -> W [N,K]: once at compile time for constants (and into the packed image), one transpose kernel per
    // call otherwise
    int w;
    bool w_image = false;
    const std::string wkey = constant_key("transposed_weight_image", {node->input_value(1).get_node()});
    if (as_constant(node->input_value(1)) && have_saved_constant(wkey))
    {
        w = upload_constant(wkey, nullptr, size_t(b200_packed_weights_bytes(N, K, 128)));
        w_image = true;
    }
    else if (auto cb = as_constant(node->input_value(1)))
    {
        const int8_t* src = static_cast<const int8_t*>(cb->get_data_ptr());
        std::vector<int8_t> t(size_t(N) * K);
        for (int64_t k = 0; k < K; ++k)
            for (int64_t n = 0; n < N; ++n)
                t[n * K + k] = src[k * N + n];
        std::vector<int8_t> image(size_t(b200_packed_weights_bytes(N, K, 128)));
        kernel_check(b200_pack_weights_host(t.data(), image.data(), N, K, 128), "b200_pack_weights_host");
        w = upload_constant(wkey, image.data(), image.size());
        w_image = true;
    }
    else
    {
        int b = canonical_slot(node->input_value(1));
        w = new_slot(Slot::ARENA, size_t(N) * K);
        emit(node, "transpose_b", [=](const Ptrs& p, cudaStream_t st) { return b200_transpose_u8(p[b], p[w], K, N, st); });
    }
    int y = new_slot(Slot::ARENA, shape_size(node->get_output_shape(0)) * node->get_output_element_type(0).size());
    if (za != 0 || zb != 0)
    {
        // sum_k (a - za) * (b - zb) = A.B - zb * rowsum(A) - za * colsum(B) + K * za * zb (zero_points.cu)
        b200_zero_point_params z;
        memset(&z, 0, sizeof(z));
        z.N = 1; z.P = M; z.Q = 1; z.K = N; z.H = M; z.W = 1; z.C = K; z.R = z.S = 1;
        z.stride_h = z.stride_w = z.dilation_h = z.dilation_w = 1;
        z.input_zero_point = za; z.filter_zero_point = zb;
        const int acc = new_slot(Slot::ARENA, size_t(M) * N * 4);
        emit(node, "qgemm_raw", [=](const Ptrs& p, cudaStream_t st) {
            b200_epilogue e;
            memset(&e, 0, sizeof(e));
            e.round_half_away = 2;
            e.out_type = B200_I32;
            return w_image ? b200_qgemm_packed(p[a], operands, static_cast<const int8_t*>(p[w]), p[acc], M, N, K, &e, st)
                           : b200_qgemm(p[a], operands, static_cast<const int8_t*>(p[w]), p[acc], M, N, K, &e, st);
        });
        int cols = -1, rows = -1;
        if (za != 0)
        {
            const int b = canonical_slot(node->input_value(1)); // B as the graph has it: [K, N]
            const int bt_code = bt == element::u8 ? B200_U8 : B200_I8;
            cols = new_slot(Slot::ARENA, size_t(N) * 4);
            emit(node, "column_sums", [=](const Ptrs& p, cudaStream_t st) {
                return b200_strided_sums(p[b], bt_code, static_cast<int32_t*>(p[cols]), N, 1, K, 1, 0, N, st);
            });
        }
        if (zb != 0)
        {
            rows = new_slot(Slot::ARENA, size_t(M) * 4);
            emit(node, "row_sums", [=](const Ptrs& p, cudaStream_t st) {
                return b200_strided_sums(p[a], B200_U8, static_cast<int32_t*>(p[rows]), M, 1, K, K, 0, 1, st);
            });
        }
        emit(node, "requant_zero_points", [=](const Ptrs& p, cudaStream_t st) {
            b200_epilogue e;
            memset(&e, 0, sizeof(e));
            e.scale = static_cast<const float*>(p[scale]);
            e.scale_count = 1;
            e.round_half_away = 1;
            e.out_zero_point = out_zp;
            e.out_type = out_t;
            return b200_requant_zero_points(static_cast<const int32_t*>(p[acc]), cols >= 0 ? static_cast<const int32_t*>(p[cols]) : nullptr,
                                            rows >= 0 ? static_cast<const int32_t*>(p[rows]) : nullptr, &z, &e, p[y], st);
        });
    }
    else
    emit(node, "qgemm_core", [=](const Ptrs& p, cudaStream_t st) {
        b200_epilogue e;
        memset(&e, 0, sizeof(e));
        e.scale = static_cast<const float*>(p[scale]);
        e.scale_count = 1;
        e.round_half_away = 1;
        e.out_zero_point = out_zp;
        e.out_type = out_t;
        return w_image ? b200_qgemm_packed(p[a], operands, static_cast<const int8_t*>(p[w]), p[y], M, N, K, &e, st)
                       : b200_qgemm(p[a], operands, static_cast<const int8_t*>(p[w]), p[y], M, N, K, &e, st);
    });
    value_of(node->output(0)).canonical = y;
}

void B200Executable::compile_max_pool(const std::shared_ptr<Node>& node)
{
    auto op = as_type_ptr<op::v0::MaxPool>(node);
    const Shape is = node->get_input_shape(0), os = node->get_output_shape(0);
    const bool is_signed = node->get_input_element_type(0) == element::i8;
    if ((node->get_input_element_type(0) != element::u8 && !is_signed) || is.size() != 4 || is[1] % 16 != 0)
        unsupported(*node, "u8 / i8 NCHW input with a multiple of 16 channels");
    int x = nhwc_slot(node->input_value(0));
    int y = new_slot(Slot::ARENA, shape_size(os));
    int64_t N = is[0], C = is[1], H = is[2], W = is[3];
    int64_t wh = op->get_window_shape()[0], ww = op->get_window_shape()[1];
    int64_t sh = op->get_window_movement_strides()[0], sw = op->get_window_movement_strides()[1];
    int64_t pb0 = op->get_padding_below()[0], pb1 = op->get_padding_below()[1];
    int64_t pa0 = op->get_padding_above()[0], pa1 = op->get_padding_above()[1];
    // The kernel derives the output extent from the padded input with the floor formula.  In ceil mode the node's output
    // may have one more row / column whose window hangs over the padded input; taps outside the image are skipped either
    // way (reference::max_pool only visits source coordinates that exist), so padding above is widened until the floor
    // formula gives the node's own output shape.
    const int64_t need0 = (int64_t(os[2]) - 1) * sh + wh - H - pb0, need1 = (int64_t(os[3]) - 1) * sw + ww - W - pb1;
    if (need0 > pa0) pa0 = need0;
    if (need1 > pa1) pa1 = need1;
    if ((H + pb0 + pa0 - wh) / sh + 1 != int64_t(os[2]) || (W + pb1 + pa1 - ww) / sw + 1 != int64_t(os[3]))
        unsupported(*node, "an output shape the pooling geometry does not produce");
    emit(node, "maxpool", [=](const Ptrs& p, cudaStream_t st) {
        return is_signed ? b200_maxpool_nhwc_i8(p[x], p[y], N, H, W, C, wh, ww, sh, sw, pb0, pb1, pa0, pa1, st)
                         : b200_maxpool_nhwc_u8(p[x], p[y], N, H, W, C, wh, ww, sh, sw, pb0, pb1, pa0, pa1, st);
    });
    value_of(node->output(0)).nhwc = y;
}

// ------------------------------------------------------------------------------------ executable: call
bool B200Executable::call(const std::vector<std::shared_ptr<runtime::Tensor>>& outputs,
                          const std::vector<std::shared_ptr<runtime::Tensor>>& inputs)
{
    std::lock_guard<std::mutex> lock(m_call_mutex);
    // Chrome-trace events like the INTERPRETER's (int_executable.cpp:122,171), written when NGRAPH_ENABLE_TRACING is set:
    // one for the call and one per lowered step.  Kernels are asynchronous, so with tracing on each step is followed by
    // a stream synchronisation: the step's event then spans its device time, and the call is no longer asynchronous.
    const bool tracing = event::Manager::is_tracing_enabled();
    event::Duration call_event("call", "B200");
    m_ctx->make_current();
    if (inputs.size() != m_function->get_parameters().size() || outputs.size() != m_function->get_results().size())
        throw std::runtime_error("B200 backend: call() tensor count does not match the Function");
    Ptrs ptrs(m_slots.size(), nullptr);
    for (size_t i = 0; i < m_slots.size(); ++i)
    {
        const Slot& s = m_slots[i];
        switch (s.kind)
        {
        case Slot::ARENA: ptrs[i] = static_cast<char*>(m_arena) + s.offset; break;
        case Slot::CONSTANT: ptrs[i] = static_cast<char*>(m_constants) + s.offset; break;
        case Slot::PARAMETER:
        case Slot::RESULT:
        {
            auto t = std::dynamic_pointer_cast<B200Tensor>(s.kind == Slot::PARAMETER ? inputs[s.index] : outputs[s.index]);
            if (!t)
                throw std::invalid_argument("B200 backend: call() was given a tensor that another backend created");
            if (t->context()->device != m_ctx->device)
                throw std::invalid_argument("B200 backend: tensor lives on another device");
            if (t->get_size_in_bytes() < s.bytes)
                throw std::invalid_argument("B200 backend: tensor smaller than the Function's parameter/result");
            ptrs[i] = t->device_ptr();
            break;
        }
        }
    }
    cudaStream_t st = m_ctx->stream;
    for (size_t i = 0; i < m_steps.size(); ++i)
    {
        if (m_perf) cudaEventRecord(m_events[2 * i], st);
        if (tracing)
        {
            event::Duration step_event(m_steps[i].node->description(), "B200",
                                       "{\"name\": \"" + m_steps[i].node->get_name() + "\", \"kernel\": \"" + m_steps[i].what + "\"}");
            kernel_check(m_steps[i].run(ptrs, st), m_steps[i].what + " for " + m_steps[i].node->get_name());
            cuda_check(cudaStreamSynchronize(st), "cudaStreamSynchronize");
        }
        else
            kernel_check(m_steps[i].run(ptrs, st), m_steps[i].what + " for " + m_steps[i].node->get_name());
        if (m_perf) cudaEventRecord(m_events[2 * i + 1], st);
    }
    for (auto& rc : m_result_copies)
        if (ptrs[rc.first] != ptrs[rc.second])
            cuda_check(cudaMemcpyAsync(ptrs[rc.second], ptrs[rc.first], m_slots[rc.second].bytes, cudaMemcpyDeviceToDevice, st),
                       "result copy");
    if (m_perf)
    {
        m_ctx->synchronize();
        for (size_t i = 0; i < m_steps.size(); ++i)
        {
            float ms = 0;
            cudaEventElapsedTime(&ms, m_events[2 * i], m_events[2 * i + 1]);
            m_step_us[i] += ms * 1000.0;
        }
        ++m_calls;
    }
    // no synchronisation here: Tensor::read() / write() order themselves after this call through the tensor
    for (auto& t : inputs)
        if (auto bt = std::dynamic_pointer_cast<B200Tensor>(t))
            bt->mark_used(st);
    for (auto& t : outputs)
        if (auto bt = std::dynamic_pointer_cast<B200Tensor>(t))
            bt->mark_used(st);
    return true;
}

// Executable::save (src/ngraph/runtime/executable.hpp:76-78): a cpio archive like the INTERPRETER's
// (int_executable.cpp:345-352), holding what compile() produced so that Backend::load does not redo it:
//   save_info  format tag
//   model      the Function after the plugin's graph passes, in the plugin's own binary form (function_io.hpp)
//   constants  the device constant image: packed filter / weight images, folded scales, plain constants, at the offsets
//              the lowering assigned
//   meta       text: hashes of the two entries above, arena size and the lowered step list
void B200Executable::save(std::ostream& out)
{
    std::lock_guard<std::mutex> lock(m_call_mutex);
    m_ctx->make_current();
    const std::string model = write_function(*m_function);
    std::vector<char> constants(m_constant_bytes);
    if (m_constant_bytes)
    {
        cuda_check(cudaStreamSynchronize(m_ctx->stream), "cudaStreamSynchronize");
        cuda_check(cudaMemcpy(constants.data(), m_constants, m_constant_bytes, cudaMemcpyDeviceToHost), "cudaMemcpy(constants -> host)");
    }
    std::ostringstream meta;
    meta << "model_fnv1a " << fnv1a(model.data(), model.size()) << "\nconstants_fnv1a " << fnv1a(constants.data(), constants.size())
         << "\narena_bytes " << m_arena_bytes << "\nsteps " << m_steps.size() << "\n";
    for (const auto& st : m_steps)
        meta << st.what << " " << st.node->get_name() << "\n";
    const std::string meta_text = meta.str();
    cpio::Writer writer(out);
    writer.write("save_info", SAVE_INFO, uint32_t(strlen(SAVE_INFO)));
    writer.write("model", model.data(), uint32_t(model.size()));
    if (constants.size() >= (size_t(1) << 32) || model.size() >= (size_t(1) << 32))
        throw std::runtime_error("B200 backend: executable too large for the cpio container (4 GiB per entry)");
    writer.write("constants", constants.data(), uint32_t(constants.size()));
    std::ostringstream index; // key, offset and size of every constant inside the image
    for (const auto& e : m_constant_index)
        index << e.first << " " << e.second.first << " " << e.second.second << "\n";
    const std::string index_text = index.str();
    writer.write("constants_index", index_text.data(), uint32_t(index_text.size()));
    writer.write("meta", meta_text.data(), uint32_t(meta_text.size()));
}

// Backend::load (src/ngraph/runtime/backend.hpp:122-125; INTERPRETER: int_backend.cpp:81-110)
std::shared_ptr<runtime::Executable> B200Backend::load(std::istream& in)
{
    cpio::Reader reader(in);
    std::string info, model, meta, index_text;
    std::vector<char> constants;
    bool have_constants = false;
    for (const cpio::FileInfo& f : reader.get_file_info())
    {
        if (f.get_name() == "save_info" || f.get_name() == "model" || f.get_name() == "meta" || f.get_name() == "constants_index")
        {
            std::vector<char> b = reader.read(f);
            (f.get_name() == "save_info" ? info : f.get_name() == "model" ? model : f.get_name() == "meta" ? meta : index_text)
                .assign(b.data(), b.size());
        }
        else if (f.get_name() == "constants")
        {
            constants = reader.read(f);
            have_constants = true;
        }
    }
    if (info != SAVE_INFO)
        throw std::runtime_error("B200 backend: not an executable saved by this plugin version (save_info '" + info + "')");
    if (model.empty() || !have_constants)
        throw std::runtime_error("B200 backend: saved executable lacks its model or its constant image");
    // the hashes in `meta` tie the two entries to each other
    {
        std::istringstream ms(meta);
        std::string key;
        uint64_t value = 0, want_model = 0, want_constants = 0;
        while (ms >> key >> value)
        {
            if (key == "model_fnv1a") want_model = value;
            else if (key == "constants_fnv1a") want_constants = value;
            else if (key == "steps") break;
        }
        if (want_model != fnv1a(model.data(), model.size()) || want_constants != fnv1a(constants.data(), constants.size()))
            throw std::runtime_error("B200 backend: saved executable is damaged (hash mismatch)");
    }
    std::map<std::string, std::pair<size_t, size_t>> index;
    {
        std::istringstream is(index_text);
        std::string key;
        size_t offset = 0, bytes = 0;
        while (is >> key >> offset >> bytes)
            index[key] = std::make_pair(offset, bytes);
    }
    // nodes are rebuilt in the saved order, which is the order the keys of the index count in
    std::vector<std::shared_ptr<Node>> order;
    std::shared_ptr<Function> function = read_function(model, &order);
    std::lock_guard<std::mutex> lock(m_mutex);
    return std::make_shared<B200Executable>(m_ctx, function, false, &constants, &index, &order);
}

std::vector<runtime::PerformanceCounter> B200Executable::get_performance_data() const
{
    std::vector<runtime::PerformanceCounter> rc;
    std::map<const Node*, size_t> index;
    for (size_t i = 0; i < m_steps.size(); ++i)
    {
        const Node* n = m_steps[i].node.get();
        size_t us = m_perf ? size_t(m_step_us[i]) : 0;
        auto it = index.find(n);
        if (it == index.end())
        {
            index[n] = rc.size();
            rc.emplace_back(m_steps[i].node, us, m_calls);
        }
        else
            rc[it->second].m_total_microseconds += us;
    }
    return rc;
}

std::shared_ptr<runtime::Tensor> B200Executable::create_input_tensor(size_t input_index)
{
    auto p = get_parameters().at(input_index);
    return std::make_shared<B200Tensor>(m_ctx, p->get_output_element_type(0), p->get_output_shape(0));
}

std::shared_ptr<runtime::Tensor> B200Executable::create_output_tensor(size_t output_index)
{
    auto r = get_results().at(output_index);
    return std::make_shared<B200Tensor>(m_ctx, r->get_output_element_type(0), r->get_output_shape(0));
}

std::vector<std::shared_ptr<runtime::Tensor>> B200Executable::create_input_tensor(size_t input_index, size_t pipeline_depth)
{
    std::vector<std::shared_ptr<runtime::Tensor>> v;
    for (size_t i = 0; i < pipeline_depth; ++i)
        v.push_back(create_input_tensor(input_index));
    return v;
}

std::vector<std::shared_ptr<runtime::Tensor>> B200Executable::create_output_tensor(size_t output_index, size_t pipeline_depth)
{
    std::vector<std::shared_ptr<runtime::Tensor>> v;
    for (size_t i = 0; i < pipeline_depth; ++i)
        v.push_back(create_output_tensor(output_index));
    return v;
}

// Multi-device backend option (see multi_device.hpp).
#include "multi_device.hpp"

#include <sstream>

#include "b200_kernels.h"
#include "function_io.hpp"
#include "graph_passes.hpp"
#include "ngraph/cpio.hpp"
#include "ngraph/descriptor/layout/dense_tensor_layout.hpp"
#include "ngraph/graph_util.hpp"

using namespace ngraph;
using namespace ngraph::runtime::b200;

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
}

// ------------------------------------------------------------------------------------ tensor
ShardedTensor::ShardedTensor(const std::vector<std::shared_ptr<DeviceContext>>& devices, const element::Type& type, const Shape& shape)
    : runtime::Tensor(std::make_shared<descriptor::Tensor>(type, shape, "external"))
{
    m_descriptor->set_tensor_layout(std::make_shared<descriptor::layout::DenseTensorLayout>(*m_descriptor));
    m_bytes = shape_size(shape) * type.size();
    m_rows = shape.empty() ? 1 : shape[0];
    m_row_bytes = m_rows ? m_bytes / m_rows : 0;
    for (const auto& ctx : devices)
        m_parts.push_back(std::make_shared<B200Tensor>(ctx, type, shape));
}

void ShardedTensor::prefer_rows(const std::vector<size_t>& begin)
{
    std::lock_guard<std::mutex> lock(m_mutex);
    m_preferred = begin;
}

void ShardedTensor::set_valid_rows(const std::vector<size_t>& begin)
{
    std::lock_guard<std::mutex> lock(m_mutex);
    m_valid = begin;
}

bool ShardedTensor::holds(size_t d, size_t from, size_t to) const
{
    std::lock_guard<std::mutex> lock(m_mutex);
    return m_valid.empty() || (m_valid[d] <= from && to <= m_valid[d + 1]) || from >= to;
}

void ShardedTensor::write(const void* p, size_t n)
{
    if (n > m_bytes)
        throw std::out_of_range("B200 tensor write: access past the end of the tensor");
    std::lock_guard<std::mutex> lock(m_mutex);
    const char* src = static_cast<const char*>(p);
    if (n == m_bytes && !m_preferred.empty())
    {
        // each device gets the rows it works on; all the copies are in flight together
        for (size_t d = 0; d < m_parts.size(); ++d)
        {
            const size_t off = m_preferred[d] * m_row_bytes, len = (m_preferred[d + 1] - m_preferred[d]) * m_row_bytes;
            if (len)
                m_parts[d]->write_async(src + off, off, len);
        }
        for (auto& part : m_parts)
            part->finish_copies();
        m_valid = m_preferred;
        return;
    }
    for (auto& part : m_parts)
        part->write_async(src, 0, n);
    for (auto& part : m_parts)
        part->finish_copies();
    if (n == m_bytes)
        m_valid.clear(); // the whole tensor, everywhere
}

void ShardedTensor::read(void* p, size_t n) const
{
    if (n > m_bytes)
        throw std::out_of_range("B200 tensor read: access past the end of the tensor");
    std::lock_guard<std::mutex> lock(m_mutex);
    char* dst = static_cast<char*>(p);
    if (m_valid.empty())
    {
        m_parts[0]->read_async(dst, 0, n);
        m_parts[0]->finish_copies();
        return;
    }
    for (size_t d = 0; d < m_parts.size(); ++d)
    {
        const size_t off = m_valid[d] * m_row_bytes, end = std::min(n, m_valid[d + 1] * m_row_bytes);
        if (off < end)
            m_parts[d]->read_async(dst + off, off, end - off);
    }
    for (auto& part : m_parts)
        part->finish_copies();
}

void ShardedTensor::make_whole_everywhere()
{
    std::lock_guard<std::mutex> lock(m_mutex);
    if (m_valid.empty())
        return;
    // every member device idle: the copies below then need no ordering against work in flight
    for (auto& part : m_parts)
        part->context()->synchronize();
    for (size_t d = 0; d < m_parts.size(); ++d)
    {
        const size_t off = m_valid[d] * m_row_bytes, len = (m_valid[d + 1] - m_valid[d]) * m_row_bytes;
        if (!len)
            continue;
        for (size_t e = 0; e < m_parts.size(); ++e)
            if (e != d && m_parts[e]->device_ptr() != m_parts[d]->device_ptr())
                cuda_check(cudaMemcpyPeer(static_cast<char*>(m_parts[e]->device_ptr()) + off, m_parts[e]->context()->device,
                                          static_cast<const char*>(m_parts[d]->device_ptr()) + off, m_parts[d]->context()->device, len),
                           "cudaMemcpyPeer");
    }
    m_valid.clear();
}

// ------------------------------------------------------------------------------------ issuing threads
IssueThread::IssueThread()
    : m_thread([this] { loop(); })
{
}

IssueThread::~IssueThread()
{
    {
        std::lock_guard<std::mutex> lock(m_mutex);
        m_stop = true;
    }
    m_wake.notify_all();
    m_thread.join();
}

void IssueThread::post(std::function<void()> work)
{
    {
        std::lock_guard<std::mutex> lock(m_mutex);
        m_queue.push_back(std::move(work));
    }
    m_wake.notify_one();
}

void IssueThread::wait()
{
    std::unique_lock<std::mutex> lock(m_mutex);
    m_idle.wait(lock, [this] { return m_queue.empty() && !m_busy; });
    if (m_error)
    {
        std::exception_ptr e = m_error;
        m_error = nullptr;
        std::rethrow_exception(e);
    }
}

void IssueThread::loop()
{
    std::unique_lock<std::mutex> lock(m_mutex);
    for (;;)
    {
        m_wake.wait(lock, [this] { return m_stop || !m_queue.empty(); });
        if (m_queue.empty())
            return; // stopping
        std::function<void()> work = std::move(m_queue.front());
        m_queue.pop_front();
        m_busy = true;
        lock.unlock();
        std::exception_ptr error;
        try
        {
            work();
        }
        catch (...)
        {
            error = std::current_exception();
        }
        lock.lock();
        m_busy = false;
        if (error && !m_error)
            m_error = error;
        if (m_queue.empty())
            m_idle.notify_all();
    }
}

// ------------------------------------------------------------------------------------ executable
ShardedExecutable::ShardedExecutable(const std::vector<std::shared_ptr<B200Backend>>& members, const std::shared_ptr<Function>& func,
                                     bool enable_performance_data)
    : m_members(members)
    , m_function(func)
{
    set_parameters_and_results(*func);
    for (const auto& m : m_members)
        m_devices.push_back(m->context());
    const size_t D = m_members.size();
    if (D > 1)
    {
        // the split is decided on the graph the devices will lower: after the plugin's own passes
        std::shared_ptr<Function> lowered = clone_function(*func);
        run_graph_passes(lowered);
        m_batch = batch_of(*lowered);
        if (m_batch < 2)
            m_why = "a batch of fewer than two samples";
        else
        {
            // balanced shares: the first (batch % D) members take one sample more; with fewer samples than members the last
            // members take none and stay idle
            const size_t lo = m_batch / D, extra = m_batch % D;
            BatchSplit more, fewer;
            const bool ok = (extra == 0 || split_batch(*lowered, lo + 1, more, m_why)) && (lo == 0 || split_batch(*lowered, lo, fewer, m_why));
            if (ok)
            {
                m_split = true;
                m_parameter_split = extra ? more.parameter_split : fewer.parameter_split;
                m_result_split = extra ? more.result_split : fewer.result_split;
                m_begin.push_back(0);
                for (size_t d = 0; d < D; ++d)
                    m_begin.push_back(m_begin.back() + lo + (d < extra ? 1 : 0));
                for (size_t d = 0; d < D; ++d)
                {
                    const size_t rows = m_begin[d + 1] - m_begin[d];
                    m_subs.push_back(rows == 0 ? nullptr
                                               : m_members[d]->compile(rows == lo + 1 && extra ? more.function : fewer.function, enable_performance_data));
                    m_threads.emplace_back(rows == 0 ? nullptr : new IssueThread());
                }
            }
        }
    }
    if (!m_split)
        m_subs.push_back(m_members[0]->compile(func, enable_performance_data));
}

std::vector<size_t> ShardedExecutable::tensor_rows(const ShardedTensor& t) const
{
    // a batch-carrying tensor's leading extent is a multiple of the batch (batch-major rows)
    const size_t k = t.rows() / m_batch;
    std::vector<size_t> v;
    for (size_t b : m_begin)
        v.push_back(b * k);
    return v;
}

std::shared_ptr<runtime::Tensor> ShardedExecutable::view(size_t d, const ShardedTensor& t, const Shape& shard_shape, size_t row0)
{
    void* p = static_cast<char*>(t.part(d)->device_ptr()) + row0 * t.row_bytes();
    const auto key = std::make_tuple(d, static_cast<const void*>(p), shape_size(shard_shape) * t.get_element_type().size());
    auto it = m_views.find(key);
    if (it != m_views.end())
        return it->second;
    if (m_views.size() >= 4096)
        m_views.clear(); // views of tensors long gone; the ones a call is using are held by that call
    auto v = std::make_shared<B200Tensor>(m_devices[d], t.get_element_type(), shard_shape, p);
    m_views.emplace(key, v);
    return v;
}

bool ShardedExecutable::call(const std::vector<std::shared_ptr<runtime::Tensor>>& outputs,
                             const std::vector<std::shared_ptr<runtime::Tensor>>& inputs)
{
    std::lock_guard<std::mutex> lock(m_call_mutex);
    if (inputs.size() != get_parameters().size() || outputs.size() != get_results().size())
        throw std::runtime_error("B200 backend: call() tensor count does not match the Function");
    std::vector<std::shared_ptr<ShardedTensor>> ins, outs;
    for (const auto& t : inputs)
        ins.push_back(std::dynamic_pointer_cast<ShardedTensor>(t));
    for (const auto& t : outputs)
        outs.push_back(std::dynamic_pointer_cast<ShardedTensor>(t));
    for (size_t i = 0; i < ins.size() + outs.size(); ++i)
    {
        const auto& t = i < ins.size() ? ins[i] : outs[i - ins.size()];
        if (!t || t->devices() != m_members.size())
            throw std::invalid_argument("B200 backend: call() was given a tensor that another backend created");
        for (size_t d = 0; d < m_members.size(); ++d)
            if (t->part(d)->context()->device != m_devices[d]->device)
                throw std::invalid_argument("B200 backend: tensor lives on other devices");
    }
    const size_t D = m_members.size();
    if (!m_split)
    {
        // whole Function on the first member device
        std::vector<std::shared_ptr<runtime::Tensor>> in0, out0;
        for (auto& t : ins)
        {
            if (!t->holds(0, 0, t->rows()))
                t->make_whole_everywhere();
            in0.push_back(t->part(0));
        }
        for (auto& t : outs)
            out0.push_back(t->part(0));
        m_subs[0]->call(out0, in0);
        for (auto& t : outs)
        {
            std::vector<size_t> only_first(D + 1, t->rows());
            only_first[0] = 0;
            t->set_valid_rows(only_first);
        }
        return true;
    }
    // per device: the rows it works on, as single-device tensors over slices of the members' buffers
    std::vector<std::vector<std::shared_ptr<runtime::Tensor>>> in_d(D), out_d(D);
    for (size_t i = 0; i < ins.size(); ++i)
    {
        ShardedTensor& t = *ins[i];
        if (!m_parameter_split[i])
        {
            for (size_t d = 0; d < D; ++d)
                if (!t.holds(d, 0, t.rows()))
                    t.make_whole_everywhere();
            for (size_t d = 0; d < D; ++d)
                in_d[d].push_back(t.part(d));
            continue;
        }
        if (t.rows() % m_batch != 0 || t.get_shape() != get_parameters()[i]->get_output_shape(0))
            throw std::invalid_argument("B200 backend: input tensor shape does not match the Function's parameter");
        const std::vector<size_t> rows = tensor_rows(t);
        for (size_t d = 0; d < D; ++d)
            if (!t.holds(d, rows[d], rows[d + 1]))
                t.make_whole_everywhere();
        t.prefer_rows(rows); // from now on write() sends each device its rows only
        for (size_t d = 0; d < D; ++d)
        {
            if (!m_subs[d])
                continue;
            Shape s = t.get_shape();
            s[0] = rows[d + 1] - rows[d];
            in_d[d].push_back(view(d, t, s, rows[d]));
        }
    }
    for (size_t i = 0; i < outs.size(); ++i)
    {
        ShardedTensor& t = *outs[i];
        if (t.rows() % m_batch != 0 || t.get_shape() != get_results()[i]->get_output_shape(0))
            throw std::invalid_argument("B200 backend: output tensor shape does not match the Function's result");
        const std::vector<size_t> rows = tensor_rows(t);
        for (size_t d = 0; d < D; ++d)
        {
            if (!m_subs[d])
                continue;
            Shape s = t.get_shape();
            s[0] = rows[d + 1] - rows[d];
            out_d[d].push_back(view(d, t, s, rows[d]));
        }
    }
    // all devices at once: each member's launches are issued by its own thread (a call only enqueues)
    for (size_t d = 0; d < D; ++d)
    {
        if (!m_subs[d])
            continue; // fewer samples than members: this one has no share
        m_threads[d]->post([this, d, &in_d, &out_d, &ins, &outs] {
            m_subs[d]->call(out_d[d], in_d[d]);
            // copies of the whole tensors (write / read) order themselves after this call on this device
            for (auto& t : ins)
                t->part(d)->mark_used(m_devices[d]->stream);
            for (auto& t : outs)
                t->part(d)->mark_used(m_devices[d]->stream);
        });
    }
    std::exception_ptr first;
    for (size_t d = 0; d < D; ++d)
    {
        try
        {
            if (m_threads[d])
                m_threads[d]->wait();
        }
        catch (...)
        {
            if (!first)
                first = std::current_exception();
        }
    }
    if (first)
        std::rethrow_exception(first);
    for (auto& t : outs)
        t->set_valid_rows(tensor_rows(*t));
    return true;
}

std::vector<runtime::PerformanceCounter> ShardedExecutable::get_performance_data() const
{
    return m_subs[0]->get_performance_data(); // the first member's view (every member with a share runs the same steps)
}

void ShardedExecutable::save(std::ostream& out)
{
    if (!m_split)
        return m_subs[0]->save(out);
    auto whole = m_members[0]->compile(m_function, false);
    whole->save(out);
    m_members[0]->remove_compiled_function(whole);
}

std::shared_ptr<runtime::Tensor> ShardedExecutable::create_input_tensor(size_t input_index)
{
    auto p = get_parameters().at(input_index);
    auto t = std::make_shared<ShardedTensor>(m_devices, p->get_output_element_type(0), p->get_output_shape(0));
    if (m_split && m_parameter_split[input_index])
        t->prefer_rows(tensor_rows(*t));
    return t;
}

std::shared_ptr<runtime::Tensor> ShardedExecutable::create_output_tensor(size_t output_index)
{
    auto r = get_results().at(output_index);
    return std::make_shared<ShardedTensor>(m_devices, r->get_output_element_type(0), r->get_output_shape(0));
}

std::vector<std::shared_ptr<runtime::Tensor>> ShardedExecutable::create_input_tensor(size_t input_index, size_t pipeline_depth)
{
    std::vector<std::shared_ptr<runtime::Tensor>> v;
    for (size_t i = 0; i < pipeline_depth; ++i)
        v.push_back(create_input_tensor(input_index));
    return v;
}

std::vector<std::shared_ptr<runtime::Tensor>> ShardedExecutable::create_output_tensor(size_t output_index, size_t pipeline_depth)
{
    std::vector<std::shared_ptr<runtime::Tensor>> v;
    for (size_t i = 0; i < pipeline_depth; ++i)
        v.push_back(create_output_tensor(output_index));
    return v;
}

// ------------------------------------------------------------------------------------ backend
bool ShardedBackend::wants(const std::string& options)
{
    return options == "all" || options.find('+') != std::string::npos;
}

ShardedBackend::ShardedBackend(const std::string& options)
{
    std::vector<int> ordinals;
    if (options == "all")
    {
        int count = 0;
        cuda_check(cudaGetDeviceCount(&count), "cudaGetDeviceCount");
        for (int d = 0; d < count; ++d)
            ordinals.push_back(d);
    }
    else
    {
        std::stringstream ss(options);
        std::string item;
        while (std::getline(ss, item, '+'))
        {
            try
            {
                size_t used = 0;
                ordinals.push_back(std::stoi(item, &used));
                if (used != item.size())
                    throw std::invalid_argument(item);
            }
            catch (...)
            {
                throw std::runtime_error("B200 backend: bad option '" + options + "' (expected 'all' or '<device>+<device>...')");
            }
        }
    }
    if (ordinals.empty())
        throw std::runtime_error("B200 backend: no CUDA device");
    for (int d : ordinals)
    {
        m_members.push_back(std::make_shared<B200Backend>(std::to_string(d)));
        m_devices.push_back(m_members.back()->context());
    }
}

std::shared_ptr<runtime::Tensor> ShardedBackend::create_tensor()
{
    throw std::runtime_error("B200 backend does not support dynamic tensors");
}

std::shared_ptr<runtime::Tensor> ShardedBackend::create_tensor(const element::Type& type, const Shape& shape)
{
    return std::make_shared<ShardedTensor>(m_devices, type, shape);
}

std::shared_ptr<runtime::Tensor> ShardedBackend::create_tensor(const element::Type&, const Shape&, void*)
{
    throw std::runtime_error("B200 backend: a tensor over caller-owned memory belongs to one device; create it with "
                             "Backend::create(\"B200:<device>\")");
}

std::shared_ptr<runtime::Executable> ShardedBackend::compile(std::shared_ptr<Function> func, bool enable_performance_data)
{
    std::lock_guard<std::mutex> lock(m_mutex);
    const auto key = std::make_pair(func, enable_performance_data);
    auto it = m_cache.find(key);
    if (it != m_cache.end())
        return it->second;
    auto exec = std::make_shared<ShardedExecutable>(m_members, func, enable_performance_data);
    m_cache.insert({key, exec});
    return exec;
}

std::shared_ptr<runtime::Executable> ShardedBackend::load(std::istream& in)
{
    cpio::Reader reader(in);
    std::string info, model;
    for (const cpio::FileInfo& f : reader.get_file_info())
        if (f.get_name() == "save_info" || f.get_name() == "model")
        {
            std::vector<char> b = reader.read(f);
            (f.get_name() == "save_info" ? info : model).assign(b.data(), b.size());
        }
    if (info != SAVE_INFO)
        throw std::runtime_error("B200 backend: not an executable saved by this plugin version (save_info '" + info + "')");
    if (model.empty())
        throw std::runtime_error("B200 backend: saved executable lacks its model");
    return compile(read_function(model));
}

bool ShardedBackend::is_supported(const Node& node) const
{
    return m_members[0]->is_supported(node);
}

void ShardedBackend::remove_compiled_function(std::shared_ptr<runtime::Executable> exec)
{
    std::lock_guard<std::mutex> lock(m_mutex);
    for (auto it = m_cache.begin(); it != m_cache.end(); ++it)
        if (it->second == exec)
        {
            m_cache.erase(it);
            break;
        }
}

// The multi-device form of the backend: Backend::create("B200:all") or Backend::create("B200:0+1+2") (the text after ':'
// is nGraph's backend option string, src/ngraph/runtime/backend_manager.cpp:83-89,141).  One Backend, one Executable and
// one Tensor per logical object, as for a single device; behind them one B200Backend / B200Executable / B200Tensor per
// member device.  compile() splits the Function along the batch (batch_split.hpp), every device gets the same graph for
// its contiguous share of the rows, constants replicated; call() hands every batch-carrying tensor to the devices by
// rows and enqueues all the sub-executables at once.  Nothing crosses between devices on the data path: Tensor::write
// sends each device its rows, Tensor::read collects them.  A Function that cannot be split runs whole on the first
// member device.
#pragma once

#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <thread>
#include <tuple>

#include "b200_backend.hpp"
#include "batch_split.hpp"

namespace ngraph
{
    namespace runtime
    {
        namespace b200
        {
            /// One logical tensor with a full-size buffer on every member device.  Either the whole tensor is valid on
            /// every device, or device d holds rows [m_valid[d], m_valid[d + 1]) of the leading axis at their place.
            class ShardedTensor : public runtime::Tensor
            {
            public:
                ShardedTensor(const std::vector<std::shared_ptr<DeviceContext>>& devices, const element::Type& type, const Shape& shape);
                void write(const void* p, size_t n) override;
                void read(void* p, size_t n) const override;

                size_t devices() const { return m_parts.size(); }
                const std::shared_ptr<B200Tensor>& part(size_t d) const { return m_parts[d]; }
                size_t rows() const { return m_rows; }
                size_t row_bytes() const { return m_row_bytes; }
                /// later whole-tensor write()s send device d rows [begin[d], begin[d + 1]) only
                void prefer_rows(const std::vector<size_t>& begin);
                /// a call() has written these rows on these devices (and nothing else of the tensor is valid)
                void set_valid_rows(const std::vector<size_t>& begin);
                /// does device d hold rows [from, to)
                bool holds(size_t d, size_t from, size_t to) const;
                /// peer copies until every device holds the whole tensor (synchronises the member devices: the slow path
                /// for a tensor that one Function produced by rows and another consumes whole)
                void make_whole_everywhere();

            private:
                std::vector<std::shared_ptr<B200Tensor>> m_parts;
                size_t m_rows = 1, m_row_bytes = 0, m_bytes = 0;
                std::vector<size_t> m_valid;     // empty: whole tensor on every device
                std::vector<size_t> m_preferred; // empty: write() sends everything to every device
                mutable std::mutex m_mutex;
            };

            /// one thread that runs closures in order (one per member device: a device's launches are issued by its own thread)
            class IssueThread
            {
            public:
                IssueThread();
                ~IssueThread();
                void post(std::function<void()> work);
                void wait(); // until everything posted has run; rethrows the first exception of the batch
            private:
                void loop();
                std::mutex m_mutex;
                std::condition_variable m_wake, m_idle;
                std::deque<std::function<void()>> m_queue;
                bool m_stop = false, m_busy = false;
                std::exception_ptr m_error;
                std::thread m_thread;
            };

            class ShardedBackend;

            class ShardedExecutable : public runtime::Executable
            {
            public:
                ShardedExecutable(const std::vector<std::shared_ptr<B200Backend>>& members, const std::shared_ptr<Function>& func,
                                  bool enable_performance_data);
                bool call(const std::vector<std::shared_ptr<runtime::Tensor>>& outputs,
                          const std::vector<std::shared_ptr<runtime::Tensor>>& inputs) override;
                std::vector<PerformanceCounter> get_performance_data() const override;
                /// the archive a single-device executable of the whole Function writes (compiled on the first member for the
                /// purpose): either form of the backend can load it
                void save(std::ostream& output_stream) override;
                std::shared_ptr<runtime::Tensor> create_input_tensor(size_t input_index) override;
                std::shared_ptr<runtime::Tensor> create_output_tensor(size_t output_index) override;
                std::vector<std::shared_ptr<runtime::Tensor>> create_input_tensor(size_t input_index, size_t pipeline_depth) override;
                std::vector<std::shared_ptr<runtime::Tensor>> create_output_tensor(size_t output_index, size_t pipeline_depth) override;
                /// number of devices the Function runs on (1 when it could not be split) and, then, why
                size_t shards() const { return m_split ? m_members.size() : 1; }
                const std::string& why_not_split() const { return m_why; }

            private:
                std::vector<size_t> tensor_rows(const ShardedTensor& t) const; // m_begin scaled to t's leading extent
                std::shared_ptr<runtime::Tensor> view(size_t d, const ShardedTensor& t, const Shape& shard_shape, size_t row0);

                std::vector<std::shared_ptr<B200Backend>> m_members;
                std::vector<std::shared_ptr<DeviceContext>> m_devices;
                std::shared_ptr<Function> m_function;                     // as given to compile()
                std::vector<std::shared_ptr<runtime::Executable>> m_subs; // per member device, or one
                std::vector<std::unique_ptr<IssueThread>> m_threads;
                bool m_split = false;
                std::string m_why;
                size_t m_batch = 0;
                std::vector<size_t> m_begin; // device d takes samples [m_begin[d], m_begin[d + 1])
                std::vector<bool> m_parameter_split, m_result_split;
                // non-owning single-device tensors over a slice of a ShardedTensor's buffer, by (device, address, bytes)
                std::map<std::tuple<size_t, const void*, size_t>, std::shared_ptr<runtime::Tensor>> m_views;
                std::mutex m_call_mutex;
            };

            class ShardedBackend : public runtime::Backend
            {
            public:
                /// "all", or device ordinals joined by '+'
                explicit ShardedBackend(const std::string& options);
                static bool wants(const std::string& options);
                std::shared_ptr<runtime::Tensor> create_tensor() override;
                std::shared_ptr<runtime::Tensor> create_tensor(const element::Type& type, const Shape& shape) override;
                std::shared_ptr<runtime::Tensor>
                    create_tensor(const element::Type& type, const Shape& shape, void* memory_pointer) override;
                std::shared_ptr<runtime::Executable> compile(std::shared_ptr<Function> func,
                                                             bool enable_performance_data = false) override;
                bool is_supported(const Node& node) const override;
                void remove_compiled_function(std::shared_ptr<runtime::Executable> exec) override;
                /// rebuilds the saved Function and compiles it for the member devices (the saved constant image belongs to a
                /// whole-batch executable and is not used: every member packs the weights for its share again)
                std::shared_ptr<runtime::Executable> load(std::istream& input_stream) override;
                size_t devices() const { return m_members.size(); }

            private:
                std::vector<std::shared_ptr<B200Backend>> m_members;
                std::vector<std::shared_ptr<DeviceContext>> m_devices;
                std::mutex m_mutex;
                std::map<std::pair<std::shared_ptr<Function>, bool>, std::shared_ptr<runtime::Executable>> m_cache;
            };
        }
    }
}

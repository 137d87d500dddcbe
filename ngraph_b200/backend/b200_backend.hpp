// nGraph runtime backend "B200": runtime::Backend / Executable / Tensor on top of the C ABI of
// include/b200_kernels.h.  Loaded by runtime::BackendManager through
// ngraph_register_b200_backend() (src/ngraph/runtime/backend_manager.cpp:78-142 in nGraph).
//
// Backend options (the text after ':' in Backend::create("B200:<options>")):
// "<CUDA device ordinal>[,stream=<cudaStream_t as an integer>]", default device 0 and a stream of its own; or "all" /
// "<ordinal>+<ordinal>...": several devices behind one Backend (multi_device.hpp).
#pragma once

#include <cuda_runtime.h>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "ngraph/function.hpp"
#include "ngraph/node.hpp"
#include "ngraph/runtime/backend.hpp"
#include "ngraph/runtime/executable.hpp"
#include "ngraph/runtime/performance_counter.hpp"
#include "ngraph/runtime/tensor.hpp"

#define B200_BACKEND_API __attribute__((visibility("default")))

namespace ngraph
{
    namespace runtime
    {
        namespace b200
        {
            // format tag of Executable::save's archive (entry "save_info"); Backend::load refuses any other
            constexpr char SAVE_INFO[] = "B200 Save File 1.0";

            // Per-backend CUDA state: device ordinal and the one stream every tensor copy and
            // kernel of this backend instance is ordered on.
            struct DeviceContext
            {
                int device = 0;
                cudaStream_t stream = nullptr;
                // Tensor::write / read copy on a stream of their own, ordered against the compute stream only through
                // the tensor they touch: a host thread can fill the next input while the previous call still runs
                cudaStream_t copy_stream = nullptr;
                bool owns_stream = true;
                explicit DeviceContext(int dev);
                DeviceContext(int dev, cudaStream_t external); // enqueue on the caller's stream
                ~DeviceContext();
                void make_current() const;
                void synchronize() const; // waits for the stream, then raises on a device status word
            };

            class B200Tensor : public runtime::Tensor
            {
            public:
                B200Tensor(const std::shared_ptr<DeviceContext>& ctx,
                           const element::Type& type,
                           const Shape& shape,
                           void* device_pointer = nullptr);
                ~B200Tensor() override;
                void write(const void* p, size_t n) override;
                void read(void* p, size_t n) const override;
                void copy_from(const runtime::Tensor& source) override;
                void* device_ptr() const { return m_ptr; }
                // The pieces write() / read() are made of, for a caller that keeps copies to several devices in flight at
                // once (the multi-device tensor): enqueue on this tensor's copy stream, then wait for them.
                void write_async(const void* p, size_t offset, size_t n);
                void read_async(void* p, size_t offset, size_t n) const;
                void finish_copies() const; // waits for the copy stream; raises on a device status word
                // orders this tensor's next copies after `event` (recorded on another device's stream)
                void order_copies_after(cudaEvent_t event) const;
                // called by Executable::call after its last kernel: later write()s and read()s of this tensor wait for it
                void mark_used(cudaStream_t compute_stream);
                const std::shared_ptr<DeviceContext>& context() const { return m_ctx; }
            private:
                std::shared_ptr<DeviceContext> m_ctx;
                void* m_ptr = nullptr;
                size_t m_bytes = 0;
                bool m_owned = false;
                cudaEvent_t m_last_use = nullptr; // recorded on the compute stream by the last call() that used the tensor
                void order_copy_after_use() const;
            };

            class B200Executable;

            class B200Backend : public runtime::Backend
            {
            public:
                explicit B200Backend(const std::string& options);
                std::shared_ptr<runtime::Tensor> create_tensor() override;
                std::shared_ptr<runtime::Tensor> create_tensor(const element::Type& type, const Shape& shape) override;
                std::shared_ptr<runtime::Tensor>
                    create_tensor(const element::Type& type, const Shape& shape, void* memory_pointer) override;
                std::shared_ptr<runtime::Executable> compile(std::shared_ptr<Function> func,
                                                             bool enable_performance_data = false) override;
                bool is_supported(const Node& node) const override;
                void remove_compiled_function(std::shared_ptr<runtime::Executable> exec) override;
                std::shared_ptr<runtime::Executable> load(std::istream& input_stream) override;
                bool is_device_memory(void* ptr) override;
                const std::shared_ptr<DeviceContext>& context() const { return m_ctx; }
            private:
                std::shared_ptr<DeviceContext> m_ctx;
                std::mutex m_mutex;
                // one executable per (Function, performance counters on / off)
                std::map<std::pair<std::shared_ptr<Function>, bool>, std::shared_ptr<runtime::Executable>> m_cache;
            };

            class B200Executable : public runtime::Executable
            {
            public:
                /// saved_constants != nullptr (Backend::load): `func` is an already lowered graph and *saved_constants the
                /// constant image compile() built for it; the image is taken over
                B200Executable(const std::shared_ptr<DeviceContext>& ctx,
                               const std::shared_ptr<Function>& func,
                               bool enable_performance_data,
                               std::vector<char>* saved_constants = nullptr,
                               const std::map<std::string, std::pair<size_t, size_t>>* saved_index = nullptr,
                               const std::vector<std::shared_ptr<Node>>* saved_order = nullptr);
                ~B200Executable() override;
                bool call(const std::vector<std::shared_ptr<runtime::Tensor>>& outputs,
                          const std::vector<std::shared_ptr<runtime::Tensor>>& inputs) override;
                std::vector<PerformanceCounter> get_performance_data() const override;
                void save(std::ostream& output_stream) override;
                std::shared_ptr<runtime::Tensor> create_input_tensor(size_t input_index) override;
                std::shared_ptr<runtime::Tensor> create_output_tensor(size_t output_index) override;
                std::vector<std::shared_ptr<runtime::Tensor>> create_input_tensor(size_t input_index,
                                                                                 size_t pipeline_depth) override;
                std::vector<std::shared_ptr<runtime::Tensor>> create_output_tensor(size_t output_index,
                                                                                  size_t pipeline_depth) override;
                size_t kernel_steps() const { return m_steps.size(); }

            private:
                // a device buffer known at compile time (arena / constant) or bound per call (parameter / result)
                struct Slot
                {
                    enum Kind { ARENA, CONSTANT, PARAMETER, RESULT } kind;
                    size_t offset = 0; // ARENA / CONSTANT: byte offset in the respective pool
                    size_t index = 0;  // PARAMETER / RESULT: position in the call's tensor vectors
                    size_t bytes = 0;
                };
                using Ptrs = std::vector<void*>;
                struct Step
                {
                    std::shared_ptr<const Node> node;
                    std::string what;
                    std::function<int(const Ptrs&, cudaStream_t)> run;
                };
                // one logical nGraph tensor and the device materialisations made of it so far
                struct Value
                {
                    int canonical = -1; // slot holding nGraph's row-major layout (NCHW for images)
                    int nhwc = -1;      // slot holding the channels-last copy (4-D one-byte tensors only)
                    element::Type et;
                    Shape shape;
                    std::shared_ptr<const Node> constant; // set for Constant nodes (host bytes available)
                    bool skipped = false; // produced inside a fused pattern, never materialised
                };

                int new_slot(Slot::Kind kind, size_t bytes, size_t index = 0);
                int upload_constant(const std::string& key, const void* data, size_t bytes);
                std::string constant_key(const char* purpose, std::initializer_list<const Node*> sources) const;
                bool have_saved_constant(const std::string& key) const;
                Value& value_of(const Output<Node>& out);
                int canonical_slot(const Output<Node>& out);
                int nhwc_slot(const Output<Node>& out);
                void emit(const std::shared_ptr<const Node>& node, const std::string& what,
                          std::function<int(const Ptrs&, cudaStream_t)> run);
                void compile_node(const std::shared_ptr<Node>& node);
                void lower_node(const std::shared_ptr<Node>& node);
                void plan_arena();
                void compile_quantize(const std::shared_ptr<Node>& node);
                void compile_dequantize(const std::shared_ptr<Node>& node);
                void compile_fused_conv(const std::shared_ptr<Node>& node);
                void compile_core_conv(const std::shared_ptr<Node>& node);
                void compile_dot_bias(const std::shared_ptr<Node>& node);
                void compile_core_dot(const std::shared_ptr<Node>& node);
                void compile_max_pool(const std::shared_ptr<Node>& node);
                void compile_avg_pool(const std::shared_ptr<Node>& node);
                int dilate_and_crop_input(const std::shared_ptr<Node>& node, int x, Shape& ds, Strides& data_dilation,
                                          CoordinateDiff& below, CoordinateDiff& above, size_t c_dev);
                bool compile_f32_glue(const std::shared_ptr<Node>& node);
                bool try_compile_avgpool_head(const std::shared_ptr<Node>& quantize_node);
                int packed_filters(const Output<Node>& filters, size_t c_pad, bool* is_image = nullptr);
                int scalar_product_scale(const Output<Node>& a, const Output<Node>& b, const Output<Node>& c);
                static bool constant_is_zero(const Output<Node>& out);
                static bool avgpool_head_member(const Node* node);

                std::shared_ptr<DeviceContext> m_ctx;
                std::shared_ptr<Function> m_function;
                bool m_perf = false;
                std::vector<Slot> m_slots;
                std::vector<Step> m_steps;
                std::map<const descriptor::Tensor*, Value> m_values;
                std::vector<char> m_constant_host; // staged constants, uploaded once at the end of compile
                std::vector<char> m_preloaded;     // Backend::load: the saved constant image, consumed in lowering order
                std::map<std::string, std::pair<size_t, size_t>> m_constant_index; // key -> (offset, bytes) in the image
                std::map<const Node*, size_t> m_node_index;                         // position in the Function's node order
                bool m_use_preloaded = false;
                size_t m_constant_bytes = 0;       // size of the device constant image
                // lifetimes of the slots, in step indices: first step that may write / last step that reads
                std::vector<size_t> m_birth, m_last;
                std::vector<int> m_touched; // slots requested while the current node is lowered
                size_t m_arena_bytes = 0;
                void* m_arena = nullptr;
                void* m_constants = nullptr;
                std::vector<std::pair<int, int>> m_result_copies; // (source slot, result slot)
                mutable std::mutex m_call_mutex;
                std::vector<cudaEvent_t> m_events; // 2 per step when performance data is enabled
                std::vector<double> m_step_us;
                size_t m_calls = 0;
            };
        }
    }
}

extern "C" B200_BACKEND_API void ngraph_register_b200_backend();

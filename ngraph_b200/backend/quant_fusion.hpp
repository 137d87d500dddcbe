// Quantisation fusion for the B200 plugin.
//
// nGraph's CPU backend owns a graph rewrite (CPUQuantFusion, src/ngraph/runtime/cpu/pass/cpu_fusion.cpp:2025-2609)
// that turns "quantized op -> Dequantize -> f32 op -> Quantize" chains into the fused quantized ops its kernels
// implement.  That pass is part of the CPU backend and never runs for a plugin, so a graph written with the un-fused
// chains (what a bridge or an importer emits) would reach this backend as separate Dequantize / Relu / Add / Quantize
// steps over f32 tensors.  QuantFusion is the plugin's own statement of the same rewrites, written as a plain walk over
// the graph:
//
//   Relu(Dequantize(QuantizedConvolutionBias))                 -> Dequantize(QuantizedConvolutionBias[relu])
//   Relu(Dequantize(QuantizedConvolution[zero points 0]))      -> Dequantize(QuantizedConvolutionRelu)
//   Relu(Add(Dequantize(QuantizedConvolutionBias), Dequantize(s)))
//                                                              -> Dequantize(QuantizedConvolutionBias(Signed)Add[relu])
//   MaxPool(Dequantize(x))                                     -> Dequantize(MaxPool(x))
//   Concat(Dequantize(x0), Dequantize(x1), ...)  [same scale]  -> Dequantize(Concat(x0, x1, ...))
//   Quantize(Dequantize(x))  [same scale and type]             -> x
//
// It is registered under the name "B200QuantFusion"; NGRAPH_PASS_ENABLES="B200QuantFusion:0" switches it off, the way
// "CPUQuantFusion:0" does for the CPU backend (cpu_external_function.cpp:215-226, :1321).
//
// Not restated: the CPU backend's Dequantize/AvgPool swap (the INTERPRETER's integer avg_pool accumulates in the
// element type and wraps, so there is no reference result to agree with) and its QuantizedDot -> QuantizedMatmul
// rewrite (a layout change for DNNL; this backend runs QuantizedDot as it is).
#pragma once

#include <memory>

#include "ngraph/pass/pass.hpp"

namespace ngraph
{
    namespace runtime
    {
        namespace b200
        {
            namespace pass
            {
                class QuantFusion : public ngraph::pass::FunctionPass
                {
                public:
                    bool run_on_function(std::shared_ptr<ngraph::Function> function) override;
                    // how many rewrites of each kind the last run made (for tests and diagnostics)
                    struct Counts
                    {
                        int conv_relu = 0, conv_bias_relu = 0, conv_bias_add = 0, max_pool = 0, concat = 0, dq_q = 0;
                        int total() const { return conv_relu + conv_bias_relu + conv_bias_add + max_pool + concat + dq_q; }
                    };
                    const Counts& counts() const { return m_counts; }

                private:
                    Counts m_counts;
                };

                // true unless NGRAPH_PASS_ENABLES holds "B200QuantFusion:0"
                bool quant_fusion_enabled();
            }
        }
    }
}

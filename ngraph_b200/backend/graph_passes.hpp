// The graph-level pipeline the B200 plugin runs in compile(), before lowering: needs nGraph's core library only, no
// device.  Kept apart from the plugin's Backend / Executable classes so that tools and tests can apply exactly the same
// passes to a Function without the plugin exporting anything besides its registration symbol.
#pragma once

#include <memory>

#include "ngraph/function.hpp"
#include "ngraph/node.hpp"

namespace ngraph
{
    namespace runtime
    {
        namespace b200
        {
            /// A fused op (LayerNorm over the last axis with scale and bias, Gelu, on f32) that the device runs as ONE kernel with
            /// the arithmetic of its decomposition, and that FusedOpDecomposition therefore leaves whole.
            bool runs_undecomposed(const Node& node);

            /// Rewrites `function` in place: LikeReplacement, FusedOpDecomposition (LayerNorm / Gelu of the shapes the device
            /// runs as one kernel stay whole unless `decompose_all`), ImplicitBroadcastElimination, the quantisation fusion
            /// (pass::QuantFusion, unless switched off through NGRAPH_PASS_ENABLES) and ConstantFolding.
            void run_graph_passes(const std::shared_ptr<Function>& function, bool decompose_all = false);
        }
    }
}

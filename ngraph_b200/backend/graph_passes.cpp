// compile()'s graph-level passes (see graph_passes.hpp).
#include "graph_passes.hpp"

#include "quant_fusion.hpp"
#include "ngraph/op/broadcast.hpp"
#include "ngraph/op/constant.hpp"
#include "ngraph/op/gelu.hpp"
#include "ngraph/op/layer_norm.hpp"
#include "ngraph/op/stop_gradient.hpp"
#include "ngraph/pass/constant_folding.hpp"
#include "ngraph/pass/fused_op_decomposition.hpp"
#include "ngraph/pass/implicit_broadcast_elimination.hpp"
#include "ngraph/pass/like_replacement.hpp"
#include "ngraph/pass/manager.hpp"

using namespace ngraph;

// The graph-level pipeline of compile(): what nGraph's backends run before they lower (cpu_external_function.cpp:1289-1335
// keeps the CPU backend's list), with the plugin's own quantisation fusion in the place CPUQuantFusion has there.
// Fused ops the device runs as one kernel with the arithmetic of their decomposition; everything else is decomposed.
bool ngraph::runtime::b200::runs_undecomposed(const Node& node)
{
    if (auto ln = as_type<const op::v0::LayerNorm>(&node))
    {
        if (!ln->get_use_affine() || ln->get_keep_stats() || node.get_input_element_type(0) != element::f32 ||
            !node.get_input_partial_shape(0).is_static())
            return false;
        const Shape shape = node.get_input_shape(0);
        const int64_t rank = int64_t(shape.size());
        const int64_t axis = ln->get_begin_norm_axis() >= 0 ? ln->get_begin_norm_axis() : rank + ln->get_begin_norm_axis();
        return rank >= 1 && axis == rank - 1 && shape.back() >= 1 && shape.back() <= 1535 && node.get_input_shape(1).size() == 1 &&
               node.get_input_shape(2).size() == 1;
    }
    if (is_type<op::v0::Gelu>(&node))
        return node.get_input_element_type(0) == element::f32;
    return false;
}

// ConstantFolding turns Broadcast(Constant) into a Constant as large as the broadcast's output: a 768-element bias
// row added to 24 576 rows becomes 75 MB of constant data, per layer.  Broadcasts of that kind (new leading axes only,
// at least 64 Ki output elements) are fenced off with an identity op that has no folder (StopGradient) while the pass
// runs; the elementwise op that reads the Broadcast then indexes the small constant directly (compile_f32_glue).
static void fence_large_constant_broadcasts(const std::shared_ptr<Function>& function)
{
    for (auto& node : function->get_ordered_ops())
    {
        auto bc = as_type_ptr<op::v0::Broadcast>(node);
        if (!bc || !is_type<op::v0::Constant>(bc->input_value(0).get_node()) || shape_size(bc->get_output_shape(0)) < 65536)
            continue;
        const AxisSet& added = bc->get_broadcast_axes();
        bool leading = !added.empty();
        for (size_t i = 0; i < added.size() && leading; ++i)
            leading = added.count(i) == 1;
        if (leading)
            bc->input(0).replace_source_output(std::make_shared<op::v0::StopGradient>(bc->input_value(0))->output(0));
    }
}

static void remove_fences(const std::shared_ptr<Function>& function)
{
    for (auto& node : function->get_ordered_ops())
        if (is_type<op::v0::StopGradient>(node))
            node->output(0).replace(node->input_value(0));
}

void ngraph::runtime::b200::run_graph_passes(const std::shared_ptr<Function>& function, bool decompose_all)
{
    bool fenced = false;
    for (auto& node : function->get_ordered_ops()) // a graph that has such nodes of its own is left as it is
        fenced = fenced || is_type<op::v0::StopGradient>(node);
    {
        ngraph::pass::Manager pre;
        pre.register_pass<ngraph::pass::LikeReplacement>();
        if (decompose_all) // the float islands as chains of elementwise ops and reductions (for comparison)
            pre.register_pass<ngraph::pass::FusedOpDecomposition>();
        else
            pre.register_pass<ngraph::pass::FusedOpDecomposition>(ngraph::runtime::b200::runs_undecomposed);
        pre.register_pass<ngraph::pass::ImplicitBroadcastElimination>(); // NumPy-style operands become explicit Broadcast nodes
        pre.run_passes(function);
    }
    if (!fenced)
        fence_large_constant_broadcasts(function);
    {
        ngraph::pass::Manager pm;
        if (ngraph::runtime::b200::pass::quant_fusion_enabled())
            pm.register_pass<ngraph::runtime::b200::pass::QuantFusion>();
        pm.register_pass<ngraph::pass::ConstantFolding>(); // also folds the scale arithmetic the fusion leaves behind
        pm.run_passes(function);
    }
    if (!fenced)
        remove_fences(function);
}

// Splitting a lowered Function along the batch: the same graph for `rows` of the `batch` leading rows of every
// batch-carrying tensor.  Used by the multi-device backend option ("B200:all", "B200:0+1"): every device runs the split
// graph on its own contiguous slice of each batch-carrying input and writes its slice of each result; no data crosses
// between devices.  Needs nGraph's core library only, no device.
#pragma once

#include <memory>
#include <string>
#include <vector>

#include "ngraph/function.hpp"

namespace ngraph
{
    namespace runtime
    {
        namespace b200
        {
            struct BatchSplit
            {
                /// the rebuilt Function: every batch-carrying tensor has `rows / batch` of its leading extent
                std::shared_ptr<Function> function;
                /// per Parameter / Result of the original Function: does its leading axis carry the batch
                std::vector<bool> parameter_split, result_split;
            };

            /// `function` must have been through run_graph_passes (explicit Broadcasts, fused quantized ops).  The batch is the
            /// leading extent of Parameter 0.  Returns false, with the reason in `why`, when the graph cannot be proven
            /// independent along the batch by the per-op rules of batch_split.cpp (a reduction over the batch axis, a
            /// transposition that moves it, a Constant that spans it, an op the rules do not know): the caller then runs the
            /// whole Function on one device.
            bool split_batch(const Function& function, size_t rows, BatchSplit& out, std::string& why);

            /// the batch of `function` as split_batch understands it, 0 when there is none
            size_t batch_of(const Function& function);
        }
    }
}

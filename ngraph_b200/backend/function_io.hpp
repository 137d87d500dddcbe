// A compact binary form of an nGraph Function restricted to the op set the B200 plugin lowers, used by
// B200Executable::save / B200Backend::load.  nGraph's own serializer (src/ngraph/serializer.cpp) needs the JSON library, which
// a build with NGRAPH_JSON_ENABLE=OFF does not have; the INTERPRETER backend's save / load
// (src/ngraph/runtime/interpreter/int_executable.cpp:345-352, int_backend.cpp:81-110) then is not available either.
// The format is private to the plugin: nodes in topological order, each with its type, its inputs and its attributes.
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
            /// Serialises `function`.  Throws ngraph::unsupported_op for an op type outside the plugin's set.
            std::string write_function(const Function& function);
            /// Rebuilds a Function from write_function's output.  Throws std::runtime_error on malformed data.
            /// `nodes_in_saved_order`, when given, receives the rebuilt nodes in the order they were written.
            std::shared_ptr<Function> read_function(const std::string& bytes,
                                                    std::vector<std::shared_ptr<Node>>* nodes_in_saved_order = nullptr);
            /// FNV-1a of a byte string (identifies a saved model / constant image pair)
            uint64_t fnv1a(const void* data, size_t bytes);
        }
    }
}

// An int8 BERT-base-shaped encoder as an nGraph Function, for the tests: token / segment / position
// embeddings, then per layer self-attention and a feed-forward block whose six matrix products (Q, K, V,
// attention output, FFN in, FFN out) are QuantizedDotBias with per-channel i8 weights and a dynamic
// per-tensor i8 activation scale (max |x| / 127 computed in the graph); softmax, LayerNorm, GELU and the
// residual adds stay in f32.  With `decomposed` the QuantizedDotBias nodes are replaced by the ops the
// INTERPRETER backend implements (Dot on i32 Converts, then the f32 scale), which is their definition:
// float(acc + bias) * scale[n] with an int32 accumulator.  Weights are drawn here from a seeded generator so
// that two builds with the same arguments are the same network.  Part of the ng_capi facade library.
#include <cmath>
#include <memory>
#include <random>
#include <string>
#include <vector>

#include "ngraph/ngraph.hpp"
#include "ngraph/op/experimental/batch_mat_mul.hpp"
#include "ngraph/op/experimental/quantized_dot_bias.hpp"
#include "ngraph/op/gelu.hpp"
#include "ngraph/op/layer_norm.hpp"
#include "ngraph/pass/constant_folding.hpp"
#include "ngraph/pass/fused_op_decomposition.hpp"
#include "ngraph/pass/like_replacement.hpp"
#include "ngraph/pass/manager.hpp"

using namespace ngraph;

namespace
{
    struct Builder
    {
        std::mt19937_64 rng;
        bool decomposed;
        size_t hidden, heads, ffn, seq, batch;

        std::shared_ptr<Node> f32_const(const Shape& s, double sigma, double mean = 0.0)
        {
            std::normal_distribution<double> d(mean, sigma);
            std::vector<float> v(shape_size(s));
            for (auto& x : v)
                x = float(sigma == 0.0 ? mean : d(rng));
            return op::v0::Constant::create(element::f32, s, v);
        }

        // y[M,N] = x[M,K] . W[N,K]^T + b, the product in int8 with a dynamic activation scale
        Output<Node> qlinear(const Output<Node>& x, size_t K, size_t N)
        {
            // weights N(0, 0.02), quantised per output channel: s_w[n] = max|w[n,:]| / 127
            std::normal_distribution<double> d(0.0, 0.02);
            std::vector<float> w(N * K);
            for (auto& v : w)
                v = float(d(rng));
            std::vector<int8_t> wq(N * K);
            std::vector<float> sw(N);
            for (size_t n = 0; n < N; ++n)
            {
                float m = 0;
                for (size_t k = 0; k < K; ++k)
                    m = std::max(m, std::fabs(w[n * K + k]));
                sw[n] = m / 127.0f;
                for (size_t k = 0; k < K; ++k)
                    wq[n * K + k] = int8_t(std::max(-127.0f, std::min(127.0f, std::nearbyint(w[n * K + k] / sw[n]))));
            }
            const Shape xs = x.get_shape();
            const size_t M = xs[0];
            AxisSet all;
            for (size_t i = 0; i < xs.size(); ++i)
                all.insert(i);
            auto amax = std::make_shared<op::v0::Max>(std::make_shared<op::v0::Abs>(x), all);
            auto s_x = std::make_shared<op::v1::Divide>(amax, op::v0::Constant::create(element::f32, Shape{}, {127.0f}));
            auto zp = op::v0::Constant::create(element::i8, Shape{}, {0});
            auto xq = std::make_shared<op::v0::Quantize>(x, s_x, zp, element::i8, AxisSet{},
                                                         op::v0::Quantize::RoundMode::ROUND_NEAREST_TOWARD_EVEN);
            auto s_w = op::v0::Constant::create(element::f32, Shape{N}, sw);
            auto scale = std::make_shared<op::v1::Multiply>(std::make_shared<op::v0::Broadcast>(s_x, Shape{N}, AxisSet{0}), s_w);
            Output<Node> y;
            if (!decomposed)
            {
                auto W = op::v0::Constant::create(element::i8, Shape{N, K}, wq);
                auto zero_bias = op::v0::Constant::create(element::i32, Shape{N}, std::vector<int32_t>(N, 0));
                y = std::make_shared<op::v0::QuantizedDotBias>(xq, W, zero_bias, scale, false, false);
            }
            else
            {
                std::vector<int32_t> wt(K * N);
                for (size_t n = 0; n < N; ++n)
                    for (size_t k = 0; k < K; ++k)
                        wt[k * N + n] = wq[n * K + k];
                auto Wt = op::v0::Constant::create(element::i32, Shape{K, N}, wt);
                auto acc = std::make_shared<op::v0::Dot>(std::make_shared<op::v0::Convert>(xq, element::i32), Wt, 1);
                y = std::make_shared<op::v1::Multiply>(std::make_shared<op::v0::Convert>(acc, element::f32),
                                                       std::make_shared<op::v0::Broadcast>(scale, Shape{M, N}, AxisSet{0}));
            }
            auto b = f32_const(Shape{N}, 0.02);
            return std::make_shared<op::v1::Add>(y, std::make_shared<op::v0::Broadcast>(b, Shape{M, N}, AxisSet{0}));
        }

        Output<Node> layer_norm(const Output<Node>& x)
        {
            auto g = f32_const(Shape{hidden}, 0.05, 1.0), b = f32_const(Shape{hidden}, 0.05);
            return std::make_shared<op::v0::LayerNorm>(x, g, b, false, 1, 1e-5);
        }

        // [B*S, H] -> [B*heads, S, d] (or [B*heads, d, S] when transposed)
        Output<Node> split_heads(const Output<Node>& x, bool transposed)
        {
            const size_t d = hidden / heads;
            auto r = std::make_shared<op::v0::Reshape>(x, AxisVector{0, 1}, Shape{batch, seq, heads, d});
            if (transposed)
                return std::make_shared<op::v0::Reshape>(r, AxisVector{0, 2, 3, 1}, Shape{batch * heads, d, seq});
            return std::make_shared<op::v0::Reshape>(r, AxisVector{0, 2, 1, 3}, Shape{batch * heads, seq, d});
        }

        Output<Node> encoder_layer(const Output<Node>& x)
        {
            const size_t d = hidden / heads, M = batch * seq;
            auto q = split_heads(qlinear(x, hidden, hidden), false);
            auto kt = split_heads(qlinear(x, hidden, hidden), true);
            auto v = split_heads(qlinear(x, hidden, hidden), false);
            Output<Node> scores = std::make_shared<op::v0::BatchMatMul>(q, kt); // [B*heads, S, S]
            auto inv = op::v0::Constant::create(element::f32, Shape{}, {float(1.0 / std::sqrt(double(d)))});
            scores = std::make_shared<op::v1::Multiply>(
                scores, std::make_shared<op::v0::Broadcast>(inv, scores.get_shape(), AxisSet{0, 1, 2}));
            auto probs = std::make_shared<op::v0::Softmax>(scores, AxisSet{2});
            auto ctx = std::make_shared<op::v0::BatchMatMul>(probs, v); // [B*heads, S, d]
            auto ctx4 = std::make_shared<op::v0::Reshape>(ctx, AxisVector{0, 1, 2}, Shape{batch, heads, seq, d});
            auto merged = std::make_shared<op::v0::Reshape>(ctx4, AxisVector{0, 2, 1, 3}, Shape{M, hidden});
            auto attn = qlinear(merged, hidden, hidden);
            auto x1 = layer_norm(std::make_shared<op::v1::Add>(x, attn));
            auto h = std::make_shared<op::v0::Gelu>(qlinear(x1, hidden, ffn));
            auto y = qlinear(h, ffn, hidden);
            return layer_norm(std::make_shared<op::v1::Add>(x1, y));
        }
    };
}

#define NGC_API extern "C" __attribute__((visibility("default")))

// Function(ids i32 [B*S], segments i32 [B*S]) -> f32 [B*S, hidden].  Returns a new std::shared_ptr<Function>*
// (released with ngc_function_free) or null.
NGC_API void* ngc_bert_encoder(int layers, int hidden, int heads, int ffn, int seq, int batch, int vocab, uint64_t seed,
                               int decomposed)
{
    try
    {
        Builder b{std::mt19937_64(seed), decomposed != 0, size_t(hidden), size_t(heads), size_t(ffn), size_t(seq), size_t(batch)};
        const size_t M = size_t(batch) * seq, H = size_t(hidden);
        auto ids = std::make_shared<op::v0::Parameter>(element::i32, Shape{M});
        auto seg = std::make_shared<op::v0::Parameter>(element::i32, Shape{M});
        auto tok = b.f32_const(Shape{size_t(vocab), H}, 0.02), segt = b.f32_const(Shape{2, H}, 0.02),
             pos = b.f32_const(Shape{size_t(seq), H}, 0.02);
        Output<Node> x = std::make_shared<op::v1::Add>(std::make_shared<op::v0::Gather>(tok, ids, 0),
                                                       std::make_shared<op::v0::Gather>(segt, seg, 0));
        auto pos_b = std::make_shared<op::v0::Reshape>(
            std::make_shared<op::v0::Broadcast>(pos, Shape{size_t(batch), size_t(seq), H}, AxisSet{0}), AxisVector{0, 1, 2},
            Shape{M, H});
        x = b.layer_norm(std::make_shared<op::v1::Add>(x, pos_b));
        for (int l = 0; l < layers; ++l)
            x = b.encoder_layer(x);
        return new std::shared_ptr<Function>(std::make_shared<Function>(OutputVector{x}, ParameterVector{ids, seg}));
    }
    catch (const std::exception&)
    {
        return nullptr;
    }
}

// Op type names of the Function, one per line, after the pass pipeline a backend runs before lowering
// (LikeReplacement, FusedOpDecomposition, ConstantFolding) when `lowered` is set.  Returns the byte count.
NGC_API int ngc_function_op_names(void* function, int lowered, char* buf, int n)
{
    try
    {
        auto f = *static_cast<std::shared_ptr<Function>*>(function);
        if (lowered)
        {
            f = clone_function(*f);
            pass::Manager pm;
            pm.register_pass<pass::LikeReplacement>();
            pm.register_pass<pass::FusedOpDecomposition>();
            pm.register_pass<pass::ConstantFolding>();
            pm.run_passes(f);
        }
        std::string all;
        for (auto& node : f->get_ordered_ops())
            all += std::string(node->get_type_info().name) + "\n";
        if (int(all.size()) + 1 > n)
            return -int(all.size()) - 1;
        memcpy(buf, all.c_str(), all.size() + 1);
        return int(all.size());
    }
    catch (const std::exception&)
    {
        return -1;
    }
}

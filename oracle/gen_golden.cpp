// gen_golden.cpp - produces the golden fixtures under tests/golden/ by running the
// REFERENCE ITSELF (nGraph core + its INTERPRETER backend, built by oracle/Makefile.ngraph
// into oracle/_ref/lib) on small seeded inputs.  Test infrastructure only.
//
//   gen_golden interp  <out.json>   seeded cases through INTERPRETER (inputs + outputs)
//   gen_golden scales  <builder> <requantize> <relu> <min/max values...>
//                                  the scale constants nGraph's own builders + ConstantFolding
//                                  produce for a set of min/max ranges (one JSON object on stdout)
//
// f32 arrays are written as their uint32 bit patterns so the fixture is exact.
#include <cstdio>
#include <cstring>
#include <fstream>
#include <functional>
#include <iostream>
#include <random>
#include <sstream>

#include "ngraph/builder/quantized_conv_builder.hpp"
#include "ngraph/builder/quantized_dot_builder.hpp"
#include "ngraph/ngraph.hpp"
#include "ngraph/op/experimental/quantized_conv_bias.hpp"
#include "ngraph/op/experimental/quantized_dot_bias.hpp"
#include "ngraph/pass/constant_folding.hpp"
#include "ngraph/pass/manager.hpp"
#include "ngraph/runtime/backend.hpp"

using namespace ngraph;
using std::make_shared;
using std::shared_ptr;
using std::string;
using std::vector;

// ---------------------------------------------------------------- tiny JSON writer
struct Json
{
    std::ostringstream os;
    bool first_case = true;
};

static const char* et_name(const element::Type& t)
{
    if (t == element::u8) return "u8";
    if (t == element::i8) return "i8";
    if (t == element::i32) return "i32";
    if (t == element::f32) return "f32";
    if (t == element::i64) return "i64";
    throw std::runtime_error("unsupported element type in fixture");
}

struct Blob
{
    element::Type et;
    Shape shape;
    vector<char> bytes;
    size_t count() const { return shape_size(shape); }
};

template <typename T>
static Blob make_blob(const element::Type& et, const Shape& shape, const vector<T>& v)
{
    Blob b{et, shape, vector<char>(v.size() * sizeof(T))};
    if (v.size() != shape_size(shape)) throw std::runtime_error("blob size mismatch");
    memcpy(b.bytes.data(), v.data(), b.bytes.size());
    return b;
}

static void write_blob(std::ostream& os, const Blob& b)
{
    os << "{\"dtype\":\"" << et_name(b.et) << "\",\"shape\":[";
    for (size_t i = 0; i < b.shape.size(); ++i) os << (i ? "," : "") << b.shape[i];
    os << "],\"data\":[";
    size_t n = b.count();
    for (size_t i = 0; i < n; ++i)
    {
        if (i) os << ",";
        if (b.et == element::u8) os << unsigned(reinterpret_cast<const uint8_t*>(b.bytes.data())[i]);
        else if (b.et == element::i8) os << int(reinterpret_cast<const int8_t*>(b.bytes.data())[i]);
        else if (b.et == element::i32) os << reinterpret_cast<const int32_t*>(b.bytes.data())[i];
        else if (b.et == element::i64) os << reinterpret_cast<const int64_t*>(b.bytes.data())[i];
        else os << reinterpret_cast<const uint32_t*>(b.bytes.data())[i]; // f32 bit pattern
    }
    os << "]}";
}

struct Case
{
    string name, op;
    vector<std::pair<string, string>> attrs; // already-JSON values
    vector<std::pair<string, Blob>> inputs, outputs;
};

static void write_case(Json& j, const Case& c)
{
    j.os << (j.first_case ? "" : ",\n") << "{\"name\":\"" << c.name << "\",\"op\":\"" << c.op << "\",\"attrs\":{";
    j.first_case = false;
    for (size_t i = 0; i < c.attrs.size(); ++i)
        j.os << (i ? "," : "") << "\"" << c.attrs[i].first << "\":" << c.attrs[i].second;
    j.os << "},\"inputs\":{";
    for (size_t i = 0; i < c.inputs.size(); ++i)
    {
        j.os << (i ? "," : "") << "\"" << c.inputs[i].first << "\":";
        write_blob(j.os, c.inputs[i].second);
    }
    j.os << "},\"outputs\":{";
    for (size_t i = 0; i < c.outputs.size(); ++i)
    {
        j.os << (i ? "," : "") << "\"" << c.outputs[i].first << "\":";
        write_blob(j.os, c.outputs[i].second);
    }
    j.os << "}}";
}

template <typename T>
static string jlist(const vector<T>& v)
{
    std::ostringstream os;
    os << "[";
    for (size_t i = 0; i < v.size(); ++i) os << (i ? "," : "") << (long long)v[i];
    os << "]";
    return os.str();
}

// ---------------------------------------------------------------- running the reference
static shared_ptr<runtime::Backend> interp()
{
    static shared_ptr<runtime::Backend> b = runtime::Backend::create("INTERPRETER");
    return b;
}

static vector<Blob> run(const shared_ptr<Function>& f, const vector<Blob>& in)
{
    auto be = interp();
    vector<shared_ptr<runtime::Tensor>> tin, tout;
    auto params = f->get_parameters();
    if (params.size() != in.size()) throw std::runtime_error("parameter count mismatch");
    for (size_t i = 0; i < in.size(); ++i)
    {
        auto t = be->create_tensor(params[i]->get_output_element_type(0), params[i]->get_output_shape(0));
        t->write(in[i].bytes.data(), in[i].bytes.size());
        tin.push_back(t);
    }
    for (auto& r : f->get_results()) tout.push_back(be->create_tensor(r->get_output_element_type(0), r->get_output_shape(0)));
    auto exe = be->compile(f);
    exe->call_with_validate(tout, tin);
    vector<Blob> out;
    for (auto& t : tout)
    {
        Blob b{t->get_element_type(), t->get_shape(), vector<char>(t->get_size_in_bytes())};
        t->read(b.bytes.data(), b.bytes.size());
        out.push_back(b);
    }
    return out;
}

static shared_ptr<Node> param_of(const Blob& b) { return make_shared<op::v0::Parameter>(b.et, b.shape); }

static ParameterVector as_params(const vector<shared_ptr<Node>>& v)
{
    ParameterVector p;
    for (auto& n : v) p.push_back(std::static_pointer_cast<op::v0::Parameter>(n));
    return p;
}

// ---------------------------------------------------------------- seeded data
struct Rng
{
    std::mt19937_64 g;
    explicit Rng(uint64_t s) : g(s) {}
    double uni() { return (g() >> 11) * (1.0 / 9007199254740992.0); }
    int irange(int lo, int hi) { return lo + int(g() % uint64_t(hi - lo + 1)); }
    double normal()
    {
        double u1 = uni() + 1e-12, u2 = uni();
        return std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2);
    }
};

template <typename T>
static Blob rand_int_blob(Rng& r, const element::Type& et, const Shape& s, int lo, int hi)
{
    vector<T> v(shape_size(s));
    for (auto& x : v) x = T(r.irange(lo, hi));
    return make_blob(et, s, v);
}

static Blob f32_blob(const Shape& s, const vector<float>& v) { return make_blob(element::f32, s, v); }

static Shape sub_shape(const Shape& s, const AxisSet& axes)
{
    Shape r;
    for (size_t i = 0; i < s.size(); ++i)
        if (axes.count(i)) r.push_back(s[i]);
    return r;
}

// ---------------------------------------------------------------- case families
static void quantize_cases(Json& j)
{
    Shape shape{2, 3, 4, 6};
    vector<AxisSet> axis_sets{AxisSet{}, AxisSet{1}, AxisSet{0, 2}};
    const element::Type qts[3] = {element::u8, element::i8, element::i32};
    int id = 0;
    for (int mode = 0; mode < 9; ++mode)
        for (size_t a = 0; a < axis_sets.size(); ++a)
            for (int qt = 0; qt < 3; ++qt)
            {
                if (qt == 2 && a != 0) continue; // i32 only per tensor
                Rng r(1000 + id);
                const AxisSet& axes = axis_sets[a];
                Shape ss = sub_shape(shape, axes);
                size_t ns = shape_size(ss);
                vector<float> scale(ns);
                for (auto& s : scale) s = float(std::exp(std::log(1e-3) + r.uni() * (std::log(1e-1) - std::log(1e-3))));
                if (a == 0) scale[0] = 0.05f;
                Blob zp;
                if (qt == 0) zp = rand_int_blob<uint8_t>(r, element::u8, ss, a == 0 ? 128 : 100, a == 0 ? 128 : 150);
                else if (qt == 1) zp = rand_int_blob<int8_t>(r, element::i8, ss, a == 0 ? 0 : -20, a == 0 ? 0 : 20);
                else zp = rand_int_blob<int32_t>(r, element::i32, ss, -7, 7);
                // data: exact ties (k+0.5)*scale, near-ties, plain normals, values beyond the clamp
                vector<float> x(shape_size(shape));
                CoordinateTransform ct(shape), st(ss);
                size_t i = 0;
                for (const Coordinate& c : ct)
                {
                    float s = scale[st.index(project(c, axes))];
                    int kind = r.irange(0, 5);
                    int k = r.irange(-140, 140);
                    if (kind == 0) x[i] = (float(k) + 0.5f) * s;
                    else if (kind == 1) x[i] = std::nextafterf((float(k) + 0.5f) * s, r.irange(0, 1) ? 1e9f : -1e9f);
                    else if (kind == 2) x[i] = float(k) * s;
                    else if (kind == 3) x[i] = float(r.normal() * 400.0) * s;
                    else x[i] = float(r.normal());
                    ++i;
                }
                Blob bx = f32_blob(shape, x), bs = f32_blob(ss, scale);
                auto X = param_of(bx), S = param_of(bs), Z = param_of(zp);
                auto q = make_shared<op::v0::Quantize>(X, S, Z, qts[qt], axes,
                                                       static_cast<op::v0::Quantize::RoundMode>(mode));
                auto out = run(make_shared<Function>(OutputVector{q}, as_params({X, S, Z})), {bx, bs, zp});
                Case c;
                c.name = "quantize_" + std::to_string(id++);
                c.op = "Quantize";
                c.attrs = {{"round_mode", std::to_string(mode)}, {"axes", jlist(vector<size_t>(axes.begin(), axes.end()))}};
                c.inputs = {{"x", bx}, {"scale", bs}, {"zero_point", zp}};
                c.outputs = {{"y", out[0]}};
                write_case(j, c);

                // and the way back
                auto Qin = param_of(out[0]);
                auto dq = make_shared<op::v0::Dequantize>(Qin, S, Z, element::f32, axes);
                auto back = run(make_shared<Function>(OutputVector{dq}, as_params({Qin, S, Z})), {out[0], bs, zp});
                Case d;
                d.name = "dequantize_" + std::to_string(id - 1);
                d.op = "Dequantize";
                d.attrs = {{"axes", jlist(vector<size_t>(axes.begin(), axes.end()))}};
                d.inputs = {{"x", out[0]}, {"scale", bs}, {"zero_point", zp}};
                d.outputs = {{"y", back[0]}};
                write_case(j, d);
            }
}

template <typename T>
static shared_ptr<Node> scalar(const element::Type& et, T v)
{
    return op::v0::Constant::create(et, Shape{}, {v});
}

static void qdot_core_cases(Json& j)
{
    struct Combo { element::Type b, out; int zb, zo; };
    Combo combos[4] = {{element::i8, element::i8, 0, 0}, {element::u8, element::u8, 3, 5},
                       {element::i8, element::i32, -2, 7}, {element::u8, element::i32, 0, 0}};
    for (int ci = 0; ci < 4; ++ci)
    {
        Rng r(2000 + ci);
        size_t M = 5, K = 24, N = 6;
        Blob A = rand_int_blob<uint8_t>(r, element::u8, Shape{M, K}, 0, 40);
        Blob B = combos[ci].b == element::i8 ? rand_int_blob<int8_t>(r, element::i8, Shape{K, N}, -30, 30)
                                             : rand_int_blob<uint8_t>(r, element::u8, Shape{K, N}, 0, 30);
        int za = ci == 1 ? 2 : 0;
        float sa = 0.5f, sb = 0.25f, so = combos[ci].out == element::i32 ? 0.125f : 16.0f;
        auto PA = param_of(A), PB = param_of(B);
        shared_ptr<Node> zB = combos[ci].b == element::i8 ? scalar<int8_t>(element::i8, combos[ci].zb)
                                                          : scalar<uint8_t>(element::u8, combos[ci].zb);
        shared_ptr<Node> zO = combos[ci].out == element::i8 ? scalar<int8_t>(element::i8, combos[ci].zo)
                              : combos[ci].out == element::u8 ? scalar<uint8_t>(element::u8, combos[ci].zo)
                                                              : scalar<int32_t>(element::i32, combos[ci].zo);
        auto d = make_shared<op::v0::QuantizedDot>(PA, PB, 1, scalar<float>(element::f32, sa),
                                                   scalar<uint8_t>(element::u8, za), scalar<float>(element::f32, sb),
                                                   zB, scalar<float>(element::f32, so), zO, combos[ci].out);
        auto out = run(make_shared<Function>(OutputVector{d}, as_params({PA, PB})), {A, B});
        Case c;
        c.name = "qdot_core_" + std::to_string(ci);
        c.op = "QuantizedDot";
        c.attrs = {{"za", std::to_string(za)}, {"zb", std::to_string(combos[ci].zb)}, {"zo", std::to_string(combos[ci].zo)}};
        c.inputs = {{"a", A}, {"b", B}, {"sa", f32_blob(Shape{}, {sa})}, {"sb", f32_blob(Shape{}, {sb})},
                    {"so", f32_blob(Shape{}, {so})}};
        c.outputs = {{"y", out[0]}};
        write_case(j, c);
    }
}

struct ConvGeom
{
    Shape data, filt;
    Strides stride, dil;
    CoordinateDiff below, above;
};

static vector<std::pair<string, string>> geom_attrs(const ConvGeom& g)
{
    return {{"stride", jlist(vector<size_t>(g.stride.begin(), g.stride.end()))},
            {"dilation", jlist(vector<size_t>(g.dil.begin(), g.dil.end()))},
            {"pad_below", jlist(vector<std::ptrdiff_t>(g.below.begin(), g.below.end()))},
            {"pad_above", jlist(vector<std::ptrdiff_t>(g.above.begin(), g.above.end()))}};
}

static void qconv_core_cases(Json& j)
{
    ConvGeom geoms[2] = {{Shape{2, 4, 6, 5}, Shape{3, 4, 3, 3}, Strides{1, 1}, Strides{1, 1}, CoordinateDiff{1, 1}, CoordinateDiff{1, 1}},
                         {Shape{1, 3, 9, 8}, Shape{2, 3, 2, 3}, Strides{2, 1}, Strides{2, 1}, CoordinateDiff{0, 2}, CoordinateDiff{1, 0}}};
    struct Combo { element::Type f, out; int zf, zo; };
    Combo combos[4] = {{element::i8, element::i8, 0, 0}, {element::u8, element::u8, 3, 5},
                       {element::i8, element::i32, -2, 7}, {element::u8, element::i32, 0, 0}};
    int id = 0;
    for (auto& g : geoms)
        for (int ci = 0; ci < 4; ++ci)
        {
            Rng r(3000 + id);
            Blob D = rand_int_blob<uint8_t>(r, element::u8, g.data, 0, 40);
            Blob F = combos[ci].f == element::i8 ? rand_int_blob<int8_t>(r, element::i8, g.filt, -20, 20)
                                                 : rand_int_blob<uint8_t>(r, element::u8, g.filt, 0, 20);
            int zd = ci == 1 ? 2 : 0;
            float sd = 0.5f, sf = 0.25f, so = combos[ci].out == element::i32 ? 0.125f : 32.0f;
            auto PD = param_of(D), PF = param_of(F);
            shared_ptr<Node> zF = combos[ci].f == element::i8 ? scalar<int8_t>(element::i8, combos[ci].zf)
                                                              : scalar<uint8_t>(element::u8, combos[ci].zf);
            shared_ptr<Node> zO = combos[ci].out == element::i8 ? scalar<int8_t>(element::i8, combos[ci].zo)
                                  : combos[ci].out == element::u8 ? scalar<uint8_t>(element::u8, combos[ci].zo)
                                                                  : scalar<int32_t>(element::i32, combos[ci].zo);
            auto cv = make_shared<op::v0::QuantizedConvolution>(
                PD, PF, g.stride, g.dil, g.below, g.above, Strides{1, 1}, scalar<float>(element::f32, sd),
                scalar<uint8_t>(element::u8, zd), scalar<float>(element::f32, sf), zF, scalar<float>(element::f32, so), zO,
                combos[ci].out);
            auto out = run(make_shared<Function>(OutputVector{cv}, as_params({PD, PF})), {D, F});
            Case c;
            c.name = "qconv_core_" + std::to_string(id++);
            c.op = "QuantizedConvolution";
            c.attrs = geom_attrs(g);
            c.attrs.push_back({"zd", std::to_string(zd)});
            c.attrs.push_back({"zf", std::to_string(combos[ci].zf)});
            c.attrs.push_back({"zo", std::to_string(combos[ci].zo)});
            c.inputs = {{"data", D}, {"filters", F}, {"sd", f32_blob(Shape{}, {sd})}, {"sf", f32_blob(Shape{}, {sf})},
                        {"so", f32_blob(Shape{}, {so})}};
            c.outputs = {{"y", out[0]}};
            write_case(j, c);
        }
}

// The tail shared by the decomposed fused ops: acc(i32) [+bias] -> f32 * scale [+ sum_scale*sum] [relu] -> Quantize RNE
static shared_ptr<Node> fused_tail(shared_ptr<Node> acc_i32, shared_ptr<Node> bias, size_t chan_axis,
                                   shared_ptr<Node> scale, shared_ptr<Node> sum_in, shared_ptr<Node> sum_scale,
                                   bool relu, const element::Type& out_et)
{
    Shape os = acc_i32->get_output_shape(0);
    AxisSet bc;
    for (size_t i = 0; i < os.size(); ++i)
        if (i != chan_axis) bc.insert(i);
    shared_ptr<Node> v = acc_i32;
    if (bias) v = make_shared<op::v1::Add>(v, make_shared<op::v0::Broadcast>(bias, os, bc));
    v = make_shared<op::v0::Convert>(v, element::f32);
    shared_ptr<Node> sc = scale;
    if (shape_size(scale->get_output_shape(0)) == 1)
    {
        AxisSet all;
        for (size_t i = 0; i < os.size(); ++i) all.insert(i);
        sc = make_shared<op::v0::Broadcast>(make_shared<op::v0::Reshape>(scale, AxisVector{0}, Shape{}), os, all);
    }
    else
        sc = make_shared<op::v0::Broadcast>(scale, os, bc);
    v = make_shared<op::v1::Multiply>(v, sc);
    if (sum_in)
    {
        AxisSet all;
        for (size_t i = 0; i < os.size(); ++i) all.insert(i);
        auto ss = make_shared<op::v0::Broadcast>(make_shared<op::v0::Reshape>(sum_scale, AxisVector{0}, Shape{}), os, all);
        v = make_shared<op::v1::Add>(v, make_shared<op::v1::Multiply>(ss, make_shared<op::v0::Convert>(sum_in, element::f32)));
    }
    if (relu) v = make_shared<op::v0::Relu>(v);
    if (out_et == element::f32) return v;
    shared_ptr<Node> zp = out_et == element::u8 ? scalar<uint8_t>(element::u8, 0) : scalar<int8_t>(element::i8, 0);
    return make_shared<op::v0::Quantize>(v, scalar<float>(element::f32, 1.0f), zp, out_et, AxisSet{},
                                         op::v0::Quantize::RoundMode::ROUND_NEAREST_TOWARD_EVEN);
}

static vector<float> log_uniform(Rng& r, size_t n, double lo, double hi)
{
    vector<float> v(n);
    for (auto& s : v) s = float(std::exp(std::log(lo) + r.uni() * (std::log(hi) - std::log(lo))));
    return v;
}

static void fused_dot_cases(Json& j)
{
    int id = 0;
    for (int per_channel = 0; per_channel < 2; ++per_channel)
        for (int mode = 0; mode < 4; ++mode) // f32, f32+relu, i8, u8+relu
        {
            bool requant = mode >= 2, relu = mode & 1;
            element::Type out_et = requant ? (relu ? element::u8 : element::i8) : element::f32;
            Rng r(4000 + id);
            size_t M = 7, K = 48, N = 10;
            Blob A = rand_int_blob<uint8_t>(r, element::u8, Shape{M, K}, 0, 255);
            Blob W = rand_int_blob<int8_t>(r, element::i8, Shape{N, K}, -127, 127);
            Blob Bi = rand_int_blob<int32_t>(r, element::i32, Shape{N}, -1000, 1000);
            Blob S = f32_blob(Shape{per_channel ? N : 1}, log_uniform(r, per_channel ? N : 1, 2e-4, 2e-3));
            auto PA = param_of(A), PW = param_of(W), PB = param_of(Bi), PS = param_of(S);
            auto a32 = make_shared<op::v0::Convert>(PA, element::i32);
            auto w32 = make_shared<op::v0::Reshape>(make_shared<op::v0::Convert>(PW, element::i32), AxisVector{1, 0}, Shape{K, N});
            auto acc = make_shared<op::v0::Dot>(a32, w32, 1);
            auto y = fused_tail(acc, PB, 1, PS, nullptr, nullptr, relu, out_et);
            auto out = run(make_shared<Function>(OutputVector{y}, as_params({PA, PW, PB, PS})), {A, W, Bi, S});
            Case c;
            c.name = "qdot_bias_" + std::to_string(id++);
            c.op = "QuantizedDotBias";
            c.attrs = {{"requantize", requant ? "1" : "0"}, {"relu", relu ? "1" : "0"}};
            c.inputs = {{"data", A}, {"weights", W}, {"bias", Bi}, {"scale", S}};
            c.outputs = {{"y", out[0]}};
            write_case(j, c);
        }
}

static void fused_conv_cases(Json& j)
{
    ConvGeom geoms[3] = {{Shape{2, 64, 6, 5}, Shape{8, 64, 3, 3}, Strides{1, 1}, Strides{1, 1}, CoordinateDiff{1, 1}, CoordinateDiff{1, 1}},
                         {Shape{1, 64, 9, 8}, Shape{4, 64, 3, 3}, Strides{2, 2}, Strides{1, 1}, CoordinateDiff{1, 1}, CoordinateDiff{1, 1}},
                         {Shape{2, 128, 4, 4}, Shape{16, 128, 1, 1}, Strides{1, 1}, Strides{1, 1}, CoordinateDiff{0, 0}, CoordinateDiff{0, 0}}};
    // kind: 0 bias, 1 bias+relu, 2 bias+add+relu (u8 sum), 3 bias+signed add+relu (i8 sum, i8 out then Convert u8), 4 relu only
    int id = 0;
    for (auto& g : geoms)
        for (int kind = 0; kind < 5; ++kind)
            {
                const int per_channel = (id & 1);
                Rng r(5000 + id);
                size_t Kc = g.filt[0];
                Blob D = rand_int_blob<uint8_t>(r, element::u8, g.data, 0, 255);
                Blob F = rand_int_blob<int8_t>(r, element::i8, g.filt, -127, 127);
                Blob Bi = rand_int_blob<int32_t>(r, element::i32, Shape{Kc}, -1000, 1000);
                Blob S = f32_blob(Shape{per_channel ? Kc : 1}, log_uniform(r, per_channel ? Kc : 1, 4e-4, 4e-3));
                bool relu = kind >= 1;
                element::Type out_et = (kind == 0 || kind == 3) ? element::i8 : element::u8;
                auto PD = param_of(D), PF = param_of(F), PB = param_of(Bi), PS = param_of(S);
                auto acc = make_shared<op::v0::QuantizedConvolution>(
                    PD, PF, g.stride, g.dil, g.below, g.above, Strides{1, 1}, scalar<float>(element::f32, 1.0f),
                    scalar<uint8_t>(element::u8, 0), scalar<float>(element::f32, 1.0f), scalar<int8_t>(element::i8, 0),
                    scalar<float>(element::f32, 1.0f), scalar<int32_t>(element::i32, 0), element::i32);
                Shape os = acc->get_output_shape(0);
                vector<shared_ptr<Node>> params{PD, PF, PB, PS};
                vector<Blob> ins{D, F, Bi, S};
                shared_ptr<Node> sum_in, sum_scale;
                Case c;
                if (kind == 2 || kind == 3)
                {
                    Blob Sum = kind == 2 ? rand_int_blob<uint8_t>(r, element::u8, os, 0, 255)
                                         : rand_int_blob<int8_t>(r, element::i8, os, -128, 127);
                    Blob SS = f32_blob(Shape{1}, {float(0.25 + r.uni())});
                    sum_in = param_of(Sum);
                    sum_scale = param_of(SS);
                    params.push_back(sum_in);
                    params.push_back(sum_scale);
                    ins.push_back(Sum);
                    ins.push_back(SS);
                    c.inputs = {{"sum_in", Sum}, {"sum_scale", SS}};
                }
                shared_ptr<Node> y = fused_tail(acc, kind == 4 ? nullptr : PB, 1, PS, sum_in, sum_scale, relu, out_et);
                if (kind == 3) y = make_shared<op::v0::Convert>(y, element::u8);
                auto out = run(make_shared<Function>(OutputVector{y}, as_params(params)), ins);
                static const char* names[5] = {"QuantizedConvolutionBias", "QuantizedConvolutionBiasRelu",
                                               "QuantizedConvolutionBiasAdd", "QuantizedConvolutionBiasSignedAdd",
                                               "QuantizedConvolutionRelu"};
                c.name = "qconv_fused_" + std::to_string(id++);
                c.op = names[kind];
                c.attrs = geom_attrs(g);
                c.attrs.push_back({"relu", relu ? "1" : "0"});
                c.inputs.push_back({"data", D});
                c.inputs.push_back({"filters", F});
                if (kind != 4) c.inputs.push_back({"bias", Bi});
                c.inputs.push_back({"scale", S});
                c.outputs = {{"y", out[0]}};
                write_case(j, c);
            }
}

static void pool_cases(Json& j)
{
    Rng r(6000);
    {
        Blob X = rand_int_blob<uint8_t>(r, element::u8, Shape{2, 16, 9, 9}, 0, 255);
        auto P = param_of(X);
        auto mp = make_shared<op::v0::MaxPool>(P, Shape{3, 3}, Strides{2, 2}, Shape{1, 1}, Shape{1, 1});
        auto out = run(make_shared<Function>(OutputVector{mp}, as_params({P})), {X});
        Case c;
        c.name = "maxpool_u8_0";
        c.op = "MaxPool";
        c.attrs = {{"window", "[3,3]"}, {"stride", "[2,2]"}, {"pad_below", "[1,1]"}, {"pad_above", "[1,1]"}};
        c.inputs = {{"x", X}};
        c.outputs = {{"y", out[0]}};
        write_case(j, c);
    }
    {
        // the global-average head: Dequantize -> AvgPool(f32) -> Quantize (u8 AvgPool itself wraps in uint8)
        Blob X = rand_int_blob<uint8_t>(r, element::u8, Shape{3, 32, 7, 7}, 0, 255);
        float s_in = 0.031f, s_out = 0.017f;
        auto P = param_of(X);
        auto dq = make_shared<op::v0::Dequantize>(P, scalar<float>(element::f32, s_in), scalar<uint8_t>(element::u8, 0),
                                                  element::f32, AxisSet{});
        auto ap = make_shared<op::v0::AvgPool>(dq, Shape{7, 7}, Strides{1, 1});
        auto q = make_shared<op::v0::Quantize>(ap, scalar<float>(element::f32, s_out), scalar<uint8_t>(element::u8, 0),
                                               element::u8, AxisSet{}, op::v0::Quantize::RoundMode::ROUND_NEAREST_TOWARD_EVEN);
        auto out = run(make_shared<Function>(OutputVector{q}, as_params({P})), {X});
        Case c;
        c.name = "global_avgpool_u8_0";
        c.op = "GlobalAvgPoolQ";
        c.inputs = {{"x", X}, {"s_in", f32_blob(Shape{}, {s_in})}, {"s_out", f32_blob(Shape{}, {s_out})}};
        c.outputs = {{"y", out[0]}};
        write_case(j, c);
    }
}

// ---------------------------------------------------------------- builder scales
static shared_ptr<Node> c1(float v) { return op::v0::Constant::create(element::f32, Shape{1}, {v}); }

static vector<float> const_values(const Output<Node>& o)
{
    auto c = std::dynamic_pointer_cast<op::v0::Constant>(o.get_node_shared_ptr());
    if (!c) throw std::runtime_error("scale did not fold to a Constant");
    return c->get_vector<float>();
}

static int scales_main(int argc, char** argv)
{
    if (argc < 11) { fprintf(stderr, "usage: scales <builder> <requantize> <relu> 6 or 8 range values\n"); return 2; }
    string kind = argv[2];
    bool requantize = atoi(argv[3]) != 0, relu = atoi(argv[4]) != 0;
    vector<float> v;
    for (int i = 5; i < argc; ++i) v.push_back(strtof(argv[i], nullptr));
    auto A = make_shared<op::v0::Parameter>(element::u8, Shape{1, 1, 3, 3});
    auto F = make_shared<op::v0::Parameter>(element::i8, Shape{1, 1, 3, 3});
    auto Bi = make_shared<op::v0::Parameter>(element::i32, Shape{1});
    shared_ptr<Node> n;
    ParameterVector pv{A, F, Bi};
    Strides one{1, 1};
    CoordinateDiff pad{1, 1};
    if (kind == "QuantizedConvolutionBiasBuilder")
        n = builder::QuantizedConvolutionBiasBuilder(A, F, Bi, one, one, pad, pad, one, c1(v[0]), c1(v[1]), c1(v[2]), c1(v[3]), c1(v[4]), c1(v[5]), relu);
    else if (kind == "QuantizedConvolutionBiasAddBuilder" || kind == "QuantizedConvolutionBiasSignedAddBuilder")
    {
        bool sgn = kind == "QuantizedConvolutionBiasSignedAddBuilder";
        auto Sum = make_shared<op::v0::Parameter>(sgn ? element::i8 : element::u8, Shape{1, 1, 3, 3});
        pv.push_back(Sum);
        n = sgn ? builder::QuantizedConvolutionBiasSignedAddBuilder(A, F, Bi, Sum, one, one, pad, pad, one, c1(v[0]), c1(v[1]), c1(v[2]), c1(v[3]), c1(v[4]), c1(v[5]), c1(v[6]), c1(v[7]), relu)
                : builder::QuantizedConvolutionBiasAddBuilder(A, F, Bi, Sum, one, one, pad, pad, one, c1(v[0]), c1(v[1]), c1(v[2]), c1(v[3]), c1(v[4]), c1(v[5]), c1(v[6]), c1(v[7]), relu);
    }
    else if (kind == "QuantizedDotBiasBuilder")
    {
        auto A2 = make_shared<op::v0::Parameter>(element::u8, Shape{4, 3});
        auto W2 = make_shared<op::v0::Parameter>(element::i8, Shape{3, 3});
        auto B2 = make_shared<op::v0::Parameter>(element::i32, Shape{3});
        pv = ParameterVector{A2, W2, B2};
        n = builder::QuantizedDotBiasBuilder(A2, W2, B2, c1(v[0]), c1(v[1]), c1(v[2]), c1(v[3]), c1(v[4]), c1(v[5]), requantize, relu);
    }
    else { fprintf(stderr, "unknown builder %s\n", kind.c_str()); return 2; }
    auto f = make_shared<Function>(OutputVector{n}, pv);
    pass::Manager pm;
    pm.register_pass<pass::ConstantFolding>();
    pm.run_passes(f);
    // find the fused node (the SignedAdd builder wraps it in a Convert)
    shared_ptr<Node> fused;
    for (auto& node : f->get_ordered_ops())
        if (string(node->get_type_name()).find("Quantized") == 0) fused = node;
    if (!fused) throw std::runtime_error("no fused node found");
    size_t scale_idx = string(fused->get_type_name()) == "QuantizedDotBias" ? 3
                       : fused->get_input_size() == 4 ? 3 : 4;
    auto bits = [](float x) { uint32_t u; memcpy(&u, &x, 4); return u; };
    std::cout << "{\"op\":\"" << fused->get_type_name() << "\",\"scale_bits\":" << bits(const_values(fused->input_value(scale_idx))[0]);
    if (fused->get_input_size() == 6)
        std::cout << ",\"sum_scale_bits\":" << bits(const_values(fused->input_value(5))[0]);
    std::cout << "}\n";
    return 0;
}

int main(int argc, char** argv)
{
    try
    {
        if (argc >= 3 && string(argv[1]) == "interp")
        {
            Json j;
            j.os << "[\n";
            quantize_cases(j);
            qdot_core_cases(j);
            qconv_core_cases(j);
            fused_dot_cases(j);
            fused_conv_cases(j);
            pool_cases(j);
            j.os << "\n]\n";
            std::ofstream(argv[2]) << j.os.str();
            return 0;
        }
        if (argc >= 2 && string(argv[1]) == "scales") return scales_main(argc, argv);
        fprintf(stderr, "usage: gen_golden interp <out.json> | scales ...\n");
        return 2;
    }
    catch (const std::exception& e)
    {
        fprintf(stderr, "gen_golden: %s\n", e.what());
        return 1;
    }
}

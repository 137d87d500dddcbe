// Non-zero input / filter zero points for the core quantized contractions.
//
// runtime::reference::convolution (src/ngraph/runtime/reference/convolution.hpp:236-258) and reference::dot
// (dot.hpp:134-159) subtract the zero points from every operand pair before they multiply,
//     acc = sum over the taps INSIDE the image, over channels, of (a - za) * (w - zw)
// (a padded tap is skipped altogether, i.e. padding behaves like the zero point), and requantise acc once.
// The tensor-core contraction computes S = sum a * w with zero padding; the rest is rank-one:
//     acc = S - zw * A(n,p,q) - za * W(k, valid taps) + (number of valid taps) * C * za * zw
// with A = the sum of the input window (padding counts 0) and W = the sum of the filter over the valid taps.  Both sums
// are tiny next to S, so they are made by plain kernels and applied in one pass over the int32 accumulators that also
// does the reference's requantisation.  Everything is int32 arithmetic like the reference's accumulator.
#include "common.cuh"

namespace b200
{
    // out[o * n_inner + i] = sum_{c < n_sum} x[o * outer_stride + i * inner_stride + c * sum_stride]
    template <typename T>
    __global__ void __launch_bounds__(256) strided_sums_kernel(const T* __restrict__ x, int32_t* __restrict__ out, int64_t n_outer,
                                                               int64_t n_inner, int64_t n_sum, int64_t outer_stride, int64_t inner_stride,
                                                               int64_t sum_stride)
    {
        const int64_t total = n_outer * n_inner;
        for (int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += int64_t(gridDim.x) * blockDim.x)
        {
            const T* base = x + (t / n_inner) * outer_stride + (t % n_inner) * inner_stride;
            int32_t s = 0;
            for (int64_t c = 0; c < n_sum; ++c)
                s += int32_t(base[c * sum_stride]);
            out[t] = s;
        }
    }

    struct Window
    {
        int N, P, Q, K, H, W, C, R, S, stride_h, stride_w, dil_h, dil_w, pad_h, pad_w;
    };

    // out[n, p, q] = the sum of pixel_sums[n, h, w] over the taps of output (p, q) that fall inside the image
    __global__ void __launch_bounds__(256) window_sums_kernel(const int32_t* __restrict__ pixel_sums, int32_t* __restrict__ out, Window g)
    {
        const int64_t total = int64_t(g.N) * g.P * g.Q;
        for (int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += int64_t(gridDim.x) * blockDim.x)
        {
            const int q = int(t % g.Q), p = int((t / g.Q) % g.P);
            const int64_t n = t / (int64_t(g.Q) * g.P);
            int32_t s = 0;
            for (int r = 0; r < g.R; ++r)
            {
                const int h = p * g.stride_h - g.pad_h + r * g.dil_h;
                if (h < 0 || h >= g.H)
                    continue;
                for (int c = 0; c < g.S; ++c)
                {
                    const int w = q * g.stride_w - g.pad_w + c * g.dil_w;
                    if (w >= 0 && w < g.W)
                        s += pixel_sums[(n * g.H + h) * g.W + w];
                }
            }
            out[t] = s;
        }
    }

    template <int OUT>
    __global__ void __launch_bounds__(256) requant_zero_points_kernel(const int32_t* __restrict__ acc, const int32_t* __restrict__ tap_sums,
                                                                      const int32_t* __restrict__ window_sums, Window g, int32_t za, int32_t zw,
                                                                      const float* __restrict__ scale_p, int32_t out_zp, void* __restrict__ out)
    {
        const float scale = __ldg(scale_p);
        const int64_t total = int64_t(g.N) * g.P * g.Q * g.K;
        const int taps = g.R * g.S;
        for (int64_t t = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; t < total; t += int64_t(gridDim.x) * blockDim.x)
        {
            const int k = int(t % g.K);
            const int64_t pix = t / g.K; // (n, p, q)
            const int q = int(pix % g.Q), p = int((pix / g.Q) % g.P);
            uint32_t filter_part = 0, valid = 0;
            for (int r = 0; r < g.R; ++r)
            {
                const int h = p * g.stride_h - g.pad_h + r * g.dil_h;
                if (h < 0 || h >= g.H)
                    continue;
                for (int c = 0; c < g.S; ++c)
                {
                    const int w = q * g.stride_w - g.pad_w + c * g.dil_w;
                    if (w < 0 || w >= g.W)
                        continue;
                    ++valid;
                    if (tap_sums)
                        filter_part += uint32_t(tap_sums[k * taps + r * g.S + c]);
                }
            }
            // modulo 2^32 like the reference's int32 accumulator on two's-complement hardware
            uint32_t u = uint32_t(acc[t]);
            if (window_sums)
                u -= uint32_t(zw) * uint32_t(window_sums[pix]);
            u -= uint32_t(za) * filter_part;
            u += valid * uint32_t(g.C) * uint32_t(za) * uint32_t(zw);
            const int32_t a = int32_t(u);
            // dot.hpp:152-159 / convolution.hpp:252-258: (OUT)round(float(acc) * scale) + zero point, saturated here
            const float r = roundf(__fmul_rn(__int2float_rn(a), scale));
            long long v = __float2ll_rn(r) + static_cast<long long>(out_zp);
            const long long lo = OUT == B200_U8 ? 0ll : OUT == B200_I8 ? -128ll : -2147483648ll;
            const long long hi = OUT == B200_U8 ? 255ll : OUT == B200_I8 ? 127ll : 2147483647ll;
            v = v < lo ? lo : (v > hi ? hi : v);
            if (r != r)
                v = 0;
            if (OUT == B200_I32)
                static_cast<int32_t*>(out)[t] = int32_t(v);
            else
                static_cast<uint8_t*>(out)[t] = uint8_t(v);
        }
    }

    static unsigned blocks_for(int64_t n)
    {
        const int64_t blocks = (n + 255) / 256, cap = b200::sm_count() * 16;
        return unsigned(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
    }

    static bool to_window(const b200_zero_point_params* z, Window& g)
    {
        const int64_t v[] = {z->N, z->P, z->Q, z->K, z->H, z->W, z->C, z->R, z->S, z->stride_h, z->stride_w, z->dilation_h, z->dilation_w};
        for (int64_t x : v)
            if (x < 1 || x > 0x7FFFFFFF)
                return false;
        if (z->pad_h < 0 || z->pad_w < 0 || z->pad_h > 0x7FFFFFFF || z->pad_w > 0x7FFFFFFF || z->R * z->S > 0x7FFFFFFF)
            return false;
        g = Window{int(z->N), int(z->P), int(z->Q), int(z->K), int(z->H), int(z->W), int(z->C), int(z->R), int(z->S), int(z->stride_h),
                   int(z->stride_w), int(z->dilation_h), int(z->dilation_w), int(z->pad_h), int(z->pad_w)};
        return true;
    }
}

extern "C" int b200_strided_sums(const void* x, int x_type, int32_t* out, int64_t n_outer, int64_t n_inner, int64_t n_sum,
                                 int64_t outer_stride, int64_t inner_stride, int64_t sum_stride, void* stream)
{
    using namespace b200;
    if (n_outer < 0 || n_inner < 0 || n_sum < 0 || outer_stride < 0 || inner_stride < 0 || sum_stride < 0 ||
        (x_type != B200_U8 && x_type != B200_I8))
        return B200_ERR_INVALID_ARGUMENT;
    if (n_outer * n_inner == 0)
        return B200_OK;
    if (!out || (!x && n_sum > 0))
        return B200_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (x_type == B200_U8)
        strided_sums_kernel<uint8_t><<<blocks_for(n_outer * n_inner), 256, 0, st>>>(static_cast<const uint8_t*>(x), out, n_outer, n_inner,
                                                                                     n_sum, outer_stride, inner_stride, sum_stride);
    else
        strided_sums_kernel<int8_t><<<blocks_for(n_outer * n_inner), 256, 0, st>>>(static_cast<const int8_t*>(x), out, n_outer, n_inner,
                                                                                    n_sum, outer_stride, inner_stride, sum_stride);
    return after_launch("b200_strided_sums");
}

extern "C" int b200_window_sums(const int32_t* pixel_sums, int32_t* out, const b200_zero_point_params* z, void* stream)
{
    using namespace b200;
    Window g;
    if (!z || !to_window(z, g) || !pixel_sums || !out)
        return B200_ERR_INVALID_ARGUMENT;
    window_sums_kernel<<<blocks_for(int64_t(g.N) * g.P * g.Q), 256, 0, static_cast<cudaStream_t>(stream)>>>(pixel_sums, out, g);
    return after_launch("b200_window_sums");
}

extern "C" int b200_requant_zero_points(const int32_t* acc, const int32_t* filter_tap_sums, const int32_t* window_sums,
                                        const b200_zero_point_params* z, const b200_epilogue* e, void* out, void* stream)
{
    using namespace b200;
    Window g;
    if (!z || !e || !to_window(z, g) || !acc || !out || !e->scale || e->round_half_away != 1 || e->scale_count != 1 || e->bias ||
        e->sum_in || e->relu)
        return B200_ERR_INVALID_ARGUMENT;
    // a sum that a non-zero zero point multiplies has to be there
    if ((z->input_zero_point != 0 && !filter_tap_sums) || (z->filter_zero_point != 0 && !window_sums))
        return B200_ERR_INVALID_ARGUMENT;
    const int32_t za = z->input_zero_point, zw = z->filter_zero_point;
    const int32_t* taps = za != 0 ? filter_tap_sums : nullptr;
    const int32_t* wins = zw != 0 ? window_sums : nullptr;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = blocks_for(int64_t(g.N) * g.P * g.Q * g.K);
    switch (e->out_type)
    {
    case B200_U8: requant_zero_points_kernel<B200_U8><<<grid, 256, 0, st>>>(acc, taps, wins, g, za, zw, e->scale, e->out_zero_point, out); break;
    case B200_I8: requant_zero_points_kernel<B200_I8><<<grid, 256, 0, st>>>(acc, taps, wins, g, za, zw, e->scale, e->out_zero_point, out); break;
    case B200_I32: requant_zero_points_kernel<B200_I32><<<grid, 256, 0, st>>>(acc, taps, wins, g, za, zw, e->scale, e->out_zero_point, out); break;
    default: return B200_ERR_INVALID_ARGUMENT;
    }
    return after_launch("b200_requant_zero_points");
}

// Layout conversions for 1-byte tensors (graph edges and weight packing), and the u8
// pooling glue of whole-graph inference.  All of them are plain HBM-bound byte movers.
#include "common.cuh"

#include <type_traits>

namespace b200
{
    constexpr int TT = 32; // transpose tile edge

    // in: [batch, rows, cols] -> out: [batch, cols, rows_pad]; columns >= rows of the output are zero.
    __global__ void __launch_bounds__(256) transpose_bytes_kernel(const uint8_t* __restrict__ in,
                                                                  uint8_t* __restrict__ out, int64_t rows,
                                                                  int64_t cols, int64_t rows_pad)
    {
        __shared__ uint8_t tile[TT][TT + 4];
        const int64_t b = blockIdx.z;
        const int64_t r0 = int64_t(blockIdx.y) * TT, c0 = int64_t(blockIdx.x) * TT;
        const uint8_t* ip = in + b * rows * cols;
        uint8_t* op = out + b * cols * rows_pad;
        const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5; // 32 x 8
        for (int j = ty; j < TT; j += 8)
        {
            int64_t r = r0 + j, c = c0 + tx;
            tile[j][tx] = (r < rows && c < cols) ? ip[r * cols + c] : uint8_t(0);
        }
        __syncthreads();
        for (int j = ty; j < TT; j += 8)
        {
            int64_t c = c0 + j, r = r0 + tx;
            if (c < cols && r < rows_pad)
                op[c * rows_pad + r] = tile[tx][j];
        }
    }

    // in: [batch, rows, cols_pad] (only cols < cols_used... ) -> out [batch, cols, rows]
    __global__ void __launch_bounds__(256) untranspose_bytes_kernel(const uint8_t* __restrict__ in,
                                                                    uint8_t* __restrict__ out, int64_t rows,
                                                                    int64_t cols, int64_t cols_pad)
    {
        __shared__ uint8_t tile[TT][TT + 4];
        const int64_t b = blockIdx.z;
        const int64_t r0 = int64_t(blockIdx.y) * TT, c0 = int64_t(blockIdx.x) * TT;
        const uint8_t* ip = in + b * rows * cols_pad;
        uint8_t* op = out + b * cols * rows;
        const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
        for (int j = ty; j < TT; j += 8)
        {
            int64_t r = r0 + j, c = c0 + tx;
            tile[j][tx] = (r < rows && c < cols) ? ip[r * cols_pad + c] : uint8_t(0);
        }
        __syncthreads();
        for (int j = ty; j < TT; j += 8)
        {
            int64_t c = c0 + j, r = r0 + tx;
            if (c < cols && r < rows)
                op[c * rows + r] = tile[tx][j];
        }
    }

    static int launch_transpose(const void* in, void* out, int64_t batch, int64_t rows, int64_t cols, int64_t rows_pad,
                                cudaStream_t st, const char* what)
    {
        if (batch == 0 || rows == 0 || cols == 0)
            return B200_OK;
        int64_t rmax = rows_pad > rows ? rows_pad : rows;
        dim3 grid(unsigned((cols + TT - 1) / TT), unsigned((rmax + TT - 1) / TT), unsigned(batch));
        if (grid.y > 65535 || grid.z > 65535)
            return B200_ERR_TOO_LARGE;
        transpose_bytes_kernel<<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), rows,
                                                     cols, rows_pad);
        return after_launch(what);
    }

    // ---- pooling on channels-last u8 --------------------------------------------------------

    // MaxPool: runtime::reference::max_pool (runtime/reference/max_pool.hpp:124-236), padding positions skipped.
    // One thread per 16 channels of one output pixel (128-bit loads, __vmaxu4; SIGNED: i8 elements, __vmaxs4).
    template <bool SIGNED>
    __global__ void __launch_bounds__(256) maxpool_nhwc_u8_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out,
                                                                  int N, int H, int W, int C16, int P, int Q, int win_h,
                                                                  int win_w, int stride_h, int stride_w, int pad_h,
                                                                  int pad_w)
    {
        int64_t total = int64_t(N) * P * Q * C16;
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x)
        {
            int c = int(i % C16);
            int64_t t = i / C16;
            int q = int(t % Q);
            t /= Q;
            int p = int(t % P);
            int n = int(t / P);
            const uint32_t lowest = SIGNED ? 0x80808080u : 0u; // the identity of the max: -128 / 0 in every byte
            uint4 m = make_uint4(lowest, lowest, lowest, lowest);
            for (int r = 0; r < win_h; ++r)
            {
                int h = p * stride_h - pad_h + r;
                if (h < 0 || h >= H)
                    continue;
                for (int s = 0; s < win_w; ++s)
                {
                    int w = q * stride_w - pad_w + s;
                    if (w < 0 || w >= W)
                        continue;
                    uint4 v = reinterpret_cast<const uint4*>(in)[((int64_t(n) * H + h) * W + w) * C16 + c];
                    m.x = SIGNED ? __vmaxs4(m.x, v.x) : __vmaxu4(m.x, v.x);
                    m.y = SIGNED ? __vmaxs4(m.y, v.y) : __vmaxu4(m.y, v.y);
                    m.z = SIGNED ? __vmaxs4(m.z, v.z) : __vmaxu4(m.z, v.z);
                    m.w = SIGNED ? __vmaxs4(m.w, v.w) : __vmaxu4(m.w, v.w);
                }
            }
            reinterpret_cast<uint4*>(out)[i] = m;
        }
    }

    // The same with the window size known at compile time: all window loads are issued before the first
    // max (out-of-image taps read as 0, the identity of an unsigned max), index arithmetic in 32 bits.
    template <int WH, int WW>
    __global__ void __launch_bounds__(256) maxpool_nhwc_u8_fixed_kernel(const uint4* __restrict__ in, uint4* __restrict__ out,
                                                                        int N, int H, int W, int C16, int P, int Q, int stride_h,
                                                                        int stride_w, int pad_h, int pad_w)
    {
        const uint32_t total = uint32_t(N) * P * Q * C16;
        for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x)
        {
            uint32_t c = i % C16, t = i / C16;
            uint32_t q = t % Q;
            t /= Q;
            uint32_t p = t % P, n = t / P;
            const int h0 = int(p) * stride_h - pad_h, w0 = int(q) * stride_w - pad_w;
            uint4 v[WH * WW];
#pragma unroll
            for (int r = 0; r < WH; ++r)
#pragma unroll
                for (int s = 0; s < WW; ++s)
                {
                    const int h = h0 + r, w = w0 + s;
                    const bool ok = h >= 0 && h < H && w >= 0 && w < W;
                    v[r * WW + s] = ok ? in[(size_t(n) * H + h) * W * C16 + size_t(w) * C16 + c] : make_uint4(0, 0, 0, 0);
                }
            uint4 m = v[0];
#pragma unroll
            for (int k = 1; k < WH * WW; ++k)
            {
                m.x = __vmaxu4(m.x, v[k].x);
                m.y = __vmaxu4(m.y, v[k].y);
                m.z = __vmaxu4(m.z, v[k].z);
                m.w = __vmaxu4(m.w, v[k].w);
            }
            out[i] = m;
        }
    }

    // The 3x3 / stride 2 window of the network stems with TWO neighbouring output pixels per thread: their windows share a
    // column, so 15 instead of 18 loads serve 32 output bytes, and a thread keeps 240 bytes in flight (the kernel is bound by
    // load latency).  Out-of-image taps read as 0, the identity of an unsigned max.
    __global__ void __launch_bounds__(256) maxpool_nhwc_u8_3x3s2_pair_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int N, int H,
                                                                             int W, int C16, int P, int Q, int pad_h, int pad_w)
    {
        const uint32_t Q2 = uint32_t(Q + 1) / 2;
        const uint32_t total = uint32_t(N) * P * Q2 * C16;
        for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x)
        {
            uint32_t c = i % C16, t = i / C16;
            const uint32_t q2 = t % Q2;
            t /= Q2;
            const uint32_t p = t % P, n = t / P;
            const int h0 = 2 * int(p) - pad_h, w0 = 4 * int(q2) - pad_w; // columns w0 .. w0 + 4 serve outputs 2 q2 and 2 q2 + 1
            uint4 v[3][5];
#pragma unroll
            for (int r = 0; r < 3; ++r)
#pragma unroll
                for (int sx = 0; sx < 5; ++sx)
                {
                    const int h = h0 + r, w = w0 + sx;
                    const bool ok = h >= 0 && h < H && w >= 0 && w < W;
                    v[r][sx] = ok ? in[(size_t(n) * H + h) * W * C16 + size_t(w) * C16 + c] : make_uint4(0, 0, 0, 0);
                }
            // Byte-wise maxima through the three-input 16-bit-lane maximum the hardware has (__vimax3_u16x2), since the byte-lane
            // SIMD maximum is emulated: the even and the odd bytes of a word are spread into two words of 16-bit lanes (one byte
            // permute each), three rows give a column's maximum in one instruction per word half, three columns an output's, and
            // a last permute interleaves the halves again.
            const uint32_t(*vw)[5][4] = reinterpret_cast<const uint32_t(*)[5][4]>(v);
            uint32_t ce[5][4], co[5][4]; // per column and word: maxima of the even / odd bytes over the three rows
#pragma unroll
            for (int sx = 0; sx < 5; ++sx)
#pragma unroll
                for (int k = 0; k < 4; ++k)
                {
                    ce[sx][k] = __vimax3_u16x2(__byte_perm(vw[0][sx][k], 0, 0x4240), __byte_perm(vw[1][sx][k], 0, 0x4240),
                                               __byte_perm(vw[2][sx][k], 0, 0x4240));
                    co[sx][k] = __vimax3_u16x2(__byte_perm(vw[0][sx][k], 0, 0x4341), __byte_perm(vw[1][sx][k], 0, 0x4341),
                                               __byte_perm(vw[2][sx][k], 0, 0x4341));
                }
            auto max3 = [&](int s0) {
                uint32_t r[4];
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    r[k] = __byte_perm(__vimax3_u16x2(ce[s0][k], ce[s0 + 1][k], ce[s0 + 2][k]),
                                       __vimax3_u16x2(co[s0][k], co[s0 + 1][k], co[s0 + 2][k]), 0x6240);
                return make_uint4(r[0], r[1], r[2], r[3]);
            };
            const size_t o = ((size_t(n) * P + p) * Q + 2 * size_t(q2)) * C16 + c;
            out[o] = max3(0);
            if (2 * q2 + 1 < uint32_t(Q))
                out[o + C16] = max3(2);
        }
    }

    // Global average head on channels-last u8: Dequantize(s_in, zp 0) -> AvgPool over H x W
    // (runtime::reference::avg_pool: sequential float sum in H,W order, one division by the count)
    // -> Quantize(s_out, zp 0, ROUND_NEAREST_TOWARD_EVEN).  One thread per (n, c); threads of a warp
    // read consecutive channels, so every pixel row is a coalesced read.
    __global__ void __launch_bounds__(256) global_avgpool_q_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out,
                                                                   const float* __restrict__ s_in,
                                                                   const float* __restrict__ s_out, int N, int HW, int C)
    {
        int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
        if (i >= int64_t(N) * C)
            return;
        int n = int(i / C), c = int(i % C);
        const float si = *s_in, so = *s_out;
        const uint8_t* ip = in + int64_t(n) * HW * C + c;
        float acc = 0.0f;
        for (int j = 0; j < HW; ++j)
            acc = __fadd_rn(acc, __fmul_rn(static_cast<float>(int(ip[int64_t(j) * C])), si));
        float avg = __fdiv_rn(acc, static_cast<float>(HW));
        out[i] = quantize_one<uint8_t, B200_ROUND_NEAREST_TOWARD_EVEN>(avg, so, 0.0f);
    }
}

namespace b200
{
    // ---- AvgPool ------------------------------------------------------------------------------------------------
    // runtime::reference::avg_pool (runtime/reference/avg_pool.hpp:160-236): the window is walked in (h, w) order over the
    // PADDED image; a position inside the image adds its value and counts, a padding position adds 0 and counts only when
    // include_padding_in_avg_computation is set; the result is sum / count, summed sequentially in the element type.
    // Window positions beyond the padded image (ceil mode) do not exist for the reference (it refuses them): they are
    // never counted here.
    struct PoolGeom
    {
        int N, C, H, W, P, Q, win_h, win_w, stride_h, stride_w, pad_h, pad_w, pad_h_above, pad_w_above, include_padding;
    };

    // f32, NCHW in and out: one thread per output element
    __global__ void __launch_bounds__(256) avgpool_f32_nchw_kernel(const float* __restrict__ in, float* __restrict__ out, PoolGeom g)
    {
        const int64_t total = int64_t(g.N) * g.C * g.P * g.Q;
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x)
        {
            const int q = int(i % g.Q);
            int64_t t = i / g.Q;
            const int p = int(t % g.P);
            const int64_t nc = t / g.P;
            const float* img = in + nc * g.H * g.W;
            float acc = 0.0f;
            int count = 0;
            for (int r = 0; r < g.win_h; ++r)
            {
                const int h = p * g.stride_h - g.pad_h + r;
                if (h >= g.H + g.pad_h_above)
                    break;
                for (int sx = 0; sx < g.win_w; ++sx)
                {
                    const int w = q * g.stride_w - g.pad_w + sx;
                    if (w >= g.W + g.pad_w_above)
                        break;
                    const bool inside = h >= 0 && h < g.H && w >= 0 && w < g.W;
                    if (inside || g.include_padding)
                    {
                        acc = __fadd_rn(acc, inside ? img[int64_t(h) * g.W + w] : 0.0f);
                        ++count;
                    }
                }
            }
            // the reference throws when a window holds no element; the host side refuses such geometries
            out[i] = __fdiv_rn(acc, static_cast<float>(count));
        }
    }

    // u8 / i8 AvgPool op, channels-last: the reference instantiated for a one-byte element type keeps the running sum IN
    // that type (it wraps modulo 256) and stores nearbyint(float(sum) / count); reproduced literally.
    template <bool SIGNED>
    __global__ void __launch_bounds__(256) avgpool_bytes_nhwc_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, PoolGeom g)
    {
        const int64_t total = int64_t(g.N) * g.P * g.Q * g.C;
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x)
        {
            const int c = int(i % g.C);
            int64_t t = i / g.C;
            const int q = int(t % g.Q);
            t /= g.Q;
            const int p = int(t % g.P);
            const int n = int(t / g.P);
            uint32_t sum = 0; // only the low byte is the reference's running sum
            int count = 0;
            for (int r = 0; r < g.win_h; ++r)
            {
                const int h = p * g.stride_h - g.pad_h + r;
                if (h >= g.H + g.pad_h_above)
                    break;
                for (int sx = 0; sx < g.win_w; ++sx)
                {
                    const int w = q * g.stride_w - g.pad_w + sx;
                    if (w >= g.W + g.pad_w_above)
                        break;
                    const bool inside = h >= 0 && h < g.H && w >= 0 && w < g.W;
                    if (inside || g.include_padding)
                    {
                        if (inside)
                            sum += in[((int64_t(n) * g.H + h) * g.W + w) * g.C + c];
                        ++count;
                    }
                }
            }
            const float s = SIGNED ? static_cast<float>(static_cast<int8_t>(sum & 0xFF)) : static_cast<float>(sum & 0xFF);
            const float avg = rintf(__fdiv_rn(s, static_cast<float>(count))); // nearbyint under round-to-nearest-even
            out[i] = SIGNED ? uint8_t(static_cast<int8_t>(avg)) : static_cast<uint8_t>(avg);
        }
    }

    // Dequantize(s_in, zp 0) -> AvgPool(f32, any window) -> Quantize(s_out, zp 0, ROUND_NEAREST_TOWARD_EVEN) on channels-last
    // bytes in one pass, every float operation of the three ops in their order: the windowed form of the pooling head.
    template <typename IN, typename OUT>
    __global__ void __launch_bounds__(256) avgpool_q_nhwc_kernel(const IN* __restrict__ in, OUT* __restrict__ out,
                                                                 const float* __restrict__ s_in, const float* __restrict__ s_out,
                                                                 PoolGeom g)
    {
        const float si = *s_in, so = *s_out;
        const int64_t total = int64_t(g.N) * g.P * g.Q * g.C;
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x)
        {
            const int c = int(i % g.C);
            int64_t t = i / g.C;
            const int q = int(t % g.Q);
            t /= g.Q;
            const int p = int(t % g.P);
            const int n = int(t / g.P);
            float acc = 0.0f;
            int count = 0;
            for (int r = 0; r < g.win_h; ++r)
            {
                const int h = p * g.stride_h - g.pad_h + r;
                if (h >= g.H + g.pad_h_above)
                    break;
                for (int sx = 0; sx < g.win_w; ++sx)
                {
                    const int w = q * g.stride_w - g.pad_w + sx;
                    if (w >= g.W + g.pad_w_above)
                        break;
                    const bool inside = h >= 0 && h < g.H && w >= 0 && w < g.W;
                    if (inside || g.include_padding)
                    {
                        const float v = inside ? __fmul_rn(static_cast<float>(int(in[((int64_t(n) * g.H + h) * g.W + w) * g.C + c])), si) : 0.0f;
                        acc = __fadd_rn(acc, v);
                        ++count;
                    }
                }
            }
            out[i] = quantize_one<OUT, B200_ROUND_NEAREST_TOWARD_EVEN>(__fdiv_rn(acc, static_cast<float>(count)), so, 0.0f);
        }
    }

    // every output window must hold at least one counted element, and the sizes must fit the kernels' int fields
    static int check_pool_geom(const b200_pool_params* g, PoolGeom& k)
    {
        if (!g || g->N < 0 || g->C <= 0 || g->H <= 0 || g->W <= 0 || g->P < 0 || g->Q < 0 || g->win_h <= 0 || g->win_w <= 0 ||
            g->stride_h <= 0 || g->stride_w <= 0 || g->pad_h < 0 || g->pad_w < 0 || g->pad_h_above < 0 || g->pad_w_above < 0)
            return B200_ERR_INVALID_ARGUMENT;
        const int64_t big = int64_t(1) << 30;
        if (g->N >= big || g->C >= big || g->H >= big || g->W >= big || g->P >= big || g->Q >= big || g->win_h >= big || g->win_w >= big ||
            g->stride_h >= big || g->stride_w >= big || g->pad_h >= big || g->pad_w >= big || g->pad_h_above >= big || g->pad_w_above >= big)
            return B200_ERR_TOO_LARGE;
        if (g->P > 0 && g->Q > 0)
        {
            // the last window starts inside the padded image, and (without include_padding) reaches the image itself;
            // the first windows must reach it too
            const int64_t h_last = (g->P - 1) * g->stride_h - g->pad_h, w_last = (g->Q - 1) * g->stride_w - g->pad_w;
            if (h_last >= g->H + g->pad_h_above || w_last >= g->W + g->pad_w_above)
                return B200_ERR_INVALID_ARGUMENT;
            if (!g->include_padding && (h_last >= g->H || w_last >= g->W || g->win_h <= g->pad_h || g->win_w <= g->pad_w))
                return B200_ERR_INVALID_ARGUMENT;
        }
        k = PoolGeom{int(g->N), int(g->C), int(g->H), int(g->W), int(g->P), int(g->Q), int(g->win_h), int(g->win_w), int(g->stride_h),
                     int(g->stride_w), int(g->pad_h), int(g->pad_w), int(g->pad_h_above), int(g->pad_w_above), g->include_padding ? 1 : 0};
        return B200_OK;
    }

    static unsigned pool_grid(int64_t total)
    {
        const int64_t blocks = (total + 255) / 256, cap = int64_t(sm_count()) * 32;
        return unsigned(blocks < cap ? blocks : cap);
    }
}

extern "C" int b200_avgpool_f32_nchw(const float* in, float* out, const b200_pool_params* geometry, void* stream)
{
    using namespace b200;
    PoolGeom g;
    int rc = check_pool_geom(geometry, g);
    if (rc != B200_OK)
        return rc;
    const int64_t total = int64_t(g.N) * g.C * g.P * g.Q;
    if (total == 0)
        return B200_OK;
    if (!in || !out)
        return B200_ERR_INVALID_ARGUMENT;
    avgpool_f32_nchw_kernel<<<pool_grid(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(in, out, g);
    return after_launch("b200_avgpool_f32_nchw");
}

extern "C" int b200_avgpool_nhwc_bytes(const void* in, void* out, int type, const b200_pool_params* geometry, void* stream)
{
    using namespace b200;
    PoolGeom g;
    int rc = check_pool_geom(geometry, g);
    if (rc != B200_OK)
        return rc;
    if (type != B200_U8 && type != B200_I8)
        return B200_ERR_INVALID_ARGUMENT;
    const int64_t total = int64_t(g.N) * g.C * g.P * g.Q;
    if (total == 0)
        return B200_OK;
    if (!in || !out)
        return B200_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (type == B200_I8)
        avgpool_bytes_nhwc_kernel<true><<<pool_grid(total), 256, 0, st>>>(static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), g);
    else
        avgpool_bytes_nhwc_kernel<false><<<pool_grid(total), 256, 0, st>>>(static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), g);
    return after_launch("b200_avgpool_nhwc_bytes");
}

extern "C" int b200_avgpool_q_nhwc(const void* in, int in_type, void* out, int out_type, const float* scale_in, const float* scale_out,
                                   const b200_pool_params* geometry, void* stream)
{
    using namespace b200;
    PoolGeom g;
    int rc = check_pool_geom(geometry, g);
    if (rc != B200_OK)
        return rc;
    if ((in_type != B200_U8 && in_type != B200_I8) || (out_type != B200_U8 && out_type != B200_I8))
        return B200_ERR_INVALID_ARGUMENT;
    const int64_t total = int64_t(g.N) * g.C * g.P * g.Q;
    if (total == 0)
        return B200_OK;
    if (!in || !out || !scale_in || !scale_out)
        return B200_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned grid = pool_grid(total);
    const uint8_t* iu = static_cast<const uint8_t*>(in);
    const int8_t* is = static_cast<const int8_t*>(in);
    if (in_type == B200_U8 && out_type == B200_U8)
        avgpool_q_nhwc_kernel<uint8_t, uint8_t><<<grid, 256, 0, st>>>(iu, static_cast<uint8_t*>(out), scale_in, scale_out, g);
    else if (in_type == B200_U8)
        avgpool_q_nhwc_kernel<uint8_t, int8_t><<<grid, 256, 0, st>>>(iu, static_cast<int8_t*>(out), scale_in, scale_out, g);
    else if (out_type == B200_U8)
        avgpool_q_nhwc_kernel<int8_t, uint8_t><<<grid, 256, 0, st>>>(is, static_cast<uint8_t*>(out), scale_in, scale_out, g);
    else
        avgpool_q_nhwc_kernel<int8_t, int8_t><<<grid, 256, 0, st>>>(is, static_cast<int8_t*>(out), scale_in, scale_out, g);
    return after_launch("b200_avgpool_q_nhwc");
}

namespace b200
{
    // Data dilation and negative padding of a convolution, materialised: the channels-last input with dil - 1 zero pixels
    // inserted between neighbours and crop pixels cut off each border of the dilated image.  Inserted pixels are zero BYTES:
    // the reference never visits them (they are not source coordinates, runtime/reference/convolution.hpp:227-251), and a zero
    // byte contributes nothing to the accumulator.  One thread per 16 channels of one output pixel.
    __global__ void __launch_bounds__(256) dilate_crop_nhwc_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, int N, int H, int W,
                                                                   int C16, int Ho, int Wo, int dil_h, int dil_w, int crop_h, int crop_w)
    {
        const int64_t total = int64_t(N) * Ho * Wo * C16;
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x)
        {
            const int c = int(i % C16);
            int64_t t = i / C16;
            const int x = int(t % Wo);
            t /= Wo;
            const int y = int(t % Ho);
            const int n = int(t / Ho);
            const int yy = y + crop_h, xx = x + crop_w;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (yy % dil_h == 0 && xx % dil_w == 0 && yy / dil_h < H && xx / dil_w < W)
                v = in[((int64_t(n) * H + yy / dil_h) * W + xx / dil_w) * C16 + c];
            out[i] = v;
        }
    }
}

extern "C" int b200_dilate_crop_nhwc_u8(const void* in, void* out, int64_t N, int64_t H, int64_t W, int64_t C, int64_t dilation_h,
                                        int64_t dilation_w, int64_t crop_h_below, int64_t crop_w_below, int64_t crop_h_above,
                                        int64_t crop_w_above, void* stream)
{
    using namespace b200;
    if (N < 0 || H <= 0 || W <= 0 || C <= 0 || dilation_h <= 0 || dilation_w <= 0 || crop_h_below < 0 || crop_w_below < 0 ||
        crop_h_above < 0 || crop_w_above < 0)
        return B200_ERR_INVALID_ARGUMENT;
    if (C % 16 != 0 || (reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
        return B200_ERR_UNSUPPORTED;
    const int64_t Ho = (H - 1) * dilation_h + 1 - crop_h_below - crop_h_above, Wo = (W - 1) * dilation_w + 1 - crop_w_below - crop_w_above;
    if (N == 0 || Ho <= 0 || Wo <= 0)
        return B200_OK;
    if (!in || !out)
        return B200_ERR_INVALID_ARGUMENT;
    const int64_t big = int64_t(1) << 30;
    if (N >= big || H >= big || W >= big || Ho >= big || Wo >= big || C >= big)
        return B200_ERR_TOO_LARGE;
    const int64_t total = N * Ho * Wo * (C / 16), blocks = (total + 255) / 256, cap = int64_t(sm_count()) * 32;
    dilate_crop_nhwc_kernel<<<unsigned(blocks < cap ? blocks : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(in), static_cast<uint4*>(out), int(N), int(H), int(W), int(C / 16), int(Ho), int(Wo), int(dilation_h),
        int(dilation_w), int(crop_h_below), int(crop_w_below));
    return after_launch("b200_dilate_crop_nhwc_u8");
}

extern "C" int b200_nchw_to_nhwc_u8(const void* in, void* out, int64_t N, int64_t C, int64_t H, int64_t W,
                                    int64_t c_pad, void* stream)
{
    if (N < 0 || C < 0 || H < 0 || W < 0 || c_pad < C)
        return B200_ERR_INVALID_ARGUMENT;
    if (N * C * H * W == 0)
        return B200_OK;
    if (!in || !out)
        return B200_ERR_INVALID_ARGUMENT;
    // per image: [C, HW] -> [HW, c_pad]
    return b200::launch_transpose(in, out, N, C, H * W, c_pad, static_cast<cudaStream_t>(stream), "b200_nchw_to_nhwc_u8");
}

extern "C" int b200_nhwc_to_nchw_u8(const void* in, void* out, int64_t N, int64_t C, int64_t H, int64_t W,
                                    int64_t c_pad, void* stream)
{
    using namespace b200;
    if (N < 0 || C < 0 || H < 0 || W < 0 || c_pad < C)
        return B200_ERR_INVALID_ARGUMENT;
    if (N * C * H * W == 0)
        return B200_OK;
    if (!in || !out)
        return B200_ERR_INVALID_ARGUMENT;
    // per image: [HW, c_pad] -> [C, HW]
    int64_t rows = H * W, cols = C;
    dim3 grid(unsigned((cols + TT - 1) / TT), unsigned((rows + TT - 1) / TT), unsigned(N));
    if (grid.y > 65535 || grid.z > 65535)
        return B200_ERR_TOO_LARGE;
    untranspose_bytes_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), rows, cols, c_pad);
    return after_launch("b200_nhwc_to_nchw_u8");
}

namespace b200
{
    // rows of `row_bytes` bytes from a dense source into rows `dst_pitch` bytes apart: one operand of a Concat.
    // V = 16: everything (pointers, row length, pitch) is a multiple of 16 bytes; V = 1: byte by byte.
    template <int V>
    __global__ void __launch_bounds__(256) copy_rows_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t rows,
                                                            int64_t row_units, int64_t dst_pitch_units)
    {
        using T = typename std::conditional<V == 16, uint4, uint8_t>::type;
        const T* s = reinterpret_cast<const T*>(src);
        T* d = reinterpret_cast<T*>(dst);
        const int64_t total = rows * row_units;
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x)
            d[(i / row_units) * dst_pitch_units + i % row_units] = s[i];
    }
}

extern "C" int b200_copy_rows(const void* src, void* dst, int64_t rows, int64_t row_bytes, int64_t dst_pitch_bytes, void* stream)
{
    if (rows < 0 || row_bytes < 0 || dst_pitch_bytes < row_bytes)
        return B200_ERR_INVALID_ARGUMENT;
    if (rows * row_bytes == 0)
        return B200_OK;
    if (!src || !dst)
        return B200_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool wide = ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) | uintptr_t(row_bytes) | uintptr_t(dst_pitch_bytes)) & 15) == 0;
    const int64_t units = wide ? rows * (row_bytes / 16) : rows * row_bytes;
    const int64_t blocks = (units + 255) / 256, cap = b200::sm_count() * 16;
    const unsigned grid = unsigned(blocks < cap ? blocks : cap);
    if (wide)
        b200::copy_rows_kernel<16><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), rows, row_bytes / 16,
                                                         dst_pitch_bytes / 16);
    else
        b200::copy_rows_kernel<1><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), rows, row_bytes,
                                                        dst_pitch_bytes);
    return b200::after_launch("b200_copy_rows");
}

extern "C" int b200_transpose_u8(const void* in, void* out, int64_t rows, int64_t cols, void* stream)
{
    if (rows < 0 || cols < 0)
        return B200_ERR_INVALID_ARGUMENT;
    if (rows * cols == 0)
        return B200_OK;
    if (!in || !out)
        return B200_ERR_INVALID_ARGUMENT;
    return b200::launch_transpose(in, out, 1, rows, cols, rows, static_cast<cudaStream_t>(stream), "b200_transpose_u8");
}

static int maxpool_nhwc_bytes(bool is_signed, const void* in, void* out, int64_t N, int64_t H, int64_t W, int64_t C, int64_t win_h,
                              int64_t win_w, int64_t stride_h, int64_t stride_w, int64_t pad_h, int64_t pad_w, int64_t pad_h_above,
                              int64_t pad_w_above, void* stream, const char* what)
{
    using namespace b200;
    if (N < 0 || H <= 0 || W <= 0 || C <= 0 || win_h <= 0 || win_w <= 0 || stride_h <= 0 || stride_w <= 0)
        return B200_ERR_INVALID_ARGUMENT;
    if (C % 16 != 0 || (reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
        return B200_ERR_UNSUPPORTED;
    int64_t P = (H + pad_h + pad_h_above - win_h) / stride_h + 1, Q = (W + pad_w + pad_w_above - win_w) / stride_w + 1;
    if (N == 0 || P <= 0 || Q <= 0)
        return B200_OK;
    if (!in || !out)
        return B200_ERR_INVALID_ARGUMENT;
    int64_t total = N * P * Q * (C / 16);
    int64_t blocks = (total + 255) / 256;
    unsigned grid = unsigned(blocks < b200::sm_count() * 32 ? blocks : b200::sm_count() * 32);
    const bool small = total < (int64_t(1) << 31) && N * H * W * (C / 16) < (int64_t(1) << 31);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint4* in4 = static_cast<const uint4*>(in);
    uint4* out4 = static_cast<uint4*>(out);
    if (is_signed)
        maxpool_nhwc_u8_kernel<true><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), int(N), int(H),
                                                           int(W), int(C / 16), int(P), int(Q), int(win_h), int(win_w),
                                                           int(stride_h), int(stride_w), int(pad_h), int(pad_w));
    else if (small && win_h == 3 && win_w == 3 && stride_h == 2 && stride_w == 2)
    {
        const int64_t threads = N * P * ((Q + 1) / 2) * (C / 16), pair_blocks = (threads + 255) / 256;
        maxpool_nhwc_u8_3x3s2_pair_kernel<<<unsigned(pair_blocks < b200::sm_count() * 32 ? pair_blocks : b200::sm_count() * 32), 256, 0, st>>>(
            in4, out4, int(N), int(H), int(W), int(C / 16), int(P), int(Q), int(pad_h), int(pad_w));
    }
    else if (small && win_h == 3 && win_w == 3)
        maxpool_nhwc_u8_fixed_kernel<3, 3><<<grid, 256, 0, st>>>(in4, out4, int(N), int(H), int(W), int(C / 16), int(P), int(Q),
                                                                 int(stride_h), int(stride_w), int(pad_h), int(pad_w));
    else if (small && win_h == 2 && win_w == 2)
        maxpool_nhwc_u8_fixed_kernel<2, 2><<<grid, 256, 0, st>>>(in4, out4, int(N), int(H), int(W), int(C / 16), int(P), int(Q),
                                                                 int(stride_h), int(stride_w), int(pad_h), int(pad_w));
    else
        maxpool_nhwc_u8_kernel<false><<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), int(N), int(H),
                                                     int(W), int(C / 16), int(P), int(Q), int(win_h), int(win_w),
                                                     int(stride_h), int(stride_w), int(pad_h), int(pad_w));
    return after_launch(what);
}

extern "C" int b200_maxpool_nhwc_u8(const void* in, void* out, int64_t N, int64_t H, int64_t W, int64_t C, int64_t win_h, int64_t win_w,
                                    int64_t stride_h, int64_t stride_w, int64_t pad_h, int64_t pad_w, int64_t pad_h_above,
                                    int64_t pad_w_above, void* stream)
{
    return maxpool_nhwc_bytes(false, in, out, N, H, W, C, win_h, win_w, stride_h, stride_w, pad_h, pad_w, pad_h_above, pad_w_above, stream,
                              "b200_maxpool_nhwc_u8");
}

extern "C" int b200_maxpool_nhwc_i8(const void* in, void* out, int64_t N, int64_t H, int64_t W, int64_t C, int64_t win_h, int64_t win_w,
                                    int64_t stride_h, int64_t stride_w, int64_t pad_h, int64_t pad_w, int64_t pad_h_above,
                                    int64_t pad_w_above, void* stream)
{
    return maxpool_nhwc_bytes(true, in, out, N, H, W, C, win_h, win_w, stride_h, stride_w, pad_h, pad_w, pad_h_above, pad_w_above, stream,
                              "b200_maxpool_nhwc_i8");
}

extern "C" int b200_global_avgpool_q_nhwc_u8(const void* in, void* out, const float* scale_in, const float* scale_out,
                                             int64_t N, int64_t H, int64_t W, int64_t C, void* stream)
{
    using namespace b200;
    if (N < 0 || H <= 0 || W <= 0 || C <= 0)
        return B200_ERR_INVALID_ARGUMENT;
    if (N == 0)
        return B200_OK;
    if (!in || !out || !scale_in || !scale_out)
        return B200_ERR_INVALID_ARGUMENT;
    int64_t total = N * C;
    global_avgpool_q_kernel<<<unsigned((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), scale_in, scale_out, int(N), int(H * W), int(C));
    return after_launch("b200_global_avgpool_q_nhwc_u8");
}

namespace b200
{
    // Patch matrix of a small-channel convolution (the network stem): input channels-last with
    // 4 channels per pixel, output row m = (n, p, q), R segments of 32 bytes = 8 taps x 4 channels
    // (taps s >= S and out-of-image pixels are zero).  One thread per (m, r) segment.
    __global__ void __launch_bounds__(256) im2col_c4_kernel(const uint32_t* __restrict__ in, uint4* __restrict__ out,
                                                            int N, int H, int W, int P, int Q, int R, int S,
                                                            int stride_h, int stride_w, int pad_h, int pad_w)
    {
        int64_t total = int64_t(N) * P * Q * R;
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x)
        {
            int r = int(i % R);
            int64_t m = i / R;
            int q = int(m % Q);
            int64_t t = m / Q;
            int p = int(t % P);
            int n = int(t / P);
            int h = p * stride_h - pad_h + r;
            int w0 = q * stride_w - pad_w;
            uint32_t v[8];
#pragma unroll
            for (int s = 0; s < 8; ++s)
            {
                int w = w0 + s;
                bool ok = s < S && h >= 0 && h < H && w >= 0 && w < W;
                v[s] = ok ? in[(int64_t(n) * H + h) * W + w] : 0u;
            }
            out[2 * i] = make_uint4(v[0], v[1], v[2], v[3]);
            out[2 * i + 1] = make_uint4(v[4], v[5], v[6], v[7]);
        }
    }

    __global__ void requant_scale_kernel(const float* a, const float* b, const float* c, float* out)
    {
        // runtime/reference/dot.hpp:154: scale = input0_scale * input1_scale / output_scale, left to right
        out[0] = __fdiv_rn(__fmul_rn(a[0], b[0]), c[0]);
    }
}

extern "C" int b200_im2col_c4_u8(const void* in, void* out, int64_t N, int64_t H, int64_t W, int64_t R, int64_t S,
                                 int64_t stride_h, int64_t stride_w, int64_t pad_h, int64_t pad_w,
                                 int64_t pad_h_above, int64_t pad_w_above, void* stream)
{
    using namespace b200;
    if (N < 0 || H <= 0 || W <= 0 || R <= 0 || S <= 0 || stride_h <= 0 || stride_w <= 0)
        return B200_ERR_INVALID_ARGUMENT;
    if (S > 8)
        return B200_ERR_UNSUPPORTED;
    int64_t P = (H + pad_h + pad_h_above - R) / stride_h + 1, Q = (W + pad_w + pad_w_above - S) / stride_w + 1;
    if (N == 0 || P <= 0 || Q <= 0)
        return B200_OK;
    if (!in || !out || (reinterpret_cast<uintptr_t>(out) & 15) || (reinterpret_cast<uintptr_t>(in) & 3))
        return B200_ERR_INVALID_ARGUMENT;
    int64_t total = N * P * Q * R;
    int64_t blocks = (total + 255) / 256;
    unsigned grid = unsigned(blocks < b200::sm_count() * 64 ? blocks : b200::sm_count() * 64);
    im2col_c4_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint32_t*>(in), static_cast<uint4*>(out), int(N), int(H), int(W), int(P), int(Q), int(R), int(S),
        int(stride_h), int(stride_w), int(pad_h), int(pad_w));
    return after_launch("b200_im2col_c4_u8");
}

extern "C" int b200_requant_scale(const float* input_scale, const float* filter_scale, const float* output_scale,
                                  float* out, void* stream)
{
    using namespace b200;
    if (!input_scale || !filter_scale || !output_scale || !out)
        return B200_ERR_INVALID_ARGUMENT;
    requant_scale_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(input_scale, filter_scale, output_scale, out);
    return after_launch("b200_requant_scale");
}

namespace b200
{
    // [batch, rows, cols] -> [batch, cols, rows] for 4-byte elements (int32 / f32 convolution outputs)
    __global__ void __launch_bounds__(256) transpose_b32_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out,
                                                                int64_t rows, int64_t cols)
    {
        __shared__ uint32_t tile[TT][TT + 1];
        const int64_t b = blockIdx.z;
        const int64_t r0 = int64_t(blockIdx.y) * TT, c0 = int64_t(blockIdx.x) * TT;
        const uint32_t* ip = in + b * rows * cols;
        uint32_t* op = out + b * rows * cols;
        const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
        for (int j = ty; j < TT; j += 8)
        {
            int64_t r = r0 + j, c = c0 + tx;
            if (r < rows && c < cols)
                tile[j][tx] = ip[r * cols + c];
        }
        __syncthreads();
        for (int j = ty; j < TT; j += 8)
        {
            int64_t c = c0 + j, r = r0 + tx;
            if (c < cols && r < rows)
                op[c * rows + r] = tile[tx][j];
        }
    }
}

extern "C" int b200_nhwc_to_nchw_b32(const void* in, void* out, int64_t N, int64_t C, int64_t HW, void* stream)
{
    using namespace b200;
    if (N < 0 || C < 0 || HW < 0)
        return B200_ERR_INVALID_ARGUMENT;
    if (N * C * HW == 0)
        return B200_OK;
    if (!in || !out)
        return B200_ERR_INVALID_ARGUMENT;
    dim3 grid(unsigned((C + TT - 1) / TT), unsigned((HW + TT - 1) / TT), unsigned(N));
    if (grid.y > 65535 || grid.z > 65535)
        return B200_ERR_TOO_LARGE;
    transpose_b32_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint32_t*>(in),
                                                                           static_cast<uint32_t*>(out), HW, C);
    return after_launch("b200_nhwc_to_nchw_b32");
}

// ---- stride-2, few-channel convolutions (network stems) as a space-to-depth problem --------------
//
// A stride-2 convolution over <= 4 channels reads, for output (p,q) and filter row r, the input row
// 2p - pad + r.  Grouping input pixels into 2x2 cells of 4 channels (16 bytes per cell, rows/cols shifted by
// the padding rounded up to even, zero outside the image) turns it into a stride-1 convolution over cells:
// filter row r and column s land in cell row (r+e_h)/2, cell column (s+e_w)/2 (e = pad & 1), at sub-pixel
// ((r+e_h)&1, (s+e_w)&1).  With at most 4 cell columns per filter row, the cells one output pixel needs from
// one cell row are 64 CONTIGUOUS bytes, i.e. one K-block of the tensor-core kernel, fetched by a tensor map
// whose pixel dimension advances 16 bytes per step (overlapping windows).
namespace b200
{
    __global__ void __launch_bounds__(256) s2d_pack_kernel(const uint8_t* __restrict__ in, uint4* __restrict__ out, int N, int C,
                                                           int H, int W, int Hc, int Wc, int eh, int ew)
    {
        // eh / ew: even shift of image rows / columns inside the cell grid
        int64_t total = int64_t(N) * Hc * Wc;
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x)
        {
            int cw = int(i % Wc);
            int64_t t = i / Wc;
            int ch = int(t % Hc);
            int n = int(t / Hc);
            uint32_t words[4] = {0, 0, 0, 0}; // (dy,dx) -> 4 channel bytes
#pragma unroll
            for (int dy = 0; dy < 2; ++dy)
#pragma unroll
                for (int dx = 0; dx < 2; ++dx)
                {
                    int h = 2 * ch + dy - eh, w = 2 * cw + dx - ew;
                    if (h >= 0 && h < H && w >= 0 && w < W)
                    {
                        uint32_t v = 0;
                        for (int c = 0; c < C; ++c)
                            v |= uint32_t(in[((int64_t(n) * C + c) * H + h) * W + w]) << (8 * c);
                        words[dy * 2 + dx] = v;
                    }
                }
            out[i] = make_uint4(words[0], words[1], words[2], words[3]);
        }
    }
}

namespace b200
{
    // Quantize (per-tensor scale and zero point, any round mode) fused into the cell packing: the f32 NCHW image is
    // read once and the one-byte NCHW intermediate never exists.  Same arithmetic as quantize_one in the Quantize
    // kernels (IEEE division, the reference's rounding sequence, clamp).
    template <typename Q>
    __device__ __forceinline__ uint32_t quantize_byte(float x, float scale, float zp, int mode)
    {
        Q v;
        switch (mode)
        {
        case B200_ROUND_NEAREST_TOWARD_INFINITY: v = quantize_one<Q, B200_ROUND_NEAREST_TOWARD_INFINITY>(x, scale, zp); break;
        case B200_ROUND_NEAREST_TOWARD_ZERO: v = quantize_one<Q, B200_ROUND_NEAREST_TOWARD_ZERO>(x, scale, zp); break;
        case B200_ROUND_NEAREST_UPWARD: v = quantize_one<Q, B200_ROUND_NEAREST_UPWARD>(x, scale, zp); break;
        case B200_ROUND_NEAREST_DOWNWARD: v = quantize_one<Q, B200_ROUND_NEAREST_DOWNWARD>(x, scale, zp); break;
        case B200_ROUND_NEAREST_TOWARD_EVEN: v = quantize_one<Q, B200_ROUND_NEAREST_TOWARD_EVEN>(x, scale, zp); break;
        case B200_ROUND_TOWARD_INFINITY: v = quantize_one<Q, B200_ROUND_TOWARD_INFINITY>(x, scale, zp); break;
        case B200_ROUND_TOWARD_ZERO: v = quantize_one<Q, B200_ROUND_TOWARD_ZERO>(x, scale, zp); break;
        case B200_ROUND_UP: v = quantize_one<Q, B200_ROUND_UP>(x, scale, zp); break;
        default: v = quantize_one<Q, B200_ROUND_DOWN>(x, scale, zp); break;
        }
        return uint32_t(uint8_t(v));
    }

    // One thread per cell.  FAST: round-to-nearest-even with a scale that allows the division-free quotient.
    // PAIRS: W even and the image 8-byte aligned, so the two pixels of a cell row are one float2 load.
    template <typename Q, bool FAST, bool PAIRS>
    __global__ void __launch_bounds__(256) s2d_pack_f32_kernel(const float* __restrict__ in, const float* __restrict__ scale,
                                                               const Q* __restrict__ zero_point, int mode, uint4* __restrict__ out,
                                                               int N, int C, int H, int W, int Hc, int Wc, int eh, int ew)
    {
        const float s = __ldg(scale);
        const int zi = int(__ldg(zero_point));
        const float zp = float(zi), y = __frcp_rn(s);
        const int lo = int(QLimits<Q>::lo) - zi, hi = int(QLimits<Q>::hi) - zi;
        const bool fast = FAST && scale_allows_fast_division(s); // the scale is only known here
        auto quant = [&](float x) -> uint32_t {
            if (fast)
                return uint32_t(quantize_rne_fast<Q>(x, s, y, lo, hi, zi)) & 0xFFu;
            return quantize_byte<Q>(x, s, zp, mode);
        };
        // pixels outside the image stay zero BYTES: the convolution pads the quantized tensor (the reference skips
        // padding positions), not the real-valued one
        const uint32_t total = uint32_t(N) * Hc * Wc;
        const size_t plane = size_t(H) * W;
        for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x)
        {
            const uint32_t cw = i % Wc, t = i / Wc;
            const uint32_t ch = t % Hc, n = t / Hc;
            const int w0 = 2 * int(cw) - ew, h0 = 2 * int(ch) - eh;
            float v[2][2][4];
#pragma unroll
            for (int dy = 0; dy < 2; ++dy)
            {
                const int h = h0 + dy;
                const bool row_ok = h >= 0 && h < H;
#pragma unroll
                for (int c = 0; c < 4; ++c)
                {
                    v[dy][0][c] = v[dy][1][c] = 0.0f;
                    if (c < C && row_ok)
                    {
                        const float* rowp = in + (size_t(n) * C + c) * plane + size_t(h) * W;
                        if (PAIRS)
                        {
                            if (w0 >= 0 && w0 + 1 < W)
                            {
                                const float2 f = *reinterpret_cast<const float2*>(rowp + w0);
                                v[dy][0][c] = f.x;
                                v[dy][1][c] = f.y;
                            }
                        }
                        else
                        {
                            if (w0 >= 0 && w0 < W)
                                v[dy][0][c] = rowp[w0];
                            if (w0 + 1 >= 0 && w0 + 1 < W)
                                v[dy][1][c] = rowp[w0 + 1];
                        }
                    }
                }
            }
            uint32_t words[4];
#pragma unroll
            for (int dy = 0; dy < 2; ++dy)
#pragma unroll
                for (int dx = 0; dx < 2; ++dx)
                {
                    const int h = h0 + dy, w = w0 + dx;
                    uint32_t word = 0;
                    if (h >= 0 && h < H && w >= 0 && w < W)
                    {
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            if (c < C)
                                word |= quant(v[dy][dx][c]) << (8 * c);
                    }
                    words[dy * 2 + dx] = word;
                }
            out[i] = make_uint4(words[0], words[1], words[2], words[3]);
        }
    }

    // The same for images whose rows can be read four floats at a time (W and the column shift multiples of 4, 16-byte
    // aligned rows): one thread makes TWO neighbouring cells from six 16-byte loads, all issued before the first use,
    // which doubles the bytes a thread keeps in flight (the kernel is bound by load latency, not by arithmetic).
    template <typename Q, bool FAST>
    __global__ void __launch_bounds__(256) s2d_pack_f32_quad_kernel(const float* __restrict__ in, const float* __restrict__ scale,
                                                                    const Q* __restrict__ zero_point, int mode, uint4* __restrict__ out,
                                                                    int N, int C, int H, int W, int Hc, int Wc, int eh, int ew)
    {
        const float s = __ldg(scale);
        const int zi = int(__ldg(zero_point));
        const float zp = float(zi), y = __frcp_rn(s);
        const int lo = int(QLimits<Q>::lo) - zi, hi = int(QLimits<Q>::hi) - zi;
        const bool fast = FAST && scale_allows_fast_division(s);
        auto quant = [&](float x) -> uint32_t {
            if (fast)
                return uint32_t(quantize_rne_fast<Q>(x, s, y, lo, hi, zi)) & 0xFFu;
            return quantize_byte<Q>(x, s, zp, mode);
        };
        const uint32_t Wc2 = uint32_t(Wc + 1) / 2;
        const uint32_t total = uint32_t(N) * Hc * Wc2;
        const size_t plane = size_t(H) * W;
        const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
        if (i >= total)
            return;
        const uint32_t cp = i % Wc2, t = i / Wc2;
        const uint32_t ch = t % Hc, n = t / Hc;
        const int w0 = 4 * int(cp) - ew, h0 = 2 * int(ch) - eh; // four pixels w0 .. w0 + 3: cells 2 cp and 2 cp + 1
        const bool cols_ok = w0 >= 0 && w0 + 3 < W;              // W and w0 are multiples of 4: all four inside, or none
        float4 v[2][4];
#pragma unroll
        for (int dy = 0; dy < 2; ++dy)
        {
            const int h = h0 + dy;
            const bool ok = cols_ok && h >= 0 && h < H;
#pragma unroll
            for (int c = 0; c < 4; ++c)
            {
                v[dy][c] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (c < C && ok)
                    v[dy][c] = *reinterpret_cast<const float4*>(in + (size_t(n) * C + c) * plane + size_t(h) * W + w0);
            }
        }
        // pixels outside the image stay zero BYTES (the convolution pads the quantized tensor)
        uint32_t words[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}}; // [cell][dy * 2 + dx]
#pragma unroll
        for (int dy = 0; dy < 2; ++dy)
        {
            const int h = h0 + dy;
            if (cols_ok && h >= 0 && h < H)
            {
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    if (c < C)
                    {
                        words[0][dy * 2 + 0] |= quant(v[dy][c].x) << (8 * c);
                        words[0][dy * 2 + 1] |= quant(v[dy][c].y) << (8 * c);
                        words[1][dy * 2 + 0] |= quant(v[dy][c].z) << (8 * c);
                        words[1][dy * 2 + 1] |= quant(v[dy][c].w) << (8 * c);
                    }
            }
        }
        const size_t cell = (size_t(n) * Hc + ch) * Wc + 2 * size_t(cp);
        out[cell] = make_uint4(words[0][0], words[0][1], words[0][2], words[0][3]);
        if (2 * cp + 1 < uint32_t(Wc))
            out[cell + 1] = make_uint4(words[1][0], words[1][1], words[1][2], words[1][3]);
    }
}

extern "C" int b200_stem_geometry(int64_t H, int64_t W, int64_t R, int64_t S, int64_t pad_h, int64_t pad_w,
                                  int64_t pad_h_above, int64_t pad_w_above, int64_t* P, int64_t* Q, int64_t* Hc, int64_t* Wc,
                                  int64_t* Rc)
{
    if (H <= 0 || W <= 0 || R <= 0 || S <= 0 || pad_h < 0 || pad_w < 0 || !P || !Q || !Hc || !Wc || !Rc)
        return B200_ERR_INVALID_ARGUMENT;
    const int64_t eh = pad_h & 1, ew = pad_w & 1;
    const int64_t rc = (R - 1 + eh) / 2 + 1, sc = (S - 1 + ew) / 2 + 1;
    if (sc > 4)
        return B200_ERR_UNSUPPORTED;
    *P = (H + pad_h + pad_h_above - R) / 2 + 1;
    *Q = (W + pad_w + pad_w_above - S) / 2 + 1;
    if (*P <= 0 || *Q <= 0)
        return B200_ERR_INVALID_ARGUMENT;
    *Rc = rc;
    *Hc = *P + rc - 1;
    *Wc = *Q + 3; // four cell columns per window
    return B200_OK;
}

extern "C" int b200_stem_pack_filter_host(const int8_t* kcrs, int8_t* packed, int64_t K, int64_t C, int64_t R, int64_t S,
                                          int64_t pad_h, int64_t pad_w)
{
    if (!kcrs || !packed || K <= 0 || C <= 0 || C > 4 || R <= 0 || S <= 0)
        return B200_ERR_INVALID_ARGUMENT;
    const int64_t eh = pad_h & 1, ew = pad_w & 1;
    const int64_t rc = (R - 1 + eh) / 2 + 1, sc = (S - 1 + ew) / 2 + 1;
    if (sc > 4)
        return B200_ERR_UNSUPPORTED;
    for (int64_t i = 0; i < K * rc * 64; ++i)
        packed[i] = 0;
    for (int64_t k = 0; k < K; ++k)
        for (int64_t c = 0; c < C; ++c)
            for (int64_t r = 0; r < R; ++r)
                for (int64_t s = 0; s < S; ++s)
                {
                    const int64_t rr = (r + eh) / 2, dy = (r + eh) & 1, ss = (s + ew) / 2, dx = (s + ew) & 1;
                    packed[(k * rc + rr) * 64 + ss * 16 + (dy * 2 + dx) * 4 + c] = kcrs[((k * C + c) * R + r) * S + s];
                }
    return B200_OK;
}

extern "C" int b200_stem_pack_input(const void* in_nchw, void* cells, int64_t N, int64_t C, int64_t H, int64_t W, int64_t R,
                                    int64_t S, int64_t pad_h, int64_t pad_w, int64_t pad_h_above, int64_t pad_w_above,
                                    void* stream)
{
    using namespace b200;
    if (N < 0 || C <= 0 || C > 4)
        return B200_ERR_INVALID_ARGUMENT;
    int64_t P, Q, Hc, Wc, Rc;
    int rc = b200_stem_geometry(H, W, R, S, pad_h, pad_w, pad_h_above, pad_w_above, &P, &Q, &Hc, &Wc, &Rc);
    if (rc != B200_OK)
        return rc;
    if (N == 0)
        return B200_OK;
    if (!in_nchw || !cells || (reinterpret_cast<uintptr_t>(cells) & 15))
        return B200_ERR_INVALID_ARGUMENT;
    const int64_t eh = pad_h + (pad_h & 1), ew = pad_w + (pad_w & 1);
    int64_t total = N * Hc * Wc;
    int64_t blocks = (total + 255) / 256;
    unsigned grid = unsigned(blocks < b200::sm_count() * 32 ? blocks : b200::sm_count() * 32);
    s2d_pack_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint8_t*>(in_nchw),
                                                                       static_cast<uint4*>(cells), int(N), int(C), int(H), int(W),
                                                                       int(Hc), int(Wc), int(eh), int(ew));
    return after_launch("b200_stem_pack_input");
}

extern "C" int b200_stem_pack_input_f32(const float* in_nchw, const float* scale, const void* zero_point, int q_type,
                                        int round_mode, void* cells, int64_t N, int64_t C, int64_t H, int64_t W, int64_t R,
                                        int64_t S, int64_t pad_h, int64_t pad_w, int64_t pad_h_above, int64_t pad_w_above,
                                        void* stream)
{
    using namespace b200;
    if (N < 0 || C <= 0 || C > 4 || (q_type != B200_U8 && q_type != B200_I8) || round_mode < 0 || round_mode > B200_ROUND_DOWN)
        return B200_ERR_INVALID_ARGUMENT;
    int64_t P, Q, Hc, Wc, Rc;
    int rc = b200_stem_geometry(H, W, R, S, pad_h, pad_w, pad_h_above, pad_w_above, &P, &Q, &Hc, &Wc, &Rc);
    if (rc != B200_OK)
        return rc;
    if (N == 0)
        return B200_OK;
    if (!in_nchw || !scale || !zero_point || !cells || (reinterpret_cast<uintptr_t>(cells) & 15))
        return B200_ERR_INVALID_ARGUMENT;
    const int64_t eh = pad_h + (pad_h & 1), ew = pad_w + (pad_w & 1);
    int64_t total = N * Hc * Wc;
    int64_t blocks = (total + 255) / 256;
    unsigned grid = unsigned(blocks); // one cell per thread: the kernel is a single wave of loads, not a loop
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (total >= (int64_t(1) << 31))
        return B200_ERR_TOO_LARGE;
    // float2 loads need an even width, an even column shift (always) and an 8-byte aligned image
    const bool pairs = (W % 2 == 0) && (reinterpret_cast<uintptr_t>(in_nchw) & 7) == 0;
    // round-to-nearest-even may take the division-free quotient; the kernel checks the scale (it lives on the device)
    const bool rne = round_mode == B200_ROUND_NEAREST_TOWARD_EVEN && (g_fast_division.load(std::memory_order_relaxed) != 0);
#define B200_S2D_LAUNCH(Q, FAST, PAIRS)                                                                                         \
    s2d_pack_f32_kernel<Q, FAST, PAIRS><<<grid, 256, 0, st>>>(in_nchw, scale, static_cast<const Q*>(zero_point), round_mode,     \
                                                              static_cast<uint4*>(cells), int(N), int(C), int(H), int(W), int(Hc), \
                                                              int(Wc), int(eh), int(ew))
    // rows that can be read four floats at a time: two cells per thread
    const bool quads = (W % 4 == 0) && (ew % 4 == 0) && (reinterpret_cast<uintptr_t>(in_nchw) & 15) == 0;
    if (quads)
    {
        const int64_t threads = N * Hc * ((Wc + 1) / 2);
        const unsigned qgrid = unsigned((threads + 255) / 256);
#define B200_S2D_QUAD(Q, FAST)                                                                                                  \
    s2d_pack_f32_quad_kernel<Q, FAST><<<qgrid, 256, 0, st>>>(in_nchw, scale, static_cast<const Q*>(zero_point), round_mode,      \
                                                             static_cast<uint4*>(cells), int(N), int(C), int(H), int(W), int(Hc), \
                                                             int(Wc), int(eh), int(ew))
        if (q_type == B200_U8)
        {
            if (rne) B200_S2D_QUAD(uint8_t, true);
            else B200_S2D_QUAD(uint8_t, false);
        }
        else
        {
            if (rne) B200_S2D_QUAD(int8_t, true);
            else B200_S2D_QUAD(int8_t, false);
        }
#undef B200_S2D_QUAD
        return after_launch("b200_stem_pack_input_f32");
    }
    if (q_type == B200_U8)
    {
        if (rne && pairs) B200_S2D_LAUNCH(uint8_t, true, true);
        else if (rne) B200_S2D_LAUNCH(uint8_t, true, false);
        else if (pairs) B200_S2D_LAUNCH(uint8_t, false, true);
        else B200_S2D_LAUNCH(uint8_t, false, false);
    }
    else
    {
        if (rne && pairs) B200_S2D_LAUNCH(int8_t, true, true);
        else if (rne) B200_S2D_LAUNCH(int8_t, true, false);
        else if (pairs) B200_S2D_LAUNCH(int8_t, false, true);
        else B200_S2D_LAUNCH(int8_t, false, false);
    }
#undef B200_S2D_LAUNCH
    return after_launch("b200_stem_pack_input_f32");
}

// Layout conversions for 1-byte tensors (graph edges and weight packing), and the u8
// pooling glue of whole-graph inference.  All of them are plain HBM-bound byte movers.
#include "common.cuh"

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
    // One thread per 16 channels of one output pixel (128-bit loads, __vmaxu4).
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
            uint4 m = make_uint4(0, 0, 0, 0);
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
                    m.x = __vmaxu4(m.x, v.x);
                    m.y = __vmaxu4(m.y, v.y);
                    m.z = __vmaxu4(m.z, v.z);
                    m.w = __vmaxu4(m.w, v.w);
                }
            }
            reinterpret_cast<uint4*>(out)[i] = m;
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

extern "C" int b200_maxpool_nhwc_u8(const void* in, void* out, int64_t N, int64_t H, int64_t W, int64_t C,
                                    int64_t win_h, int64_t win_w, int64_t stride_h, int64_t stride_w, int64_t pad_h,
                                    int64_t pad_w, int64_t pad_h_above, int64_t pad_w_above, void* stream)
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
    unsigned grid = unsigned(blocks < 148 * 32 ? blocks : 148 * 32);
    maxpool_nhwc_u8_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out), int(N), int(H), int(W), int(C / 16), int(P), int(Q),
        int(win_h), int(win_w), int(stride_h), int(stride_w), int(pad_h), int(pad_w));
    return after_launch("b200_maxpool_nhwc_u8");
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
    unsigned grid = unsigned(blocks < 148 * 64 ? blocks : 148 * 64);
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

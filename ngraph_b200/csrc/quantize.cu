// Quantize / Dequantize: HBM-streaming kernels (5 bytes per element for 8-bit types).
//
// Arithmetic follows runtime::reference::quantize / dequantize
// (src/ngraph/runtime/reference/quantize.hpp:30-117, dequantize.hpp:32-52) exactly;
// the iteration order does not matter because every element is independent.
//
// Two launch shapes:
//   rows    - the tensor is viewed as [rows, inner] where every row has ONE scale /
//             zero point (per-tensor: a single row; per-axis on axis a: rows =
//             prod(shape[0..a]), inner = prod(shape[a+1..])).  128-bit loads,
//             packed 32-bit (or 128-bit) stores, 4 independent loads in flight per thread.
//   generic - one element per thread with the scale index recomputed from the
//             coordinates; any axis set, any alignment.
#include "common.cuh"

namespace b200
{
    constexpr int QT = 256;         // threads per block
    constexpr int QU = 4;           // independent 4-element vectors per thread
    constexpr int QCHUNK = QT * QU * 4; // elements per block

    struct ProjDims
    {
        int rank;
        int64_t shape[B200_MAX_RANK];
        int64_t sstride[B200_MAX_RANK]; // stride into scale/zero_point (0 for non-axes)
    };

    __device__ __forceinline__ int64_t project_index(const ProjDims& d, int64_t idx)
    {
        int64_t s = 0;
#pragma unroll 1
        for (int i = d.rank - 1; i >= 0; --i)
        {
            int64_t q = idx / d.shape[i];
            int64_t c = idx - q * d.shape[i];
            s += c * d.sstride[i];
            idx = q;
        }
        return s;
    }

    template <typename Q>
    __device__ __forceinline__ void store4(Q* p, Q a, Q b, Q c, Q d);
    template <>
    __device__ __forceinline__ void store4<uint8_t>(uint8_t* p, uint8_t a, uint8_t b, uint8_t c, uint8_t d)
    {
        *reinterpret_cast<uint32_t*>(p) = uint32_t(a) | (uint32_t(b) << 8) | (uint32_t(c) << 16) | (uint32_t(d) << 24);
    }
    template <>
    __device__ __forceinline__ void store4<int8_t>(int8_t* p, int8_t a, int8_t b, int8_t c, int8_t d)
    {
        *reinterpret_cast<uint32_t*>(p) = uint32_t(uint8_t(a)) | (uint32_t(uint8_t(b)) << 8) |
                                          (uint32_t(uint8_t(c)) << 16) | (uint32_t(uint8_t(d)) << 24);
    }
    template <>
    __device__ __forceinline__ void store4<int32_t>(int32_t* p, int32_t a, int32_t b, int32_t c, int32_t d)
    {
        *reinterpret_cast<int4*>(p) = make_int4(a, b, c, d);
    }

    template <typename Q, int MODE, bool FAST>
    __global__ void __launch_bounds__(QT) quantize_rows_kernel(const float* __restrict__ x,
                                                               const float* __restrict__ scale,
                                                               const Q* __restrict__ zp,
                                                               Q* __restrict__ out,
                                                               int64_t inner,
                                                               uint32_t chunks_per_row,
                                                               int64_t n_scales)
    {
        const int64_t row = blockIdx.x / chunks_per_row;
        const uint32_t chunk = blockIdx.x - uint32_t(row) * chunks_per_row;
        const int64_t sidx = row % n_scales;
        const float s = scale[sidx];
        const float z = static_cast<float>(zp[sidx]);
        const int64_t row_off = int64_t(chunk) * QCHUNK;
        const int64_t rem = inner - row_off; // elements of this row from the chunk start
        const float* xp = x + row * inner + row_off;
        Q* op = out + row * inner + row_off;
        // one scale per block: the division becomes two multiply-adds where that is exact (8-bit outputs only; an
        // int32 output can be large enough for the last bit of a quotient beyond 2^24 to matter)
        const bool fast = FAST && sizeof(Q) == 1 && scale_allows_fast_division(s);
        const float y = __frcp_rn(s);
        const float s_low = __fmul_rn(fabsf(s), 5.9604644775390625e-8f); // |s| * 2^-24 (quantize4_directed_fast)
        const int zi = static_cast<int>(zp[sidx]);
        const int lo = sizeof(Q) == 1 ? int(QLimits<Q>::lo) - zi : 0, hi = sizeof(Q) == 1 ? int(QLimits<Q>::hi) - zi : 0; // 8-bit path only

        float4 v[QU];
#pragma unroll
        for (int u = 0; u < QU; ++u)
        {
            int64_t off = (int64_t(u) * QT + threadIdx.x) * 4;
            if (off + 4 <= rem)
                v[u] = *reinterpret_cast<const float4*>(xp + off);
        }
#pragma unroll
        for (int u = 0; u < QU; ++u)
        {
            int64_t off = (int64_t(u) * QT + threadIdx.x) * 4;
            if (off + 4 <= rem && fast)
            {
                constexpr bool directed = MODE == B200_ROUND_TOWARD_INFINITY || MODE == B200_ROUND_TOWARD_ZERO ||
                                          MODE == B200_ROUND_UP || MODE == B200_ROUND_DOWN;
                if (directed)
                {
                    int r[4];
                    quantize4_directed_fast<MODE>(v[u], s, y, s_low, lo, hi, zi, r);
                    store4<Q>(op + off, static_cast<Q>(r[0]), static_cast<Q>(r[1]), static_cast<Q>(r[2]), static_cast<Q>(r[3]));
                }
                else
                    store4<Q>(op + off,
                              static_cast<Q>(quantize_int_fast<Q, MODE>(v[u].x, s, y, lo, hi, zi)),
                              static_cast<Q>(quantize_int_fast<Q, MODE>(v[u].y, s, y, lo, hi, zi)),
                              static_cast<Q>(quantize_int_fast<Q, MODE>(v[u].z, s, y, lo, hi, zi)),
                              static_cast<Q>(quantize_int_fast<Q, MODE>(v[u].w, s, y, lo, hi, zi)));
            }
            else if (off + 4 <= rem)
            {
                store4<Q>(op + off,
                          quantize_one<Q, MODE>(v[u].x, s, z),
                          quantize_one<Q, MODE>(v[u].y, s, z),
                          quantize_one<Q, MODE>(v[u].z, s, z),
                          quantize_one<Q, MODE>(v[u].w, s, z));
            }
            else
            {
                for (int64_t e = off; e < rem && e < off + 4; ++e)
                    op[e] = quantize_one<Q, MODE>(xp[e], s, z);
            }
        }
    }

    // Round-to-nearest-even Quantize to 8 bits with the division strength-reduced per row.
    //
    // The row's scale s is uniform, so y = RN(1/s) is computed once (correctly rounded reciprocal)
    // and each quotient is  q0 = RN(x*y);  e = x - q0*s (exact in one FMA);  q = RN(q0 + e*y),
    // which is the correctly rounded x/s (Markstein's division theorem) whenever s is a normal
    // number whose significand is not all ones and nothing over/underflows.  Blocks whose scale
    // fails that test, and quotients of magnitude >= 2^24 (whose result saturates regardless of
    // the last bit), take the other branches below, so every output byte equals the plain
    // x / s -> floor(q+0.5)/ceil(q-0.5)/parity -> +zero_point -> clamp sequence of the reference.
    // (For |q| < 2^23 that rounding sequence is round-half-even, i.e. one cvt.rni; beyond it clamps.)
    template <typename Q>
    __global__ void __launch_bounds__(QT) quantize_rows_rne8_kernel(const float* __restrict__ x,
                                                                   const float* __restrict__ scale,
                                                                   const Q* __restrict__ zp,
                                                                   Q* __restrict__ out,
                                                                   int64_t inner,
                                                                   uint32_t chunks_per_row,
                                                                   int64_t n_scales)
    {
        const int64_t row = blockIdx.x / chunks_per_row;
        const uint32_t chunk = blockIdx.x - uint32_t(row) * chunks_per_row;
        const int64_t sidx = row % n_scales;
        const float s = scale[sidx];
        const int zi = static_cast<int>(zp[sidx]);
        const float z = static_cast<float>(zi);
        const int64_t row_off = int64_t(chunk) * QCHUNK;
        const int64_t rem = inner - row_off;
        const float* xp = x + row * inner + row_off;
        Q* op = out + row * inner + row_off;
        const bool fast = scale_allows_fast_division(s);
        const float y = __frcp_rn(s);
        const int lo = int(QLimits<Q>::lo) - zi, hi = int(QLimits<Q>::hi) - zi;

        float4 v[QU];
#pragma unroll
        for (int u = 0; u < QU; ++u)
        {
            int64_t off = (int64_t(u) * QT + threadIdx.x) * 4;
            if (off + 4 <= rem)
                v[u] = *reinterpret_cast<const float4*>(xp + off);
        }
#pragma unroll
        for (int u = 0; u < QU; ++u)
        {
            int64_t off = (int64_t(u) * QT + threadIdx.x) * 4;
            if (off + 4 <= rem)
            {
                if (fast)
                {
                    const int a = quantize_rne_fast<Q>(v[u].x, s, y, lo, hi, zi), b = quantize_rne_fast<Q>(v[u].y, s, y, lo, hi, zi);
                    const int c = quantize_rne_fast<Q>(v[u].z, s, y, lo, hi, zi), d = quantize_rne_fast<Q>(v[u].w, s, y, lo, hi, zi);
                    *reinterpret_cast<uint32_t*>(op + off) =
                        uint32_t(a & 0xFF) | (uint32_t(b & 0xFF) << 8) | (uint32_t(c & 0xFF) << 16) | (uint32_t(d & 0xFF) << 24);
                }
                else
                {
                    store4<Q>(op + off, quantize_one<Q, 4>(v[u].x, s, z), quantize_one<Q, 4>(v[u].y, s, z),
                              quantize_one<Q, 4>(v[u].z, s, z), quantize_one<Q, 4>(v[u].w, s, z));
                }
            }
            else
            {
                for (int64_t e = off; e < rem && e < off + 4; ++e)
                    op[e] = quantize_one<Q, 4>(xp[e], s, z);
            }
        }
    }

    template <typename Q, int MODE>
    __global__ void __launch_bounds__(QT) quantize_generic_kernel(const float* __restrict__ x,
                                                                  const float* __restrict__ scale,
                                                                  const Q* __restrict__ zp,
                                                                  Q* __restrict__ out,
                                                                  int64_t total,
                                                                  ProjDims dims)
    {
        for (int64_t i = int64_t(blockIdx.x) * QT + threadIdx.x; i < total; i += int64_t(gridDim.x) * QT)
        {
            int64_t sidx = project_index(dims, i);
            out[i] = quantize_one<Q, MODE>(x[i], scale[sidx], static_cast<float>(zp[sidx]));
        }
    }

    // out = (float)(in - zp) * scale   (dequantize.hpp:47-51; the subtraction is exact in int)
    template <typename Q>
    __device__ __forceinline__ float dequantize_one(Q v, int zp, float s)
    {
        return __fmul_rn(static_cast<float>(int(v) - zp), s);
    }
    template <>
    __device__ __forceinline__ float dequantize_one<int32_t>(int32_t v, int zp, float s)
    {
        // int32 - int32 as the reference computes it (wraps on overflow here; UB there)
        return __fmul_rn(static_cast<float>(int32_t(uint32_t(v) - uint32_t(zp))), s);
    }

    template <typename Q>
    struct Vec4;
    template <>
    struct Vec4<uint8_t>
    {
        uint32_t w;
        __device__ __forceinline__ void load(const uint8_t* p) { w = *reinterpret_cast<const uint32_t*>(p); }
        __device__ __forceinline__ uint8_t get(int i) const { return uint8_t(w >> (8 * i)); }
    };
    template <>
    struct Vec4<int8_t>
    {
        uint32_t w;
        __device__ __forceinline__ void load(const int8_t* p) { w = *reinterpret_cast<const uint32_t*>(p); }
        __device__ __forceinline__ int8_t get(int i) const { return int8_t(uint8_t(w >> (8 * i))); }
    };
    template <>
    struct Vec4<int32_t>
    {
        int4 w;
        __device__ __forceinline__ void load(const int32_t* p) { w = *reinterpret_cast<const int4*>(p); }
        __device__ __forceinline__ int32_t get(int i) const { return i == 0 ? w.x : i == 1 ? w.y : i == 2 ? w.z : w.w; }
    };

    template <typename Q>
    __global__ void __launch_bounds__(QT) dequantize_rows_kernel(const Q* __restrict__ in,
                                                                 const float* __restrict__ scale,
                                                                 const Q* __restrict__ zp,
                                                                 float* __restrict__ out,
                                                                 int64_t inner,
                                                                 uint32_t chunks_per_row,
                                                                 int64_t n_scales)
    {
        const int64_t row = blockIdx.x / chunks_per_row;
        const uint32_t chunk = blockIdx.x - uint32_t(row) * chunks_per_row;
        const int64_t sidx = row % n_scales;
        const float s = scale[sidx];
        const int z = static_cast<int>(zp[sidx]);
        const int64_t row_off = int64_t(chunk) * QCHUNK;
        const int64_t rem = inner - row_off;
        const Q* ip = in + row * inner + row_off;
        float* op = out + row * inner + row_off;

        Vec4<Q> v[QU];
#pragma unroll
        for (int u = 0; u < QU; ++u)
        {
            int64_t off = (int64_t(u) * QT + threadIdx.x) * 4;
            if (off + 4 <= rem)
                v[u].load(ip + off);
        }
#pragma unroll
        for (int u = 0; u < QU; ++u)
        {
            int64_t off = (int64_t(u) * QT + threadIdx.x) * 4;
            if (off + 4 <= rem)
            {
                float4 r;
                r.x = dequantize_one<Q>(v[u].get(0), z, s);
                r.y = dequantize_one<Q>(v[u].get(1), z, s);
                r.z = dequantize_one<Q>(v[u].get(2), z, s);
                r.w = dequantize_one<Q>(v[u].get(3), z, s);
                *reinterpret_cast<float4*>(op + off) = r;
            }
            else
            {
                for (int64_t e = off; e < rem && e < off + 4; ++e)
                    op[e] = dequantize_one<Q>(ip[e], z, s);
            }
        }
    }

    template <typename Q>
    __global__ void __launch_bounds__(QT) dequantize_generic_kernel(const Q* __restrict__ in,
                                                                    const float* __restrict__ scale,
                                                                    const Q* __restrict__ zp,
                                                                    float* __restrict__ out,
                                                                    int64_t total,
                                                                    ProjDims dims)
    {
        for (int64_t i = int64_t(blockIdx.x) * QT + threadIdx.x; i < total; i += int64_t(gridDim.x) * QT)
        {
            int64_t sidx = project_index(dims, i);
            out[i] = dequantize_one<Q>(in[i], static_cast<int>(zp[sidx]), scale[sidx]);
        }
    }

    // How the (shape, axes) pair maps onto the two launch shapes.
    struct QuantPlan
    {
        int64_t total;
        bool rows_ok;     // [rows, inner] view with one scale per row exists
        int64_t rows, inner, n_scales;
        ProjDims dims;
    };

    static int make_plan(const int64_t* shape, int rank, const int64_t* axes, int n_axes, QuantPlan& p)
    {
        if (rank < 0 || rank > B200_MAX_RANK || n_axes < 0 || n_axes > rank || (rank > 0 && !shape) ||
            (n_axes > 0 && !axes))
            return B200_ERR_INVALID_ARGUMENT;
        bool is_axis[B200_MAX_RANK] = {false};
        for (int i = 0; i < n_axes; ++i)
        {
            if (axes[i] < 0 || axes[i] >= rank || is_axis[axes[i]] || (i > 0 && axes[i] <= axes[i - 1]))
                return B200_ERR_INVALID_ARGUMENT;
            is_axis[axes[i]] = true;
        }
        p.total = 1;
        for (int i = 0; i < rank; ++i)
        {
            if (shape[i] < 0)
                return B200_ERR_INVALID_ARGUMENT;
            p.total *= shape[i];
        }
        p.dims.rank = rank;
        int64_t ss = 1;
        for (int i = rank - 1; i >= 0; --i)
        {
            p.dims.shape[i] = shape[i];
            p.dims.sstride[i] = is_axis[i] ? ss : 0;
            if (is_axis[i])
                ss *= shape[i];
        }
        p.n_scales = ss;
        // rows view: the axes are one contiguous run [a..b]; every dim before a only repeats the scales
        p.rows_ok = false;
        if (n_axes == 0)
        {
            p.rows_ok = true;
            p.rows = 1;
            p.inner = p.total;
        }
        else if (axes[n_axes - 1] - axes[0] == n_axes - 1)
        {
            int64_t inner = 1, rows = 1;
            for (int i = int(axes[n_axes - 1]) + 1; i < rank; ++i)
                inner *= shape[i];
            for (int i = 0; i <= int(axes[n_axes - 1]); ++i)
                rows *= shape[i];
            p.rows_ok = true;
            p.rows = rows;
            p.inner = inner;
        }
        return B200_OK;
    }

    static bool use_rows(const QuantPlan& p, const void* a, const void* b)
    {
        if (!p.rows_ok || p.total == 0)
            return false;
        if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15)
            return false;
        if (p.rows > 1 && ((p.inner & 3) || p.inner < 512))
            return false;
        int64_t chunks = (p.inner + QCHUNK - 1) / QCHUNK;
        return chunks * p.rows < (int64_t(1) << 31) && chunks < (int64_t(1) << 31);
    }

    static unsigned generic_grid(int64_t total)
    {
        int64_t b = (total + QT - 1) / QT;
        const int64_t cap = b200::sm_count() * 8 * 4;
        return unsigned(b < cap ? (b > 0 ? b : 1) : cap);
    }

    std::atomic<int> g_fast_division{1};

    template <typename Q>
    static void launch_rne8(const float* x, const float* scale, const void* zp, void* out, const QuantPlan& p,
                            uint32_t chunks, cudaStream_t st)
    {
        quantize_rows_rne8_kernel<Q><<<unsigned(chunks * p.rows), QT, 0, st>>>(
            x, scale, static_cast<const Q*>(zp), static_cast<Q*>(out), p.inner, chunks, p.n_scales);
    }
    template <>
    void launch_rne8<int32_t>(const float*, const float*, const void*, void*, const QuantPlan&, uint32_t, cudaStream_t)
    {
    }

    template <typename Q, int MODE>
    static int launch_quantize(const float* x, const float* scale, const void* zp, void* out,
                               const QuantPlan& p, cudaStream_t st)
    {
        if (use_rows(p, x, out) && MODE == B200_ROUND_NEAREST_TOWARD_EVEN && sizeof(Q) == 1 &&
            g_fast_division.load(std::memory_order_relaxed))
        {
            uint32_t chunks = uint32_t((p.inner + QCHUNK - 1) / QCHUNK);
            launch_rne8<Q>(x, scale, zp, out, p, chunks, st);
        }
        else if (use_rows(p, x, out))
        {
            uint32_t chunks = uint32_t((p.inner + QCHUNK - 1) / QCHUNK);
            if (sizeof(Q) == 1 && g_fast_division.load(std::memory_order_relaxed))
                quantize_rows_kernel<Q, MODE, true><<<unsigned(chunks * p.rows), QT, 0, st>>>(
                    x, scale, static_cast<const Q*>(zp), static_cast<Q*>(out), p.inner, chunks, p.n_scales);
            else
                quantize_rows_kernel<Q, MODE, false><<<unsigned(chunks * p.rows), QT, 0, st>>>(
                    x, scale, static_cast<const Q*>(zp), static_cast<Q*>(out), p.inner, chunks, p.n_scales);
        }
        else
        {
            quantize_generic_kernel<Q, MODE><<<generic_grid(p.total), QT, 0, st>>>(
                x, scale, static_cast<const Q*>(zp), static_cast<Q*>(out), p.total, p.dims);
        }
        return after_launch("b200_quantize");
    }

    template <typename Q>
    static int dispatch_quantize_mode(int mode, const float* x, const float* scale, const void* zp, void* out,
                                      const QuantPlan& p, cudaStream_t st)
    {
        switch (mode)
        {
        case 0: return launch_quantize<Q, 0>(x, scale, zp, out, p, st);
        case 1: return launch_quantize<Q, 1>(x, scale, zp, out, p, st);
        case 2: return launch_quantize<Q, 2>(x, scale, zp, out, p, st);
        case 3: return launch_quantize<Q, 3>(x, scale, zp, out, p, st);
        case 4: return launch_quantize<Q, 4>(x, scale, zp, out, p, st);
        case 5: return launch_quantize<Q, 5>(x, scale, zp, out, p, st);
        case 6: return launch_quantize<Q, 6>(x, scale, zp, out, p, st);
        case 7: return launch_quantize<Q, 7>(x, scale, zp, out, p, st);
        case 8: return launch_quantize<Q, 8>(x, scale, zp, out, p, st);
        default: return B200_ERR_INVALID_ARGUMENT;
        }
    }

    template <typename Q>
    static int launch_dequantize(const void* in, const float* scale, const void* zp, float* out,
                                 const QuantPlan& p, cudaStream_t st)
    {
        if (use_rows(p, in, out))
        {
            uint32_t chunks = uint32_t((p.inner + QCHUNK - 1) / QCHUNK);
            dequantize_rows_kernel<Q><<<unsigned(chunks * p.rows), QT, 0, st>>>(
                static_cast<const Q*>(in), scale, static_cast<const Q*>(zp), out, p.inner, chunks, p.n_scales);
        }
        else
        {
            dequantize_generic_kernel<Q><<<generic_grid(p.total), QT, 0, st>>>(
                static_cast<const Q*>(in), scale, static_cast<const Q*>(zp), out, p.total, p.dims);
        }
        return after_launch("b200_dequantize");
    }
}

extern "C" int b200_set_fast_division(int enable)
{
    int old = b200::g_fast_division.exchange(enable ? 1 : 0);
    return old;
}

extern "C" int b200_quantize(const float* input, const float* scale, const void* zero_point, void* output,
                             int quant_type, const int64_t* shape, int rank, const int64_t* axes, int n_axes,
                             int round_mode, void* stream)
{
    using namespace b200;
    QuantPlan p;
    int rc = make_plan(shape, rank, axes, n_axes, p);
    if (rc != B200_OK)
        return rc;
    if (round_mode < 0 || round_mode > 8)
        return B200_ERR_INVALID_ARGUMENT;
    if (quant_type != B200_U8 && quant_type != B200_I8 && quant_type != B200_I32)
        return B200_ERR_INVALID_ARGUMENT;
    if (p.total == 0)
        return B200_OK;
    if (!input || !scale || !zero_point || !output)
        return B200_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (quant_type)
    {
    case B200_U8: return dispatch_quantize_mode<uint8_t>(round_mode, input, scale, zero_point, output, p, st);
    case B200_I8: return dispatch_quantize_mode<int8_t>(round_mode, input, scale, zero_point, output, p, st);
    default: return dispatch_quantize_mode<int32_t>(round_mode, input, scale, zero_point, output, p, st);
    }
}

extern "C" int b200_dequantize(const void* input, const float* scale, const void* zero_point, float* output,
                               int quant_type, const int64_t* shape, int rank, const int64_t* axes, int n_axes,
                               void* stream)
{
    using namespace b200;
    QuantPlan p;
    int rc = make_plan(shape, rank, axes, n_axes, p);
    if (rc != B200_OK)
        return rc;
    if (quant_type != B200_U8 && quant_type != B200_I8 && quant_type != B200_I32)
        return B200_ERR_INVALID_ARGUMENT;
    if (p.total == 0)
        return B200_OK;
    if (!input || !scale || !zero_point || !output)
        return B200_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (quant_type)
    {
    case B200_U8: return launch_dequantize<uint8_t>(input, scale, zero_point, output, p, st);
    case B200_I8: return launch_dequantize<int8_t>(input, scale, zero_point, output, p, st);
    default: return launch_dequantize<int32_t>(input, scale, zero_point, output, p, st);
    }
}

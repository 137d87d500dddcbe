// f32 glue operators of quantized graphs (the float islands between int8 contractions: softmax, LayerNorm,
// GELU, residual adds, dynamic activation scales) with the arithmetic of nGraph's reference kernels:
//
//   elementwise +, -, *, /, max, min, abs, neg, sqrt, relu   IEEE single, one rounding each, nothing contracted
//   exp, erf                                                   reference: std::exp / std::erf on float; here the double
//                                                              routine rounded to float (differs from a given libm in
//                                                              the last bit on a small share of inputs)
//   Sum          runtime/reference/sum.hpp:56-90     Kahan-compensated, inputs taken in row-major order
//   Max          runtime/reference/max.hpp:32-58     start at -inf, replace when x > max
//   Broadcast    runtime/reference/broadcast.hpp     output coordinate with the broadcast axes dropped
//   BatchMatMul  runtime/reference/batch_mat_mul.hpp -> dot.hpp:108-160: the sum over k runs in DOUBLE, in order,
//                over exact products, and is rounded to float once
//   Gather       runtime/reference/gather.hpp        rows of a matrix picked by an index vector
//   Reshape      runtime/reference/reshape.hpp       axis permutation followed by a free re-interpretation
//
// All are HBM-bound (or, for the reductions and the matrix product, latency-bound on purpose: they keep the
// reference's summation order so that results are identical, not merely close).
#include <cuda_runtime.h>
#include <math.h>
#include <initializer_list>
#include "common.cuh"

namespace b200
{
    constexpr int MAX_RANK = 8;
    struct Dims
    {
        int rank;
        int64_t out_dim[MAX_RANK];    // shape of the tensor the thread index runs over
        int64_t in_stride[MAX_RANK];  // element stride in the other tensor for each of those axes (0: axis absent)
    };

    __device__ __forceinline__ int64_t mapped_offset(const Dims& d, int64_t idx)
    {
        int64_t off = 0;
#pragma unroll 1
        for (int a = d.rank - 1; a >= 0; --a)
        {
            const int64_t c = idx % d.out_dim[a];
            idx /= d.out_dim[a];
            off += c * d.in_stride[a];
        }
        return off;
    }

    template <int OP>
    __device__ __forceinline__ float binary_op(float a, float b)
    {
        switch (OP)
        {
        case B200_F32_ADD: return __fadd_rn(a, b);
        case B200_F32_SUB: return __fsub_rn(a, b);
        case B200_F32_MUL: return __fmul_rn(a, b);
        case B200_F32_DIV: return __fdiv_rn(a, b);
        case B200_F32_MAX: return a > b ? a : b; // reference::maximum
        default: return a < b ? a : b;           // reference::minimum
        }
    }

    template <int OP>
    __global__ void __launch_bounds__(256) binary_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                         float* __restrict__ out, int64_t n)
    {
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
            out[i] = binary_op<OP>(a[i], b[i]);
    }

    // One operand is a small tensor that op::v0::Broadcast would repeat along new leading axes (a bias row, a scalar
    // factor): element i of the large operand meets v[i % period] instead of a materialised copy.  V_LEFT: v is the
    // left-hand operand.  Four neighbours at a time when `period` allows it.
    template <int OP, bool V_LEFT, bool VEC>
    __global__ void __launch_bounds__(256) binary_periodic_kernel(const float* __restrict__ a, const float* __restrict__ v,
                                                                  float* __restrict__ out, int64_t n, int64_t period)
    {
        if (VEC)
        {
            const int64_t n4 = n >> 2, p4 = period >> 2; // period == 1: p4 == 0
            const float4* a4 = reinterpret_cast<const float4*>(a);
            const float s = p4 == 0 ? __ldg(v) : 0.0f;
            for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += int64_t(gridDim.x) * blockDim.x)
            {
                const float4 x = a4[i];
                const float4 y = p4 == 0 ? make_float4(s, s, s, s) : __ldg(reinterpret_cast<const float4*>(v) + i % p4);
                float4 r;
                r.x = V_LEFT ? binary_op<OP>(y.x, x.x) : binary_op<OP>(x.x, y.x);
                r.y = V_LEFT ? binary_op<OP>(y.y, x.y) : binary_op<OP>(x.y, y.y);
                r.z = V_LEFT ? binary_op<OP>(y.z, x.z) : binary_op<OP>(x.z, y.z);
                r.w = V_LEFT ? binary_op<OP>(y.w, x.w) : binary_op<OP>(x.w, y.w);
                reinterpret_cast<float4*>(out)[i] = r;
            }
        }
        else
            for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
            {
                const float x = a[i], y = __ldg(v + i % period);
                out[i] = V_LEFT ? binary_op<OP>(y, x) : binary_op<OP>(x, y);
            }
    }

    template <int OP>
    void launch_binary_periodic(const float* a, const float* v, float* out, int64_t n, int64_t period, bool v_left, cudaStream_t st)
    {
        const bool vec = n % 4 == 0 && (period == 1 || period % 4 == 0) &&
                         ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(out) | (period == 1 ? 0 : reinterpret_cast<uintptr_t>(v))) & 15) == 0;
        const int64_t work = vec ? n / 4 : n, blocks = (work + 255) / 256, cap = b200::sm_count() * 16;
        const unsigned g = unsigned(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
        if (vec && v_left) binary_periodic_kernel<OP, true, true><<<g, 256, 0, st>>>(a, v, out, n, period);
        else if (vec) binary_periodic_kernel<OP, false, true><<<g, 256, 0, st>>>(a, v, out, n, period);
        else if (v_left) binary_periodic_kernel<OP, true, false><<<g, 256, 0, st>>>(a, v, out, n, period);
        else binary_periodic_kernel<OP, false, false><<<g, 256, 0, st>>>(a, v, out, n, period);
    }

    template <int OP>
    __device__ __forceinline__ float unary_op(float x)
    {
        switch (OP)
        {
        case B200_F32_ABS: return fabsf(x);
        case B200_F32_NEG: return -x;
        case B200_F32_SQRT: return __fsqrt_rn(x);
        case B200_F32_EXP: return static_cast<float>(exp(static_cast<double>(x)));
        case B200_F32_ERF: return static_cast<float>(erf(static_cast<double>(x)));
        default: return x > 0.0f ? x : 0.0f; // reference::relu
        }
    }

    template <int OP>
    __global__ void __launch_bounds__(256) unary_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t n)
    {
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
            out[i] = unary_op<OP>(x[i]);
    }

    // out[idx] = in[mapped(idx)] for 4-byte elements: Broadcast (stride 0 on the new axes) and axis permutations.
    // T: one element (uint32_t) or four neighbours along a last axis that both tensors share (uint4); IDX: 32-bit index
    // arithmetic when every index and offset fits (a 64-bit division costs several times a 32-bit one).
    template <typename T, typename IDX>
    __global__ void __launch_bounds__(256) remap_kernel(const T* __restrict__ in, T* __restrict__ out, Dims d, int64_t n)
    {
        IDX dim[MAX_RANK], stride[MAX_RANK];
#pragma unroll
        for (int a = 0; a < MAX_RANK; ++a)
        {
            dim[a] = a < d.rank ? IDX(d.out_dim[a]) : IDX(1);
            stride[a] = a < d.rank ? IDX(d.in_stride[a]) : IDX(0);
        }
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
        {
            IDX idx = IDX(i), off = 0;
#pragma unroll
            for (int a = MAX_RANK - 1; a >= 0; --a)
                if (a < d.rank)
                {
                    const IDX q = idx / dim[a];
                    off += (idx - q * dim[a]) * stride[a];
                    idx = q;
                }
            out[i] = in[off];
        }
    }

    // Picks the widest form the tensors allow.  `d` describes the output axes and the input stride of each.
    static void launch_remap(const void* in, void* out, Dims d, int64_t n, int64_t in_elements, cudaStream_t st)
    {
        const int last = d.rank - 1;
        bool wide = d.rank >= 1 && d.in_stride[last] == 1 && d.out_dim[last] % 4 == 0 &&
                    ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
        for (int a = 0; wide && a < last; ++a)
            wide = d.in_stride[a] % 4 == 0;
        if (wide)
        {
            d.out_dim[last] /= 4;
            for (int a = 0; a < last; ++a)
                d.in_stride[a] /= 4;
            n /= 4;
            in_elements /= 4;
        }
        const bool small = n < (int64_t(1) << 31) && in_elements < (int64_t(1) << 31);
        const int64_t blocks = (n + 255) / 256, cap = b200::sm_count() * 16;
        const unsigned grid = unsigned(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
        if (wide && small)
            remap_kernel<uint4, uint32_t><<<grid, 256, 0, st>>>(static_cast<const uint4*>(in), static_cast<uint4*>(out), d, n);
        else if (wide)
            remap_kernel<uint4, int64_t><<<grid, 256, 0, st>>>(static_cast<const uint4*>(in), static_cast<uint4*>(out), d, n);
        else if (small)
            remap_kernel<uint32_t, uint32_t><<<grid, 256, 0, st>>>(static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out), d, n);
        else
            remap_kernel<uint32_t, int64_t><<<grid, 256, 0, st>>>(static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out), d, n);
    }

    // One thread per output element; the reduced coordinates are walked in row-major order, as the reference does.
    // keep: the kept axes (thread index -> input offset); red: the reduced axes.
    // One step of the reference's compensated sum (runtime/reference/sum.hpp:56-90).
    __device__ __forceinline__ void kahan_step(float& z, float& c, float x)
    {
        if (isfinite(x) && isfinite(z))
        {
            const float y = __fsub_rn(x, c);
            const float t = __fadd_rn(z, y);
            c = __fsub_rn(__fsub_rn(t, z), y);
            z = t;
        }
        else
            z = __fadd_rn(z, x);
    }

    template <int OP> // b200_reduce_op
    __global__ void __launch_bounds__(128) reduce_kernel(const float* __restrict__ in, float* __restrict__ out, Dims keep, Dims red,
                                                         int64_t n_out, int64_t n_red)
    {
        for (int64_t o = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; o < n_out; o += int64_t(gridDim.x) * blockDim.x)
        {
            const float* base = in + mapped_offset(keep, o);
            if (OP == B200_REDUCE_SUM)
            {
                float z = 0.0f, c = 0.0f;
                for (int64_t r = 0; r < n_red; ++r)
                    kahan_step(z, c, base[mapped_offset(red, r)]);
                out[o] = z;
            }
            else
            {
                // max.hpp:32-58 / min.hpp: start from -inf / +inf, replace on a strict comparison (a NaN never wins)
                float m = OP == B200_REDUCE_MIN ? INFINITY : -INFINITY;
                for (int64_t r = 0; r < n_red; ++r)
                {
                    float x = base[mapped_offset(red, r)];
                    if (OP == B200_REDUCE_MAX_ABS)
                        x = fabsf(x);
                    if (OP == B200_REDUCE_MIN ? x < m : x > m)
                        m = x;
                }
                out[o] = m;
            }
        }
    }

    // Max with few outputs and long reductions (a whole-tensor max for a dynamic activation scale): one block per
    // output.  The result of a max does not depend on the order the inputs are taken in (NaNs never win the
    // x > max test, in any order), so this equals the sequential reference loop.
    __global__ void __launch_bounds__(256) reduce_max_block_kernel(const float* __restrict__ in, float* __restrict__ out, Dims keep,
                                                                   Dims red, int64_t n_red)
    {
        __shared__ float partial[8];
        const float* base = in + mapped_offset(keep, blockIdx.x);
        float m = -INFINITY;
        for (int64_t r = threadIdx.x; r < n_red; r += blockDim.x)
        {
            const float x = base[mapped_offset(red, r)];
            if (x > m)
                m = x;
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1)
        {
            const float o = __shfl_xor_sync(0xffffffffu, m, d);
            if (o > m)
                m = o;
        }
        if ((threadIdx.x & 31) == 0)
            partial[threadIdx.x >> 5] = m;
        __syncthreads();
        if (threadIdx.x == 0)
        {
            for (int w = 1; w < 8; ++w)
                if (partial[w] > m)
                    m = partial[w];
            out[blockIdx.x] = m;
        }
    }

    // Whole-tensor max (one output): many blocks, each over a contiguous slice, combined with an atomic on the ordered
    // integer image of the float (non-negative floats order like signed ints, negative ones like reversed unsigned
    // ints).  NaNs never win, as in the reference loop; the output must hold -inf on entry.
    template <bool ABS> // the max of |x|: op::v0::Max over op::v0::Abs without the tensor in between
    __global__ void __launch_bounds__(256) reduce_max_all_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t n)
    {
        __shared__ float partial[8];
        float m = -INFINITY;
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
        {
            const float x = ABS ? fabsf(in[i]) : in[i];
            if (x > m)
                m = x;
        }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1)
        {
            const float o = __shfl_xor_sync(0xffffffffu, m, d);
            if (o > m)
                m = o;
        }
        if ((threadIdx.x & 31) == 0)
            partial[threadIdx.x >> 5] = m;
        __syncthreads();
        if (threadIdx.x == 0)
        {
            for (int w = 1; w < 8; ++w)
                if (partial[w] > m)
                    m = partial[w];
            if (m >= 0.0f)
                atomicMax(reinterpret_cast<int*>(out), __float_as_int(m));
            else if (m > -INFINITY)
                atomicMin(reinterpret_cast<unsigned int*>(out), __float_as_uint(m));
        }
    }

    __global__ void fill_f32_kernel(float* out, float value, int64_t n)
    {
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
            out[i] = value;
    }

    // Softmax and LayerNorm over the LAST axis of a [rows, L] matrix.  Their compensated sums have to walk a row in
    // order, so a row belongs to one thread; reading it straight from memory would make the 32 lanes of a warp touch 32
    // different rows per load.  A block therefore stages 32 rows in shared memory, lets all its threads do the
    // order-free parts (max, exp, normalise, divide) and one warp the 32 ordered sums, one row per lane.
    // VEC: L is a multiple of 4 and the pointers are 16-byte aligned, so rows move as float4 with eight loads in flight
    // per thread (row stride L + 4: the ordered walks then meet 4-way bank conflicts, hidden behind the dependent
    // additions); otherwise element by element with an odd row stride.
    constexpr int ROWS_PER_TILE = 32;
    __host__ __device__ inline int staged_row_stride(int L, bool vec) { return vec ? L + 4 : (L | 1); }

    // The elementwise op that produced the rows can be applied while they are staged (one rounding, the same value the
    // op's own kernel would have written): factor != nullptr multiplies by the scalar *factor (op::v1::Multiply by a
    // broadcast scalar), addend != nullptr adds the rows of a second tensor (op::v1::Add).
    template <bool VEC>
    __device__ __forceinline__ void stage_rows(const float* __restrict__ src, float* tile, int n_rows, int L, int stride,
                                               const float* __restrict__ factor, const float* __restrict__ addend)
    {
        const float f = factor ? __ldg(factor) : 1.0f;
        if (VEC)
        {
            const int L4 = L >> 2, total = n_rows * L4;
            const float4* src4 = reinterpret_cast<const float4*>(src);
            const float4* add4 = reinterpret_cast<const float4*>(addend);
            for (int i0 = threadIdx.x; i0 < total; i0 += blockDim.x * 8)
            {
                float4 v[8], w[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                {
                    const int i = i0 + j * blockDim.x;
                    if (i < total)
                    {
                        v[j] = __ldg(src4 + i);
                        if (addend)
                            w[j] = __ldg(add4 + i);
                    }
                }
#pragma unroll
                for (int j = 0; j < 8; ++j)
                {
                    const int i = i0 + j * blockDim.x;
                    if (i < total)
                    {
                        float4 r = v[j];
                        if (factor)
                            r = make_float4(__fmul_rn(r.x, f), __fmul_rn(r.y, f), __fmul_rn(r.z, f), __fmul_rn(r.w, f));
                        if (addend)
                            r = make_float4(__fadd_rn(r.x, w[j].x), __fadd_rn(r.y, w[j].y), __fadd_rn(r.z, w[j].z), __fadd_rn(r.w, w[j].w));
                        *reinterpret_cast<float4*>(tile + (i / L4) * stride + 4 * (i % L4)) = r;
                    }
                }
            }
        }
        else
            for (int i = threadIdx.x; i < n_rows * L; i += blockDim.x)
            {
                float r = src[i];
                if (factor)
                    r = __fmul_rn(r, f);
                if (addend)
                    r = __fadd_rn(r, addend[i]);
                tile[(i / L) * stride + i % L] = r;
            }
    }

    template <bool VEC>
    __global__ void __launch_bounds__(128) softmax_rows_kernel(const float* __restrict__ in, const float* __restrict__ factor, float* __restrict__ out,
                                                               int64_t rows, int L)
    {
        extern __shared__ __align__(16) float tile[];
        __shared__ float row_max[ROWS_PER_TILE], row_sum[ROWS_PER_TILE];
        const int stride = staged_row_stride(L, VEC);
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int64_t n_tiles = (rows + ROWS_PER_TILE - 1) / ROWS_PER_TILE;
        for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x)
        {
            const int64_t row0 = t * ROWS_PER_TILE;
            const int n_rows = int(rows - row0 < ROWS_PER_TILE ? rows - row0 : ROWS_PER_TILE);
            stage_rows<VEC>(in + row0 * L, tile, n_rows, L, stride, factor, nullptr);
            __syncthreads();
            // softmax.hpp: max over the axis (the largest value whatever the order), then exp(x - max)
            for (int r = warp; r < n_rows; r += 4)
            {
                float m = -INFINITY;
                for (int c = lane; c < L; c += 32)
                {
                    const float x = tile[r * stride + c];
                    m = x > m ? x : m;
                }
                for (int d = 16; d; d >>= 1)
                {
                    const float o = __shfl_xor_sync(0xFFFFFFFFu, m, d);
                    m = o > m ? o : m;
                }
                // the same warp owns the row in the next step too, so no block-wide barrier is needed in between
                for (int c = lane; c < L; c += 32)
                {
                    float& v = tile[r * stride + c];
                    v = static_cast<float>(exp(static_cast<double>(__fsub_rn(v, m))));
                }
            }
            __syncthreads();
            if (warp == 0 && lane < n_rows)
            {
                const float* row = tile + lane * stride;
                float z = 0.0f, c = 0.0f;
                for (int k = 0; k < L; ++k)
                    kahan_step(z, c, row[k]);
                row_sum[lane] = z;
            }
            __syncthreads();
            float* dst = out + row0 * L;
            if (VEC)
            {
                const int L4 = L >> 2, total = n_rows * L4;
                for (int i = threadIdx.x; i < total; i += blockDim.x)
                {
                    const int r = i / L4;
                    float4 v = *reinterpret_cast<const float4*>(tile + r * stride + 4 * (i % L4));
                    const float sum = row_sum[r];
                    v.x = __fdiv_rn(v.x, sum), v.y = __fdiv_rn(v.y, sum), v.z = __fdiv_rn(v.z, sum), v.w = __fdiv_rn(v.w, sum);
                    reinterpret_cast<float4*>(dst)[i] = v;
                }
            }
            else
                for (int i = threadIdx.x; i < n_rows * L; i += blockDim.x)
                {
                    const int r = i / L;
                    dst[i] = __fdiv_rn(tile[r * stride + i % L], row_sum[r]);
                }
            __syncthreads();
        }
    }

    // op::v0::LayerNorm over the last axis with scale and bias, as ONE kernel with the rounding steps of its
    // decomposition (src/ngraph/op/layer_norm.cpp:68-150 with builder::mean / builder::variance,
    // src/ngraph/builder/reduce_ops.cpp:68-127), in that order:
    //   mean = KahanSum(x) / N;  var = KahanSum((x - mean) * (x - mean)) / N;  sd = sqrt(var + eps);
    //   y = ((x - mean) / sd) * gamma + beta          (every operation a separate IEEE rounding, no fused multiply-add)
    template <bool VEC>
    __global__ void __launch_bounds__(128) layer_norm_rows_kernel(const float* __restrict__ in, const float* __restrict__ addend,
                                                                  const float* __restrict__ gamma, const float* __restrict__ beta,
                                                                  float* __restrict__ out, int64_t rows, int L, float count, float eps)
    {
        extern __shared__ __align__(16) float tile[];
        __shared__ float row_mean[ROWS_PER_TILE], row_sd[ROWS_PER_TILE];
        const int stride = staged_row_stride(L, VEC);
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int64_t n_tiles = (rows + ROWS_PER_TILE - 1) / ROWS_PER_TILE;
        for (int64_t t = blockIdx.x; t < n_tiles; t += gridDim.x)
        {
            const int64_t row0 = t * ROWS_PER_TILE;
            const int n_rows = int(rows - row0 < ROWS_PER_TILE ? rows - row0 : ROWS_PER_TILE);
            stage_rows<VEC>(in + row0 * L, tile, n_rows, L, stride, nullptr, addend ? addend + row0 * L : nullptr);
            __syncthreads();
            if (warp == 0 && lane < n_rows)
            {
                const float* row = tile + lane * stride;
                float z = 0.0f, c = 0.0f;
                for (int k = 0; k < L; ++k)
                    kahan_step(z, c, row[k]);
                const float mean = __fdiv_rn(z, count);
                z = 0.0f, c = 0.0f;
                for (int k = 0; k < L; ++k)
                {
                    const float d = __fsub_rn(row[k], mean);
                    kahan_step(z, c, __fmul_rn(d, d));
                }
                row_mean[lane] = mean;
                row_sd[lane] = __fsqrt_rn(__fadd_rn(__fdiv_rn(z, count), eps));
            }
            __syncthreads();
            float* dst = out + row0 * L;
            if (VEC)
            {
                const int L4 = L >> 2, total = n_rows * L4;
                for (int i = threadIdx.x; i < total; i += blockDim.x)
                {
                    const int r = i / L4, k4 = i % L4;
                    float4 v = *reinterpret_cast<const float4*>(tile + r * stride + 4 * k4);
                    const float4 g = __ldg(reinterpret_cast<const float4*>(gamma) + k4), b = __ldg(reinterpret_cast<const float4*>(beta) + k4);
                    const float mean = row_mean[r], sd = row_sd[r];
                    v.x = __fadd_rn(__fmul_rn(__fdiv_rn(__fsub_rn(v.x, mean), sd), g.x), b.x);
                    v.y = __fadd_rn(__fmul_rn(__fdiv_rn(__fsub_rn(v.y, mean), sd), g.y), b.y);
                    v.z = __fadd_rn(__fmul_rn(__fdiv_rn(__fsub_rn(v.z, mean), sd), g.z), b.z);
                    v.w = __fadd_rn(__fmul_rn(__fdiv_rn(__fsub_rn(v.w, mean), sd), g.w), b.w);
                    reinterpret_cast<float4*>(dst)[i] = v;
                }
            }
            else
                for (int i = threadIdx.x; i < n_rows * L; i += blockDim.x)
                {
                    const int r = i / L, k = i % L;
                    const float norm = __fdiv_rn(__fsub_rn(tile[r * stride + k], row_mean[r]), row_sd[r]);
                    dst[i] = __fadd_rn(__fmul_rn(norm, __ldg(gamma + k)), __ldg(beta + k));
                }
            __syncthreads();
        }
    }

    // op::v0::Gelu with the rounding steps of its decomposition (src/ngraph/op/gelu.cpp:46-60):
    //   (0.5 * x) * (1 + erf(x / float(sqrt(2.0))))
    __global__ void __launch_bounds__(256) gelu_kernel(const float* __restrict__ x, float* __restrict__ out, int64_t n)
    {
        const float sqrt_two = static_cast<float>(1.4142135623730951);
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
        {
            const float v = x[i];
            const float e = static_cast<float>(erf(static_cast<double>(__fdiv_rn(v, sqrt_two))));
            out[i] = __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, e));
        }
    }

    // Sum over the last axis for rows of any length: a warp owns 32 rows, one per lane, and walks them 64 columns at a
    // time; each 32 x 64 panel is fetched with coalesced loads into shared memory (row stride 65: the lanes' walks hit
    // 32 different banks) and then added in column order with the reference's compensated step.  Many one-warp blocks per
    // SM overlap one block's loads with another's additions.
    __global__ void __launch_bounds__(32) sum_rows_kernel(const float* __restrict__ in, float* __restrict__ out, int64_t rows, int64_t L)
    {
        constexpr int CH = 64;
        __shared__ float panel[32][CH + 1];
        const int lane = threadIdx.x;
        for (int64_t row0 = int64_t(blockIdx.x) * 32; row0 < rows; row0 += int64_t(gridDim.x) * 32)
        {
            const int n_rows = int(rows - row0 < 32 ? rows - row0 : 32);
            float z = 0.0f, c = 0.0f;
            for (int64_t col0 = 0; col0 < L; col0 += CH)
            {
                const int n_col = int(L - col0 < CH ? L - col0 : CH);
                // lane l fetches columns l and l + 32 of every row: 16 rows at a time, 32 loads in flight
#pragma unroll
                for (int r0 = 0; r0 < 32; r0 += 16)
                {
                    float v[16][2];
#pragma unroll
                    for (int r = 0; r < 16; ++r)
#pragma unroll
                        for (int h = 0; h < 2; ++h)
                            v[r][h] = (r0 + r < n_rows && lane + 32 * h < n_col) ? in[(row0 + r0 + r) * L + col0 + lane + 32 * h] : 0.0f;
#pragma unroll
                    for (int r = 0; r < 16; ++r)
#pragma unroll
                        for (int h = 0; h < 2; ++h)
                            panel[r0 + r][lane + 32 * h] = v[r][h];
                }
                __syncwarp();
                if (lane < n_rows)
                    for (int cc = 0; cc < n_col; ++cc)
                        kahan_step(z, c, panel[lane][cc]);
                __syncwarp();
            }
            if (lane < n_rows)
                out[row0 + lane] = z;
        }
    }

    // Grid and shared memory of the two staged kernels: as many 32-row tiles per SM as fit.
    template <typename Kernel>
    bool staged_launch_shape(Kernel kernel, int64_t rows, int L, bool vec, unsigned& grid, size_t& bytes)
    {
        bytes = size_t(ROWS_PER_TILE) * staged_row_stride(L, vec) * sizeof(float);
        if (bytes > 48 * 1024 && // the attribute belongs to the current device's copy of the kernel: set it on each use
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
            return false;
        const int64_t tiles = (rows + ROWS_PER_TILE - 1) / ROWS_PER_TILE;
        const int64_t per_sm = (200 * 1024) / int64_t(bytes) < 8 ? (200 * 1024) / int64_t(bytes) : 8;
        grid = unsigned(tiles < b200::sm_count() * per_sm ? tiles : b200::sm_count() * per_sm);
        return true;
    }

    inline bool all_aligned16(std::initializer_list<const void*> ptrs)
    {
        uintptr_t bits = 0;
        for (const void* p : ptrs)
            bits |= reinterpret_cast<uintptr_t>(p);
        return (bits & 15) == 0;
    }

    // out[b, m, n] = float(sum_k double(a[b, m, k]) * double(b[b, k, n])), k ascending.  One thread owns a 4 x 4 block
    // of outputs, each with its own double accumulator walked in k order (so every output sees exactly the reference's
    // sequence of additions); the block shares 4 + 4 operand loads per 16 multiply-adds.
    __global__ void __launch_bounds__(128) bmm_f32_kernel(const float* __restrict__ a, const float* __restrict__ bm,
                                                          float* __restrict__ out, int64_t B, int M, int K, int N)
    {
        const int tiles_n = (N + 3) / 4, tiles_m = (M + 3) / 4;
        const int64_t total = B * tiles_m * tiles_n;
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x)
        {
            const int tn = int(i % tiles_n);
            const int64_t t = i / tiles_n;
            const int tm = int(t % tiles_m);
            const int64_t b = t / tiles_m;
            const int m0 = tm * 4, n0 = tn * 4;
            const float* ap = a + (b * M + m0) * K;
            const float* bp = bm + b * K * N + n0;
            // rows / columns beyond the matrix read the last valid one (their results are not stored)
            const int r1 = m0 + 1 < M ? 1 : 0, r2 = m0 + 2 < M ? 2 : r1, r3 = m0 + 3 < M ? 3 : r2;
            const int c1 = n0 + 1 < N ? 1 : 0, c2 = n0 + 2 < N ? 2 : c1, c3 = n0 + 3 < N ? 3 : c2;
            double acc[4][4];
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    acc[r][c] = 0.0;
            for (int k = 0; k < K; ++k)
            {
                const double x0 = ap[k], x1 = ap[int64_t(r1) * K + k], x2 = ap[int64_t(r2) * K + k], x3 = ap[int64_t(r3) * K + k];
                const float* brow = bp + int64_t(k) * N;
                const double y0 = brow[0], y1 = brow[c1], y2 = brow[c2], y3 = brow[c3];
                const double xs[4] = {x0, x1, x2, x3}, ys[4] = {y0, y1, y2, y3};
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        acc[r][c] = fma(xs[r], ys[c], acc[r][c]); // a product of two floats is exact in double: one rounding, like mul + add
            }
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    if (m0 + r < M && n0 + c < N)
                        out[(b * M + m0 + r) * N + n0 + c] = static_cast<float>(acc[r][c]);
        }
    }

    // The same product for large matrices: a block of 256 threads owns a TM x TN tile of one batch entry.  Operands are
    // converted to double ONCE per block and K chunk into shared memory (the conversion, not the multiply-add, limits
    // the register-only kernel above), and every thread keeps (TM/16) x (TN/16) double accumulators for the outputs
    // (ty + 16 i, tx + 16 j).  Each accumulator still receives its products in ascending k, one rounding each, so the
    // result is bit-identical to the kernel above.  Zero-filled padding beyond M, N or K adds fma(0, 0, acc) = acc.
    template <int TM, int TN, int KC>
    __global__ void __launch_bounds__(256) bmm_f32_tiled_kernel(const float* __restrict__ a, const float* __restrict__ bm,
                                                                float* __restrict__ out, int M, int K, int N, int tiles_m, int tiles_n)
    {
        constexpr int RM = TM / 16, RN = TN / 16;
        constexpr int LDA = TM + 2, LDB = TN; // LDA: the transposing store of the A panel spreads over the banks
        extern __shared__ double panels[];
        double* As = panels;            // [KC][LDA]  As[k][m]
        double* Bs = panels + KC * LDA; // [KC][LDB]  Bs[k][n]
        const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
        const int tile = blockIdx.x;
        const int tn = tile % tiles_n, tm = (tile / tiles_n) % tiles_m;
        const int64_t batch = tile / (tiles_n * tiles_m);
        const int m0 = tm * TM, n0 = tn * TN;
        const float* ab = a + batch * int64_t(M) * K;
        const float* bb = bm + batch * int64_t(K) * N;
        double acc[RM][RN];
#pragma unroll
        for (int i = 0; i < RM; ++i)
#pragma unroll
            for (int j = 0; j < RN; ++j)
                acc[i][j] = 0.0;
        // the panels of chunk c + 1 travel from memory into registers while chunk c is multiplied out of shared memory
        constexpr int A_PER = TM * KC / 256, B_PER = KC * TN / 256;
        float ra[A_PER], rb[B_PER];
        auto fetch = [&](int k0) {
#pragma unroll
            for (int j = 0; j < A_PER; ++j)
            {
                const int i = tid + j * 256, m = i / KC, k = i % KC; // consecutive threads along k (contiguous in memory)
                ra[j] = (m0 + m < M && k0 + k < K) ? ab[int64_t(m0 + m) * K + k0 + k] : 0.0f;
            }
#pragma unroll
            for (int j = 0; j < B_PER; ++j)
            {
                const int i = tid + j * 256, k = i / TN, n = i % TN; // consecutive threads along n
                rb[j] = (k0 + k < K && n0 + n < N) ? bb[int64_t(k0 + k) * N + n0 + n] : 0.0f;
            }
        };
        auto stash = [&]() {
#pragma unroll
            for (int j = 0; j < A_PER; ++j)
            {
                const int i = tid + j * 256;
                As[(i % KC) * LDA + i / KC] = double(ra[j]);
            }
#pragma unroll
            for (int j = 0; j < B_PER; ++j)
            {
                const int i = tid + j * 256;
                Bs[(i / TN) * LDB + i % TN] = double(rb[j]);
            }
        };
        fetch(0);
        stash();
        __syncthreads();
        for (int k0 = 0; k0 < K; k0 += KC)
        {
            const bool more = k0 + KC < K;
            if (more)
                fetch(k0 + KC);
#pragma unroll 4
            for (int k = 0; k < KC; ++k)
            {
                double x[RM], y[RN];
#pragma unroll
                for (int i = 0; i < RM; ++i)
                    x[i] = As[k * LDA + ty + 16 * i];
#pragma unroll
                for (int j = 0; j < RN; ++j)
                    y[j] = Bs[k * LDB + tx + 16 * j];
#pragma unroll
                for (int i = 0; i < RM; ++i)
#pragma unroll
                    for (int j = 0; j < RN; ++j)
                        acc[i][j] = fma(x[i], y[j], acc[i][j]);
            }
            __syncthreads();
            if (more)
            {
                stash();
                __syncthreads();
            }
        }
        float* ob = out + batch * int64_t(M) * N;
#pragma unroll
        for (int i = 0; i < RM; ++i)
#pragma unroll
            for (int j = 0; j < RN; ++j)
            {
                const int m = m0 + ty + 16 * i, n = n0 + tx + 16 * j;
                if (m < M && n < N)
                    ob[int64_t(m) * N + n] = static_cast<float>(acc[i][j]);
            }
    }

    template <int TM, int TN, int KC>
    bool launch_bmm_tiled(const float* a, const float* b, float* out, int64_t batch, int M, int K, int N, cudaStream_t st)
    {
        constexpr size_t bytes = size_t(KC) * (TM + 2 + TN) * sizeof(double);
        if (cudaFuncSetAttribute(bmm_f32_tiled_kernel<TM, TN, KC>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes)) != cudaSuccess)
            return false;
        const int tiles_m = (M + TM - 1) / TM, tiles_n = (N + TN - 1) / TN;
        const int64_t tiles = batch * tiles_m * tiles_n;
        if (tiles > 0x7FFFFFFF)
            return false;
        bmm_f32_tiled_kernel<TM, TN, KC><<<unsigned(tiles), 256, bytes, st>>>(a, b, out, M, K, N, tiles_m, tiles_n);
        return true;
    }

    template <typename I>
    __global__ void __launch_bounds__(256) gather_rows_kernel(const uint32_t* __restrict__ table, const I* __restrict__ idx,
                                                              uint32_t* __restrict__ out, int64_t n_idx, int64_t row_words,
                                                              int64_t n_rows)
    {
        const int64_t total = n_idx * row_words;
        for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x)
        {
            const int64_t r = i / row_words, w = i - r * row_words;
            const int64_t src = int64_t(idx[r]);
            out[i] = (src >= 0 && src < n_rows) ? table[src * row_words + w] : 0u; // the reference does not check
        }
    }

    static unsigned grid_for(int64_t n, int threads)
    {
        int64_t blocks = (n + threads - 1) / threads;
        const int64_t cap = int64_t(b200::sm_count()) * 16;
        return unsigned(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
    }
}

extern "C" int b200_f32_binary(int op, const float* a, const float* b, float* out, int64_t n, void* stream)
{
    using namespace b200;
    if (n < 0 || op < B200_F32_ADD || op > B200_F32_MIN)
        return B200_ERR_INVALID_ARGUMENT;
    if (n == 0)
        return B200_OK;
    if (!a || !b || !out)
        return B200_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned g = grid_for(n, 256);
    switch (op)
    {
    case B200_F32_ADD: binary_kernel<B200_F32_ADD><<<g, 256, 0, st>>>(a, b, out, n); break;
    case B200_F32_SUB: binary_kernel<B200_F32_SUB><<<g, 256, 0, st>>>(a, b, out, n); break;
    case B200_F32_MUL: binary_kernel<B200_F32_MUL><<<g, 256, 0, st>>>(a, b, out, n); break;
    case B200_F32_DIV: binary_kernel<B200_F32_DIV><<<g, 256, 0, st>>>(a, b, out, n); break;
    case B200_F32_MAX: binary_kernel<B200_F32_MAX><<<g, 256, 0, st>>>(a, b, out, n); break;
    default: binary_kernel<B200_F32_MIN><<<g, 256, 0, st>>>(a, b, out, n); break;
    }
    return after_launch("b200_f32_binary");
}

extern "C" int b200_f32_binary_periodic(int op, const float* a, const float* v, float* out, int64_t n, int64_t period, int v_is_left,
                                        void* stream)
{
    using namespace b200;
    if (n < 0 || period < 1 || op < B200_F32_ADD || op > B200_F32_MIN)
        return B200_ERR_INVALID_ARGUMENT;
    if (n == 0)
        return B200_OK;
    if (!a || !v || !out || n % period != 0)
        return B200_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool left = v_is_left != 0;
    switch (op)
    {
    case B200_F32_ADD: launch_binary_periodic<B200_F32_ADD>(a, v, out, n, period, left, st); break;
    case B200_F32_SUB: launch_binary_periodic<B200_F32_SUB>(a, v, out, n, period, left, st); break;
    case B200_F32_MUL: launch_binary_periodic<B200_F32_MUL>(a, v, out, n, period, left, st); break;
    case B200_F32_DIV: launch_binary_periodic<B200_F32_DIV>(a, v, out, n, period, left, st); break;
    case B200_F32_MAX: launch_binary_periodic<B200_F32_MAX>(a, v, out, n, period, left, st); break;
    default: launch_binary_periodic<B200_F32_MIN>(a, v, out, n, period, left, st); break;
    }
    return after_launch("b200_f32_binary_periodic");
}

extern "C" int b200_f32_unary(int op, const float* x, float* out, int64_t n, void* stream)
{
    using namespace b200;
    if (n < 0 || op < B200_F32_ABS || op > B200_F32_RELU)
        return B200_ERR_INVALID_ARGUMENT;
    if (n == 0)
        return B200_OK;
    if (!x || !out)
        return B200_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned g = grid_for(n, 256);
    switch (op)
    {
    case B200_F32_ABS: unary_kernel<B200_F32_ABS><<<g, 256, 0, st>>>(x, out, n); break;
    case B200_F32_NEG: unary_kernel<B200_F32_NEG><<<g, 256, 0, st>>>(x, out, n); break;
    case B200_F32_SQRT: unary_kernel<B200_F32_SQRT><<<g, 256, 0, st>>>(x, out, n); break;
    case B200_F32_EXP: unary_kernel<B200_F32_EXP><<<g, 256, 0, st>>>(x, out, n); break;
    case B200_F32_ERF: unary_kernel<B200_F32_ERF><<<g, 256, 0, st>>>(x, out, n); break;
    default: unary_kernel<B200_F32_RELU><<<g, 256, 0, st>>>(x, out, n); break;
    }
    return after_launch("b200_f32_unary");
}

namespace b200
{
    static bool valid_shape(const int64_t* shape, int rank)
    {
        if (rank < 0 || rank > MAX_RANK || (rank > 0 && !shape))
            return false;
        for (int i = 0; i < rank; ++i)
            if (shape[i] < 0)
                return false;
        return true;
    }
    static int64_t count_of(const int64_t* shape, int rank)
    {
        int64_t n = 1;
        for (int i = 0; i < rank; ++i)
            n *= shape[i];
        return n;
    }
}

extern "C" int b200_broadcast_b32(const void* in, void* out, const int64_t* out_shape, int rank, const int64_t* broadcast_axes,
                                  int n_axes, void* stream)
{
    using namespace b200;
    if (!valid_shape(out_shape, rank) || n_axes < 0 || n_axes > rank || (n_axes > 0 && !broadcast_axes))
        return B200_ERR_INVALID_ARGUMENT;
    bool is_new[MAX_RANK] = {false};
    for (int i = 0; i < n_axes; ++i)
    {
        if (broadcast_axes[i] < 0 || broadcast_axes[i] >= rank || is_new[broadcast_axes[i]])
            return B200_ERR_INVALID_ARGUMENT;
        is_new[broadcast_axes[i]] = true;
    }
    const int64_t n = count_of(out_shape, rank);
    if (n == 0)
        return B200_OK;
    if (!in || !out)
        return B200_ERR_INVALID_ARGUMENT;
    Dims d;
    d.rank = rank;
    int64_t stride = 1;
    for (int a = rank - 1; a >= 0; --a)
    {
        d.out_dim[a] = out_shape[a];
        d.in_stride[a] = is_new[a] ? 0 : stride;
        if (!is_new[a])
            stride *= out_shape[a];
    }
    launch_remap(in, out, d, n, stride, static_cast<cudaStream_t>(stream)); // stride: the input's element count by now
    return after_launch("b200_broadcast_b32");
}

extern "C" int b200_permute_b32(const void* in, void* out, const int64_t* in_shape, int rank, const int64_t* order, void* stream)
{
    using namespace b200;
    if (!valid_shape(in_shape, rank) || (rank > 0 && !order))
        return B200_ERR_INVALID_ARGUMENT;
    bool seen[MAX_RANK] = {false};
    for (int i = 0; i < rank; ++i)
    {
        if (order[i] < 0 || order[i] >= rank || seen[order[i]])
            return B200_ERR_INVALID_ARGUMENT;
        seen[order[i]] = true;
    }
    const int64_t n = count_of(in_shape, rank);
    if (n == 0)
        return B200_OK;
    if (!in || !out)
        return B200_ERR_INVALID_ARGUMENT;
    int64_t in_stride[MAX_RANK];
    int64_t s = 1;
    for (int a = rank - 1; a >= 0; --a)
    {
        in_stride[a] = s;
        s *= in_shape[a];
    }
    Dims d;
    d.rank = rank;
    for (int a = 0; a < rank; ++a)
    {
        d.out_dim[a] = in_shape[order[a]];
        d.in_stride[a] = in_stride[order[a]];
    }
    launch_remap(in, out, d, n, n, static_cast<cudaStream_t>(stream));
    return after_launch("b200_permute_b32");
}

extern "C" int b200_reduce_f32(int op, const float* in, float* out, const int64_t* shape, int rank, const int64_t* axes, int n_axes,
                               void* stream)
{
    using namespace b200;
    if (op < B200_REDUCE_SUM || op > B200_REDUCE_MAX_ABS || !valid_shape(shape, rank) || n_axes < 0 || n_axes > rank ||
        (n_axes > 0 && !axes))
        return B200_ERR_INVALID_ARGUMENT;
    bool reduced[MAX_RANK] = {false};
    for (int i = 0; i < n_axes; ++i)
    {
        if (axes[i] < 0 || axes[i] >= rank || reduced[axes[i]])
            return B200_ERR_INVALID_ARGUMENT;
        reduced[axes[i]] = true;
    }
    int64_t stride[MAX_RANK];
    int64_t s = 1;
    for (int a = rank - 1; a >= 0; --a)
    {
        stride[a] = s;
        s *= shape[a];
    }
    Dims keep, red;
    keep.rank = red.rank = 0;
    int64_t n_out = 1, n_red = 1;
    for (int a = 0; a < rank; ++a)
    {
        Dims& d = reduced[a] ? red : keep;
        d.out_dim[d.rank] = shape[a];
        d.in_stride[d.rank] = stride[a];
        ++d.rank;
        (reduced[a] ? n_red : n_out) *= shape[a];
    }
    if (n_out == 0)
        return B200_OK;
    if (!out || (!in && n_red > 0))
        return B200_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool any_max = op == B200_REDUCE_MAX || op == B200_REDUCE_MAX_ABS;
    if (any_max && n_out == 1 && n_red >= (int64_t(1) << 16))
    {
        // every axis reduced: the input is one contiguous run
        fill_f32_kernel<<<1, 32, 0, st>>>(out, -INFINITY, 1);
        if (op == B200_REDUCE_MAX_ABS)
            reduce_max_all_kernel<true><<<grid_for(n_red / 4, 256), 256, 0, st>>>(in, out, n_red);
        else
            reduce_max_all_kernel<false><<<grid_for(n_red / 4, 256), 256, 0, st>>>(in, out, n_red);
        g_launches.fetch_add(1, std::memory_order_relaxed);
    }
    else if (op == B200_REDUCE_MAX && n_out <= 4096 && n_red >= 1024)
        reduce_max_block_kernel<<<unsigned(n_out), 256, 0, st>>>(in, out, keep, red, n_red);
    else if (op == B200_REDUCE_SUM && n_axes == 1 && axes[0] == rank - 1 && n_out >= 64)
    {
        // the last axis of a matrix with many rows: panels staged through shared memory
        const int64_t warps = (n_out + 31) / 32, cap = b200::sm_count() * 16;
        sum_rows_kernel<<<unsigned(warps < cap ? warps : cap), 32, 0, st>>>(in, out, n_out, n_red);
    }
    else if (op == B200_REDUCE_SUM)
        reduce_kernel<B200_REDUCE_SUM><<<grid_for(n_out, 128), 128, 0, st>>>(in, out, keep, red, n_out, n_red);
    else if (op == B200_REDUCE_MAX)
        reduce_kernel<B200_REDUCE_MAX><<<grid_for(n_out, 128), 128, 0, st>>>(in, out, keep, red, n_out, n_red);
    else if (op == B200_REDUCE_MAX_ABS)
        reduce_kernel<B200_REDUCE_MAX_ABS><<<grid_for(n_out, 128), 128, 0, st>>>(in, out, keep, red, n_out, n_red);
    else
        reduce_kernel<B200_REDUCE_MIN><<<grid_for(n_out, 128), 128, 0, st>>>(in, out, keep, red, n_out, n_red);
    return after_launch("b200_reduce_f32");
}

extern "C" int b200_softmax_rows_f32(const float* x, float* out, int64_t rows, int64_t row_elements, void* stream)
{
    return b200_softmax_rows_scaled_f32(x, nullptr, out, rows, row_elements, stream);
}

extern "C" int b200_softmax_rows_scaled_f32(const float* x, const float* factor, float* out, int64_t rows, int64_t row_elements,
                                            void* stream)
{
    using namespace b200;
    if (rows < 0 || row_elements < 0)
        return B200_ERR_INVALID_ARGUMENT;
    if (rows * row_elements == 0)
        return B200_OK;
    if (!x || !out)
        return B200_ERR_INVALID_ARGUMENT;
    if (row_elements > 1535)
        return B200_ERR_UNSUPPORTED; // a row too long to stage: the caller composes the five steps instead
    const int L = int(row_elements);
    const bool vec = L % 4 == 0 && all_aligned16({x, out});
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    unsigned grid;
    size_t bytes;
    if (!(vec ? staged_launch_shape(softmax_rows_kernel<true>, rows, L, vec, grid, bytes)
              : staged_launch_shape(softmax_rows_kernel<false>, rows, L, vec, grid, bytes)))
        return B200_ERR_CUDA;
    if (vec)
        softmax_rows_kernel<true><<<grid, 128, bytes, st>>>(x, factor, out, rows, L);
    else
        softmax_rows_kernel<false><<<grid, 128, bytes, st>>>(x, factor, out, rows, L);
    return after_launch("b200_softmax_rows_f32");
}

extern "C" int b200_layer_norm_rows_f32(const float* x, const float* gamma, const float* beta, float* out, int64_t rows,
                                        int64_t row_elements, float epsilon, void* stream)
{
    return b200_layer_norm_rows_sum_f32(x, nullptr, gamma, beta, out, rows, row_elements, epsilon, stream);
}

extern "C" int b200_layer_norm_rows_sum_f32(const float* x, const float* addend, const float* gamma, const float* beta, float* out,
                                            int64_t rows, int64_t row_elements, float epsilon, void* stream)
{
    using namespace b200;
    if (rows < 0 || row_elements < 0)
        return B200_ERR_INVALID_ARGUMENT;
    if (rows * row_elements == 0)
        return B200_OK;
    if (!x || !gamma || !beta || !out)
        return B200_ERR_INVALID_ARGUMENT;
    if (row_elements > 1535)
        return B200_ERR_UNSUPPORTED; // a row too long to stage: the caller runs the decomposition
    const int L = int(row_elements);
    const bool vec = L % 4 == 0 && all_aligned16({x, addend, gamma, beta, out});
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const float count = static_cast<float>(row_elements);
    unsigned grid;
    size_t bytes;
    if (!(vec ? staged_launch_shape(layer_norm_rows_kernel<true>, rows, L, vec, grid, bytes)
              : staged_launch_shape(layer_norm_rows_kernel<false>, rows, L, vec, grid, bytes)))
        return B200_ERR_CUDA;
    if (vec)
        layer_norm_rows_kernel<true><<<grid, 128, bytes, st>>>(x, addend, gamma, beta, out, rows, L, count, epsilon);
    else
        layer_norm_rows_kernel<false><<<grid, 128, bytes, st>>>(x, addend, gamma, beta, out, rows, L, count, epsilon);
    return after_launch("b200_layer_norm_rows_f32");
}

extern "C" int b200_gelu_f32(const float* x, float* out, int64_t n, void* stream)
{
    using namespace b200;
    if (n < 0)
        return B200_ERR_INVALID_ARGUMENT;
    if (n == 0)
        return B200_OK;
    if (!x || !out)
        return B200_ERR_INVALID_ARGUMENT;
    gelu_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(x, out, n);
    return after_launch("b200_gelu_f32");
}

extern "C" int b200_bmm_f32(const float* a, const float* b, float* out, int64_t batch, int64_t M, int64_t K, int64_t N, void* stream)
{
    using namespace b200;
    if (batch < 0 || M < 0 || K < 0 || N < 0 || M > 0x7FFFFFFF || K > 0x7FFFFFFF || N > 0x7FFFFFFF)
        return B200_ERR_INVALID_ARGUMENT;
    if (batch * M * N == 0)
        return B200_OK;
    if (!out || (K > 0 && (!a || !b)))
        return B200_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // large products go through the shared-memory kernel; both kernels give the same bits
    // the wide tile pays off once there are enough K chunks to prefetch behind (measured: K = 64 runs 7 % faster on the narrow one)
    if (M >= 64 && N >= 96 && K >= 256 && launch_bmm_tiled<128, 128, 16>(a, b, out, batch, int(M), int(K), int(N), st))
        return after_launch("b200_bmm_f32");
    if (M >= 64 && N >= 48 && K >= 16 && launch_bmm_tiled<128, 64, 32>(a, b, out, batch, int(M), int(K), int(N), st))
        return after_launch("b200_bmm_f32");
    const int64_t blocks4 = batch * ((M + 3) / 4) * ((N + 3) / 4);
    bmm_f32_kernel<<<grid_for(blocks4, 128), 128, 0, st>>>(a, b, out, batch, int(M), int(K), int(N));
    return after_launch("b200_bmm_f32");
}

extern "C" int b200_gather_rows_b32(const void* table, int64_t n_rows, int64_t row_elements, const void* indices, int index_type,
                                    int64_t n_indices, void* out, void* stream)
{
    using namespace b200;
    if (n_rows < 0 || row_elements < 0 || n_indices < 0 || (index_type != B200_I32 && index_type != B200_I64))
        return B200_ERR_INVALID_ARGUMENT;
    const int64_t total = n_indices * row_elements;
    if (total == 0)
        return B200_OK;
    if (!table || !indices || !out)
        return B200_ERR_INVALID_ARGUMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (index_type == B200_I32)
        gather_rows_kernel<int32_t><<<grid_for(total, 256), 256, 0, st>>>(static_cast<const uint32_t*>(table),
                                                                          static_cast<const int32_t*>(indices),
                                                                          static_cast<uint32_t*>(out), n_indices, row_elements, n_rows);
    else
        gather_rows_kernel<int64_t><<<grid_for(total, 256), 256, 0, st>>>(static_cast<const uint32_t*>(table),
                                                                          static_cast<const int64_t*>(indices),
                                                                          static_cast<uint32_t*>(out), n_indices, row_elements, n_rows);
    return after_launch("b200_gather_rows_b32");
}

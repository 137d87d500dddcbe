// Shared host/device helpers for the B200 kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <atomic>
#include "b200_kernels.h"

namespace b200
{
    // Count of kernels launched through this library (read by b200_launch_count).
    extern std::atomic<uint64_t> g_launches;
    // b200_set_fast_division: 0 makes every Quantize kernel use the plain IEEE division
    extern std::atomic<int> g_fast_division;

    // Records the CUDA error text for b200_last_cuda_error and maps to a status.
    int cuda_status(cudaError_t err, const char* where);

    inline int after_launch(const char* where)
    {
        g_launches.fetch_add(1, std::memory_order_relaxed);
        return cuda_status(cudaGetLastError(), where);
    }

    // Multiprocessors of the current device (grids of the streaming kernels are sized in multiples of it); 148 on a B200,
    // which is also the answer if the query fails.
    inline int sm_count()
    {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        return n;
    }

    inline size_t dtype_size(int t)
    {
        return (t == B200_U8 || t == B200_I8) ? 1 : 4;
    }

    template <typename T>
    struct QLimits;
    template <>
    struct QLimits<uint8_t>
    {
        static constexpr float lo = 0.0f, hi = 255.0f;
    };
    template <>
    struct QLimits<int8_t>
    {
        static constexpr float lo = -128.0f, hi = 127.0f;
    };
    template <>
    struct QLimits<int32_t>
    {
        static constexpr float lo = -2147483648.0f, hi = 2147483648.0f;
    };

    // The rounding step of reference::quantize (runtime/reference/quantize.hpp:51-103),
    // written with explicit round-to-nearest adds so the compiler can neither contract
    // nor reassociate them.
    template <int MODE>
    __device__ __forceinline__ float round_quant(float q)
    {
        if (MODE == B200_ROUND_NEAREST_TOWARD_INFINITY)
        {
            float a = floorf(__fadd_rn(fabsf(q), 0.5f));
            return (q < 0.0f) ? -a : a;
        }
        else if (MODE == B200_ROUND_NEAREST_TOWARD_ZERO)
        {
            float a = ceilf(__fsub_rn(fabsf(q), 0.5f));
            return (q < 0.0f) ? -a : a;
        }
        else if (MODE == B200_ROUND_NEAREST_UPWARD)
        {
            return floorf(__fadd_rn(q, 0.5f));
        }
        else if (MODE == B200_ROUND_NEAREST_DOWNWARD)
        {
            return ceilf(__fsub_rn(q, 0.5f));
        }
        else if (MODE == B200_ROUND_NEAREST_TOWARD_EVEN)
        {
            float up = floorf(__fadd_rn(q, 0.5f));
            float dn = ceilf(__fsub_rn(q, 0.5f));
            // fmod(up, 2.0) == 0  <=>  up/2 is an integer (exact: halving is exact in binary fp)
            float h = __fmul_rn(up, 0.5f);
            return (floorf(h) == h) ? up : dn;
        }
        else if (MODE == B200_ROUND_TOWARD_INFINITY)
        {
            float a = ceilf(fabsf(q));
            return (q < 0.0f) ? -a : a;
        }
        else if (MODE == B200_ROUND_TOWARD_ZERO)
        {
            float a = floorf(fabsf(q));
            return (q < 0.0f) ? -a : a;
        }
        else if (MODE == B200_ROUND_UP)
        {
            return ceilf(q);
        }
        else
        {
            return floorf(q);
        }
    }

    // clamp + cast of reference::quantize (quantize.hpp:109-115).  NaN -> 0.
    template <typename Q>
    __device__ __forceinline__ Q clamp_cast(float q)
    {
        float c = fminf(fmaxf(q, QLimits<Q>::lo), QLimits<Q>::hi);
        int v = __float2int_rz(c); // saturating for the int32 upper edge
        return (q != q) ? Q(0) : static_cast<Q>(v);
    }

    template <typename Q, int MODE>
    __device__ __forceinline__ Q quantize_one(float x, float scale, float zp)
    {
        float q = __fdiv_rn(x, scale);
        q = round_quant<MODE>(q);
        q = __fadd_rn(q, zp);
        return clamp_cast<Q>(q);
    }

    // Fast path of round-to-nearest-even Quantize to 8 bits (see quantize_rows_rne8_kernel): is the scale one for
    // which y = RN(1/s), q0 = RN(x*y), e = fma(-q0,s,x), q = fma(e,y,q0) is the correctly rounded x / s.
    __device__ __forceinline__ bool scale_allows_fast_division(float s)
    {
        const uint32_t b = __float_as_uint(s);
        const uint32_t ex = (b >> 23) & 0xFF, man = b & 0x7FFFFF;
        return ex >= 127 - 40 && ex <= 127 + 40 && man != 0x7FFFFF;
    }

    // The same strength-reduced division for the other rounding modes (8-bit outputs): the quotient has to be the
    // correctly rounded x / s itself, because ceil / floor see its last bit.  q1 is that quotient while nothing
    // underflows, which |x| >= 2^-60 guarantees for the admitted scales (2^-40 <= |s| < 2^41); zeros divide to zero;
    // quotients of magnitude >= 2^24 (and inf / NaN) saturate or become 0 whatever their last bit; the few remaining
    // inputs (0 < |x| < 2^-60) take the IEEE division.
    template <typename Q, int MODE>
    __device__ __forceinline__ Q quantize_one_fast(float x, float s, float y, float zp)
    {
        const float q0 = __fmul_rn(x, y);
        const float e = __fmaf_rn(-q0, s, x);
        const float q1 = __fmaf_rn(e, y, q0);
        const float ax = fabsf(x);
        float q;
        if (!(fabsf(q0) < 16777216.0f) || ax == 0.0f)
            q = q0;
        else if (ax >= 8.673617379884035e-19f) // 2^-60
            q = q1;
        else
            q = __fdiv_rn(x, s);
        q = round_quant<MODE>(q);
        q = __fadd_rn(q, zp);
        return clamp_cast<Q>(q);
    }

    template <typename Q>
    __device__ __forceinline__ int quantize_rne_fast(float x, float s, float y, int lo_minus_zp, int hi_minus_zp, int zp)
    {
        const float q0 = __fmul_rn(x, y);
        const float e = __fmaf_rn(-q0, s, x);
        const float q1 = __fmaf_rn(e, y, q0);
        const float q = (fabsf(q0) < 16777216.0f) ? q1 : q0; // huge, inf and NaN quotients skip the correction
        const int i = __float2int_rn(q);                     // saturating
        const int r = min(max(i, lo_minus_zp), hi_minus_zp) + zp;
        return (x != x) ? 0 : r;                             // NaN -> 0, as clamp_cast
    }

}

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

    // The rounding step of reference::quantize as ONE float -> int32 conversion with a directed rounding mode (plus the
    // literal +-0.5 add of the half-way modes and a sign fix for the modes defined on |q|).  Equal to
    // int(round_quant<MODE>(q)) wherever that integer is representable, saturated beyond, 0 for NaN; the caller clamps
    // to the 8-bit range, so saturation never shows.  (floorf / ceilf followed by a float add of the zero point, two
    // float clamps and a truncating conversion is what this replaces.)
    template <int MODE>
    __device__ __forceinline__ int round_quant_to_int(float q)
    {
        if (MODE == B200_ROUND_NEAREST_TOWARD_INFINITY)
        {
            const int a = __float2int_rd(__fadd_rn(fabsf(q), 0.5f));
            return (q < 0.0f) ? -a : a;
        }
        else if (MODE == B200_ROUND_NEAREST_TOWARD_ZERO)
        {
            const int a = __float2int_ru(__fsub_rn(fabsf(q), 0.5f));
            return (q < 0.0f) ? -a : a;
        }
        else if (MODE == B200_ROUND_NEAREST_UPWARD)
            return __float2int_rd(__fadd_rn(q, 0.5f));
        else if (MODE == B200_ROUND_NEAREST_DOWNWARD)
            return __float2int_ru(__fsub_rn(q, 0.5f));
        else if (MODE == B200_ROUND_NEAREST_TOWARD_EVEN)
            return __float2int_rn(q); // the floor / ceil / parity sequence is round-half-even for |q| < 2^23; beyond, both saturate
        else if (MODE == B200_ROUND_TOWARD_INFINITY)
        {
            const int a = __float2int_ru(fabsf(q));
            return (q < 0.0f) ? -a : a;
        }
        else if (MODE == B200_ROUND_TOWARD_ZERO)
            return __float2int_rz(q); // sign * floor|q|
        else if (MODE == B200_ROUND_UP)
            return __float2int_ru(q);
        else
            return __float2int_rd(q);
    }

    // The strength-reduced division for the modes other than round-half-even (8-bit outputs): the quotient has to be the
    // correctly rounded x / s itself, because the directed conversions see its last bit.  q1 is that quotient while nothing
    // underflows, which |x| >= 2^-60 guarantees for the admitted scales (2^-40 <= |s| < 2^41).  Quotients of magnitude
    // >= 2^24 (and inf / NaN) saturate or become 0 whatever their last bit, so q0 serves.  Smaller inputs take the IEEE
    // division in the directed modes: whether such a quotient is a tiny non-zero number (ceil gives 1) or underflows to
    // zero (ceil gives 0) is decided by the division's own rounding.  The branch is all but never taken.
    // lo_minus_zp / hi_minus_zp / zp as in quantize_rne_fast.
    template <typename Q, int MODE>
    __device__ __forceinline__ int quantize_int_fast(float x, float s, float y, int lo_minus_zp, int hi_minus_zp, int zp)
    {
        const float q0 = __fmul_rn(x, y);
        const float e = __fmaf_rn(-q0, s, x);
        const float q1 = __fmaf_rn(e, y, q0);
        float q = (fabsf(q0) < 16777216.0f) ? q1 : q0;
        constexpr bool nearest = MODE == B200_ROUND_NEAREST_TOWARD_INFINITY || MODE == B200_ROUND_NEAREST_TOWARD_ZERO ||
                                 MODE == B200_ROUND_NEAREST_UPWARD || MODE == B200_ROUND_NEAREST_DOWNWARD ||
                                 MODE == B200_ROUND_NEAREST_TOWARD_EVEN;
        if (!nearest && fabsf(x) < 8.673617379884035e-19f) // 2^-60; the half-way modes send every |q| < 2^-19 to 0 anyway
            q = __fdiv_rn(x, s);
        const int i = round_quant_to_int<MODE>(q);
        const int r = min(max(i, lo_minus_zp), hi_minus_zp) + zp;
        return (x != x) ? 0 : r; // NaN -> 0, as clamp_cast
    }

    // Four elements at once for the directed modes (round toward infinity / zero / up / down), without a test per element on
    // the way.  For the admitted scales (2^-40 <= |s| < 2^41) q1 below is the correctly rounded x / s whenever nothing
    // underflows, and where something does (|x| < 2^-60, hence |x / s| < 2^-20) it still is within one denormal step of it.
    // A directed rounding of a quotient of magnitude below 1 depends only on its sign and on whether it is zero, so q1 can
    // only give a wrong integer when the IEEE quotient is 0 or +-2^-149 and q1 is the other of the two: |q1| <= 2^-149.
    // Those (and every x = 0, harmlessly) are settled exactly: RN(x / s) != 0  <=>  |x| / |s| > 2^-150 (a tie at 2^-150 goes to
    // the even neighbour, 0)  <=>  |x| * 2^126 > |s| * 2^-24, both products exact here (|x| <= 2^-148 * 2^41; |s| * 2^-24 is
    // normal).  `s_low` = |s| * 2^-24.  One test per group of four on the common path.
    template <int MODE>
    __device__ __forceinline__ void quantize4_directed_fast(const float4& x4, float s, float y, float s_low, int lo_minus_zp,
                                                            int hi_minus_zp, int zp, int (&r)[4])
    {
        const float x[4] = {x4.x, x4.y, x4.z, x4.w};
        float q[4];
        bool risky = false;
#pragma unroll
        for (int i = 0; i < 4; ++i)
        {
            const float q0 = __fmul_rn(x[i], y);
            const float e = __fmaf_rn(-q0, s, x[i]);
            const float q1 = __fmaf_rn(e, y, q0);
            q[i] = (fabsf(q0) < 16777216.0f) ? q1 : q0;
            risky = risky || fabsf(q[i]) <= 1.401298464e-45f;
        }
        if (risky)
        {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (fabsf(q[i]) <= 1.401298464e-45f)
                {
                    const bool nonzero = __fmul_rn(fabsf(x[i]), 8.507059173e37f) > s_low; // 2^126
                    const uint32_t sign = (__float_as_uint(x[i]) ^ __float_as_uint(s)) & 0x80000000u;
                    q[i] = __uint_as_float(sign | (nonzero ? 1u : 0u)); // +-2^-149 or +-0
                }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
        {
            const int v = min(max(round_quant_to_int<MODE>(q[i]), lo_minus_zp), hi_minus_zp) + zp;
            r[i] = (x[i] != x[i]) ? 0 : v; // NaN -> 0, as clamp_cast
        }
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

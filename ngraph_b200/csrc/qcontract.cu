// Int8 contractions on the tcgen05 tensor cores: one persistent, warp-specialised kernel
// serves both the matrix product (QuantizedDot / QuantizedDotBias) and the implicit-GEMM
// convolution (QuantizedConvolutionBias and friends).
//
//   D[128 x BN] (int32, in TMEM) += A[128 x BK] * B[BN x BK]^T        per k-block
//
// * A and B tiles arrive by TMA (tiled mode, no multicast) into a ring of shared-memory
//   stages, stored with the 64- or 128-byte swizzle the MMA descriptors name.
// * For the convolution A is never materialised: the activation tensor is channels-last
//   [N,H,W,C]; an output tile is a patch TN x TH x TW of output pixels (128 of them) and the
//   A tile of filter tap (r,s), channel block c0 is the same patch of the INPUT displaced by
//   the tap offset - a single 4-D TMA box.  Out-of-image coordinates are zero-filled by the
//   TMA unit, which is exactly the reference's "padding positions are skipped"
//   (runtime/reference/convolution.hpp:227-251).  A stride s > 1 is handled with s*s tensor
//   maps over the s-strided pixel sub-lattices of the input (no element strides, no gather).
//   The filter [K,R,S,C] is a plain [K, R*S*C] row-major matrix, so B tiles are 2-D boxes.
// * warp 0: TMA producer; warp 1: TMEM allocation + MMA issue (one elected thread);
//   warps 2-9: epilogue (tcgen05.ld -> bias/scale/sum/ReLU/round/saturate -> global).
//   Two TMEM accumulator buffers let the epilogue of tile i overlap the MMAs of tile i+1.
// * Every wait is bounded (ptx::mbar_wait); a timeout sets g_contract_status, the CTA
//   drains and frees its TMEM, and the host reports B200_ERR_DEVICE_STATUS.
#include <cuda.h>
#include <cstdio>
#include <cstring>
#include <mutex>
#include "common.cuh"
#include "ptx.cuh"

namespace b200
{
#ifdef B200_PROFILE_WAITS
    // debug build only: wait cycles per role of CTA 0 ([0] producer/empty, [1] mma/full, [2] mma/tempty,
    // [3] epilogue/tfull, [4] epilogue body, [5] kernel total, [6] tiles of CTA 0)
    __device__ long long g_wait_cycles[8];
#define PROF_T0() long long prof_t0 = clock64()
#define PROF_ADD(i) do { if (blockIdx.x == 0) atomicAdd(reinterpret_cast<unsigned long long*>(&g_wait_cycles[i]), (unsigned long long)(clock64() - prof_t0)); } while (0)
#else
#define PROF_T0() do { } while (0)
#define PROF_ADD(i) do { } while (0)
#endif

    __device__ int g_contract_status = 0; // 0 ok; otherwise 1000*role + detail of the wait that gave up

    struct ContractParams
    {
        int M, N;           // GEMM rows (conv: unused) and output channels
        int num_kblocks;
        int tiles_m, tiles_n;
        // convolution
        int conv;
        int S, cblocks;     // filter width, channel blocks per tap
        int dil_h, dil_w, pad_h, pad_w, stride_h, stride_w;
        int TW, TH, TN;     // output patch covered by one tile (TW*TH*TN == 128)
        int tiles_q, tiles_p; // patches along Q and P (tiles_m = tiles_q*tiles_p*ceil(NB/TN))
        int NB, P, Q;       // batch and output spatial size
        // epilogue
        const int32_t* bias;
        const float* scale;
        int scale_per_channel;
        const void* sum_in;
        int sum_type;
        const float* sum_scale;
        int relu, half_away, out_zp, out_type;
        void* out;
        uint32_t idesc;
    };

    struct TensorMaps
    {
        CUtensorMap a[4]; // GEMM: a[0] (2-D).  Conv: one 4-D map per (h parity, w parity) sub-lattice
        CUtensorMap b;
    };

    constexpr int BM = 128;
    constexpr int NUM_THREADS = 320; // producer warp, MMA warp, 8 epilogue warps

    template <int BN, int BK>
    struct Cfg
    {
        static constexpr int A_BYTES = BM * BK;
        static constexpr int B_BYTES = BN * BK;
        static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
        static constexpr int STAGES = (196608 / STAGE_BYTES) > 8 ? 8 : (196608 / STAGE_BYTES);
        static constexpr int TMEM_COLS = 2 * BN;
        static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
    };

    __device__ __forceinline__ int floor_div(int a, int b)
    {
        int q = a / b;
        return (a % b != 0 && ((a < 0) != (b < 0))) ? q - 1 : q;
    }

    // ---- epilogue arithmetic ----------------------------------------------------------------
    __device__ __forceinline__ float load_sum(const void* p, int type, int64_t i)
    {
        return type == B200_U8 ? static_cast<float>(static_cast<const uint8_t*>(p)[i])
                               : static_cast<float>(static_cast<const int8_t*>(p)[i]);
    }

    struct EpiRow
    {
        bool valid;
        int64_t off; // element offset of column 0 of this row in out / sum_in
    };

    // Core requantisation of one accumulator (reference::dot / convolution, dot.hpp:152-159):
    // (OUT)round(float(acc) * scale) + zero_point, saturated.  Returns the integer as raw 32 bits.
    __device__ __forceinline__ uint32_t epilogue_core(const ContractParams& p, int32_t acc, float scale)
    {
        float r = roundf(__fmul_rn(__int2float_rn(acc), scale));
        long long v = __float2ll_rn(r) + static_cast<long long>(p.out_zp);
        long long lo = p.out_type == B200_U8 ? 0ll : p.out_type == B200_I8 ? -128ll : -2147483648ll;
        long long hi = p.out_type == B200_U8 ? 255ll : p.out_type == B200_I8 ? 127ll : 2147483647ll;
        v = v < lo ? lo : (v > hi ? hi : v);
        return (r != r) ? 0u : static_cast<uint32_t>(static_cast<int32_t>(v));
    }

    template <int BN, int BK>
    __global__ void __launch_bounds__(NUM_THREADS, 1)
        qcontract_kernel(const __grid_constant__ TensorMaps maps, const __grid_constant__ ContractParams p)
    {
        using C = Cfg<BN, BK>;
        extern __shared__ uint8_t smem_raw[];
        __shared__ int abort_flag;
        __shared__ uint32_t tmem_base_slot;
        __shared__ __align__(16) float epi_scale[8][BN / 2];   // per epilogue warp: its column half of the tile
        __shared__ __align__(16) int32_t epi_bias[8][BN / 2];

        const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
        const uint32_t bars = smem_base + C::STAGES * C::STAGE_BYTES;
        auto full_bar = [&](int s) { return bars + 8u * s; };
        auto empty_bar = [&](int s) { return bars + 8u * (C::STAGES + s); };
        auto tfull_bar = [&](int b) { return bars + 8u * (2 * C::STAGES + b); };
        auto tempty_bar = [&](int b) { return bars + 8u * (2 * C::STAGES + 2 + b); };

        const int warp = threadIdx.x >> 5;
        const int lane = threadIdx.x & 31;
        volatile int* abortp = &abort_flag;

        if (threadIdx.x == 0)
        {
            abort_flag = 0;
            for (int s = 0; s < C::STAGES; ++s)
            {
                ptx::mbar_init(full_bar(s), 1);
                ptx::mbar_init(empty_bar(s), 1);
            }
            for (int b = 0; b < 2; ++b)
            {
                ptx::mbar_init(tfull_bar(b), 1);
                ptx::mbar_init(tempty_bar(b), 8);
            }
            ptx::fence_barrier_init();
        }
        if (warp == 1)
        {
            ptx::tmem_alloc(ptx::smem_u32(&tmem_base_slot), C::TMEM_COLS);
            ptx::tmem_relinquish();
        }
        ptx::tc_fence_before_sync();
        __syncthreads();
        ptx::tc_fence_after_sync();
        const uint32_t tmem_base = tmem_base_slot;

        const int num_tiles = p.tiles_m * p.tiles_n;
        int fail = 0;
#ifdef B200_PROFILE_WAITS
        const long long prof_kernel_t0 = clock64();
#endif

        if (warp == 0)
        {
            // ------------------------------------------------------------ TMA producer
            if (ptx::elect_one())
            {
                ptx::prefetch_tmap(&maps.b);
                ptx::prefetch_tmap(&maps.a[0]);
                uint32_t it = 0;
                for (int tile = blockIdx.x; tile < num_tiles && !fail; tile += gridDim.x)
                {
                    const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
                    int q0 = 0, p0 = 0, n0 = 0;
                    if (p.conv)
                    {
                        int t = tm;
                        q0 = (t % p.tiles_q) * p.TW;
                        t /= p.tiles_q;
                        p0 = (t % p.tiles_p) * p.TH;
                        n0 = (t / p.tiles_p) * p.TN;
                    }
                    for (int kb = 0; kb < p.num_kblocks; ++kb, ++it)
                    {
                        const int s = it % C::STAGES;
                        const uint32_t ph = (it / C::STAGES) & 1;
                        PROF_T0();
                        if (!ptx::mbar_wait(empty_bar(s), ph ^ 1, abortp))
                        {
                            fail = 1001;
                            break;
                        }
                        PROF_ADD(0);
                        const uint32_t a_dst = smem_base + s * C::STAGE_BYTES;
                        const uint32_t b_dst = a_dst + C::A_BYTES;
                        ptx::mbar_expect_tx(full_bar(s), C::STAGE_BYTES);
                        if (p.conv)
                        {
                            const int rs = kb / p.cblocks, cb = kb - rs * p.cblocks;
                            const int r = rs / p.S, sx = rs - r * p.S;
                            const int off_h = r * p.dil_h - p.pad_h, off_w = sx * p.dil_w - p.pad_w;
                            const int dh = floor_div(off_h, p.stride_h), dw = floor_div(off_w, p.stride_w);
                            const int par_h = off_h - dh * p.stride_h, par_w = off_w - dw * p.stride_w;
                            ptx::tma_load_4d(a_dst, &maps.a[par_h * p.stride_w + par_w], full_bar(s), cb * BK, q0 + dw,
                                             p0 + dh, n0);
                        }
                        else
                        {
                            ptx::tma_load_2d(a_dst, &maps.a[0], full_bar(s), kb * BK, tm * BM);
                        }
                        ptx::tma_load_2d(b_dst, &maps.b, full_bar(s), kb * BK, tn * BN);
                    }
                }
            }
        }
        else if (warp == 1)
        {
            // ------------------------------------------------------------ MMA issuer
            if (ptx::elect_one())
            {
                uint32_t it = 0, tile_it = 0;
                for (int tile = blockIdx.x; tile < num_tiles && !fail; tile += gridDim.x, ++tile_it)
                {
                    const int acc = tile_it & 1;
                    const uint32_t acc_ph = (tile_it >> 1) & 1;
                    {
                        PROF_T0();
                        if (!ptx::mbar_wait(tempty_bar(acc), acc_ph ^ 1, abortp))
                        {
                            fail = 2001;
                            break;
                        }
                        PROF_ADD(2);
                    }
                    ptx::tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + acc * BN;
                    for (int kb = 0; kb < p.num_kblocks; ++kb, ++it)
                    {
                        const int s = it % C::STAGES;
                        const uint32_t ph = (it / C::STAGES) & 1;
                        {
                            PROF_T0();
                            if (!ptx::mbar_wait(full_bar(s), ph, abortp))
                            {
                                fail = 2002;
                                break;
                            }
                            PROF_ADD(1);
                        }
                        ptx::tc_fence_after_sync();
                        const uint32_t a_src = smem_base + s * C::STAGE_BYTES;
                        const uint32_t b_src = a_src + C::A_BYTES;
                        const uint64_t a_desc = ptx::smem_desc_kmajor(a_src, BK);
                        const uint64_t b_desc = ptx::smem_desc_kmajor(b_src, BK);
#pragma unroll
                        for (int k = 0; k < BK / 32; ++k)
                        {
                            // advance 32 bytes (one K=32 int8 MMA) inside the swizzled row: +2 in 16-byte units
                            ptx::mma_i8(d_tmem, a_desc + uint64_t(2 * k), b_desc + uint64_t(2 * k), p.idesc,
                                        (kb | k) != 0 ? 1u : 0u);
                        }
                        ptx::mma_commit(empty_bar(s)); // frees the stage once these MMAs have read it
                    }
                    if (fail)
                        break;
                    ptx::mma_commit(tfull_bar(acc)); // accumulator complete
                }
            }
        }
        else
        {
            // ------------------------------------------------------------ epilogue (warps 2..9)
            // TMEM lane quarter (warp id % 4) is fixed by the hardware; the two warps that share a
            // quarter split the tile's columns between them.
            const int quarter = warp & 3;
            const int half = (warp - 2) >> 2;
            const int row = quarter * 32 + lane; // accumulator row of this thread
            const bool has_sum = p.sum_in != nullptr;
            const float sum_scale = has_sum ? __ldg(p.sum_scale) : 0.0f;
            const int esz = (p.out_type == B200_U8 || p.out_type == B200_I8) ? 1 : 4;
            const bool vec_ok = ((esz == 1) ? ((p.N & 15) == 0) : ((p.N & 3) == 0)) &&
                                ((reinterpret_cast<uintptr_t>(p.out) | reinterpret_cast<uintptr_t>(p.sum_in)) & 15) == 0;
            uint32_t tile_it = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !fail; tile += gridDim.x, ++tile_it)
            {
                const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
                const int acc = tile_it & 1;
                const uint32_t acc_ph = (tile_it >> 1) & 1;
                // stage this warp's share of the tile's per-channel scale and bias (warp-private buffer,
                // so a warp-level sync is all the ordering it needs)
                __syncwarp();
                for (int j = lane; j < BN / 2; j += 32)
                {
                    const int col = tn * BN + half * (BN / 2) + j;
                    const bool in_n = col < p.N;
                    epi_scale[warp - 2][j] = in_n ? __ldg(p.scale + (p.scale_per_channel ? col : 0)) : 0.0f;
                    epi_bias[warp - 2][j] = (in_n && p.bias) ? __ldg(p.bias + col) : 0;
                }
                __syncwarp();
                EpiRow er;
                if (p.conv)
                {
                    int t = tm;
                    const int q0 = (t % p.tiles_q) * p.TW;
                    t /= p.tiles_q;
                    const int p0 = (t % p.tiles_p) * p.TH;
                    const int n0 = (t / p.tiles_p) * p.TN;
                    const int tw = row % p.TW, th = (row / p.TW) % p.TH, tnn = row / (p.TW * p.TH);
                    const int q = q0 + tw, pp = p0 + th, n = n0 + tnn;
                    er.valid = q < p.Q && pp < p.P && n < p.NB;
                    er.off = ((int64_t(n) * p.P + pp) * p.Q + q) * p.N;
                }
                else
                {
                    const int m = tm * BM + row;
                    er.valid = m < p.M;
                    er.off = int64_t(m) * p.N;
                }
                {
                    PROF_T0();
                    if (!ptx::mbar_wait(tfull_bar(acc), acc_ph, abortp))
                    {
                        fail = 3001;
                        break;
                    }
                    if (warp == 2 && lane == 0)
                        PROF_ADD(3);
                }
                ptx::tc_fence_after_sync();
                PROF_T0();
#pragma unroll 1
                for (int c0 = half * (BN / 2); c0 < (half + 1) * (BN / 2); c0 += 32)
                {
                    uint32_t v[32];
                    __syncwarp();
                    ptx::tmem_ld_32x32(tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN + c0, v);
                    ptx::tmem_ld_wait();
                    const int col0 = tn * BN + c0;
                    if (col0 >= p.N)
                        continue; // warp-uniform
                    const bool full_chunk = col0 + 32 <= p.N;
                    const bool fast = full_chunk && vec_ok;
                    const float* sc = &epi_scale[warp - 2][c0 - half * (BN / 2)];
                    const int32_t* bi = &epi_bias[warp - 2][c0 - half * (BN / 2)];
                    if (p.half_away)
                    {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            v[j] = epilogue_core(p, int32_t(v[j]), sc[j]);
                    }
                    else
                    {
                        // v <- float(acc + bias) * scale  [+ sum_scale * float(sum)]  [relu]
                        float f[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            f[j] = __fmul_rn(__int2float_rn(int32_t(v[j]) + bi[j]), sc[j]);
                        if (has_sum && er.valid)
                        {
                            if (fast)
                            {
                                const uint4* sp = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.sum_in) + er.off + col0);
                                const uint4 s0 = sp[0], s1 = sp[1];
                                const uint32_t sw[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
                                for (int j = 0; j < 32; ++j)
                                {
                                    const uint32_t byte = (sw[j >> 2] >> (8 * (j & 3))) & 0xFF;
                                    const float sv = p.sum_type == B200_U8 ? float(byte) : float(int(int8_t(byte)));
                                    f[j] = __fadd_rn(f[j], __fmul_rn(sum_scale, sv));
                                }
                            }
                            else
                            {
#pragma unroll
                                for (int j = 0; j < 32; ++j)
                                    if (col0 + j < p.N)
                                        f[j] = __fadd_rn(f[j], __fmul_rn(sum_scale, load_sum(p.sum_in, p.sum_type, er.off + col0 + j)));
                            }
                        }
                        if (p.relu)
                        {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                f[j] = (f[j] > 0.0f) ? f[j] : 0.0f; // reference::relu; NaN -> 0 as there
                        }
                        if (p.out_type == B200_F32)
                        {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                v[j] = __float_as_uint(f[j]);
                        }
                        else if (p.out_type == B200_I32)
                        {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                v[j] = uint32_t(clamp_cast<int32_t>(round_quant<B200_ROUND_NEAREST_TOWARD_EVEN>(f[j])));
                        }
                        else
                        {
                            // Quantize(scale 1, zp 0, ROUND_NEAREST_TOWARD_EVEN) to 8 bits: the literal
                            // floor(v+0.5)/ceil(v-0.5)/parity sequence equals round-to-nearest-even for
                            // |v| < 2^23 and everything beyond saturates, so one saturating cvt.rni
                            // (NaN -> 0) followed by the integer clamp gives the same byte.
                            const int lo = p.out_type == B200_U8 ? 0 : -128, hi = p.out_type == B200_U8 ? 255 : 127;
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                v[j] = uint32_t(min(max(__float2int_rn(f[j]), lo), hi));
                        }
                    }
                    if (er.valid && esz == 1)
                    {
                        uint8_t* op = static_cast<uint8_t*>(p.out) + er.off + col0;
                        if (fast)
                        {
                            uint32_t w[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                w[j] = (v[4 * j] & 0xFF) | ((v[4 * j + 1] & 0xFF) << 8) | ((v[4 * j + 2] & 0xFF) << 16) |
                                       ((v[4 * j + 3] & 0xFF) << 24);
                            reinterpret_cast<uint4*>(op)[0] = make_uint4(w[0], w[1], w[2], w[3]);
                            reinterpret_cast<uint4*>(op)[1] = make_uint4(w[4], w[5], w[6], w[7]);
                        }
                        else
                        {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < p.N)
                                    op[j] = uint8_t(v[j]);
                        }
                    }
                    else if (er.valid)
                    {
                        uint32_t* op = static_cast<uint32_t*>(p.out) + er.off + col0;
                        if (fast)
                        {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                reinterpret_cast<uint4*>(op)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                        }
                        else
                        {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < p.N)
                                    op[j] = v[j];
                        }
                    }
                }
                if (warp == 2 && lane == 0)
                {
                    PROF_ADD(4);
#ifdef B200_PROFILE_WAITS
                    if (blockIdx.x == 0)
                        atomicAdd(reinterpret_cast<unsigned long long*>(&g_wait_cycles[6]), 1ull);
#endif
                }
                // all of this warp's TMEM reads are done: hand the accumulator back
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0)
                    ptx::mbar_arrive(tempty_bar(acc));
            }
        }

        // ------------------------------------------------------------ common tail
#ifdef B200_PROFILE_WAITS
        if (blockIdx.x == 0 && threadIdx.x == 0)
            atomicAdd(reinterpret_cast<unsigned long long*>(&g_wait_cycles[5]), (unsigned long long)(clock64() - prof_kernel_t0));
#endif
        if (fail)
            atomicCAS(&g_contract_status, 0, fail);
        __syncwarp();
        ptx::tc_fence_before_sync();
        __syncthreads();
        if (abort_flag)
        {
            // give copies still in flight time to land before shared memory is released
            for (int i = 0; i < 50; ++i)
                __nanosleep(1000);
            __syncthreads();
        }
        if (warp == 1)
        {
            ptx::tc_fence_after_sync();
            ptx::tmem_dealloc(tmem_base, C::TMEM_COLS);
        }
    }

    // ---------------------------------------------------------------------------- host side
    typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

    static EncodeTiledFn encode_fn()
    {
        static EncodeTiledFn fn = nullptr;
        static std::once_flag once;
        std::call_once(once, [] {
            void* f = nullptr;
            cudaDriverEntryPointQueryResult q;
            if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) == cudaSuccess &&
                q == cudaDriverEntryPointSuccess)
                fn = reinterpret_cast<EncodeTiledFn>(f);
        });
        return fn;
    }

    void set_error_text(const char* text);

    // rank-`rank` u8 tensor map; dims/strides innermost first (strides[i] = byte pitch of dim i+1)
    static int make_map(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides,
                        const uint32_t* box, int swizzle_bytes)
    {
        EncodeTiledFn fn = encode_fn();
        if (!fn)
        {
            set_error_text("cuTensorMapEncodeTiled entry point not available");
            return B200_ERR_CUDA;
        }
        cuuint32_t estr[5] = {1, 1, 1, 1, 1};
        CUtensorMapSwizzle sw = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                                : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
        CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS)
        {
            char buf[200];
            snprintf(buf, sizeof(buf),
                     "cuTensorMapEncodeTiled failed (%d): rank %d dims %llu %llu %llu %llu box %u %u %u %u", int(r), rank,
                     (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 0),
                     (unsigned long long)(rank > 2 ? dims[2] : 0), (unsigned long long)(rank > 3 ? dims[3] : 0), box[0],
                     rank > 1 ? box[1] : 0, rank > 2 ? box[2] : 0, rank > 3 ? box[3] : 0);
            set_error_text(buf);
            return B200_ERR_CUDA;
        }
        return B200_OK;
    }

    static int num_sms()
    {
        static int n = 0;
        if (n == 0)
        {
            int dev = 0;
            if (cudaGetDevice(&dev) != cudaSuccess ||
                cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
                n = 148;
        }
        return n;
    }

    template <int BN, int BK>
    static int launch_contract(const TensorMaps& maps, const ContractParams& p, cudaStream_t st)
    {
        using C = Cfg<BN, BK>;
        static bool attr_set[64] = {false};
        int dev = 0;
        cudaGetDevice(&dev);
        dev &= 63;
        if (!attr_set[dev])
        {
            cudaError_t e = cudaFuncSetAttribute(qcontract_kernel<BN, BK>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 C::SMEM_BYTES);
            if (e != cudaSuccess)
                return cuda_status(e, "cudaFuncSetAttribute(qcontract)");
            attr_set[dev] = true;
        }
        int tiles = p.tiles_m * p.tiles_n;
        int grid = tiles < num_sms() ? tiles : num_sms();
        qcontract_kernel<BN, BK><<<grid, NUM_THREADS, C::SMEM_BYTES, st>>>(maps, p);
        return after_launch("qcontract_kernel");
    }

    static int dispatch_contract(int bn, int bk, const TensorMaps& maps, const ContractParams& p, cudaStream_t st)
    {
        if (bk == 128)
        {
            if (bn == 64) return launch_contract<64, 128>(maps, p, st);
            if (bn == 128) return launch_contract<128, 128>(maps, p, st);
            return launch_contract<256, 128>(maps, p, st);
        }
        if (bn == 64) return launch_contract<64, 64>(maps, p, st);
        if (bn == 128) return launch_contract<128, 64>(maps, p, st);
        return launch_contract<256, 64>(maps, p, st);
    }

    static int check_epilogue(const b200_epilogue* e, int64_t n_out)
    {
        if (!e || !e->scale)
            return B200_ERR_INVALID_ARGUMENT;
        if (e->scale_count != 1 && e->scale_count != n_out)
            return B200_ERR_INVALID_ARGUMENT;
        if (e->out_type < B200_U8 || e->out_type > B200_F32)
            return B200_ERR_INVALID_ARGUMENT;
        if (e->sum_in && (!e->sum_scale || (e->sum_type != B200_U8 && e->sum_type != B200_I8)))
            return B200_ERR_INVALID_ARGUMENT;
        if (e->round_half_away && (e->out_type == B200_F32 || e->sum_in || e->bias || e->relu || e->scale_count != 1))
            return B200_ERR_INVALID_ARGUMENT;
        return B200_OK;
    }

    static void fill_epilogue(ContractParams& p, const b200_epilogue* e, void* out, int a_type)
    {
        p.bias = e->bias;
        p.scale = e->scale;
        p.scale_per_channel = e->scale_count > 1;
        p.sum_in = e->sum_in;
        p.sum_type = e->sum_type;
        p.sum_scale = e->sum_scale;
        p.relu = e->relu;
        p.half_away = e->round_half_away;
        p.out_zp = e->out_zero_point;
        p.out_type = e->out_type;
        p.out = out;
        (void)a_type;
    }

    // tcgen05 instruction descriptor, kind::i8: [4,6) D format (2 = s32), [7,10) A format
    // (0 = u8, 1 = s8), [10,13) B format, bits 15/16 A/B major (0 = K-major), [17,23) N>>3, [24,29) M>>4.
    static uint32_t make_idesc(int a_type, int bn)
    {
        uint32_t a_fmt = a_type == B200_I8 ? 1u : 0u;
        return (2u << 4) | (a_fmt << 7) | (1u << 10) | (uint32_t(bn >> 3) << 17) | (uint32_t(BM >> 4) << 24);
    }

    static int pick_bn(int64_t n_out, int64_t tiles_m)
    {
        if (n_out <= 64)
            return 64;
        if (n_out <= 128)
            return 128;
        // wide outputs: 256-wide tiles halve the A re-reads, but keep enough tiles to fill the SMs
        int64_t tiles256 = tiles_m * ((n_out + 255) / 256);
        return (tiles256 >= 2 * num_sms() && n_out % 256 == 0) ? 256 : 128;
    }
}

#ifdef B200_PROFILE_WAITS
extern "C" __attribute__((visibility("default"))) int b200_debug_wait_cycles(long long* out8, int reset)
{
    long long z[8] = {0};
    cudaDeviceSynchronize();
    cudaMemcpyFromSymbol(out8, b200::g_wait_cycles, sizeof(z));
    if (reset)
        cudaMemcpyToSymbol(b200::g_wait_cycles, z, sizeof(z));
    return 0;
}
#endif

extern "C" int b200_device_status(int* status_out)
{
    using namespace b200;
    int v = 0, zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_contract_status, sizeof(int));
    if (e != cudaSuccess)
        return cuda_status(e, "b200_device_status");
    if (v != 0)
        cudaMemcpyToSymbol(g_contract_status, &zero, sizeof(int));
    if (status_out)
        *status_out = v;
    return v == 0 ? B200_OK : B200_ERR_DEVICE_STATUS;
}

extern "C" int b200_qgemm(const void* A, int a_type, const int8_t* W, void* out, int64_t M, int64_t N, int64_t K,
                          const b200_epilogue* epilogue, void* stream)
{
    using namespace b200;
    if (M < 0 || N < 0 || K < 0 || (a_type != B200_U8 && a_type != B200_I8))
        return B200_ERR_INVALID_ARGUMENT;
    int rc = check_epilogue(epilogue, N);
    if (rc != B200_OK)
        return rc;
    if (M == 0 || N == 0)
        return B200_OK;
    if (!A || !W || !out || K == 0)
        return B200_ERR_INVALID_ARGUMENT;
    if (K % 16 != 0 || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
        return B200_ERR_UNSUPPORTED;
    if (M > 0x7FFFFFFF || N > 0x7FFFFFFF || K > 0x7FFFFFFF)
        return B200_ERR_TOO_LARGE;

    const int bk = 128;
    ContractParams p = {};
    p.M = int(M);
    p.N = int(N);
    p.num_kblocks = int((K + bk - 1) / bk);
    p.tiles_m = int((M + BM - 1) / BM);
    const int bn = pick_bn(N, p.tiles_m);
    p.tiles_n = int((N + bn - 1) / bn);
    p.conv = 0;
    fill_epilogue(p, epilogue, out, a_type);
    p.idesc = make_idesc(a_type, bn);

    TensorMaps maps;
    memset(&maps, 0, sizeof(maps));
    uint64_t dims_a[2] = {uint64_t(K), uint64_t(M)}, str[1] = {uint64_t(K)};
    uint32_t box_a[2] = {uint32_t(bk), uint32_t(BM)};
    rc = make_map(&maps.a[0], A, 2, dims_a, str, box_a, bk);
    if (rc != B200_OK)
        return rc;
    uint64_t dims_b[2] = {uint64_t(K), uint64_t(N)};
    uint32_t box_b[2] = {uint32_t(bk), uint32_t(bn)};
    rc = make_map(&maps.b, W, 2, dims_b, str, box_b, bk);
    if (rc != B200_OK)
        return rc;
    return dispatch_contract(bn, bk, maps, p, static_cast<cudaStream_t>(stream));
}

static int64_t conv_out_dim(int64_t in, int64_t lo, int64_t hi, int64_t win, int64_t dil, int64_t stride)
{
    int64_t eff = (win - 1) * dil + 1, padded = in + lo + hi;
    return padded < eff ? 0 : (padded - eff) / stride + 1;
}

extern "C" int b200_qconv_out_shape(const b200_conv_params* c, int64_t* P, int64_t* Q)
{
    if (!c || !P || !Q || c->stride_h <= 0 || c->stride_w <= 0 || c->dilation_h <= 0 || c->dilation_w <= 0 ||
        c->R <= 0 || c->S <= 0)
        return B200_ERR_INVALID_ARGUMENT;
    *P = conv_out_dim(c->H, c->pad_h, c->pad_h_above, c->R, c->dilation_h, c->stride_h);
    *Q = conv_out_dim(c->W, c->pad_w, c->pad_w_above, c->S, c->dilation_w, c->stride_w);
    return B200_OK;
}

// Chooses the output patch TW x TH x TN (product 128, all powers of two) that wastes the fewest
// accumulator rows on positions outside the output.
static void pick_patch(int64_t NB, int64_t P, int64_t Q, int& TW, int& TH, int& TN)
{
    double best = -1.0;
    for (int tw = 1; tw <= 128; tw *= 2)
        for (int th = 1; tw * th <= 128; th *= 2)
        {
            int tn = 128 / (tw * th);
            int64_t tiles = ((Q + tw - 1) / tw) * ((P + th - 1) / th) * ((NB + tn - 1) / tn);
            double eff = double(NB * P * Q) / double(tiles * 128);
            // prefer wider patches on ties (longer contiguous runs for the TMA unit)
            if (eff > best + 1e-9 || (eff > best - 1e-9 && tw * th > TW * TH))
            {
                best = eff;
                TW = tw;
                TH = th;
                TN = tn;
            }
        }
}

extern "C" int b200_qconv(const void* data, int data_type, const int8_t* filters, void* out,
                          const b200_conv_params* c, const b200_epilogue* epilogue, void* stream)
{
    using namespace b200;
    if (!c || (data_type != B200_U8 && data_type != B200_I8))
        return B200_ERR_INVALID_ARGUMENT;
    int64_t P, Q;
    int rc = b200_qconv_out_shape(c, &P, &Q);
    if (rc != B200_OK)
        return rc;
    if (c->N < 0 || c->H <= 0 || c->W <= 0 || c->C <= 0 || c->K <= 0)
        return B200_ERR_INVALID_ARGUMENT;
    rc = check_epilogue(epilogue, c->K);
    if (rc != B200_OK)
        return rc;
    if (c->N == 0 || P == 0 || Q == 0)
        return B200_OK;
    if (!data || !filters || !out)
        return B200_ERR_INVALID_ARGUMENT;
    if (c->C % 64 != 0 || (reinterpret_cast<uintptr_t>(data) & 15) || (reinterpret_cast<uintptr_t>(filters) & 15))
        return B200_ERR_UNSUPPORTED;
    if (c->stride_h * c->stride_w > 4 || c->pad_h < 0 || c->pad_w < 0 || c->H < c->stride_h || c->W < c->stride_w)
        return B200_ERR_UNSUPPORTED;
    if (c->N * P * Q > 0x7FFFFFFF || c->R * c->S * c->C > 0x7FFFFFFF)
        return B200_ERR_TOO_LARGE;

    const int bk = (c->C % 128 == 0) ? 128 : 64;
    ContractParams p = {};
    p.conv = 1;
    p.N = int(c->K);
    p.S = int(c->S);
    p.cblocks = int(c->C / bk);
    p.num_kblocks = int(c->R * c->S * p.cblocks);
    p.dil_h = int(c->dilation_h);
    p.dil_w = int(c->dilation_w);
    p.pad_h = int(c->pad_h);
    p.pad_w = int(c->pad_w);
    p.stride_h = int(c->stride_h);
    p.stride_w = int(c->stride_w);
    p.NB = int(c->N);
    p.P = int(P);
    p.Q = int(Q);
    pick_patch(c->N, P, Q, p.TW, p.TH, p.TN);
    p.tiles_q = int((Q + p.TW - 1) / p.TW);
    p.tiles_p = int((P + p.TH - 1) / p.TH);
    p.tiles_m = p.tiles_q * p.tiles_p * int((c->N + p.TN - 1) / p.TN);
    const int bn = pick_bn(c->K, p.tiles_m);
    p.tiles_n = int((c->K + bn - 1) / bn);
    fill_epilogue(p, epilogue, out, data_type);
    p.idesc = make_idesc(data_type, bn);

    TensorMaps maps;
    memset(&maps, 0, sizeof(maps));
    // one map per pixel sub-lattice (h % stride_h, w % stride_w) of the channels-last input
    for (int ph = 0; ph < p.stride_h; ++ph)
        for (int pw = 0; pw < p.stride_w; ++pw)
        {
            uint64_t dims[4] = {uint64_t(c->C), uint64_t((c->W - pw + p.stride_w - 1) / p.stride_w),
                                uint64_t((c->H - ph + p.stride_h - 1) / p.stride_h), uint64_t(c->N)};
            uint64_t str[3] = {uint64_t(c->C) * p.stride_w, uint64_t(c->C) * c->W * p.stride_h,
                               uint64_t(c->C) * c->W * c->H};
            uint32_t box[4] = {uint32_t(bk), uint32_t(p.TW), uint32_t(p.TH), uint32_t(p.TN)};
            const uint8_t* base = static_cast<const uint8_t*>(data) + (int64_t(ph) * c->W + pw) * c->C;
            rc = make_map(&maps.a[ph * p.stride_w + pw], base, 4, dims, str, box, bk);
            if (rc != B200_OK)
                return rc;
        }
    const uint64_t kg = uint64_t(c->R * c->S * c->C);
    uint64_t dims_b[2] = {kg, uint64_t(c->K)}, str_b[1] = {kg};
    uint32_t box_b[2] = {uint32_t(bk), uint32_t(bn)};
    rc = make_map(&maps.b, filters, 2, dims_b, str_b, box_b, bk);
    if (rc != B200_OK)
        return rc;
    return dispatch_contract(bn, bk, maps, p, static_cast<cudaStream_t>(stream));
}

// Thin inline-PTX wrappers for the sm_100a features the contraction kernels use:
// mbarrier, TMA tiled loads (no multicast), tcgen05 MMA / TMEM.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200
{
    namespace ptx
    {
        __device__ __forceinline__ uint32_t smem_u32(const void* p)
        {
            return static_cast<uint32_t>(__cvta_generic_to_shared(p));
        }

        __device__ __forceinline__ bool elect_one()
        {
            uint32_t pred = 0;
            asm volatile(
                "{\n\t"
                ".reg .pred P;\n\t"
                "elect.sync _|P, 0xffffffff;\n\t"
                "selp.b32 %0, 1, 0, P;\n\t"
                "}"
                : "=r"(pred));
            return pred != 0;
        }

        __device__ __forceinline__ uint64_t globaltimer()
        {
            uint64_t t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            return t;
        }

        // ---- mbarrier ----------------------------------------------------------------
        __device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
        {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
        }
        __device__ __forceinline__ void fence_barrier_init()
        {
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
        {
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
        }
        __device__ __forceinline__ void mbar_arrive(uint32_t bar)
        {
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
        }
        __device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
        {
            uint32_t ok;
            asm volatile(
                "{\n\t"
                ".reg .pred P;\n\t"
                "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
                "selp.b32 %0, 1, 0, P;\n\t"
                "}"
                : "=r"(ok)
                : "r"(bar), "r"(parity)
                : "memory");
            return ok != 0;
        }

        // The same with cluster scope, for a barrier that threads of the peer CTA arrive on (mbar_arrive_remote), as a plain
        // test (no system-chosen nap between polls).
        __device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity)
        {
            uint32_t ok;
            asm volatile(
                "{\n\t"
                ".reg .pred P;\n\t"
                "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 P, [%1], %2;\n\t"
                "selp.b32 %0, 1, 0, P;\n\t"
                "}"
                : "=r"(ok)
                : "r"(bar), "r"(parity)
                : "memory");
            return ok != 0;
        }

        // ---- thread-block clusters (CTA pairs) ----------------------------------------------------
        __device__ __forceinline__ uint32_t cluster_ctarank()
        {
            uint32_t r;
            asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
            return r;
        }
        // every thread of every CTA of the cluster arrives, then waits: a cluster-wide __syncthreads
        __device__ __forceinline__ void cluster_sync()
        {
            asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
            asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        }
        // the address, in the cluster's shared window, of this CTA's shared-memory address `addr` in CTA `rank`
        __device__ __forceinline__ uint32_t mapa(uint32_t addr, uint32_t rank)
        {
            uint32_t r;
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
            return r;
        }
        // arrive on a barrier of another CTA of the cluster (address from mapa)
        __device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr)
        {
            asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
        }

        // Bounded wait: gives up after `limit_ns` (or as soon as another thread of the CTA
        // has given up), records that in *abort_flag and returns false.  Never spins forever.
        // `backoff_ns` > 0 sleeps between polls so that a waiting warp does not take issue slots
        // from the warps that do the arithmetic on the same scheduler.
        template <bool CLUSTER_SCOPE = false>
        __device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  uint32_t backoff_ns = 0, uint64_t limit_ns = 2000000000ull)
        {
            uint32_t spins = 0;
            uint64_t t0 = 0;
            while (!(CLUSTER_SCOPE ? mbar_try_wait_cluster(bar, parity) : mbar_try_wait(bar, parity)))
            {
                if (backoff_ns)
                    __nanosleep(backoff_ns);
                if ((++spins & 0xFF) == 0)
                {
                    if (*abort_flag)
                        return false;
                    uint64_t now = globaltimer();
                    if (t0 == 0)
                        t0 = now;
                    else if (now - t0 > limit_ns)
                    {
                        *abort_flag = 1;
                        return false;
                    }
                }
            }
            return true;
        }

        // ---- TMA tiled loads (global -> shared, completion on an mbarrier) ---------------
        __device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y)
        {
            asm volatile(
                "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
                : "memory");
        }
        __device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                                    int c2, int c3)
        {
            asm volatile(
                "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
                : "memory");
        }
        // Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), completion on an mbarrier.
        __device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
        {
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
                         : "memory");
        }
        __device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map)
        {
            asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
        }

        // ---- tcgen05 / TMEM ----------------------------------------------------------------
        __device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols)
        {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
                         : "memory");
        }
        __device__ __forceinline__ void tmem_relinquish()
        {
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
        __device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
        {
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
        }
        // The same for a CTA pair (cta_group::2): the allocating warp of BOTH CTAs issues each of these, the pair gets the
        // same columns in both tensor memories.
        __device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols)
        {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
                         : "memory");
        }
        __device__ __forceinline__ void tmem_relinquish_pair()
        {
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        }
        __device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols)
        {
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
        }
        __device__ __forceinline__ void tc_fence_before_sync()
        {
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        }
        __device__ __forceinline__ void tc_fence_after_sync()
        {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        // D[tmem] (+)= A[smem] * B[smem]^T, int8 operands, int32 accumulate; issued by ONE thread.
        __device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate)
        {
            asm volatile(
                "{\n\t"
                ".reg .pred p;\n\t"
                "setp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
                "}"
                ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                : "memory");
        }
        // One instruction for a CTA pair: D is 256 rows (128 in each CTA's tensor memory), A comes from both CTAs' shared
        // memory at the descriptor's offset (128 rows each), B likewise (N / 2 rows each).  Issued by ONE thread of the
        // even CTA of the pair.
        __device__ __forceinline__ void mma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                    uint32_t accumulate)
        {
            asm volatile(
                "{\n\t"
                ".reg .pred p;\n\t"
                "setp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t"
                "}"
                ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
                : "memory");
        }
        // Arrive, in BOTH CTAs of the pair, on the barrier at this shared-memory offset once every pair MMA issued so far
        // by this thread has completed (the multicast is of the barrier arrival, not of data).
        __device__ __forceinline__ void mma_commit_pair(uint32_t bar)
        {
            const uint16_t both = 3;
            asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                         ::"r"(bar), "h"(both)
                         : "memory");
        }
        // Arrive on an mbarrier once every MMA issued so far by this thread has completed.
        __device__ __forceinline__ void mma_commit(uint32_t bar)
        {
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                         : "memory");
        }
        // 32 lanes x 32 columns of 32-bit accumulators -> 32 registers per thread (thread = lane/row).
        __device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32])
        {
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                  "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                  "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
                  "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
                  "=r"(r[30]), "=r"(r[31])
                : "r"(taddr)
                : "memory");
        }
        __device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

        // Shared-memory matrix descriptor for a K-major operand tile whose rows are `row_bytes`
        // (64 or 128) long and stored with the matching TMA swizzle; 8-row groups are
        // 8*row_bytes apart (the stride byte offset).  Bits: [0,14) start>>4, [16,30) LBO>>4,
        // [32,46) SBO>>4, [46,48) descriptor version (1 on sm_100), [61,64) swizzle mode.
        // The start may be any whole number of rows (and, for the K steps of one tile, 32-byte pieces) into a tile
        // that the TMA unit wrote: the 16-byte swizzle is a function of the shared-memory address bits alone, so a
        // descriptor that starts r rows into the tile reads rows r, r+1, ... correctly (measured; base-offset field 0).
        __device__ __forceinline__ uint64_t smem_desc_kmajor(uint32_t smem_addr, uint32_t row_bytes)
        {
            const uint64_t layout = row_bytes == 128 ? 2ull : row_bytes == 64 ? 4ull : 6ull;
            uint64_t d = 0;
            d |= uint64_t((smem_addr & 0x3FFFF) >> 4);
            d |= uint64_t(1) << 16;
            d |= uint64_t((8 * row_bytes) >> 4) << 32;
            d |= uint64_t(1) << 46;
            d |= layout << 61;
            return d;
        }

        // Shared-memory matrix descriptor, K-major, no swizzle, for an operand whose rows are overlapping windows of a
        // linear byte run: row r starts at 16*r bytes.  Canonical no-swizzle layout: 8-row groups of 16-byte pieces;
        // leading byte offset (between K pieces) = 16, stride byte offset (between 8-row groups) = 128.
        __device__ __forceinline__ uint64_t smem_desc_overlapping_rows(uint32_t smem_addr)
        {
            uint64_t d = 0;
            d |= uint64_t((smem_addr & 0x3FFFF) >> 4);
            d |= uint64_t(16 >> 4) << 16;
            d |= uint64_t(128 >> 4) << 32;
            d |= uint64_t(1) << 46;
            return d;
        }
    }
}

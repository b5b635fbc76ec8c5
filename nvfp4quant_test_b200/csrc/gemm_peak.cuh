// Tensor-pipe rate probe for the NVFP4 GEMM's instruction: tcgen05.mma.kind::mxf4nvf4.block_scale (M = 128,
// N = 256, K = 64 per instruction, one CTA per SM) issued back to back on operands that stay in shared memory.
// No global-memory traffic inside the timed loop, so the result is what the tensor pipe of this GPU sustains for
// this instruction at the clock it runs at: the denominator the GEMM's "fraction of FP4 peak" is quoted against.
// Results of the MMAs are never read; operands are a fixed pseudo-random byte pattern (E2M1 nibbles of all
// values, scale bytes 0x30..0x3f) so that the data path toggles like real data.
#pragma once

#include "gemm_pair.cuh"

namespace nvfp4 {
namespace gemm {
namespace peak {

constexpr int kPeakThreads = 64;
constexpr int kABytes = 128 * kBKBytes;          // 128 rows x 256 elements
constexpr int kBBytes = 256 * kBKBytes;          // 256 rows x 256 elements
constexpr int kSfBytes = 2048 + 4096;            // scales of A (one 128-row group) and B (two groups), 256 elements of K
constexpr int kSmemBytes = kABytes + kBBytes + kSfBytes + 1024 + 64;
constexpr int kBatch = 16;                       // K stages (4 MMAs each) per commit

// skip_last_commit != 0 (testing hook): the last batch is issued without its tcgen05.commit, so the wait for it can
// only end by running into the wait limit; the kernel then records its status word, lets the queued MMAs finish,
// frees its TMEM and returns like any other launch.
__global__ void __launch_bounds__(kPeakThreads, 1) fp4_peak_kernel(int stages, int skip_last_commit) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - raw_addr);
    uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + kABytes + kBBytes + kSfBytes);
    const uint32_t bar_base = smem_u32(bars);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    const int warp = threadIdx.x >> 5;

    // operands: any byte pattern is a valid E2M1 pair; scale bytes kept in 0x30..0x3f (finite, near 1)
    for (int i = threadIdx.x; i < (kABytes + kBBytes) / 4; i += kPeakThreads) {
        uint32_t h = (static_cast<uint32_t>(i) + 1u) * 2654435761u + blockIdx.x * 40503u;
        h ^= h >> 15;
        h *= 2246822519u;
        h ^= h >> 13;
        reinterpret_cast<uint32_t*>(aligned)[i] = h;
    }
    for (int i = threadIdx.x; i < kSfBytes / 4; i += kPeakThreads) {
        uint32_t h = (static_cast<uint32_t>(i) + 7u) * 2246822519u;
        h ^= h >> 13;
        reinterpret_cast<uint32_t*>(aligned + kABytes + kBBytes)[i] = 0x30303030u | (h & 0x0f0f0f0fu);
    }
    if (threadIdx.x == 0) {
        mbar_init(bar_base, 1);
        mbar_init(bar_base + 8, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes above -> async proxy (MMA, tcgen05.cp)
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(const_cast<uint32_t*>(tmem_slot))),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 1) {
        const bool issuer = elect_one();
        constexpr uint32_t idesc = instr_desc<256>();
        const uint32_t a_lo = ((base & 0x3ffffu) >> 4) | (1u << 16);
        const uint32_t b_lo = a_lo + (kABytes >> 4);
        const uint32_t sfa_lo = ((base + kABytes + kBBytes) & 0x3ffffu) >> 4;
        const uint32_t sfb_lo = sfa_lo + (2048 >> 4);
        const uint32_t sfa_t = tmem_base + 256, sfb_t = tmem_base + 256 + 16;
        if (issuer) {
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                tc_cp_lohi(sfa_t + 4 * kb, sfa_lo + 32 * kb);
                tc_cp_lohi(sfb_t + 8 * kb, sfb_lo + 32 * kb);
                tc_cp_lohi(sfb_t + 8 * kb + 4, sfb_lo + 128 + 32 * kb);
            }
        }
        __syncwarp();
        bool ok = true;
        uint32_t phase0 = 0, phase1 = 0;
        int batch = 0;
        for (int s0 = 0; ok && s0 < stages; s0 += kBatch, ++batch) {
            const int b = batch & 1;
            // the batch committed two rounds ago used this barrier: wait for it, so that at most two batches are queued
            if (batch >= 2) {
                ok = mbar_wait_warp(bar_base + 8u * b, b ? phase1 : phase0, abort_flag, (4u << 24) | (batch & 0xffff));
                if (b) phase1 ^= 1u; else phase0 ^= 1u;
                if (!ok) break;
            }
            if (issuer) {
                const int n = min(kBatch, stages - s0);
                for (int s = 0; s < n; ++s) {
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb)
                        tc_mma_lohi(tmem_base, a_lo + 2 * kb, b_lo + 2 * kb, idesc, sfa_t + 4 * kb, sfb_t + 8 * kb,
                                    (s0 + s + kb) > 0 ? 1u : 0u);
                }
                if (!(skip_last_commit && s0 + kBatch >= stages)) tc_commit(bar_base + 8u * b);
            }
            __syncwarp();
        }
        // drain: every committed batch must have completed before TMEM is released
        for (int k = 0; ok && k < 2 && k < batch; ++k) {
            const int b = (batch - 1 - k) & 1;
            ok = mbar_wait_warp(bar_base + 8u * b, b ? phase1 : phase0, abort_flag, (4u << 24) | 0xfff0u | k);
            if (b) phase1 ^= 1u; else phase0 ^= 1u;
        }
    }
    if (*abort_flag) {   // a wait gave up: let queued MMAs finish before TMEM and shared memory are released
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// The same probe with the instruction the large-shape kernels use: cta_group::2, a CTA pair per 256 x 256 x 64 MMA.
// Each CTA holds its 128 rows of A and 128 of the 256 B rows, so an MMA reads 8 KiB of shared memory per CTA instead
// of 12 KiB, which is what lets the tensor pipe run at its full rate.
constexpr int kPairBBytes = 128 * kBKBytes;
constexpr int kPairSmemBytes = kABytes + kPairBBytes + kSfBytes + 1024 + 64;

__global__ void __launch_bounds__(kPeakThreads, 1) fp4_peak_pair_kernel(int stages) {
    using namespace pair;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* aligned = smem_raw + (base - raw_addr);
    uint64_t* bars = reinterpret_cast<uint64_t*>(aligned + kABytes + kPairBBytes + kSfBytes);
    const uint32_t bar_base = smem_u32(bars);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 2);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    const int warp = threadIdx.x >> 5;
    const uint32_t rank = cluster_ctarank();

    for (int i = threadIdx.x; i < (kABytes + kPairBBytes) / 4; i += kPeakThreads) {
        uint32_t h = (static_cast<uint32_t>(i) + 1u) * 2654435761u + blockIdx.x * 40503u;
        h ^= h >> 15;
        h *= 2246822519u;
        h ^= h >> 13;
        reinterpret_cast<uint32_t*>(aligned)[i] = h;
    }
    for (int i = threadIdx.x; i < kSfBytes / 4; i += kPeakThreads) {
        uint32_t h = (static_cast<uint32_t>(i) + 7u) * 2246822519u;
        h ^= h >> 13;
        reinterpret_cast<uint32_t*>(aligned + kABytes + kPairBBytes)[i] = 0x30303030u | (h & 0x0f0f0f0fu);
    }
    if (threadIdx.x == 0) {
        mbar_init(bar_base, 1);
        mbar_init(bar_base + 8, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(const_cast<uint32_t*>(tmem_slot))),
                     "r"(kTmemCols)
                     : "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // both CTAs' operands, barriers and TMEM exist before the leader issues anything
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 1 && rank == 0) {
        const bool issuer = elect_one();
        constexpr uint32_t idesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(256 >> 3) << 17) |
                                   (static_cast<uint32_t>(256 >> 4) << 24);
        const uint32_t a_lo = ((base & 0x3ffffu) >> 4) | (1u << 16);
        const uint32_t b_lo = a_lo + (kABytes >> 4);
        const uint32_t sfa_lo = ((base + kABytes + kPairBBytes) & 0x3ffffu) >> 4;
        const uint32_t sfb_lo = sfa_lo + (2048 >> 4);
        const uint32_t sfa_t = tmem_base + 256, sfb_t = tmem_base + 256 + 16;
        if (issuer) {
#pragma unroll
            for (int kb = 0; kb < 4; ++kb) {
                tc_cp_pair(sfa_t + 4 * kb, sfa_lo + 32 * kb);
                tc_cp_pair(sfb_t + 8 * kb, sfb_lo + 32 * kb);
                tc_cp_pair(sfb_t + 8 * kb + 4, sfb_lo + 128 + 32 * kb);
            }
        }
        __syncwarp();
        bool ok = true;
        uint32_t phase0 = 0, phase1 = 0;
        int batch = 0;
        for (int s0 = 0; ok && s0 < stages; s0 += kBatch, ++batch) {
            const int b = batch & 1;
            if (batch >= 2) {
                ok = mbar_wait_warp(bar_base + 8u * b, b ? phase1 : phase0, abort_flag, (5u << 24) | (batch & 0xffff));
                if (b) phase1 ^= 1u; else phase0 ^= 1u;
                if (!ok) break;
            }
            if (issuer) {
                const int n = min(kBatch, stages - s0);
                for (int s = 0; s < n; ++s) {
#pragma unroll
                    for (int kb = 0; kb < 4; ++kb)
                        tc_mma_pair(tmem_base, a_lo + 2 * kb, b_lo + 2 * kb, idesc, sfa_t + 4 * kb, sfb_t + 8 * kb,
                                    (s0 + s + kb) > 0 ? 1u : 0u);
                }
                // arrive on the leader's barrier only: the peer waits on nothing, and an arrival it never observes
                // could still be on its way when it leaves
                asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_base + 8u * b)
                             : "memory");
            }
            __syncwarp();
        }
        for (int k = 0; ok && k < 2 && k < batch; ++k) {
            const int b = (batch - 1 - k) & 1;
            ok = mbar_wait_warp(bar_base + 8u * b, b ? phase1 : phase0, abort_flag, (5u << 24) | 0xfff0u | k);
            if (b) phase1 ^= 1u; else phase0 ^= 1u;
        }
    }
    if (*abort_flag) {
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();   // the leader's MMAs read the peer's shared memory and TMEM: nobody leaves before they are done
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
    cluster_sync_all();   // both CTAs stay until both deallocations of the pair have been issued (see gemm_pair_kernel)
}

}  // namespace peak
}  // namespace gemm
}  // namespace nvfp4

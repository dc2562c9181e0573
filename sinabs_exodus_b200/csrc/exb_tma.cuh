// TMA + mbarrier plumbing for the time-major kernels.
//
// A CTA owns a tile of W adjacent neurons of one batch item and walks through
// time.  A producer warp streams [TC time steps x W neurons] chunks of every
// input tensor into a ring of S shared-memory stages with
// cp.async.bulk.tensor (TMA); consumer warps read one float4 per thread and
// step from the stage, keep all neuron state in registers, and write results
// straight to global memory.  The bytes in flight are set by S*TC*W, not by
// the number of resident threads, so small problems and the last partial wave
// of large ones still keep HBM busy.
//
// Every wait on an mbarrier is bounded: after a limit of polls (WAIT_LIMIT unless
// exb_set_wait_limit changed it) the kernel records a code in a device status
// word (read by exb_device_status), stops issuing work, poisons its per-neuron
// results with NaN, waits -- again bounded -- for its own copies in flight, and
// returns normally.  No multicast loads are used anywhere.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace exb {

// Status word: 0 = fine; otherwise the code of the first wait that ran out.  One per
// translation unit that includes this header (static); each such unit exports a reader, and
// exb_device_status looks at all of them.
static __device__ unsigned int g_exb_status = 0;

enum { EXB_STATUS_FULL_WAIT = 1, EXB_STATUS_EMPTY_WAIT = 2, EXB_STATUS_DRAIN_WAIT = 3, EXB_STATUS_LOOKBACK_WAIT = 4,
       EXB_STATUS_PEER_WAIT = 5 };

constexpr uint32_t WAIT_LIMIT = 1u << 22;

// Polls a wait may take before it gives up.  One copy per translation unit, like the status word;
// exb_set_wait_limit writes all of them.  The drain at the end of a kernel always uses WAIT_LIMIT.
static __constant__ unsigned int c_exb_wait_limit = WAIT_LIMIT;

__device__ __forceinline__ uint32_t smem_u32(const void *p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0u;
}

// Bounded wait for the completion of the phase with the given parity.  The limit is read only
// when the first poll fails.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity)
{
    if (mbar_try_wait(bar, parity)) return true;
    const uint32_t limit = c_exb_wait_limit;
    for (uint32_t i = 1; i < limit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// The same with the compile-time limit: for the drain of a kernel that gave up, which must outlast
// its own copies in flight whatever limit the host has set.
__device__ __forceinline__ bool mbar_wait_drain(uint32_t bar, uint32_t parity)
{
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// Host side: set this translation unit's copy of the limit on the current device (0 = default).
static inline cudaError_t set_wait_limit_here(unsigned int polls)
{
    const unsigned int v = polls ? polls : WAIT_LIMIT;
    return cudaMemcpyToSymbol(c_exb_wait_limit, &v, sizeof(v));
}

__device__ __forceinline__ void report_timeout(unsigned int code) { atomicCAS(&g_exb_status, 0u, code); }

// 3-D tiled load (x = neuron, y = time step, z = batch item) into shared memory,
// completion signalled on `bar` as transferred bytes.  x must be a multiple of 4.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, int x, int y, int z, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}

// Orders this thread's shared-memory writes before later accesses of the async (TMA) proxy to the same bytes.
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ float4 lds128(const float *p) { return *reinterpret_cast<const float4 *>(p); }

// Ring of up to MAX_STAGES stages with one "full" (bytes landed) and one "empty" (all
// consumer warps done) barrier per stage.  Lives at the end of the CTA's dynamic shared memory.
constexpr int MAX_STAGES = 8;

struct Ring {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    int issued;     // chunks the producer has issued (written before the final barrier)
    int aborted;    // set by any thread whose wait ran out
    unsigned int ticket;   // work item of this CTA (time-parallel scan kernels)
};

__device__ __forceinline__ void ring_init(Ring *r, int stages, int consumer_warps)
{
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(smem_u32(&r->full[s]), 1);
            mbar_init(smem_u32(&r->empty[s]), consumer_warps);
        }
        r->issued = 0;
        r->aborted = 0;
        mbar_fence_init();
    }
    __syncthreads();
}

// Called by all threads at the end of the kernel.  In the normal case consumers
// have waited for every issued chunk, so nothing is in flight.  After an abort,
// thread 0 waits (bounded) for the newest chunk of every stage so that no copy
// can land in shared memory that has already been handed to another CTA.
__device__ __forceinline__ void ring_finish(Ring *r, int stages)
{
    __syncthreads();
    if (threadIdx.x == 0 && r->aborted) {
        const int issued = r->issued;
        for (int s = 0; s < stages; ++s) {
            int k = issued - 1;
            while (k >= 0 && (k % stages) != s) --k;
            if (k >= 0 && !mbar_wait_drain(smem_u32(&r->full[s]), (uint32_t)((k / stages) & 1)))
                report_timeout(EXB_STATUS_DRAIN_WAIT);
        }
    }
}

}  // namespace exb

// bulk.cuh - bulk-copy (cp.async.bulk) and mbarrier primitives for kernels that stream weights
// HBM -> shared memory. Every wait is bounded: a wait that runs out stores a code through `err`
// (mapped host memory the engine checks after each call) and returns false.
#pragma once

#include "common.cuh"

namespace g5b {

constexpr int ST_WAIT_LIMIT = 1 << 22;       // try_wait attempts before giving up (~ a second)

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false (and an error code in *err) when the barrier never completes.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int *err, int code)
{
    for (int i = 0; i < ST_WAIT_LIMIT; i++)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(err, code);
    return false;
}
// The same wait for a whole warp that has nothing else to do: one lane polls, with a pause
// between polls, so that 32 lanes do not fill the shared-memory pipe with polls that the
// producer warp's copies and shuffles would queue behind. Every lane then observes the
// completed phase itself. The result is uniform over the warp.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t *bar, uint32_t parity, int *err, int code)
{
    bool ok = true;
    if ((threadIdx.x & 31) == 0) {
        ok = false;
        for (int i = 0; i < ST_WAIT_LIMIT; i++) {
            if (mbar_try_wait(bar, parity)) { ok = true; break; }
            __nanosleep(20);
        }
        if (!ok) atomicExch(err, code);
    }
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
        ok = false;
        for (int i = 0; i < 1024 && !ok; i++) ok = mbar_try_wait(bar, parity);
        ok = __all_sync(0xffffffffu, ok);
    }
    return ok;
}
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src, uint32_t bytes, uint64_t *bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst_smem)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

}  // namespace g5b

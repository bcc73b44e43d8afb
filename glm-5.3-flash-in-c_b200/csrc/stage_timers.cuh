// stage_timers.cuh - optional clock stamps inside moe_decode_kernel. A normal build defines none
// of this (every macro is empty); building with -DG5B_STAGE_TIMERS makes each CTA record, relative
// to its own start, the clock64() at which it passed the numbered points of the kernel, plus the
// global nanosecond timer at kernel entry (slot 10) and exit (slot 11), and exports
// g5b_debug_decode_timers() to read the table back. Slots: 0 router rows done, 6 activation split
// done, 7 first stage in shared memory, 8 first routed stage, 9 router scores visible (grid point
// 0), 13 top-k done, 14 picks published, 1 plan made, 2 gate/up done (grid point 1 signalled),
// 3 first down stage, 4 down done, 5 combine done, 15 this rank's step word published (expert
// parallel), 12 every rank's step word seen.
#pragma once

#ifdef G5B_STAGE_TIMERS
__device__ unsigned long long g_decode_timers[160][16];
#define DT_GLOBAL_NS(k)                                                        \
    do {                                                                       \
        if (threadIdx.x == 0 && blockIdx.x < 160) {                            \
            unsigned long long gt_;                                            \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt_));            \
            g_decode_timers[blockIdx.x][k] = gt_;                              \
        }                                                                      \
    } while (0)
#define DT_BEGIN() const long long t_begin = clock64(); DT_GLOBAL_NS(10)
#define DT_MARK(k) do { if (ctid == 0 && blockIdx.x < 160) g_decode_timers[blockIdx.x][k] = clock64() - t_begin; } while (0)
#define DT_MARK_P(k) do { if (lane == 0 && blockIdx.x < 160) g_decode_timers[blockIdx.x][k] = clock64() - t_begin; } while (0)
#define DT_END() do { __syncthreads(); DT_GLOBAL_NS(11); } while (0)
#define DT_EXPORT()                                                                                  \
    extern "C" int g5b_debug_decode_timers(unsigned long long *dst)                                   \
    {                                                                                                \
        return cudaMemcpyFromSymbol(dst, g_decode_timers, sizeof g_decode_timers) == cudaSuccess ? 0 : -1; \
    }
#else
#define DT_BEGIN() do { } while (0)
#define DT_MARK(k) do { } while (0)
#define DT_MARK_P(k) do { } while (0)
#define DT_END() do { } while (0)
#define DT_EXPORT()
#endif

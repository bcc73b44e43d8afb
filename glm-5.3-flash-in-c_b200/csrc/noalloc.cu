// noalloc.cu - RMSNorm on device buffers with no allocation of any kind.
//
// Some hosts of this library cannot allocate device memory while they run: an inference server
// that handed every byte of HBM to weights and KV cache at start-up and runs with a zero
// allocation budget afterwards, a real-time decode loop where a driver allocation would stall
// every stream of the device, or a plugin host that owns the allocator and forbids its guests to
// call cudaMalloc. The engine's RMSNorm needs one float of scratch per row (the normalisation
// factor written by the first kernel and read by the second); here that scratch is a fixed array
// compiled into the library image, so the call touches no allocator: not cudaMalloc/cudaFree,
// not torch, not a memory pool.
//
// The price: the array is part of the module, so every GPU that loads the library holds its 16 KB
// until the process exits; the row count is capped at the array's size; and all calls on a
// device share the one array.
#include <stdio.h>

#include "kernels.h"

namespace g5b {
void set_last_error(const char *msg);   // engine.cu: the message g5b_last_error() returns
}

namespace {

constexpr int NOALLOC_MAX_ROWS = 4096;
constexpr int NOALLOC_MAX_DEVICES = 64;

// One normalisation factor per row. In host code this name is only a handle for the runtime's
// symbol table, not a device address; the address is resolved once per device below.
static __device__ __align__(256) float g_noalloc_rms_factor[NOALLOC_MAX_ROWS];

// Resolved device address, per device ordinal. Filled by the first call on a device and never
// locked: the library's contract is one caller thread at a time, and two first calls that did race
// would both store the same value. It is not refreshed: after cudaDeviceReset the process has to
// reload the library before it calls this entry point again.
float *g_factor_addr[NOALLOC_MAX_DEVICES];

}  // namespace

extern "C" int g5b_rmsnorm_noalloc(float *y_dev, const float *x_dev, const float *w_dev, int n, int rows,
                                   float eps, void *stream)
{
    char msg[192];
    if (!y_dev || !x_dev || n < 1 || rows < 1) {
        g5b::set_last_error("g5b_rmsnorm_noalloc: null buffer or empty shape");
        return -1;
    }
    if (rows > NOALLOC_MAX_ROWS) {
        snprintf(msg, sizeof msg, "g5b_rmsnorm_noalloc: %d rows exceed the built-in scratch of %d rows; "
                                  "split the call or use an entry point that may allocate", rows, NOALLOC_MAX_ROWS);
        g5b::set_last_error(msg);
        return -1;
    }
    int dev = -1;
    cudaError_t rc = cudaGetDevice(&dev);
    if (rc != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) {
        g5b::set_last_error("g5b_rmsnorm_noalloc: no usable current CUDA device");
        return -1;
    }
    if (!g_factor_addr[dev]) {
        // First call on this device: ask the runtime where this device's copy of the array lives.
        float *p = nullptr;
        rc = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_noalloc_rms_factor);
        if (rc != cudaSuccess || !p) {
            snprintf(msg, sizeof msg, "g5b_rmsnorm_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(rc));
            g5b::set_last_error(msg);
            return -1;
        }
        g_factor_addr[dev] = p;
    }
    float *factor = g_factor_addr[dev];
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // Every factor the second kernel reads is written by the first one in this same call, so
    // nothing of the previous call's contents needs clearing.
    g5b::rms_factor(st, x_dev, n, n, rows, eps, factor);
    g5b::rms_apply(st, y_dev, x_dev, w_dev, factor, n, n, rows);
    rc = cudaGetLastError();
    if (rc != cudaSuccess) {
        snprintf(msg, sizeof msg, "g5b_rmsnorm_noalloc: launch failed: %s", cudaGetErrorString(rc));
        g5b::set_last_error(msg);
        return -1;
    }
    return 0;
}

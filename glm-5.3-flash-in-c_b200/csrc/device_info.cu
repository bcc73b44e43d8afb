// device_info.cu - per-device facts and one-time kernel set-up, keyed by device ordinal.
//
// A process may hold engines on several GPUs (g5b_engine_create takes a device). The opt-in to
// more than 48 KB of dynamic shared memory is a per-device attribute of a kernel, and SM counts
// or cooperative-launch support may differ between devices, so nothing here is cached in a
// single static: every answer belongs to the device that is current when it is asked for.
#include <stdio.h>

#include "kernels.h"

namespace g5b {

static int g_sms[G5B_MAX_DEVICES], g_coop[G5B_MAX_DEVICES];

int dev_now()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return 0; }
    return dev < 0 || dev >= G5B_MAX_DEVICES ? 0 : dev;
}

int dev_sms()
{
    const int dev = dev_now();
    if (g_sms[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) { cudaGetLastError(); n = 148; }
        g_sms[dev] = n;
    }
    return g_sms[dev];
}

bool dev_cooperative()
{
    const int dev = dev_now();
    if (g_coop[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess) { cudaGetLastError(); v = 0; }
        g_coop[dev] = v ? 1 : -1;
    }
    return g_coop[dev] == 1;
}

bool dev_opt_in_smem(const void *kernel, size_t bytes, SmemGrant &grant)
{
    if (bytes <= 48 * 1024) return true;
    const int dev = dev_now();
    if (grant.bytes[dev] >= bytes) return true;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes) != cudaSuccess) {
        cudaGetLastError();
        char msg[160];
        snprintf(msg, sizeof msg, "device %d refuses %zu bytes of dynamic shared memory for a kernel", dev, bytes);
        set_last_error(msg);
        return false;
    }
    grant.bytes[dev] = bytes;
    return true;
}

}  // namespace g5b

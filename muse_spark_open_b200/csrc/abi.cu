// Small entry points of the C ABI that need no kernel.
#include <cuda_runtime.h>

#include "msk.h"
#include "status.cuh"

extern "C" int msk_version(void) { return 100; }

extern "C" int msk_device_info(int* sm_count, int* l2_bytes) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return MSK_ERR_CUDA;
    int sms = 0, l2 = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return MSK_ERR_CUDA;
    if (cudaDeviceGetAttribute(&l2, cudaDevAttrL2CacheSize, dev) != cudaSuccess) return MSK_ERR_CUDA;
    if (sm_count != nullptr) *sm_count = sms;
    if (l2_bytes != nullptr) *l2_bytes = l2;
    return 0;
}

// Library-wide host helpers: status strings, last CUDA error, per-device SM count.
#include <stdio.h>
#include <string.h>

#include "ck_common.cuh"

namespace ck {

static thread_local char g_last_error[512] = "";

void set_last_cuda_error(cudaError_t err, const char *where) {
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s (%s)", where, cudaGetErrorName(err), cudaGetErrorString(err));
}

int num_sms() {
    static int cached[64];  // 0 = unknown
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cached[dev] = v;
    }
    return cached[dev];
}

}  // namespace ck

extern "C" const char *ck_status_string(int status) {
    switch (status) {
        case CK_OK: return "CK_OK";
        case CK_ERR_SHAPE: return "CK_ERR_SHAPE";
        case CK_ERR_RANGE: return "CK_ERR_RANGE";
        case CK_ERR_TIMEOUT: return "CK_ERR_TIMEOUT";
        case CK_ERR_CUDA: return "CK_ERR_CUDA";
        case CK_ERR_UNSUPPORTED: return "CK_ERR_UNSUPPORTED";
        case CK_ERR_WORKSPACE: return "CK_ERR_WORKSPACE";
        default: return "CK_ERR_UNKNOWN";
    }
}

extern "C" const char *ck_last_cuda_error(void) { return ck::g_last_error; }

extern "C" int ck_abi_version(void) { return 3; }

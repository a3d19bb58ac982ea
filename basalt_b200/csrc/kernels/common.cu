#include "common.cuh"

#include <cstdio>
#include <cstring>

#include "../../../include/basalt_b200_kernels.h"

namespace basalt_k {

static thread_local char g_msg[256] = "";

int sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

int record(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return 0;
    snprintf(g_msg, sizeof g_msg, "%s: %s", what, cudaGetErrorString(e));
    return (int)e;
}

int record_msg(int code, const char* what, const char* msg) {
    snprintf(g_msg, sizeof g_msg, "%s: %s", what, msg);
    return code;
}

}  // namespace basalt_k

extern "C" const char* basalt_k_last_error(void) { return basalt_k::g_msg; }

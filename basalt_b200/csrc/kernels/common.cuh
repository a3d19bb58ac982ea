// Shared helpers of the hand-written kernels' host launchers.
#pragma once
#include <cuda_runtime.h>

namespace basalt_k {

// SM count of the current device (148 on a B200), cached per device.
int sm_count();
// Stores a failing error code with its text for basalt_k_last_error(); returns the code.
int record(cudaError_t e, const char* what);
int record_msg(int code, const char* what, const char* msg);

// Resident CTAs per SM for `kernel` at the given block size, from the occupancy calculator.
template <class K>
int resident_ctas(K kernel, int threads, size_t dyn_smem = 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, dyn_smem) != cudaSuccess || n < 1) n = 1;
    return n;
}

}  // namespace basalt_k

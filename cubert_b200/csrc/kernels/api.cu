// Library-wide pieces of the C ABI: version and the last CUDA error of a failed launch.
#include "common.cuh"

namespace cubk {

static thread_local cudaError_t g_last_error = cudaSuccess;

void set_last_error(cudaError_t err) {
    g_last_error = err;
}

}  // namespace cubk

extern "C" {

int cubk_version(void) {
    return 100;  // 1.0.0
}

const char *cubk_last_cuda_error(void) {
    return cudaGetErrorString(cubk::g_last_error);
}

}

#include "runtime.h"

#include <cstdlib>
#include <cstring>
#include <sstream>

#include "cubert_kernels.h"

namespace cubert {

void cuda_check(cudaError_t err, const char *what, const char *file, int line) {
    if (err == cudaSuccess) {
        return;
    }
    std::ostringstream os;
    os << "CUDA failure " << (int) err << " (" << cudaGetErrorString(err) << ") in " << what << " at " << file
       << ":" << line;
    throw RuntimeError(os.str());
}

void cublas_check(cublasStatus_t st, const char *what, const char *file, int line) {
    if (st == CUBLAS_STATUS_SUCCESS) {
        return;
    }
    std::ostringstream os;
    os << "cuBLAS failure " << (int) st << " in " << what << " at " << file << ":" << line;
    throw RuntimeError(os.str());
}

void kernel_check(int rc, const char *what, const char *file, int line) {
    if (rc == CUBK_OK) {
        return;
    }
    std::ostringstream os;
    os << "kernel launch layer returned " << rc;
    if (rc == CUBK_ERR_LAUNCH) {
        os << " (" << cubk_last_cuda_error() << ")";
    }
    os << " in " << what << " at " << file << ":" << line;
    throw RuntimeError(os.str());
}

void DeviceBuffer::allocate(size_t bytes) {
    release();
    if (bytes == 0) {
        return;
    }
    cudaError_t err = cudaMalloc(&ptr_, bytes);
    if (err != cudaSuccess) {
        size_t free_b = 0, total_b = 0;
        cudaMemGetInfo(&free_b, &total_b);
        std::ostringstream os;
        os << "CUDA " << cudaGetErrorString(err) << ". Tried to allocate " << bytes << " (" << total_b
           << " total; " << free_b << " free)";
        ptr_ = nullptr;
        throw RuntimeError(os.str());
    }
    bytes_ = bytes;
}

void DeviceBuffer::release() {
    if (ptr_ != nullptr) {
        cudaFree(ptr_);
        ptr_ = nullptr;
        bytes_ = 0;
    }
}

void DeviceBuffer::upload(const void *host, size_t bytes) {
    if (bytes > bytes_) {
        throw RuntimeError("DeviceBuffer::upload: source larger than the allocation");
    }
    if (bytes > 0) {
        CUDA_CHECK(cudaMemcpy(ptr_, host, bytes, cudaMemcpyHostToDevice));
    }
}

void convert(const float *in, float *out, size_t n) {
    std::memcpy(out, in, n * sizeof(float));
}

void convert(const float *in, __half *out, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        out[i] = __float2half_rn(in[i]);
    }
}

void convert(const __half *in, float *out, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        out[i] = __half2float(in[i]);
    }
}

void convert(const __half *in, __half *out, size_t n) {
    std::memcpy(out, in, n * sizeof(__half));
}

int env_int(const char *name, int fallback) {
    const char *v = std::getenv(name);
    if (v == nullptr || *v == '\0') {
        return fallback;
    }
    return std::atoi(v);
}

}  // namespace cubert

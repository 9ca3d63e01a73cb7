// Host-side runtime helpers: error types, CUDA/cuBLAS checking, device buffers.
#pragma once

#include <cublasLt.h>
#include <cublas_v2.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>

namespace cubert {

// Failures of the CUDA runtime, cuBLAS or a kernel launch. The reference prints and exits
// (src/cuBERT/common.cpp:79-93); a library should not end its host process, so this is an
// exception that the C API lets propagate and the status-returning API converts.
struct RuntimeError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

void cuda_check(cudaError_t err, const char *what, const char *file, int line);
void cublas_check(cublasStatus_t st, const char *what, const char *file, int line);
void kernel_check(int rc, const char *what, const char *file, int line);

#define CUDA_CHECK(expr) ::cubert::cuda_check((expr), #expr, __FILE__, __LINE__)
#define CUBLAS_CHECK(expr) ::cubert::cublas_check((expr), #expr, __FILE__, __LINE__)
#define KERNEL_CHECK(expr) ::cubert::kernel_check((expr), #expr, __FILE__, __LINE__)

// Owning device allocation.
class DeviceBuffer {
public:
    DeviceBuffer() = default;
    explicit DeviceBuffer(size_t bytes) { allocate(bytes); }
    ~DeviceBuffer() { release(); }
    DeviceBuffer(const DeviceBuffer &) = delete;
    DeviceBuffer &operator=(const DeviceBuffer &) = delete;
    DeviceBuffer(DeviceBuffer &&o) noexcept : ptr_(o.ptr_), bytes_(o.bytes_) {
        o.ptr_ = nullptr;
        o.bytes_ = 0;
    }
    DeviceBuffer &operator=(DeviceBuffer &&o) noexcept {
        if (this != &o) {
            release();
            ptr_ = o.ptr_;
            bytes_ = o.bytes_;
            o.ptr_ = nullptr;
            o.bytes_ = 0;
        }
        return *this;
    }

    void allocate(size_t bytes);
    void release();
    void upload(const void *host, size_t bytes);  // synchronous host-to-device copy

    template <typename T>
    T *as() const {
        return static_cast<T *>(ptr_);
    }
    void *get() const { return ptr_; }
    size_t bytes() const { return bytes_; }

private:
    void *ptr_ = nullptr;
    size_t bytes_ = 0;
};

// Storage type traits: float or __half.
template <typename T>
struct Storage;

template <>
struct Storage<float> {
    static constexpr cudaDataType_t cuda_type = CUDA_R_32F;
    static constexpr bool is_half = false;
};

template <>
struct Storage<__half> {
    static constexpr cudaDataType_t cuda_type = CUDA_R_16F;
    static constexpr bool is_half = true;
};

// Round-to-nearest-even conversions on the host, bit-identical to the reference's half_float
// based float2half / half2float (src/cuBERT/common.h:94-106, src/half.hpp:374).
void convert(const float *in, float *out, size_t n);
void convert(const float *in, __half *out, size_t n);
void convert(const __half *in, float *out, size_t n);
void convert(const __half *in, __half *out, size_t n);

int env_int(const char *name, int fallback);

}  // namespace cubert

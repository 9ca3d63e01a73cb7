// cuBLAS / cuBLASLt calls of one model replica. The matrix products are library calls and
// not part of the product; this wrapper only fixes conventions:
//   * column-major BLAS semantics exactly as the reference passes them
//     (src/cuBERT/common.cpp:224-419), so the layouts documented there carry over;
//   * float32 accumulation for both storage types; float32 storage computes to float32 accuracy
//     (CUBLAS_COMPUTE_32F, never TF32), as the reference does (CUDA_R_32F compute type): on the
//     float32 pipes or, where cuBLAS offers it, as error-free three-way bfloat16 splits on the
//     tensor cores;
//   * a fixed workspace, so that no call allocates and all of them can be captured in a graph;
//   * the reference's GEMM_ALGO_* environment variables still select a cublasGemmAlgo_t
//     (src/cuBERT/common.cpp:443-469).
#pragma once

#include <map>
#include <tuple>

#include "runtime.h"

namespace cubert {

int gemm_algo_from_env(const char *env, bool half);

class Blas {
public:
    // fp32_emulation_workspace > 0 (float32 models): float32 products may run as nine bfloat16
    // tensor-core products of operands split three ways (cuBLAS 12.9 "BF16x9", results as accurate as
    // float32 arithmetic), which needs that much workspace for the split operands. Off with
    // CUBERT_FP32_EMULATION=0 or an older cuBLAS. CUBERT_BLAS_WORKSPACE_MB overrides the size.
    explicit Blas(cudaStream_t stream, size_t fp32_emulation_workspace = 0, size_t workspace_bytes = 0);
    bool fp32_emulation() const { return fp32_emulation_; }
    ~Blas();
    Blas(const Blas &) = delete;
    Blas &operator=(const Blas &) = delete;

    // C = alpha * op(A) * op(B) + beta * C
    template <typename T>
    void gemm(bool trans_a, bool trans_b, int m, int n, int k, float alpha, const T *A, int lda, const T *B,
              int ldb, float beta, T *C, int ldc, int algo);

    // Pointer-array batched product (device arrays of device pointers).
    template <typename T>
    void gemm_batched(bool trans_a, bool trans_b, int m, int n, int k, float alpha, const T *const *A, int lda,
                      const T *const *B, int ldb, float beta, T *const *C, int ldc, int batch, int algo);

    // C = A * B + bias (bias of length m broadcast over the n columns), through the cuBLASLt
    // bias epilogue. Used where no fused kernel follows the product (the Q/K/V projection).
    template <typename T>
    void gemm_bias(int m, int n, int k, const T *A, int lda, const T *B, int ldb, const T *bias, T *C, int ldc);

private:
    struct LtPlan {
        cublasLtMatmulDesc_t desc = nullptr;
        cublasLtMatrixLayout_t a = nullptr, b = nullptr, c = nullptr;
        cublasLtMatmulAlgo_t algo;
        size_t workspace = 0;
    };
    typedef std::tuple<int, int, int, int, int, int, int> LtKey;  // m, n, k, lda, ldb, ldc, is_half

    cudaStream_t stream_;
    cublasHandle_t handle_ = nullptr;
    cublasLtHandle_t lt_ = nullptr;
    DeviceBuffer workspace_;
    bool fp32_emulation_ = false;
    std::map<LtKey, LtPlan> plans_;
};

}  // namespace cubert

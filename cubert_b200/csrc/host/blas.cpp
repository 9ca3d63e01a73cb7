#include "blas.h"

#include <cstdlib>

namespace cubert {

namespace {
constexpr size_t kWorkspaceBytes = 64u << 20;
}

int gemm_algo_from_env(const char *env, bool half) {
    const char *val = std::getenv(env);
    if (val == nullptr) {
        return half ? (int) CUBLAS_GEMM_DEFAULT_TENSOR_OP : (int) CUBLAS_GEMM_DEFAULT;
    }
    return std::atoi(val);
}

Blas::Blas(cudaStream_t stream, size_t fp32_emulation_workspace, size_t workspace_bytes) : stream_(stream) {
    CUBLAS_CHECK(cublasCreate(&handle_));
    CUBLAS_CHECK(cublasSetStream(handle_, stream_));
    CUBLAS_CHECK(cublasLtCreate(&lt_));
    // float32 storage must not be demoted to TF32
    CUBLAS_CHECK(cublasSetMathMode(handle_, CUBLAS_DEFAULT_MATH));
    size_t bytes = workspace_bytes > 0 ? workspace_bytes : kWorkspaceBytes;
    if (fp32_emulation_workspace > 0 && env_int("CUBERT_FP32_EMULATION", 1) != 0) {
        // A cuBLAS older than 12.9 refuses the mode and the products stay on the float32 pipes.
        fp32_emulation_ = cublasSetMathMode(handle_, CUBLAS_FP32_EMULATED_BF16X9_MATH) == CUBLAS_STATUS_SUCCESS;
        if (fp32_emulation_ && fp32_emulation_workspace > bytes) {
            bytes = fp32_emulation_workspace;
        }
    }
    const int ws_mb = env_int("CUBERT_BLAS_WORKSPACE_MB", 0);
    if (ws_mb > 0) {
        bytes = (size_t) ws_mb << 20;
    }
    workspace_.allocate(bytes);
    CUBLAS_CHECK(cublasSetWorkspace(handle_, workspace_.get(), workspace_.bytes()));
}

Blas::~Blas() {
    for (auto &kv : plans_) {
        LtPlan &p = kv.second;
        if (p.a) cublasLtMatrixLayoutDestroy(p.a);
        if (p.b) cublasLtMatrixLayoutDestroy(p.b);
        if (p.c) cublasLtMatrixLayoutDestroy(p.c);
        if (p.desc) cublasLtMatmulDescDestroy(p.desc);
    }
    if (lt_) cublasLtDestroy(lt_);
    if (handle_) cublasDestroy(handle_);
}

template <typename T>
void Blas::gemm(bool trans_a, bool trans_b, int m, int n, int k, float alpha, const T *A, int lda, const T *B,
                int ldb, float beta, T *C, int ldc, int algo) {
    if (m == 0 || n == 0) {
        return;
    }
    constexpr cudaDataType_t dt = Storage<T>::cuda_type;
    CUBLAS_CHECK(cublasGemmEx(handle_, trans_a ? CUBLAS_OP_T : CUBLAS_OP_N, trans_b ? CUBLAS_OP_T : CUBLAS_OP_N, m,
                              n, k, &alpha, A, dt, lda, B, dt, ldb, &beta, C, dt, ldc, CUBLAS_COMPUTE_32F,
                              (cublasGemmAlgo_t) algo));
}

template <typename T>
void Blas::gemm_batched(bool trans_a, bool trans_b, int m, int n, int k, float alpha, const T *const *A, int lda,
                        const T *const *B, int ldb, float beta, T *const *C, int ldc, int batch, int algo) {
    if (m == 0 || n == 0 || batch == 0) {
        return;
    }
    constexpr cudaDataType_t dt = Storage<T>::cuda_type;
    CUBLAS_CHECK(cublasGemmBatchedEx(handle_, trans_a ? CUBLAS_OP_T : CUBLAS_OP_N,
                                     trans_b ? CUBLAS_OP_T : CUBLAS_OP_N, m, n, k, &alpha,
                                     reinterpret_cast<const void *const *>(A), dt, lda,
                                     reinterpret_cast<const void *const *>(B), dt, ldb, &beta,
                                     reinterpret_cast<void *const *>(C), dt, ldc, batch, CUBLAS_COMPUTE_32F,
                                     (cublasGemmAlgo_t) algo));
}

template <typename T>
void Blas::gemm_bias(int m, int n, int k, const T *A, int lda, const T *B, int ldb, const T *bias, T *C,
                     int ldc) {
    if (m == 0 || n == 0) {
        return;
    }
    constexpr cudaDataType_t dt = Storage<T>::cuda_type;
    const LtKey key(m, n, k, lda, ldb, ldc, Storage<T>::is_half ? 1 : 0);
    auto it = plans_.find(key);
    if (it == plans_.end()) {
        LtPlan p;
        CUBLAS_CHECK(cublasLtMatrixLayoutCreate(&p.a, dt, m, k, lda));
        CUBLAS_CHECK(cublasLtMatrixLayoutCreate(&p.b, dt, k, n, ldb));
        CUBLAS_CHECK(cublasLtMatrixLayoutCreate(&p.c, dt, m, n, ldc));
        cublasLtMatmulHeuristicResult_t result;
        // the emulated float32 compute type first where it was asked for, plain float32 otherwise or after it
        const bool try_emulated = fp32_emulation_ && !Storage<T>::is_half;
        for (int attempt = try_emulated ? 0 : 1; attempt < 2; ++attempt) {
            const cublasComputeType_t compute = attempt == 0 ? CUBLAS_COMPUTE_32F_EMULATED_16BFX9 : CUBLAS_COMPUTE_32F;
            if (cublasLtMatmulDescCreate(&p.desc, compute, CUDA_R_32F) != CUBLAS_STATUS_SUCCESS) {
                p.desc = nullptr;
                continue;
            }
            const cublasOperation_t op_n = CUBLAS_OP_N;
            CUBLAS_CHECK(cublasLtMatmulDescSetAttribute(p.desc, CUBLASLT_MATMUL_DESC_TRANSA, &op_n, sizeof(op_n)));
            CUBLAS_CHECK(cublasLtMatmulDescSetAttribute(p.desc, CUBLASLT_MATMUL_DESC_TRANSB, &op_n, sizeof(op_n)));
            const cublasLtEpilogue_t epilogue = CUBLASLT_EPILOGUE_BIAS;
            CUBLAS_CHECK(
                cublasLtMatmulDescSetAttribute(p.desc, CUBLASLT_MATMUL_DESC_EPILOGUE, &epilogue, sizeof(epilogue)));
            CUBLAS_CHECK(
                cublasLtMatmulDescSetAttribute(p.desc, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &bias, sizeof(bias)));
            cublasLtMatmulPreference_t pref = nullptr;
            CUBLAS_CHECK(cublasLtMatmulPreferenceCreate(&pref));
            const size_t ws = workspace_.bytes();
            CUBLAS_CHECK(cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &ws,
                                                              sizeof(ws)));
            int found = 0;
            cublasStatus_t st =
                cublasLtMatmulAlgoGetHeuristic(lt_, p.desc, p.a, p.b, p.c, p.c, pref, 1, &result, &found);
            cublasLtMatmulPreferenceDestroy(pref);
            if (st == CUBLAS_STATUS_SUCCESS && found > 0) {
                break;
            }
            cublasLtMatmulDescDestroy(p.desc);
            p.desc = nullptr;
        }
        if (p.desc == nullptr) {
            cublasLtMatrixLayoutDestroy(p.a);
            cublasLtMatrixLayoutDestroy(p.b);
            cublasLtMatrixLayoutDestroy(p.c);
            throw RuntimeError("cuBLASLt found no algorithm for the biased projection");
        }
        p.algo = result.algo;
        p.workspace = result.workspaceSize;
        it = plans_.emplace(key, p).first;
    }
    LtPlan &p = it->second;
    CUBLAS_CHECK(cublasLtMatmulDescSetAttribute(p.desc, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &bias, sizeof(bias)));
    const float alpha = 1.f, beta = 0.f;
    CUBLAS_CHECK(cublasLtMatmul(lt_, p.desc, &alpha, A, p.a, B, p.b, &beta, C, p.c, C, p.c, &p.algo,
                                workspace_.get(), workspace_.bytes(), stream_));
}

#define INSTANTIATE(T)                                                                                              \
    template void Blas::gemm<T>(bool, bool, int, int, int, float, const T *, int, const T *, int, float, T *, int,  \
                                int);                                                                               \
    template void Blas::gemm_batched<T>(bool, bool, int, int, int, float, const T *const *, int, const T *const *,  \
                                        int, float, T *const *, int, int, int);                                     \
    template void Blas::gemm_bias<T>(int, int, int, const T *, int, const T *, int, const T *, T *, int);

INSTANTIATE(float)
INSTANTIATE(__half)
#undef INSTANTIATE

}  // namespace cubert

/*
 * Stand-in for Intel's <mkl.h>, used only to compile the reference's CPU path
 * (HAVE_MKL) into oracle/_ref. TEST INFRASTRUCTURE ONLY.
 *
 * The reference's runtime shim uses four MKL entry points
 * (src/cuBERT/common.cpp:164,172,247-257,285-298,336-348):
 *   cblas_sgemm        -> forwarded to the Fortran BLAS symbol sgemm_
 *   cblas_sgemm_batch  -> declared here; resolved at link time (the MKL symbol is
 *                         exported by torch's libtorch_cpu.so), or by the loop in
 *                         mkl_shim_fallback.c when ORACLE_BLAS_FALLBACK is set
 *   mkl_malloc/mkl_free -> posix_memalign / free
 */
#ifndef ORACLE_MKL_SHIM_H
#define ORACLE_MKL_SHIM_H

#include <stdlib.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_LAYOUT;
typedef enum { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;

#ifndef MKL_INT
#define MKL_INT int
#endif

void sgemm_(const char *transa, const char *transb, const int *m, const int *n, const int *k,
            const float *alpha, const float *a, const int *lda, const float *b, const int *ldb,
            const float *beta, float *c, const int *ldc);

void cblas_sgemm_batch(const CBLAS_LAYOUT layout,
                       const CBLAS_TRANSPOSE *transa_array, const CBLAS_TRANSPOSE *transb_array,
                       const MKL_INT *m_array, const MKL_INT *n_array, const MKL_INT *k_array,
                       const float *alpha_array,
                       const float **a_array, const MKL_INT *lda_array,
                       const float **b_array, const MKL_INT *ldb_array,
                       const float *beta_array,
                       float **c_array, const MKL_INT *ldc_array,
                       const MKL_INT group_count, const MKL_INT *group_size);

/* The reference only ever passes CblasColMajor, which is Fortran BLAS order. */
static inline void cblas_sgemm(const CBLAS_LAYOUT layout,
                               const CBLAS_TRANSPOSE transa, const CBLAS_TRANSPOSE transb,
                               const int m, const int n, const int k,
                               const float alpha, const float *a, const int lda,
                               const float *b, const int ldb,
                               const float beta, float *c, const int ldc) {
    const char ta = transa == CblasNoTrans ? 'N' : 'T';
    const char tb = transb == CblasNoTrans ? 'N' : 'T';
    if (layout != CblasColMajor) {
        abort();
    }
    sgemm_(&ta, &tb, &m, &n, &k, &alpha, a, &lda, b, &ldb, &beta, c, &ldc);
}

static inline void *mkl_malloc(size_t size, int alignment) {
    void *p = NULL;
    if (posix_memalign(&p, (size_t) alignment, size ? size : (size_t) alignment) != 0) {
        return NULL;
    }
    return p;
}

static inline void mkl_free(void *p) {
    free(p);
}

#ifdef __cplusplus
}
#endif
#endif

/* Minimal declaration of the one BLAS entry point the reference CPU path calls
 * (cblas_sgemm). Test infrastructure only: used when building the unmodified
 * reference into oracle/_ref against an OpenBLAS that ships inside a Python wheel. */
#ifndef ORACLE_SHIM_CBLAS_H
#define ORACLE_SHIM_CBLAS_H
#ifdef __cplusplus
extern "C" {
#endif
enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 };
#ifdef ORACLE_SCIPY_OPENBLAS
#define cblas_sgemm scipy_cblas_sgemm
#define openblas_set_num_threads scipy_openblas_set_num_threads
#endif
void cblas_sgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE ta, enum CBLAS_TRANSPOSE tb,
                 int M, int N, int K, float alpha, const float* A, int lda,
                 const float* B, int ldb, float beta, float* C, int ldc);
void openblas_set_num_threads(int n);
#ifdef __cplusplus
}
#endif
#endif

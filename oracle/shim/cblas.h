/* Minimal CBLAS declarations (standard CBLAS interface constants and the one routine the
 * reference's BLAS build calls) so that the reference can be compiled against an OpenBLAS shared
 * object that ships without headers. Test infrastructure only. */
#ifndef ORACLE_SHIM_CBLAS_H
#define ORACLE_SHIM_CBLAS_H
#ifdef __cplusplus
extern "C" {
#endif
enum CBLAS_ORDER { CblasRowMajor = 101, CblasColMajor = 102 };
enum CBLAS_TRANSPOSE { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 };
void cblas_sgemm(enum CBLAS_ORDER order, enum CBLAS_TRANSPOSE transa, enum CBLAS_TRANSPOSE transb, int m, int n,
                 int k, float alpha, const float *a, int lda, const float *b, int ldb, float beta, float *c,
                 int ldc);
void openblas_set_num_threads(int n);
int openblas_get_num_threads(void);
#ifdef __cplusplus
}
#endif
#endif

/* Minimal stand-in for the parts of Intel MKL the reference benchmark touches
 * (mlp_omp.cc:9,474,566,657; Rand.cc:7-49; Matrix.h:12), so that the unmodified
 * reference sources compile on a machine without MKL.  Checker infrastructure.
 *
 *  - cblas_sgemm is forwarded to the OpenBLAS build shipped inside the scipy
 *    wheel (symbol scipy_cblas_sgemm, 32-bit integer interface), loaded at run
 *    time; one OpenBLAS thread per call, because the reference already tiles the
 *    GEMM over its own OpenMP threads.
 *  - the VSL uniform generator is replaced by the portable counter-based stream
 *    of b2_rng.h consumed sequentially (MKL's Niederreiter sequence is not
 *    reproducible without MKL); b2shim_rng_reset() rewinds it.
 */
#ifndef B2_SHIM_MKL_H
#define B2_SHIM_MKL_H

#include <algorithm>
#include <array>
#include <cstddef>
#include <string>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_LAYOUT;
typedef enum { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;

void cblas_sgemm(CBLAS_LAYOUT layout, CBLAS_TRANSPOSE transa, CBLAS_TRANSPOSE transb, int m,
                 int n, int k, float alpha, const float* a, int lda, const float* b, int ldb,
                 float beta, float* c, int ldc);
double dsecnd(void);
void mkl_set_num_threads(int n);

typedef void* VSLStreamStatePtr;
#define VSL_BRNG_NIEDERR 0
#define VSL_RNG_METHOD_UNIFORM_STD 0
int vslNewStream(VSLStreamStatePtr* stream, int brng, unsigned seed);
int vsRngUniform(int method, VSLStreamStatePtr stream, int n, float* r, float a, float b);
int vdRngUniform(int method, VSLStreamStatePtr stream, int n, double* r, double a, double b);

/* Not MKL: rewind the sequential stream used by v?RngUniform. */
void b2shim_rng_reset(void);
/* Not MKL: name of the BLAS actually bound ("openblas:<path>" or "loops"). */
const char* b2shim_blas_name(void);

#ifdef __cplusplus
}
#endif
#endif

/* CPU oracle for the MLP training step of jspark1105/tbb_test (mlp_omp.cc /
 * mlp_tbb.cc).  TEST INFRASTRUCTURE ONLY: this is the checker the CUDA path is
 * compared against; it is never linked into, called from, or shipped with the
 * product library.
 *
 * It restates, in plain C, the reference's call sequence
 *   forward   A[l+1] = A[l] * W[l]^T                 (mlp_omp.cc:441-510)
 *   wgrad     dW[l]  = dZ[l]^T * A[l]  per socket    (mlp_omp.cc:527-600)
 *   dgrad     dA[l]  = dZ[l] * W[l]                  (mlp_omp.cc:624-691)
 *   update    W[l]  -= alpha * sum_sockets dW[l]     (mlp_omp.cc:56-323)
 * with two modes:
 *   ORC_MODE_REF       exactly the C++ reference: no ReLU, dZ[L-1] = A[L]
 *                      (mlp_omp.cc:565,655), no 1/B scaling.
 *   ORC_MODE_BASELINE  ReLU between layers, dZ[L-1] = (A[L] - T) / B_global,
 *                      semantics of c2_bench/mlp_caffe2.py:208-235,257-267.
 *
 * Parity pinning: ref mode is checked against the unmodified reference binary
 * built under oracle/_ref (final weights, activations and gradients after the
 * reference's own 272 iterations) and against the reference's allreduce+SGD
 * known-answer test (mlp_omp.cc:325-373); see tests/golden/.
 */
#ifndef MLP_ORACLE_H
#define MLP_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { ORC_MODE_REF = 0, ORC_MODE_BASELINE = 1 };
/* Operand rounding applied where the device path stores reduced precision. */
enum { ORC_ROUND_NONE = 0, ORC_ROUND_TF32 = 1, ORC_ROUND_BF16 = 2 };

typedef struct {
  int nlayers;
  const int* nfeatures; /* nlayers + 1 entries: F_0 .. F_L */
  int batch;            /* global batch */
  int nranks;           /* sockets / GPUs the batch is split over */
  int mode;             /* ORC_MODE_* */
  int rounding;         /* ORC_ROUND_* */
  int grad_bf16;        /* round each rank's dW to bf16 before the sum */
  float lr;
} orc_config;

typedef struct orc_mlp orc_mlp;

/* cblas_sgemm-compatible signature (row-major only is ever passed). */
typedef void (*orc_sgemm_fn)(int order, int transa, int transb, int m, int n, int k,
                             float alpha, const float* a, int lda, const float* b,
                             int ldb, float beta, float* c, int ldc);
/* Route the oracle's GEMMs through an external BLAS (NULL = built-in loops). */
void orc_set_sgemm(orc_sgemm_fn fn);

/* s > 1: every GEMM is summed as s partial products over consecutive ranges of the
 * contraction index (same mathematics, another fp32 addition order); 1 = off. */
void orc_set_ksplit(int s);

/* Row-major C = alpha*op(A)*op(B) + beta*C with cblas argument meaning. */
void orc_sgemm(int transa, int transb, int m, int n, int k, float alpha,
               const float* a, int lda, const float* b, int ldb, float beta,
               float* c, int ldc);

orc_mlp* orc_create(const orc_config* cfg);
void orc_destroy(orc_mlp* o);

void orc_set_weights(orc_mlp* o, int l, const float* w, size_t ld);
void orc_get_weights(const orc_mlp* o, int l, float* w, size_t ld);
void orc_set_input(orc_mlp* o, const float* x, size_t ld);
void orc_set_target(orc_mlp* o, const float* t, size_t ld);

/* n training steps. After the call the taps below hold the last step's values. */
void orc_step(orc_mlp* o, int n);

/* Forward activation A[l], l in [0, L] (post-ReLU in baseline mode). */
void orc_get_activation(const orc_mlp* o, int l, float* a, size_t ld);
/* Gradient w.r.t. the output of layer l (dZ[l]), l in [0, L-1]. */
void orc_get_dz(const orc_mlp* o, int l, float* g, size_t ld);
/* Gradient w.r.t. the network input (dA[0]; the reference's spare buffer,
 * mlp_omp.cc:656). */
void orc_get_input_grad(const orc_mlp* o, float* g, size_t ld);
/* Sum over ranks of dW[l]. */
void orc_get_weight_grad(const orc_mlp* o, int l, float* g, size_t ld);
/* 0.5 * sum((Y - T)^2) / B_global (baseline) or 0.5 * sum(Y^2) (ref). */
double orc_loss(const orc_mlp* o);

/* Batch rows [begin,end) of `rank`: Partition.cc:34-51 with one thread/socket. */
void orc_batch_range(int batch, int nranks, int rank, int* begin, int* end);

/* The reference's allreduce + SGD known-answer data (mlp_omp.cc:336-337,
 * 356-360): grad(s*R+i, j) = s+i+j, w = i*j, alpha = 1. `expected` receives
 * i*j - ((i+j)*N + N(N-1)/2). */
void orc_kat_fill(int nsockets, int nrows, int ncols, int sid, float* w, float* g, size_t ld);
void orc_kat_expected(int nsockets, int nrows, int ncols, float* expected, size_t ld);

/* Ring reduce-scatter + SGD + allgather over `nsockets` stacked replicas,
 * following the chunk schedule of mlp_omp.cc:80-146,227-271 with one thread
 * per socket (ring order = socket order for nsockets < 8, the table of
 * mlp_bench_common.cc:13 for 8). w, g, push: (nsockets*nrows) x ld floats. */
void orc_ring_update(int nsockets, int nrows, int ncols, size_t ld, float* w,
                     float* g, float* push, float alpha);

/* print_checksum (mlp_bench_common.cc:152-168): l1, l2, trace in double. */
void orc_checksum(const float* w, int nrows, int ncols, size_t ld, double out[3]);

/* Seeded synthetic data from the counter-based generator of include/b2_rng.h;
 * element (i,j) uses counter start + i*ncols + j. */
void orc_fill_uniform(float* a, int nrows, int ncols, size_t ld, uint64_t seed, uint64_t start,
                      float lo, float hi);
void orc_fill_normal(float* a, int nrows, int ncols, size_t ld, uint64_t seed, uint64_t start,
                     float stddev);
void orc_fill_sign(float* a, int nrows, int ncols, size_t ld, uint64_t seed, uint64_t start);

/* Rounding helpers (round-to-nearest-even bf16; tf32 = 13 low mantissa bits cleared). */
float orc_round_bf16(float x);
float orc_round_tf32(float x);

#ifdef __cplusplus
}
#endif
#endif

// Harness linked with the UNMODIFIED reference sources (compiled where they lie,
// with main renamed to mlp_omp_main) into oracle/_ref/libref_mlp_omp.so.  It
// exposes the reference's own functions and global state through a C ABI so that
// golden vectors can be generated from, and the CPU oracle pinned against, the
// reference itself.  Checker infrastructure only.
#include <omp.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "mkl.h"
#include "Matrix.h"
#include "Partition.h"
#include "TwistedHyperCube.h"
#include "mlp_bench_common.h"

int mlp_omp_main(int argc, char** argv);

// defined in mlp_omp.cc:297
void update_weight(Matrix<float, PAD>* weight, Matrix<float, PAD>* weight_grad,
                   Matrix<float, PAD>* weight_grad_push_buf, double alpha, int layer,
                   bool measure_time, int nthreads_per_socket, int tid_in_socket);

// mlp_omp.cc:50,53: handshake flags and the per-thread phase counter of the ring
// steps. Threads of the OpenMP pool keep their phase between calls, and the
// handshake only works while every participating thread is at the same phase
// (always true inside the reference's own main, where all threads run the same
// number of steps), so both are cleared before each direct call.
extern volatile int done_flags[];
extern thread_local int done_flag_phase;

extern "C" {

int ref_nlayers() { return nlayers; }
int ref_nfeatures(int i) { return nfeatures[i]; }
int ref_pad() { return PAD; }
int ref_nsockets() { return nsockets; }
const char* ref_blas_name() { return b2shim_blas_name(); }

// Runs the reference benchmark end to end (allocation, self-check, init, 16+256
// steps, report). The global matrices stay allocated afterwards.
int ref_run_main(int nsock, int nthr_per_socket) {
  char a0[] = "mlp_omp", a1[16], a2[16];
  snprintf(a1, sizeof a1, "%d", nsock);
  snprintf(a2, sizeof a2, "%d", nthr_per_socket);
  char* argv[] = {a0, a1, a2, nullptr};
  b2shim_rng_reset();
  return mlp_omp_main(3, argv);
}

// Re-creates the initial inputs and weights in the global matrices (same stream
// position as at the start of ref_run_main).
void ref_reinit() {
  b2shim_rng_reset();
  init_matrices();
}

static void copy_out(Matrix<float, PAD>* m, int row0, int rows, float* out, size_t ld) {
  for (int i = 0; i < rows; ++i)
    memcpy(out + (size_t)i * ld, m->rawData(row0 + i, 0), sizeof(float) * m->ncols());
}
int ref_batch() { return activations[0]->nrows(); }
void ref_get_weights(int l, int replica, float* out, size_t ld) {
  copy_out(weights[l].get(), replica * nfeatures[l + 1], nfeatures[l + 1], out, ld);
}
void ref_get_weight_grad(int l, int replica, float* out, size_t ld) {
  copy_out(weight_grads[l].get(), replica * nfeatures[l + 1], nfeatures[l + 1], out, ld);
}
void ref_get_activation(int l, float* out, size_t ld) {
  copy_out(activations[l].get(), 0, activations[l]->nrows(), out, ld);
}
void ref_checksum() { print_checksum(); }

// The reference's ring reduce-scatter + SGD + allgather on caller data:
// w, g are (nsock*nrows) x ncols dense; runs update_weight with alpha on
// nsock*nthr OpenMP threads and writes the updated stacked weights back.
void ref_update_weight(int nsock, int nthr, int nrows, int ncols, float* w, const float* g,
                       double alpha) {
  nsockets = nsock;
  nthreads_per_socket = nthr;
  nthreads = nsock * nthr;
  omp_set_num_threads(nthreads);
  Matrix<float, PAD> W(nsock * nrows, ncols), G(nsock * nrows, ncols), P(nsock * nrows, ncols);
  // the padded buffer takes part in the reduction (mlp_omp.cc:73-74): clear it
  memset(W.rawData(), 0, sizeof(float) * (size_t)(nsock * nrows + PAD) * (ncols + PAD));
  memset(G.rawData(), 0, sizeof(float) * (size_t)(nsock * nrows + PAD) * (ncols + PAD));
  memset(P.rawData(), 0, sizeof(float) * (size_t)(nsock * nrows + PAD) * (ncols + PAD));
  for (int i = 0; i < nsock * nrows; ++i) {
    memcpy(W.rawData(i, 0), w + (size_t)i * ncols, sizeof(float) * ncols);
    memcpy(G.rawData(i, 0), g + (size_t)i * ncols, sizeof(float) * ncols);
  }
  for (int i = 0; i < nthreads * 16; ++i) done_flags[i] = 0;
#pragma omp parallel
  done_flag_phase = 0;
#pragma omp parallel
  update_weight(&W, &G, &P, alpha, 0, false, get_num_threads_per_socket(),
                get_thread_num_in_socket());
  for (int i = 0; i < nsock * nrows; ++i)
    memcpy(w + (size_t)i * ncols, W.rawData(i, 0), sizeof(float) * ncols);
}

// Seconds per call of the reference's update_weight (ring reduce-scatter + SGD +
// allgather, mlp_omp.cc:297-323) on (nsock*nrows) x ncols buffers that stay allocated
// across `iters` timed calls after one warm-up call: the CPU side of the allreduce sweep.
double ref_time_update_weight(int nsock, int nthr, int nrows, int ncols, int iters) {
  nsockets = nsock;
  nthreads_per_socket = nthr;
  nthreads = nsock * nthr;
  omp_set_num_threads(nthreads);
  Matrix<float, PAD> W(nsock * nrows, ncols), G(nsock * nrows, ncols), P(nsock * nrows, ncols);
  const size_t n = (size_t)(nsock * nrows + PAD) * (ncols + PAD);
#pragma omp parallel for
  for (size_t i = 0; i < n; ++i) {
    W.rawData()[i] = 0.f;
    G.rawData()[i] = 1e-3f;
    P.rawData()[i] = 0.f;
  }
  double t0 = 0;
  for (int it = -1; it < iters; ++it) {
    if (it == 0) t0 = dsecnd();
    for (int i = 0; i < nthreads * 16; ++i) done_flags[i] = 0;
#pragma omp parallel
    {
      done_flag_phase = 0;
      update_weight(&W, &G, &P, 1e-10, 0, false, get_num_threads_per_socket(), get_thread_num_in_socket());
    }
  }
  return (dsecnd() - t0) / iters;
}

// Partition.cc:34-51
void ref_get_partition(int nsock, int work, int socket_id, int nthr, int tid, int* out2) {
  nsockets = nsock;
  auto p = get_partition(work, socket_id, nthr, tid);
  out2[0] = p.first;
  out2[1] = p.second;
}
// Partition.cc:75-166
void ref_intra_socket_2d(int m, int n, double ar, int m_align, int nthr, int tid, int* out4) {
  get_intra_socket_2dpartition(&out4[0], &out4[1], &out4[2], &out4[3], m, n, ar, m_align != 0,
                               nthr, tid);
}
// Partition.cc:193-222
void ref_2dpartition(int nsock, int m, int n, double ar, int m_align, int socket_id, int nthr,
                     int tid, int* out4) {
  nsockets = nsock;
  get_2dpartition(&out4[0], &out4[1], &out4[2], &out4[3], m, n, ar, m_align != 0, socket_id, nthr,
                  tid);
}
int ref_work_per_socket(int nsock, int work) {
  nsockets = nsock;
  return get_work_per_socket(work);
}
// TwistedHyperCube.cc: peer / recv / send
void ref_hypercube(int twisted, int num_nodes, int shift, int id, int dim, int* out3) {
  if (twisted) {
    TwistedHyperCube c(num_nodes, shift);
    out3[0] = c.Peer(id, dim);
    out3[1] = c.RecvLocation(id, dim);
    out3[2] = c.SendLocation(id, dim);
  } else {
    HyperCube c(num_nodes, shift);
    out3[0] = c.Peer(id, dim);
    out3[1] = c.RecvLocation(id, dim);
    out3[2] = c.SendLocation(id, dim);
  }
}
int ref_hypercube_dim(int num_nodes) { return HyperCube(num_nodes).Dimension(); }
// mlp_bench_common.cc:170-190
void ref_ring_info(int nsock, int sid, int task, int* out3) {
  nsockets = nsock;
  get_my_ring_info(sid, task, &out3[0], &out3[1], &out3[2]);
}
}

// C exports of the host-side mirror (Partition, TwistedHyperCube, ring tables,
// Matrix layout, seeded fills) so that the test-suite can compare them, through
// ctypes, with golden vectors produced by the reference's own functions.
#include <chrono>
#include <cstring>
#include <vector>

#include "../csrc/bucket_plan.h"
#include "HyperCubeAllReduce.h"
#include "b2_rng.h"
#include "TwistedHyperCube.h"
#include "mlp_bench_common.h"

extern "C" {

void b2h_get_partition(int nsock, int work, int socket_id, int nthr, int tid, int* out2) {
  nsockets = nsock;
  auto p = get_partition(work, socket_id, nthr, tid);
  out2[0] = p.first;
  out2[1] = p.second;
}

int b2h_work_per_socket(int nsock, int work) {
  nsockets = nsock;
  return get_work_per_socket(work);
}

void b2h_intra_socket_2d(int m, int n, double ar, int m_align, int nthr, int tid, int* out4) {
  get_intra_socket_2dpartition(&out4[0], &out4[1], &out4[2], &out4[3], m, n, ar, m_align != 0, nthr, tid);
}

void b2h_2dpartition(int nsock, int m, int n, double ar, int m_align, int socket_id, int nthr, int tid, int* out4) {
  nsockets = nsock;
  get_2dpartition(&out4[0], &out4[1], &out4[2], &out4[3], m, n, ar, m_align != 0, socket_id, nthr, tid);
}

void b2h_hypercube(int twisted, int num_nodes, int shift, int id, int dim, int* out3) {
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

// Allreduce of `num_nodes` buffers of `count` floats through the hypercube addressing.
// Returns 1 on success, 0 when the addressing is not a consistent schedule.
int b2h_hypercube_allreduce(int twisted, int num_nodes, int shift, float* const* bufs, size_t count, int threaded) {
  if (twisted) return hypercube_allreduce(TwistedHyperCube(num_nodes, shift), bufs, count, threaded != 0) ? 1 : 0;
  return hypercube_allreduce(HyperCube(num_nodes, shift), bufs, count, threaded != 0) ? 1 : 0;
}

// Seconds per allreduce of `count` floats over `num_nodes` host threads (one per node), buffers
// U(-1,1) from seed = node id; 0 when the addressing is inconsistent.
double b2h_time_hypercube_allreduce(int twisted, int num_nodes, int shift, size_t count, int iterations) {
  std::vector<std::vector<float>> store(num_nodes, std::vector<float>(count));
  std::vector<float*> bufs(num_nodes);
  for (int i = 0; i < num_nodes; ++i) {
    for (size_t k = 0; k < count; ++k) store[i][k] = b2_rng_uniform((uint64_t)i, k, -1.f, 1.f);
    bufs[i] = store[i].data();
  }
  HyperCube plain(num_nodes, shift);
  TwistedHyperCube twist(twisted ? num_nodes : 2, twisted ? shift : 0);
  const HyperCube& cube = twisted ? static_cast<const HyperCube&>(twist) : plain;
  if (!hypercube_allreduce(cube, bufs.data(), count, true, 1)) return 0.0;  // warm-up
  // keep the values bounded over the timed repetitions
  for (int i = 0; i < num_nodes; ++i)
    for (size_t k = 0; k < count; ++k) store[i][k] *= 1e-6f;
  const auto t0 = std::chrono::steady_clock::now();
  hypercube_allreduce(cube, bufs.data(), count, true, iterations);
  return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() / iterations;
}

// The 2 * log2(num_nodes) steps of node `id`, 5 ints each: dim, peer, first_chunk, num_chunks, reduce.
int b2h_hypercube_steps(int twisted, int num_nodes, int shift, int id, int* out, int max_steps) {
  std::vector<HyperCubeStep> st = twisted ? hypercube_allreduce_steps(TwistedHyperCube(num_nodes, shift), id)
                                          : hypercube_allreduce_steps(HyperCube(num_nodes, shift), id);
  int n = 0;
  for (const auto& s : st) {
    if (n >= max_steps) break;
    int* o = out + 5 * n++;
    o[0] = s.dim; o[1] = s.peer; o[2] = s.first_chunk; o[3] = s.num_chunks; o[4] = s.reduce ? 1 : 0;
  }
  return (int)st.size();
}

// The library's gradient-bucket rule (csrc/bucket_plan.h): lowest / highest layer of each layer's bucket.
void b2h_plan_buckets(const size_t* layer_bytes, int nlayers, int world_size, int allreduce, int ar_bucket_mb,
                      double growth, int* bucket_low, int* bucket_high) {
  b2::plan_gradient_buckets(layer_bytes, nlayers, world_size, allreduce != 0, ar_bucket_mb, growth, bucket_low,
                            bucket_high);
}

// The library's slab layout and slice ownership under the sharded update (csrc/bucket_plan.h).
size_t b2h_slab_layout(const size_t* layer_elems, int nlayers, int world_size, size_t* offset, size_t* padded) {
  return b2::plan_slab_layout(layer_elems, nlayers, world_size, offset, padded);
}
void b2h_bucket_slice(const size_t* offset, const size_t* padded, int low, int high, int world_size, int rank,
                      size_t* out4) {
  b2::plan_bucket_slice(offset, padded, low, high, world_size, rank, &out4[0], &out4[1], &out4[2], &out4[3]);
}

// The rule as the library applies it with the sharded update and the default bucket size: layer 0 in
// a bucket of its own.
void b2h_plan_buckets_sharded(const size_t* layer_bytes, int nlayers, int world_size, int ar_bucket_mb, double growth,
                              int* bucket_low, int* bucket_high) {
  b2::plan_gradient_buckets(layer_bytes, nlayers, world_size, true, ar_bucket_mb, growth, bucket_low, bucket_high);
  if (ar_bucket_mb < 0 && world_size > 1) b2::plan_split_lowest_layer(nlayers, bucket_low, bucket_high);
}

void b2h_ring_info(int nsock, int sid, int task, int* out3) {
  nsockets = nsock;
  get_my_ring_info(sid, task, &out3[0], &out3[1], &out3[2]);
}

// Matrix<float, 16> layout facts: ld, allocation alignment, element addressing.
void b2h_matrix_layout(int rows, int cols, int* ld, int* aligned4k, long long* offset_last) {
  Matrix<float, PAD> m(rows, cols);
  *ld = m.ld();
  *aligned4k = (reinterpret_cast<uintptr_t>(m.rawData()) % 4096) == 0;
  *offset_last = m.rawData(rows - 1, cols - 1) - m.rawData();
}

// init_matrices() on a fresh model; returns the input and the weights densely.
void b2h_init_matrices(int nlayers_, const int* widths, int batch, int nsock, float* x, float** w) {
  nsockets = nsock;
  set_model(std::vector<int>(widths, widths + nlayers_ + 1));
  activations[0].reset(new Matrix<float, PAD>(batch, nfeatures[0]));
  for (int l = 0; l < nlayers; ++l)
    weights[l].reset(new Matrix<float, PAD>(nsock * nfeatures[l + 1], nfeatures[l]));
  randSeed(3);
  init_matrices();
  for (int i = 0; i < batch; ++i) memcpy(x + (size_t)i * nfeatures[0], activations[0]->rawData(i, 0), 4 * nfeatures[0]);
  for (int l = 0; l < nlayers; ++l)
    for (int i = 0; i < nsock * nfeatures[l + 1]; ++i)
      memcpy(w[l] + (size_t)i * nfeatures[l], weights[l]->rawData(i, 0), 4 * nfeatures[l]);
}

// print_checksum arithmetic on a dense matrix: l1, l2, trace.
void b2h_checksum(const float* w, int rows, int cols, double* out3) {
  double l1 = 0, l2 = 0, tr = 0;
  for (int i = 0; i < rows; ++i) {
    for (int j = 0; j < cols; ++j) {
      float v = w[(size_t)i * cols + j];
      l1 += std::abs(v);
      l2 += v * v;
    }
    if (i < std::min(rows, cols)) tr += w[(size_t)i * cols + i];
  }
  out3[0] = l1;
  out3[1] = std::sqrt(l2);
  out3[2] = tr;
}
}

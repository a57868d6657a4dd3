#include "mlp_bench_common.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>

std::vector<int> nfeatures = {1024, 1024, 1024, 1024, 1024, 1024, 1024, 1};
int nlayers = 7;
int NWARMUP = 16, NITER = 256;
int nthreads_per_socket = 1, nthreads = 1;
double wall_clock_time = 0;

std::vector<std::vector<std::array<double, NUM_BREAKDOWNS>>> sum_times;
std::vector<std::array<double, NUM_BREAKDOWNS>> sum_flops;

std::vector<std::unique_ptr<Matrix<float, PAD>>> weights, weight_grads, weight_grad_push_bufs, activations;

std::vector<std::array<int, 8>> rings = {{0, 1, 2, 4, 7, 6, 5, 3}, {0, 3, 5, 6, 7, 4, 2, 1}};

void set_model(const std::vector<int>& widths) {
  nfeatures = widths;
  nlayers = (int)widths.size() - 1;
  weights.clear();
  weight_grads.clear();
  weight_grad_push_bufs.clear();
  activations.clear();
  weights.resize(nlayers);
  weight_grads.resize(nlayers);
  weight_grad_push_bufs.resize(nlayers);
  activations.resize(nlayers + 2);
  sum_flops.assign(nlayers, {});
  sum_times.clear();
}

void init_matrices() {
  activations[0]->randFill(0.f, 1.f);
  for (int l = 0; l < nlayers; ++l) {
    Matrix<float, PAD>& w = *weights[l];
    const int rows = nfeatures[l + 1];
    for (int r = 0; r < rows; ++r) randFill(w.rawData(r, 0), (size_t)w.ncols(), -0.1f, 0.1f);
    // every socket starts from the same replica
    const size_t replica_bytes = sizeof(float) * (size_t)rows * w.ld();
    for (int s = 1; s * rows < w.nrows(); ++s) memcpy(w.rawData(s * rows, 0), w.rawData(), replica_bytes);
  }
}

namespace {
struct PhaseStat {
  double max = 0, imbalance = 1;
};

// max over workers and max/avg over the workers that take part in `phase`
PhaseStat phase_stat(int layer, int phase) {
  PhaseStat st;
  double total = 0;
  int active = 0;
  for (const auto& worker : sum_times) {
    const double t = worker[layer][phase];
    total += t;
    st.max = std::max(st.max, t);
    if (t > 0) ++active;
  }
  if (active > 0 && total > 0) st.imbalance = st.max / (total / active);
  return st;
}

double rate(double work, double seconds, double divisor) {
  return seconds > 0 ? work / seconds / divisor / 1e9 : 0.0;
}
}  // namespace

void report_timing() {
  // wgt_update = reduce-scatter + allgather, as in the reference (mlp_bench_common.cc:43-51)
  for (int l = 0; l < nlayers; ++l) {
    for (auto& worker : sum_times)
      worker[l][WGT_UPDATE] = worker[l][WGT_UPDATE_REDUCE_SCATTER] + worker[l][WGT_UPDATE_ALLGATHER];
    sum_flops[l][WGT_UPDATE] = sum_flops[l][WGT_UPDATE_REDUCE_SCATTER] + sum_flops[l][WGT_UPDATE_ALLGATHER];
  }
  static const char* names[NUM_BREAKDOWNS] = {"fwd", "wgt_grad", "bwd", "wgt_update", "wgt_update_reduce_scatter",
                                              "wgt_update_allgather"};
  const int workers = std::max<int>(1, (int)sum_times.size());
  double total_time[NUM_BREAKDOWNS] = {0}, total_work[NUM_BREAKDOWNS] = {0};
  for (int l = 0; l < nlayers; ++l) {
    printf("[layer %d]", l);
    for (int ph = FWD; ph < NUM_BREAKDOWNS; ++ph) {
      const PhaseStat st = phase_stat(l, ph);
      const bool gemm = ph <= BWD;
      printf("%s %s %g ms/iter (%g %s) imbalance %g", ph == FWD ? "" : ",", names[ph], st.max / NITER * 1e3,
             rate(sum_flops[l][ph], st.max, gemm ? workers : nsockets), gemm ? "GF/s/gpu" : "GB/s/gpu",
             st.imbalance);
      total_time[ph] += st.max;
      total_work[ph] += sum_flops[l][ph];
    }
    printf("\n");
  }
  printf("total");
  for (int ph = FWD; ph < NUM_BREAKDOWNS; ++ph) {
    const bool gemm = ph <= BWD;
    printf("%s %s %g ms/iter (%g %s)", ph == FWD ? "" : ",", names[ph], total_time[ph] / NITER * 1e3,
           rate(total_work[ph], total_time[ph], gemm ? workers : nsockets), gemm ? "GF/s/gpu" : "GB/s/gpu");
  }
  printf("\nwall clock time %g ms/iter\n", wall_clock_time / NITER * 1e3);
}

void print_checksum() {
  // replica 0 only, double accumulation (mlp_bench_common.cc:152-168)
  for (int l = 0; l < nlayers; ++l) {
    const Matrix<float, PAD>& w = *weights[l];
    const int rows = nfeatures[l + 1], cols = nfeatures[l];
    double l1 = 0, l2 = 0, trace = 0;
    for (int i = 0; i < rows; ++i) {
      for (int j = 0; j < cols; ++j) {
        const float v = w(i, j);
        l1 += std::abs(v);
        l2 += v * v;
      }
      if (i < std::min(rows, cols)) trace += w(i, i);
    }
    printf("layer %d l1 %g l2 %g trace %g\n", l, l1, std::sqrt(l2), trace);
  }
}

void get_my_ring_info(int sid, int task, int* idx_in_ring, int* prev_sid, int* next_sid) {
  const int which = task % (int)rings.size();
  if (nsockets < 8) {
    // fewer than 8 sockets: plain socket order; odd tasks travel the other way but keep
    // idx_in_ring = sid (the reference's behaviour, mlp_bench_common.cc:182-188)
    const int up = (sid + 1) % nsockets, down = (sid - 1 + nsockets) % nsockets;
    *idx_in_ring = sid;
    *prev_sid = which ? up : down;
    *next_sid = which ? down : up;
    return;
  }
  const auto& ring = rings[which];
  const int pos = (int)(std::find(ring.begin(), ring.end(), sid) - ring.begin());
  *idx_in_ring = pos;
  *prev_sid = ring[(pos - 1 + nsockets) % nsockets];
  *next_sid = ring[(pos + 1) % nsockets];
}

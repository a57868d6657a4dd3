// Shared state and reporting of the MLP benchmark drivers: the counterpart of the
// reference's mlp_bench_common.h:9-68 for the GPU driver (mlp_cuda.cc).  Same
// names; the model (layer widths, batch, iteration counts) is a run-time setting
// instead of compile-time constants, with the reference's values as defaults.
#pragma once

#include <array>
#include <memory>
#include <vector>

#include "Matrix.h"
#include "Partition.h"

constexpr int PAD = 16;
constexpr int CACHE_LINE_LEN = 16;

enum Breakdown {
  FWD = 0,
  WGT_GRAD,
  BWD,
  WGT_UPDATE,
  WGT_UPDATE_REDUCE_SCATTER,
  WGT_UPDATE_ALLGATHER,
  NUM_BREAKDOWNS,
};

// Layer widths F_0..F_L (default: the reference's {1024 x 7, 1}) and derived count.
extern std::vector<int> nfeatures;
extern int nlayers;
extern int NWARMUP, NITER;  // 16 and 256 in the reference
extern int nthreads_per_socket, nthreads;
void set_model(const std::vector<int>& widths);

constexpr int MAX_NUM_THREADS = 1024;
// sum_times[worker][layer][breakdown] in seconds over the timed iterations;
// a worker is a socket's thread in the reference and a GPU here.
extern std::vector<std::vector<std::array<double, NUM_BREAKDOWNS>>> sum_times;
// flops (GEMM phases) or bytes (update phases) per layer and breakdown
extern std::vector<std::array<double, NUM_BREAKDOWNS>> sum_flops;
extern double wall_clock_time;

// Threads per socket the reference takes away from the GEMMs to run the allreduce
// (index = threads per socket). The GPU driver has no use for it - the side stream
// plays that role - but report_timing keeps the same averaging rule.
constexpr int nthreads_per_socket_for_allreduce[29] = {
    0, 0, 0, 0, 0, 1, 1, 1, 1, 1, 2, 2, 2, 2, 2, 2, 2, 2, 2, 2, 4, 4, 4, 4, 4, 4, 4, 4, 4,
};

// Two rings over 8 sockets running in opposite directions.
extern std::vector<std::array<int, 8>> rings;

extern std::vector<std::unique_ptr<Matrix<float, PAD>>> weights, weight_grads, weight_grad_push_bufs,
    activations;

// Inputs U(0,1), weights U(-0.1,0.1) on replica 0, copied to the other replicas.
void init_matrices();
void report_timing();
void print_checksum();
void get_my_ring_info(int sid, int task, int* idx_in_ring, int* prev_sid, int* next_sid);

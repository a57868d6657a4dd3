// Work split of the benchmark: batch rows over sockets (one GPU each here), then
// over the threads of a socket; and the 2-D (m, n) tiling of one GEMM inside a
// socket.  Same functions and argument meaning as the reference's Partition.h:8-76.
//
// On the GPU path the socket-level split decides each rank's batch shard
// (get_partition(batch, rank, 1, 0)); the intra-socket 2-D split is kept for
// drivers that tile host-side work and as the documented counterpart of the CTA
// tile grid.
#pragma once

#include <algorithm>
#include <cassert>
#include <cmath>
#include <utility>

extern int nsockets;

// Position of the calling thread. Inside an OpenMP parallel region it comes from
// OpenMP, like the reference; other threads (one host thread per GPU, say) declare
// theirs once with set_thread_position().
void set_thread_position(int thread_num, int num_threads);
int get_num_threads_per_socket();
int get_socket_num();
int get_thread_num_in_socket();

int get_work_per_socket(int work);
std::pair<int, int> get_partition(int work);
std::pair<int, int> get_partition(int work, int nthreads_per_socket, int tid_in_socket);
std::pair<int, int> get_partition(int work, int socket_id, int nthreads_per_socket, int tid_in_socket);

void get_intra_socket_2dpartition(int* m_begin, int* m_end, int* n_begin, int* n_end, int m, int n,
                                  double aspect_ratio, bool m_align);
void get_intra_socket_2dpartition(int* m_begin, int* m_end, int* n_begin, int* n_end, int m, int n,
                                  double aspect_ratio, bool m_align, int nthreads_per_socket,
                                  int tid_in_socket);

void get_2dpartition(int* m_begin, int* m_end, int* n_begin, int* n_end, int m, int n,
                     double aspect_ratio, bool m_align);
void get_2dpartition(int* m_begin, int* m_end, int* n_begin, int* n_end, int m, int n,
                     double aspect_ratio, bool m_align, int nthreads_per_socket, int tid_in_socket);
void get_2dpartition(int* m_begin, int* m_end, int* n_begin, int* n_end, int m, int n,
                     double aspect_ratio, bool m_align, int socket_id, int nthreads_per_socket,
                     int tid_in_socket);

#include "Partition.h"

#ifdef _OPENMP
#include <omp.h>
#endif

int nsockets = 1;

namespace {

thread_local int tl_thread_num = 0;
thread_local int tl_num_threads = 1;

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

struct ThreadPos {
  int tid, count;
};

ThreadPos where_am_i() {
#ifdef _OPENMP
  if (omp_in_parallel()) return {omp_get_thread_num(), omp_get_num_threads()};
#endif
  return {tl_thread_num, tl_num_threads};
}

// Rows per block when `extent` is cut into `blocks` pieces; whole multiples of 16
// when `align16` (the reference aligns n always and m on request, Partition.cc:93-99).
inline int block_extent(int extent, int blocks, bool align16) {
  return align16 ? ceil_div(ceil_div(extent, 16), blocks) * 16 : ceil_div(extent, blocks);
}

}  // namespace

void set_thread_position(int thread_num, int num_threads) {
  tl_thread_num = thread_num;
  tl_num_threads = num_threads;
}

int get_num_threads_per_socket() {
  ThreadPos p = where_am_i();
  assert(p.count % nsockets == 0);
  return p.count / nsockets;
}

int get_socket_num() { return where_am_i().tid / get_num_threads_per_socket(); }

int get_thread_num_in_socket() { return where_am_i().tid % get_num_threads_per_socket(); }

int get_work_per_socket(int work) { return ceil_div(work, nsockets); }

std::pair<int, int> get_partition(int work, int socket_id, int nthreads_per_socket, int tid_in_socket) {
  // level 1: equal ceil-div shards per socket; level 2: the same inside the shard
  const int shard = get_work_per_socket(work);
  const int shard_begin = std::min(socket_id * shard, work);
  const int chunk = ceil_div(shard, nthreads_per_socket);
  const int lo = std::min(tid_in_socket * chunk, shard);
  const int hi = std::min(lo + chunk, shard);
  return {std::min(shard_begin + lo, work), std::min(shard_begin + hi, work)};
}

std::pair<int, int> get_partition(int work, int nthreads_per_socket, int tid_in_socket) {
  return get_partition(work, get_socket_num(), nthreads_per_socket, tid_in_socket);
}

std::pair<int, int> get_partition(int work) {
  return get_partition(work, get_num_threads_per_socket(), get_thread_num_in_socket());
}

void get_intra_socket_2dpartition(int* m_begin, int* m_end, int* n_begin, int* n_end, int m, int n,
                                  double aspect_ratio, bool m_align, int nthreads_per_socket,
                                  int tid_in_socket) {
  // Choose mb x nb = nthreads_per_socket blocks so that (rows per block) / (cols per
  // block) is as close as possible to aspect_ratio. Candidates are the divisors of the
  // thread count in increasing mb; the search stops at the first divisor that does
  // not improve on the best so far (Partition.cc:93-152).
  const int T = nthreads_per_socket;
  int mb = 1, nb = T;
  int bm = block_extent(m, mb, m_align);
  int bn = block_extent(n, nb, true);
  double best = std::abs((double)bm / bn - aspect_ratio);

  for (int cand_mb = 2; cand_mb <= T; ++cand_mb) {
    if (T % cand_mb) continue;
    const int cand_nb = T / cand_mb;
    const int rows_each = ceil_div(m, cand_mb), cols_each = ceil_div(n, cand_nb);
    if (m_align) {
      if (aspect_ratio < 1 && bm == 16 && rows_each < 16) continue;  // already at the 16-row floor
      if (rows_each <= 8) continue;
    }
    if (cols_each <= 8) continue;
    const int cand_bm = block_extent(m, cand_mb, m_align);
    const int cand_bn = block_extent(n, cand_nb, true);
    const double delta = std::abs((double)cand_bm / cand_bn - aspect_ratio);
    if (!(delta < best)) break;
    best = delta;
    mb = cand_mb;
    nb = cand_nb;
    bm = cand_bm;
    bn = cand_bn;
  }

  const int row_block = tid_in_socket / nb, col_block = tid_in_socket % nb;
  *m_begin = std::min(row_block * bm, m);
  *m_end = std::min(*m_begin + bm, m);
  *n_begin = std::min(col_block * bn, n);
  *n_end = std::min(*n_begin + bn, n);
}

void get_intra_socket_2dpartition(int* m_begin, int* m_end, int* n_begin, int* n_end, int m, int n,
                                  double aspect_ratio, bool m_align) {
  get_intra_socket_2dpartition(m_begin, m_end, n_begin, n_end, m, n, aspect_ratio, m_align,
                               get_num_threads_per_socket(), get_thread_num_in_socket());
}

void get_2dpartition(int* m_begin, int* m_end, int* n_begin, int* n_end, int m, int n,
                     double aspect_ratio, bool m_align, int socket_id, int nthreads_per_socket,
                     int tid_in_socket) {
  // rows are first cut per socket, then the socket's slab is tiled in 2-D
  const int slab = get_work_per_socket(m);
  get_intra_socket_2dpartition(m_begin, m_end, n_begin, n_end, slab, n, aspect_ratio, m_align,
                               nthreads_per_socket, tid_in_socket);
  const int slab_begin = std::min(socket_id * slab, m);
  *m_begin = std::min(slab_begin + *m_begin, m);
  *m_end = std::min(slab_begin + *m_end, m);
}

void get_2dpartition(int* m_begin, int* m_end, int* n_begin, int* n_end, int m, int n,
                     double aspect_ratio, bool m_align, int nthreads_per_socket, int tid_in_socket) {
  get_2dpartition(m_begin, m_end, n_begin, n_end, m, n, aspect_ratio, m_align, get_socket_num(),
                  nthreads_per_socket, tid_in_socket);
}

void get_2dpartition(int* m_begin, int* m_end, int* n_begin, int* n_end, int m, int n,
                     double aspect_ratio, bool m_align) {
  get_2dpartition(m_begin, m_end, n_begin, n_end, m, n, aspect_ratio, m_align,
                  get_num_threads_per_socket(), get_thread_num_in_socket());
}

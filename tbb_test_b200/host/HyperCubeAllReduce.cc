#include "HyperCubeAllReduce.h"

#include <algorithm>
#include <atomic>
#include <cstring>
#include <thread>

std::vector<HyperCubeStep> hypercube_allreduce_steps(const HyperCube& cube, int id) {
  const int D = cube.Dimension();
  std::vector<HyperCubeStep> steps;
  for (int d = D - 1; d >= 0; --d)
    steps.push_back({d, cube.Peer(id, d), cube.RecvLocation(id, d), 1 << d, true});
  for (int d = 0; d < D; ++d) {
    const int peer = cube.Peer(id, d);
    // what the peer finished (or gathered so far) in this dimension
    steps.push_back({d, peer, cube.RecvLocation(peer, d), 1 << d, false});
  }
  return steps;
}

bool hypercube_schedule_is_consistent(const HyperCube& cube) {
  const int N = cube.NumNodes(), D = cube.Dimension();
  std::vector<int> lo(N, 0), len(N, N);  // chunk range each node is still responsible for
  for (int d = D - 1; d >= 0; --d) {
    for (int i = 0; i < N; ++i) {
      const int p = cube.Peer(i, d);
      if (p < 0 || p >= N || p == i || cube.Peer(p, d) != i) return false;
      if (cube.SendLocation(i, d) != cube.RecvLocation(p, d)) return false;
      // partners must split one common range into its two halves
      if (lo[i] != lo[p] || len[i] != (2 << d)) return false;
      const int r = cube.RecvLocation(i, d), s = cube.SendLocation(i, d);
      if (!((r == lo[i] && s == lo[i] + (1 << d)) || (s == lo[i] && r == lo[i] + (1 << d)))) return false;
    }
    for (int i = 0; i < N; ++i) {
      lo[i] = cube.RecvLocation(i, d);
      len[i] = 1 << d;
    }
  }
  std::vector<int> owned(lo);
  std::sort(owned.begin(), owned.end());
  for (int i = 0; i < N; ++i)
    if (owned[i] != i) return false;
  return true;
}

namespace {

struct ChunkRange {
  size_t begin, end;
};

ChunkRange chunk_span(size_t count, int N, int first_chunk, int num_chunks) {
  const size_t chunk = (count + N - 1) / N;
  ChunkRange r;
  r.begin = std::min(count, chunk * (size_t)first_chunk);
  r.end = std::min(count, chunk * (size_t)(first_chunk + num_chunks));
  return r;
}

void run_step(const HyperCubeStep& s, float* mine, const float* theirs, size_t count, int N) {
  const ChunkRange r = chunk_span(count, N, s.first_chunk, s.num_chunks);
  if (s.reduce) {
    for (size_t k = r.begin; k < r.end; ++k) mine[k] += theirs[k];
  } else if (r.end > r.begin) {
    memcpy(mine + r.begin, theirs + r.begin, (r.end - r.begin) * sizeof(float));
  }
}

// Reusable barrier for the per-node threads: counts arrivals, the last one opens the next
// generation; waiters spin briefly, then yield (the nodes may outnumber the cores).
class StepBarrier {
 public:
  explicit StepBarrier(int n) : n_(n) {}
  void wait() {
    const unsigned gen = gen_.load(std::memory_order_acquire);
    if (arrived_.fetch_add(1, std::memory_order_acq_rel) + 1 == n_) {
      arrived_.store(0, std::memory_order_relaxed);
      gen_.store(gen + 1, std::memory_order_release);
      return;
    }
    for (int spins = 0; gen_.load(std::memory_order_acquire) == gen; ++spins)
      if (spins > 2000) std::this_thread::yield();
  }

 private:
  const int n_;
  std::atomic<int> arrived_{0};
  std::atomic<unsigned> gen_{0};
};

}  // namespace

bool hypercube_allreduce(const HyperCube& cube, float* const* bufs, size_t count, bool threaded,
                         int iterations) {
  if (!hypercube_schedule_is_consistent(cube)) return false;
  const int N = cube.NumNodes();
  std::vector<std::vector<HyperCubeStep>> steps(N);
  for (int i = 0; i < N; ++i) steps[i] = hypercube_allreduce_steps(cube, i);
  const size_t nsteps = steps[0].size();
  // Within a step every node reads chunks its partner does not write in that step (the two
  // halves of a range while halving, disjoint finished ranges while doubling), so a barrier
  // between steps is all the ordering needed.
  if (!threaded) {
    for (int it = 0; it < iterations; ++it)
      for (size_t s = 0; s < nsteps; ++s)
        for (int i = 0; i < N; ++i) run_step(steps[i][s], bufs[i], bufs[steps[i][s].peer], count, N);
    return true;
  }
  StepBarrier barrier(N);
  std::vector<std::thread> pool;
  for (int i = 0; i < N; ++i)
    pool.emplace_back([&, i] {
      for (int it = 0; it < iterations; ++it)
        for (size_t s = 0; s < nsteps; ++s) {
          run_step(steps[i][s], bufs[i], bufs[steps[i][s].peer], count, N);
          barrier.wait();
        }
    });
  for (auto& t : pool) t.join();
  return true;
}

// Small-message gradient allreduce over peer memory (NVLink loads and stores), for the
// messages where a library collective is latency-bound (the 1 MiB layers of the deep narrow
// configuration). Two-shot: every rank sums the chunk it owns by reading that chunk from all
// ranks' gradient slabs, in rank order (so all ranks end with identical bits), and stores the
// sum into every rank's slab. Ordering between ranks is by two flag exchanges per call,
// "my input is ready" and "my stores are done"; flags carry a call counter (epoch) that only
// grows, so they are never reset. Every wait is bounded: after P2pParams::wait_ns the kernel
// records a status code and returns without signalling, so that the peers time out too and
// every rank reports the failure; a launch that finds a failure already recorded returns at
// once, so that the calls queued behind a failed one do not each wait out the limit.
//
// No TMA, no multicast: plain peer loads/stores issued per CTA.
#include "common.cuh"

namespace b2 {

namespace {

constexpr int THREADS = 512;
constexpr int MAX_CTAS = 32;

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Spin until *flag has reached `epoch` (wrap-safe). False after `limit_ns`.
__device__ bool wait_flag(const unsigned int* flag, unsigned int epoch, unsigned long long limit_ns,
                          unsigned int* status, unsigned int code) {
  if ((int)(ld_acquire_sys(flag) - epoch) >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned int spins = 0;
  while ((int)(ld_acquire_sys(flag) - epoch) < 0) {
    if ((++spins & 0x3F) == 0 && globaltimer_ns() - t0 > limit_ns) {
      atomicCAS(status, 0u, code);
      return false;
    }
  }
  return true;
}

// One rank's part of one allreduce; `cta` of `nctas` CTAs of that rank.
__device__ void p2p_allreduce_body(const P2pParams& p, int cta, int nctas) {
  __shared__ int abort_s;
  __shared__ int last_s;
  const int t = threadIdx.x;
  const int world = p.world, rank = p.rank;
  unsigned int* my_flags = p.flags[rank];
  if (t == 0) {
    // a wait of an earlier call already gave up: the call counters of the ranks no longer agree
    abort_s = (*reinterpret_cast<volatile unsigned int*>(p.status) >= 100u) ? 1 : 0;
    last_s = 0;
  }
  __syncthreads();
  if (abort_s) return;

  // ---- 1. my input is ready (it was written by earlier work of this stream); wait for the peers'
  if (t < world && t != rank) {
    if (cta == 0) {
      __threadfence_system();
      st_release_sys(p.flags[t] + P2P_FLAG_ARRIVE + rank, p.epoch);
    }
    if (!wait_flag(my_flags + P2P_FLAG_ARRIVE + t, p.epoch, p.wait_ns, p.status, 101u)) abort_s = 1;
  }
  __syncthreads();
  if (abort_s) return;  // no "done" signal: the peers give up as well and report it

  // ---- 2. sum the chunk this rank owns, rank 0 first, and store it to every rank
  const unsigned long long per = (((p.count + world - 1) / world) + 3ull) & ~3ull;  // multiple of 4 elements
  const unsigned long long begin = per * rank < p.count ? per * rank : p.count;
  const unsigned long long end = begin + per < p.count ? begin + per : p.count;
  const unsigned long long n4 = (end - begin) >> 2;
  const unsigned long long base = p.offset + begin;  // 16-byte aligned: offset and `per` are multiples of 4
  for (unsigned long long i = (unsigned long long)cta * blockDim.x + t; i < n4;
       i += (unsigned long long)nctas * blockDim.x) {
    float4 v[P2P_MAX_RANKS];
#pragma unroll
    for (int r = 0; r < P2P_MAX_RANKS; ++r)
      if (r < world) v[r] = __ldcv(reinterpret_cast<const float4*>(p.slab[r] + base) + i);
    float4 acc = v[0];
#pragma unroll
    for (int r = 1; r < P2P_MAX_RANKS; ++r)
      if (r < world) {
        acc.x += v[r].x;
        acc.y += v[r].y;
        acc.z += v[r].z;
        acc.w += v[r].w;
      }
#pragma unroll
    for (int r = 0; r < P2P_MAX_RANKS; ++r)
      if (r < world) reinterpret_cast<float4*>(p.slab[r] + base)[i] = acc;
  }
  if (cta == 0 && t == 0) {  // the up to three elements after the last whole vector of the chunk
    for (unsigned long long k = begin + (n4 << 2); k < end; ++k) {
      float acc = __ldcv(p.slab[0] + p.offset + k);
      for (int r = 1; r < world; ++r) acc += __ldcv(p.slab[r] + p.offset + k);
      for (int r = 0; r < world; ++r) p.slab[r][p.offset + k] = acc;
    }
  }

  // ---- 3. the last CTA of this rank to finish tells the peers, then waits for theirs
  __threadfence_system();
  __syncthreads();
  if (t == 0) {
    const unsigned int prev = atomicAdd(p.ctas_done, 1u);
    if (prev == (unsigned int)nctas - 1u) {
      *p.ctas_done = 0;  // ready for the next call (calls of one rank run one after another)
      last_s = 1;
    }
    __threadfence();
  }
  __syncthreads();
  if (!last_s) return;
  if (t < world && t != rank) {
    __threadfence_system();
    st_release_sys(p.flags[t] + P2P_FLAG_DONE + rank, p.epoch);
    wait_flag(my_flags + P2P_FLAG_DONE + t, p.epoch, p.wait_ns, p.status, 102u);
  }
}

__global__ void __launch_bounds__(THREADS) p2p_allreduce_kernel(const __grid_constant__ P2pParams p) {
  p2p_allreduce_body(p, blockIdx.x, gridDim.x);
}

// All ranks in one launch on one GPU (blockIdx.y = rank): the ranks wait on one another, so
// the launch is cooperative, which guarantees that every CTA is resident.
__global__ void __launch_bounds__(THREADS) p2p_allreduce_emulated_kernel(const P2pParams* ranks) {
  p2p_allreduce_body(ranks[blockIdx.y], blockIdx.x, gridDim.x);
}

int ctas_for(const P2pParams& p, int limit) {
  const unsigned long long per = (p.count + p.world - 1) / p.world;
  long long n = (long long)((per / 4 + THREADS - 1) / THREADS);
  if (n < 1) n = 1;
  if (n > MAX_CTAS) n = MAX_CTAS;
  if (limit > 0 && n > limit) n = limit;
  return (int)n;
}

}  // namespace

cudaError_t p2p_allreduce_launch(const P2pParams& p, int cta_limit, cudaStream_t stream) {
  if (p.world < 2 || p.world > P2P_MAX_RANKS || p.rank < 0 || p.rank >= p.world || (p.offset & 3ull))
    return cudaErrorInvalidValue;
  p2p_allreduce_kernel<<<ctas_for(p, cta_limit), THREADS, 0, stream>>>(p);
  return cudaGetLastError();
}

cudaError_t p2p_allreduce_emulated_launch(const P2pParams* ranks_dev, const P2pParams& any_rank,
                                          cudaStream_t stream) {
  if (any_rank.world < 2 || any_rank.world > P2P_MAX_RANKS || (any_rank.offset & 3ull)) return cudaErrorInvalidValue;
  int dev = 0, coop = 0, sms = 0, per_sm = 0;
  cudaError_t e;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
  if ((e = cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev)) != cudaSuccess) return e;
  if (!coop) return cudaErrorNotSupported;
  if ((e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess) return e;
  if ((e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, p2p_allreduce_emulated_kernel, THREADS, 0)) !=
      cudaSuccess)
    return e;
  int ctas = ctas_for(any_rank, 0);
  while (ctas > 1 && ctas * any_rank.world > sms * per_sm) --ctas;
  if (ctas * any_rank.world > sms * per_sm) return cudaErrorCooperativeLaunchTooLarge;
  dim3 grid(ctas, any_rank.world), block(THREADS);
  void* args[] = {(void*)&ranks_dev};
  return cudaLaunchCooperativeKernel((const void*)p2p_allreduce_emulated_kernel, grid, block, args, 0, stream);
}

}  // namespace b2

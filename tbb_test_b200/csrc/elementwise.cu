// Bandwidth-bound kernels of the training step: the SGD weight update, the
// output gradient, precision conversion and seeded fills.  All of them are
// grid-stride loops over 16-byte vectors with a scalar tail.
#include "common.cuh"

namespace b2 {
namespace {

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// ---------------------------------------------------------------- SGD update
// Replaces the AVX-512 loops of update_weight_allgather (mlp_omp.cc:217-223 for
// one socket, :240-252 for the owned chunk after the reduce-scatter):
//   w = fma(-alpha, g, w)
// Algorithmic traffic per parameter: read w (4) + read g (4 or 2) + write w (4)
// (+ write the bf16 operand copy (2) in BF16 precision).
__device__ __forceinline__ float tf32_lo(float v) {  // v - tf32(v): what a tf32 read of v drops (exact)
  return v - __uint_as_float(__float_as_uint(v) & 0xFFFFE000u);
}

template <bool G_BF16, bool W16, bool W_LO>
__global__ void __launch_bounds__(256) sgd_kernel(float* __restrict__ w, const void* __restrict__ gv,
                                                  __nv_bfloat16* __restrict__ w16, float* __restrict__ w_lo,
                                                  size_t n, float neg_lr) {
  const size_t nvec = n / 4;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  float4* w4 = reinterpret_cast<float4*>(w);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float4 wv = w4[i];
    float g0, g1, g2, g3;
    if (G_BF16) {
      uint2 raw = __ldg(reinterpret_cast<const uint2*>(gv) + i);
      __nv_bfloat162 lo = *reinterpret_cast<__nv_bfloat162*>(&raw.x);
      __nv_bfloat162 hi = *reinterpret_cast<__nv_bfloat162*>(&raw.y);
      g0 = __low2float(lo); g1 = __high2float(lo); g2 = __low2float(hi); g3 = __high2float(hi);
    } else {
      float4 g = __ldg(reinterpret_cast<const float4*>(gv) + i);
      g0 = g.x; g1 = g.y; g2 = g.z; g3 = g.w;
    }
    wv.x = fmaf(neg_lr, g0, wv.x);
    wv.y = fmaf(neg_lr, g1, wv.y);
    wv.z = fmaf(neg_lr, g2, wv.z);
    wv.w = fmaf(neg_lr, g3, wv.w);
    w4[i] = wv;
    if (W16) {
      __nv_bfloat162 a = __floats2bfloat162_rn(wv.x, wv.y);
      __nv_bfloat162 b = __floats2bfloat162_rn(wv.z, wv.w);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&a);
      o.y = *reinterpret_cast<uint32_t*>(&b);
      reinterpret_cast<uint2*>(w16)[i] = o;
    }
    if (W_LO)
      reinterpret_cast<float4*>(w_lo)[i] = make_float4(tf32_lo(wv.x), tf32_lo(wv.y), tf32_lo(wv.z), tf32_lo(wv.w));
  }
  // tail (n % 4 elements)
  for (size_t i = nvec * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float g = G_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(gv)[i])
                     : reinterpret_cast<const float*>(gv)[i];
    float v = fmaf(neg_lr, g, w[i]);
    w[i] = v;
    if (W16) w16[i] = __float2bfloat16_rn(v);
    if (W_LO) w_lo[i] = tf32_lo(v);
  }
}

// ------------------------------------------------------------ output gradient
// REF: dZ[L-1] = A[L] (the reference feeds the forward output back as the
// gradient, mlp_omp.cc:565,655). BASELINE: dZ[L-1] = (A[L] - T) / B_global.
template <typename TO>
__global__ void __launch_bounds__(256) loss_grad_kernel(const float* __restrict__ y,
                                                        const float* __restrict__ t,
                                                        TO* __restrict__ dz, float* __restrict__ dz_lo, size_t n,
                                                        int baseline, float inv_batch, double loss_scale,
                                                        double* __restrict__ loss) {
  // fp32 partial sums per thread (a few hundred terms each), double from the block level up
  float local = 0.f;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t nvec = n / 4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float4 d = __ldg(reinterpret_cast<const float4*>(y) + i);
    float4 g = d;
    if (baseline) {
      const float4 tv = __ldg(reinterpret_cast<const float4*>(t) + i);
      d.x -= tv.x; d.y -= tv.y; d.z -= tv.z; d.w -= tv.w;
      g.x = d.x * inv_batch; g.y = d.y * inv_batch; g.z = d.z * inv_batch; g.w = d.w * inv_batch;
    }
    local += 0.5f * (d.x * d.x + d.y * d.y + d.z * d.z + d.w * d.w);
    if (sizeof(TO) == 4) {
      reinterpret_cast<float4*>(dz)[i] = g;
      if (dz_lo) reinterpret_cast<float4*>(dz_lo)[i] = make_float4(tf32_lo(g.x), tf32_lo(g.y), tf32_lo(g.z), tf32_lo(g.w));
    } else {
      __nv_bfloat162 a = __floats2bfloat162_rn(g.x, g.y);
      __nv_bfloat162 b = __floats2bfloat162_rn(g.z, g.w);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&a);
      o.y = *reinterpret_cast<uint32_t*>(&b);
      reinterpret_cast<uint2*>(dz)[i] = o;
    }
  }
  for (size_t i = nvec * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    float d = y[i];
    float g = d;
    if (baseline) {
      d -= t[i];
      g = d * inv_batch;
    }
    local += 0.5f * d * d;
    if (sizeof(TO) == 4) {
      reinterpret_cast<float*>(dz)[i] = g;
      if (dz_lo) dz_lo[i] = tf32_lo(g);
    } else {
      reinterpret_cast<__nv_bfloat16*>(dz)[i] = __float2bfloat16_rn(g);
    }
  }
  __shared__ double red[256];
  red[threadIdx.x] = (double)local;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0) atomicAdd(loss, red[0] * loss_scale);
}

__global__ void __launch_bounds__(256) f32_to_bf16_kernel(const float* __restrict__ src,
                                                          __nv_bfloat16* __restrict__ dst, size_t n) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t nvec = n / 4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float4 v = __ldg(reinterpret_cast<const float4*>(src) + i);
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y);
    __nv_bfloat162 b = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t*>(&a);
    o.y = *reinterpret_cast<uint32_t*>(&b);
    reinterpret_cast<uint2*>(dst)[i] = o;
  }
  for (size_t i = nvec * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = __float2bfloat16_rn(src[i]);
}

__global__ void __launch_bounds__(256) split_lo_kernel(const float* __restrict__ src, float* __restrict__ dst, size_t n) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = tf32_lo(src[i]);
}

__global__ void __launch_bounds__(256) bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ src,
                                                          float* __restrict__ dst, size_t n) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = __bfloat162float(src[i]);
}

// U(lo,hi) from the same counter-based stream as include/b2_rng.h (element i of
// stream `seed`), for the allreduce sweep's device-resident buffers.
template <typename T>
__global__ void __launch_bounds__(256) fill_uniform_kernel(T* __restrict__ buf, size_t n, uint64_t seed,
                                                           float lo, float hi) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const uint64_t s = mix64(seed);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    double u = (double)(mix64(s + i) >> 40) * (1.0 / 16777216.0);
    float v = (float)((double)lo + ((double)hi - (double)lo) * u);
    if (sizeof(T) == 4) reinterpret_cast<float*>(buf)[i] = v;
    else reinterpret_cast<__nv_bfloat16*>(buf)[i] = __float2bfloat16_rn(v);
  }
}

// Order-independent fingerprint of a buffer: the sum of its 32-bit words modulo 2^64
// (exact whatever the order of additions, unlike a floating-point checksum).
__global__ void __launch_bounds__(256) fingerprint_kernel(const uint32_t* __restrict__ words, size_t n,
                                                          unsigned long long* __restrict__ out) {
  unsigned long long local = 0;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) local += words[i];
  __shared__ unsigned long long red[256];
  red[threadIdx.x] = local;
  __syncthreads();
  for (int s = 128; s > 0; s >>= 1) {
    if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
    __syncthreads();
  }
  if (threadIdx.x == 0) atomicAdd(out, red[0]);
}

int grid_for(size_t work_items, int sm_count, int per_sm) {
  size_t blocks = (work_items + 255) / 256;
  size_t cap = (size_t)sm_count * per_sm;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

int device_sms() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

}  // namespace

cudaError_t sgd_launch(float* w, const void* g, int g_type, __nv_bfloat16* w16, size_t n, float lr,
                       int sm_count, cudaStream_t s, float* w_lo) {
  if (n == 0) return cudaSuccess;
  // 8 resident CTAs of 256 threads per SM keep enough 16-byte loads in flight
  int grid = grid_for(n / 4 + 1, sm_count, 8);
  float neg = -lr;
  if (w_lo) {
    sgd_kernel<false, false, true><<<grid, 256, 0, s>>>(w, g, nullptr, w_lo, n, neg);
  } else if (g_type == T_BF16) {
    if (w16) sgd_kernel<true, true, false><<<grid, 256, 0, s>>>(w, g, w16, nullptr, n, neg);
    else sgd_kernel<true, false, false><<<grid, 256, 0, s>>>(w, g, w16, nullptr, n, neg);
  } else {
    if (w16) sgd_kernel<false, true, false><<<grid, 256, 0, s>>>(w, g, w16, nullptr, n, neg);
    else sgd_kernel<false, false, false><<<grid, 256, 0, s>>>(w, g, w16, nullptr, n, neg);
  }
  return cudaGetLastError();
}

cudaError_t split_lo_launch(const float* src, float* dst, size_t n, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  split_lo_kernel<<<grid_for(n, device_sms(), 8), 256, 0, s>>>(src, dst, n);
  return cudaGetLastError();
}

cudaError_t loss_grad_launch(const float* y, const float* target, void* dz, int dz_type, size_t n,
                             int baseline, float inv_batch, double loss_scale, double* loss,
                             cudaStream_t s, float* dz_lo) {
  if (n == 0) return cudaSuccess;
  int grid = grid_for(n / 4 + 1, device_sms(), 8);
  if (dz_type == T_BF16)
    loss_grad_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(y, target, (__nv_bfloat16*)dz, nullptr, n, baseline,
                                                         inv_batch, loss_scale, loss);
  else
    loss_grad_kernel<float><<<grid, 256, 0, s>>>(y, target, (float*)dz, dz_lo, n, baseline, inv_batch,
                                                 loss_scale, loss);
  return cudaGetLastError();
}

cudaError_t convert_f32_to_bf16(const float* src, __nv_bfloat16* dst, size_t n, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  f32_to_bf16_kernel<<<grid_for(n / 4 + 1, device_sms(), 8), 256, 0, s>>>(src, dst, n);
  return cudaGetLastError();
}

cudaError_t convert_bf16_to_f32(const __nv_bfloat16* src, float* dst, size_t n, cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  bf16_to_f32_kernel<<<grid_for(n, device_sms(), 8), 256, 0, s>>>(src, dst, n);
  return cudaGetLastError();
}

cudaError_t fingerprint_launch(const void* buf, size_t bytes, unsigned long long* out, cudaStream_t s) {
  const size_t n = bytes / 4;  // whole 32-bit words (the buffers fingerprinted here are multiples of 4 bytes)
  if (n == 0) return cudaSuccess;
  fingerprint_kernel<<<grid_for(n, device_sms(), 8), 256, 0, s>>>(static_cast<const uint32_t*>(buf), n, out);
  return cudaGetLastError();
}

cudaError_t fill_uniform_launch(void* buf, int type, size_t n, uint64_t seed, float lo, float hi,
                                cudaStream_t s) {
  if (n == 0) return cudaSuccess;
  int grid = grid_for(n, device_sms(), 8);
  if (type == T_BF16)
    fill_uniform_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((__nv_bfloat16*)buf, n, seed, lo, hi);
  else
    fill_uniform_kernel<float><<<grid, 256, 0, s>>>((float*)buf, n, seed, lo, hi);
  return cudaGetLastError();
}

}  // namespace b2

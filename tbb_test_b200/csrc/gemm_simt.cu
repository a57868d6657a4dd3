// CUDA-core GEMM: the fp32 parity path of the training step and the fallback for
// shapes the tensor-core kernel does not take (unaligned leading dimensions, the
// N = 1 tail layer of the reference topology, mlp_bench_common.h:26).
//
// Stands in for the reference's cblas_sgemm calls (mlp_omp.cc:474,566,657):
// C = alpha * op(A) * op(B) + beta * C with fp32 accumulation in k order.
// 128 x 128 x 16 tiles, 256 threads, an 8 x 8 register block per thread.
#include "common.cuh"

namespace b2 {
namespace {

constexpr int BM = 128, BN = 128, BK = 16, NT = 256;

template <typename T>
__device__ __forceinline__ float ldf(const T* p);
template <>
__device__ __forceinline__ float ldf<float>(const float* p) { return __ldg(p); }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}

__device__ __forceinline__ float ldplain(const float* p) { return *p; }
__device__ __forceinline__ float ldplain(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T>
__device__ __forceinline__ void stf(T* p, float v);
template <>
__device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(NT) gemm_simt_kernel(GemmDesc g) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const TI* __restrict__ A = static_cast<const TI*>(g.A);
  const TI* __restrict__ B = static_cast<const TI*>(g.B);
  const int t = threadIdx.x;
  const int tx = t % 16, ty = t / 16;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const bool a_kmajor = (g.sAk == 1), b_kmajor = (g.sBk == 1);

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < g.K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int idx = t + i * NT;
      int mm, kk;
      if (a_kmajor) { kk = idx % BK; mm = idx / BK; } else { mm = idx % BM; kk = idx / BM; }
      int gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < g.M && gk < g.K) ? ldf(A + gm * g.sAm + gk * g.sAk) : 0.f;
      int nn;
      if (b_kmajor) { kk = idx % BK; nn = idx / BK; } else { nn = idx % BN; kk = idx / BN; }
      int gn = n0 + nn;
      gk = k0 + kk;
      Bs[kk][nn] = (gn < g.N && gk < g.K) ? ldf(B + gk * g.sBk + gn * g.sBn) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[8], b[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = As[kk][ty * 8 + i];
#pragma unroll
      for (int j = 0; j < 8; ++j) b[j] = Bs[kk][tx * 8 + j];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

  TO* __restrict__ C = static_cast<TO*>(g.C);
  const TI* __restrict__ X = static_cast<const TI*>(g.aux);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    int gm = m0 + ty * 8 + i;
    if (gm >= g.M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      int gn = n0 + tx * 8 + j;
      if (gn >= g.N) continue;
      float v = g.alpha * acc[i][j];
      TO* c = C + (long long)gm * g.ldc + gn;
      if (g.beta != 0.f) v += g.beta * ldplain(c);
      if (g.epilogue == EPI_RELU) v = v > 0.f ? v : 0.f;
      if (g.epilogue == EPI_MASK) v = ldf(X + (long long)gm * g.ldaux + gn) > 0.f ? v : 0.f;
      stf(c, v);
    }
  }
}

}  // namespace

cudaError_t gemm_simt_launch(const GemmDesc& g, cudaStream_t stream) {
  if (g.M <= 0 || g.N <= 0) return cudaSuccess;
  dim3 grid((g.N + BN - 1) / BN, (g.M + BM - 1) / BM);
  if (g.in_type == T_F32 && g.out_type == T_F32)
    gemm_simt_kernel<float, float><<<grid, NT, 0, stream>>>(g);
  else if (g.in_type == T_BF16 && g.out_type == T_BF16)
    gemm_simt_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, NT, 0, stream>>>(g);
  else if (g.in_type == T_BF16 && g.out_type == T_F32)
    gemm_simt_kernel<__nv_bfloat16, float><<<grid, NT, 0, stream>>>(g);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

}  // namespace b2

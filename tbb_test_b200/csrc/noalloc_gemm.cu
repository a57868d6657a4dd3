// b2_gemm_bf16_noalloc: the bf16 tensor-core GEMM for callers that must not
// allocate device memory.
//
// Who that is: a host program that has handed all device memory to its own pool
// (a framework's caching allocator, an inference server's arena) - a cudaMalloc
// made behind its back by a library can fail outright, fragment the little that
// is left, or block on the implicit device-wide synchronisation cudaMalloc and
// cudaFree carry; and a caller on a latency-critical path that cannot afford that
// synchronisation at all. Such a caller already owns device buffers for the fp32
// operands and the result and only needs the library to bring no allocations of
// its own.
//
// The bf16 GEMM needs scratch memory beyond its inputs and outputs: bf16 copies
// of both fp32 operands (what b2_sgemm_host obtains from cudaMalloc on every call)
// and the status word the tensor-core kernel reports a timed-out wait in. Here
// that scratch is a file-scope __device__ array of fixed size. Consequences the
// caller has to know about:
//   * every GPU that loads this library holds the array (16 MiB + 256 bytes)
//     until the process exits;
//   * operands larger than B2_NOALLOC_MAX_OPERAND_ELEMS elements are refused;
//   * all calls share the one array: two calls whose GPU work overlaps (different
//     streams, different host threads) race on it - serialise them;
//   * the first call on a device looks the array's device address up
//     (cudaGetSymbolAddress, once per device); make that first call outside any
//     stream capture.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>
#include <string>

#include "../../include/b200mlp.h"
#include "common.cuh"

using namespace b2;

namespace {

constexpr size_t kMaxOperandElems = B2_NOALLOC_MAX_OPERAND_ELEMS;
constexpr size_t kStatusBytes = 256;
constexpr size_t kScratchBytes = kStatusBytes + 2 * kMaxOperandElems * sizeof(__nv_bfloat16);

// [0, 256): status word of the tensor-core kernel (cleared before every launch);
// then the bf16 copy of A, then the bf16 copy of B. In host code this name is only a
// handle for cudaGetSymbolAddress - it is not a device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
unsigned char* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;
thread_local std::string g_noalloc_error;

int fail(int code, const char* fmt, const char* detail = "") {
  char buf[320];
  snprintf(buf, sizeof buf, fmt, detail);
  g_noalloc_error = buf;
  return code;
}

// fp32 (rows x cols, leading dimension ld) -> dense bf16 (rows x cols)
__global__ void __launch_bounds__(256) pack_bf16_kernel(const float* __restrict__ src, size_t ld,
                                                        __nv_bfloat16* __restrict__ dst, int rows, int cols) {
  const size_t total = (size_t)rows * cols;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const size_t r = i / cols, c = i % cols;
    dst[i] = __float2bfloat16_rn(src[r * ld + c]);
  }
}

// Device address of the scratch array on the current device (looked up once per device).
int scratch_for_current_device(unsigned char** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(B2_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(B2_ERR_UNSUPPORTED, "device ordinal beyond %s", "63");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_addr[dev]) {
    unsigned char* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p)
      return fail(B2_ERR_CUDA, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return B2_OK;
}

}  // namespace

extern "C" {

const char* b2_noalloc_last_error(void) { return g_noalloc_error.c_str(); }

int b2_gemm_bf16_noalloc(int transa, int transb, int m, int n, int k, const float* a, size_t lda, const float* b,
                         size_t ldb, float* c, size_t ldc, void* stream) {
  if (m < 1 || n < 1 || k < 1 || !a || !b || !c) return fail(B2_ERR_INVALID, "bad GEMM arguments%s");
  const int ar = transa ? k : m, ac = transa ? m : k;
  const int br = transb ? n : k, bc = transb ? k : n;
  if (lda < (size_t)ac || ldb < (size_t)bc || ldc < (size_t)n)
    return fail(B2_ERR_INVALID, "leading dimension smaller than the row length%s");
  if ((size_t)ar * ac > kMaxOperandElems || (size_t)br * bc > kMaxOperandElems) {
    char lim[64];
    snprintf(lim, sizeof lim, "%zu", kMaxOperandElems);
    return fail(B2_ERR_UNSUPPORTED,
                "operand too large for the fixed scratch: each of A and B may hold at most %s elements", lim);
  }
  unsigned char* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc != B2_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned int* status = reinterpret_cast<unsigned int*>(scratch);
  __nv_bfloat16* a16 = reinterpret_cast<__nv_bfloat16*>(scratch + kStatusBytes);
  __nv_bfloat16* b16 = a16 + kMaxOperandElems;

  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;

  GemmDesc d{};
  d.M = m; d.N = n; d.K = k;
  d.A = a16; d.sAm = transa ? 1 : ac; d.sAk = transa ? ac : 1;
  d.B = b16; d.sBk = transb ? 1 : bc; d.sBn = transb ? bc : 1;
  d.C = c; d.ldc = (long long)ldc;
  d.alpha = 1.f; d.beta = 0.f;
  d.epilogue = EPI_NONE;
  d.in_type = T_BF16; d.out_type = T_F32;
  char why[128] = "";
  TcPlan* plan = gemm_tc_plan_create(d, sms, why, sizeof why);  // host-side only: tensor maps, tile choice
  if (!plan) return fail(B2_ERR_UNSUPPORTED, "shape not served by the tensor-core kernel: %s", why);

  cudaError_t e = cudaMemsetAsync(status, 0, sizeof(unsigned int), st);  // the array keeps the last call's contents
  if (e == cudaSuccess) {
    const int grid = sms * 8;
    pack_bf16_kernel<<<grid, 256, 0, st>>>(a, lda, a16, ar, ac);
    pack_bf16_kernel<<<grid, 256, 0, st>>>(b, ldb, b16, br, bc);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = gemm_tc_launch(plan, st, status);
  gemm_tc_plan_destroy(plan);
  if (e != cudaSuccess) return fail(B2_ERR_CUDA, "launch failed: %s", cudaGetErrorString(e));
  unsigned int st_host = 0;
  e = cudaMemcpyAsync(&st_host, status, sizeof st_host, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return fail(B2_ERR_CUDA, "GEMM failed: %s", cudaGetErrorString(e));
  if (st_host != 0) return fail(B2_ERR_TIMEOUT, "tensor-core GEMM gave up waiting on a pipeline barrier%s");
  return B2_OK;
}

}  // extern "C"

// Shared declarations of the b200mlp CUDA sources (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b2 {

enum Epilogue : int {
  EPI_NONE = 0,  // C = alpha * acc (+ beta * C)
  EPI_RELU = 1,  // C = max(acc, 0)                    forward of a hidden layer
  EPI_MASK = 2   // C = aux > 0 ? acc : 0              input gradient through a ReLU
};

enum ElemType : int { T_F32 = 0, T_BF16 = 1 };

// One GEMM, C[M x N] = op(A) * op(B), described by element strides so that the
// three call forms of the training step share every kernel:
//   forward  (NoTrans x Trans)   A(m,k) = A[m*lda + k]   B(k,n) = B[n*ldb + k]
//   wgrad    (Trans   x NoTrans) A(m,k) = A[k*lda + m]   B(k,n) = B[k*ldb + n]
//   dgrad    (NoTrans x NoTrans) A(m,k) = A[m*lda + k]   B(k,n) = B[k*ldb + n]
struct GemmDesc {
  int M, N, K;
  const void* A;
  long long sAm, sAk;
  const void* B;
  long long sBk, sBn;
  void* C;
  long long ldc;
  const void* aux;  // EPI_MASK only, same element type as A/B operands
  long long ldaux;
  float alpha, beta;
  int epilogue;
  int in_type;   // ElemType of A, B and aux
  int out_type;  // ElemType of C
  // Optional stream-K workspace of the tensor-core kernel (null = whole tiles per CTA):
  // TC_WS_SLOT_BYTES per SM and one zero-initialised flag word per SM. GEMMs that share a
  // workspace must not overlap on the GPU.
  float* ws;
  unsigned int* ws_flags;
  // fp32-class tensor-core mode (in_type T_F32 only): low-order twins x - tf32(x) of both
  // operands (same shapes and strides as A and B). With both set the kernel issues three tf32
  // MMAs per k-step (A*B + A*B_lo + A_lo*B), which restores fp32-class accuracy. C_lo (same
  // shape and ldc as C, fp32) receives the twin of the result for the GEMM that reads C next.
  const void* A_lo;
  const void* B_lo;
  void* C_lo;
  // Optional in-kernel timeline of the tensor-core kernel (null = off): CTA 0 stamps %globaltimer
  // per tile into trace[tile * 4 + {0: first MMA issued, 1: accumulator complete (seen by the
  // epilogue), 2: accumulator released, 3: last store of the tile issued}], up to TC_TRACE_TILES tiles.
  // Behind them, for the first TC_TRACE_KBLOCKS k-blocks of CTA 0's second tile: when the MMA warp
  // saw the k-block's operands in shared memory, when the TMA warp saw the k-block's slot free, and
  // (CTA-pair kernel) when the peer CTA's TMA warp saw it free.
  unsigned long long* trace;
};
constexpr int TC_TRACE_TILES = 64;
constexpr int TC_TRACE_KBLOCKS = 64;
constexpr int TC_TRACE_WORDS = TC_TRACE_TILES * 4 + 3 * TC_TRACE_KBLOCKS;
constexpr size_t TC_WS_SLOT_BYTES = 2 * 128 * 256 * sizeof(float);

// CUDA-core GEMM for any shape, stride and alignment (fp32 accumulate).
cudaError_t gemm_simt_launch(const GemmDesc& g, cudaStream_t stream);

// Tensor-core (tcgen05 + TMA + TMEM) GEMM. in_type T_BF16 -> kind::f16 (bf16),
// in_type T_F32 -> kind::tf32. Returns cudaErrorNotSupported when the shape or
// alignment cannot be served (caller falls back to gemm_simt_launch).
// `status` is a device word the kernel sets non-zero if a bounded wait gave up.
struct TcPlan;  // opaque: tensor maps + tile choice for one GEMM site
TcPlan* gemm_tc_plan_create(const GemmDesc& g, int sm_count, char* err, size_t errlen);
void gemm_tc_plan_destroy(TcPlan* p);
// ReLU bit plane of a plan (one bit per element of C, words of 32 columns, ld_words words per
// row): mask_out on a forward plan with the ReLU epilogue, mask_in on an input-gradient plan with
// the mask epilogue (read instead of the activation). False when the plan cannot use one.
bool gemm_tc_plan_set_mask(TcPlan* plan, uint32_t* mask_out, const uint32_t* mask_in, long long ld_words);
cudaError_t gemm_tc_launch(const TcPlan* p, cudaStream_t stream, unsigned int* status);

// Small-message allreduce over peer memory (p2p_allreduce.cu). Every rank's gradient slab and
// flag block are addressable from every rank (peer access within a process, IPC mappings
// between processes). A flag block is 2 * P2P_MAX_RANKS words, written by the peers: word
// P2P_FLAG_ARRIVE + r = "rank r's input of call `epoch` is ready", P2P_FLAG_DONE + r = "rank r's
// stores of call `epoch` are done".
constexpr int P2P_MAX_RANKS = 8;
constexpr int P2P_FLAG_ARRIVE = 0;
constexpr int P2P_FLAG_DONE = P2P_MAX_RANKS;
constexpr size_t P2P_FLAG_BYTES = 2 * P2P_MAX_RANKS * sizeof(unsigned int);
struct P2pParams {
  float* slab[P2P_MAX_RANKS];          // index = rank; slab[rank] is this rank's own
  unsigned int* flags[P2P_MAX_RANKS];  // index = rank
  int world, rank;
  unsigned long long offset;  // first element of the message in every slab (multiple of 4)
  unsigned long long count;   // elements
  unsigned int epoch;         // call counter, > 0, the same on every rank for the same call
  unsigned int* ctas_done;    // this rank's own counter, zero between calls
  unsigned int* status;       // this rank's own word, set non-zero when a wait gave up
  unsigned long long wait_ns; // how long a flag wait may last before the rank gives up
};
// One rank's launch (every rank launches its own, each on its own GPU).
cudaError_t p2p_allreduce_launch(const P2pParams& p, int cta_limit, cudaStream_t stream);
// All ranks in one cooperative launch on one GPU: `ranks_dev` = device array of world entries.
cudaError_t p2p_allreduce_emulated_launch(const P2pParams* ranks_dev, const P2pParams& any_rank, cudaStream_t stream);

// Element-wise kernels.
cudaError_t convert_f32_to_bf16(const float* src, __nv_bfloat16* dst, size_t n, cudaStream_t s);
cudaError_t convert_bf16_to_f32(const __nv_bfloat16* src, float* dst, size_t n, cudaStream_t s);
// dz = y (ref) or (y - t) * inv_batch (baseline); loss += 0.5 * sum(d^2) * loss_scale
cudaError_t loss_grad_launch(const float* y, const float* target, void* dz, int dz_type, size_t n,
                             int baseline, float inv_batch, double loss_scale, double* loss,
                             cudaStream_t s, float* dz_lo = nullptr);
// w = fma(-lr, g, w); optional bf16 copy of the new weights, optional low-order twin w - tf32(w)
cudaError_t sgd_launch(float* w, const void* g, int g_type, __nv_bfloat16* w_bf16, size_t n, float lr,
                       int sm_count, cudaStream_t s, float* w_lo = nullptr);
// *out += sum of the 32-bit words of buf modulo 2^64 (out must be zeroed by the caller)
cudaError_t fingerprint_launch(const void* buf, size_t bytes, unsigned long long* out, cudaStream_t s);
// dst = src - tf32(src): the part of an fp32 value the tensor core drops when it reads it as tf32
cudaError_t split_lo_launch(const float* src, float* dst, size_t n, cudaStream_t s);
cudaError_t fill_uniform_launch(void* buf, int type, size_t n, uint64_t seed, float lo, float hi,
                                cudaStream_t s);

}  // namespace b2

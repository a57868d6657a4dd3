/* b200mlp: C ABI of the B200 (sm_100a) implementation of the MLP training step
 * benchmarked by jspark1105/tbb_test (mlp_omp.cc / mlp_tbb.cc).
 *
 * The reference has no FFI layer: its hot path is reached at source level from
 * main() (mlp_omp.cc:375-750) through the globals of mlp_bench_common.h:53-55.
 * Each entry point below replaces one phase of that main; the citation names the
 * reference code it stands in for.  One handle drives one GPU (the reference's
 * "socket"); a data-parallel job creates one handle per GPU, in one process or in
 * one process per GPU, all with the same configuration except `rank`/`device`.
 *
 * Conventions: plain pointers and sizes only; host matrices are row-major with a
 * caller-given leading dimension in ELEMENTS (the reference's Matrix has
 * ld = ncols + 16, Matrix.h:148); every function returns a b2_status (0 = ok,
 * negative = error, b2_last_error() gives the text) and never exits or throws
 * (the reference asserts or calls exit(-1), mlp_omp.cc:368).  There is no CPU
 * fallback: without a usable CUDA device b2_create fails.
 */
#ifndef B200MLP_H
#define B200MLP_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct b2_handle b2_handle;

typedef enum {
  B2_OK = 0,
  B2_ERR_INVALID = -1,     /* bad argument or shape */
  B2_ERR_CUDA = -2,        /* a CUDA runtime/driver call failed */
  B2_ERR_NCCL = -3,        /* NCCL missing or a collective failed */
  B2_ERR_UNSUPPORTED = -4, /* valid request this build cannot serve */
  B2_ERR_TIMEOUT = -5,     /* a bounded device-side wait gave up */
  B2_ERR_STATE = -6        /* call made in the wrong state */
} b2_status;

/* What the step computes. */
typedef enum {
  B2_MODE_REF = 0,     /* the C++ reference as written: no ReLU, dZ[L-1] = A[L]
                          (mlp_omp.cc:565,655), no 1/B scaling */
  B2_MODE_BASELINE = 1 /* ReLU between layers, dZ[L-1] = (A[L]-T)/B_global
                          (c2_bench/mlp_caffe2.py:208-235) */
} b2_mode;

/* Arithmetic of the three GEMMs; accumulation is fp32 and the master weights and
 * the SGD update are fp32 in every case. */
typedef enum {
  B2_PREC_FP32 = 0, /* fp32 operands, CUDA-core FMA (parity mode) */
  B2_PREC_TF32 = 1, /* fp32 storage, tcgen05 kind::tf32 */
  B2_PREC_BF16 = 2, /* bf16 operands (activations, gradients, a bf16 weight copy),
                       tcgen05 kind::f16 */
  B2_PREC_FP32_TC = 3 /* fp32 storage and fp32-class results on the tensor cores: every operand x
                       is kept with its low-order twin x - tf32(x), and each k-step issues three
                       kind::tf32 MMAs (A*B + A*B_lo + A_lo*B) into the same fp32 accumulator;
                       same tolerance class as B2_PREC_FP32 (the reference's sgemm), about a
                       third of the TF32 rate */
} b2_precision;

typedef enum { B2_DTYPE_F32 = 0, B2_DTYPE_BF16 = 1 } b2_dtype;

/* Replaces the compile-time model of mlp_bench_common.h:26-38 and the argv of
 * mlp_omp.cc:376-386. Fill with b2_config_default() first. */
typedef struct {
  int nlayers;              /* number of fully-connected layers L */
  const int* nfeatures;     /* L+1 widths F_0..F_L (mlp_bench_common.h:26) */
  int batch;                /* GLOBAL batch, split over ranks like
                               get_partition(batch, rank, 1, 0) (Partition.cc:34-51) */
  int rank;                 /* this handle's shard, 0 <= rank < world_size  (socket id) */
  int world_size;           /* number of GPUs in the job                   (nsockets) */
  int device;               /* CUDA device ordinal */
  int mode;                 /* b2_mode */
  int precision;            /* b2_precision */
  int grad_bf16;            /* 1: weight gradients are produced, summed and read in bf16
                               (BF16 precision only) */
  int allreduce;            /* 0 = the reference's NO_ALL_REDUCE build (mlp_omp.cc:21) */
  int overlap;              /* 1 = allreduce/update on a side stream, overlapped with the
                               remaining backward GEMMs (OVERLAP_ALL_REDUCE, mlp_omp.cc:23) */
  int input_grad;           /* 1 = also compute dA[0] like the reference (mlp_omp.cc:656) */
  int collect_timing;       /* 1 = per-phase CUDA-event timing (sum_times, mlp_bench_common.h:35) */
  int use_graph;            /* 1 = replay each step as one CUDA graph (refused with B2_ERR_UNSUPPORTED
                               when world_size > 1 and allreduce = 1) */
  int force_simt;           /* 1 = never use the tensor-core kernels (debugging aid) */
  int comm_sms;             /* SMs the persistent GEMM kernels leave free for the collective's CTAs
                               while allreduce and GEMMs overlap (the counterpart of the threads the
                               reference takes away from the GEMMs, mlp_bench_common.h:40-48);
                               -1 = default: 20 on 4 or more GPUs, 0 otherwise */
  int ar_bucket_mb;         /* gradient allreduce granularity: 0 = one collective per layer, issued as
                               soon as that layer's weight gradient is done (what the reference does per
                               layer, mlp_omp.cc:692-705); N > 0 = consecutive layers are summed
                               together once they add up to N MiB; -1 = default: the first collective
                               takes about a quarter of all gradient bytes (large messages use NVLink
                               far better) and, with 4 or more GPUs, each later one 1.5 times the
                               bytes of the one before (the sums then limit the step, so the first
                               should start early and the rest be few) */
  int shard_update;         /* how the summed gradient reaches the weights on 2 or more GPUs:
                               1 = like the reference (mlp_omp.cc:90-146, 240-258): reduce-scatter of each
                               gradient bucket, SGD on the 1/world slice of the weights this rank owns,
                               allgather of the updated weights (of their bf16 operand copy in BF16
                               precision: 25 % fewer bytes on the wire, and only the owner keeps that
                               slice's fp32 master weights current until b2_download_weights or
                               b2_allreduce_sgd gathers them, which makes those two calls collective);
                               0 = allreduce, then every rank updates all weights; -1 = default: 1 */
  float lr;                 /* SGD step (the reference hard-codes 1e-10, mlp_omp.cc:609) */
  const void* nccl_unique_id; /* B2_NCCL_ID_BYTES bytes from b2_nccl_unique_id(), shared by all
                                 ranks; NULL when world_size == 1 */
} b2_config;

#define B2_NCCL_ID_BYTES 128

/* Phases of the step, in the order of the reference's Breakdown enum
 * (mlp_bench_common.h:12-20). */
enum { B2_T_FWD = 0, B2_T_WGT_GRAD = 1, B2_T_BWD = 2, B2_T_WGT_UPDATE = 3,
       B2_T_ALLREDUCE = 4, /* gradient allreduce, or reduce-scatter with shard_update (WGT_UPDATE_REDUCE_SCATTER) */
       B2_T_ALLGATHER = 5, /* allgather of the updated weights with shard_update (WGT_UPDATE_ALLGATHER) */
       B2_T_NUM = 6 };

/* Defaults: mode BASELINE, precision FP32, world 1, allreduce/overlap/input_grad on, comm_sms -1. */
int b2_config_default(b2_config* cfg);

/* Library version string and the CUDA architecture it was built for. */
const char* b2_version(void);

/* Root rank: create the id every rank passes in b2_config.nccl_unique_id. One id
 * founds one communicator: every set of handles created together needs a fresh id. */
int b2_nccl_unique_id(void* out_bytes);

/* Allocation phase of main (mlp_omp.cc:390-409): device buffers for weights,
 * gradients and activations of this rank's batch shard, streams, events and the
 * communicator. */
int b2_create(const b2_config* cfg, b2_handle** out);
int b2_destroy(b2_handle* h);

/* Text of the last error recorded on the handle (or on the calling thread when
 * h is NULL, e.g. after a failed b2_create). */
const char* b2_last_error(const b2_handle* h);

/* Rows [begin,end) of the global batch this handle owns (Partition.cc:34-51). */
int b2_batch_range(const b2_handle* h, int* begin, int* end);

/* init_matrices (mlp_bench_common.cc:16-33): weights[l] replica rows, F_{l+1} x F_l.
 * With shard_update in BF16 precision b2_download_weights is collective after steps have run:
 * every rank has to call it (for the same layers in the same order), because each rank holds
 * current fp32 master weights only for the slices it owns and the call gathers them first. */
int b2_upload_weights(b2_handle* h, int layer, const float* host, size_t ld);
int b2_download_weights(b2_handle* h, int layer, float* host, size_t ld);
/* activations[0] (mlp_bench_common.cc:18) and the +-1 targets of BASELINE mode.
 * `host` is the GLOBAL batch x F matrix; the handle copies its own rows. */
int b2_upload_input(b2_handle* h, const float* host, size_t ld);
int b2_upload_target(b2_handle* h, const float* host, size_t ld);

/* Parity taps. `host` is the GLOBAL batch x F matrix; only this handle's rows are
 * written. Activation l in [0,L]; dz l in [0,L-1] is the gradient w.r.t. layer l's
 * output (what the reference leaves in activations[l+1], mlp_omp.cc:655-671). */
int b2_download_activation(b2_handle* h, int layer, float* host, size_t ld);
int b2_download_dz(b2_handle* h, int layer, float* host, size_t ld);
int b2_download_input_grad(b2_handle* h, float* host, size_t ld);
/* weight_grads[l] (mlp_omp.cc:579): this rank's gradient, after the allreduce if
 * one has run. */
int b2_download_weight_grad(b2_handle* h, int layer, float* host, size_t ld);
int b2_upload_weight_grad(b2_handle* h, int layer, const float* host, size_t ld);

int b2_set_lr(b2_handle* h, float lr);

/* The loop body of mlp_omp.cc:435-737, `iters` times: forward GEMMs, output
 * gradient, then per layer (last to first) weight-gradient GEMM, gradient
 * allreduce + SGD on the side stream, input-gradient GEMM. Returns after both
 * streams have drained. */
int b2_step(b2_handle* h, int iters);

/* One step fed from host memory: uploads this rank's rows of `x` (and `t`),
 * runs b2_step(h, 1) and returns this rank's share of the loss
 * (0.5*sum((Y-T)^2)/B_global, or 0.5*sum(Y^2) in REF mode). Pinned host memory
 * (b2_host_alloc) makes the copies asynchronous. */
int b2_train_step_host(b2_handle* h, const float* x, size_t ldx, const float* t, size_t ldt,
                       double* loss);
/* Pipelined form of the same call for input streams: enqueues the copy of this
 * step's inputs (on a copy stream, into one of two input slots) and the step, and
 * returns without waiting, so that the copy of step i+1 overlaps the compute of
 * step i. At most two steps may be in flight; b2_wait_loss() blocks until the
 * oldest one has finished and returns its loss share. `x` and `t` must stay valid
 * and unchanged until that step's b2_wait_loss() returns, and should be pinned.
 * Needs collect_timing = 0 and use_graph = 0. The reference has no counterpart
 * (its inputs never change, mlp_bench_common.cc:18); this is the form a data-loader
 * driven caller of the training step uses. */
int b2_train_step_host_async(b2_handle* h, const float* x, size_t ldx, const float* t, size_t ldt);
int b2_wait_loss(b2_handle* h, double* loss);
/* Loss of the most recent step (this rank's share). */
int b2_loss(b2_handle* h, double* loss);

int b2_host_alloc(void** ptr, size_t bytes); /* pinned host memory */
/* Pinned host memory on the NUMA node the GPU `device` hangs off, the counterpart of
 * create_matrix_with_numa_aware_allocation (mlp_omp.cc:27-47), which binds each socket's
 * matrices to that socket's node. The node and its CPUs are read from sysfs
 * (/sys/bus/pci/devices/<bus id>/numa_node, /sys/devices/system/node/node<N>/cpulist); the
 * calling thread runs on those CPUs while the pages are allocated and touched, then gets its
 * affinity back. *numa_node (optional) receives the node, or -1 when the system does not tell
 * (no sysfs entry, a single node, no allowed CPU on that node): the call then behaves like
 * b2_host_alloc. Freed by b2_host_free. */
int b2_host_alloc_near(void** ptr, size_t bytes, int device, int* numa_node);
int b2_host_free(void* ptr);

/* The three cblas_sgemm call sites (mlp_omp.cc:474,566,657) with cblas argument
 * meaning, row-major, on HOST matrices (copied in and out): C = op(A)*op(B) in the
 * given b2_precision, optional fused ReLU (epilogue 1) or mask by aux>0
 * (epilogue 2, aux is m x n with leading dimension ldaux). */
int b2_sgemm_host(b2_handle* h, int precision, int transa, int transb, int m, int n, int k,
                  const float* a, size_t lda, const float* b, size_t ldb, float* c, size_t ldc,
                  int epilogue, const float* aux, size_t ldaux);
/* Same on fp32 DEVICE pointers of this handle's GPU, alpha/beta like cblas
 * (FP32 precision: any alpha/beta; TF32: beta must be 0; FP32_TC is served by
 * b2_sgemm_host only, which has room for the operand twins). Asynchronous on the
 * handle's main stream; b2_sync() waits. */
int b2_sgemm(b2_handle* h, int precision, int transa, int transb, int m, int n, int k, float alpha,
             const float* a, size_t lda, const float* b, size_t ldb, float beta, float* c,
             size_t ldc);
int b2_sync(b2_handle* h);

/* No counterpart in the reference. The bf16 tensor-core GEMM (same call meaning as
 * b2_sgemm, alpha = 1, beta = 0) on fp32 DEVICE operands, for callers that must not
 * allocate device memory: programs that gave all of it to their own pool, where a
 * library's cudaMalloc can fail or stall, and latency-critical paths that cannot take
 * the device-wide synchronisation cudaMalloc/cudaFree imply. It needs no handle and
 * calls no cudaMalloc/cudaFree: the bf16 operand copies and the kernel's status word
 * live in a fixed __device__ array of 16 MiB + 256 bytes that every GPU loading the
 * library holds until the process exits. Limits: op(A) and op(B) may each hold at most
 * B2_NOALLOC_MAX_OPERAND_ELEMS elements. `a` and `b` need no alignment (they are repacked
 * into the scratch), but the packed copies must be addressable by TMA: the number of
 * COLUMNS of each matrix as stored (k for a non-transposed A, m for a transposed one; n for
 * a non-transposed B, k for a transposed one) must be a multiple of 8, `c` must be 16-byte
 * aligned with ldc a multiple of 4, and n at least 16. A call outside these limits returns
 * B2_ERR_UNSUPPORTED with the reason in b2_noalloc_last_error(). The array is shared by all
 * calls and keeps the previous call's contents: calls whose GPU work overlaps race.
 * The first call on a device looks up the array's address and should be made outside
 * stream capture. `stream` is a cudaStream_t (NULL = default stream); the call returns
 * after the result is in `c`. b2_noalloc_last_error() has the text of a failure. */
#define B2_NOALLOC_MAX_OPERAND_ELEMS (4u * 1024u * 1024u)
int b2_gemm_bf16_noalloc(int transa, int transb, int m, int n, int k, const float* a, size_t lda,
                         const float* b, size_t ldb, float* c, size_t ldc, void* stream);
const char* b2_noalloc_last_error(void);

/* update_weight (mlp_omp.cc:297-323) on layer `l`: sum weight_grads[l] over all
 * ranks, then w = fma(-lr, sum, w). The reference's known-answer test
 * (mlp_omp.cc:325-373) runs through this call. With shard_update it takes the reference's
 * own route: reduce-scatter, SGD on the owned slice, allgather of the weights. */
int b2_allreduce_sgd(b2_handle* h, int layer);

/* In-place sum over all ranks of `count` elements of `dtype` (b2_dtype) at the DEVICE pointer
 * `dev_buf` of this handle's GPU, through the handle's communicator on its main stream;
 * returns after the result is there. The gradient-allreduce sweep on caller-owned buffers
 * (the reference sums caller-owned Matrix buffers, update_weight(Matrix*, ...), mlp_omp.cc:297);
 * with one rank the buffer is left as it is. */
int b2_allreduce(b2_handle* h, void* dev_buf, size_t count, int dtype);

/* Gradient-allreduce sweep: sums `count` elements of `dtype` filled with
 * U(-1,1) from seed = rank across all ranks, `iters` timed repetitions after
 * `warmup`; *ms_per_iter is the device time of one allreduce on this rank and
 * checksum (optional) the sum of the first min(count,4096) result elements. */
int b2_allreduce_bench(b2_handle* h, size_t count, int dtype, int warmup, int iters,
                       double* ms_per_iter, double* checksum);
/* The same sweep for each of the three collectives of the step: kind 0 = allreduce, 1 =
 * reduce-scatter (mlp_omp.cc:56-169: each rank ends with the sum of its 1/world slice), 2 =
 * allgather (mlp_omp.cc:171-295 after its SGD: each rank's slice to all); `count` is the whole
 * buffer in elements and must divide by the number of ranks for kinds 1 and 2. */
int b2_collective_bench(b2_handle* h, int kind, size_t count, int dtype, int warmup, int iters,
                        double* ms_per_iter, double* checksum);

/* The SGD kernel alone on `nparams` parameters (w = fma(-lr, g, w), gradients of grad_dtype,
 * optionally also writing the bf16 operand copy), on parameter sets used in rotation that
 * together exceed the L2 several times: *ms_per_iter = device time of one launch,
 * *bytes_per_iter = the algorithmic bytes it moves (read w, read g, write w, write copy). */
int b2_sgd_bench(b2_handle* h, size_t nparams, int grad_dtype, int with_bf16_copy, int warmup, int iters,
                 double* ms_per_iter, double* bytes_per_iter);

/* Switches the per-phase event timing of b2_step (b2_config.collect_timing) on or off. */
int b2_set_timing(b2_handle* h, int collect_timing);

/* Order-independent fingerprint (sum of the 32-bit words modulo 2^64) of layer l's weights as
 * the next forward pass reads them (the bf16 operand copy in BF16 precision, the fp32 weights
 * otherwise): equal on every rank of a data-parallel job exactly when the replicas hold the
 * same bits. The device counterpart of comparing print_checksum lines by eye
 * (mlp_bench_common.cc:152-168). */
int b2_weights_fingerprint(b2_handle* h, int layer, unsigned long long* fingerprint);

/* One GEMM of the step alone, for roofline measurements per call form and shape: form 0 = forward
 * (mlp_omp.cc:474-488: A m x k, B n x k), 1 = weight gradient (:565-580: A stored k x m, B stored
 * k x n), 2 = input gradient (:655-671: A m x k, B k x n); `precision`, `epilogue` and the output
 * type as in the step (out_dtype a b2_dtype; bf16 output needs BF16 precision); sms = number of SMs
 * the persistent tensor-core grid may use (0 = all). Operands are seeded U(-1,1) device buffers,
 * as many sets as it takes to exceed the L2 several times over, used in rotation so that every
 * launch reads its operands from HBM like the launches of a step do. *ms_per_iter = device time
 * of one launch (CUDA events around `iters` back-to-back launches after `warmup`). */
int b2_gemm_bench(b2_handle* h, int form, int m, int n, int k, int precision, int epilogue, int out_dtype,
                  int sms, int warmup, int iters, double* ms_per_iter);

/* Peer-memory path for small gradient messages (the 1 MiB layers of the deep narrow
 * configuration, where a library collective is latency-bound). The reference moves its
 * gradients between sockets by plain loads and stores to the other sockets' buffers
 * (mlp_omp.cc:94-160); this is the same idea between GPUs over NVLink: each rank sums the
 * chunk it owns straight out of every rank's gradient buffer, in rank order, and stores the
 * sum into every rank's buffer, with two bounded flag exchanges per call.
 *   1. every rank: b2_p2p_describe(h, desc)            B2_P2P_DESC_BYTES bytes
 *   2. exchange the descriptors between the ranks (threads: an array; processes: any transport)
 *   3. every rank: b2_p2p_connect(h, all_descs, max_bytes) with all_descs in rank order
 * From then on gradient sums of at most max_bytes (fp32 gradients, no graph replay) bypass
 * NCCL; larger ones still use it. All ranks must pass the same max_bytes, and none may destroy
 * its handle while another still runs steps. A rank that waits longer than the wait limit (one
 * second unless b2_p2p_set_wait_ms changed it; the reference spins without a limit,
 * mlp_omp.cc:120-121,267-268) for another gets B2_ERR_TIMEOUT from its next synchronising call
 * (b2_step, b2_sync, b2_allreduce_sgd, b2_wait_loss) and falls back to NCCL-only; the peer
 * launches still queued behind the one that gave up return at once. */
#define B2_P2P_DESC_BYTES 128
int b2_p2p_describe(b2_handle* h, void* desc);
int b2_p2p_connect(b2_handle* h, const void* descs, size_t max_bytes);
/* How long one flag wait of the peer-memory path may last, 1 .. 60000 ms (default 1000). Ranks
 * that reach a gradient sum further apart than this (first-call module loads, a slow host
 * thread) time out, so embedders with loosely coupled ranks raise it. */
int b2_p2p_set_wait_ms(b2_handle* h, int ms);
/* The same kernel with all `world` ranks emulated on ONE GPU (one cooperative launch; for
 * machines with fewer GPUs than ranks): bufs[r] = rank r's `count` host floats, replaced by the
 * sum over ranks. No handle needed. The reference has no counterpart. */
int b2_p2p_emulate(int device, int world, float* const* bufs, size_t count);
/* Same with a chosen wait limit and, when lagging_rank >= 0, with that rank one call behind
 * the others, so that every wait on it runs out: the call then returns B2_ERR_TIMEOUT after
 * about two wait limits and leaves bufs untouched (how a lost rank looks to the others, made
 * on the host side without any fault on the device). lagging_rank = -1: no rank lags. */
int b2_p2p_emulate_opts(int device, int world, float* const* bufs, size_t count, int wait_ms,
                        int lagging_rank);

/* Device times in milliseconds accumulated since the last reset:
 * phase_ms[l * B2_T_NUM + phase] per layer (needs collect_timing), and
 * *step_ms / *steps for whole steps (always collected). Feeds report_timing
 * (mlp_bench_common.cc:38-150). Pointers may be NULL. */
int b2_get_timing(b2_handle* h, double* phase_ms, double* step_ms, long long* steps);
/* Milliseconds since the last reset during which at least one GEMM of the steps was running
 * (needs collect_timing). The weight-gradient GEMMs run next to the input-gradient GEMMs on a
 * second stream, so the per-phase sums of b2_get_timing count overlapped time twice; a GEMM
 * rate is flops / this number. */
int b2_get_gemm_busy_ms(b2_handle* h, double* ms);
int b2_reset_timing(b2_handle* h);
/* Chrome-trace ("trace event") JSON of the most recent b2_step call made with collect_timing:
 * one complete event per layer and phase, pid = rank, tid = stream (0 main, 1 weight-gradient
 * stream, 2 side stream). Same idea as the reference's COLLECT_TRACE dump (mlp_tbb.cc:82-108,
 * 1378-1392), with GPUs for sockets and streams for threads. */
int b2_write_trace(b2_handle* h, const char* path);

/* Which kernel serves the GEMM sites of the step (three per layer, plus the second input slot's):
 * in the tensor-core precisions a site whose shape or alignment the tensor-core kernel cannot
 * address (a leading dimension that is not a multiple of 16 bytes, fewer than 16 output columns,
 * such as the 1-wide tail layer of the reference's topology, mlp_bench_common.h:26) falls to the
 * CUDA-core kernel, about 30 times slower. The counts and the reason given for the first such
 * site make that visible; with B2_VERBOSE set in the environment it is also printed once. */
int b2_site_report(const b2_handle* h, int* tensor_core_sites, int* cuda_core_sites, char* first_reason,
                   size_t reason_len);

/* Number of kernels of this library launched on the handle since creation, and
 * how many of them were tensor-core (tcgen05) GEMMs. */
int b2_launch_counts(const b2_handle* h, long long* total, long long* tensor_core);

#ifdef __cplusplus
}
#endif
#endif /* B200MLP_H */

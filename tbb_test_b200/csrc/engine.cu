// Handle, step schedule and C ABI of b200mlp (see include/b200mlp.h).
//
// One handle = one GPU = one "socket" of the reference.  The step mirrors the loop
// body of mlp_omp.cc:435-737 and the dependency graph of mlp_tbb.cc:1288-1367:
//
//   main stream   fwd(0) .. fwd(L-1), output gradient,
//                 then for l = L-1 .. 0:  wgrad(l), dgrad(l)
//   side stream   for l = L-1 .. 0:  [after wgrad(l)] allreduce(dW[l]),
//                 [after dgrad(l), which still reads W[l]] SGD(l)
//
// and fwd(l) of the next step waits for SGD(l) only, so the reduction and update of
// a layer overlap the backward GEMMs of the layers below it and, for the first
// layers, the start of the next forward pass (the reference overlaps the same way
// by dedicating threads: mlp_omp.cc:520-527,601-615,692-723).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <sched.h>
#include <unistd.h>

#include <algorithm>
#include <cctype>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/b200mlp.h"
#include "bucket_plan.h"
#include "common.cuh"
#include "nccl_dyn.h"

using namespace b2;

namespace {

thread_local std::string g_tls_error;

struct Site {
  GemmDesc d;
  TcPlan* plan = nullptr;  // null: CUDA-core kernel
  bool active = false;
};

}  // namespace

struct b2_handle {
  b2_config cfg;
  std::vector<int> nf;
  int L = 0, b0 = 0, b1 = 0, bl = 0, sms = 148;
  int gemm_sms = 148;  // SMs the persistent GEMM kernels of the step occupy (sms - comm_sms)
  int op_type = T_F32;    // element type of GEMM operands held on the device
  int grad_type = T_F32;  // element type of dW
  cudaStream_t s_main = nullptr, s_comm = nullptr;
  // Weight-gradient GEMMs run on a stream of their own next to the input-gradient chain:
  // both are persistent kernels, so the CTAs of one start on the SMs the other's last,
  // partial wave leaves idle instead of waiting for the whole kernel to drain.
  cudaStream_t s_wg = nullptr;
  cudaStream_t s_upd = nullptr;  // SGD updates: off the collective's stream so that the next bucket's sum starts at once
  cudaEvent_t ev_join_upd = nullptr;
  std::vector<cudaEvent_t> ev_ar;  // per layer that closes a bucket: its allreduce is done
  cudaEvent_t ev_dz_last = nullptr;
  bool wg_stream = false;
  // Weights live in slabs laid out like the gradient slab (same element offsets), so that a
  // bucket of consecutive layers is one contiguous range in all three: the reduce-scatter of
  // the gradients, the SGD of the owned slice and the allgather of the weights each take one call.
  float* w_slab = nullptr;
  __nv_bfloat16* w16_slab = nullptr;
  std::vector<float*> w;             // w_slab + dw_off[l]
  std::vector<__nv_bfloat16*> w16;   // w16_slab + dw_off[l]
  // fp32-class tensor-core mode (B2_PREC_FP32_TC): low-order twins x - tf32(x) of every GEMM
  // operand, produced where the operand itself is produced (uploads, GEMM epilogues, the
  // output-gradient kernel, SGD)
  bool x3 = false;
  float* w_lo_slab = nullptr;
  std::vector<float*> w_lo, act_lo, dz_lo;
  float* act0_alt_lo = nullptr;
  // B2_NCCL_UB=1 (2 or more GPUs): the gradient and weight slabs come from ncclMemAlloc and are
  // registered with the communicator, so that its collectives run on them in place
  bool nccl_ub = false;
  void* ub_handle[3] = {nullptr, nullptr, nullptr};
  bool ag_deferred = true;     // allgathers behind all reduce-scatters of a step, lowest bucket first
  bool ag_grouped = false;     // B2_AG_ORDER=grouped: each allgather in one NCCL group with the next reduce-scatter
  bool shard = false;          // reduce-scatter + owned-slice SGD + allgather instead of allreduce + full SGD
  bool masters_stale = false;  // BF16 precision with shard: ranks hold current fp32 masters only for their slices
  std::vector<size_t> dw_pad;  // padded element count of layer l in the slabs (multiple of 128 * world)
  std::vector<char> bucket_full;  // for the layer closing a bucket: 1 = this bucket is summed in full on every rank
  std::vector<cudaEvent_t> ev_shard;  // per bucket-closing layer: owned-slice SGD done
  std::vector<void*> dw, act, dz;
  // ReLU bit planes (BASELINE mode, tensor-core kernels): relu_bits[l] holds one bit per element
  // of act[l], l = 1 .. L-1, written by the forward epilogue of layer l-1 and read by the
  // input-gradient epilogue of layer l in place of the activation (1/16 of its bytes)
  std::vector<uint32_t*> relu_bits;
  // All weight gradients live in one slab, last layer first (the order backward produces
  // them), so that consecutive layers can be summed by one collective call ("bucket").
  void* dw_slab = nullptr;
  // Peer-memory path for small gradient messages (b2_p2p_connect): every rank's slab and the
  // flag block at its end are mapped here; messages up to p2p_max_bytes bypass NCCL.
  size_t slab_bytes = 0, p2p_flags_off = 0;
  bool p2p_ready = false;
  size_t p2p_max_bytes = 0;
  unsigned int p2p_epoch = 0;
  unsigned long long p2p_wait_ns = 1000000000ull;  // b2_p2p_set_wait_ms
  unsigned int* p2p_ctas_done = nullptr;
  float* p2p_slab[P2P_MAX_RANKS] = {};
  unsigned int* p2p_flags[P2P_MAX_RANKS] = {};
  void* p2p_opened[P2P_MAX_RANKS] = {};  // IPC mappings of other processes' slabs
  std::vector<size_t> dw_off;       // element offset of dw[l] in the slab
  std::vector<int> bucket_low;      // for layer l: lowest layer index of its bucket
  std::vector<int> bucket_high;     // for layer l: highest layer index of its bucket
  float* y = nullptr;
  float* target = nullptr;
  void* dinput = nullptr;
  float* stage = nullptr;  // fp32 staging for converted up/downloads
  size_t stage_elems = 0;
  double* loss_dev = nullptr;  // [2]: one accumulator per input slot
  unsigned int* status_dev = nullptr;
  unsigned long long* fp_dev = nullptr;  // accumulator of b2_weights_fingerprint
  float* tc_ws = nullptr;           // stream-K workspace shared by this handle's GEMMs (they
  unsigned int* tc_ws_flags = nullptr;  // all run on the main stream, one after the other)
  std::vector<cudaEvent_t> ev_wgrad, ev_dgrad, ev_upd;
  std::vector<char> upd_pending;
  cudaEvent_t ev_t0 = nullptr, ev_t1 = nullptr, ev_join = nullptr, ev_fork = nullptr;
  std::vector<cudaEvent_t> ev_phase;  // [iters][L][B2_T_NUM][2], alive during one b2_step call
  int ev_iter = 0;                    // step of the current call the recorder is in
  std::vector<Site> fwd, wgrad, dgrad;
  // second input slot of the pipelined host-fed path (b2_train_step_host_async): while a
  // step computes on slot 0 the next step's inputs are copied into slot 1 and vice versa
  void* act0_alt = nullptr;
  float* target_alt = nullptr;
  float* xstage[2] = {nullptr, nullptr};  // fp32 landing buffers when the operands are bf16
  Site fwd0_alt, wgrad0_alt;
  cudaStream_t s_copy = nullptr;
  cudaEvent_t ev_copied[2] = {nullptr, nullptr}, ev_slot_free[2] = {nullptr, nullptr},
              ev_loss[2] = {nullptr, nullptr};
  bool slot_used[2] = {false, false};
  double* loss_host = nullptr;  // pinned, one value per slot
  long long async_issued = 0, async_waited = 0;
  ncclComm_t comm = nullptr;
  std::vector<double> phase_ms;
  struct TraceEvent {
    int step, layer, phase;
    float start_ms, dur_ms;  // relative to the start of the b2_step call
  };
  std::vector<TraceEvent> trace;  // phases of the most recent timed b2_step call
  double gemm_busy_ms = 0;        // time during which at least one GEMM of the step was running
  double step_ms = 0;
  long long steps = 0, launches = 0, tc_launches = 0;
  cudaGraphExec_t graph_exec = nullptr;
  int tensor_core_sites = 0, cuda_core_sites = 0;  // GEMM sites of the step by the kernel that serves them
  std::string cuda_core_reason;                    // why the first refused site was refused
  std::string err;
};

namespace {

int fail(b2_handle* h, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (h) h->err = buf;
  g_tls_error = buf;
  return code;
}

#define CK(h, call)                                                                              \
  do {                                                                                           \
    cudaError_t e_ = (call);                                                                     \
    if (e_ != cudaSuccess)                                                                       \
      return fail(h, B2_ERR_CUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, \
                  __LINE__);                                                                     \
  } while (0)

#define NCK(h, call)                                                                         \
  do {                                                                                       \
    int r_ = (call);                                                                         \
    if (r_ != ncclSuccess)                                                                   \
      return fail(h, B2_ERR_NCCL, "%s failed: %s", #call, nccl_api().GetErrorString(r_));    \
  } while (0)

size_t esize(int type) { return type == T_BF16 ? 2 : 4; }

void batch_range(int batch, int world, int rank, int* b, int* e) {
  // get_partition(work, socket, 1, 0), Partition.cc:34-51
  int per = (batch + world - 1) / world;
  int lo = rank * per < batch ? rank * per : batch;
  int hi = lo + per < batch ? lo + per : batch;
  *b = lo;
  *e = hi;
}

int make_site(b2_handle* h, Site& s, bool want_tc, int sms = 0) {
  s.d.ws = h->tc_ws;
  s.d.ws_flags = h->tc_ws_flags;
  s.active = s.d.M > 0 && s.d.N > 0 && s.d.K > 0;
  s.plan = nullptr;
  if (!s.active || !want_tc) return B2_OK;
  char why[128] = "";
  s.plan = gemm_tc_plan_create(s.d, sms > 0 ? sms : h->gemm_sms, why, sizeof why);
  if (!s.plan) {
    // the CUDA-core kernel serves this site (about 30 x slower): counted, the first reason kept
    // for b2_site_report, and announced once per handle when B2_VERBOSE is set
    if (h->cuda_core_sites++ == 0) {
      char buf[256];
      snprintf(buf, sizeof buf, "GEMM %d x %d x %d: %s", s.d.M, s.d.N, s.d.K, why);
      h->cuda_core_reason = buf;
      if (getenv("B2_VERBOSE"))
        fprintf(stderr, "b200mlp: rank %d: tensor-core kernel refused, CUDA-core kernel used: %s\n", h->cfg.rank, buf);
    }
  } else {
    ++h->tensor_core_sites;
  }
  return B2_OK;
}

int run_site(b2_handle* h, const Site& s, cudaStream_t st) {
  if (!s.active) return B2_OK;
  ++h->launches;
  if (s.plan) {
    ++h->tc_launches;
    CK(h, gemm_tc_launch(s.plan, st, h->status_dev));
  } else {
    CK(h, gemm_simt_launch(s.d, st));
    if (s.d.C_lo) {  // fp32-class mode: the CUDA-core kernel served this site, so its result's twin is made here
      CK(h, split_lo_launch(static_cast<const float*>(s.d.C), static_cast<float*>(s.d.C_lo), (size_t)s.d.M * s.d.N, st));
      ++h->launches;
    }
  }
  return B2_OK;
}

bool use_tc(const b2_handle* h) { return h->cfg.precision != B2_PREC_FP32 && !h->cfg.force_simt; }

cudaEvent_t phase_ev(b2_handle* h, int l, int phase, int end) {
  return h->ev_phase[(((size_t)h->ev_iter * h->L + l) * B2_T_NUM + phase) * 2 + end];
}

int check_comm(b2_handle* h);

int check_status(b2_handle* h) {
  unsigned int st = 0;
  CK(h, cudaMemcpy(&st, h->status_dev, sizeof st, cudaMemcpyDeviceToHost));
  if (st != 0) {
    cudaMemset(h->status_dev, 0, sizeof st);
    if (h->tc_ws_flags) cudaMemset(h->tc_ws_flags, 0, (size_t)h->sms * sizeof(unsigned int));
    if (st >= 100u) {  // a flag wait of the peer-memory allreduce: its call counters no longer agree
      h->p2p_ready = false;
      cudaMemset(h->p2p_ctas_done, 0, sizeof(unsigned int));
      return fail(h, B2_ERR_TIMEOUT, "peer-memory allreduce gave up waiting for another rank (code %u); "
                  "the peer path is switched off for this handle", st);
    }
    return fail(h, B2_ERR_TIMEOUT, "tensor-core GEMM gave up waiting on a pipeline barrier (role %u)", st);
  }
  return check_comm(h);
}

// Asynchronous errors of the communicator (a peer process that died, a network fault): reported
// as B2_ERR_NCCL, and the communicator is aborted so that no later call blocks on it.
int check_comm(b2_handle* h) {
  if (!h->comm || !nccl_api().CommGetAsyncError) return B2_OK;
  int async = ncclSuccess;
  if (nccl_api().CommGetAsyncError(h->comm, &async) != ncclSuccess) return B2_OK;
  if (async != ncclSuccess && async != ncclInProgress) {
    const char* what = nccl_api().GetErrorString(async);
    if (nccl_api().CommAbort) nccl_api().CommAbort(h->comm);
    h->comm = nullptr;
    return fail(h, B2_ERR_NCCL, "the communicator reported an asynchronous error (%s) and was aborted; "
                "destroy the handles of this job", what ? what : "?");
  }
  return B2_OK;
}

// Rows of `width` bytes between two pitched buffers: one flat copy when both are dense.
cudaError_t copy_rows(void* dst, size_t dpitch, const void* src, size_t spitch, size_t width, size_t rows,
                      cudaMemcpyKind kind, cudaStream_t st) {
  if (dpitch == width && spitch == width) return cudaMemcpyAsync(dst, src, width * rows, kind, st);
  return cudaMemcpy2DAsync(dst, dpitch, src, spitch, width, rows, kind, st);
}

// Host (ld) <-> dense device matrix of `type`, through the fp32 staging buffer when
// the device holds bf16.
int upload_matrix(b2_handle* h, void* dev, int type, const float* host, size_t ld, int rows, int cols) {
  if (rows <= 0 || cols <= 0) return B2_OK;
  if (type == T_F32) {
    CK(h, copy_rows(dev, (size_t)cols * 4, host, ld * 4, (size_t)cols * 4, (size_t)rows, cudaMemcpyHostToDevice,
                    h->s_main));
  } else {
    if ((size_t)rows * cols > h->stage_elems) return fail(h, B2_ERR_INVALID, "staging buffer too small");
    CK(h, copy_rows(h->stage, (size_t)cols * 4, host, ld * 4, (size_t)cols * 4, (size_t)rows,
                    cudaMemcpyHostToDevice, h->s_main));
    CK(h, convert_f32_to_bf16(h->stage, (__nv_bfloat16*)dev, (size_t)rows * cols, h->s_main));
    ++h->launches;
  }
  return B2_OK;
}

int download_matrix(b2_handle* h, const void* dev, int type, float* host, size_t ld, int rows, int cols) {
  if (rows <= 0 || cols <= 0) return B2_OK;
  const void* src = dev;
  if (type == T_BF16) {
    if ((size_t)rows * cols > h->stage_elems) return fail(h, B2_ERR_INVALID, "staging buffer too small");
    CK(h, convert_bf16_to_f32((const __nv_bfloat16*)dev, h->stage, (size_t)rows * cols, h->s_main));
    ++h->launches;
    src = h->stage;
  }
  CK(h, cudaMemcpy2DAsync(host, ld * 4, src, (size_t)cols * 4, (size_t)cols * 4, rows, cudaMemcpyDeviceToHost,
                          h->s_main));
  CK(h, cudaStreamSynchronize(h->s_main));
  return B2_OK;
}

int build_sites(b2_handle* h) {
  const int L = h->L, bl = h->bl;
  const bool baseline = h->cfg.mode == B2_MODE_BASELINE;
  const bool tc = use_tc(h);
  h->fwd.assign(L, Site());
  h->wgrad.assign(L, Site());
  h->dgrad.assign(L, Site());
  // B2_BWD_SPLIT=p (experimental): while the weight-gradient stream is in use, its grids take
  // p percent of the GEMM SMs and the input-gradient grids the rest, so that the two
  // concurrent persistent kernels together stay inside the SMs not set aside for the collective
  int wg_sms = 0, dg_sms = 0;
  if (const char* e = getenv("B2_BWD_SPLIT")) {
    const int pct = atoi(e);
    if (h->wg_stream && pct > 0 && pct < 100) {
      wg_sms = h->gemm_sms * pct / 100;
      if (wg_sms < 1) wg_sms = 1;
      dg_sms = h->gemm_sms - wg_sms;
      if (dg_sms < 1) dg_sms = 1;
    }
  }
  for (int l = 0; l < L; ++l) {
    const int fi = h->nf[l], fo = h->nf[l + 1];
    const void* wop = h->op_type == T_BF16 ? (const void*)h->w16[l] : (const void*)h->w[l];
    // forward: A[l+1] = A[l] * W[l]^T (mlp_omp.cc:474-488)
    GemmDesc f{};
    f.M = bl; f.N = fo; f.K = fi;
    f.A = h->act[l]; f.sAm = fi; f.sAk = 1;
    f.B = wop; f.sBk = 1; f.sBn = fi;
    f.C = (l == L - 1) ? (void*)h->y : h->act[l + 1];
    f.ldc = fo;
    f.alpha = 1.f; f.beta = 0.f;
    f.epilogue = (baseline && l < L - 1) ? EPI_RELU : EPI_NONE;
    f.in_type = h->op_type;
    f.out_type = (l == L - 1) ? T_F32 : h->op_type;
    if (h->x3) {
      f.A_lo = h->act_lo[l];
      f.B_lo = h->w_lo[l];
      f.C_lo = (l == L - 1) ? nullptr : h->act_lo[l + 1];
    }
    h->fwd[l].d = f;
    make_site(h, h->fwd[l], tc);
    // weight gradient: dW[l] = dZ[l]^T * A[l] over this rank's rows (mlp_omp.cc:565-580)
    GemmDesc g{};
    g.M = fo; g.N = fi; g.K = bl;
    g.A = h->dz[l]; g.sAm = 1; g.sAk = fo;
    g.B = h->act[l]; g.sBk = fi; g.sBn = 1;
    g.C = h->dw[l]; g.ldc = fi;
    g.alpha = 1.f; g.beta = 0.f;
    g.epilogue = EPI_NONE;
    g.in_type = h->op_type;
    g.out_type = h->grad_type;
    if (h->x3) {
      g.A_lo = h->dz_lo[l];
      g.B_lo = h->act_lo[l];
    }
    h->wgrad[l].d = g;
    make_site(h, h->wgrad[l], tc, wg_sms);
    // input gradient: dA[l] = dZ[l] * W[l] (mlp_omp.cc:655-671), masked by ReLU'(A[l])
    GemmDesc b{};
    b.M = bl; b.N = fi; b.K = fo;
    b.A = h->dz[l]; b.sAm = fo; b.sAk = 1;
    b.B = wop; b.sBk = fi; b.sBn = 1;
    b.C = (l == 0) ? h->dinput : h->dz[l - 1];
    b.ldc = fi;
    b.alpha = 1.f; b.beta = 0.f;
    b.epilogue = (baseline && l > 0) ? EPI_MASK : EPI_NONE;
    b.aux = h->act[l]; b.ldaux = fi;
    b.in_type = h->op_type;
    b.out_type = h->op_type;
    if (h->x3) {
      b.A_lo = h->dz_lo[l];
      b.B_lo = h->w_lo[l];
      b.C_lo = (l == 0) ? nullptr : h->dz_lo[l - 1];
    }
    h->dgrad[l].d = b;
    make_site(h, h->dgrad[l], tc, dg_sms);
    if (l == 0 && !h->cfg.input_grad) h->dgrad[l].active = false;
    if (l == 0) {  // layer 0 reads the network input: one more pair of sites for the second slot
      h->fwd0_alt.d = f;
      h->fwd0_alt.d.A = h->act0_alt;
      if (h->x3) h->fwd0_alt.d.A_lo = h->act0_alt_lo;
      make_site(h, h->fwd0_alt, tc);
      h->wgrad0_alt.d = g;
      h->wgrad0_alt.d.B = h->act0_alt;
      if (h->x3) h->wgrad0_alt.d.B_lo = h->act0_alt_lo;
      make_site(h, h->wgrad0_alt, tc, wg_sms);
    }
  }
  // ReLU bit planes: used for a layer only if both its producer (forward of the layer below) and
  // its consumer (input gradient of the layer itself) run on the tensor-core kernel
  for (int l = 1; l < L; ++l) {
    if (!h->relu_bits[l] || !h->fwd[l - 1].plan || !h->dgrad[l].plan) continue;
    const long long ldw = h->nf[l] / 32;
    if (l == 1 && !h->fwd0_alt.plan) continue;
    if (!gemm_tc_plan_set_mask(h->fwd[l - 1].plan, h->relu_bits[l], nullptr, ldw)) continue;
    if (!gemm_tc_plan_set_mask(h->dgrad[l].plan, nullptr, h->relu_bits[l], ldw)) {
      gemm_tc_plan_set_mask(h->fwd[l - 1].plan, nullptr, nullptr, ldw);
      continue;
    }
    if (l == 1) gemm_tc_plan_set_mask(h->fwd0_alt.plan, h->relu_bits[l], nullptr, ldw);
  }
  return B2_OK;
}

// Sum of `count` gradient elements starting `begin` elements into the slab, over all ranks:
// through peer memory when the ranks are connected and the message is small, else NCCL.
int sum_gradients(b2_handle* h, size_t begin, size_t count, cudaStream_t st) {
  const size_t es = esize(h->grad_type);
  if (h->p2p_ready && h->grad_type == T_F32 && !h->cfg.use_graph && count * es <= h->p2p_max_bytes) {
    P2pParams p{};
    for (int r = 0; r < h->cfg.world_size; ++r) {
      p.slab[r] = h->p2p_slab[r];
      p.flags[r] = h->p2p_flags[r];
    }
    p.world = h->cfg.world_size;
    p.rank = h->cfg.rank;
    p.offset = begin;
    p.count = count;
    p.epoch = ++h->p2p_epoch;
    p.ctas_done = h->p2p_ctas_done;
    p.status = h->status_dev;
    p.wait_ns = h->p2p_wait_ns;
    ++h->launches;
    CK(h, p2p_allreduce_launch(p, h->cfg.comm_sms, st));
    return B2_OK;
  }
  char* base = static_cast<char*>(h->dw_slab) + begin * es;
  NCK(h, nccl_api().AllReduce(base, base, count, h->grad_type == T_BF16 ? ncclBfloat16 : ncclFloat32, ncclSum,
                              h->comm, st));
  return B2_OK;
}

int layer_update(b2_handle* h, int l, cudaStream_t st, bool timed) {
  const size_t n = (size_t)h->nf[l + 1] * h->nf[l];
  if (h->cfg.world_size > 1 && h->cfg.allreduce) {
    if (timed) CK(h, cudaEventRecord(phase_ev(h, l, B2_T_ALLREDUCE, 0), st));
    int rc = sum_gradients(h, h->dw_off[l], n, st);
    if (rc) return rc;
    if (timed) CK(h, cudaEventRecord(phase_ev(h, l, B2_T_ALLREDUCE, 1), st));
  }
  return B2_OK;
}

// Element range of the bucket of layers [low, high] in the slabs (`high` first), padding included.
void bucket_range(const b2_handle* h, int low, int high, size_t* begin, size_t* count) {
  plan_bucket_slice(h->dw_off.data(), h->dw_pad.data(), low, high, h->cfg.world_size, h->cfg.rank, begin, count,
                    nullptr, nullptr);
}

// Sum of the gradients of layers [low, high] (contiguous in the slab, `high` first) over all ranks.
int bucket_allreduce(b2_handle* h, int low, int high, cudaStream_t st, bool timed) {
  if (!(h->cfg.world_size > 1 && h->cfg.allreduce)) return B2_OK;
  const size_t begin = h->dw_off[high];
  const size_t end = h->dw_off[low] + (size_t)h->nf[low + 1] * h->nf[low];
  if (timed) CK(h, cudaEventRecord(phase_ev(h, low, B2_T_ALLREDUCE, 0), st));
  int rc = sum_gradients(h, begin, end - begin, st);
  if (rc) return rc;
  if (timed) CK(h, cudaEventRecord(phase_ev(h, low, B2_T_ALLREDUCE, 1), st));
  return B2_OK;
}

// The reference's route (mlp_omp.cc:90-146, 240-258) for one bucket, in three calls:
// reduce-scatter of the gradients (rank r receives the sum of slice r, in place) ...
int bucket_reduce_scatter(b2_handle* h, int low, int high, cudaStream_t st, bool timed) {
  size_t begin, count;
  bucket_range(h, low, high, &begin, &count);
  const size_t es = esize(h->grad_type), per = count / h->cfg.world_size;
  char* base = static_cast<char*>(h->dw_slab) + begin * es;
  if (timed) CK(h, cudaEventRecord(phase_ev(h, low, B2_T_ALLREDUCE, 0), st));
  NCK(h, nccl_api().ReduceScatter(base, base + (size_t)h->cfg.rank * per * es, per,
                                  h->grad_type == T_BF16 ? ncclBfloat16 : ncclFloat32, ncclSum, h->comm, st));
  if (timed) CK(h, cudaEventRecord(phase_ev(h, low, B2_T_ALLREDUCE, 1), st));
  return B2_OK;
}
// ... w = fma(-lr, g, w) on the slice this rank owns (1/world of the bucket's SGD traffic) ...
int bucket_shard_sgd(b2_handle* h, int low, int high, cudaStream_t st, bool timed) {
  size_t begin, count;
  bucket_range(h, low, high, &begin, &count);
  const size_t per = count / h->cfg.world_size, off = begin + (size_t)h->cfg.rank * per;
  if (timed) CK(h, cudaEventRecord(phase_ev(h, low, B2_T_WGT_UPDATE, 0), st));
  CK(h, sgd_launch(h->w_slab + off, static_cast<char*>(h->dw_slab) + off * esize(h->grad_type), h->grad_type,
                   h->op_type == T_BF16 ? h->w16_slab + off : nullptr, per, h->cfg.lr, h->sms, st,
                   h->x3 ? h->w_lo_slab + off : nullptr));
  ++h->launches;
  if (timed) CK(h, cudaEventRecord(phase_ev(h, low, B2_T_WGT_UPDATE, 1), st));
  if (h->op_type == T_BF16) h->masters_stale = true;
  return B2_OK;
}
// ... and allgather of the updated weights: of the bf16 operand copy in BF16 precision (half the
// bytes; the fp32 masters stay with their owners), of the fp32 weights otherwise.
int bucket_allgather(b2_handle* h, int low, int high, cudaStream_t st, bool timed) {
  size_t begin, count;
  bucket_range(h, low, high, &begin, &count);
  const size_t per = count / h->cfg.world_size;
  if (timed) CK(h, cudaEventRecord(phase_ev(h, low, B2_T_ALLGATHER, 0), st));
  if (h->op_type == T_BF16) {
    __nv_bfloat16* base = h->w16_slab + begin;
    NCK(h, nccl_api().AllGather(base + (size_t)h->cfg.rank * per, base, per, ncclBfloat16, h->comm, st));
  } else {
    float* base = h->w_slab + begin;
    NCK(h, nccl_api().AllGather(base + (size_t)h->cfg.rank * per, base, per, ncclFloat32, h->comm, st));
    if (h->x3) {  // the twins of the slices that arrived from the other ranks
      CK(h, split_lo_launch(base, h->w_lo_slab + begin, count, st));
      ++h->launches;
    }
  }
  if (timed) CK(h, cudaEventRecord(phase_ev(h, low, B2_T_ALLGATHER, 1), st));
  return B2_OK;
}

// Whether the bucket closed by layer `low` takes the sharded route (else: full sum + full SGD).
// Reduce-scatter of bucket [low, high] and allgather of bucket [ag_low, ag_high] (updated before)
// in one NCCL group: one launch in which the two run side by side on separate channels.
int bucket_rs_ag_grouped(b2_handle* h, int low, int high, int ag_low, int ag_high, cudaStream_t st, bool timed) {
  size_t rb, rc_, ab, ac;
  bucket_range(h, low, high, &rb, &rc_);
  bucket_range(h, ag_low, ag_high, &ab, &ac);
  const int world = h->cfg.world_size, rank = h->cfg.rank;
  const size_t es = esize(h->grad_type), rper = rc_ / world, aper = ac / world;
  char* gbase = static_cast<char*>(h->dw_slab) + rb * es;
  if (timed) CK(h, cudaEventRecord(phase_ev(h, low, B2_T_ALLREDUCE, 0), st));
  NCK(h, nccl_api().GroupStart());
  NCK(h, nccl_api().ReduceScatter(gbase, gbase + (size_t)rank * rper * es, rper,
                                  h->grad_type == T_BF16 ? ncclBfloat16 : ncclFloat32, ncclSum, h->comm, st));
  if (h->op_type == T_BF16) {
    __nv_bfloat16* base = h->w16_slab + ab;
    NCK(h, nccl_api().AllGather(base + (size_t)rank * aper, base, aper, ncclBfloat16, h->comm, st));
  } else {
    float* base = h->w_slab + ab;
    NCK(h, nccl_api().AllGather(base + (size_t)rank * aper, base, aper, ncclFloat32, h->comm, st));
  }
  NCK(h, nccl_api().GroupEnd());
  if (h->op_type != T_BF16 && h->x3) {
    CK(h, split_lo_launch(h->w_slab + ab, h->w_lo_slab + ab, ac, st));
    ++h->launches;
  }
  if (timed) {  // the pair counts as the reduce-scatter's phase; the allgather's own phase is empty
    CK(h, cudaEventRecord(phase_ev(h, low, B2_T_ALLREDUCE, 1), st));
    CK(h, cudaEventRecord(phase_ev(h, ag_low, B2_T_ALLGATHER, 0), st));
    CK(h, cudaEventRecord(phase_ev(h, ag_low, B2_T_ALLGATHER, 1), st));
  }
  return B2_OK;
}

bool bucket_sharded(const b2_handle* h, int low) {
  return h->shard && !h->bucket_full[low];
}

// Brings every rank's fp32 master weights up to date (collective; BF16 precision with
// shard_update only): each rank contributes the slices it owns.
int gather_masters(b2_handle* h) {
  if (!h->masters_stale) return B2_OK;
  if (!h->comm) return fail(h, B2_ERR_STATE, "the communicator of this job was aborted after an error");
  for (int l = h->L - 1; l >= 0; --l) {
    if (h->bucket_low[l] != l || !bucket_sharded(h, l)) continue;
    size_t begin, count;
    bucket_range(h, l, h->bucket_high[l], &begin, &count);
    const size_t per = count / h->cfg.world_size;
    float* base = h->w_slab + begin;
    NCK(h, nccl_api().AllGather(base + (size_t)h->cfg.rank * per, base, per, ncclFloat32, h->comm, h->s_main));
  }
  CK(h, cudaStreamSynchronize(h->s_main));
  h->masters_stale = false;
  return B2_OK;
}

int layer_sgd(b2_handle* h, int l, cudaStream_t st, bool timed) {
  const size_t n = (size_t)h->nf[l + 1] * h->nf[l];
  if (timed) CK(h, cudaEventRecord(phase_ev(h, l, B2_T_WGT_UPDATE, 0), st));
  CK(h, sgd_launch(h->w[l], h->dw[l], h->grad_type, h->op_type == T_BF16 ? h->w16[l] : nullptr, n, h->cfg.lr,
                   h->sms, st, h->x3 ? h->w_lo[l] : nullptr));
  ++h->launches;
  if (timed) CK(h, cudaEventRecord(phase_ev(h, l, B2_T_WGT_UPDATE, 1), st));
  return B2_OK;
}

// Enqueue one training step on the two streams (no host synchronisation).
int enqueue_step(b2_handle* h, bool timed, int slot = 0) {
  const int L = h->L;
  double* loss_acc = h->loss_dev + slot;
  const float* target = slot ? h->target_alt : h->target;
  const bool overlap = h->cfg.overlap != 0;
  const bool wg = overlap && h->wg_stream;
  cudaStream_t sm = h->s_main, sc = overlap ? h->s_comm : h->s_main, sw = wg ? h->s_wg : h->s_main;
  cudaStream_t su = overlap ? h->s_upd : h->s_main;
  const bool has_ar = h->cfg.world_size > 1 && h->cfg.allreduce;
  int rc;
  if (has_ar && !h->comm)
    return fail(h, B2_ERR_STATE, "the communicator of this job was aborted after an error; destroy the handles");
  int pending_ag = -1;  // bucket (its lowest layer) whose allgather is still to be issued
  // Allgathers are issued behind ALL reduce-scatters of the step, lowest layers first: the next
  // forward pass needs layer 0 first and the top layers last, while backward produced the
  // gradients in the opposite order. So once the last gradient exists the collective stream
  // only has to finish reduce-scatter + allgather of the LOWEST bucket before fwd(0) may start;
  // the allgathers of the upper buckets run under the next forward pass. (B2_AG_ORDER=eager:
  // each bucket's allgather right behind the next bucket's reduce-scatter, top bucket first.)
  const bool ag_deferred = h->ag_deferred;
  int deferred[64];
  int ndeferred = 0;
  CK(h, cudaMemsetAsync(loss_acc, 0, sizeof(double), sm));
  for (int l = 0; l < L; ++l) {
    if (overlap && h->upd_pending[l]) {
      CK(h, cudaStreamWaitEvent(sm, h->ev_upd[l], 0));
      h->upd_pending[l] = 0;
    }
    if (timed) CK(h, cudaEventRecord(phase_ev(h, l, B2_T_FWD, 0), sm));
    if ((rc = run_site(h, (l == 0 && slot) ? h->fwd0_alt : h->fwd[l], sm))) return rc;
    if (timed) CK(h, cudaEventRecord(phase_ev(h, l, B2_T_FWD, 1), sm));
  }
  {
    const size_t n = (size_t)h->bl * h->nf[L];
    const bool baseline = h->cfg.mode == B2_MODE_BASELINE;
    CK(h, loss_grad_launch(h->y, target, h->dz[L - 1], h->op_type, n, baseline ? 1 : 0,
                           1.0f / (float)h->cfg.batch, baseline ? 1.0 / (double)h->cfg.batch : 1.0, loss_acc, sm,
                           h->x3 ? h->dz_lo[L - 1] : nullptr));
    if (n) ++h->launches;
    if (wg) CK(h, cudaEventRecord(h->ev_dz_last, sm));
  }
  for (int l = L - 1; l >= 0; --l) {
    // wgrad(l) needs dZ[l]: the output gradient for the last layer, dgrad(l+1) otherwise
    if (wg) CK(h, cudaStreamWaitEvent(sw, l == L - 1 ? h->ev_dz_last : h->ev_dgrad[l + 1], 0));
    if (timed) CK(h, cudaEventRecord(phase_ev(h, l, B2_T_WGT_GRAD, 0), sw));
    if (h->wgrad[l].active) {
      if ((rc = run_site(h, (l == 0 && slot) ? h->wgrad0_alt : h->wgrad[l], sw))) return rc;
    } else {  // a rank without batch rows contributes a zero gradient
      CK(h, cudaMemsetAsync(h->dw[l], 0, (size_t)h->nf[l + 1] * h->nf[l] * esize(h->grad_type), sw));
    }
    if (timed) CK(h, cudaEventRecord(phase_ev(h, l, B2_T_WGT_GRAD, 1), sw));
    const bool closes_bucket = (h->bucket_low[l] == l);
    const bool sharded = closes_bucket && has_ar && bucket_sharded(h, l);
    if (overlap) {
      CK(h, cudaEventRecord(h->ev_wgrad[l], sw));
      // in-order weight-gradient stream: the event covers every layer of the bucket
      if (closes_bucket) CK(h, cudaStreamWaitEvent(has_ar ? sc : su, h->ev_wgrad[l], 0));
    }
    if (sharded) {
      // reduce-scatter of this bucket; behind it, on the same stream, the allgather of the bucket
      // before (its owned-slice SGD ran while this reduce-scatter was in flight)
      if (h->ag_grouped && pending_ag >= 0) {
        if (overlap) CK(h, cudaStreamWaitEvent(sc, h->ev_shard[pending_ag], 0));
        if ((rc = bucket_rs_ag_grouped(h, l, h->bucket_high[l], pending_ag, h->bucket_high[pending_ag], sc, timed)))
          return rc;
        for (int k = pending_ag; k <= h->bucket_high[pending_ag]; ++k) {
          if (overlap) {
            CK(h, cudaEventRecord(h->ev_upd[k], sc));
            h->upd_pending[k] = 1;
          }
        }
        pending_ag = -1;
      } else if ((rc = bucket_reduce_scatter(h, l, h->bucket_high[l], sc, timed))) {
        return rc;
      }
      if (overlap) CK(h, cudaEventRecord(h->ev_ar[l], sc));
      if (pending_ag >= 0 && ag_deferred && ndeferred < 64) {
        deferred[ndeferred++] = pending_ag;
        pending_ag = -1;
      }
      if (pending_ag >= 0) {
        if (overlap) CK(h, cudaStreamWaitEvent(sc, h->ev_shard[pending_ag], 0));
        if ((rc = bucket_allgather(h, pending_ag, h->bucket_high[pending_ag], sc, timed))) return rc;
        for (int k = pending_ag; k <= h->bucket_high[pending_ag]; ++k) {
          if (overlap) {
            CK(h, cudaEventRecord(h->ev_upd[k], sc));
            h->upd_pending[k] = 1;
          }
        }
        pending_ag = -1;
      }
    } else if (closes_bucket && has_ar) {
      if ((rc = bucket_allreduce(h, l, h->bucket_high[l], sc, timed))) return rc;
      if (overlap) {
        CK(h, cudaEventRecord(h->ev_ar[l], sc));
        CK(h, cudaStreamWaitEvent(su, h->ev_ar[l], 0));
      }
    }
    if (timed) CK(h, cudaEventRecord(phase_ev(h, l, B2_T_BWD, 0), sm));
    if ((rc = run_site(h, h->dgrad[l], sm))) return rc;
    if (timed) CK(h, cudaEventRecord(phase_ev(h, l, B2_T_BWD, 1), sm));
    if (overlap) CK(h, cudaEventRecord(h->ev_dgrad[l], sm));
    if (sharded) {
      // SGD of the owned slice: after the reduce-scatter and after dgrad(l), the last reader of the
      // bucket's old weights on the in-order main stream
      if (overlap) {
        CK(h, cudaStreamWaitEvent(su, h->ev_ar[l], 0));
        CK(h, cudaStreamWaitEvent(su, h->ev_dgrad[l], 0));
      }
      if ((rc = bucket_shard_sgd(h, l, h->bucket_high[l], su, timed))) return rc;
      if (overlap) CK(h, cudaEventRecord(h->ev_shard[l], su));
      pending_ag = l;
    } else if (closes_bucket) {
      // SGD of every layer of the bucket, on its own stream so that the next bucket's sum does
      // not queue behind it: after this bucket's sum, and after dgrad(l), the last reader of the
      // bucket's old weights on the in-order main stream. Lowest layer first: it is the first
      // one the next forward pass needs.
      if (overlap) CK(h, cudaStreamWaitEvent(su, h->ev_dgrad[l], 0));
      for (int k = l; k <= h->bucket_high[l]; ++k) {
        if ((rc = layer_sgd(h, k, su, timed))) return rc;
        if (overlap) {
          CK(h, cudaEventRecord(h->ev_upd[k], su));
          h->upd_pending[k] = 1;
        }
      }
    }
  }
  // the allgather of the last (lowest) bucket, then the deferred ones from the lowest layers up
  for (int i = ndeferred; i >= 0; --i) {
    const int b = (i == ndeferred) ? pending_ag : deferred[i];
    if (b < 0) continue;
    if (overlap) CK(h, cudaStreamWaitEvent(sc, h->ev_shard[b], 0));
    if ((rc = bucket_allgather(h, b, h->bucket_high[b], sc, timed))) return rc;
    for (int k = b; k <= h->bucket_high[b]; ++k) {
      if (overlap) {
        CK(h, cudaEventRecord(h->ev_upd[k], sc));
        h->upd_pending[k] = 1;
      }
    }
  }
  // the step's inputs (read by wgrad(0)) are free, and the step is over on the main stream,
  // only once the last weight-gradient GEMM is done
  if (wg) CK(h, cudaStreamWaitEvent(sm, h->ev_wgrad[0], 0));
  return B2_OK;
}

int join_streams(b2_handle* h) {
  if (h->cfg.overlap) {
    CK(h, cudaEventRecord(h->ev_join, h->s_comm));
    CK(h, cudaStreamWaitEvent(h->s_main, h->ev_join, 0));
    CK(h, cudaEventRecord(h->ev_join_upd, h->s_upd));
    CK(h, cudaStreamWaitEvent(h->s_main, h->ev_join_upd, 0));
    for (auto& p : h->upd_pending) p = 0;
  }
  return B2_OK;
}

void free_all(b2_handle* h) {
  if (!h) return;
  cudaSetDevice(h->cfg.device);
  if (h->s_main) cudaStreamSynchronize(h->s_main);
  if (h->s_comm) cudaStreamSynchronize(h->s_comm);
  if (h->s_upd) {
    cudaStreamSynchronize(h->s_upd);
    cudaStreamDestroy(h->s_upd);
  }
  if (h->ev_join_upd) cudaEventDestroy(h->ev_join_upd);
  for (auto e : h->ev_ar)
    if (e) cudaEventDestroy(e);
  if (h->s_copy) cudaStreamSynchronize(h->s_copy);
  if (h->s_wg) {
    cudaStreamSynchronize(h->s_wg);
    cudaStreamDestroy(h->s_wg);
  }
  if (h->ev_dz_last) cudaEventDestroy(h->ev_dz_last);
  if (h->comm && nccl_api().ok) {
    for (void* rh : h->ub_handle)
      if (rh && nccl_api().CommDeregister) nccl_api().CommDeregister(h->comm, rh);
    nccl_api().CommDestroy(h->comm);
  }
  if (h->graph_exec) cudaGraphExecDestroy(h->graph_exec);
  for (auto& s : h->fwd) gemm_tc_plan_destroy(s.plan);
  for (auto& s : h->wgrad) gemm_tc_plan_destroy(s.plan);
  for (auto& s : h->dgrad) gemm_tc_plan_destroy(s.plan);
  if (h->nccl_ub && nccl_api().MemFree) {
    if (h->w_slab) nccl_api().MemFree(h->w_slab);
    if (h->w16_slab) nccl_api().MemFree(h->w16_slab);
    if (h->dw_slab) nccl_api().MemFree(h->dw_slab);
    h->dw_slab = nullptr;
  } else {
    cudaFree(h->w_slab);
    cudaFree(h->w16_slab);
  }
  cudaFree(h->w_lo_slab);
  for (auto p : h->act_lo) cudaFree(p);
  for (auto p : h->dz_lo) cudaFree(p);
  cudaFree(h->act0_alt_lo);
  for (auto e : h->ev_shard)
    if (e) cudaEventDestroy(e);
  for (int r = 0; r < P2P_MAX_RANKS; ++r)
    if (h->p2p_opened[r]) cudaIpcCloseMemHandle(h->p2p_opened[r]);
  cudaFree(h->p2p_ctas_done);
  cudaFree(h->dw_slab);
  for (auto p : h->act) cudaFree(p);
  for (auto p : h->relu_bits) cudaFree(p);
  for (auto p : h->dz) cudaFree(p);
  cudaFree(h->y);
  cudaFree(h->target);
  cudaFree(h->dinput);
  cudaFree(h->stage);
  cudaFree(h->loss_dev);
  cudaFree(h->act0_alt);
  cudaFree(h->target_alt);
  cudaFree(h->xstage[0]);
  cudaFree(h->xstage[1]);
  if (h->loss_host) cudaFreeHost(h->loss_host);
  gemm_tc_plan_destroy(h->fwd0_alt.plan);
  gemm_tc_plan_destroy(h->wgrad0_alt.plan);
  for (int i = 0; i < 2; ++i) {
    if (h->ev_copied[i]) cudaEventDestroy(h->ev_copied[i]);
    if (h->ev_slot_free[i]) cudaEventDestroy(h->ev_slot_free[i]);
    if (h->ev_loss[i]) cudaEventDestroy(h->ev_loss[i]);
  }
  if (h->s_copy) cudaStreamDestroy(h->s_copy);
  cudaFree(h->status_dev);
  cudaFree(h->fp_dev);
  cudaFree(h->tc_ws);
  cudaFree(h->tc_ws_flags);
  for (auto e : h->ev_wgrad) cudaEventDestroy(e);
  for (auto e : h->ev_dgrad) cudaEventDestroy(e);
  for (auto e : h->ev_upd) cudaEventDestroy(e);
  for (auto e : h->ev_phase)
    if (e) cudaEventDestroy(e);
  if (h->ev_t0) cudaEventDestroy(h->ev_t0);
  if (h->ev_t1) cudaEventDestroy(h->ev_t1);
  if (h->ev_join) cudaEventDestroy(h->ev_join);
  if (h->ev_fork) cudaEventDestroy(h->ev_fork);
  if (h->s_main) cudaStreamDestroy(h->s_main);
  if (h->s_comm) cudaStreamDestroy(h->s_comm);
  delete h;
}

template <typename T>
int dev_alloc(b2_handle* h, T** p, size_t bytes) {
  *p = nullptr;
  if (bytes == 0) bytes = 16;
  CK(h, cudaMalloc((void**)p, bytes));
  CK(h, cudaMemset(*p, 0, bytes));
  return B2_OK;
}

}  // namespace

extern "C" {

int b2_config_default(b2_config* c) {
  if (!c) return B2_ERR_INVALID;
  memset(c, 0, sizeof *c);
  c->world_size = 1;
  c->mode = B2_MODE_BASELINE;
  c->precision = B2_PREC_FP32;
  c->allreduce = 1;
  c->overlap = 1;
  c->input_grad = 1;
  c->comm_sms = -1;
  c->ar_bucket_mb = -1;
  c->shard_update = -1;
  c->lr = 0.01f;
  return B2_OK;
}

const char* b2_version(void) { return "b200mlp 0.1 (sm_100a)"; }

const char* b2_last_error(const b2_handle* h) { return h ? h->err.c_str() : g_tls_error.c_str(); }

int b2_nccl_unique_id(void* out) {
  if (!out) return fail(nullptr, B2_ERR_INVALID, "null output");
  NcclApi& n = nccl_api();
  if (!n.ok) return fail(nullptr, B2_ERR_NCCL, "%s", n.error.c_str());
  ncclUniqueId id;
  NCK(nullptr, n.GetUniqueId(&id));
  memcpy(out, &id, sizeof id);
  return B2_OK;
}

int b2_create(const b2_config* cfg, b2_handle** out) {
  if (!cfg || !out) return fail(nullptr, B2_ERR_INVALID, "null argument");
  *out = nullptr;
  if (cfg->nlayers < 1 || !cfg->nfeatures) return fail(nullptr, B2_ERR_INVALID, "nlayers/nfeatures");
  if (cfg->batch < 1) return fail(nullptr, B2_ERR_INVALID, "batch must be positive");
  if (cfg->world_size < 1 || cfg->rank < 0 || cfg->rank >= cfg->world_size)
    return fail(nullptr, B2_ERR_INVALID, "rank %d outside world of %d", cfg->rank, cfg->world_size);
  if (cfg->precision < B2_PREC_FP32 || cfg->precision > B2_PREC_FP32_TC)
    return fail(nullptr, B2_ERR_INVALID, "unknown precision %d", cfg->precision);
  if (cfg->mode != B2_MODE_REF && cfg->mode != B2_MODE_BASELINE)
    return fail(nullptr, B2_ERR_INVALID, "unknown mode %d", cfg->mode);
  if (cfg->grad_bf16 && cfg->precision != B2_PREC_BF16)
    return fail(nullptr, B2_ERR_INVALID, "grad_bf16 needs BF16 precision");
  for (int i = 0; i <= cfg->nlayers; ++i)
    if (cfg->nfeatures[i] < 1) return fail(nullptr, B2_ERR_INVALID, "nfeatures[%d] must be positive", i);
  if (cfg->world_size > 1 && cfg->allreduce && !cfg->nccl_unique_id)
    return fail(nullptr, B2_ERR_INVALID, "world_size > 1 needs nccl_unique_id");
  // A captured step that contains collectives did not complete on two GPUs. Probable cause: the
  // communicator's first collective was issued under stream capture, while NCCL connects its
  // channels lazily at the first collective of each kind. b2_step now issues every bucket's
  // collective once, uncaptured, before it captures; until that has been confirmed on GPUs the
  // combination stays refused unless B2_GRAPH_WITH_ALLREDUCE=1 is set.
  if (cfg->use_graph && cfg->world_size > 1 && cfg->allreduce) {
    const char* e = getenv("B2_GRAPH_WITH_ALLREDUCE");
    if (!(e && e[0] == '1'))
      return fail(nullptr, B2_ERR_UNSUPPORTED, "use_graph is not supported together with the gradient allreduce");
  }

  int ndev = 0;
  cudaError_t e = cudaGetDeviceCount(&ndev);
  if (e != cudaSuccess || ndev == 0)
    return fail(nullptr, B2_ERR_CUDA, "no CUDA device (%s); this library has no CPU path",
                e == cudaSuccess ? "count 0" : cudaGetErrorString(e));
  if (cfg->device < 0 || cfg->device >= ndev) return fail(nullptr, B2_ERR_INVALID, "device %d of %d", cfg->device, ndev);

  b2_handle* h = new b2_handle();
  h->cfg = *cfg;
  h->L = cfg->nlayers;
  h->nf.assign(cfg->nfeatures, cfg->nfeatures + cfg->nlayers + 1);
  h->cfg.nfeatures = h->nf.data();
  h->cfg.nccl_unique_id = nullptr;
  batch_range(cfg->batch, cfg->world_size, cfg->rank, &h->b0, &h->b1);
  h->bl = h->b1 - h->b0;
  h->op_type = cfg->precision == B2_PREC_BF16 ? T_BF16 : T_F32;
  h->grad_type = cfg->grad_bf16 ? T_BF16 : T_F32;
  h->x3 = cfg->precision == B2_PREC_FP32_TC && !cfg->force_simt;
  int rc = B2_OK;
#define TRY(x)            \
  do {                    \
    rc = (x);             \
    if (rc != B2_OK) {    \
      g_tls_error = h->err; \
      free_all(h);        \
      return rc;          \
    }                     \
  } while (0)
#define TRYCK(call)                                                                                  \
  do {                                                                                               \
    cudaError_t e_ = (call);                                                                         \
    if (e_ != cudaSuccess) {                                                                         \
      rc = fail(h, B2_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e_));                     \
      free_all(h);                                                                                   \
      return rc;                                                                                     \
    }                                                                                                \
  } while (0)

  TRYCK(cudaSetDevice(cfg->device));
  cudaDeviceProp prop;
  TRYCK(cudaGetDeviceProperties(&prop, cfg->device));
  if (prop.major != 10)
    TRY(fail(h, B2_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", cfg->device,
             prop.major, prop.minor));
  h->sms = prop.multiProcessorCount;
  {
    const bool comm = cfg->world_size > 1 && cfg->allreduce && cfg->overlap;
    // default: 20 on 4 or more GPUs, none on 2 (measured there: 3.28 ms per step of configuration 4
    // with none against 3.36 ms with 20; on 8 GPUs 2.07 against 2.09)
    int reserve = cfg->comm_sms < 0 ? (comm && cfg->world_size >= 4 ? 20 : 0) : cfg->comm_sms;
    if (reserve > h->sms / 2) reserve = h->sms / 2;
    h->gemm_sms = h->sms - reserve;
    h->cfg.comm_sms = reserve;
  }
  TRYCK(cudaStreamCreateWithFlags(&h->s_main, cudaStreamNonBlocking));
  {
    // the side stream's kernels (collective, SGD) should take free SMs before the next GEMM does
    int lo = 0, hi = 0;
    TRYCK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    TRYCK(cudaStreamCreateWithPriority(&h->s_comm, cudaStreamNonBlocking, hi));
    TRYCK(cudaStreamCreateWithPriority(&h->s_upd, cudaStreamNonBlocking, hi));
  }

  TRYCK(cudaStreamCreateWithFlags(&h->s_wg, cudaStreamNonBlocking));
  TRYCK(cudaEventCreateWithFlags(&h->ev_dz_last, cudaEventDisableTiming));
  {
    // off when the stream-K schedule is requested: its workspace is shared by the handle's GEMMs
    const char* e = getenv("B2_WGRAD_STREAM");
    const char* sk = getenv("B2_TC_STREAMK");
    h->wg_stream = (e ? e[0] != '0' : true) && !(sk && sk[0] == '1');
  }
  const int L = h->L;
  const size_t bl = (size_t)h->bl;
  h->w.assign(L, nullptr);
  h->w16.assign(L, nullptr);
  h->dw.assign(L, nullptr);
  h->dz.assign(L, nullptr);
  h->act.assign(L + 1, nullptr);
  h->relu_bits.assign(L + 1, nullptr);
  h->w_lo.assign(L, nullptr);
  h->act_lo.assign(L + 1, nullptr);
  h->dz_lo.assign(L, nullptr);
  size_t max_elems = 16;
  for (int l = 0; l < L; ++l) {
    const size_t nw = (size_t)h->nf[l + 1] * h->nf[l];
    TRY(dev_alloc(h, &h->dz[l], bl * h->nf[l + 1] * esize(h->op_type)));
    TRY(dev_alloc(h, &h->act[l], bl * h->nf[l] * esize(h->op_type)));
    if (h->x3) {
      TRY(dev_alloc(h, &h->dz_lo[l], bl * h->nf[l + 1] * 4));
      TRY(dev_alloc(h, &h->act_lo[l], bl * h->nf[l] * 4));
    }
    if (l > 0 && cfg->mode == B2_MODE_BASELINE && cfg->precision != B2_PREC_FP32 && !cfg->force_simt &&
        h->nf[l] % 32 == 0)
      TRY(dev_alloc(h, &h->relu_bits[l], bl * (size_t)(h->nf[l] / 32) * sizeof(uint32_t)));
    if (nw > max_elems) max_elems = nw;
    if (bl * h->nf[l] > max_elems) max_elems = bl * h->nf[l];
    if (bl * h->nf[l + 1] > max_elems) max_elems = bl * h->nf[l + 1];
  }
  {
    // gradient and weight slabs, last layer first; every layer is padded to a multiple of
    // 128 * world elements, so that it starts on a 256-byte boundary in each slab and every
    // bucket of layers divides evenly among the ranks (the padding stays zero: 0 - lr * 0)
    h->dw_off.assign(L, 0);
    h->dw_pad.assign(L, 0);
    const size_t es = esize(h->grad_type);
    std::vector<size_t> layer_elems(L);
    for (int l = 0; l < L; ++l) layer_elems[l] = (size_t)h->nf[l + 1] * h->nf[l];
    const size_t total = plan_slab_layout(layer_elems.data(), L, cfg->world_size, h->dw_off.data(), h->dw_pad.data());
    {
      const char* ub = getenv("B2_NCCL_UB");
      h->nccl_ub = ub && ub[0] == '1' && cfg->world_size > 1 && cfg->allreduce && nccl_api().ok &&
                   nccl_api().MemAlloc && nccl_api().MemFree && nccl_api().CommRegister && nccl_api().CommDeregister;
    }
    auto slab_alloc = [&](void** ptr, size_t bytes) -> int {
      if (!h->nccl_ub) return dev_alloc(h, reinterpret_cast<char**>(ptr), bytes);
      if (nccl_api().MemAlloc(ptr, bytes) != ncclSuccess) return fail(h, B2_ERR_NCCL, "ncclMemAlloc of %zu bytes failed", bytes);
      cudaError_t e_ = cudaMemset(*ptr, 0, bytes);
      if (e_ != cudaSuccess) return fail(h, B2_ERR_CUDA, "cudaMemset: %s", cudaGetErrorString(e_));
      return B2_OK;
    };
    TRY(slab_alloc(reinterpret_cast<void**>(&h->w_slab), total * 4));
    if (h->op_type == T_BF16) TRY(slab_alloc(reinterpret_cast<void**>(&h->w16_slab), total * 2));
    if (h->x3) TRY(dev_alloc(h, &h->w_lo_slab, total * 4));
    for (int l = 0; l < L; ++l) {
      h->w[l] = h->w_slab + h->dw_off[l];
      if (h->w16_slab) h->w16[l] = h->w16_slab + h->dw_off[l];
      if (h->w_lo_slab) h->w_lo[l] = h->w_lo_slab + h->dw_off[l];
    }
    h->shard = cfg->world_size > 1 && cfg->allreduce && cfg->shard_update != 0;
    h->p2p_flags_off = (total * es + 255) / 256 * 256;
    h->slab_bytes = h->p2p_flags_off + 256;  // zero-filled flag block (P2P_FLAG_BYTES) behind the gradients
    TRY(slab_alloc(&h->dw_slab, h->slab_bytes));
    TRY(dev_alloc(h, &h->p2p_ctas_done, sizeof(unsigned int)));
    for (int l = 0; l < L; ++l) h->dw[l] = static_cast<char*>(h->dw_slab) + h->dw_off[l] * es;
    // buckets of consecutive layers (rule and rationale: bucket_plan.h); B2_BUCKET_GROWTH
    // overrides the factor between consecutive buckets
    std::vector<size_t> layer_bytes(L);
    for (int l = 0; l < L; ++l) layer_bytes[l] = (size_t)h->nf[l + 1] * h->nf[l] * es;
    double growth = 0.0;
    if (const char* e = getenv("B2_BUCKET_GROWTH")) growth = atof(e);
    h->bucket_low.assign(L, 0);
    h->bucket_high.assign(L, 0);
    plan_gradient_buckets(layer_bytes.data(), L, cfg->world_size, cfg->allreduce != 0, cfg->ar_bucket_mb, growth,
                          h->bucket_low.data(), h->bucket_high.data());
    {
      const char* e = getenv("B2_AG_ORDER");
      h->ag_deferred = !(e && (e[0] == 'e' || e[0] == 'g'));
      h->ag_grouped = e && e[0] == 'g' && nccl_api().GroupStart && nccl_api().GroupEnd;
      // layer 0 in a bucket of its own (bucket_plan.h) unless the bucket size was given explicitly
      // (ar_bucket_mb >= 0) or B2_SPLIT_LAST=0
      const char* sl = getenv("B2_SPLIT_LAST");
      if (h->shard && cfg->ar_bucket_mb < 0 && !(sl && sl[0] == '0'))
        plan_split_lowest_layer(L, h->bucket_low.data(), h->bucket_high.data());
    }
    // B2_BUCKET_LAYERS=a,b,c,... (experiments): layers per bucket, from the last layer down; the
    // counts must add up to the number of layers, else the variable is ignored
    if (const char* e = getenv("B2_BUCKET_LAYERS")) {
      std::vector<int> counts;
      int sum = 0;
      for (const char* q = e; *q;) {
        int v = atoi(q);
        if (v < 1) { sum = -1; break; }
        counts.push_back(v);
        sum += v;
        while (*q && *q != ',') ++q;
        if (*q == ',') ++q;
      }
      if (sum == L && cfg->world_size > 1 && cfg->allreduce) {
        int high = L - 1;
        for (int c : counts) {
          const int low = high - c + 1;
          for (int k = low; k <= high; ++k) {
            h->bucket_low[k] = low;
            h->bucket_high[k] = high;
          }
          high = low - 1;
        }
      }
    }
  }
  TRY(dev_alloc(h, &h->y, bl * h->nf[L] * 4));
  TRY(dev_alloc(h, &h->target, bl * h->nf[L] * 4));
  TRY(dev_alloc(h, &h->dinput, bl * h->nf[0] * esize(h->op_type)));
  if (h->op_type == T_BF16 || h->grad_type == T_BF16) {
    h->stage_elems = max_elems;
    TRY(dev_alloc(h, &h->stage, max_elems * 4));
  }
  TRY(dev_alloc(h, &h->act0_alt, bl * h->nf[0] * esize(h->op_type)));
  if (h->x3) TRY(dev_alloc(h, &h->act0_alt_lo, bl * h->nf[0] * 4));
  TRY(dev_alloc(h, &h->target_alt, bl * h->nf[L] * 4));
  if (h->op_type == T_BF16)
    for (int i = 0; i < 2; ++i) TRY(dev_alloc(h, &h->xstage[i], bl * h->nf[0] * 4));
  TRY(dev_alloc(h, &h->loss_dev, 2 * sizeof(double)));
  TRYCK(cudaHostAlloc((void**)&h->loss_host, 2 * sizeof(double), cudaHostAllocDefault));
  TRYCK(cudaStreamCreateWithFlags(&h->s_copy, cudaStreamNonBlocking));
  for (int i = 0; i < 2; ++i) {
    TRYCK(cudaEventCreateWithFlags(&h->ev_copied[i], cudaEventDisableTiming));
    TRYCK(cudaEventCreateWithFlags(&h->ev_slot_free[i], cudaEventDisableTiming));
    TRYCK(cudaEventCreateWithFlags(&h->ev_loss[i], cudaEventDisableTiming));
  }
  TRY(dev_alloc(h, &h->status_dev, sizeof(unsigned int)));
  TRY(dev_alloc(h, &h->fp_dev, sizeof(unsigned long long)));
  if (cfg->precision != B2_PREC_FP32 && !cfg->force_simt) {
    TRY(dev_alloc(h, &h->tc_ws, (size_t)h->sms * TC_WS_SLOT_BYTES));
    TRY(dev_alloc(h, &h->tc_ws_flags, (size_t)h->sms * sizeof(unsigned int)));
  }

  h->ev_wgrad.assign(L, nullptr);
  h->ev_dgrad.assign(L, nullptr);
  h->ev_upd.assign(L, nullptr);
  h->ev_ar.assign(L, nullptr);
  h->ev_shard.assign(L, nullptr);
  h->bucket_full.assign(L, 0);
  h->upd_pending.assign(L, 0);
  for (int l = 0; l < L; ++l) {
    TRYCK(cudaEventCreateWithFlags(&h->ev_shard[l], cudaEventDisableTiming));
    TRYCK(cudaEventCreateWithFlags(&h->ev_wgrad[l], cudaEventDisableTiming));
    TRYCK(cudaEventCreateWithFlags(&h->ev_dgrad[l], cudaEventDisableTiming));
    TRYCK(cudaEventCreateWithFlags(&h->ev_upd[l], cudaEventDisableTiming));
    TRYCK(cudaEventCreateWithFlags(&h->ev_ar[l], cudaEventDisableTiming));
  }
  TRYCK(cudaEventCreate(&h->ev_t0));
  TRYCK(cudaEventCreate(&h->ev_t1));
  TRYCK(cudaEventCreateWithFlags(&h->ev_join, cudaEventDisableTiming));
  TRYCK(cudaEventCreateWithFlags(&h->ev_join_upd, cudaEventDisableTiming));
  TRYCK(cudaEventCreateWithFlags(&h->ev_fork, cudaEventDisableTiming));
  h->phase_ms.assign((size_t)L * B2_T_NUM, 0.0);

  if (cfg->world_size > 1 && cfg->allreduce) {
    NcclApi& n = nccl_api();
    if (!n.ok) TRY(fail(h, B2_ERR_NCCL, "%s", n.error.c_str()));
    ncclUniqueId id;
    memcpy(&id, cfg->nccl_unique_id, sizeof id);
    int r = -1;
    int nccl_version = 0;
    if (n.GetVersion) n.GetVersion(&nccl_version);
    // B2_NCCL_MAX_CTAS=n creates the communicator with at most n CTAs per collective; unset
    // or 0 leaves the library's choice, which measured faster than a cap equal to the SMs
    // the GEMM grids leave free (8 GPUs: 2.71 ms against 2.81 ms per step)
    int max_ctas = 0;
    if (const char* e = getenv("B2_NCCL_MAX_CTAS")) max_ctas = atoi(e);
    if (n.CommInitRankConfig && nccl_version >= 22703 && max_ctas > 0) {
      ncclConfigCompat c = nccl_config_unset();
      c.maxCTAs = max_ctas;
      r = n.CommInitRankConfig(&h->comm, cfg->world_size, id, cfg->rank, &c);
      // a library that rejects the configuration does so before any rank exchange
      if (r == 4 /* ncclInvalidArgument */) r = n.CommInitRank(&h->comm, cfg->world_size, id, cfg->rank);
    } else {
      r = n.CommInitRank(&h->comm, cfg->world_size, id, cfg->rank);
    }
    if (r != ncclSuccess) TRY(fail(h, B2_ERR_NCCL, "ncclCommInitRank failed: %s", n.GetErrorString(r)));
    if (h->nccl_ub) {
      const size_t es_ = esize(h->grad_type);
      size_t welems = 0;
      for (int l = 0; l < L; ++l) welems += h->dw_pad[l];
      (void)es_;
      if (n.CommRegister(h->comm, h->dw_slab, h->slab_bytes, &h->ub_handle[0]) != ncclSuccess ||
          n.CommRegister(h->comm, h->w_slab, welems * 4, &h->ub_handle[1]) != ncclSuccess ||
          (h->w16_slab && n.CommRegister(h->comm, h->w16_slab, welems * 2, &h->ub_handle[2]) != ncclSuccess))
        TRY(fail(h, B2_ERR_NCCL, "ncclCommRegister failed"));
    }
  }
  TRY(build_sites(h));
  TRYCK(cudaDeviceSynchronize());
#undef TRY
#undef TRYCK
  *out = h;
  return B2_OK;
}

int b2_destroy(b2_handle* h) {
  free_all(h);
  return B2_OK;
}

int b2_batch_range(const b2_handle* h, int* begin, int* end) {
  if (!h) return B2_ERR_INVALID;
  if (begin) *begin = h->b0;
  if (end) *end = h->b1;
  return B2_OK;
}

#define ENTER(h)                                                \
  if (!(h)) return fail(nullptr, B2_ERR_INVALID, "null handle"); \
  CK(h, cudaSetDevice((h)->cfg.device))

#define LAYER_OK(h, l, hi) \
  if ((l) < 0 || (l) > (hi)) return fail(h, B2_ERR_INVALID, "layer %d out of range", (l))

int b2_upload_weights(b2_handle* h, int l, const float* host, size_t ld) {
  ENTER(h);
  LAYER_OK(h, l, h->L - 1);
  if (!host || ld < (size_t)h->nf[l]) return fail(h, B2_ERR_INVALID, "bad host matrix");
  const int rows = h->nf[l + 1], cols = h->nf[l];
  CK(h, cudaMemcpy2DAsync(h->w[l], (size_t)cols * 4, host, ld * 4, (size_t)cols * 4, rows, cudaMemcpyHostToDevice,
                          h->s_main));
  if (h->op_type == T_BF16) {
    CK(h, convert_f32_to_bf16(h->w[l], h->w16[l], (size_t)rows * cols, h->s_main));
    ++h->launches;
  }
  if (h->x3) {
    CK(h, split_lo_launch(h->w[l], h->w_lo[l], (size_t)rows * cols, h->s_main));
    ++h->launches;
  }
  CK(h, cudaStreamSynchronize(h->s_main));
  return B2_OK;
}

int b2_download_weights(b2_handle* h, int l, float* host, size_t ld) {
  ENTER(h);
  LAYER_OK(h, l, h->L - 1);
  if (!host || ld < (size_t)h->nf[l]) return fail(h, B2_ERR_INVALID, "bad host matrix");
  int rc = gather_masters(h);  // collective when ranks hold current masters only for their own slices
  if (rc) return rc;
  return download_matrix(h, h->w[l], T_F32, host, ld, h->nf[l + 1], h->nf[l]);
}

int b2_upload_input(b2_handle* h, const float* host, size_t ld) {
  ENTER(h);
  if (!host || ld < (size_t)h->nf[0]) return fail(h, B2_ERR_INVALID, "bad host matrix");
  int rc = upload_matrix(h, h->act[0], h->op_type, host + (size_t)h->b0 * ld, ld, h->bl, h->nf[0]);
  if (rc) return rc;
  if (h->x3 && h->bl > 0) {
    CK(h, split_lo_launch(static_cast<const float*>(h->act[0]), h->act_lo[0], (size_t)h->bl * h->nf[0], h->s_main));
    ++h->launches;
  }
  CK(h, cudaStreamSynchronize(h->s_main));
  return B2_OK;
}

int b2_upload_target(b2_handle* h, const float* host, size_t ld) {
  ENTER(h);
  if (!host || ld < (size_t)h->nf[h->L]) return fail(h, B2_ERR_INVALID, "bad host matrix");
  int rc = upload_matrix(h, h->target, T_F32, host + (size_t)h->b0 * ld, ld, h->bl, h->nf[h->L]);
  if (rc) return rc;
  CK(h, cudaStreamSynchronize(h->s_main));
  return B2_OK;
}

int b2_download_activation(b2_handle* h, int l, float* host, size_t ld) {
  ENTER(h);
  LAYER_OK(h, l, h->L);
  if (!host || ld < (size_t)h->nf[l]) return fail(h, B2_ERR_INVALID, "bad host matrix");
  if (l == h->L) return download_matrix(h, h->y, T_F32, host + (size_t)h->b0 * ld, ld, h->bl, h->nf[l]);
  return download_matrix(h, h->act[l], h->op_type, host + (size_t)h->b0 * ld, ld, h->bl, h->nf[l]);
}

int b2_download_dz(b2_handle* h, int l, float* host, size_t ld) {
  ENTER(h);
  LAYER_OK(h, l, h->L - 1);
  if (!host || ld < (size_t)h->nf[l + 1]) return fail(h, B2_ERR_INVALID, "bad host matrix");
  return download_matrix(h, h->dz[l], h->op_type, host + (size_t)h->b0 * ld, ld, h->bl, h->nf[l + 1]);
}

int b2_download_input_grad(b2_handle* h, float* host, size_t ld) {
  ENTER(h);
  if (!host || ld < (size_t)h->nf[0]) return fail(h, B2_ERR_INVALID, "bad host matrix");
  return download_matrix(h, h->dinput, h->op_type, host + (size_t)h->b0 * ld, ld, h->bl, h->nf[0]);
}

int b2_download_weight_grad(b2_handle* h, int l, float* host, size_t ld) {
  ENTER(h);
  LAYER_OK(h, l, h->L - 1);
  if (!host || ld < (size_t)h->nf[l]) return fail(h, B2_ERR_INVALID, "bad host matrix");
  return download_matrix(h, h->dw[l], h->grad_type, host, ld, h->nf[l + 1], h->nf[l]);
}

int b2_upload_weight_grad(b2_handle* h, int l, const float* host, size_t ld) {
  ENTER(h);
  LAYER_OK(h, l, h->L - 1);
  if (!host || ld < (size_t)h->nf[l]) return fail(h, B2_ERR_INVALID, "bad host matrix");
  int rc = upload_matrix(h, h->dw[l], h->grad_type, host, ld, h->nf[l + 1], h->nf[l]);
  if (rc) return rc;
  CK(h, cudaStreamSynchronize(h->s_main));
  return B2_OK;
}

int b2_set_lr(b2_handle* h, float lr) {
  if (!h) return B2_ERR_INVALID;
  if (h->graph_exec) {  // the step graph has the old value baked in
    cudaGraphExecDestroy(h->graph_exec);
    h->graph_exec = nullptr;
  }
  h->cfg.lr = lr;
  return B2_OK;
}

int b2_sync(b2_handle* h) {
  ENTER(h);
  CK(h, cudaStreamSynchronize(h->s_main));
  CK(h, cudaStreamSynchronize(h->s_comm));
  CK(h, cudaStreamSynchronize(h->s_upd));
  CK(h, cudaStreamSynchronize(h->s_wg));
  return check_status(h);
}

static int capture_graph(b2_handle* h) {
  cudaGraph_t graph = nullptr;
  CK(h, cudaStreamBeginCapture(h->s_main, cudaStreamCaptureModeThreadLocal));
  int rc = B2_OK;
  if (h->cfg.overlap) {  // fork the side stream into the capture
    cudaEventRecord(h->ev_fork, h->s_main);
    cudaStreamWaitEvent(h->s_comm, h->ev_fork, 0);
  }
  for (auto& p : h->upd_pending) p = 0;
  const long long l0 = h->launches, t0 = h->tc_launches;
  rc = enqueue_step(h, false);
  if (rc == B2_OK) rc = join_streams(h);
  h->launches = l0;  // launches are counted per replay
  h->tc_launches = t0;
  cudaError_t e = cudaStreamEndCapture(h->s_main, &graph);
  if (rc != B2_OK) {
    if (graph) cudaGraphDestroy(graph);
    return rc;
  }
  if (e != cudaSuccess) return fail(h, B2_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
  e = cudaGraphInstantiate(&h->graph_exec, graph, 0);
  cudaGraphDestroy(graph);
  if (e != cudaSuccess) return fail(h, B2_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
  return B2_OK;
}

static long long launches_per_step(const b2_handle* h, long long* tc) {
  long long n = 0, t = 0;
  for (int l = 0; l < h->L; ++l) {
    for (const Site* s : {&h->fwd[l], &h->wgrad[l], &h->dgrad[l]})
      if (s->active) {
        ++n;
        if (s->plan) ++t;
      }
    ++n;  // SGD
  }
  if ((size_t)h->bl * h->nf[h->L]) ++n;  // output gradient
  if (tc) *tc = t;
  return n;
}

int b2_step(b2_handle* h, int iters) {
  ENTER(h);
  if (iters < 0) return fail(h, B2_ERR_INVALID, "iters < 0");
  if (h->async_issued != h->async_waited) return fail(h, B2_ERR_STATE, "pipelined steps in flight: b2_wait_loss first");
  if (iters == 0) return B2_OK;
  const bool timed = h->cfg.collect_timing != 0;
  const bool graph = h->cfg.use_graph && !timed;
  int rc;
  if (graph && !h->graph_exec) {
    CK(h, cudaStreamSynchronize(h->s_main));
    CK(h, cudaStreamSynchronize(h->s_comm));
    CK(h, cudaStreamSynchronize(h->s_upd));
    if (h->comm) {
      // connect the communicator outside the capture: each bucket's collective once, in place on
      // the gradient slab, whose contents are dead until the step's weight-gradient GEMMs rewrite them
      for (int l = h->L - 1; l >= 0; --l) {
        if (h->bucket_low[l] != l) continue;
        if (bucket_sharded(h, l)) {  // the weights of all ranks are equal: gathering them changes nothing
          if ((rc = bucket_reduce_scatter(h, l, h->bucket_high[l], h->s_comm, false))) return rc;
          if ((rc = bucket_allgather(h, l, h->bucket_high[l], h->s_comm, false))) return rc;
        } else if ((rc = bucket_allreduce(h, l, h->bucket_high[l], h->s_comm, false))) {
          return rc;
        }
      }
      CK(h, cudaStreamSynchronize(h->s_comm));
    }
    if ((rc = capture_graph(h))) return rc;
  }
  if (timed) {  // one event pair per (step, layer, phase): nothing is read back before the end
    h->ev_phase.assign((size_t)iters * h->L * B2_T_NUM * 2, nullptr);
    for (auto& ev : h->ev_phase) CK(h, cudaEventCreate(&ev));
  }
  CK(h, cudaEventRecord(h->ev_t0, h->s_main));
  for (int it = 0; it < iters; ++it) {
    if (graph) {
      CK(h, cudaGraphLaunch(h->graph_exec, h->s_main));
      long long t = 0;
      h->launches += launches_per_step(h, &t);
      h->tc_launches += t;
    } else {
      h->ev_iter = it;
      if ((rc = enqueue_step(h, timed))) return rc;
    }
  }
  if (!graph && (rc = join_streams(h))) return rc;
  CK(h, cudaEventRecord(h->ev_t1, h->s_main));
  CK(h, cudaStreamSynchronize(h->s_main));
  CK(h, cudaStreamSynchronize(h->s_comm));
  CK(h, cudaStreamSynchronize(h->s_upd));
  float ms = 0.f;
  CK(h, cudaEventElapsedTime(&ms, h->ev_t0, h->ev_t1));
  h->step_ms += ms;
  h->steps += iters;
  if (timed) {
    h->trace.clear();
    for (int it = 0; it < iters; ++it) {
      h->ev_iter = it;
      for (int l = 0; l < h->L; ++l)
        for (int ph = 0; ph < B2_T_NUM; ++ph) {
          float pm = 0.f, t0 = 0.f;
          if (cudaEventElapsedTime(&pm, phase_ev(h, l, ph, 0), phase_ev(h, l, ph, 1)) == cudaSuccess) {
            h->phase_ms[(size_t)l * B2_T_NUM + ph] += pm;
            if (cudaEventElapsedTime(&t0, h->ev_t0, phase_ev(h, l, ph, 0)) == cudaSuccess)
              h->trace.push_back({it, l, ph, t0, pm});
          } else {
            cudaGetLastError();  // phase not recorded in this configuration (e.g. no allreduce)
          }
        }
    }
    for (auto ev : h->ev_phase) cudaEventDestroy(ev);
    h->ev_phase.clear();
    h->ev_iter = 0;
    // forward / weight-gradient / input-gradient GEMMs overlap each other (two streams): the
    // length of the union of their intervals is the time the GEMMs really occupied
    std::vector<std::pair<float, float>> iv;
    for (const auto& e : h->trace)
      if (e.phase == B2_T_FWD || e.phase == B2_T_WGT_GRAD || e.phase == B2_T_BWD)
        iv.push_back({e.start_ms, e.start_ms + e.dur_ms});
    std::sort(iv.begin(), iv.end());
    float cur_b = 0.f, cur_e = -1.f;
    for (const auto& x : iv) {
      if (cur_e < 0.f) { cur_b = x.first; cur_e = x.second; }
      else if (x.first <= cur_e) { if (x.second > cur_e) cur_e = x.second; }
      else { h->gemm_busy_ms += cur_e - cur_b; cur_b = x.first; cur_e = x.second; }
    }
    if (cur_e >= 0.f) h->gemm_busy_ms += cur_e - cur_b;
  }
  return check_status(h);
}

int b2_loss(b2_handle* h, double* loss) {
  ENTER(h);
  if (!loss) return fail(h, B2_ERR_INVALID, "null output");
  CK(h, cudaMemcpyAsync(loss, h->loss_dev, sizeof(double), cudaMemcpyDeviceToHost, h->s_main));
  CK(h, cudaStreamSynchronize(h->s_main));
  return B2_OK;
}

int b2_train_step_host(b2_handle* h, const float* x, size_t ldx, const float* t, size_t ldt, double* loss) {
  ENTER(h);
  if (!x || ldx < (size_t)h->nf[0]) return fail(h, B2_ERR_INVALID, "bad input matrix");
  int rc;
  // fwd(0) of this step must not start before the copy; the copy must not start
  // before the previous step stopped reading act[0] - both hold on the main stream.
  if ((rc = upload_matrix(h, h->act[0], h->op_type, x + (size_t)h->b0 * ldx, ldx, h->bl, h->nf[0]))) return rc;
  if (h->x3 && h->bl > 0) {
    CK(h, split_lo_launch(static_cast<const float*>(h->act[0]), h->act_lo[0], (size_t)h->bl * h->nf[0], h->s_main));
    ++h->launches;
  }
  if (t) {
    if (ldt < (size_t)h->nf[h->L]) return fail(h, B2_ERR_INVALID, "bad target matrix");
    if ((rc = upload_matrix(h, h->target, T_F32, t + (size_t)h->b0 * ldt, ldt, h->bl, h->nf[h->L]))) return rc;
  }
  if ((rc = b2_step(h, 1))) return rc;
  if (loss) return b2_loss(h, loss);
  return B2_OK;
}

int b2_train_step_host_async(b2_handle* h, const float* x, size_t ldx, const float* t, size_t ldt) {
  ENTER(h);
  if (!x || ldx < (size_t)h->nf[0]) return fail(h, B2_ERR_INVALID, "bad input matrix");
  if (t && ldt < (size_t)h->nf[h->L]) return fail(h, B2_ERR_INVALID, "bad target matrix");
  if (h->cfg.collect_timing || h->cfg.use_graph)
    return fail(h, B2_ERR_STATE, "the pipelined host-fed step needs collect_timing = 0 and use_graph = 0");
  if (h->async_issued - h->async_waited >= 2)
    return fail(h, B2_ERR_STATE, "two steps already in flight: call b2_wait_loss first");
  const int slot = (int)(h->async_issued & 1);
  const int rows = h->bl, f0 = h->nf[0], fl = h->nf[h->L];
  int rc;
  // the copy may start once the step that last computed on this slot is done with it
  if (h->slot_used[slot]) CK(h, cudaStreamWaitEvent(h->s_copy, h->ev_slot_free[slot], 0));
  if (rows > 0) {
    void* act0 = slot ? h->act0_alt : h->act[0];
    void* land = h->op_type == T_BF16 ? (void*)h->xstage[slot] : act0;
    CK(h, copy_rows(land, (size_t)f0 * 4, x + (size_t)h->b0 * ldx, ldx * 4, (size_t)f0 * 4, (size_t)rows,
                    cudaMemcpyHostToDevice, h->s_copy));
    if (h->op_type == T_BF16) {
      CK(h, convert_f32_to_bf16(h->xstage[slot], (__nv_bfloat16*)act0, (size_t)rows * f0, h->s_copy));
      ++h->launches;
    }
    if (h->x3) {
      CK(h, split_lo_launch(static_cast<const float*>(act0), slot ? h->act0_alt_lo : h->act_lo[0], (size_t)rows * f0,
                            h->s_copy));
      ++h->launches;
    }
    if (t)
      CK(h, copy_rows(slot ? h->target_alt : h->target, (size_t)fl * 4, t + (size_t)h->b0 * ldt, ldt * 4,
                      (size_t)fl * 4, (size_t)rows, cudaMemcpyHostToDevice, h->s_copy));
  }
  CK(h, cudaEventRecord(h->ev_copied[slot], h->s_copy));
  CK(h, cudaStreamWaitEvent(h->s_main, h->ev_copied[slot], 0));
  if ((rc = enqueue_step(h, false, slot))) return rc;
  CK(h, cudaEventRecord(h->ev_slot_free[slot], h->s_main));
  h->slot_used[slot] = true;
  CK(h, cudaMemcpyAsync(h->loss_host + slot, h->loss_dev + slot, sizeof(double), cudaMemcpyDeviceToHost,
                        h->s_main));
  CK(h, cudaEventRecord(h->ev_loss[slot], h->s_main));
  ++h->async_issued;
  ++h->steps;
  return B2_OK;
}

int b2_wait_loss(b2_handle* h, double* loss) {
  ENTER(h);
  if (h->async_waited >= h->async_issued) return fail(h, B2_ERR_STATE, "no step in flight");
  const int slot = (int)(h->async_waited & 1);
  CK(h, cudaEventSynchronize(h->ev_loss[slot]));
  if (loss) *loss = h->loss_host[slot];
  ++h->async_waited;
  if (h->async_waited == h->async_issued) {  // pipeline drained: also let the updates finish
    int rc = join_streams(h);
    if (rc) return rc;
    CK(h, cudaStreamSynchronize(h->s_main));
    return check_status(h);
  }
  return B2_OK;
}

int b2_host_alloc(void** ptr, size_t bytes) {
  if (!ptr) return B2_ERR_INVALID;
  cudaError_t e = cudaHostAlloc(ptr, bytes, cudaHostAllocDefault);
  if (e != cudaSuccess) return fail(nullptr, B2_ERR_CUDA, "cudaHostAlloc: %s", cudaGetErrorString(e));
  return B2_OK;
}

int b2_host_alloc_near(void** ptr, size_t bytes, int device, int* numa_node) {
  if (!ptr) return B2_ERR_INVALID;
  if (numa_node) *numa_node = -1;
  cpu_set_t old_set, node_set;
  bool bound = false;
  int node = -1;
  char bus[32] = "";
  if (cudaDeviceGetPCIBusId(bus, sizeof bus, device) == cudaSuccess &&
      sched_getaffinity(0, sizeof old_set, &old_set) == 0) {
    for (char* c = bus; *c; ++c) *c = (char)tolower((unsigned char)*c);
    char path[128];
    snprintf(path, sizeof path, "/sys/bus/pci/devices/%s/numa_node", bus);
    if (FILE* f = fopen(path, "r")) {
      if (fscanf(f, "%d", &node) != 1) node = -1;
      fclose(f);
    }
    if (node >= 0) {
      // "0-31,64-95": the CPUs of the node, kept only where this thread may already run
      CPU_ZERO(&node_set);
      int kept = 0;
      snprintf(path, sizeof path, "/sys/devices/system/node/node%d/cpulist", node);
      if (FILE* f = fopen(path, "r")) {
        int lo, hi;
        while (fscanf(f, "%d", &lo) == 1) {
          hi = lo;
          int ch = fgetc(f);
          if (ch == '-') {
            if (fscanf(f, "%d", &hi) != 1) break;
            ch = fgetc(f);
          }
          for (int c = lo; c <= hi && c < CPU_SETSIZE; ++c)
            if (c >= 0 && CPU_ISSET(c, &old_set)) {
              CPU_SET(c, &node_set);
              ++kept;
            }
          if (ch != ',') break;
        }
        fclose(f);
      }
      if (kept > 0 && sched_setaffinity(0, sizeof node_set, &node_set) == 0) bound = true;
    }
  }
  cudaError_t e = cudaHostAlloc(ptr, bytes, cudaHostAllocDefault);
  if (e == cudaSuccess && bound) memset(*ptr, 0, bytes);  // touched from the node's CPUs
  if (bound) sched_setaffinity(0, sizeof old_set, &old_set);
  if (e != cudaSuccess) return fail(nullptr, B2_ERR_CUDA, "cudaHostAlloc: %s", cudaGetErrorString(e));
  if (numa_node && bound) *numa_node = node;
  return B2_OK;
}

int b2_host_free(void* ptr) {
  cudaError_t e = cudaFreeHost(ptr);
  if (e != cudaSuccess) return fail(nullptr, B2_ERR_CUDA, "cudaFreeHost: %s", cudaGetErrorString(e));
  return B2_OK;
}

int b2_allreduce_sgd(b2_handle* h, int l) {
  ENTER(h);
  LAYER_OK(h, l, h->L - 1);
  int rc;
  const bool has_ar = h->cfg.world_size > 1 && h->cfg.allreduce;
  if (has_ar && !h->comm)
    return fail(h, B2_ERR_STATE, "the communicator of this job was aborted after an error; destroy the handles");
  if (has_ar && h->bucket_low[l] == l && h->bucket_high[l] == l && bucket_sharded(h, l)) {
    // the layer is a bucket of its own: the reference's route (mlp_omp.cc:297-323)
    if ((rc = bucket_reduce_scatter(h, l, l, h->s_main, false))) return rc;
    if ((rc = bucket_shard_sgd(h, l, l, h->s_main, false))) return rc;
    if ((rc = bucket_allgather(h, l, l, h->s_main, false))) return rc;
  } else {
    // a layer inside a larger bucket: the slices of the ranks follow the bucket, not the layer,
    // so sum the whole layer everywhere and update it everywhere (needs current masters everywhere)
    if ((rc = gather_masters(h))) return rc;
    if ((rc = layer_update(h, l, h->s_main, false))) return rc;
    if ((rc = layer_sgd(h, l, h->s_main, false))) return rc;
  }
  CK(h, cudaStreamSynchronize(h->s_main));
  return check_status(h);  // a peer-memory sum that gave up must not pass for a result
}

int b2_allreduce(b2_handle* h, void* dev_buf, size_t count, int dtype) {
  ENTER(h);
  if (!dev_buf || count == 0) return fail(h, B2_ERR_INVALID, "bad buffer");
  if (dtype != B2_DTYPE_F32 && dtype != B2_DTYPE_BF16) return fail(h, B2_ERR_INVALID, "bad dtype");
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, dev_buf) != cudaSuccess || attr.type != cudaMemoryTypeDevice ||
      attr.device != h->cfg.device) {
    cudaGetLastError();
    return fail(h, B2_ERR_INVALID, "not a device pointer of GPU %d", h->cfg.device);
  }
  if (h->cfg.world_size > 1) {
    if (!h->comm) return fail(h, B2_ERR_STATE, "the handle was created without a communicator (allreduce = 0)");
    NCK(h, nccl_api().AllReduce(dev_buf, dev_buf, count, dtype == B2_DTYPE_BF16 ? ncclBfloat16 : ncclFloat32, ncclSum,
                                h->comm, h->s_main));
  }
  CK(h, cudaStreamSynchronize(h->s_main));
  return check_comm(h);
}

namespace {
// What b2_p2p_describe writes: where this rank's gradient slab lives and how to map it.
struct P2pDesc {
  uint32_t magic;
  int32_t device;
  int64_t pid;
  uint64_t ptr, slab_bytes, flags_off;
  cudaIpcMemHandle_t ipc;
};
static_assert(sizeof(P2pDesc) <= B2_P2P_DESC_BYTES, "descriptor does not fit");
constexpr uint32_t P2P_MAGIC = 0x62327032u;
}  // namespace

int b2_p2p_describe(b2_handle* h, void* desc) {
  ENTER(h);
  if (!desc) return fail(h, B2_ERR_INVALID, "null descriptor");
  if (h->cfg.world_size < 2 || h->cfg.world_size > P2P_MAX_RANKS)
    return fail(h, B2_ERR_UNSUPPORTED, "the peer-memory path serves 2 to %d ranks", P2P_MAX_RANKS);
  if (h->grad_type != T_F32) return fail(h, B2_ERR_UNSUPPORTED, "the peer-memory path sums fp32 gradients only");
  if (h->nccl_ub) return fail(h, B2_ERR_UNSUPPORTED, "the peer-memory path cannot share slabs allocated by NCCL (B2_NCCL_UB)");
  P2pDesc d;
  memset(&d, 0, sizeof d);
  d.magic = P2P_MAGIC;
  d.device = h->cfg.device;
  d.pid = (int64_t)getpid();
  d.ptr = (uint64_t)(uintptr_t)h->dw_slab;
  d.slab_bytes = h->slab_bytes;
  d.flags_off = h->p2p_flags_off;
  CK(h, cudaIpcGetMemHandle(&d.ipc, h->dw_slab));
  memset(desc, 0, B2_P2P_DESC_BYTES);
  memcpy(desc, &d, sizeof d);
  return B2_OK;
}

int b2_p2p_connect(b2_handle* h, const void* descs, size_t max_bytes) {
  ENTER(h);
  if (!descs) return fail(h, B2_ERR_INVALID, "null descriptors");
  if (h->p2p_ready) return fail(h, B2_ERR_STATE, "already connected");
  const int world = h->cfg.world_size, rank = h->cfg.rank;
  if (world < 2 || world > P2P_MAX_RANKS)
    return fail(h, B2_ERR_UNSUPPORTED, "the peer-memory path serves 2 to %d ranks", P2P_MAX_RANKS);
  if (h->grad_type != T_F32) return fail(h, B2_ERR_UNSUPPORTED, "the peer-memory path sums fp32 gradients only");
  for (int r = 0; r < world; ++r) {
    P2pDesc d;
    memcpy(&d, static_cast<const char*>(descs) + (size_t)r * B2_P2P_DESC_BYTES, sizeof d);
    if (d.magic != P2P_MAGIC) return fail(h, B2_ERR_INVALID, "descriptor %d is not one of b2_p2p_describe", r);
    if (d.slab_bytes != h->slab_bytes || d.flags_off != h->p2p_flags_off)
      return fail(h, B2_ERR_INVALID, "rank %d was created for a different model", r);
    char* base = nullptr;
    if (r == rank) {
      if (d.ptr != (uint64_t)(uintptr_t)h->dw_slab) return fail(h, B2_ERR_INVALID, "descriptor %d is not this rank's", r);
      base = static_cast<char*>(h->dw_slab);
    } else if (d.pid == (int64_t)getpid()) {
      // another handle of this process: its pointer is valid here once peer access is on
      if (d.device != h->cfg.device) {
        int can = 0;
        CK(h, cudaDeviceCanAccessPeer(&can, h->cfg.device, d.device));
        if (!can) return fail(h, B2_ERR_UNSUPPORTED, "device %d cannot access device %d", h->cfg.device, d.device);
        cudaError_t e = cudaDeviceEnablePeerAccess(d.device, 0);
        if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
        else if (e != cudaSuccess) return fail(h, B2_ERR_CUDA, "cudaDeviceEnablePeerAccess: %s", cudaGetErrorString(e));
      }
      base = reinterpret_cast<char*>((uintptr_t)d.ptr);
    } else {
      void* mapped = nullptr;
      CK(h, cudaIpcOpenMemHandle(&mapped, d.ipc, cudaIpcMemLazyEnablePeerAccess));
      h->p2p_opened[r] = mapped;
      base = static_cast<char*>(mapped);
    }
    h->p2p_slab[r] = reinterpret_cast<float*>(base);
    h->p2p_flags[r] = reinterpret_cast<unsigned int*>(base + h->p2p_flags_off);
  }
  // buckets small enough for the peer path are summed in full on every rank and updated by every
  // rank from now on (also when the peer path later falls back to NCCL), so bring the masters up
  // to date first (every rank is in this call)
  int rc = gather_masters(h);
  if (rc) return rc;
  const size_t es = esize(h->grad_type);
  for (int l = 0; l < h->L; ++l) {
    if (h->bucket_low[l] != l) continue;
    const size_t bytes = (h->dw_off[l] + (size_t)h->nf[l + 1] * h->nf[l] - h->dw_off[h->bucket_high[l]]) * es;
    h->bucket_full[l] = (max_bytes > 0 && bytes <= max_bytes) ? 1 : 0;
  }
  h->p2p_max_bytes = max_bytes;
  h->p2p_epoch = 0;
  h->p2p_ready = max_bytes > 0;
  return B2_OK;
}

int b2_p2p_set_wait_ms(b2_handle* h, int ms) {
  if (!h) return B2_ERR_INVALID;
  if (ms < 1 || ms > 60000) return fail(h, B2_ERR_INVALID, "wait limit must be 1 .. 60000 ms");
  h->p2p_wait_ns = (unsigned long long)ms * 1000000ull;
  return B2_OK;
}

int b2_p2p_emulate(int device, int world, float* const* bufs, size_t count) {
  return b2_p2p_emulate_opts(device, world, bufs, count, 1000, -1);
}

int b2_p2p_emulate_opts(int device, int world, float* const* bufs, size_t count, int wait_ms, int lagging_rank) {
  if (world < 2 || world > P2P_MAX_RANKS || !bufs || count == 0 || wait_ms < 1 || wait_ms > 60000 ||
      lagging_rank >= world)
    return fail(nullptr, B2_ERR_INVALID, "bad arguments");
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) return fail(nullptr, B2_ERR_CUDA, "cudaSetDevice: %s", cudaGetErrorString(e));
  // one allocation: world slabs (count floats, padded) + world flag blocks + counters + status + parameters
  const size_t slab = (count * sizeof(float) + 255) / 256 * 256;
  const size_t off_flags = slab * world, off_cnt = off_flags + 256 * (size_t)world;
  const size_t off_status = off_cnt + 256, off_params = off_status + 256;
  const size_t total = off_params + sizeof(P2pParams) * world;
  char* mem = nullptr;
  unsigned int status = 0;
  int rc = B2_OK;
  P2pParams host[P2P_MAX_RANKS];
  if ((e = cudaMalloc((void**)&mem, total)) != cudaSuccess)
    return fail(nullptr, B2_ERR_CUDA, "cudaMalloc: %s", cudaGetErrorString(e));
  do {
    if ((e = cudaMemset(mem, 0, total)) != cudaSuccess) break;
    for (int r = 0; r < world; ++r) {
      if ((e = cudaMemcpy(mem + slab * r, bufs[r], count * sizeof(float), cudaMemcpyHostToDevice)) != cudaSuccess) break;
      P2pParams& p = host[r];
      memset(&p, 0, sizeof p);
      for (int q = 0; q < world; ++q) {
        p.slab[q] = reinterpret_cast<float*>(mem + slab * q);
        p.flags[q] = reinterpret_cast<unsigned int*>(mem + off_flags + 256 * (size_t)q);
      }
      p.world = world;
      p.rank = r;
      p.offset = 0;
      p.count = count;
      // a lagging rank is one call behind the others: it announces call 1 while they wait for call 2
      p.epoch = (r == lagging_rank) ? 1u : 2u;
      p.wait_ns = (unsigned long long)wait_ms * 1000000ull;
      p.ctas_done = reinterpret_cast<unsigned int*>(mem + off_cnt) + r;
      p.status = reinterpret_cast<unsigned int*>(mem + off_status);
    }
    if (e != cudaSuccess) break;
    if ((e = cudaMemcpy(mem + off_params, host, sizeof(P2pParams) * world, cudaMemcpyHostToDevice)) != cudaSuccess) break;
    if ((e = p2p_allreduce_emulated_launch(reinterpret_cast<const P2pParams*>(mem + off_params), host[0], 0)) !=
        cudaSuccess)
      break;
    if ((e = cudaDeviceSynchronize()) != cudaSuccess) break;
    if ((e = cudaMemcpy(&status, mem + off_status, sizeof status, cudaMemcpyDeviceToHost)) != cudaSuccess) break;
    if (status != 0) {
      rc = fail(nullptr, B2_ERR_TIMEOUT, "emulated ranks gave up waiting for one another (code %u)", status);
      break;
    }
    for (int r = 0; r < world && e == cudaSuccess; ++r)
      e = cudaMemcpy(bufs[r], mem + slab * r, count * sizeof(float), cudaMemcpyDeviceToHost);
  } while (0);
  cudaFree(mem);
  if (e != cudaSuccess) return fail(nullptr, B2_ERR_CUDA, "peer-allreduce emulation: %s", cudaGetErrorString(e));
  return rc;
}

int b2_collective_bench(b2_handle* h, int kind, size_t count, int dtype, int warmup, int iters, double* ms_per_iter,
                        double* checksum) {
  ENTER(h);
  if (count == 0 || iters < 1 || warmup < 0) return fail(h, B2_ERR_INVALID, "bad sweep arguments");
  if (dtype != B2_DTYPE_F32 && dtype != B2_DTYPE_BF16) return fail(h, B2_ERR_INVALID, "bad dtype");
  if (kind < 0 || kind > 2) return fail(h, B2_ERR_INVALID, "kind: 0 allreduce, 1 reduce-scatter, 2 allgather");
  const int type = dtype == B2_DTYPE_BF16 ? T_BF16 : T_F32;
  const int ntype = dtype == B2_DTYPE_BF16 ? ncclBfloat16 : ncclFloat32;
  const int world = h->cfg.world_size;
  const bool multi = world > 1 && h->comm;
  if (kind != 0 && count % (size_t)world != 0) return fail(h, B2_ERR_INVALID, "count must divide by the number of ranks");
  const size_t per = count / (size_t)world;
  void *src = nullptr, *dst = nullptr;
  CK(h, cudaMalloc(&src, count * esize(type)));
  cudaError_t e = cudaMalloc(&dst, count * esize(type));
  if (e != cudaSuccess) {
    cudaFree(src);
    return fail(h, B2_ERR_CUDA, "cudaMalloc: %s", cudaGetErrorString(e));
  }
  int rc = B2_OK;
  auto run = [&]() -> int {
    if (!multi) return B2_OK;  // one rank: nothing to exchange
    char* s8 = static_cast<char*>(src);
    char* d8 = static_cast<char*>(dst);
    if (kind == 0) {
      NCK(h, nccl_api().AllReduce(src, dst, count, ntype, ncclSum, h->comm, h->s_main));
    } else if (kind == 1) {
      NCK(h, nccl_api().ReduceScatter(src, d8 + (size_t)h->cfg.rank * per * esize(type), per, ntype, ncclSum, h->comm,
                                      h->s_main));
    } else {
      NCK(h, nccl_api().AllGather(s8 + (size_t)h->cfg.rank * per * esize(type), dst, per, ntype, h->comm, h->s_main));
    }
    return B2_OK;
  };
  do {
    if (fill_uniform_launch(src, type, count, (uint64_t)h->cfg.rank, -1.f, 1.f, h->s_main) != cudaSuccess) {
      rc = fail(h, B2_ERR_CUDA, "fill failed");
      break;
    }
    ++h->launches;
    if (!multi) cudaMemcpyAsync(dst, src, count * esize(type), cudaMemcpyDeviceToDevice, h->s_main);
    for (int i = 0; i < warmup && rc == B2_OK; ++i) rc = run();
    if (rc) break;
    cudaEventRecord(h->ev_t0, h->s_main);
    for (int i = 0; i < iters && rc == B2_OK; ++i) rc = run();
    if (rc) break;
    cudaEventRecord(h->ev_t1, h->s_main);
    if (cudaStreamSynchronize(h->s_main) != cudaSuccess) {
      rc = fail(h, B2_ERR_CUDA, "collective sweep: %s", cudaGetErrorString(cudaGetLastError()));
      break;
    }
    float ms = 0.f;
    cudaEventElapsedTime(&ms, h->ev_t0, h->ev_t1);
    if (ms_per_iter) *ms_per_iter = multi ? (double)ms / iters : 0.0;
    if (checksum) {
      const size_t n = count < 4096 ? count : 4096;
      std::vector<float> host(n);
      if (type == T_BF16) {
        std::vector<__nv_bfloat16> hb(n);
        cudaMemcpy(hb.data(), dst, n * 2, cudaMemcpyDeviceToHost);
        for (size_t i = 0; i < n; ++i) host[i] = __bfloat162float(hb[i]);
      } else {
        cudaMemcpy(host.data(), dst, n * 4, cudaMemcpyDeviceToHost);
      }
      double s = 0;
      for (size_t i = 0; i < n; ++i) s += host[i];
      *checksum = s;
    }
    rc = check_comm(h);
  } while (0);
  cudaFree(src);
  cudaFree(dst);
  return rc;
}

int b2_allreduce_bench(b2_handle* h, size_t count, int dtype, int warmup, int iters, double* ms_per_iter,
                       double* checksum) {
  return b2_collective_bench(h, 0, count, dtype, warmup, iters, ms_per_iter, checksum);
}

int b2_sgd_bench(b2_handle* h, size_t nparams, int grad_dtype, int with_bf16_copy, int warmup, int iters,
                 double* ms_per_iter, double* bytes_per_iter) {
  ENTER(h);
  if (nparams == 0 || iters < 1 || warmup < 0) return fail(h, B2_ERR_INVALID, "bad arguments");
  if (grad_dtype != B2_DTYPE_F32 && grad_dtype != B2_DTYPE_BF16) return fail(h, B2_ERR_INVALID, "bad dtype");
  const int gt = grad_dtype == B2_DTYPE_BF16 ? T_BF16 : T_F32;
  const size_t per_param = 4 + esize(gt) + 4 + (with_bf16_copy ? 2 : 0);  // read w, read g, write w (+ write bf16 copy)
  // parameter sets in rotation, together several times the L2, so that every launch streams from HBM
  int sets = (int)((size_t(512) << 20) / (nparams * per_param)) + 1;
  if (sets > 16) sets = 16;
  if (sets < 2) sets = 2;
  std::vector<float*> w(sets, nullptr);
  std::vector<void*> g(sets, nullptr);
  std::vector<__nv_bfloat16*> w16(sets, nullptr);
  int rc = B2_OK;
  do {
    for (int i = 0; i < sets; ++i) {
      if (cudaMalloc((void**)&w[i], nparams * 4) != cudaSuccess || cudaMalloc(&g[i], nparams * esize(gt)) != cudaSuccess ||
          (with_bf16_copy && cudaMalloc((void**)&w16[i], nparams * 2) != cudaSuccess)) {
        rc = fail(h, B2_ERR_CUDA, "cudaMalloc: %s", cudaGetErrorString(cudaGetLastError()));
        break;
      }
      fill_uniform_launch(w[i], T_F32, nparams, 11 + i, -1.f, 1.f, h->s_main);
      fill_uniform_launch(g[i], gt, nparams, 31 + i, -1.f, 1.f, h->s_main);
    }
    if (rc) break;
    cudaError_t e = cudaSuccess;
    for (int i = 0; i < warmup && e == cudaSuccess; ++i)
      e = sgd_launch(w[i % sets], g[i % sets], gt, w16[i % sets], nparams, 1e-6f, h->sms, h->s_main);
    if (e == cudaSuccess) e = cudaEventRecord(h->ev_t0, h->s_main);
    for (int i = 0; i < iters && e == cudaSuccess; ++i) {
      e = sgd_launch(w[(warmup + i) % sets], g[(warmup + i) % sets], gt, w16[(warmup + i) % sets], nparams, 1e-6f,
                     h->sms, h->s_main);
      ++h->launches;
    }
    if (e == cudaSuccess) e = cudaEventRecord(h->ev_t1, h->s_main);
    if (e == cudaSuccess) e = cudaStreamSynchronize(h->s_main);
    if (e != cudaSuccess) {
      rc = fail(h, B2_ERR_CUDA, "SGD benchmark: %s", cudaGetErrorString(e));
      break;
    }
    float ms = 0.f;
    cudaEventElapsedTime(&ms, h->ev_t0, h->ev_t1);
    if (ms_per_iter) *ms_per_iter = (double)ms / iters;
    if (bytes_per_iter) *bytes_per_iter = (double)(nparams * per_param);
  } while (0);
  for (int i = 0; i < sets; ++i) {
    cudaFree(w[i]); cudaFree(g[i]); cudaFree(w16[i]);
  }
  return rc;
}

int b2_set_timing(b2_handle* h, int collect_timing) {
  if (!h) return B2_ERR_INVALID;
  if (h->async_issued != h->async_waited) return fail(h, B2_ERR_STATE, "pipelined steps in flight");
  h->cfg.collect_timing = collect_timing ? 1 : 0;
  return B2_OK;
}

int b2_weights_fingerprint(b2_handle* h, int l, unsigned long long* out) {
  ENTER(h);
  LAYER_OK(h, l, h->L - 1);
  if (!out) return fail(h, B2_ERR_INVALID, "null output");
  unsigned long long* acc = h->fp_dev;
  const size_t n = (size_t)h->nf[l + 1] * h->nf[l];
  CK(h, cudaStreamSynchronize(h->s_main));
  CK(h, cudaMemsetAsync(acc, 0, sizeof *acc, h->s_main));
  if (h->op_type == T_BF16)
    CK(h, fingerprint_launch(h->w16[l], n * 2, acc, h->s_main));
  else
    CK(h, fingerprint_launch(h->w[l], n * 4, acc, h->s_main));
  ++h->launches;
  CK(h, cudaMemcpyAsync(out, acc, sizeof *out, cudaMemcpyDeviceToHost, h->s_main));
  CK(h, cudaStreamSynchronize(h->s_main));
  return B2_OK;
}

int b2_gemm_bench(b2_handle* h, int form, int m, int n, int k, int precision, int epilogue, int out_dtype, int sms,
                  int warmup, int iters, double* ms_per_iter) {
  ENTER(h);
  if (form < 0 || form > 2 || m < 1 || n < 1 || k < 1 || iters < 1 || warmup < 0)
    return fail(h, B2_ERR_INVALID, "bad GEMM benchmark arguments");
  if (precision < B2_PREC_FP32 || precision > B2_PREC_FP32_TC)
    return fail(h, B2_ERR_INVALID, "unknown precision %d", precision);
  if (epilogue < EPI_NONE || epilogue > EPI_MASK) return fail(h, B2_ERR_INVALID, "bad epilogue");
  const int in_type = precision == B2_PREC_BF16 ? T_BF16 : T_F32;
  const int out_type = out_dtype == B2_DTYPE_BF16 ? T_BF16 : T_F32;
  if (out_type == T_BF16 && in_type != T_BF16) return fail(h, B2_ERR_INVALID, "bf16 output needs BF16 precision");
  const size_t ea = (size_t)m * k, eb = (size_t)k * n, ec = (size_t)m * n;
  const size_t set_bytes = (ea + eb) * esize(in_type) + ec * esize(out_type) + (epilogue != EPI_NONE ? ec * esize(in_type) : 0);
  // operand sets used in rotation so that consecutive launches find nothing of theirs in the L2
  int sets = (int)((size_t(384) << 20) / set_bytes) + 1;
  if (sets > 16) sets = 16;
  if (sets < 1) sets = 1;
  struct Set { void *a, *b, *c, *x; float *a_lo, *b_lo, *c_lo; TcPlan* plan; GemmDesc d; };
  std::vector<Set> S(sets, Set{nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, GemmDesc{}});
  const bool x3 = precision == B2_PREC_FP32_TC && !h->cfg.force_simt;
  int rc = B2_OK;
  const bool tc = precision != B2_PREC_FP32 && !h->cfg.force_simt;
  // B2_TC_TRACE=1: per-tile timeline of CTA 0 of the last timed launch, printed to stderr
  unsigned long long* trace_dev = nullptr;
  if (tc && getenv("B2_TC_TRACE")) {
    cudaMalloc((void**)&trace_dev, TC_TRACE_WORDS * sizeof(unsigned long long));
    cudaMemset(trace_dev, 0, TC_TRACE_WORDS * sizeof(unsigned long long));
  }
  do {
    for (int i = 0; i < sets && rc == B2_OK; ++i) {
      Set& s = S[i];
      if (cudaMalloc(&s.a, ea * esize(in_type)) != cudaSuccess || cudaMalloc(&s.b, eb * esize(in_type)) != cudaSuccess ||
          cudaMalloc(&s.c, ec * esize(out_type)) != cudaSuccess ||
          (epilogue != EPI_NONE && cudaMalloc(&s.x, ec * esize(in_type)) != cudaSuccess)) {
        rc = fail(h, B2_ERR_CUDA, "cudaMalloc: %s", cudaGetErrorString(cudaGetLastError()));
        break;
      }
      fill_uniform_launch(s.a, in_type, ea, 7 + 3 * i, -1.f, 1.f, h->s_main);
      fill_uniform_launch(s.b, in_type, eb, 8 + 3 * i, -1.f, 1.f, h->s_main);
      if (x3) {
        if (cudaMalloc((void**)&s.a_lo, ea * 4) != cudaSuccess || cudaMalloc((void**)&s.b_lo, eb * 4) != cudaSuccess ||
            cudaMalloc((void**)&s.c_lo, ec * 4) != cudaSuccess) {
          rc = fail(h, B2_ERR_CUDA, "cudaMalloc: %s", cudaGetErrorString(cudaGetLastError()));
          break;
        }
        split_lo_launch(static_cast<const float*>(s.a), s.a_lo, ea, h->s_main);
        split_lo_launch(static_cast<const float*>(s.b), s.b_lo, eb, h->s_main);
      }
      if (s.x) fill_uniform_launch(s.x, in_type, ec, 9 + 3 * i, -1.f, 1.f, h->s_main);
      GemmDesc& d = s.d;
      d.M = m; d.N = n; d.K = k;
      d.A = s.a; d.B = s.b; d.C = s.c; d.ldc = n;
      if (form == 0) {         // forward: A m x k, B n x k
        d.sAm = k; d.sAk = 1; d.sBk = 1; d.sBn = k;
      } else if (form == 1) {  // weight gradient: A stored k x m, B stored k x n
        d.sAm = 1; d.sAk = m; d.sBk = n; d.sBn = 1;
      } else {                 // input gradient: A m x k, B k x n
        d.sAm = k; d.sAk = 1; d.sBk = n; d.sBn = 1;
      }
      d.aux = s.x; d.ldaux = n;
      d.alpha = 1.f; d.beta = 0.f;
      d.epilogue = epilogue;
      d.in_type = in_type; d.out_type = out_type;
      d.ws = nullptr; d.ws_flags = nullptr;
      d.A_lo = s.a_lo; d.B_lo = s.b_lo;
      d.C_lo = (x3 && form != 1) ? s.c_lo : nullptr;  // like the step: activations and gradients get a twin
      d.trace = trace_dev;
      if (tc) {
        char why[128] = "";
        s.plan = gemm_tc_plan_create(d, sms > 0 && sms <= h->sms ? sms : h->sms, why, sizeof why);
        if (!s.plan) rc = fail(h, B2_ERR_UNSUPPORTED, "tensor-core kernel refuses this GEMM: %s", why);
        // like the step: the ReLU bit plane (here: the first bytes of the auxiliary buffer) is written
        // by a forward epilogue and read by an input-gradient epilogue instead of the activation
        if (s.plan && n % 32 == 0 && epilogue == EPI_RELU)
          gemm_tc_plan_set_mask(s.plan, static_cast<uint32_t*>(s.x), nullptr, n / 32);
        if (s.plan && n % 32 == 0 && epilogue == EPI_MASK)
          gemm_tc_plan_set_mask(s.plan, nullptr, static_cast<const uint32_t*>(s.x), n / 32);
      }
    }
    if (rc) break;
    auto run = [&](int i) -> cudaError_t {
      Set& s = S[i % sets];
      ++h->launches;
      if (s.plan) {
        ++h->tc_launches;
        return gemm_tc_launch(s.plan, h->s_main, h->status_dev);
      }
      return gemm_simt_launch(s.d, h->s_main);
    };
    cudaError_t e = cudaSuccess;
    for (int i = 0; i < warmup && e == cudaSuccess; ++i) e = run(i);
    if (e == cudaSuccess) e = cudaEventRecord(h->ev_t0, h->s_main);
    for (int i = 0; i < iters && e == cudaSuccess; ++i) e = run(warmup + i);
    if (e == cudaSuccess) e = cudaEventRecord(h->ev_t1, h->s_main);
    if (e == cudaSuccess) e = cudaStreamSynchronize(h->s_main);
    if (e != cudaSuccess) {
      rc = fail(h, B2_ERR_CUDA, "GEMM benchmark: %s", cudaGetErrorString(e));
      break;
    }
    float ms = 0.f;
    cudaEventElapsedTime(&ms, h->ev_t0, h->ev_t1);
    if (ms_per_iter) *ms_per_iter = (double)ms / iters;
    if (trace_dev) {
      std::vector<unsigned long long> t(TC_TRACE_WORDS);
      cudaMemcpy(t.data(), trace_dev, t.size() * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
      fprintf(stderr, "tile: first MMA -> accumulator complete | complete -> released | released -> last store issued | "
                      "accumulator complete -> next tile's first MMA   (ns, CTA 0)\n");
      for (int i = 0; i < TC_TRACE_TILES && t[i * 4 + 1]; ++i)
        fprintf(stderr, "%3d: %8lld | %8lld | %8lld | %8lld\n", i, (long long)(t[i * 4 + 1] - t[i * 4]),
                (long long)(t[i * 4 + 2] - t[i * 4 + 1]), (long long)(t[i * 4 + 3] - t[i * 4 + 2]),
                (i + 1 < TC_TRACE_TILES && t[(i + 1) * 4]) ? (long long)(t[(i + 1) * 4] - t[i * 4 + 1]) : -1LL);
      const unsigned long long* c = t.data() + TC_TRACE_TILES * 4;
      if (c[0]) {
        fprintf(stderr, "second tile, per k-block (ns since its first): operands seen by the MMA warp | slot seen free by the "
                        "TMA warp | by the peer CTA's TMA warp (CTA-pair kernel)\n");
        for (int kb = 0; kb < TC_TRACE_KBLOCKS && c[kb]; ++kb)
          fprintf(stderr, "  k-block %2d: %7lld | %7lld | %7lld\n", kb, (long long)(c[kb] - c[0]),
                  c[TC_TRACE_KBLOCKS + kb] ? (long long)(c[TC_TRACE_KBLOCKS + kb] - c[0]) : 0LL,
                  c[2 * TC_TRACE_KBLOCKS + kb] ? (long long)(c[2 * TC_TRACE_KBLOCKS + kb] - c[0]) : 0LL);
      }
    }
    rc = check_status(h);
  } while (0);
  cudaFree(trace_dev);
  for (auto& s : S) {
    gemm_tc_plan_destroy(s.plan);
    cudaFree(s.a); cudaFree(s.b); cudaFree(s.c); cudaFree(s.x);
    cudaFree(s.a_lo); cudaFree(s.b_lo); cudaFree(s.c_lo);
  }
  return rc;
}

int b2_get_timing(b2_handle* h, double* phase_ms, double* step_ms, long long* steps) {
  if (!h) return B2_ERR_INVALID;
  if (phase_ms) memcpy(phase_ms, h->phase_ms.data(), h->phase_ms.size() * sizeof(double));
  if (step_ms) *step_ms = h->step_ms;
  if (steps) *steps = h->steps;
  return B2_OK;
}

int b2_write_trace(b2_handle* h, const char* path) {
  if (!h || !path) return fail(h, B2_ERR_INVALID, "null argument");
  if (h->trace.empty()) return fail(h, B2_ERR_STATE, "no timed step recorded (needs collect_timing = 1)");
  FILE* f = fopen(path, "w");
  if (!f) return fail(h, B2_ERR_INVALID, "cannot open %s", path);
  static const char* names[B2_T_NUM] = {"fwd", "wgt_grad", "bwd", "wgt_update", "allreduce", "allgather"};
  // one "thread" per stream: main (fwd, bwd), weight-gradient stream, collective stream, update stream
  static const int tid[B2_T_NUM] = {0, 1, 0, 3, 2, 2};
  fprintf(f, "[\n");
  for (size_t i = 0; i < h->trace.size(); ++i) {
    const auto& e = h->trace[i];
    fprintf(f, "{\"name\": \"%s %d\", \"ph\": \"X\", \"pid\": %d, \"tid\": %d, \"ts\": %.3f, \"dur\": %.3f, "
               "\"args\": {\"step\": %d}}%s\n",
            names[e.phase], e.layer, h->cfg.rank, tid[e.phase], e.start_ms * 1e3, e.dur_ms * 1e3, e.step,
            i + 1 < h->trace.size() ? "," : "");
  }
  fprintf(f, "]\n");
  fclose(f);
  return B2_OK;
}

int b2_get_gemm_busy_ms(b2_handle* h, double* ms) {
  if (!h || !ms) return B2_ERR_INVALID;
  *ms = h->gemm_busy_ms;
  return B2_OK;
}

int b2_reset_timing(b2_handle* h) {
  if (!h) return B2_ERR_INVALID;
  h->gemm_busy_ms = 0;
  std::fill(h->phase_ms.begin(), h->phase_ms.end(), 0.0);
  h->step_ms = 0;
  h->steps = 0;
  return B2_OK;
}

int b2_site_report(const b2_handle* h, int* tensor_core_sites, int* cuda_core_sites, char* first_reason,
                   size_t reason_len) {
  if (!h) return B2_ERR_INVALID;
  if (tensor_core_sites) *tensor_core_sites = h->tensor_core_sites;
  if (cuda_core_sites) *cuda_core_sites = h->cuda_core_sites;
  if (first_reason && reason_len) snprintf(first_reason, reason_len, "%s", h->cuda_core_reason.c_str());
  return B2_OK;
}

int b2_launch_counts(const b2_handle* h, long long* total, long long* tc) {
  if (!h) return B2_ERR_INVALID;
  if (total) *total = h->launches;
  if (tc) *tc = h->tc_launches;
  return B2_OK;
}

static int gemm_common(b2_handle* h, int precision, GemmDesc& d, cudaStream_t st) {
  TcPlan* plan = nullptr;
  if (precision != B2_PREC_FP32 && !h->cfg.force_simt) {
    if (!h->tc_ws) {  // a handle created for fp32 steps gets its tensor-core workspace on first use
      int rc;
      if ((rc = dev_alloc(h, &h->tc_ws, (size_t)h->sms * TC_WS_SLOT_BYTES))) return rc;
      if ((rc = dev_alloc(h, &h->tc_ws_flags, (size_t)h->sms * sizeof(unsigned int)))) return rc;
    }
    d.ws = h->tc_ws;
    d.ws_flags = h->tc_ws_flags;
    char why[128];
    plan = gemm_tc_plan_create(d, h->sms, why, sizeof why);
  }
  ++h->launches;
  cudaError_t e;
  if (plan) {
    ++h->tc_launches;
    e = gemm_tc_launch(plan, st, h->status_dev);
    gemm_tc_plan_destroy(plan);  // the tensor maps were passed by value at launch
  } else {
    e = gemm_simt_launch(d, st);
  }
  if (e != cudaSuccess) return fail(h, B2_ERR_CUDA, "GEMM launch: %s", cudaGetErrorString(e));
  return B2_OK;
}

int b2_sgemm(b2_handle* h, int precision, int transa, int transb, int m, int n, int k, float alpha, const float* a,
             size_t lda, const float* b, size_t ldb, float beta, float* c, size_t ldc) {
  ENTER(h);
  if (precision == B2_PREC_BF16) return fail(h, B2_ERR_UNSUPPORTED, "b2_sgemm takes fp32 device operands");
  if (precision == B2_PREC_FP32_TC)
    return fail(h, B2_ERR_UNSUPPORTED, "b2_sgemm has no room for the operand twins of the fp32-class mode: b2_sgemm_host");
  if (m < 0 || n < 0 || k < 0 || !a || !b || !c) return fail(h, B2_ERR_INVALID, "bad GEMM arguments");
  GemmDesc d{};
  d.M = m; d.N = n; d.K = k;
  d.A = a; d.sAm = transa ? 1 : (long long)lda; d.sAk = transa ? (long long)lda : 1;
  d.B = b; d.sBk = transb ? 1 : (long long)ldb; d.sBn = transb ? (long long)ldb : 1;
  d.C = c; d.ldc = (long long)ldc;
  d.alpha = alpha; d.beta = beta;
  d.epilogue = EPI_NONE;
  d.in_type = T_F32; d.out_type = T_F32;
  return gemm_common(h, precision, d, h->s_main);
}

int b2_sgemm_host(b2_handle* h, int precision, int transa, int transb, int m, int n, int k, const float* a,
                  size_t lda, const float* b, size_t ldb, float* c, size_t ldc, int epilogue, const float* aux,
                  size_t ldaux) {
  ENTER(h);
  if (m < 1 || n < 1 || k < 1 || !a || !b || !c) return fail(h, B2_ERR_INVALID, "bad GEMM arguments");
  if (epilogue < EPI_NONE || epilogue > EPI_MASK) return fail(h, B2_ERR_INVALID, "bad epilogue");
  if (epilogue == EPI_MASK && !aux) return fail(h, B2_ERR_INVALID, "mask epilogue needs aux");
  const int in_type = precision == B2_PREC_BF16 ? T_BF16 : T_F32;
  // like the step: bf16 operands produce bf16 activations/gradients, fp32 otherwise
  const int out_type = (in_type == T_BF16 && epilogue != EPI_NONE) ? T_BF16 : T_F32;
  const int ar = transa ? k : m, ac = transa ? m : k;
  const int br = transb ? n : k, bc = transb ? k : n;
  void *da = nullptr, *db = nullptr, *dc = nullptr, *dx = nullptr;
  float *da_lo = nullptr, *db_lo = nullptr;
  const bool x3 = precision == B2_PREC_FP32_TC && !h->cfg.force_simt;
  float* stage = nullptr;
  size_t big = (size_t)ar * ac;
  if ((size_t)br * bc > big) big = (size_t)br * bc;
  if ((size_t)m * n > big) big = (size_t)m * n;
  int rc = B2_OK;
  auto put = [&](void** dev, const float* host, size_t ld, int rows, int cols) -> int {
    CK(h, cudaMalloc(dev, (size_t)rows * cols * esize(in_type)));
    if (in_type == T_F32) {
      CK(h, cudaMemcpy2DAsync(*dev, (size_t)cols * 4, host, ld * 4, (size_t)cols * 4, rows, cudaMemcpyHostToDevice,
                              h->s_main));
    } else {
      CK(h, cudaMemcpy2DAsync(stage, (size_t)cols * 4, host, ld * 4, (size_t)cols * 4, rows,
                              cudaMemcpyHostToDevice, h->s_main));
      CK(h, convert_f32_to_bf16(stage, (__nv_bfloat16*)*dev, (size_t)rows * cols, h->s_main));
      CK(h, cudaStreamSynchronize(h->s_main));
    }
    return B2_OK;
  };
  do {
    if (cudaMalloc((void**)&stage, big * 4) != cudaSuccess) { rc = fail(h, B2_ERR_CUDA, "cudaMalloc"); break; }
    if ((rc = put(&da, a, lda, ar, ac))) break;
    if ((rc = put(&db, b, ldb, br, bc))) break;
    if (epilogue == EPI_MASK && (rc = put(&dx, aux, ldaux, m, n))) break;
    if (cudaMalloc(&dc, (size_t)m * n * esize(out_type)) != cudaSuccess) { rc = fail(h, B2_ERR_CUDA, "cudaMalloc"); break; }
    if (x3) {
      if (cudaMalloc((void**)&da_lo, (size_t)ar * ac * 4) != cudaSuccess ||
          cudaMalloc((void**)&db_lo, (size_t)br * bc * 4) != cudaSuccess) { rc = fail(h, B2_ERR_CUDA, "cudaMalloc"); break; }
      split_lo_launch(static_cast<const float*>(da), da_lo, (size_t)ar * ac, h->s_main);
      split_lo_launch(static_cast<const float*>(db), db_lo, (size_t)br * bc, h->s_main);
    }
    GemmDesc d{};
    d.M = m; d.N = n; d.K = k;
    d.A = da; d.sAm = transa ? 1 : ac; d.sAk = transa ? ac : 1;
    d.B = db; d.sBk = transb ? 1 : bc; d.sBn = transb ? bc : 1;
    d.C = dc; d.ldc = n;
    d.aux = dx; d.ldaux = n;
    d.alpha = 1.f; d.beta = 0.f;
    d.epilogue = epilogue;
    d.in_type = in_type; d.out_type = out_type;
    d.A_lo = da_lo; d.B_lo = db_lo;
    if ((rc = gemm_common(h, precision, d, h->s_main))) break;
    const void* src = dc;
    if (out_type == T_BF16) {
      if (convert_bf16_to_f32((const __nv_bfloat16*)dc, stage, (size_t)m * n, h->s_main) != cudaSuccess) {
        rc = fail(h, B2_ERR_CUDA, "convert");
        break;
      }
      src = stage;
    }
    if (cudaMemcpy2DAsync(c, ldc * 4, src, (size_t)n * 4, (size_t)n * 4, m, cudaMemcpyDeviceToHost, h->s_main) !=
            cudaSuccess ||
        cudaStreamSynchronize(h->s_main) != cudaSuccess) {
      rc = fail(h, B2_ERR_CUDA, "GEMM readback: %s", cudaGetErrorString(cudaGetLastError()));
      break;
    }
    rc = check_status(h);
  } while (0);
  cudaFree(da); cudaFree(db); cudaFree(dc); cudaFree(dx); cudaFree(stage);
  cudaFree(da_lo); cudaFree(db_lo);
  return rc;
}

}  // extern "C"

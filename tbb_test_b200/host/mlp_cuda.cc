// mlp_cuda: GPU counterpart of the reference's mlp_omp / mlp_tbb benchmark mains
// (mlp_omp.cc:375-750).  Same phases in the same order - allocate the host
// matrices, run the allreduce+SGD known-answer self-check, initialise inputs and
// weights, run NWARMUP + NITER training steps, report timing, print the weight
// checksums - with the training step executed by libb200mlp.so through its C ABI,
// one GPU per "socket" and one host thread per GPU.
//
//   mlp_cuda <ngpus> [<nthreads_per_socket, ignored>] [options]
//     --widths 1024,1024,...   layer widths F_0..F_L     (default: reference model)
//     --batch N                global batch               (default 1024 * ngpus)
//     --precision fp32|fp32tc|tf32|bf16                   (default bf16)
//     --mode ref|baseline                                 (default ref, lr 1e-10)
//     --lr X   --warmup N   --iters N   --no-overlap   --no-allreduce   --graph
//     --p2p-bytes N            gradient sums up to N bytes through peer memory instead of NCCL
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "b200mlp.h"
#include "b2_rng.h"
#include "mlp_bench_common.h"

namespace {

struct Options {
  int ngpus = 1;
  std::vector<int> widths = {1024, 1024, 1024, 1024, 1024, 1024, 1024, 1};
  int batch = 0;
  int precision = B2_PREC_BF16;
  int mode = B2_MODE_REF;
  float lr = 1e-10f;
  int warmup = 16, iters = 256;
  int overlap = 1, allreduce = 1, graph = 0;
  long long p2p_bytes = 0;
};

bool parse(int argc, char** argv, Options* o) {
  if (argc < 2) return false;
  o->ngpus = atoi(argv[1]);
  int i = 2;
  if (i < argc && argv[i][0] != '-') ++i;  // the reference's <nthreads_per_socket>
  for (; i < argc; ++i) {
    std::string a = argv[i];
    auto next = [&]() -> const char* { return i + 1 < argc ? argv[++i] : ""; };
    if (a == "--widths") {
      o->widths.clear();
      std::string s = next();
      size_t p = 0;
      while (p < s.size()) {
        size_t q = s.find(',', p);
        if (q == std::string::npos) q = s.size();
        o->widths.push_back(atoi(s.substr(p, q - p).c_str()));
        p = q + 1;
      }
    } else if (a == "--batch") o->batch = atoi(next());
    else if (a == "--precision") {
      std::string v = next();
      o->precision = v == "fp32" ? B2_PREC_FP32 : v == "fp32tc" ? B2_PREC_FP32_TC : v == "tf32" ? B2_PREC_TF32 : B2_PREC_BF16;
    } else if (a == "--mode") {
      std::string v = next();
      o->mode = v == "baseline" ? B2_MODE_BASELINE : B2_MODE_REF;
      if (o->mode == B2_MODE_BASELINE && o->lr == 1e-10f) o->lr = 0.01f;
    } else if (a == "--lr") o->lr = (float)atof(next());
    else if (a == "--warmup") o->warmup = atoi(next());
    else if (a == "--iters") o->iters = atoi(next());
    else if (a == "--no-overlap") o->overlap = 0;
    else if (a == "--no-allreduce") o->allreduce = 0;
    else if (a == "--graph") o->graph = 1;
    else if (a == "--p2p-bytes") o->p2p_bytes = atoll(next());
    else return false;
  }
  if (o->batch <= 0) o->batch = 1024 * o->ngpus;  // weak scaling like the reference (mlp_omp.cc:386)
  return o->ngpus >= 1 && o->widths.size() >= 2;
}

Matrix<float, PAD>* new_matrix(int rows, int cols) {
  // the reference first-touches with (i + j) % 31 - 15 (mlp_omp.cc:40-45); the pattern is kept
  auto* m = new Matrix<float, PAD>(rows, cols);
  for (int i = 0; i < rows; ++i)
    for (int j = 0; j < cols; ++j) (*m)(i, j) = (float)((i + j) % 31 - 15);
  return m;
}

double now() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

struct Worker {
  b2_handle* h = nullptr;
  int rc = 0;
  std::string err;
};

// Runs fn(gpu) on one host thread per GPU and reports the first failure.
template <typename F>
bool on_all_gpus(std::vector<Worker>& ws, F fn) {
  std::vector<std::thread> ts;
  for (int g = 0; g < (int)ws.size(); ++g)
    ts.emplace_back([&, g] {
      set_thread_position(g, (int)ws.size());
      ws[g].rc = fn(g);
      if (ws[g].rc) ws[g].err = b2_last_error(ws[g].h);
    });
  for (auto& t : ts) t.join();
  for (int g = 0; g < (int)ws.size(); ++g)
    if (ws[g].rc) {
      fprintf(stderr, "gpu %d: error %d: %s\n", g, ws[g].rc, ws[g].err.c_str());
      return false;
    }
  return true;
}

// The reference's self-check (mlp_omp.cc:325-373): grad(s, i, j) = s + i + j,
// w = i * j, alpha = 1; every replica must end at i*j - ((i+j)*N + N(N-1)/2).
bool check_all_reduce_correctness(std::vector<Worker>& ws, const Options& o) {
  const int N = o.ngpus, rows = nfeatures[1], cols = nfeatures[0];
  bool ok = on_all_gpus(ws, [&](int g) -> int {
    Matrix<float, PAD> w(rows, cols), grad(rows, cols);
    for (int i = 0; i < rows; ++i)
      for (int j = 0; j < cols; ++j) {
        grad(i, j) = (float)(g + i + j);
        w(i, j) = (float)(i * j);
      }
    int rc;
    if ((rc = b2_set_lr(ws[g].h, 1.0f))) return rc;
    if ((rc = b2_upload_weights(ws[g].h, 0, w.rawData(), w.ld()))) return rc;
    if ((rc = b2_upload_weight_grad(ws[g].h, 0, grad.rawData(), grad.ld()))) return rc;
    if ((rc = b2_allreduce_sgd(ws[g].h, 0))) return rc;
    if ((rc = b2_download_weights(ws[g].h, 0, w.rawData(), w.ld()))) return rc;
    for (int i = 0; i < rows; ++i)
      for (int j = 0; j < cols; ++j) {
        const float expected = (float)(i * j - ((i + j) * N + (N - 1) * N / 2));
        if (std::abs(w(i, j) - expected) > 1e-5) {
          printf("sid %d i %d j %d expected %f actual %f\n", g, i, j, expected, w(i, j));
          return B2_ERR_STATE;
        }
      }
    return b2_set_lr(ws[g].h, o.lr);
  });
  return ok;
}

}  // namespace

int main(int argc, char** argv) {
  Options o;
  if (!parse(argc, argv, &o)) {
    fprintf(stderr,
            "%s <ngpus> [<nthreads_per_socket>] [--widths a,b,..] [--batch N] [--precision fp32|fp32tc|tf32|bf16]\n"
            "        [--mode ref|baseline] [--lr X] [--warmup N] [--iters N] [--no-overlap] [--no-allreduce] [--graph]\n"
            "        [--p2p-bytes N]\n",
            argv[0]);
    return 1;
  }
  nsockets = o.ngpus;
  nthreads_per_socket = 1;
  nthreads = nsockets;
  set_model(o.widths);
  NWARMUP = o.warmup;
  NITER = o.iters;
  const int batch_size = o.batch;

  // host matrices, as in mlp_omp.cc:390-409 (one weight replica: the device holds the others)
  for (int l = 0; l < nlayers; ++l) {
    activations[l].reset(new_matrix(batch_size, nfeatures[l]));
    weights[l].reset(new_matrix(nfeatures[l + 1], nfeatures[l]));
    weight_grads[l].reset(new_matrix(nfeatures[l + 1], nfeatures[l]));
  }
  activations[nlayers].reset(new_matrix(batch_size, nfeatures[nlayers]));
  activations[nlayers + 1].reset(new_matrix(batch_size, nfeatures[0]));

  char id[B2_NCCL_ID_BYTES] = {0};
  if (o.ngpus > 1 && o.allreduce && b2_nccl_unique_id(id) != B2_OK) {
    fprintf(stderr, "NCCL: %s\n", b2_last_error(nullptr));
    return 2;
  }
  std::vector<Worker> ws(o.ngpus);
  bool ok = on_all_gpus(ws, [&](int g) -> int {
    b2_config c;
    b2_config_default(&c);
    c.nlayers = nlayers;
    c.nfeatures = nfeatures.data();
    c.batch = batch_size;
    c.rank = g;
    c.world_size = o.ngpus;
    c.device = g;
    c.mode = o.mode;
    c.precision = o.precision;
    c.allreduce = o.allreduce;
    c.overlap = o.overlap;
    c.use_graph = o.graph;
    c.collect_timing = o.graph ? 0 : 1;
    c.lr = o.lr;
    c.nccl_unique_id = o.ngpus > 1 ? id : nullptr;
    int rc = b2_create(&c, &ws[g].h);
    if (rc) ws[g].err = b2_last_error(nullptr);
    return rc;
  });
  if (!ok) return 2;
  if (o.p2p_bytes > 0 && o.ngpus > 1 && o.allreduce) {
    // every GPU's gradient buffer becomes addressable from every other GPU (one process: peer access)
    std::vector<char> descs((size_t)o.ngpus * B2_P2P_DESC_BYTES);
    ok = on_all_gpus(ws, [&](int g) -> int { return b2_p2p_describe(ws[g].h, &descs[(size_t)g * B2_P2P_DESC_BYTES]); }) &&
         on_all_gpus(ws, [&](int g) -> int { return b2_p2p_connect(ws[g].h, descs.data(), (size_t)o.p2p_bytes); });
    if (!ok) return 2;
  }

  if (o.allreduce && !check_all_reduce_correctness(ws, o)) return -1;

  // initial values (master thread only, to be deterministic: mlp_omp.cc:419-420)
  randSeed(3);
  init_matrices();
  if (o.mode == B2_MODE_BASELINE) b2_fill_sign(activations[nlayers]->rawData(), batch_size, nfeatures[nlayers],
                                               activations[nlayers]->ld(), 2);

  ok = on_all_gpus(ws, [&](int g) -> int {
    int rc;
    for (int l = 0; l < nlayers; ++l)
      if ((rc = b2_upload_weights(ws[g].h, l, weights[l]->rawData(), weights[l]->ld()))) return rc;
    if ((rc = b2_upload_input(ws[g].h, activations[0]->rawData(), activations[0]->ld()))) return rc;
    if (o.mode == B2_MODE_BASELINE &&
        (rc = b2_upload_target(ws[g].h, activations[nlayers]->rawData(), activations[nlayers]->ld())))
      return rc;
    if ((rc = b2_step(ws[g].h, NWARMUP))) return rc;
    return b2_reset_timing(ws[g].h);
  });
  if (!ok) return 2;

  wall_clock_time = now();
  ok = on_all_gpus(ws, [&](int g) -> int { return b2_step(ws[g].h, NITER); });
  wall_clock_time = now() - wall_clock_time;
  if (!ok) return 2;

  // gather the per-phase device times into the reference's tables
  sum_times.assign(o.ngpus, std::vector<std::array<double, NUM_BREAKDOWNS>>(nlayers));
  for (int g = 0; g < o.ngpus; ++g) {
    std::vector<double> ph((size_t)nlayers * B2_T_NUM, 0.0);
    b2_get_timing(ws[g].h, ph.data(), nullptr, nullptr);
    int b0, b1;
    b2_batch_range(ws[g].h, &b0, &b1);
    for (int l = 0; l < nlayers; ++l) {
      auto& t = sum_times[g][l];
      t[FWD] = ph[l * B2_T_NUM + B2_T_FWD] * 1e-3;
      t[WGT_GRAD] = ph[l * B2_T_NUM + B2_T_WGT_GRAD] * 1e-3;
      t[BWD] = ph[l * B2_T_NUM + B2_T_BWD] * 1e-3;
      // the reduce-scatter (or allreduce) stands where the reference has its reduce-scatter, the
      // SGD kernel plus the allgather of the weights where it has the update + allgather
      t[WGT_UPDATE_REDUCE_SCATTER] = ph[l * B2_T_NUM + B2_T_ALLREDUCE] * 1e-3;
      t[WGT_UPDATE_ALLGATHER] = (ph[l * B2_T_NUM + B2_T_WGT_UPDATE] + ph[l * B2_T_NUM + B2_T_ALLGATHER]) * 1e-3;
      if (g == 0) {
        const double flops = 2.0 * batch_size * nfeatures[l] * nfeatures[l + 1] * NITER;  // mlp_omp.cc:492,584,675
        sum_flops[l][FWD] = sum_flops[l][WGT_GRAD] = sum_flops[l][BWD] = flops;
        const double bytes = (double)(nsockets - 1) * nfeatures[l + 1] * nfeatures[l] * sizeof(float) * NITER;
        sum_flops[l][WGT_UPDATE_REDUCE_SCATTER] = sum_flops[l][WGT_UPDATE_ALLGATHER] = bytes;  // mlp_omp.cc:163,288
      }
    }
  }
  report_timing();
  printf("samples/s %g\n", (double)batch_size * NITER / wall_clock_time);

  // final weights of replica 0 for the checksum (mlp_bench_common.cc:152-168). Every GPU takes
  // part in the download: with the sharded update in BF16 precision it is a collective that first
  // gathers the fp32 master weights from the ranks that own them; only replica 0's copy is kept.
  ok = on_all_gpus(ws, [&](int g) -> int {
    std::vector<float> scratch;
    for (int l = 0; l < nlayers; ++l) {
      int rc;
      if (g == 0) {
        rc = b2_download_weights(ws[g].h, l, weights[l]->rawData(), weights[l]->ld());
      } else {
        scratch.resize((size_t)nfeatures[l + 1] * nfeatures[l]);
        rc = b2_download_weights(ws[g].h, l, scratch.data(), (size_t)nfeatures[l]);
      }
      if (rc) return rc;
    }
    return 0;
  });
  if (!ok) return 2;
  print_checksum();
  for (auto& w : ws) b2_destroy(w.h);
  return 0;
}

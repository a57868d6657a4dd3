// Implementation of the MKL stand-in declared in mkl.h.  Checker infrastructure.
#include "mkl.h"

#include <dlfcn.h>
#include <glob.h>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/b2_rng.h"

namespace {
using sgemm_t = void (*)(int, int, int, int, int, int, float, const float*, int, const float*, int,
                         float, float*, int);
sgemm_t g_sgemm = nullptr;
char g_name[1024] = "unbound";
std::once_flag g_once;

void* try_open(const char* pattern) {
  glob_t g;
  void* h = nullptr;
  if (glob(pattern, 0, nullptr, &g) == 0) {
    for (size_t i = 0; i < g.gl_pathc && !h; ++i) {
      h = dlopen(g.gl_pathv[i], RTLD_NOW | RTLD_LOCAL);
      if (h) snprintf(g_name, sizeof g_name, "openblas:%s", g.gl_pathv[i]);
    }
  }
  globfree(&g);
  return h;
}

void bind_blas() {
  void* h = nullptr;
  if (const char* p = getenv("B2_OPENBLAS_PATH")) h = try_open(p);
#ifdef B2_OPENBLAS_DEFAULT
  if (!h) h = try_open(B2_OPENBLAS_DEFAULT);
#endif
  if (h) {
    g_sgemm = (sgemm_t)dlsym(h, "scipy_cblas_sgemm");
    using setn_t = void (*)(int);
    if (auto setn = (setn_t)dlsym(h, "scipy_openblas_set_num_threads")) setn(1);
  }
  if (!g_sgemm) {
    fprintf(stderr, "mkl shim: no OpenBLAS found (set B2_OPENBLAS_PATH)\n");
    abort();
  }
}

uint64_t g_rng_pos = 0;
constexpr uint64_t kShimSeed = 3;  // the reference asks for Niederreiter dimension 3 (Rand.cc:20)
}  // namespace

extern "C" {

void cblas_sgemm(CBLAS_LAYOUT layout, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n, int k,
                 float alpha, const float* a, int lda, const float* b, int ldb, float beta, float* c,
                 int ldc) {
  std::call_once(g_once, bind_blas);
  if (m <= 0 || n <= 0) return;
  g_sgemm((int)layout, (int)ta, (int)tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
}

double dsecnd(void) {
  using namespace std::chrono;
  return duration<double>(steady_clock::now().time_since_epoch()).count();
}

void mkl_set_num_threads(int) {}

int vslNewStream(VSLStreamStatePtr* stream, int, unsigned) {
  *stream = (void*)&g_rng_pos;
  return 0;
}
int vsRngUniform(int, VSLStreamStatePtr, int n, float* r, float a, float b) {
  for (int i = 0; i < n; ++i) r[i] = b2_rng_uniform(kShimSeed, g_rng_pos++, a, b);
  return 0;
}
int vdRngUniform(int, VSLStreamStatePtr, int n, double* r, double a, double b) {
  for (int i = 0; i < n; ++i) r[i] = (double)b2_rng_uniform(kShimSeed, g_rng_pos++, (float)a, (float)b);
  return 0;
}
void b2shim_rng_reset(void) { g_rng_pos = 0; }
const char* b2shim_blas_name(void) {
  std::call_once(g_once, bind_blas);
  return g_name;
}
}

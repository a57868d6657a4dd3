/* CPU oracle for the MLP training step: see mlp_oracle.h for what it restates
 * and how it is pinned.  TEST INFRASTRUCTURE ONLY (checker, never the product).
 *
 * Internal storage is dense row-major (ld = ncols); host-facing accessors take
 * the caller's leading dimension (the reference's Matrix has ld = ncols + 16,
 * Matrix.h:148).
 */
#include "mlp_oracle.h"

#include "../include/b2_rng.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ rounding */

float orc_round_bf16(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7f800000u) == 0x7f800000u) { /* inf / nan: truncate, keep nan-ness */
    u &= 0xffff0000u;
  } else {
    u += 0x7fffu + ((u >> 16) & 1u);
    u &= 0xffff0000u;
  }
  memcpy(&x, &u, 4);
  return x;
}

float orc_round_tf32(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  u &= 0xffffe000u;
  memcpy(&x, &u, 4);
  return x;
}

static float round_as(float x, int rounding) {
  if (rounding == ORC_ROUND_BF16) return orc_round_bf16(x);
  if (rounding == ORC_ROUND_TF32) return orc_round_tf32(x);
  return x;
}

/* --------------------------------------------------------------------- GEMM */

static orc_sgemm_fn g_sgemm = NULL;
void orc_set_sgemm(orc_sgemm_fn fn) { g_sgemm = fn; }

/* Built-in row-major SGEMM: every form is brought to
 *   C[i][:] += a(i,p) * Bn[p][:]
 * (B transposed into a scratch copy when it is stored n x k), which vectorises
 * over the contiguous output row without reassociating the sum over p. */
static void sgemm_loops(int transa, int transb, int m, int n, int k, float alpha,
                        const float* a, int lda, const float* b, int ldb, float beta,
                        float* c, int ldc) {
  float* bt = NULL;
  const float* bn = b;
  int ldbn = ldb;
  if (transb) { /* b is n x k -> make k x n */
    bt = (float*)malloc((size_t)k * n * sizeof(float));
#pragma omp parallel for schedule(static)
    for (int p = 0; p < k; ++p)
      for (int j = 0; j < n; ++j) bt[(size_t)p * n + j] = b[(size_t)j * ldb + p];
    bn = bt;
    ldbn = n;
  }
  enum { JB = 512 };
#pragma omp parallel for schedule(static)
  for (int i = 0; i < m; ++i) {
    float acc[JB];
    for (int j0 = 0; j0 < n; j0 += JB) {
      int jn = n - j0 < JB ? n - j0 : JB;
      for (int j = 0; j < jn; ++j) acc[j] = 0.f;
      for (int p = 0; p < k; ++p) {
        float av = transa ? a[(size_t)p * lda + i] : a[(size_t)i * lda + p];
        const float* brow = bn + (size_t)p * ldbn + j0;
        for (int j = 0; j < jn; ++j) acc[j] += av * brow[j];
      }
      float* crow = c + (size_t)i * ldc + j0;
      if (beta == 0.f) {
        for (int j = 0; j < jn; ++j) crow[j] = alpha * acc[j];
      } else {
        for (int j = 0; j < jn; ++j) crow[j] = alpha * acc[j] + beta * crow[j];
      }
    }
  }
  free(bt);
}

/* Re-association switch: with g_ksplit = s > 1 every GEMM is computed as s partial
 * products over consecutive ranges of the contraction index that are added up one
 * after the other - the same sum in another floating-point order. Two oracles that
 * differ only in this switch measure how sensitive a configuration is to the order of
 * fp32 additions (the noise floor any two correct implementations are apart). */
static int g_ksplit = 1;
void orc_set_ksplit(int s) { g_ksplit = s < 1 ? 1 : s; }

static void sgemm_one(int transa, int transb, int m, int n, int k, float alpha, const float* a,
                      int lda, const float* b, int ldb, float beta, float* c, int ldc);

void orc_sgemm(int transa, int transb, int m, int n, int k, float alpha, const float* a,
               int lda, const float* b, int ldb, float beta, float* c, int ldc) {
  if (m <= 0 || n <= 0) return;
  if (g_ksplit <= 1 || k < 2 * g_ksplit) {
    sgemm_one(transa, transb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
    return;
  }
  for (int s = 0; s < g_ksplit; ++s) {
    const int k0 = (int)((long long)k * s / g_ksplit), k1 = (int)((long long)k * (s + 1) / g_ksplit);
    const float* as = transa ? a + (size_t)k0 * lda : a + k0;
    const float* bs = transb ? b + k0 : b + (size_t)k0 * ldb;
    sgemm_one(transa, transb, m, n, k1 - k0, alpha, as, lda, bs, ldb, s == 0 ? beta : 1.f, c, ldc);
  }
}

static void sgemm_one(int transa, int transb, int m, int n, int k, float alpha, const float* a,
                      int lda, const float* b, int ldb, float beta, float* c, int ldc) {
  if (g_sgemm) {
    /* CblasRowMajor = 101, CblasNoTrans = 111, CblasTrans = 112 */
    g_sgemm(101, transa ? 112 : 111, transb ? 112 : 111, m, n, k, alpha, a, lda, b, ldb,
            beta, c, ldc);
  } else {
    sgemm_loops(transa, transb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
  }
}

/* -------------------------------------------------------------------- model */

struct orc_mlp {
  orc_config cfg;
  int* nf;
  float** w;     /* master weights, F_{l+1} x F_l */
  float** dw;    /* summed gradient */
  float** act;   /* forward activations A[0..L], batch x F_l (stored precision) */
  float** dz;    /* dZ[0..L-1], batch x F_{l+1} (stored precision) */
  float* target; /* batch x F_L */
  float* dinput; /* batch x F_0 */
  double loss;
};

void orc_batch_range(int batch, int nranks, int rank, int* begin, int* end) {
  /* get_partition(work, socket, 1, 0): ceil-div shard, clamped (Partition.cc:34-51) */
  int per = (batch + nranks - 1) / nranks;
  int b = rank * per;
  if (b > batch) b = batch;
  int e = b + per;
  if (e > batch) e = batch;
  *begin = b;
  *end = e;
}

orc_mlp* orc_create(const orc_config* cfg) {
  orc_mlp* o = (orc_mlp*)calloc(1, sizeof(orc_mlp));
  o->cfg = *cfg;
  int L = cfg->nlayers;
  o->nf = (int*)malloc(sizeof(int) * (L + 1));
  memcpy(o->nf, cfg->nfeatures, sizeof(int) * (L + 1));
  o->cfg.nfeatures = o->nf;
  o->w = (float**)calloc(L, sizeof(float*));
  o->dw = (float**)calloc(L, sizeof(float*));
  o->dz = (float**)calloc(L, sizeof(float*));
  o->act = (float**)calloc(L + 1, sizeof(float*));
  size_t B = (size_t)cfg->batch;
  for (int l = 0; l < L; ++l) {
    size_t nw = (size_t)o->nf[l + 1] * o->nf[l];
    o->w[l] = (float*)calloc(nw, sizeof(float));
    o->dw[l] = (float*)calloc(nw, sizeof(float));
    o->dz[l] = (float*)calloc(B * o->nf[l + 1], sizeof(float));
  }
  for (int l = 0; l <= L; ++l) o->act[l] = (float*)calloc(B * o->nf[l], sizeof(float));
  o->target = (float*)calloc(B * o->nf[L], sizeof(float));
  o->dinput = (float*)calloc(B * o->nf[0], sizeof(float));
  return o;
}

void orc_destroy(orc_mlp* o) {
  if (!o) return;
  int L = o->cfg.nlayers;
  for (int l = 0; l < L; ++l) {
    free(o->w[l]);
    free(o->dw[l]);
    free(o->dz[l]);
  }
  for (int l = 0; l <= L; ++l) free(o->act[l]);
  free(o->w);
  free(o->dw);
  free(o->dz);
  free(o->act);
  free(o->target);
  free(o->dinput);
  free(o->nf);
  free(o);
}

static void copy_in(float* dst, int rows, int cols, const float* src, size_t ld) {
  for (int i = 0; i < rows; ++i)
    memcpy(dst + (size_t)i * cols, src + (size_t)i * ld, sizeof(float) * cols);
}
static void copy_out(const float* src, int rows, int cols, float* dst, size_t ld) {
  for (int i = 0; i < rows; ++i)
    memcpy(dst + (size_t)i * ld, src + (size_t)i * cols, sizeof(float) * cols);
}

void orc_set_weights(orc_mlp* o, int l, const float* w, size_t ld) {
  copy_in(o->w[l], o->nf[l + 1], o->nf[l], w, ld);
}
void orc_get_weights(const orc_mlp* o, int l, float* w, size_t ld) {
  copy_out(o->w[l], o->nf[l + 1], o->nf[l], w, ld);
}
void orc_set_input(orc_mlp* o, const float* x, size_t ld) {
  copy_in(o->act[0], o->cfg.batch, o->nf[0], x, ld);
  if (o->cfg.rounding == ORC_ROUND_BF16) {
    size_t n = (size_t)o->cfg.batch * o->nf[0];
    for (size_t i = 0; i < n; ++i) o->act[0][i] = orc_round_bf16(o->act[0][i]);
  }
}
void orc_set_target(orc_mlp* o, const float* t, size_t ld) {
  copy_in(o->target, o->cfg.batch, o->nf[o->cfg.nlayers], t, ld);
}
void orc_get_activation(const orc_mlp* o, int l, float* a, size_t ld) {
  copy_out(o->act[l], o->cfg.batch, o->nf[l], a, ld);
}
void orc_get_dz(const orc_mlp* o, int l, float* g, size_t ld) {
  copy_out(o->dz[l], o->cfg.batch, o->nf[l + 1], g, ld);
}
void orc_get_input_grad(const orc_mlp* o, float* g, size_t ld) {
  copy_out(o->dinput, o->cfg.batch, o->nf[0], g, ld);
}
void orc_get_weight_grad(const orc_mlp* o, int l, float* g, size_t ld) {
  copy_out(o->dw[l], o->nf[l + 1], o->nf[l], g, ld);
}
double orc_loss(const orc_mlp* o) { return o->loss; }

/* GEMM operand view: bf16 values are already stored rounded (activations, dZ)
 * except the master weights; tf32 rounds at operand-read time. */
static const float* operand(const float* x, size_t n, int rounding, int is_master_weight,
                            float** scratch) {
  int need = (rounding == ORC_ROUND_TF32) || (rounding == ORC_ROUND_BF16 && is_master_weight);
  if (!need) {
    *scratch = NULL;
    return x;
  }
  float* t = (float*)malloc(n * sizeof(float));
#pragma omp parallel for schedule(static)
  for (size_t i = 0; i < n; ++i) t[i] = round_as(x[i], rounding);
  *scratch = t;
  return t;
}

static void one_step(orc_mlp* o) {
  const orc_config* c = &o->cfg;
  const int L = c->nlayers, B = c->batch, R = c->rounding;
  const int* nf = o->nf;
  const int store_bf16 = (R == ORC_ROUND_BF16);

  /* forward: A[l+1] = A[l] * W[l]^T (NoTrans x Trans, mlp_omp.cc:474-488) */
  for (int l = 0; l < L; ++l) {
    float *sa, *sw;
    const float* a = operand(o->act[l], (size_t)B * nf[l], R, 0, &sa);
    const float* w = operand(o->w[l], (size_t)nf[l + 1] * nf[l], R, 1, &sw);
    orc_sgemm(0, 1, B, nf[l + 1], nf[l], 1.f, a, nf[l], w, nf[l], 0.f, o->act[l + 1], nf[l + 1]);
    free(sa);
    free(sw);
    size_t n = (size_t)B * nf[l + 1];
    float* z = o->act[l + 1];
    if (c->mode == ORC_MODE_BASELINE && l < L - 1) {
      for (size_t i = 0; i < n; ++i) z[i] = z[i] > 0.f ? z[i] : 0.f;
    }
    if (store_bf16 && l < L - 1) { /* hidden activations are stored as bf16; the output stays fp32 */
      for (size_t i = 0; i < n; ++i) z[i] = orc_round_bf16(z[i]);
    }
  }

  /* output gradient */
  {
    size_t n = (size_t)B * nf[L];
    const float* y = o->act[L];
    float* g = o->dz[L - 1];
    double loss = 0;
    if (c->mode == ORC_MODE_REF) { /* the forward output is used as the gradient, mlp_omp.cc:565 */
      for (size_t i = 0; i < n; ++i) {
        g[i] = y[i];
        loss += 0.5 * (double)y[i] * y[i];
      }
    } else {
      const float inv_b = 1.0f / (float)B;
      for (size_t i = 0; i < n; ++i) {
        float d = y[i] - o->target[i];
        g[i] = d * inv_b;
        loss += 0.5 * (double)d * d;
      }
      loss /= B;
    }
    if (store_bf16)
      for (size_t i = 0; i < n; ++i) g[i] = orc_round_bf16(g[i]);
    o->loss = loss;
  }

  /* backward */
  for (int l = L - 1; l >= 0; --l) {
    size_t nw = (size_t)nf[l + 1] * nf[l];
    float *sg, *sa, *sw;
    const float* g = operand(o->dz[l], (size_t)B * nf[l + 1], R, 0, &sg);
    const float* a = operand(o->act[l], (size_t)B * nf[l], R, 0, &sa);

    /* wgrad, one partial per rank over its batch rows (mlp_omp.cc:528-531,565-580),
     * partials summed in rank order */
    float* part = (float*)malloc(nw * sizeof(float));
    memset(o->dw[l], 0, nw * sizeof(float));
    for (int r = 0; r < c->nranks; ++r) {
      int kb, ke;
      orc_batch_range(B, c->nranks, r, &kb, &ke);
      if (ke > kb) {
        orc_sgemm(1, 0, nf[l + 1], nf[l], ke - kb, 1.f, g + (size_t)kb * nf[l + 1], nf[l + 1],
                  a + (size_t)kb * nf[l], nf[l], 0.f, part, nf[l]);
      } else {
        memset(part, 0, nw * sizeof(float));
      }
      if (c->grad_bf16)
        for (size_t i = 0; i < nw; ++i) part[i] = orc_round_bf16(part[i]);
      if (r == 0)
        memcpy(o->dw[l], part, nw * sizeof(float));
      else
        for (size_t i = 0; i < nw; ++i) o->dw[l][i] += part[i];
      if (c->grad_bf16 && r > 0)
        for (size_t i = 0; i < nw; ++i) o->dw[l][i] = orc_round_bf16(o->dw[l][i]);
    }
    free(part);

    /* dgrad: dA[l] = dZ[l] * W[l] (NoTrans x NoTrans, mlp_omp.cc:655-671) with the
     * pre-update weights */
    const float* w = operand(o->w[l], nw, R, 1, &sw);
    float* da = (l == 0) ? o->dinput : o->dz[l - 1];
    orc_sgemm(0, 0, B, nf[l], nf[l + 1], 1.f, g, nf[l + 1], w, nf[l], 0.f, da, nf[l]);
    if (l > 0) {
      size_t n = (size_t)B * nf[l];
      if (c->mode == ORC_MODE_BASELINE) {
        const float* al = o->act[l];
        for (size_t i = 0; i < n; ++i) da[i] = al[i] > 0.f ? da[i] : 0.f;
      }
      if (store_bf16)
        for (size_t i = 0; i < n; ++i) da[i] = orc_round_bf16(da[i]);
    }
    free(sg);
    free(sa);
    free(sw);

    /* update: w = fma(-alpha, sum dW, w) (mlp_omp.cc:217-223,240-252) */
    {
      float na = -c->lr;
      float* wm = o->w[l];
      const float* d = o->dw[l];
      for (size_t i = 0; i < nw; ++i) wm[i] = fmaf(na, d[i], wm[i]);
    }
  }
}

void orc_step(orc_mlp* o, int n) {
  for (int i = 0; i < n; ++i) one_step(o);
}

/* ---------------------------------------------- allreduce + SGD restatement */

void orc_kat_fill(int nsockets, int nrows, int ncols, int sid, float* w, float* g, size_t ld) {
  (void)nsockets;
  for (int i = 0; i < nrows; ++i)
    for (int j = 0; j < ncols; ++j) {
      g[(size_t)i * ld + j] = (float)(sid + i + j);
      w[(size_t)i * ld + j] = (float)(i * j);
    }
}

void orc_kat_expected(int nsockets, int nrows, int ncols, float* expected, size_t ld) {
  for (int i = 0; i < nrows; ++i)
    for (int j = 0; j < ncols; ++j)
      expected[(size_t)i * ld + j] =
          (float)(i * j - ((i + j) * nsockets + (nsockets - 1) * nsockets / 2));
}

static const int ring8[8] = {0, 1, 2, 4, 7, 6, 5, 3}; /* mlp_bench_common.cc:13 */

static void ring_info(int n, int sid, int* idx, int* next) {
  if (n == 8) {
    int p = 0;
    while (ring8[p] != sid) ++p;
    *idx = p;
    *next = ring8[(p + 1) % 8];
  } else { /* mlp_bench_common.cc:182-185, task 0 */
    *idx = sid;
    *next = (sid + 1) % n;
  }
}

static void chunk_range(size_t chunk, size_t per, size_t total, size_t* b, size_t* e) {
  *b = chunk * per < total ? chunk * per : total;
  *e = *b + per < total ? *b + per : total;
}

void orc_ring_update(int n, int nrows, int ncols, size_t ld, float* w, float* g, float* push,
                     float alpha) {
  (void)ncols;
  const size_t ws = (size_t)nrows * ld; /* the padded buffer is reduced, mlp_omp.cc:73-74 */
  const size_t per = (ws + (size_t)n * 16 - 1) / n / 16 * 16; /* mlp_omp.cc:80-81 */
  const float na = -alpha;
  if (n == 1) { /* mlp_omp.cc:205-224 */
    for (size_t i = 0; i < ws; ++i) w[i] = fmaf(na, g[i], w[i]);
    return;
  }
  for (int step = 0; step < n - 1; ++step) { /* reduce-scatter, mlp_omp.cc:90-146 */
    for (int s = 0; s < n; ++s) {
      int idx, next;
      size_t b, e;
      ring_info(n, s, &idx, &next);
      chunk_range((size_t)((idx - step + n) % n), per, ws, &b, &e);
      memcpy(push + next * ws + b, g + s * ws + b, (e - b) * sizeof(float));
    }
    if (step < n - 2) {
      for (int s = 0; s < n; ++s) {
        int idx, next;
        size_t b, e;
        ring_info(n, s, &idx, &next);
        chunk_range((size_t)((idx - step - 1 + 2 * n) % n), per, ws, &b, &e);
        for (size_t i = b; i < e; ++i) g[s * ws + i] += push[s * ws + i];
      }
    }
  }
  for (int step = 0; step < n - 1; ++step) { /* allgather, mlp_omp.cc:227-271 */
    for (int s = 0; s < n; ++s) {
      int idx, next;
      size_t b, e;
      ring_info(n, s, &idx, &next);
      chunk_range((size_t)((idx + 1 - step + n) % n), per, ws, &b, &e);
      if (step == 0) {
        for (size_t i = b; i < e; ++i) {
          float t = g[s * ws + i] + push[s * ws + i];
          t = fmaf(na, t, w[s * ws + i]);
          w[s * ws + i] = t;
          w[next * ws + i] = t;
        }
      } else {
        memcpy(w + next * ws + b, w + s * ws + b, (e - b) * sizeof(float));
      }
    }
  }
}

void orc_checksum(const float* w, int nrows, int ncols, size_t ld, double out[3]) {
  double l1 = 0, l2 = 0, tr = 0;
  for (int i = 0; i < nrows; ++i) {
    for (int j = 0; j < ncols; ++j) {
      float v = w[(size_t)i * ld + j];
      l1 += fabsf(v);
      l2 += v * v; /* float product added to a double, as mlp_bench_common.cc:159 */
    }
    if (i < (nrows < ncols ? nrows : ncols)) tr += w[(size_t)i * ld + i];
  }
  out[0] = l1;
  out[1] = sqrt(l2);
  out[2] = tr;
}

/* ------------------------------------------------ seeded synthetic data */

void orc_fill_uniform(float* a, int nrows, int ncols, size_t ld, uint64_t seed, uint64_t start,
                      float lo, float hi) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < nrows; ++i)
    for (int j = 0; j < ncols; ++j)
      a[(size_t)i * ld + j] = b2_rng_uniform(seed, start + (uint64_t)i * ncols + j, lo, hi);
}

void orc_fill_normal(float* a, int nrows, int ncols, size_t ld, uint64_t seed, uint64_t start,
                     float stddev) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < nrows; ++i)
    for (int j = 0; j < ncols; ++j)
      a[(size_t)i * ld + j] = stddev * b2_rng_normal(seed, start + (uint64_t)i * ncols + j);
}

void orc_fill_sign(float* a, int nrows, int ncols, size_t ld, uint64_t seed, uint64_t start) {
#pragma omp parallel for schedule(static)
  for (int i = 0; i < nrows; ++i)
    for (int j = 0; j < ncols; ++j)
      a[(size_t)i * ld + j] = b2_rng_sign(seed, start + (uint64_t)i * ncols + j);
}

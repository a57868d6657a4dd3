// Tensor-core GEMM for sm_100a: TMA -> shared memory -> tcgen05.mma -> TMEM ->
// fused epilogue.  Replaces the three MKL cblas_sgemm call sites of the training
// step (forward mlp_omp.cc:474-488, weight gradient :565-580, input gradient
// :655-671) for bf16 (kind::f16) and fp32-as-tf32 (kind::tf32) operands with fp32
// accumulation.
//
// One persistent CTA per SM, 192 threads:
//   warp 0      TMA producer (one elected lane): fills a ring of shared-memory
//               stages, each holding a 128 x 128-byte A slab and a BN x 128-byte
//               B slab in the 128-byte-swizzled layout the MMA descriptors expect
//   warp 1      allocates TMEM; one elected lane issues tcgen05.mma (M = 128,
//               N = BN, 32 bytes of K per instruction) into one of two TMEM
//               accumulators and commits stage / accumulator completion to mbarriers
//   warps 2-5   epilogue: tcgen05.ld the finished accumulator (each warp its own
//               32-lane quarter), apply ReLU / ReLU-mask / scaling, convert, stage
//               128-byte-wide chunks in swizzled shared memory and write them with
//               TMA stores (coalesced, asynchronous, clipped at the matrix edge);
//               the accumulator is handed back to the MMA warp as soon as the last
//               chunk has left TMEM, while the stores are still draining
//
// Operand layouts.  Row-major storage gives a K-contiguous ("K-major") operand
// only for the forward GEMM; the input-gradient GEMM reads W with N contiguous
// and the weight-gradient GEMM reads both operands with M/N contiguous (the
// contraction runs over batch rows).  Both cases are served without a transpose
// pass: a K-major slab is one TMA box {128 B of K, rows}; an MN-major slab is a
// row of boxes {128 B of M/N, BLOCK_K k-rows}, and the shared-memory descriptor's
// leading/stride byte offsets plus the instruction descriptor's major bits tell
// the tensor core which one it is looking at.
//
// Every wait on an mbarrier is bounded (about two seconds of wall time); a wait
// that gives up raises an abort flag, the kernel records a code in `status`,
// releases its TMEM and returns.
#include <cuda.h>

#include <cmath>
#include <mutex>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace b2 {
namespace {

constexpr int BLOCK_M = 128;
constexpr int SLAB_BYTES = 128;          // bytes of the contiguous dimension per smem row
constexpr int KSTEP_BYTES = 32;          // bytes of K one tcgen05.mma consumes
constexpr int KSTEPS = SLAB_BYTES / KSTEP_BYTES;
constexpr int MAX_STAGES = 8;
constexpr int NUM_THREADS = 192;       // producer warp + MMA warp + 4 epilogue warps
constexpr int NUM_THREADS_SUB2 = 320;  // 256-row tiles: one group of 4 epilogue warps per 128-row accumulator
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;
constexpr uint32_t X3_CORR_COLS = 256;  // fp32-class mode: TMEM column offset of the correction accumulators

struct TcParams {
  int M, N, K;
  int num_m_blocks, num_n_blocks, num_k_blocks;  // m blocks count super-tiles of sub_m * 128 rows
  int block_n, block_k;  // block_k in elements: 128 bytes of K, or 64 in the half-k-block mode
  int ksteps;            // MMAs per k-block and 128-row accumulator: block_k bytes / 32
  uint32_t a_sub_bytes;  // bytes of one 128-row part of the A slab in a stage
  int sub_m;             // 128-row accumulators per tile: 1 (two TMEM stages) or 2 (one stage)
  int acc_stages;
  int num_items;         // work items: whole tiles, then the last partial wave cut in 128-row halves
  int split_from;        // first tile that is cut in halves
  int raster_m;          // row blocks per band of the tile order (L2 reuse, see decode_item)
  int pair;              // 1: CTA-pair kernel (cta_group::2), 256 x 256 tile per pair
  // Stream-K: the k-blocks of all tiles form one sequence that is cut into gridDim.x
  // equal contiguous ranges, so a tile may be computed by two or more CTAs. The CTA that
  // holds the tile's first k-block owns it; the others store fp32 partial accumulators
  // to their workspace slot and raise a flag.
  int streamk;
  int dp_tiles;           // leading tiles handed out whole, round-robin (full waves)
  long long total_units;  // (tiles - dp_tiles) * k-blocks: the stream-K tail
  float* ws;              // gridDim.x slots of 2 * 128 * 256 floats
  unsigned int* ws_flags; // one per CTA, all zero between launches
  int stages;
  int tmem_cols;
  uint32_t idesc;
  int kind_tf32;
  int a_mn, b_mn;                  // 1 = operand stored with M/N contiguous
  uint32_t a_lbo, a_sbo, a_kstep;  // shared-memory descriptor strides / per-k-step advance (bytes)
  uint32_t b_lbo, b_sbo, b_kstep;
  uint32_t a_layout, b_layout;     // descriptor swizzle code: 2 = 128 B, 1 = 128 B with 32-byte atoms
  int a_boxes, b_boxes;            // TMA boxes per stage
  uint32_t a_box_bytes, b_box_bytes;
  int a_box_mn, b_box_mn;          // M/N elements covered by one box
  uint32_t a_stage_bytes, b_stage_bytes;
  void* C;
  long long ldc;
  const void* aux;
  long long ldaux;
  int out_bf16, aux_bf16, epilogue;
  float alpha;
  unsigned int* status;
  // Epilogue through shared memory + TMA stores (tensor map of C as third kernel argument):
  // every epilogue warp owns epi_bufs chunk buffers of 32 rows x 128 bytes behind the stages.
  int tma_store, epi_bufs;  // tma_store: staged epilogue on (1) / direct per-lane stores (0)
  int store_by_tma;         // staged epilogue: 1 = TMA stores, 0 = coalesced st.global read back from the buffer
  uint32_t epi_off;  // byte offset of the chunk buffers from the (aligned) start of shared memory
  // ReLU bit planes: one bit per element, row-major words of 32 columns. A forward epilogue
  // writes the plane of the activation it produces, the input-gradient epilogue of the layer
  // above reads it instead of the activation itself (1/16 of the bytes, one word per lane).
  uint32_t* mask_out;
  const uint32_t* mask_in;
  long long ld_mask;  // words per row
  // fp32-class mode (three tf32 MMAs per k-step on operands split into a high and a low part):
  // x3 = the stage holds A, A_lo, B, B_lo; c_lo = the epilogue also writes the low-order twin
  // of C (v - tf32(v)) for the GEMM that will read C as an operand
  int x3, c_lo;
  void* C_lo;
  unsigned long long* trace;  // see GemmDesc::trace
};

// ------------------------------------------------------------------ PTX wrappers

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ unsigned long long globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. Returns false when it gave up or another role raised the abort flag.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned int* status, unsigned int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer();
  unsigned int spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0xFF) == 0) {
      if (*abort_flag) return false;
      if (globaltimer() - t0 > WAIT_LIMIT_NS) {
        *abort_flag = 1;
        atomicCAS(status, 0u, code);
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ void tma_load_2d(const CUtensorMap* map, uint64_t* bar, void* dst, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until at most N of this thread's bulk groups still READ their shared-memory source
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- CTA-pair (cta_group::2) forms
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `local_addr` (a shared::cta address) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load whose completion bytes are credited to an mbarrier that may live in the peer
// CTA of the pair (`mbar_cluster_addr` is a shared::cluster address). No multicast: the
// data lands in the issuing CTA's own shared memory only.
__device__ __forceinline__ void tma_load_2d_pair(const CUtensorMap* map, uint32_t mbar_cluster_addr, void* dst,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(mbar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
// commit of a pair's MMAs: arrives on the barrier at the same offset in both CTAs
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"((uint16_t)3)
      : "memory");
}
// One k-block (KSTEPS MMAs per 128-row sub-block) issued from precomputed descriptor
// templates. A single thread issues every MMA of the CTA, so the instruction count
// between two MMAs is what bounds the tensor pipe's duty cycle: the constant descriptor
// fields are assembled once per kernel, and per MMA only the 14-bit start-address field
// (address >> 4) is added in.
template <bool TF32, bool PAIR>
__device__ __forceinline__ void mma_issue(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  if (PAIR) {
    if (TF32)
      asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                   "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                   ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
    else
      asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                   "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                   ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  } else {
    if (TF32)
      asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                   "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                   ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
    else
      asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                   "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                   ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
  }
}
// With alo16 / blo16 != 0 (fp32-class mode, tf32 only) the stage also holds the low-order
// twins of both slabs, alo16 / blo16 sixteen-byte units behind the slabs themselves, and every
// k-step issues three MMAs: A*B, A*B_lo and A_lo*B (the tensor core truncates fp32 operands
// to tf32, so A and B stand for their own high parts; A_lo*B_lo, 2^-22 of the product, is dropped).
// The two correction products go to an accumulator of their own, X3_CORR_COLS TMEM columns
// behind the main one, and the epilogue adds the two: the tensor core truncates when it adds
// into an accumulator, a bias that grows with the number of additions, so the main sum should
// see K/8 of them, not 3K/8 (measured at K = 4096: 3.0e-5 relative with one accumulator).
template <int SUB_M, bool TF32, bool PAIR>
__device__ __forceinline__ void issue_kblock(uint32_t tmem_d, uint64_t a_tmpl, uint64_t b_tmpl, uint32_t sa16,
                                             uint32_t sb16, uint32_t a_step16, uint32_t b_step16, uint32_t idesc,
                                             uint32_t block_n, int sub, bool first_kblock, int ksteps,
                                             uint32_t a_sub16, uint32_t alo16 = 0, uint32_t blo16 = 0) {
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    if (ks >= ksteps) break;
    const uint64_t bdesc = b_tmpl + (uint64_t)(sb16 + ks * b_step16);
    const uint32_t accumulate = (ks == 0) ? (first_kblock ? 0u : 1u) : 1u;
#pragma unroll
    for (int i = 0; i < SUB_M; ++i) {  // the 128-row sub-blocks share the B slab
      if (i < sub) {
        const uint64_t adesc = a_tmpl + (uint64_t)(sa16 + i * a_sub16 + ks * a_step16);
        const uint32_t d = tmem_d + (uint32_t)i * block_n;
        mma_issue<TF32, PAIR>(d, adesc, bdesc, idesc, accumulate);
        if (TF32 && !PAIR && SUB_M == 1 && alo16 != 0) {
          mma_issue<TF32, PAIR>(d + X3_CORR_COLS, adesc, bdesc + (uint64_t)blo16, idesc, accumulate);
          mma_issue<TF32, PAIR>(d + X3_CORR_COLS, adesc + (uint64_t)alo16, bdesc, idesc, 1u);
        }
      }
    }
  }
}

// 64-bit shared-memory matrix descriptor (version 1) for a 128-byte-swizzled slab.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo, uint32_t layout) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version (Blackwell)
  d |= (uint64_t)layout << 61;
  return d;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Work item -> (first row, number of 128-row sub-blocks, column block). Tiles are
// numbered band by band: a band is `raster_m` row blocks tall and spans all column
// blocks, row block fastest inside it, so that the ~148 tiles in flight at any time
// cover a roughly square patch of C and share their A and B slabs in L2 (a wave that
// is one row-block column tall re-fetches A from DRAM for every column block).
// Tiles from split_from on are handed out as two 128-row halves so that the last,
// partial wave of a persistent grid costs half a tile time instead of a whole one.
struct Item {
  int m0, sub, n_blk;
};
template <int SUB_M>
__device__ __forceinline__ Item decode_item(int w, int split_from, int num_m_blocks, int num_n_blocks, int raster_m,
                                            int M) {
  int tile = w, half = -1;
  if (SUB_M == 2 && w >= split_from) {
    tile = split_from + ((w - split_from) >> 1);
    half = (w - split_from) & 1;
  }
  Item it;
  const int band_tiles = raster_m * num_n_blocks;
  const int band = tile / band_tiles;
  const int in_band = tile - band * band_tiles;
  const int m_base = band * raster_m;
  const int band_rows = min(raster_m, num_m_blocks - m_base);
  it.n_blk = in_band / band_rows;
  it.m0 = (m_base + in_band % band_rows) * (SUB_M * BLOCK_M);
  it.sub = SUB_M;
  if (SUB_M == 2) {
    if (half >= 0) {
      it.m0 += half * BLOCK_M;
      it.sub = 1;
    } else if (it.m0 + BLOCK_M >= M) {
      it.sub = 1;  // ragged last row block: the second half would be empty
    }
  }
  return it;
}

// Epilogue of one 32-column chunk of one accumulator row: scale, ReLU or ReLU-mask,
// convert, store (16-byte vectors when the chunk lies fully inside the matrix).
__device__ __forceinline__ void epilogue_chunk(const TcParams& p, int row, bool row_ok, int col0,
                                               const uint32_t (&r)[32]) {
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * p.alpha;
  const bool full = (col0 + 32 <= p.N);
  if (p.epilogue == EPI_RELU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = v[j] > 0.f ? v[j] : 0.f;
  } else if (p.epilogue == EPI_MASK && row_ok) {
    if (p.aux_bf16) {
      const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(p.aux) + (long long)row * p.ldaux + col0;
      if (full) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 u = __ldg(reinterpret_cast<const uint4*>(x) + j);
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            // a bf16 is positive iff it is non-zero with the sign bit clear
            uint32_t lo = w[t] & 0xFFFFu, hi = w[t] >> 16;
            if (!(lo != 0 && lo < 0x8000u)) v[j * 8 + t * 2] = 0.f;
            if (!(hi != 0 && hi < 0x8000u)) v[j * 8 + t * 2 + 1] = 0.f;
          }
        }
      } else {
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N && !(__bfloat162float(x[j]) > 0.f)) v[j] = 0.f;
      }
    } else {
      const float* x = static_cast<const float*>(p.aux) + (long long)row * p.ldaux + col0;
      if (full) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float4 u = __ldg(reinterpret_cast<const float4*>(x) + j);
          if (!(u.x > 0.f)) v[j * 4 + 0] = 0.f;
          if (!(u.y > 0.f)) v[j * 4 + 1] = 0.f;
          if (!(u.z > 0.f)) v[j * 4 + 2] = 0.f;
          if (!(u.w > 0.f)) v[j * 4 + 3] = 0.f;
        }
      } else {
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N && !(x[j] > 0.f)) v[j] = 0.f;
      }
    }
  }
  if (row_ok) {
    if (p.out_bf16) {
      __nv_bfloat16* c = static_cast<__nv_bfloat16*>(p.C) + (long long)row * p.ldc + col0;
      if (full) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 o;
          o.x = pack_bf16(v[j * 8 + 0], v[j * 8 + 1]);
          o.y = pack_bf16(v[j * 8 + 2], v[j * 8 + 3]);
          o.z = pack_bf16(v[j * 8 + 4], v[j * 8 + 5]);
          o.w = pack_bf16(v[j * 8 + 6], v[j * 8 + 7]);
          reinterpret_cast<uint4*>(c)[j] = o;
        }
      } else {
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) c[j] = __float2bfloat16_rn(v[j]);
      }
    } else {
      float* c = static_cast<float*>(p.C) + (long long)row * p.ldc + col0;
      if (full) {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          reinterpret_cast<float4*>(c)[j] = make_float4(v[j * 4], v[j * 4 + 1], v[j * 4 + 2], v[j * 4 + 3]);
      } else {
        for (int j = 0; j < 32; ++j)
          if (col0 + j < p.N) c[j] = v[j];
      }
    }
  }
}


// ---- epilogue through shared memory and TMA stores
//
// 32 accumulator columns of one row (this lane's), in place: scale, ReLU (returning the bits
// of the stored value being positive) or masking by `mask` (bit j = keep column j).
__device__ __forceinline__ void epilogue_math32(const TcParams& p, uint32_t (&r)[32], uint32_t mask) {
  // one pass per operation, each a loop of independent elements (the kind of epilogue is uniform)
  if (p.alpha != 1.f) {
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * p.alpha);
  }
  if (p.epilogue == EPI_RELU) {
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(fmaxf(__uint_as_float(r[j]), 0.f));
  } else if (p.epilogue == EPI_MASK) {
#pragma unroll
    for (int j = 0; j < 32; ++j) r[j] = (mask >> j) & 1u ? r[j] : 0u;
  }
}
// mask word of 32 columns from the stored activation itself (callers without a bit plane)
__device__ __forceinline__ uint32_t mask_from_values(const TcParams& p, int row, int col0) {
  uint32_t m = 0;
  if (row >= p.M) return 0;
  if (p.aux_bf16) {
    const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(p.aux) + (long long)row * p.ldaux + col0;
    if (col0 + 32 <= p.N) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(x) + j);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const uint32_t lo = w[t] & 0xFFFFu, hi = w[t] >> 16;  // positive: non-zero, sign clear
          if (lo != 0 && lo < 0x8000u) m |= 1u << (j * 8 + t * 2);
          if (hi != 0 && hi < 0x8000u) m |= 1u << (j * 8 + t * 2 + 1);
        }
      }
    } else {
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N && __bfloat162float(x[j]) > 0.f) m |= 1u << j;
    }
  } else {
    const float* x = static_cast<const float*>(p.aux) + (long long)row * p.ldaux + col0;
    if (col0 + 32 <= p.N) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 u = __ldg(reinterpret_cast<const float4*>(x) + j);
        if (u.x > 0.f) m |= 1u << (j * 4);
        if (u.y > 0.f) m |= 1u << (j * 4 + 1);
        if (u.z > 0.f) m |= 1u << (j * 4 + 2);
        if (u.w > 0.f) m |= 1u << (j * 4 + 3);
      }
    } else {
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N && x[j] > 0.f) m |= 1u << j;
    }
  }
  return m;
}

// A staged chunk (32 rows x 128 bytes, swizzled) to global memory with coalesced stores: the
// warp reads the buffer back so that one instruction covers four whole 128-byte rows (lanes
// 8i..8i+7 take the eight 16-byte pieces of one row) and writes them with st.global - four full
// lines per instruction instead of 32 lines touched by 16 bytes each when every lane stores its
// own row. These stores go through the load/store unit, not through the TMA queue, where a
// store would wait behind the producer's loads of the next tile.
__device__ __forceinline__ void store_chunk_rows(const TcParams& p, void* cbase, const uint8_t* cbuf, int row0,
                                                 int col0, int lane) {
  const int es = p.out_bf16 ? 2 : 4;
  const int per_piece = 16 / es;  // elements per 16-byte piece
  const int piece = lane & 7;
  const int gcol = col0 + piece * per_piece;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rr = 4 * i + (lane >> 3);
    const uint4 v = *reinterpret_cast<const uint4*>(cbuf + rr * 128 + ((piece ^ (rr & 7)) << 4));
    const int grow = row0 + rr;
    if (grow < p.M && gcol < p.N) {
      uint8_t* g = static_cast<uint8_t*>(cbase) + ((long long)grow * p.ldc + gcol) * es;
      if (gcol + per_piece <= p.N) {
        *reinterpret_cast<uint4*>(g) = v;
      } else {  // ragged right edge: element by element
        const int left = p.N - gcol;
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          const uint32_t word = wi == 0 ? v.x : wi == 1 ? v.y : wi == 2 ? v.z : v.w;
          if (es == 4) {
            if (wi < left) reinterpret_cast<uint32_t*>(g)[wi] = word;
          } else {
            if (2 * wi < left) reinterpret_cast<uint16_t*>(g)[2 * wi] = (uint16_t)(word & 0xFFFFu);
            if (2 * wi + 1 < left) reinterpret_cast<uint16_t*>(g)[2 * wi + 1] = (uint16_t)(word >> 16);
          }
        }
      }
    }
  }
}

// One epilogue warp's 32 rows of one accumulator: rows row0 .. row0+31 (this lane: row0 + lane),
// columns n0 .. n0 + block_n of C, accumulator at TMEM address `taddr` (lane quarter and first
// column already applied). `release()` hands the accumulator back to the MMA warp; it is called
// once, right after the last chunk has been read out of TMEM. `buf` = this warp's chunk
// buffers (EPI_BUFS x 4 KB, 1024-byte aligned), `buf_i` = the one to use next (kept between tiles).
template <int EPI_BUFS, typename Release>
__device__ __forceinline__ void epilogue_rows_tma(const TcParams& p, const CUtensorMap* tma_c,
                                                  const CUtensorMap* tma_c_lo, uint32_t taddr, int row0, int n0,
                                                  uint8_t* buf, int& buf_i, int lane, Release release) {
  const int row = row0 + lane;
  const int chunk_cols = p.out_bf16 ? 64 : 32;  // 128 bytes of C per row and chunk
  const int nchunks = p.block_n / chunk_cols;
  const uint32_t swz = (uint32_t)(lane & 7);
  for (int ch = 0; ch < nchunks; ++ch) {
    const int col0 = n0 + ch * chunk_cols;
    if (col0 >= p.N) break;  // uniform across the warp
    const bool last = (ch == nchunks - 1) || (col0 + chunk_cols >= p.N);
    uint32_t words[32];  // the chunk's 128 bytes of this row
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if (half == 1 && !p.out_bf16) break;
      const int c0 = col0 + half * 32;
      uint32_t r[32];
      tmem_ld32(taddr + (uint32_t)(ch * chunk_cols + half * 32), r);
      if (p.x3) {  // main sum + sum of the two correction products (an fp32 add with rounding)
        uint32_t r2[32];
        tmem_ld32(taddr + X3_CORR_COLS + (uint32_t)(ch * chunk_cols + half * 32), r2);
#pragma unroll
        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r2[j]));
      }
      if (last && (half == 1 || !p.out_bf16)) {
        tc_fence_before();
        __syncwarp();
        release();
      }
      uint32_t mask = 0;
      if (p.epilogue == EPI_MASK) {
        if (p.mask_in) mask = (row < p.M && c0 < p.N) ? __ldg(p.mask_in + (long long)row * p.ld_mask + (c0 >> 5)) : 0u;
        else mask = c0 < p.N ? mask_from_values(p, row, c0) : 0u;
      }
      epilogue_math32(p, r, mask);
      uint32_t bits = 0;
      if (p.out_bf16) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          words[half * 16 + j] = pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
        if (p.mask_out) {
          // the plane is written behind a ReLU, so no half is negative: a half is positive iff its low
          // 15 bits are not all zero; adding 0x7FFF carries into bit 15 (31) exactly then. Four
          // partial words keep the dependency chains short.
          uint32_t part[4] = {0, 0, 0, 0};
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const uint32_t m = ((words[half * 16 + j] & 0x7FFF7FFFu) + 0x7FFF7FFFu) & 0x80008000u;
            part[j & 3] |= (((m >> 15) | (m >> 30)) & 3u) << (2 * j);
          }
          bits = (part[0] | part[1]) | (part[2] | part[3]);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) words[j] = r[j];
        if (p.mask_out) {
          uint32_t part[4] = {0, 0, 0, 0};
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (__uint_as_float(r[j]) > 0.f) part[j & 3] |= 1u << j;
          bits = (part[0] | part[1]) | (part[2] | part[3]);
        }
      }
      if (p.mask_out && row < p.M && c0 < p.N) p.mask_out[(long long)row * p.ld_mask + (c0 >> 5)] = bits;
    }
    if (p.store_by_tma) {
      // the chunk buffer is free once the store issued EPI_BUFS chunks ago has read it
      if (lane == 0) bulk_wait_read<EPI_BUFS - 1>();
      __syncwarp();
    }
    uint8_t* cbuf = buf + (size_t)buf_i * 4096;
    {
      uint8_t* dst = cbuf + (size_t)lane * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j)  // 16-byte piece j of row `lane` sits at slot j ^ (lane & 7): 128-byte swizzle
        *reinterpret_cast<uint4*>(dst + ((j ^ swz) << 4)) =
            make_uint4(words[4 * j], words[4 * j + 1], words[4 * j + 2], words[4 * j + 3]);
    }
    if (p.store_by_tma) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && row0 < p.M) {
        tma_store_2d(tma_c, cbuf, col0, row0);
        bulk_commit();
      }
      buf_i = (buf_i + 1 == EPI_BUFS) ? 0 : buf_i + 1;
    } else {
      __syncwarp();
      store_chunk_rows(p, p.C, cbuf, row0, col0, lane);
      __syncwarp();  // every lane has read the buffer before it is written again
    }
    if (p.c_lo) {
      // fp32-class mode: the low-order twin of the chunk, v - tf32(v) (exact), the same way
      if (p.store_by_tma) {
        if (lane == 0) bulk_wait_read<EPI_BUFS - 1>();
        __syncwarp();
      }
      uint8_t* lbuf = buf + (size_t)buf_i * 4096;
      uint8_t* dst2 = lbuf + (size_t)lane * 128;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint32_t lo[4];
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          const float v = __uint_as_float(words[4 * j + t]);
          lo[t] = __float_as_uint(v - __uint_as_float(words[4 * j + t] & 0xFFFFE000u));
        }
        *reinterpret_cast<uint4*>(dst2 + ((j ^ swz) << 4)) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
      }
      if (p.store_by_tma) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && row0 < p.M) {
          tma_store_2d(tma_c_lo, lbuf, col0, row0);
          bulk_commit();
        }
        buf_i = (buf_i + 1 == EPI_BUFS) ? 0 : buf_i + 1;
      } else {
        __syncwarp();
        store_chunk_rows(p, p.C_lo, lbuf, row0, col0, lane);
        __syncwarp();
      }
    }
  }
}

// Piece of work of one CTA: k-blocks [kb0, kb1) of one tile (all of them unless stream-K
// cut the tile).
struct Work {
  int m0, sub, n_blk, kb0, kb1;
  long long unit0;  // position of kb0 in the stream-K sequence, -1 for a whole tile
};
struct WorkIter {
  int w;
  long long unit, end;
};
constexpr int WS_SLOT_FLOATS = 2 * BLOCK_M * 256;

__device__ __forceinline__ long long streamk_start(const TcParams& p, int cta) {
  return ((long long)cta * p.total_units) / (long long)gridDim.x;
}
__device__ __forceinline__ void work_begin(const TcParams& p, WorkIter& wi) {
  wi.w = blockIdx.x;
  wi.unit = streamk_start(p, blockIdx.x);
  wi.end = streamk_start(p, blockIdx.x + 1);
}
// Whole tiles first (round-robin over the grid, so that the tiles in flight stay a compact
// patch of C), then - stream-K only - this CTA's contiguous share of the k-blocks of the
// remaining tiles.
template <int SUB_M>
__device__ __forceinline__ bool work_next(const TcParams& p, WorkIter& wi, Work& wk) {
  if (p.streamk) {
    if (wi.w < p.dp_tiles) {
      const Item it = decode_item<SUB_M>(wi.w, 0x7fffffff, p.num_m_blocks, p.num_n_blocks, p.raster_m, p.M);
      wk.m0 = it.m0; wk.sub = it.sub; wk.n_blk = it.n_blk; wk.kb0 = 0; wk.kb1 = p.num_k_blocks;
      wk.unit0 = -1;
      wi.w += gridDim.x;
      return true;
    }
    if (wi.unit >= wi.end) return false;
    const int KB = p.num_k_blocks;
    const int tail_tile = (int)(wi.unit / KB);
    const int tile = p.dp_tiles + tail_tile;
    const int kb0 = (int)(wi.unit - (long long)tail_tile * KB);
    const long long rem = wi.end - wi.unit;
    const int kb1 = rem < (long long)(KB - kb0) ? kb0 + (int)rem : KB;
    const Item it = decode_item<SUB_M>(tile, 0x7fffffff, p.num_m_blocks, p.num_n_blocks, p.raster_m, p.M);
    wk.m0 = it.m0; wk.sub = it.sub; wk.n_blk = it.n_blk; wk.kb0 = kb0; wk.kb1 = kb1;
    wk.unit0 = wi.unit;
    wi.unit += kb1 - kb0;
    return true;
  }
  if (wi.w >= p.num_items) return false;
  const Item it = decode_item<SUB_M>(wi.w, p.split_from, p.num_m_blocks, p.num_n_blocks, p.raster_m, p.M);
  wk.m0 = it.m0; wk.sub = it.sub; wk.n_blk = it.n_blk; wk.kb0 = 0; wk.kb1 = p.num_k_blocks;
  wk.unit0 = -1;
  wi.w += gridDim.x;
  return true;
}
__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* ptr) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
  return v;
}
__device__ __forceinline__ void epilogue_bar_sync(int nthreads) {
  asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}

// ------------------------------------------------------------------------ kernel

// Register budget: the 320 threads of the 256-row mode get 168 registers each (the register file is
// handed out as if the CTA had 384 threads: 192 per thread was refused at launch), the 192
// threads of the other modes 255.
template <int SUB_M>
__global__ void __launch_bounds__(SUB_M == 2 ? NUM_THREADS_SUB2 : NUM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ CUtensorMap tma_a_lo,
               const __grid_constant__ CUtensorMap tma_b_lo, const __grid_constant__ CUtensorMap tma_c_lo,
               const __grid_constant__ TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t acc_full_bar[2];
  __shared__ __align__(8) uint64_t acc_empty_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // stage layout: A [A_lo] B [B_lo] (the low-order twins only in the fp32-class mode)
  const uint32_t lo_mul = p.x3 ? 2u : 1u;
  const uint32_t stage_bytes = (p.a_stage_bytes + p.b_stage_bytes) * lo_mul;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &abort_s;

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full_bar[a], 1);
      mbar_init(&acc_empty_bar[a], 4 * SUB_M);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tma_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tma_b) : "memory");
    if (p.tma_store && p.store_by_tma) asm volatile("prefetch.tensormap [%0];" ::"l"(&tma_c) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  const uint32_t acc_cols = (uint32_t)(SUB_M * p.block_n);  // TMEM columns of one accumulator stage
  constexpr int ACC_STAGES = SUB_M == 2 ? 1 : 2;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      WorkIter wi;
      Work it;
      work_begin(p, wi);
      int load_tile = 0;
      while (ok && work_next<SUB_M>(p, wi, it)) {
        const uint32_t a_bytes = (uint32_t)it.sub * p.a_sub_bytes;
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 1u)) { ok = false; break; }
          if (p.trace && blockIdx.x == 0 && load_tile == 1 && kb - it.kb0 < TC_TRACE_KBLOCKS)
            p.trace[TC_TRACE_TILES * 4 + TC_TRACE_KBLOCKS + (kb - it.kb0)] = globaltimer();
          uint8_t* sa = smem + (size_t)stage * stage_bytes;
          uint8_t* sb = sa + p.a_stage_bytes * lo_mul;
          mbar_expect_tx(&full_bar[stage], (a_bytes + p.b_stage_bytes) * lo_mul);
          const int k0 = kb * p.block_k;
          for (uint32_t part = 0; part < lo_mul; ++part) {  // the operands, then their low-order twins
            const CUtensorMap* ma = part ? &tma_a_lo : &tma_a;
            const CUtensorMap* mb = part ? &tma_b_lo : &tma_b;
            uint8_t* da = sa + part * p.a_stage_bytes;
            uint8_t* db = sb + part * p.b_stage_bytes;
            if (p.a_mn) {
              const int nbox = it.sub * p.a_boxes;  // a_boxes per 128 rows
              for (int b = 0; b < nbox; ++b)
                tma_load_2d(ma, &full_bar[stage], da + (size_t)b * p.a_box_bytes, it.m0 + b * p.a_box_mn, k0);
            } else {
#pragma unroll
              for (int i = 0; i < SUB_M; ++i)
                if (i < it.sub)
                  tma_load_2d(ma, &full_bar[stage], da + (size_t)i * p.a_sub_bytes, k0, it.m0 + i * BLOCK_M);
            }
            if (p.b_mn) {
              for (int b = 0; b < p.b_boxes; ++b)
                tma_load_2d(mb, &full_bar[stage], db + (size_t)b * p.b_box_bytes, it.n_blk * p.block_n + b * p.b_box_mn,
                            k0);
            } else {
              tma_load_2d(mb, &full_bar[stage], db, k0, it.n_blk * p.block_n);
            }
          }
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        ++load_tile;
      }
      if (!ok) {
        // give copies already in flight a bounded time to land before the CTA retires
        const unsigned long long t0 = globaltimer();
        while (globaltimer() - t0 < 2000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint64_t a_tmpl = make_smem_desc(0, p.a_lbo, p.a_sbo, p.a_layout);
      const uint64_t b_tmpl = make_smem_desc(0, p.b_lbo, p.b_sbo, p.b_layout);
      const uint32_t smem16 = smem_u32(smem) >> 4, stage16 = stage_bytes >> 4, a_stage16 = p.a_stage_bytes >> 4;
      const uint32_t a_step16 = p.a_kstep >> 4, b_step16 = p.b_kstep >> 4, idesc = p.idesc;
      const uint32_t block_n = (uint32_t)p.block_n;
      const bool tf32 = p.kind_tf32 != 0;
      const uint32_t alo16 = p.x3 ? a_stage16 : 0u, blo16 = p.x3 ? (p.b_stage_bytes >> 4) : 0u;
      const int ksteps = p.ksteps;
      const uint32_t a_sub16 = p.a_sub_bytes >> 4;
      int trace_tile = 0;
      WorkIter wi;
      Work it;
      work_begin(p, wi);
      while (ok && work_next<SUB_M>(p, wi, it)) {
        if (!mbar_wait(&acc_empty_bar[acc], acc_phase ^ 1, abort_flag, p.status, 2u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)acc * acc_cols;
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 3u)) { ok = false; break; }
          tc_fence_after();
          if (p.trace && blockIdx.x == 0) {
            if (kb == it.kb0 && trace_tile < TC_TRACE_TILES) p.trace[trace_tile * 4 + 0] = globaltimer();
            if (trace_tile == 1 && kb - it.kb0 < TC_TRACE_KBLOCKS) p.trace[TC_TRACE_TILES * 4 + (kb - it.kb0)] = globaltimer();
          }
          const uint32_t sa16 = smem16 + (uint32_t)stage * stage16;
          if (tf32)
            issue_kblock<SUB_M, true, false>(tmem_d, a_tmpl, b_tmpl, sa16, sa16 + a_stage16 * lo_mul, a_step16, b_step16,
                                             idesc, block_n, it.sub, kb == it.kb0, ksteps, a_sub16, alo16, blo16);
          else
            issue_kblock<SUB_M, false, false>(tmem_d, a_tmpl, b_tmpl, sa16, sa16 + a_stage16, a_step16, b_step16,
                                              idesc, block_n, it.sub, kb == it.kb0, ksteps, a_sub16);
          tc_commit(&empty_bar[stage]);  // frees the stage once these MMAs have read it
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&acc_full_bar[acc]);   // accumulator complete -> epilogue
        ++trace_tile;
        if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    constexpr int EPI_THREADS = 128 * SUB_M;
    constexpr int EPI_BUFS = SUB_M == 2 ? 1 : 2;  // chunk buffers per warp (shared memory left beside the stages)
    const int sub = (warp - 2) >> 2;  // each group of four epilogue warps drains one 128-row accumulator
    uint8_t* ebuf = smem + p.epi_off + (size_t)(warp - 2) * (EPI_BUFS * 4096);
    int ebuf_i = 0;
    int epi_tile = 0;
    WorkIter wi;
    Work it;
    work_begin(p, wi);
    while (work_next<SUB_M>(p, wi, it)) {
      const int n_blk = it.n_blk;
      const int KB = p.num_k_blocks;
      if (p.tma_store) {  // whole tiles only (no stream-K pieces)
        if (!mbar_wait(&acc_full_bar[acc], acc_phase, abort_flag, p.status, 4u)) break;
        tc_fence_after();
        const bool tracing = p.trace && blockIdx.x == 0 && warp == 2 && lane == 0 && epi_tile < TC_TRACE_TILES;
        if (tracing) p.trace[epi_tile * 4 + 1] = globaltimer();
        uint64_t* release_bar = &acc_empty_bar[acc];
        if (sub < it.sub) {
          epilogue_rows_tma<EPI_BUFS>(
              p, &tma_c, &tma_c_lo,
              tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * acc_cols + (uint32_t)(sub * p.block_n),
              it.m0 + sub * BLOCK_M + q * 32, n_blk * p.block_n, ebuf, ebuf_i, lane,
              [&]() {
                if (lane == 0) mbar_arrive(release_bar);
                if (tracing) p.trace[epi_tile * 4 + 2] = globaltimer();
              });
          if (tracing) p.trace[epi_tile * 4 + 3] = globaltimer();
          ++epi_tile;
        } else {  // half tile: this group's accumulator was not used
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(release_bar);
        }
        if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
        continue;
      }
      const bool contributor = it.kb0 > 0;                 // stream-K: someone else owns this tile
      const bool owner_partial = it.kb0 == 0 && it.kb1 < KB;  // stream-K: others finish this tile
      const long long tile_end = it.unit0 - it.kb0 + KB;
      if (!mbar_wait(&acc_full_bar[acc], acc_phase, abort_flag, p.status, 4u)) break;
      tc_fence_after();
      int first_contrib = 0, last_contrib = -1;
      if (owner_partial) {
        // the CTAs after this one hold the rest of the tile, each as the FIRST piece of its
        // range, so their partial sums are ready long before this CTA gets here
        first_contrib = (int)blockIdx.x + 1;
        last_contrib = first_contrib;
        while (last_contrib + 1 < (int)gridDim.x && streamk_start(p, last_contrib + 1) < tile_end) ++last_contrib;
        bool ready = true;
        for (int c = first_contrib; c <= last_contrib && ready; ++c) {
          const unsigned long long t0 = globaltimer();
          unsigned int spins = 0;
          while (ld_acquire_u32(p.ws_flags + c) == 0u) {
            if ((++spins & 0x3F) == 0 && (*abort_flag || globaltimer() - t0 > WAIT_LIMIT_NS)) {
              *abort_flag = 1;
              atomicCAS(p.status, 0u, 5u);
              ready = false;
              break;
            }
          }
        }
        epilogue_bar_sync(EPI_THREADS);  // every epilogue thread has seen the flags
        if (threadIdx.x == 64)
          for (int c = first_contrib; c <= last_contrib; ++c) p.ws_flags[c] = 0u;  // consumed: re-arm
        if (!ready) break;
      }
      if (sub < it.sub) {
      const int row = it.m0 + sub * BLOCK_M + q * 32 + lane;
      const bool row_ok = row < p.M;
      const size_t ws_row = ((size_t)sub * BLOCK_M + q * 32 + lane) * (size_t)p.block_n;
      for (int c0 = 0; c0 < p.block_n; c0 += 32) {
        const int col0 = n_blk * p.block_n + c0;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)acc * acc_cols +
                      (uint32_t)(sub * p.block_n + c0), r);
        if (contributor) {
          float4* dst = reinterpret_cast<float4*>(p.ws + (size_t)blockIdx.x * WS_SLOT_FLOATS + ws_row + c0);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            dst[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                 __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        } else {
          for (int c = first_contrib; c <= last_contrib; ++c) {
            const float4* src = reinterpret_cast<const float4*>(p.ws + (size_t)c * WS_SLOT_FLOATS + ws_row + c0);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 v = __ldcg(src + j);
              r[4 * j] = __float_as_uint(__uint_as_float(r[4 * j]) + v.x);
              r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + v.y);
              r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + v.z);
              r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + v.w);
            }
          }
          epilogue_chunk(p, row, row_ok, col0, r);
        }
      }
      }  // sub-block
      if (contributor) {
        __threadfence();                 // partial sums visible device-wide before the flag
        epilogue_bar_sync(EPI_THREADS);
        if (threadIdx.x == 64) atomicExch(p.ws_flags + blockIdx.x, 1u);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty_bar[acc]);
      if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
    }
    if (p.tma_store && p.store_by_tma && lane == 0) bulk_wait_all();  // the chunk buffers must outlive the stores that read them
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols)
                 : "memory");
  }
}

// ------------------------------------------------------ kernel, CTA-pair variant
//
// Two CTAs of a cluster (two neighbouring SMs) work on one 256 x 256 tile with
// tcgen05.mma.cta_group::2: CTA r of the pair holds rows [r*128, r*128+128) of the A
// slab and the r-th 128-column half of the B slab, the leader CTA (rank 0) issues
// every MMA, and each CTA's TMEM receives its own 128 rows x 256 columns of the
// accumulator. Each SM's shared memory then feeds 4 KB of A + 4 KB of B per MMA
// instead of 4 KB + 8 KB, and is filled with 32 KB instead of 48 KB per k-block,
// with two TMEM stages kept for epilogue overlap.
//
// Barriers: full[s] lives in the leader and collects the bytes of both CTAs' loads;
// empty[s] and acc_full[a] exist in both CTAs and are signalled by one multicast
// tcgen05.commit; acc_empty[a] lives in the leader and counts the epilogue warps of
// both CTAs (the peer's arrive remotely). A cluster barrier after initialisation keeps
// remote signals away from uninitialised barriers, one before exit keeps either CTA's
// shared memory and TMEM alive while the other may still touch it.
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const __grid_constant__ CUtensorMap tma_c, const __grid_constant__ TcParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[MAX_STAGES];
  __shared__ __align__(8) uint64_t acc_full_bar[2];
  __shared__ __align__(8) uint64_t acc_empty_bar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_s;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t stage_bytes = p.a_stage_bytes + p.b_stage_bytes;  // per CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  volatile int* abort_flag = &abort_s;

  if (threadIdx.x == 0) {
    abort_s = 0;
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full_bar[a], 1);
      mbar_init(&acc_empty_bar[a], 8);  // four epilogue warps in each CTA of the pair
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tma_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tma_b) : "memory");
    if (p.tma_store && p.store_by_tma) asm volatile("prefetch.tensormap [%0];" ::"l"(&tma_c) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  const int num_tiles = p.num_m_blocks * p.num_n_blocks;  // 256 x 256 tiles

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int load_tile = 0;
      for (int t = pair; t < num_tiles && ok; t += num_pairs, ++load_tile) {
        const Item it = decode_item<2>(t, num_tiles, p.num_m_blocks, p.num_n_blocks, p.raster_m, 1 << 30);
        const int m0 = it.m0 + (int)rank * BLOCK_M;                   // this CTA's rows of A
        const int n0 = it.n_blk * p.block_n + (int)rank * (p.block_n / 2);  // this CTA's half of B
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, 1u)) { ok = false; break; }
          if (p.trace && blockIdx.x < 2 && load_tile == 1 && kb < TC_TRACE_KBLOCKS)  // leader and peer of pair 0
            p.trace[TC_TRACE_TILES * 4 + (1 + blockIdx.x) * TC_TRACE_KBLOCKS + kb] = globaltimer();
          uint8_t* sa = smem + (size_t)stage * stage_bytes;
          uint8_t* sb = sa + p.a_stage_bytes;
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * stage_bytes);  // both CTAs' bytes
          const uint32_t full_addr = map_to_cta(smem_u32(&full_bar[stage]), 0);
          const int k0 = kb * p.block_k;
          if (p.a_mn) {
            for (int b = 0; b < p.a_boxes; ++b)
              tma_load_2d_pair(&tma_a, full_addr, sa + (size_t)b * p.a_box_bytes, m0 + b * p.a_box_mn, k0);
          } else {
            tma_load_2d_pair(&tma_a, full_addr, sa, k0, m0);
          }
          if (p.b_mn) {
            for (int b = 0; b < p.b_boxes; ++b)
              tma_load_2d_pair(&tma_b, full_addr, sb + (size_t)b * p.b_box_bytes, n0 + b * p.b_box_mn, k0);
          } else {
            tma_load_2d_pair(&tma_b, full_addr, sb, k0, n0);
          }
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer();
        while (globaltimer() - t0 < 2000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ----------------------------------------------- MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint64_t a_tmpl = make_smem_desc(0, p.a_lbo, p.a_sbo, p.a_layout);
      const uint64_t b_tmpl = make_smem_desc(0, p.b_lbo, p.b_sbo, p.b_layout);
      const uint32_t smem16 = smem_u32(smem) >> 4, stage16 = stage_bytes >> 4, a_stage16 = p.a_stage_bytes >> 4;
      const uint32_t a_step16 = p.a_kstep >> 4, b_step16 = p.b_kstep >> 4, idesc = p.idesc;
      const bool tf32 = p.kind_tf32 != 0;
      int trace_tile = 0;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        if (!mbar_wait(&acc_empty_bar[acc], acc_phase ^ 1, abort_flag, p.status, 2u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * p.block_n);
        for (int kb = 0; kb < p.num_k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, 3u)) { ok = false; break; }
          tc_fence_after();
          if (p.trace && blockIdx.x == 0) {
            if (kb == 0 && trace_tile < TC_TRACE_TILES) p.trace[trace_tile * 4 + 0] = globaltimer();
            if (trace_tile == 1 && kb < TC_TRACE_KBLOCKS) p.trace[TC_TRACE_TILES * 4 + kb] = globaltimer();
          }
          const uint32_t sa16 = smem16 + (uint32_t)stage * stage16;
          if (tf32)
            issue_kblock<1, true, true>(tmem_d, a_tmpl, b_tmpl, sa16, sa16 + a_stage16, a_step16, b_step16, idesc,
                                        0u, 1, kb == 0, p.ksteps, 0u);
          else
            issue_kblock<1, false, true>(tmem_d, a_tmpl, b_tmpl, sa16, sa16 + a_stage16, a_step16, b_step16, idesc,
                                         0u, 1, kb == 0, p.ksteps, 0u);
          tc_commit_pair(&empty_bar[stage]);
          if (++stage == p.stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit_pair(&acc_full_bar[acc]);
        ++trace_tile;
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint8_t* ebuf = smem + p.epi_off + (size_t)(warp - 2) * (2 * 4096);
    int ebuf_i = 0;
    int epi_tile = 0;
    for (int t = pair; t < num_tiles; t += num_pairs) {
      const Item it = decode_item<2>(t, num_tiles, p.num_m_blocks, p.num_n_blocks, p.raster_m, 1 << 30);
      if (!mbar_wait(&acc_full_bar[acc], acc_phase, abort_flag, p.status, 4u)) break;
      tc_fence_after();
      if (p.tma_store) {
        const uint32_t release_addr = map_to_cta(smem_u32(&acc_empty_bar[acc]), 0);
        const bool tracing = p.trace && blockIdx.x == 0 && warp == 2 && lane == 0 && epi_tile < TC_TRACE_TILES;
        if (tracing) p.trace[epi_tile * 4 + 1] = globaltimer();
        epilogue_rows_tma<2>(p, &tma_c, &tma_c, tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * p.block_n),
                             it.m0 + (int)rank * BLOCK_M + q * 32, it.n_blk * p.block_n, ebuf, ebuf_i, lane,
                             [&]() {
                               if (lane == 0) mbar_arrive_cluster(release_addr);
                               if (tracing) p.trace[epi_tile * 4 + 2] = globaltimer();
                             });
        if (tracing) p.trace[epi_tile * 4 + 3] = globaltimer();
        ++epi_tile;
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
        continue;
      }
      const int row = it.m0 + (int)rank * BLOCK_M + q * 32 + lane;
      const bool row_ok = row < p.M;
      for (int c0 = 0; c0 < p.block_n; c0 += 32) {
        const int col0 = it.n_blk * p.block_n + c0;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * p.block_n + c0), r);
        epilogue_chunk(p, row, row_ok, col0, r);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty_bar[acc]), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
    if (p.tma_store && p.store_by_tma && lane == 0) bulk_wait_all();
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols)
                 : "memory");
  }
}

// ------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D tensor map over a row-major matrix: `inner` contiguous elements per row,
// `outer` rows, `ld` elements between rows; box = box_inner x box_outer.
// swizzle: 0 = 128 bytes, 1 = 128 bytes in 32-byte atoms, 2 = 64 bytes
bool make_map(CUtensorMap* map, const void* base, int elem_bytes, long long inner, long long outer, long long ld,
              int box_inner, int box_outer, int swizzle) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return false;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                   : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace

struct TcPlan {
  CUtensorMap map_a, map_b, map_c, map_a_lo, map_b_lo, map_c_lo;
  TcParams p;
  int grid;
  size_t smem;
};

TcPlan* gemm_tc_plan_create(const GemmDesc& g, int sm_count, char* err, size_t errlen) {
  auto fail = [&](const char* why) -> TcPlan* {
    if (err && errlen) snprintf(err, errlen, "%s", why);
    return nullptr;
  };
  const int eb = g.in_type == T_BF16 ? 2 : 4;
  const int ob = g.out_type == T_BF16 ? 2 : 4;
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) return fail("empty GEMM");
  if (g.beta != 0.f) return fail("beta != 0");
  const bool x3 = g.A_lo != nullptr && g.B_lo != nullptr;
  if ((g.A_lo != nullptr) != (g.B_lo != nullptr)) return fail("fp32-class mode needs the twins of both operands");
  if (x3 && eb != 4) return fail("fp32-class mode is for fp32 operands");
  if (g.C_lo && ob != 4) return fail("a result twin needs an fp32 result");
  const bool a_mn = (g.sAm == 1 && g.sAk != 1), b_mn = (g.sBn == 1 && g.sBk != 1);
  if (!a_mn && g.sAk != 1) return fail("A has no unit stride");
  if (!b_mn && g.sBk != 1) return fail("B has no unit stride");
  const long long lda = a_mn ? g.sAk : g.sAm, ldb = b_mn ? g.sBk : g.sBn;
  auto aligned = [](const void* p, long long ld, int bytes) {
    return (reinterpret_cast<uintptr_t>(p) % 16 == 0) && ((ld * bytes) % 16 == 0);
  };
  if (!aligned(g.A, lda, eb) || !aligned(g.B, ldb, eb)) return fail("operand not 16-byte aligned");
  if (x3 && (!aligned(g.A_lo, lda, eb) || !aligned(g.B_lo, ldb, eb))) return fail("operand twin not 16-byte aligned");
  if (g.C_lo && !aligned(g.C_lo, g.ldc, ob)) return fail("result twin not 16-byte aligned");
  if (!aligned(g.C, g.ldc, ob)) return fail("output not 16-byte aligned");
  if (g.epilogue == EPI_MASK && !aligned(g.aux, g.ldaux, eb)) return fail("mask operand not 16-byte aligned");
  if (g.N < 16) return fail("N < 16");

  TcPlan* plan = new TcPlan();
  TcParams& p = plan->p;
  memset(&p, 0, sizeof p);
  p.M = g.M; p.N = g.N; p.K = g.K;
  // Tile shape: 256 x 256 (two 128-row accumulators sharing each B slab: least shared-memory
  // traffic per flop, but a single accumulator stage), 128 x 256, 128 x 128 or 128 x 64 (two
  // accumulator stages). Chosen by a cost model: waves of the persistent grid times the time
  // of one tile, where a tile's time is its area divided by the rate the tile shape sustains
  // relative to 256 x 256 (measured at 8192 x 4096 x 4096: 128 x 256 reaches 0.93 of it; a
  // 128-column MMA reads A and B from shared memory at the 128 B/clk ceiling, 0.70; 64 columns
  // 0.45). Filling every SM is not the goal: 1024 x 4096 is served faster by 128 tiles of
  // 128 x 256 on 128 SMs than by 256 tiles of 128 x 128 on all 148.
  auto tiles = [&](int rows, int n) { return (long long)((g.M + rows - 1) / rows) * ((g.N + n - 1) / n); };
  int bn = 256;
  {
    struct Cand { int sub_m, bn; double rate; };
    const Cand cands[4] = {{2, 256, 1.0}, {1, 256, 0.93}, {1, 128, 0.70}, {1, 64, 0.45}};
    double best = 1e300;
    int best_i = 3;
    for (int i = 0; i < 4; ++i) {
      const Cand& c = cands[i];
      if (c.bn / 2 >= g.N && c.bn > 64) continue;  // tile wider than twice the matrix
      if (x3 && (c.sub_m == 2 || c.bn == 256)) continue;  // twice the shared memory per stage: 128 x 128 at most
      const long long T = tiles(c.sub_m * BLOCK_M, c.bn);
      double waves;
      if (c.sub_m == 2) {
        // the last partial wave is handed out as 128-row halves when that fits in one wave
        const long long full = T / sm_count, rem = T % sm_count;
        waves = (double)full + (rem == 0 ? 0.0 : (T > sm_count && rem * 2 <= sm_count ? 0.5 : 1.0));
      } else {
        waves = (double)((T + sm_count - 1) / sm_count);
      }
      const double cost = waves * (double)(c.sub_m * BLOCK_M) * c.bn / c.rate;
      if (cost < best * 0.999) { best = cost; best_i = i; }
    }
    bn = cands[best_i].bn;
    p.sub_m = cands[best_i].sub_m;
  }
  p.block_n = bn;
  const char* force = getenv("B2_TC_SUB_M");
  if (force && (force[0] == '1' || (force[0] == '2' && bn == 256))) p.sub_m = force[0] - '0';
  if (const char* fb = getenv("B2_TC_BN")) {  // experiments: force the tile width
    const int v = atoi(fb);
    if (v == 64 || v == 128 || v == 256) { bn = v; p.block_n = v; if (v != 256) p.sub_m = 1; }
  }
  if (x3 && (bn == 256 || p.sub_m == 2)) { bn = 128; p.block_n = 128; p.sub_m = 1; }
  // CTA pairs: a 256 x 256 tile per pair of SMs once there is a tile for every pair
  {
    const char* pe = getenv("B2_TC_PAIR");
    const bool want = pe ? (pe[0] == '1' || pe[0] == '2') : false;
    const bool any_count = pe && pe[0] == '2';  // experiments: also when there are fewer tiles than CTA pairs
    p.pair = (want && !x3 && bn == 256 && (any_count || tiles(2 * BLOCK_M, bn) >= sm_count / 2)) ? 1 : 0;
    if (p.pair) p.sub_m = 2;  // tile rows for the work decomposition: 128 per CTA of the pair
  }
  // B2_TC_HALF_K=1: k-blocks of 64 bytes of K instead of 128 (64-byte swizzle for K-contiguous
  // slabs), i.e. a ring with twice the slots of half the size, handed back after half as many
  // MMAs. Off by default: measured slower (8192 x 4096 x 4096 forward 1023 against 1319 TFLOP/s);
  // 64-byte rows arrive at 62 GB/s per SM against 93 GB/s for 128-byte rows.
  bool half_k = false;
  if (const char* e = getenv("B2_TC_HALF_K")) half_k = e[0] == '1';
  const int kb_bytes = half_k ? SLAB_BYTES / 2 : SLAB_BYTES;  // bytes of K per k-block
  p.block_k = kb_bytes / eb;
  p.ksteps = kb_bytes / KSTEP_BYTES;
  p.acc_stages = (p.sub_m == 2 && !p.pair) ? 1 : 2;
  p.num_m_blocks = (g.M + p.sub_m * BLOCK_M - 1) / (p.sub_m * BLOCK_M);
  p.num_n_blocks = (g.N + bn - 1) / bn;
  p.num_k_blocks = (g.K + p.block_k - 1) / p.block_k;
  p.tmem_cols = 2 * bn < 32 ? 32 : 2 * bn;  // 128, 256 or 512: powers of two
  if (x3) p.tmem_cols = 512;                // two main accumulators (bn <= 128) and, 256 columns on, their correction twins
  {
    // band height that makes a wave of sm_count tiles about square in elements of C
    const double aspect = (double)bn / (p.sub_m * BLOCK_M);
    int rm = (int)(sqrt((double)sm_count * aspect) + 0.5);
    if (const char* r = getenv("B2_TC_RASTER")) rm = atoi(r);
    if (rm < 1) rm = 1;
    if (rm > p.num_m_blocks) rm = p.num_m_blocks;
    p.raster_m = rm;
  }
  {
    const long long T = (long long)p.num_m_blocks * p.num_n_blocks;
    const long long rem = T % sm_count;
    p.split_from = (int)T;
    if (p.sub_m == 2 && !p.pair && T > sm_count && rem > 0 && rem * 2 <= sm_count) p.split_from = (int)(T - rem);
    p.num_items = (int)(p.split_from + 2 * (T - p.split_from));
    // Stream-K when whole tiles would leave part of the last wave idle (or there are fewer
    // tiles than SMs) and the caller provided a workspace.
    p.dp_tiles = (int)((T / sm_count) * sm_count);
    p.total_units = (T - p.dp_tiles) * p.num_k_blocks;
    // Off unless B2_TC_STREAMK=1: on the shapes of the benchmark configurations the two
    // extra exposed epilogues of a stream-K tail (partial store, partial reload) cost about
    // as much as the idle part of the last wave they remove; it pays for long-K shapes only.
    const char* sk = getenv("B2_TC_STREAMK");
    const bool allow = sk ? (sk[0] == '1') : false;
    p.streamk = (allow && !p.pair && !x3 && g.ws && g.ws_flags && T % sm_count != 0 && p.total_units >= sm_count) ? 1 : 0;
    p.ws = g.ws;
    p.ws_flags = g.ws_flags;
    if (p.streamk) {
      p.split_from = (int)T;
      p.num_items = (int)T;
    }
  }
  p.kind_tf32 = (eb == 4);
  p.a_mn = a_mn; p.b_mn = b_mn;
  const uint32_t fmt = (eb == 4) ? 2u : 1u;  // tf32 : bf16
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
            ((uint32_t)(bn >> 3) << 17) | ((uint32_t)((p.pair ? 2 * BLOCK_M : BLOCK_M) >> 4) << 24);
  const int slab_elems = SLAB_BYTES / eb;
  const int cta_bn = p.pair ? bn / 2 : bn;  // B rows (columns of C) held by one CTA
  // K-contiguous slabs: rows of kb_bytes, 128-byte swizzle (8-row groups of 1024 B) or, for
  // half k-blocks, 64-byte swizzle (8-row groups of 512 B, descriptor layout code 4).
  // M/N-contiguous slabs: boxes of 128 bytes of M or N by block_k k-rows.
  p.a_sub_bytes = BLOCK_M * kb_bytes;
  p.a_stage_bytes = (p.pair ? 1 : p.sub_m) * p.a_sub_bytes;
  p.b_stage_bytes = cta_bn * kb_bytes;
  const uint32_t k_sbo = 8 * kb_bytes, k_layout = half_k ? 4u : 2u;
  const int k_swz = half_k ? 2 : 0;  // make_map's swizzle choice
  bool ok = true;
  // M/N-contiguous operands: 16-bit elements use the plain 128-byte swizzle (8 k-rows of
  // 128 B per 1024-byte group); 32-bit elements are only accepted in the variant that
  // swizzles 32-byte atoms (4 k-rows per 512-byte group).
  const bool mn_atom32 = (eb == 4);
  const uint32_t mn_group_bytes = mn_atom32 ? 512 : 1024;
  const uint32_t mn_layout = mn_atom32 ? 1 : 2;
  if (a_mn) {
    // boxes of {128 bytes of M, block_k k-rows}; 8-row groups 1024 B apart, M atoms one box apart
    p.a_boxes = BLOCK_M / slab_elems;
    p.a_box_mn = slab_elems;
    p.a_box_bytes = p.block_k * SLAB_BYTES;
    p.a_lbo = p.a_box_bytes;
    p.a_sbo = mn_group_bytes;
    p.a_layout = mn_layout;
    p.a_kstep = (KSTEP_BYTES / eb) * SLAB_BYTES;
    ok = ok && make_map(&plan->map_a, g.A, eb, g.M, g.K, lda, slab_elems, p.block_k, mn_atom32 ? 1 : 0);
    if (x3) ok = ok && make_map(&plan->map_a_lo, g.A_lo, eb, g.M, g.K, lda, slab_elems, p.block_k, mn_atom32 ? 1 : 0);
  } else {
    p.a_boxes = 1;
    p.a_box_bytes = p.a_sub_bytes;
    p.a_lbo = 16;
    p.a_sbo = k_sbo;
    p.a_kstep = KSTEP_BYTES;
    p.a_layout = k_layout;
    ok = ok && make_map(&plan->map_a, g.A, eb, g.K, g.M, lda, p.block_k, BLOCK_M, k_swz);
    if (x3) ok = ok && make_map(&plan->map_a_lo, g.A_lo, eb, g.K, g.M, lda, p.block_k, BLOCK_M, k_swz);
  }
  if (b_mn) {
    p.b_boxes = cta_bn / slab_elems;
    p.b_box_mn = slab_elems;
    p.b_box_bytes = p.block_k * SLAB_BYTES;
    p.b_lbo = p.b_box_bytes;
    p.b_sbo = mn_group_bytes;
    p.b_layout = mn_layout;
    p.b_kstep = (KSTEP_BYTES / eb) * SLAB_BYTES;
    ok = ok && make_map(&plan->map_b, g.B, eb, g.N, g.K, ldb, slab_elems, p.block_k, mn_atom32 ? 1 : 0);
    if (x3) ok = ok && make_map(&plan->map_b_lo, g.B_lo, eb, g.N, g.K, ldb, slab_elems, p.block_k, mn_atom32 ? 1 : 0);
  } else {
    p.b_boxes = 1;
    p.b_box_bytes = p.b_stage_bytes;
    p.b_lbo = 16;
    p.b_sbo = k_sbo;
    p.b_kstep = KSTEP_BYTES;
    p.b_layout = k_layout;
    ok = ok && make_map(&plan->map_b, g.B, eb, g.K, g.N, ldb, p.block_k, cta_bn, k_swz);
    if (x3) ok = ok && make_map(&plan->map_b_lo, g.B_lo, eb, g.K, g.N, ldb, p.block_k, cta_bn, k_swz);
  }
  if (!ok) {
    delete plan;
    return fail("cuTensorMapEncodeTiled failed");
  }
  if (!x3) {  // the kernel takes all six maps: unused ones are copies of valid ones
    plan->map_a_lo = plan->map_a;
    plan->map_b_lo = plan->map_b;
  }
  p.x3 = x3 ? 1 : 0;
  // Epilogue chunk buffers (32 rows x 128 bytes per buffer) behind the stages: one buffer per
  // epilogue warp in the 256-row mode (eight warps; three 64 KB stages fill the rest), two otherwise.
  memset(&plan->map_c, 0, sizeof plan->map_c);
  {
    // staged epilogue unless stream-K pieces are in play (B2_TC_EPILOGUE=direct: per-lane stores);
    // the staged chunks leave by TMA stores, or with B2_TC_TMA_STORE=0 by coalesced st.global read
    // back from the buffer (measured at 8192 x 4096 x 4096: 7.2 us against 8.2-10 us from the
    // accumulator's completion to its release)
    const char* ee = getenv("B2_TC_EPILOGUE");
    const char* e = getenv("B2_TC_TMA_STORE");
    p.tma_store = (!p.streamk && !(ee && ee[0] == 'd')) ? 1 : 0;
    p.store_by_tma = (p.tma_store && !(e && e[0] == '0')) ? 1 : 0;
    if (p.store_by_tma) {
      EncodeTiledFn enc = get_encode();
      cuuint64_t dims[2] = {(cuuint64_t)g.N, (cuuint64_t)g.M};
      cuuint64_t strides[1] = {(cuuint64_t)g.ldc * ob};
      cuuint32_t box[2] = {(cuuint32_t)(128 / ob), 32};
      cuuint32_t estr[2] = {1, 1};
      if (!enc || enc(&plan->map_c, ob == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                      g.C, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                      CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        p.store_by_tma = 0;  // e.g. a row pitch beyond the tensor map's limits
      plan->map_c_lo = plan->map_c;
      if (p.store_by_tma && g.C_lo &&
          enc(&plan->map_c_lo, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, g.C_lo, dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        p.store_by_tma = 0;
    }
  }
  p.c_lo = (g.C_lo && p.tma_store) ? 1 : 0;
  p.C_lo = g.C_lo;
  if (g.C_lo && !p.c_lo) {
    delete plan;
    return fail("the result twin needs the staged epilogue");
  }
  p.epi_bufs = (p.sub_m == 2 && !p.pair) ? 1 : 2;
  const size_t epi_bytes = p.tma_store ? (size_t)(p.pair ? 4 : 4 * p.sub_m) * p.epi_bufs * 4096 : 0;
  const size_t stage = (size_t)(p.a_stage_bytes + p.b_stage_bytes) * (x3 ? 2 : 1);
  const size_t budget = 227 * 1024 - 1024 /* alignment slack */ - 512 /* static: barriers */;
  int stages = (int)((budget - epi_bytes) / stage);
  if (stages > MAX_STAGES) stages = MAX_STAGES;
  if (const char* e = getenv("B2_TC_STAGES")) {  // experiments: fewer stages than fit
    const int want = atoi(e);
    if (want >= 2 && want < stages) stages = want;
  }
  if (stages < 2) {
    delete plan;
    return fail("tile does not fit in shared memory");
  }
  p.stages = stages;
  p.epi_off = (uint32_t)((size_t)stages * stage);
  // Always ask for the same large carve-out so that only one CTA (one TMEM
  // allocation) is ever resident per SM.
  plan->smem = 1024 + (size_t)stages * stage + epi_bytes;
  if (plan->smem < 140 * 1024) plan->smem = 140 * 1024;
  p.C = g.C; p.ldc = g.ldc; p.aux = g.aux; p.ldaux = g.ldaux;
  p.out_bf16 = g.out_type == T_BF16;
  p.aux_bf16 = g.in_type == T_BF16;
  p.epilogue = g.epilogue;
  p.alpha = g.alpha;
  p.mask_out = nullptr;
  p.mask_in = nullptr;
  p.ld_mask = 0;
  p.trace = g.trace;
  plan->grid = p.num_items < sm_count ? p.num_items : sm_count;
  if (p.streamk) plan->grid = sm_count;
  if (p.pair) {
    const int pairs = sm_count / 2;
    const int T = p.num_m_blocks * p.num_n_blocks;
    plan->grid = 2 * (T < pairs ? T : pairs);
  }
  return plan;
}

void gemm_tc_plan_destroy(TcPlan* p) { delete p; }

bool gemm_tc_plan_set_mask(TcPlan* plan, uint32_t* mask_out, const uint32_t* mask_in, long long ld_words) {
  if (!plan || !plan->p.tma_store || plan->p.N % 32 != 0 || ld_words * 32 < plan->p.N) return false;
  if (mask_out && plan->p.epilogue != EPI_RELU) return false;
  if (mask_in && plan->p.epilogue != EPI_MASK) return false;
  plan->p.mask_out = mask_out;
  plan->p.mask_in = mask_in;
  plan->p.ld_mask = ld_words;
  return true;
}

cudaError_t gemm_tc_launch(const TcPlan* plan, cudaStream_t stream, unsigned int* status) {
  // the kernels' shared-memory limit is raised once per device; host threads that drive
  // different GPUs may come here at the same time
  static std::mutex attr_mutex;
  static unsigned long long attr_set = 0;  // one bit per device ordinal
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> attr_lock(attr_mutex);
    if (!(attr_set >> (dev & 63) & 1ull)) {
      cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
      if (e != cudaSuccess) return e;
      attr_set |= 1ull << (dev & 63);
    }
  }
  TcParams p = plan->p;
  p.status = status;
  if (p.pair) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan->grid);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = plan->smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemm_tc_pair_kernel, plan->map_a, plan->map_b, plan->map_c, p);
  }
  if (p.sub_m == 2)
    gemm_tc_kernel<2><<<plan->grid, NUM_THREADS_SUB2, plan->smem, stream>>>(
        plan->map_a, plan->map_b, plan->map_c, plan->map_a_lo, plan->map_b_lo, plan->map_c_lo, p);
  else
    gemm_tc_kernel<1><<<plan->grid, NUM_THREADS, plan->smem, stream>>>(
        plan->map_a, plan->map_b, plan->map_c, plan->map_a_lo, plan->map_b_lo, plan->map_c_lo, p);
  return cudaGetLastError();
}

}  // namespace b2

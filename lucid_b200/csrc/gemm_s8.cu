// s8 x s8 -> s32 contraction on the 5th-generation tensor cores (sm_100a):
//   TMA (cp.async.bulk.tensor, 128-byte swizzle) -> shared-memory ring ->
//   tcgen05.mma kind::i8 issued by one thread -> int32 accumulators in TMEM ->
//   epilogue warps read TMEM (tcgen05.ld), apply scales / bias / activation /
//   requantisation in registers and store.
//
// One persistent CTA per SM (or one CTA pair per two SMs): warp 0 = TMA producer,
// warp 1 = MMA issuer and TMEM owner, then 8 or 16 epilogue warps (four per TMEM
// lane quadrant, each taking a share of the tile's columns).  Two accumulator
// stages in TMEM let the epilogue of one work item overlap the mainloop of the
// next.  The same mainloop serves the Linear GEMM and the NHWC implicit-GEMM
// convolution (the producer walks filter taps with shifted, optionally strided
// 4-D TMA boxes whose out-of-image elements are zero-filled, which is the padding).
//
// Work is scheduled either tile by tile (round robin over the CTAs) or, when the
// tile count does not fill whole waves, as equal contiguous runs of k-blocks per
// CTA ("stream-K"): a tile cut by a run boundary is finished by the CTA that holds
// its first k-blocks, which adds the other CTAs' int32 partial sums from an
// L2-resident scratch before the epilogue (integer addition: order-free, exact).
//
// Every wait (mbarrier, scratch flag) is bounded: when the budget runs out the CTA
// raises an abort flag, reports LQ_ERR_TIMEOUT through the status word, drains and
// frees its TMEM before returning, so the context stays usable.
#include <cuda.h>

#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "common.cuh"

namespace lq {
namespace {

constexpr int BM = 128;       // rows of the CTA tile == TMEM lanes
constexpr int BK = 128;       // bytes (= int8 elements) of K per stage: one 128B swizzle atom
constexpr int UMMA_K = 32;    // K per tcgen05.mma for 8-bit operands
// Epilogue warps per CTA (EW): 8 when the mainloop of a tile outlasts its epilogue (large K:
// more ring stages, fewer polling warps), 16 when the epilogue is the long pole (small K).
// The register file is split over the SM's four schedulers (16 K registers each): 10 warps leave
// at most 3 on one scheduler (168 registers per thread), 18 warps 5 (96 registers).
constexpr int threads_for(int ew) { return 64 + 32 * ew; }  // producer warp, MMA warp, epilogue warps
constexpr int kTmemCols = 512;
constexpr long long kWaitBudgetCycles = 1ll << 31;  // ~1 s: default budget of every device-side wait
// stream-K / exchange scratch (caller's workspace): a 4 KB header, then one slot per CTA
constexpr int kWsHeaderBytes = 4096;
constexpr int kWsMaxCtas = 192;                      // slots sized for up to 192 SMs
constexpr int kWsSlotBytes = BM * 256 * 4;           // one CTA's 128 x 256 int32 partial tile
constexpr int kWsFlagsOffset = 256;                  // header: ticket at 0, 2 words per CTA from here
static_assert(kWsFlagsOffset + kWsMaxCtas * 8 <= kWsHeaderBytes, "flags must fit the header");

template <int BN, bool PAIR, int EW>
struct Cfg {
  // PAIR: two CTAs of a cluster share one 256 x BN tile (tcgen05 cta_group::2); each
  // CTA stages its own 128 rows of A and half of the B rows.
  // the ring shares the SM's 227 KB with EW x 4 KB of epilogue staging
  static constexpr int kStages = EW == 16 ? (PAIR ? 5 : (BN == 256 ? 3 : 5)) : (PAIR ? 6 : (BN == 256 ? 4 : 6));
  static constexpr int kABytes = BM * BK;
  static constexpr int kBRows = PAIR ? BN / 2 : BN;
  static constexpr int kBBytes = kBRows * BK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // ring + 1 KB alignment slack + barriers (512 B) + per-warp output staging (EW x 4 KB)
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 512 + EW * 4096;
};

struct Geometry {
  // GEMM: rows = M.  Conv: output pixels arranged as (img, P, Q).
  int conv;            // 0 GEMM, 1 implicit-GEMM conv
  int M, N, K;         // GEMM extents (conv: M = imgs*P*Q, K = R*S*C)
  int tiles_m, tiles_n, num_kb;
  // conv only
  int P, Q, C, R, S;
  int pad_h, pad_w, stride_h, stride_w, dil_h, dil_w;
  int tile_h, tile_w, tiles_p, tiles_q;
  int cblocks;         // ceil(C / BK)
  int streamk;         // 1: contiguous runs of k-blocks per CTA instead of whole tiles
  long long wait_budget;  // clock64 cycles a device-side wait may take
#ifdef LQ_TESTING
  int test_no_loads;   // test-only build: the producer issues nothing, so the first wait runs out
#endif
};

struct Epi {
  int out_dtype, act, a_scale_mode, qmin, qmax;
  const float* a_scale;
  const float* a_zp;
  const int32_t* b_rowsum;
  const float* b_scale;
  const float* bias;
  const float* out_scale;
  const float* out_zp;
  void* out;           // first destination
  void* more_outs[7];  // further destinations of the same tiles (peer GPUs' buffers)
  int n_dst;           // number of destinations (>= 1)
  int multicast;       // `out` is an NVSwitch multicast address: one multimem store reaches every rank
  long long col0;      // column offset of this GEMM's columns inside every destination
  long long ldo;  // elements
  int n_out;      // columns of out (N, or N/2 for the gated epilogue)
  int vec_ok;     // 16-byte vector stores allowed
  int par_vec;    // per-column parameter arrays are 16-byte aligned (vector loads)
  int32_t* status;
  uint8_t* ws;    // scratch (stream-K partial tiles and flags, completion ticket) or null
  // exchange step of a sharded layer: once every CTA has stored its tiles, the last one bumps
  // this rank's counter and stores the new value into its flag word on every peer
  int32_t* signal_counter;
  int32_t* peer_flags[8];
  int n_flags;
};

// ---- PTX wrappers ----------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait.  Returns false when the CTA is aborting or the budget ran out.  SLEEP_NS > 0
// backs off between polls (long waits by warps that are not on the critical path).
template <int SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          long long budget) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t it = 1;; ++it) {
    if (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > budget) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}
// Warp-uniform wait: every lane polls, the warp agrees on the outcome.
template <int SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                               long long budget) {
  return __all_sync(0xffffffffu, mbar_wait<SLEEP_NS>(bar, parity, abort_flag, budget));
}
// Bounded wait on a global-memory word written by another CTA (ld.acquire.gpu): true once
// *p == want.
__device__ __forceinline__ bool flag_wait_eq(const unsigned int* p, unsigned int want, volatile int* abort_flag,
                                             long long budget) {
  const long long t0 = clock64();
  for (uint32_t it = 1;; ++it) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    if (v == want) return true;
    __nanosleep(100);
    if ((it & 63u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > budget) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}
// One lane of a converged warp.  The surrounding control flow stays warp-uniform so that
// loop state and descriptors can live in uniform registers.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, int x, int y,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tm), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tm, int c0, int c1,
                                            int c2, int c3, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(tm), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

// ---- cta_group::2 (CTA pair) variants -----------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `local_addr` in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
               : "memory");
}
// The pair's loads complete on the leader CTA's barrier (no multicast: each CTA fetches
// its own rows).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* tm, int x, int y,
                                                 uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tm), "r"(x), "r"(y), "r"(cluster_bar)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* tm, int c0, int c1,
                                                 int c2, int c3, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(tm), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(cluster_bar)
      : "memory");
}
// commit that arrives on the same barrier offset in both CTAs of the pair
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void tc_mma_i8_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// K-major operand tile in shared memory, 128-byte swizzle: rows are 128 B, eight
// rows form a 1024 B swizzle atom (stride-byte-offset), leading-byte-offset is 1
// (ignored for swizzled K-major), descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fffu);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor for kind::i8: D = s32, A = u8|s8, B = s8, both K-major.
__host__ __device__ constexpr uint32_t make_idesc(int a_signed, int bn, int mma_m = BM) {
  return (2u << 4) | ((uint32_t)(a_signed ? 1 : 0) << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) |
         ((uint32_t)(mma_m >> 4) << 24);
}

// ---- epilogue helpers -------------------------------------------------------------
__device__ __forceinline__ float silu_f32(float x) {
  return __fmul_rn(x, __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))));
}

__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// load and wait in one statement: the registers are defined only once the data has landed
__device__ __forceinline__ void tc_ld16_sync(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld_dep16(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]),
                 "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]),
                 "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}
// tcgen05.wait::ld that also carries the loaded registers, so that no use of them can be
// scheduled ahead of the wait.
__device__ __forceinline__ void tc_wait_ld_dep(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]),
                 "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]),
                 "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]),
                 "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
                 "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]),
                 "+r"(r[31])
               :
               : "memory");
}

enum { KIND_S32 = 0, KIND_F32 = 1, KIND_BF16 = 2, KIND_Q8 = 3 };
template <int KIND>
struct KindInfo {
  static constexpr int kEsz = KIND == KIND_Q8 ? 1 : (KIND == KIND_BF16 ? 2 : 4);
};

// Per-thread state of one tile's epilogue.
struct RowCtx {
  float sa;          // activation scale of this thread's row
  int zpa;           // activation zero point
  Divisor so;        // output grid: scale (with its hoisted reciprocal)
  float zo;          // ... and zero point
  float fqmin, fqmax;
  // the requantising epilogue's integer tail: code = bits(q + 1.5 * 2^23) + zofs, clamped to
  // [clo, chi] (a ReLU is folded into clo) unless the saturating pack already does that
  int zofs, clo, chi;
  bool need_clamp, out_signed;
  bool grid_ok;  // the output grid is inside the short division's domain (else: full-range blocks)
  uint32_t row_mask; // valid rows of this warp (bit r = tile row quad*32 + r)
  long long row0;    // global output row of the warp's first row
};

// Partial sums of a tile that other CTAs computed (stream-K): contributor i's 128 x BN int32
// tile lies in scratch slot `cta0 + i * cta_step`, as [lane quadrant][16-column block][16-byte
// piece][lane] so that a warp's store or load of one piece is one contiguous 512-byte run.
struct Partials {
  const uint8_t* slots;  // first slot of the scratch; null = nothing to add
  int n, cta0, cta_step;
};
template <int BN>
__device__ __forceinline__ size_t partial_index(int quad, int colblk, int piece, int lane) {
  return (size_t)(((quad * (BN / 16) + colblk) * 4 + piece) * 32 + lane) * 16;
}
// acc[0..16) += the contributors' sums of the same 16 columns (L2 loads: the data was written
// by other SMs during this launch)
template <int BN>
__device__ __forceinline__ void add_partials16(uint32_t (&acc)[16], const Partials& ps, int quad, int colblk,
                                               int lane) {
  for (int i = 0; i < ps.n; ++i) {
    const uint8_t* slot = ps.slots + (size_t)(ps.cta0 + i * ps.cta_step) * kWsSlotBytes;
#pragma unroll
    for (int pc = 0; pc < 4; ++pc) {
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(slot + partial_index<BN>(quad, colblk, pc, lane)));
      acc[4 * pc] += v.x, acc[4 * pc + 1] += v.y, acc[4 * pc + 2] += v.z, acc[4 * pc + 3] += v.w;
    }
  }
}
// This warp's share (32 lanes x BN / PARTS columns) of an accumulator tile, raw, into the
// CTA's scratch slot.
template <int BN, int PARTS>
__device__ __forceinline__ void dump_partial(uint32_t taddr, uint8_t* slot, int quad, int part, int lane) {
  constexpr int NB = BN / PARTS / 16;
#pragma unroll 1
  for (int blk = 0; blk < NB; ++blk) {
    const int colblk = part * NB + blk;
    uint32_t acc[16];
    tc_ld16_sync(taddr + colblk * 16, acc);
#pragma unroll
    for (int pc = 0; pc < 4; ++pc)
      __stcg(reinterpret_cast<uint4*>(slot + partial_index<BN>(quad, colblk, pc, lane)),
             make_uint4(acc[4 * pc], acc[4 * pc + 1], acc[4 * pc + 2], acc[4 * pc + 3]));
  }
}

// One 16-byte store to a multicast address: NVSwitch writes it into the buffer of every GPU
// bound to the multicast object (the issuing GPU's included), so the link carries each tile once
// instead of once per peer.
__device__ __forceinline__ void multimem_st16(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "f"(__uint_as_float(v.x)),
               "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

// Flush the warp's staging buffer (32 rows x 128 B, 16-byte pieces XOR-swizzled by row):
// eight lanes write one full 128-byte line of a row.
template <int ESZ>
__device__ __forceinline__ void flush_group(const uint8_t* stg, int lane, const Epi& ep,
                                            const RowCtx& rc, int gcol0, int pieces) {
  constexpr int EPP = 16 / ESZ;  // elements per 16-byte piece
  const int pc = lane & 7;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int r = k * 4 + (lane >> 3);
    const uint4 v = *reinterpret_cast<const uint4*>(stg + r * 128 + ((pc ^ (r & 7)) << 4));
    const int col = gcol0 + pc * EPP;
    const int nvalid = ep.n_out - col;
    if (((rc.row_mask >> r) & 1u) && pc < pieces && nvalid > 0) {
      const long long off = ((rc.row0 + r) * ep.ldo + ep.col0 + col) * ESZ;
      // the same 16 bytes go to every destination: this GPU's buffer first, then the peers'
      // (plain stores over NVLink; the exchange overlaps the mainloop of the next tile)
      for (int dsti = 0; dsti < ep.n_dst; ++dsti) {
        uint8_t* dst = reinterpret_cast<uint8_t*>(dsti == 0 ? ep.out : ep.more_outs[dsti - 1]) + off;
        if (ep.multicast) {
          multimem_st16(dst, v);  // the host admits only shapes whose pieces are all whole
        } else if (ep.vec_ok && nvalid >= EPP) {
          *reinterpret_cast<uint4*>(dst) = v;
        } else {
          const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int e = 0; e < EPP; ++e) {
            if (e < nvalid) {
              if (ESZ == 4) reinterpret_cast<uint32_t*>(dst)[e] = wv[e];
              else if (ESZ == 2) reinterpret_cast<uint16_t*>(dst)[e] = (uint16_t)(wv[e >> 1] >> (16 * (e & 1)));
              else dst[e] = (uint8_t)(wv[e >> 2] >> (8 * (e & 3)));
            }
          }
        }
      }
    }
  }
}

// Parameters of 16 consecutive columns; `fast` = the block is inside N and the arrays are
// 16-byte aligned (straight-line vector loads, every lane asks for the same address).
__device__ __forceinline__ void load_params16(const float* p, int col, int ncols, bool fast,
                                              float dflt, float (&v)[16]) {
  if (fast) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float4 t = __ldg(reinterpret_cast<const float4*>(p + col) + q);
      v[4 * q] = t.x, v[4 * q + 1] = t.y, v[4 * q + 2] = t.z, v[4 * q + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = col + j < ncols ? __ldg(p + col + j) : dflt;
  }
}

// y[j] = f32(acc[j] - zpa * rowsum[j]) * (sa * sb[j]) [+ bias[j]] for 16 columns; every float
// step is a separate binary32 operation.
__device__ __forceinline__ void dequant16(const Epi& ep, const Geometry& g, const RowCtx& rc,
                                          const uint32_t* acc, int col, float (&y)[16]) {
  const bool fast = ep.par_vec && col + 16 <= g.N;
  float p[16];
  load_params16(ep.b_scale, col, g.N, fast, 1.0f, p);
  if (ep.b_rowsum != nullptr && rc.zpa != 0) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int rs = col + j < g.N ? __ldg(ep.b_rowsum + col + j) : 0;
      y[j] = __fmul_rn((float)((int)acc[j] - rc.zpa * rs), __fmul_rn(rc.sa, p[j]));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) y[j] = __fmul_rn((float)(int)acc[j], __fmul_rn(rc.sa, p[j]));
  }
  if (ep.bias != nullptr) {
    load_params16(ep.bias, col, g.N, fast, 0.0f, p);
#pragma unroll
    for (int j = 0; j < 16; ++j) y[j] = __fadd_rn(y[j], p[j]);
  }
}

// 16 outputs of one row -> 4 * esz packed words.
template <int KIND>
__device__ __forceinline__ void finish16(const float (&y)[16], uint32_t (&w)[16], const RowCtx& rc) {
  if (KIND == KIND_F32) {
#pragma unroll
    for (int j = 0; j < 16; ++j) w[j] = __float_as_uint(y[j]);
  } else if (KIND == KIND_BF16) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(y[2 * j], y[2 * j + 1]);
      w[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float x4[4] = {y[4 * j], y[4 * j + 1], y[4 * j + 2], y[4 * j + 3]};
      float c[4];
      code4_f32(x4, rc.so, rc.zo, rc.fqmin, rc.fqmax, c);
      // identical byte patterns for both storages once the value is inside its grid
      w[j] = rc.fqmin < 0.0f ? pack4_s8(c) : pack4_u8(c);
    }
  }
}

// Epilogue of one accumulator tile for one warp: 32 TMEM lanes (rows) x 1/PARTS of the
// tile's output columns (`part` selects which), in blocks of 16 columns: TMEM -> registers ->
// outputs -> this thread's slot of the staging buffer; the warp flushes the buffer whenever a
// 128-byte group per row is complete.  Four warps share a lane quadrant, so the TMEM and
// parameter load latencies of one warp hide behind the arithmetic of the others; the short
// blocks keep the 16-warp build inside its 96-register budget.
template <int BN, int KIND, bool GATED, int PARTS>
__device__ __forceinline__ void epilogue_tile(const Epi& ep, const Geometry& g, const RowCtx& rc,
                                              uint32_t taddr, uint8_t* stg, int lane, int part,
                                              int n0, int on0, const Partials& ps, int quad) {
  constexpr int ESZ = KindInfo<KIND>::kEsz;
  constexpr int OUTC = GATED ? BN / 2 : BN;   // output columns of the tile
  constexpr int WCOLS = OUTC / PARTS;         // ... of this warp
  constexpr int NB = WCOLS / 16;              // 16-column blocks per warp
  constexpr int BPG = 8 / ESZ;                // blocks per 128-byte group
  static_assert(NB >= 1, "tile too narrow for this many column parts");
  const int c0 = part * WCOLS;                // first output column of this warp inside the tile
#pragma unroll 1
  for (int blk = 0; blk < NB; ++blk) {
    const int oc = c0 + blk * 16;             // output column inside the tile
    uint32_t acc[16], acc_u[16];
    if (GATED) {
      tc_ld16(taddr + oc, acc);
      tc_ld16(taddr + BN / 2 + oc, acc_u);
      tc_wait_ld_dep16(acc);
      tc_wait_ld_dep16(acc_u);
      if (ps.n) {
        add_partials16<BN>(acc, ps, quad, oc >> 4, lane);
        add_partials16<BN>(acc_u, ps, quad, (BN / 2 + oc) >> 4, lane);
      }
    } else {
      tc_ld16_sync(taddr + oc, acc);
      if (ps.n) add_partials16<BN>(acc, ps, quad, oc >> 4, lane);
    }
    uint32_t w[16];
    if (KIND == KIND_S32) {
      if (ep.b_rowsum != nullptr && rc.zpa != 0) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int col = n0 + oc + j;
          const int rs = col < g.N ? __ldg(ep.b_rowsum + col) : 0;
          w[j] = (uint32_t)((int)acc[j] - rc.zpa * rs);
        }
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) w[j] = acc[j];
      }
    } else {
      float y[16];
      dequant16(ep, g, rc, acc, n0 + oc, y);
      if (GATED) {
        float u[16];
        dequant16(ep, g, rc, acc_u, n0 + BN / 2 + oc, u);
#pragma unroll
        for (int j = 0; j < 16; ++j) y[j] = __fmul_rn(silu_f32(y[j]), u[j]);
      } else if (ep.act == LQ_ACT_RELU) {
#pragma unroll
        for (int j = 0; j < 16; ++j) y[j] = fmaxf(y[j], 0.0f);
      }
      finish16<KIND>(y, w, rc);
    }
    // stage: row = lane, 16-byte pieces swizzled by (row & 7)
    const int cs = blk % BPG;
#pragma unroll
    for (int i = 0; i < ESZ; ++i) {
      const int piece = cs * ESZ + i;
      *reinterpret_cast<uint4*>(stg + lane * 128 + ((piece ^ (lane & 7)) << 4)) =
          make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
    }
    if (cs == BPG - 1 || blk == NB - 1) {
      __syncwarp();
      flush_group<ESZ>(stg, lane, ep, rc, on0 + c0 + (blk - cs) * 16, (cs + 1) * ESZ);
      __syncwarp();
    }
  }
}

// Four integral floats already inside an 8-bit grid (signed or unsigned) -> four packed codes:
// the low byte of each integer.
__device__ __forceinline__ uint32_t pack4_low_bytes(const float (&c)[4]) {
  const uint32_t a = (uint32_t)__float2int_rz(c[0]), b = (uint32_t)__float2int_rz(c[1]);
  const uint32_t d = (uint32_t)__float2int_rz(c[2]), e = (uint32_t)__float2int_rz(c[3]);
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(d, e, 0x0040), 0x5410);
}

// Lean requantising epilogue: 8-bit codes to one destination, tile inside N.  Compared with
// epilogue_tile: the per-column parameters of the warp's columns are combined once per column
// of tiles into a table in the warp's staging area (scale product folded when the activation
// scale is per tensor; `fill` says the warp moved to another column of tiles) and read back with
// broadcast 16-byte shared loads, scale / bias / division run on the packed f32x2 pipe with the
// integer tail of the stream encodes (no float-to-int conversion, no clip in float), and every
// thread stores its 16 finished bytes straight to global memory (its row's next 16 bytes follow one
// block later, so L2 merges the sectors) -- no staging pass.  What the epilogue descriptor asks
// for (bias, ReLU, zero-point correction) is a template argument, so the 16-column loop has no
// branch on it; signed and unsigned grids share one byte pack (the codes are already clipped
// into their grid, so the low byte of the integer is the code either way).  Taken for a
// per-tensor activation scale, whose product with the weight scale folds into the table.
template <int BN, int PARTS, bool HAS_BIAS, bool RELU, bool HAS_ZP>
__device__ __forceinline__ void epilogue_tile_q8(const Epi& ep, const RowCtx& rc, uint32_t taddr, uint8_t* stg,
                                                 int lane, int part, int n0, bool fill, const Partials& ps,
                                                 int quad) {
  constexpr int WCOLS = BN / PARTS;
  constexpr int NB = WCOLS / 16;
  const int c0 = part * WCOLS;
  float* t_scale = reinterpret_cast<float*>(stg);
  float* t_bias = t_scale + WCOLS;
  int* t_rowsum = reinterpret_cast<int*>(t_bias + WCOLS);
  if (fill) {
    __syncwarp();
    for (int j = lane; j < WCOLS; j += 32) {
      const int col = n0 + c0 + j;
      const float sb = ep.b_scale ? __ldg(ep.b_scale + col) : 1.0f;
      t_scale[j] = __fmul_rn(rc.sa, sb);
      if (HAS_BIAS) t_bias[j] = __ldg(ep.bias + col);
      if (HAS_ZP) t_rowsum[j] = __ldg(ep.b_rowsum + col);
    }
    __syncwarp();
  }
  const bool row_ok = (rc.row_mask >> lane) & 1u;
  uint8_t* dst = reinterpret_cast<uint8_t*>(ep.out) + (rc.row0 + lane) * ep.ldo + ep.col0 + n0 + c0;
  const F2 y2 = f2_pack(rc.so.y, rc.so.y), ns2 = f2_pack(-rc.so.s, -rc.so.s);
  const F2 magic2 = f2_pack(12582912.0f, 12582912.0f);
  // one 16-column block: accumulators in registers -> 16 finished bytes in global memory
  auto finish_block = [&](uint32_t (&acc)[16], int blk) {
    if (ps.n) add_partials16<BN>(acc, ps, quad, (c0 >> 4) + blk, lane);
    uint32_t w[4];
    float big = rc.grid_ok ? 0.0f : INFINITY;
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const float4 s4 = *reinterpret_cast<const float4*>(t_scale + blk * 16 + 4 * q4);
      float a[4];
      if (HAS_ZP) {
        const int4 r4 = *reinterpret_cast<const int4*>(t_rowsum + blk * 16 + 4 * q4);
        const int rs[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = (float)((int)acc[4 * q4 + i] - rc.zpa * rs[i]);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = (float)(int)acc[4 * q4 + i];
      }
      // acc * scale (+ bias): scalar, two roundings.  (Packed, ptxas contracts mul.rn.f32x2 +
      // add.rn.f32x2 into one fused multiply-add -- one rounding, codes off by one at ties.)
      const float sc[4] = {s4.x, s4.y, s4.z, s4.w};
      float v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = __fmul_rn(a[i], sc[i]);
      if (HAS_BIAS) {
        const float4 b4 = *reinterpret_cast<const float4*>(t_bias + blk * 16 + 4 * q4);
        v[0] = __fadd_rn(v[0], b4.x), v[1] = __fadd_rn(v[1], b4.y);
        v[2] = __fadd_rn(v[2], b4.z), v[3] = __fadd_rn(v[3], b4.w);
      }
      const F2 v01 = f2_pack(v[0], v[1]), v23 = f2_pack(v[2], v[3]);
      // correctly rounded quotient by the output scale, rounded to the nearest integer (ties to
      // even) in the mantissa of q + 1.5 * 2^23; the ReLU is the lower clamp of the code
      // (rint(max(y, 0) / s) == max(rint(y / s), 0) for s > 0)
      F2 e01, e23;
      const F2 q01 = f2_div_short(v01, y2, ns2, e01), q23 = f2_div_short(v23, y2, ns2, e23);
      float e[4], t[4];
      f2_unpack(e01, e[0], e[1]), f2_unpack(e23, e[2], e[3]);
      big = fmaxf(fmaxf(big, fmaxf(fabsf(e[0]), fabsf(e[1]))), fmaxf(fabsf(e[2]), fabsf(e[3])));
      f2_unpack(f2_add(q01, magic2), t[0], t[1]), f2_unpack(f2_add(q23, magic2), t[2], t[3]);
      int c[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) c[i] = __float_as_int(t[i]) + rc.zofs;
      if (rc.need_clamp) {
#pragma unroll
        for (int i = 0; i < 4; ++i) c[i] = min(max(c[i], rc.clo), rc.chi);
      }
      w[q4] = rc.out_signed ? pack4i_s8(c) : pack4i_u8(c);
    }
    if (!(big < 0x1p22f)) {
      // a quotient outside the short division's domain (never for sane scales): the whole block
      // again through the full-range sequence
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        float y[4], c[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int col = blk * 16 + 4 * q4 + i;
          const int v = HAS_ZP ? (int)acc[4 * q4 + i] - rc.zpa * t_rowsum[col] : (int)acc[4 * q4 + i];
          y[i] = __fmul_rn((float)v, t_scale[col]);
          if (HAS_BIAS) y[i] = __fadd_rn(y[i], t_bias[col]);
          if (RELU) y[i] = fmaxf(y[i], 0.0f);
        }
        code4_f32(y, rc.so, rc.zo, rc.fqmin, rc.fqmax, c);
        w[q4] = pack4_low_bytes(c);
      }
    }
    if (row_ok) *reinterpret_cast<uint4*>(dst + blk * 16) = make_uint4(w[0], w[1], w[2], w[3]);
  };
  if constexpr (PARTS <= 2) {
    // 8 epilogue warps (168 registers)
    static_assert(NB % 2 == 0, "blocks are taken in pairs");
    // two blocks per iteration, finished in one basic block: eight independent chains of four
    // outputs for the scheduler to interleave (two epilogue warps per scheduler hide little)
    uint32_t acc_a[16], acc_b[16];
#pragma unroll 1
    for (int blk = 0; blk < NB; blk += 2) {
      tc_ld16(taddr + c0 + blk * 16, acc_a);
      tc_ld16(taddr + c0 + (blk + 1) * 16, acc_b);
      tc_wait_ld_dep16(acc_a);
      tc_wait_ld_dep16(acc_b);
      finish_block(acc_a, blk);
      finish_block(acc_b, blk + 1);
    }
  } else {
    // 16 epilogue warps (96 registers): one register set, read and wait in one statement (a
    // register that a read in flight will write must never be spilled)
#pragma unroll 1
    for (int blk = 0; blk < NB; ++blk) {
      uint32_t acc[16];
      tc_ld16_sync(taddr + c0 + blk * 16, acc);
      finish_block(acc, blk);
    }
  }
}

// The general 8-bit epilogue (ragged last column of tiles, per-row activation scales, several
// destinations), out of line: it is the rare path of the 8-bit kernels, and inlined it would
// set the register budget of their tile loop.
template <int BN, int PARTS>
static __device__ __noinline__ void epilogue_q8_generic(const Epi& ep, const Geometry& g, const RowCtx& rc, uint32_t taddr,
                                                        uint8_t* stg, int lane, int part, int n0, const Partials& ps,
                                                        int quad) {
  epilogue_tile<BN, KIND_Q8, false, PARTS>(ep, g, rc, taddr, stg, lane, part, n0, n0, ps, quad);
}

// Runtime flags -> template arguments (three uniform branches per tile, none per element).
template <int BN, int PARTS, bool... Fs>
__device__ __forceinline__ void q8_dispatch(int mask, const Epi& ep, const RowCtx& rc, uint32_t taddr, uint8_t* stg,
                                            int lane, int part, int n0, bool fill, const Partials& ps, int quad) {
  if constexpr (sizeof...(Fs) == 3) {
    epilogue_tile_q8<BN, PARTS, Fs...>(ep, rc, taddr, stg, lane, part, n0, fill, ps, quad);
  } else if (mask & 1) {
    q8_dispatch<BN, PARTS, Fs..., true>(mask >> 1, ep, rc, taddr, stg, lane, part, n0, fill, ps, quad);
  } else {
    q8_dispatch<BN, PARTS, Fs..., false>(mask >> 1, ep, rc, taddr, stg, lane, part, n0, fill, ps, quad);
  }
}

// ---- work schedule ------------------------------------------------------------------
// Tile mode: worker w takes tiles w, w + W, ... whole (M fastest, so neighbouring workers share
// a B tile in L2).  Stream-K mode handles the tiles that do not fill a whole wave: with T tiles
// and W workers the first T % W tiles form one sequence of k-block units that is dealt out in
// equal contiguous runs (worker w takes units [U*w/W, U*(w+1)/W): the tail of one tile, maybe
// whole tiles, the head of another); the other T - T % W tiles follow tile by tile, so every
// worker ends with the same number of whole tiles and the L2 footprint of the tile-by-tile order
// is kept.
struct Sched {
  int num_workers, num_kb;
  int tile, total_tiles;  // tile-by-tile part: next tile
  long long u, u_end;     // stream-K part: next unit, end of the run (empty when not stream-K)
};
__device__ __forceinline__ long long run_begin(long long units, int worker, int num_workers) {
  return units * worker / num_workers;
}
// tiles handled by the stream-K part
__device__ __forceinline__ int streamk_tiles(const Geometry& g, int total_tiles, int num_workers) {
  return g.streamk ? total_tiles % num_workers : 0;
}
__device__ __forceinline__ Sched make_sched(const Geometry& g, int worker, int raw_worker, int num_workers,
                                            int total_tiles) {
  Sched s;
  s.num_workers = num_workers, s.num_kb = g.num_kb, s.total_tiles = total_tiles;
  const int sk_tiles = streamk_tiles(g, total_tiles, num_workers);
  const long long units = (long long)sk_tiles * g.num_kb;
  s.u = run_begin(units, worker, num_workers), s.u_end = run_begin(units, worker + 1, num_workers);
  s.tile = sk_tiles + raw_worker;
  return s;
}
// Next work item: k-blocks [kb0, kb1) of `tile`.  False when the worker is done.
__device__ __forceinline__ bool sched_next(Sched& s, int& tile, int& kb0, int& kb1) {
  if (s.u < s.u_end) {
    tile = (int)(s.u / s.num_kb);
    kb0 = (int)(s.u - (long long)tile * s.num_kb);
    const long long left = s.u_end - s.u;
    kb1 = left < (long long)(s.num_kb - kb0) ? kb0 + (int)left : s.num_kb;
    s.u += kb1 - kb0;
    return true;
  }
  if (s.tile >= s.total_tiles) return false;
  tile = s.tile, kb0 = 0, kb1 = s.num_kb;
  s.tile += s.num_workers;
  return true;
}

// ---- the kernel ---------------------------------------------------------------------
// FAM selects the epilogue family compiled into the kernel: 0 = float / s32 outputs (plain and
// gated), 1 = 8-bit codes (the requantising epilogues).  One kernel with both spilled the state
// of its tile loop (96 registers with 16 epilogue warps) and reloaded it from L2 inside the
// requantising loop, which is what bounded the small-K layers.
template <int BN, bool PAIR, int EW, int FAM>
__global__ void __launch_bounds__(threads_for(EW), 1)
gemm_s8_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
               const __grid_constant__ Geometry g, const __grid_constant__ Epi ep, const uint32_t idesc) {
  using C = Cfg<BN, PAIR, EW>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~(uintptr_t)1023);
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + C::kStages * C::kABytes;
  uint8_t* tail = smem + C::kStages * C::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail);  // full[S], empty[S], tfull[2], tempty[2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tail + 256);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tail + 260);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * C::kStages;
  const uint32_t bar_tfull = bar_empty + 8 * C::kStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  const long long budget = g.wait_budget;

  // PAIR: CTA `rank` of the 2-CTA cluster owns M sub-tile 2*pair_m + rank and B rows
  // [rank*BN/2, (rank+1)*BN/2) of the tile; the leader (rank 0) issues the MMAs.
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
  const bool leader = rank == 0;
  const int num_workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int raw_worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  // Stream-K numbers the workers against the launch order: the CTA that finishes a cut tile
  // waits for partial sums of workers with higher numbers, i.e. of CTAs that were launched
  // before it, and those wait for nobody.
  const int worker = g.streamk ? num_workers - 1 - raw_worker : raw_worker;
  const int tiles_mw = PAIR ? (g.tiles_m + 1) / 2 : g.tiles_m;  // M tiles per worker
  const int total_tiles = tiles_mw * g.tiles_n;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_tfull + 8 * s, 1);
      mbar_init(bar_tempty + 8 * s, (PAIR ? 2 : 1) * EW);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tm_b) : "memory");
  }
  if (warp == 1) {
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(tmem_slot)),
                   "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(tmem_slot)),
                   "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();  // the peer's barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above touched only kernel arguments, shared memory and TMEM, and may have run
  // while the kernel before this one in the stream was still draining; global memory (operands,
  // scales, workspace, outputs) is touched from here on.
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ===== TMA producer (one per CTA) =====
    Sched sc = make_sched(g, worker, raw_worker, num_workers, total_tiles);
    int stage = 0, tile, kb0, kb1;
    uint32_t phase = 0;
    bool ok = true;
#ifdef LQ_TESTING
    if (g.test_no_loads) ok = false;
#endif
    while (ok && sched_next(sc, tile, kb0, kb1)) {
      const int tm_idx = (tile % tiles_mw) * (PAIR ? 2 : 1) + (int)rank;
      const int n0 = (tile / tiles_mw) * BN + (int)rank * C::kBRows;
      int m0 = tm_idx * BM, img = 0, y0 = 0, x0 = 0;
      if (g.conv) {
        const int per_img = g.tiles_p * g.tiles_q;
        img = tm_idx / per_img;  // >= number of images for the padding sub-tile: zero-filled
        const int rem = tm_idx - img * per_img;
        // input coordinates of the tile's first output pixel at tap (0, 0)
        y0 = (rem / g.tiles_q) * g.tile_h * g.stride_h - g.pad_h;
        x0 = (rem % g.tiles_q) * g.tile_w * g.stride_w - g.pad_w;
      }
      const uint32_t a_bytes = g.conv ? (uint32_t)(BK * g.tile_w * g.tile_h) : (uint32_t)C::kABytes;
      const uint32_t stage_tx = (a_bytes + (uint32_t)C::kBBytes) * (PAIR ? 2u : 1u);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait_warp(bar_empty + 8 * stage, phase ^ 1u, abort_flag, budget)) {
          ok = false;
          break;
        }
        const uint32_t a_dst = smem_u32(smem_a + stage * C::kABytes);
        const uint32_t b_dst = smem_u32(smem_b + stage * C::kBBytes);
        int ax = kb * BK, bx = kb * BK, ay = 0, ax2 = 0;
        if (g.conv) {
          const int tap = kb / g.cblocks;
          const int cb = kb - tap * g.cblocks;
          const int r = tap / g.S, sft = tap - r * g.S;
          ax = cb * BK, bx = tap * g.C + cb * BK;
          ay = y0 + r * g.dil_h, ax2 = x0 + sft * g.dil_w;
        }
        if (!elect_one()) {
        } else if (PAIR) {
          // both CTAs' bytes are counted on the leader's barrier
          const uint32_t full = map_to_cta(bar_full + 8 * stage, 0);
          if (leader) mbar_expect_tx(bar_full + 8 * stage, stage_tx);
          if (g.conv) tma_load_4d_pair(a_dst, &tm_a, ax, ax2, ay, img, full);
          else tma_load_2d_pair(a_dst, &tm_a, ax, m0, full);
          tma_load_2d_pair(b_dst, &tm_b, bx, n0, full);
        } else {
          const uint32_t full = bar_full + 8 * stage;
          mbar_expect_tx(full, stage_tx);
          if (g.conv) tma_load_4d(a_dst, &tm_a, ax, ax2, ay, img, full);
          else tma_load_2d(a_dst, &tm_a, ax, m0, full);
          tma_load_2d(b_dst, &tm_b, bx, n0, full);
        }
        if (++stage == C::kStages) stage = 0, phase ^= 1u;
      }
    }
  } else if (warp == 1) {
    // ===== MMA issuer (leader CTA only when paired) =====
    if (leader) {
      Sched sc = make_sched(g, worker, raw_worker, num_workers, total_tiles);
      int stage = 0, acc = 0, tile, kb0, kb1;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      while (ok && sched_next(sc, tile, kb0, kb1)) {
        if (!mbar_wait_warp(bar_tempty + 8 * acc, acc_phase ^ 1u, abort_flag, budget)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait_warp(bar_full + 8 * stage, phase, abort_flag, budget)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t adesc = make_smem_desc(smem_u32(smem_a + stage * C::kABytes));
          const uint64_t bdesc = make_smem_desc(smem_u32(smem_b + stage * C::kBBytes));
          const bool issuer = elect_one();
          const uint32_t first = kb == kb0 ? 0u : 1u;  // the first MMA of a work item overwrites
#pragma unroll
          for (int k = 0; k < BK / UMMA_K && issuer; ++k) {
            // advancing K inside the swizzle atom = advancing the start address
            const uint64_t koff = (uint64_t)(k * (UMMA_K >> 4));
            if (PAIR) tc_mma_i8_pair(d_tmem, adesc + koff, bdesc + koff, idesc, k != 0 ? 1u : first);
            else tc_mma_i8(d_tmem, adesc + koff, bdesc + koff, idesc, k != 0 ? 1u : first);
          }
          // frees the stage (in both CTAs when paired) once the MMAs have read it
          if (!issuer) {
          } else if (PAIR) tc_commit_pair(bar_empty + 8 * stage);
          else tc_commit(bar_empty + 8 * stage);
          __syncwarp();
          if (++stage == C::kStages) stage = 0, phase ^= 1u;
        }
        if (!ok) break;
        // accumulator complete
        if (elect_one()) {
          if (PAIR) tc_commit_pair(bar_tfull + 8 * acc);
          else tc_commit(bar_tfull + 8 * acc);
        }
        __syncwarp();
        if (++acc == 2) acc = 0, acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else {
    // ===== epilogue: warps 2..EW+1; TMEM lane quadrant = warp % 4, column part = (warp - 2) / 4 =====
    constexpr int PARTS = EW / 4;
    const int quad = warp & 3;
    const int row = quad * 32 + lane;  // tile-local row == TMEM lane
    uint8_t* stg = tail + 512 + (warp - 2) * 4096;  // this warp's output staging
    const int part = (warp - 2) >> 2;
    const bool gated = ep.act == LQ_ACT_SILU_GATE;
    // the lean requantising epilogue: one destination, vector stores, aligned parameter arrays
    const bool q8_lean = ep.n_dst == 1 && !ep.multicast && ep.vec_ok && ep.par_vec &&
                         ep.a_scale_mode != LQ_PER_ROW && (ep.out_dtype == LQ_S8 || ep.out_dtype == LQ_U8);
    // what does not change from tile to tile is read once
    RowCtx rc_launch;
    rc_launch.sa = (ep.a_scale && ep.a_scale_mode != LQ_PER_ROW) ? __ldcg(ep.a_scale) : 1.0f;
    rc_launch.zpa = ep.a_zp ? (int)__ldcg(ep.a_zp) : 0;
    rc_launch.so = make_divisor(ep.out_scale ? __ldcg(ep.out_scale) : 1.0f);
    rc_launch.zo = ep.out_zp ? __ldcg(ep.out_zp) : 0.0f;
    rc_launch.fqmin = (float)ep.qmin, rc_launch.fqmax = (float)ep.qmax;
    rc_launch.row_mask = 0u, rc_launch.row0 = 0;
    {
      const bool relu = ep.act == LQ_ACT_RELU;
      const int zo_i = (int)rc_launch.zo;
      rc_launch.zofs = zo_i - 0x4B400000;
      rc_launch.clo = relu && zo_i > ep.qmin ? zo_i : ep.qmin;
      rc_launch.chi = ep.qmax;
      rc_launch.out_signed = ep.out_dtype == LQ_S8;
      const int store_lo = rc_launch.out_signed ? -128 : 0, store_hi = rc_launch.out_signed ? 127 : 255;
      rc_launch.need_clamp = !(rc_launch.clo <= store_lo && rc_launch.chi >= store_hi);
    }
    // a positive output scale in the short division's range and an integral zero point
    const bool q8_lean_grid = rc_launch.so.fast && rc_launch.so.s > 0.0f && fabsf(rc_launch.zo) <= 512.0f &&
                              rc_launch.zo == rintf(rc_launch.zo);
    rc_launch.grid_ok = q8_lean_grid;
    const int q8_mask = (ep.bias != nullptr ? 1 : 0) | (ep.act == LQ_ACT_RELU ? 2 : 0) |
                        ((ep.b_rowsum != nullptr && rc_launch.zpa != 0) ? 4 : 0);
    int q8_filled_tn = -1;  // column of tiles whose parameters this warp's table holds
    // stream-K scratch of this CTA: its slot for a partial tile and its two flag words
    // (arrivals of the writing warps, departures of the reading warps)
    uint8_t* const sk_slots = ep.ws ? ep.ws + kWsHeaderBytes : nullptr;
    unsigned int* const sk_flags = ep.ws ? reinterpret_cast<unsigned int*>(ep.ws + kWsFlagsOffset) : nullptr;
    const long long units = (long long)streamk_tiles(g, total_tiles, num_workers) * g.num_kb;
    Sched sc = make_sched(g, worker, raw_worker, num_workers, total_tiles);
    int acc = 0, tile, kb0, kb1;
    uint32_t acc_phase = 0;
    const uint32_t tempty_target = PAIR ? map_to_cta(bar_tempty, 0) : bar_tempty;
    while (sched_next(sc, tile, kb0, kb1)) {
      const int tm_idx = (tile % tiles_mw) * (PAIR ? 2 : 1) + (int)rank;
      const int tn_idx = tile / tiles_mw;
      // output row of this thread; valid rows of a tile are a prefix and map to
      // consecutive output rows
      bool row_ok;
      int m_global;
      if (g.conv) {
        const int per_img = g.tiles_p * g.tiles_q;
        const int img = tm_idx / per_img;
        const int rem = tm_idx - img * per_img;
        const int ph = row / g.tile_w, qw = row - ph * g.tile_w;
        const int p = (rem / g.tiles_q) * g.tile_h + ph;
        const int q = (rem % g.tiles_q) * g.tile_w + qw;
        row_ok = tm_idx < g.tiles_m && ph < g.tile_h && p < g.P && q < g.Q;
        m_global = (img * g.P + p) * g.Q + q;
      } else {
        m_global = tm_idx * BM + row;
        row_ok = m_global < g.M;
      }
      RowCtx rc = rc_launch;
      if (ep.a_scale && ep.a_scale_mode == LQ_PER_ROW) rc.sa = row_ok ? __ldcg(ep.a_scale + m_global) : 1.0f;
      rc.row_mask = __ballot_sync(0xffffffffu, row_ok);
      rc.row0 = (long long)__shfl_sync(0xffffffffu, m_global, 0);

      if (!mbar_wait_warp<200>(bar_tfull + 8 * acc, acc_phase, abort_flag, budget)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
      const int n0 = tn_idx * BN;
      Partials ps;
      ps.slots = nullptr, ps.n = 0, ps.cta0 = 0, ps.cta_step = 0;
      if (kb0 > 0) {
        // a tile whose first k-blocks belong to another CTA: leave the raw sums in this CTA's slot
        dump_partial<BN, PARTS>(taddr, sk_slots + (size_t)blockIdx.x * kWsSlotBytes, quad, part, lane);
        __threadfence();
        __syncwarp();
        if (lane == 0) atomicAdd(sk_flags + 2 * blockIdx.x, 1u);
      } else {
        if (kb1 < g.num_kb) {
          // this CTA finishes a cut tile: the workers after it hold the rest of its k-blocks
          const long long tile_end = (long long)(tile + 1) * g.num_kb;
          int n = 0;
          while (worker + 1 + n < num_workers && run_begin(units, worker + 1 + n, num_workers) < tile_end) ++n;
          ps.slots = sk_slots, ps.n = n;
          ps.cta_step = PAIR ? -2 : -1;
          ps.cta0 = (num_workers - 1 - (worker + 1)) * (PAIR ? 2 : 1) + (int)rank;
          int ready = 1;
          if (lane == 0)
            for (int i = 0; i < n && ready; ++i)
              ready = flag_wait_eq(sk_flags + 2 * (ps.cta0 + i * ps.cta_step), (unsigned)EW, abort_flag, budget) ? 1 : 0;
          if (!__shfl_sync(0xffffffffu, ready, 0)) break;
        }
        if constexpr (FAM == 0) {
          if (gated) {
            const int on0 = tn_idx * (BN / 2);
            if (ep.out_dtype == LQ_F32) epilogue_tile<BN, KIND_F32, true, PARTS>(ep, g, rc, taddr, stg, lane, part, n0, on0, ps, quad);
            else epilogue_tile<BN, KIND_BF16, true, PARTS>(ep, g, rc, taddr, stg, lane, part, n0, on0, ps, quad);
          } else if (ep.out_dtype == LQ_BF16) {
            epilogue_tile<BN, KIND_BF16, false, PARTS>(ep, g, rc, taddr, stg, lane, part, n0, n0, ps, quad);
          } else if (ep.out_dtype == LQ_F32) {
            epilogue_tile<BN, KIND_F32, false, PARTS>(ep, g, rc, taddr, stg, lane, part, n0, n0, ps, quad);
          } else {
            epilogue_tile<BN, KIND_S32, false, PARTS>(ep, g, rc, taddr, stg, lane, part, n0, n0, ps, quad);
          }
        } else if constexpr (FAM == 2) {
          // every tile is eligible for the requantising loop (checked by the launcher); an output
          // grid outside the short division's domain sends every block through its full-range
          // sequence (rc.grid_ok)
          q8_dispatch<BN, PARTS>(q8_mask, ep, rc, taddr, stg, lane, part, n0, q8_filled_tn != tn_idx, ps, quad);
          q8_filled_tn = tn_idx;
        } else {
          if (q8_lean && q8_lean_grid && n0 + BN <= g.N) {
            q8_dispatch<BN, PARTS>(q8_mask, ep, rc, taddr, stg, lane, part, n0, q8_filled_tn != tn_idx, ps, quad);
            q8_filled_tn = tn_idx;
          } else {
            epilogue_q8_generic<BN, PARTS>(ep, g, rc, taddr, stg, lane, part, n0, ps, quad);
            q8_filled_tn = -1;  // the generic path stages through the table's memory
          }
        }
        if (ps.n) {
          // the last reading warp re-arms the contributors' flags for the next launch
          __syncwarp();
          if (lane == 0) {
            for (int i = 0; i < ps.n; ++i) {
              unsigned int* f = sk_flags + 2 * (ps.cta0 + i * ps.cta_step);
              if (atomicAdd(f + 1, 1u) == (unsigned)(EW - 1)) {
                f[1] = 0u;
                __threadfence();
                f[0] = 0u;
              }
            }
          }
        }
      }
      // hand the accumulator stage back to the MMA issuer
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) mbar_arrive_cluster(tempty_target + 8 * acc);
        else mbar_arrive(bar_tempty + 8 * acc);
      }
      if (++acc == 2) acc = 0, acc_phase ^= 1u;
    }
  }

  // ===== teardown (every role falls through to here) =====
  tc_fence_before();
  __syncthreads();
  // read after the barrier: a role that finished early (the producer once it has issued its
  // last load) must still see an abort that another role raised later
  const bool aborted = *abort_flag != 0;
  if (aborted) {
    // give copies / MMAs still in flight time to land before the CTA's shared
    // memory and TMEM are released
    for (int i = 0; i < 50; ++i) __nanosleep(20000);
    if (threadIdx.x == 0 && ep.status) atomicExch(ep.status, (int)LQ_ERR_TIMEOUT);
  }
  if (PAIR) cluster_sync_all();  // the peer may still signal this CTA's barriers / read its tiles
  if (ep.n_flags > 0 && threadIdx.x == 0 && !aborted) {
    // Exchange step: every CTA's stores into the peers' buffers are complete (barrier above) and
    // made visible system-wide before its ticket; the CTA that draws the last ticket publishes
    // this rank's new step count to its flag word on every peer.
    __threadfence_system();
    unsigned int* ticket = reinterpret_cast<unsigned int*>(ep.ws);
    if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
      *ticket = 0u;
      __threadfence_system();
      const int v = *ep.signal_counter + 1;
      *ep.signal_counter = v;
      for (int i = 0; i < ep.n_flags; ++i)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(ep.peer_flags[i]), "r"(v) : "memory");
    }
  }
  if (warp == 1) {
    tc_fence_after();
    if (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"(kTmemCols)
                   : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"(kTmemCols)
                   : "memory");
  }
}

// ---- host side -----------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

// A tensor map is a pure function of (address, extents, strides, box, traversal strides), so
// encoded maps are kept in a small table: a layer that runs the same buffers every step pays the
// driver call once.
struct MapKey {
  const void* base;
  uint64_t dims[4], strides[3];
  uint32_t box[4], estr[4], rank;
  bool operator==(const MapKey& o) const { return memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapCache {
  static constexpr int kEntries = 256;
  std::mutex mu;
  MapKey keys[kEntries];
  CUtensorMap maps[kEntries];
  bool used[kEntries] = {};
  static size_t hash(const MapKey& k) {
    const unsigned char* p = reinterpret_cast<const unsigned char*>(&k);
    size_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(MapKey); ++i) h = (h ^ p[i]) * 1099511628211ull;
    return h;
  }
};

int encode_map(CUtensorMap* tm, const MapKey& key) {
  static MapCache cache;
  const size_t slot = MapCache::hash(key) % MapCache::kEntries;
  {
    std::lock_guard<std::mutex> lock(cache.mu);
    if (cache.used[slot] && cache.keys[slot] == key) {
      *tm = cache.maps[slot];
      return LQ_OK;
    }
  }
  EncodeTiledFn enc = get_encode();
  if (!enc) return fail(LQ_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[4], strides[3];
  cuuint32_t box[4], estr[4];
  for (int i = 0; i < 4; ++i) dims[i] = key.dims[i], box[i] = key.box[i], estr[i] = key.estr[i];
  for (int i = 0; i < 3; ++i) strides[i] = key.strides[i];
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, key.rank, const_cast<void*>(key.base), dims, strides, box,
                   estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(LQ_ERR_CUDA, "cuTensorMapEncodeTiled (" + std::to_string(key.rank) + "-D) failed: " + std::to_string((int)r));
  std::lock_guard<std::mutex> lock(cache.mu);
  cache.keys[slot] = key, cache.maps[slot] = *tm, cache.used[slot] = true;
  return LQ_OK;
}

int encode_2d(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t k, uint64_t row_stride,
              uint32_t box_rows) {
  MapKey key;
  memset(&key, 0, sizeof(key));
  key.base = base, key.rank = 2;
  key.dims[0] = k, key.dims[1] = rows;
  key.strides[0] = row_stride;
  key.box[0] = (uint32_t)BK, key.box[1] = box_rows;
  key.estr[0] = key.estr[1] = 1;
  return encode_map(tm, key);
}

// NHWC activations of one channel group: extents (c, w, h, n) with pixel stride `c_stride`
// bytes; the box covers tile_w x tile_h output pixels, i.e. (tile - 1) * stride + 1 input
// positions walked with the convolution stride as the traversal stride.
int encode_nhwc(CUtensorMap* tm, const void* base, uint64_t n, uint64_t h, uint64_t w, uint64_t c,
                uint64_t c_stride, uint32_t tile_w, uint32_t tile_h, uint32_t stride_w, uint32_t stride_h) {
  MapKey key;
  memset(&key, 0, sizeof(key));
  key.base = base, key.rank = 4;
  key.dims[0] = c, key.dims[1] = w, key.dims[2] = h, key.dims[3] = n;
  key.strides[0] = c_stride, key.strides[1] = c_stride * w, key.strides[2] = c_stride * w * h;
  key.box[0] = (uint32_t)BK, key.box[1] = (tile_w - 1) * stride_w + 1, key.box[2] = (tile_h - 1) * stride_h + 1;
  key.box[3] = 1;
  key.estr[0] = 1, key.estr[1] = stride_w, key.estr[2] = stride_h, key.estr[3] = 1;
  return encode_map(tm, key);
}

int check_epilogue(const lq_epilogue_t* e, size_t N, const char* who, bool allow_gate) {
  const std::string w(who);
  if (!e) return fail(LQ_ERR_DEVICE, w + ": epilogue descriptor is null");
  switch (e->out_dtype) {
    case LQ_S32: case LQ_F32: case LQ_BF16: case LQ_S8: case LQ_U8: break;
    default: return fail(LQ_ERR_DTYPE, w + ": out_dtype must be s32|f32|bf16|s8|u8");
  }
  if (e->act < LQ_ACT_NONE || e->act > LQ_ACT_SILU_GATE) return fail(LQ_ERR_UNSUPPORTED, w + ": unknown activation");
  if (e->act == LQ_ACT_SILU_GATE) {
    if (!allow_gate) return fail(LQ_ERR_UNSUPPORTED, w + ": gated epilogue is GEMM-only");
    if (e->out_dtype != LQ_F32 && e->out_dtype != LQ_BF16) return fail(LQ_ERR_DTYPE, w + ": gated epilogue writes f32|bf16");
    if (N % 256 != 0) return fail(LQ_ERR_SHAPE, w + ": gated epilogue needs N % 256 == 0 ([gate;up] in blocks of 128 rows)");
  }
  if (e->out_dtype != LQ_S32) {
    if (!e->a_scale || !e->b_scale) return fail(LQ_ERR_DEVICE, w + ": a_scale and b_scale are required for scaled outputs");
    if (e->a_scale_mode != LQ_PER_TENSOR && e->a_scale_mode != LQ_PER_ROW) return fail(LQ_ERR_SHAPE, w + ": a_scale_mode");
  }
  if (e->a_zp && !e->b_rowsum) return fail(LQ_ERR_DEVICE, w + ": a_zp needs b_rowsum");
  if (e->out_dtype == LQ_S8 || e->out_dtype == LQ_U8) {
    if (!e->out_scale || !e->out_zp) return fail(LQ_ERR_DEVICE, w + ": requantising outputs need out_scale/out_zp");
    const int lo = e->out_dtype == LQ_S8 ? -128 : 0, hi = e->out_dtype == LQ_S8 ? 127 : 255;
    if (e->qmin < lo || e->qmax > hi || e->qmin >= e->qmax) return fail(LQ_ERR_SHAPE, w + ": qmin/qmax outside the output dtype");
  }
  return LQ_OK;
}

size_t dtype_size(int dt) {
  switch (dt) {
    case LQ_S32: case LQ_F32: return 4;
    case LQ_BF16: case LQ_S16: return 2;
    default: return 1;
  }
}

void fill_epi(Epi* d, const lq_epilogue_t* e, void* out, size_t ldo, size_t n_out, int32_t* status) {
  memset(d, 0, sizeof(Epi));
  d->out_dtype = e->out_dtype, d->act = e->act, d->a_scale_mode = e->a_scale_mode;
  d->qmin = e->qmin, d->qmax = e->qmax;
  d->a_scale = e->a_scale, d->a_zp = e->a_zp, d->b_rowsum = e->b_rowsum, d->b_scale = e->b_scale;
  d->bias = e->bias, d->out_scale = e->out_scale, d->out_zp = e->out_zp;
  d->out = out, d->ldo = (long long)ldo, d->n_out = (int)n_out, d->status = status;
  d->n_dst = 1, d->col0 = 0, d->multicast = 0;
  const size_t esz = dtype_size(e->out_dtype);
  d->vec_ok = aligned16(out) && ((ldo * esz) % 16 == 0);
  d->par_vec = aligned16(e->b_scale) && aligned16(e->bias) && aligned16(e->b_rowsum);
}

// Environment knobs (read once): LQ_GEMM_SHAPE=pair|single256|single128 and
// LQ_GEMM_EPI_WARPS=8|16 force a tile shape / epilogue width, LQ_GEMM_STREAMK=0|1 the
// schedule (the tests cover every variant this way; all of them compute the same numbers),
// LQ_GEMM_VERBOSE prints each launch's geometry.
struct Knobs {
  int shape = -1, epi_warps = 0, streamk = -1, bcast_epi_warps = 0, q8_lean_only = 1, q8_epi_warps = 8;
  // policy thresholds: stream-K when the last wave fills less than this percentage of the
  // workers and a tile has at least this many k-blocks.  Measured on the Llama-2-70B shard
  // shapes: +14 % at 4096 x 4096 x 28672 (34 of 74 clusters in the last wave, 224 k-blocks),
  // +3-4 % with 64-86 k-blocks and a last wave under half full; a loss where the last wave is
  // mostly full or a run would be a few k-blocks (the partial-tile round trip and the extra
  // exposed epilogue then cost more than the evened-out wave saves).
  int streamk_max_fill = 50, streamk_min_kb = 64;
  bool verbose = false;
  void read() {
    shape = -1, epi_warps = 0, streamk = -1, bcast_epi_warps = 0;
    if (const char* f = getenv("LQ_GEMM_BCAST_EPI_WARPS")) bcast_epi_warps = atoi(f);
    q8_lean_only = 1, q8_epi_warps = 8;
    if (const char* f = getenv("LQ_GEMM_Q8_LEAN_ONLY")) q8_lean_only = atoi(f);
    if (const char* f = getenv("LQ_GEMM_Q8_EPI_WARPS")) q8_epi_warps = atoi(f) == 16 ? 16 : 8;
    if (const char* f = getenv("LQ_GEMM_STREAMK_MAX_FILL")) streamk_max_fill = atoi(f);
    if (const char* f = getenv("LQ_GEMM_STREAMK_MIN_KB")) streamk_min_kb = atoi(f);
    if (const char* f = getenv("LQ_GEMM_SHAPE")) {
      if (!strcmp(f, "pair")) shape = 0;
      else if (!strcmp(f, "single256")) shape = 1;
      else if (!strcmp(f, "single128")) shape = 2;
    }
    if (const char* f = getenv("LQ_GEMM_EPI_WARPS")) epi_warps = atoi(f);
    if (const char* f = getenv("LQ_GEMM_STREAMK")) streamk = atoi(f) != 0;
    verbose = getenv("LQ_GEMM_VERBOSE") != nullptr;
  }
};
Knobs& knobs_storage() {
  static Knobs k = [] {
    Knobs v;
    v.read();
    return v;
  }();
  return k;
}
const Knobs& knobs() { return knobs_storage(); }

// CTA pairs that can be resident at once, per device.
template <int BN, bool PAIR, int EW, int FAM>
struct LaunchState {
  PerDeviceOnce once;
  int max_clusters[kMaxDevices] = {};
};

template <int BN, bool PAIR, int EW, int FAM>
int launch_fam(const CUtensorMap& ta, const CUtensorMap& tb, const Geometry& g_in, const Epi& ep,
               uint32_t idesc, cudaStream_t st) {
  static LaunchState<BN, PAIR, EW, FAM> state;
  auto kernel = gemm_s8_kernel<BN, PAIR, EW, FAM>;
  constexpr int smem = Cfg<BN, PAIR, EW>::kSmemBytes;
  constexpr int kGemmThreads = threads_for(EW);
  const int dev = current_device();
  const cudaError_t attr_err = state.once.run([&]() -> cudaError_t {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (PAIR && e == cudaSuccess) {
      cudaLaunchConfig_t probe = {};
      probe.gridDim = dim3(2 * sm_count(), 1, 1);
      probe.blockDim = dim3(kGemmThreads, 1, 1);
      probe.dynamicSmemBytes = smem;
      cudaLaunchAttribute at[1];
      at[0].id = cudaLaunchAttributeClusterDimension;
      at[0].val.clusterDim.x = 2, at[0].val.clusterDim.y = 1, at[0].val.clusterDim.z = 1;
      probe.attrs = at, probe.numAttrs = 1;
      int mc = 0;
      if (cudaOccupancyMaxActiveClusters(&mc, kernel, &probe) != cudaSuccess || mc <= 0) {
        cudaGetLastError();
        mc = sm_count() / 2;
      }
      state.max_clusters[dev] = mc;
    }
    return e;
  });
  if (attr_err != cudaSuccess) return check_cuda(attr_err, "cudaFuncSetAttribute(max dynamic smem)");
  const int tiles_mw = PAIR ? (g_in.tiles_m + 1) / 2 : g_in.tiles_m;
  const int total_tiles = tiles_mw * g_in.tiles_n;
  // workers that get something to do: one per tile, or (stream-K, fewer tiles than workers) one
  // per run of k-blocks
  Geometry g = g_in;
  const int workers_max = PAIR ? state.max_clusters[dev] : sm_count();
  int total = total_tiles;
  if (g.streamk) {
    const int min_run = knobs().streamk == 1 ? 2 : 8;
    if (total_tiles < workers_max) {
      const long long runs = (long long)total_tiles * g.num_kb / min_run;
      total = runs < 1 ? 1 : (runs > workers_max ? workers_max : (int)runs);
      if (total <= total_tiles) g.streamk = 0, total = total_tiles;  // nothing to gain from cutting tiles
    } else if ((long long)(total_tiles % workers_max) * g.num_kb < (long long)min_run * workers_max) {
      g.streamk = 0;  // the partial wave is too short to cut into one run per worker
    }
  }
  if (!PAIR) {
    const int grid = total < sm_count() ? total : sm_count();
    if (knobs().verbose)
      fprintf(stderr, "[lq] launch BN=%d EW=%d: %d tiles x %d k-blocks on %d CTAs%s\n", BN, EW, total_tiles, g.num_kb, grid,
              g.streamk ? " (stream-K)" : "");
    return check_cuda(launch_pdl(kernel, dim3(grid), dim3(kGemmThreads), smem, st, ta, tb, g, ep, idesc),
                      "gemm_s8_kernel launch");
  }
  const int max_clusters = state.max_clusters[dev];
  const int clusters = total < max_clusters ? total : max_clusters;
  if (knobs().verbose)
    fprintf(stderr, "[lq] paired launch EW=%d: %d tiles x %d k-blocks on %d clusters (max active %d)%s\n", EW, total_tiles,
            g.num_kb, clusters, max_clusters, g.streamk ? " (stream-K)" : "");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[2];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2, at[0].val.clusterDim.y = 1, at[0].val.clusterDim.z = 1;
  at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at, cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return check_cuda(cudaLaunchKernelEx(&cfg, kernel, ta, tb, g, ep, idesc), "gemm_s8_kernel (paired) launch");
}

template <int BN, bool PAIR, int EW>
int launch(const CUtensorMap& ta, const CUtensorMap& tb, const Geometry& g, const Epi& ep, uint32_t idesc,
           cudaStream_t st) {
  if (ep.out_dtype == LQ_S8 || ep.out_dtype == LQ_U8) {
    // every tile eligible for the requantising loop: the kernel that holds nothing else
    const bool lean_only = ep.n_dst == 1 && !ep.multicast && ep.vec_ok && ep.par_vec && ep.a_scale_mode != LQ_PER_ROW &&
                           g.N % BN == 0 && knobs().q8_lean_only;
    if (lean_only) return launch_fam<BN, PAIR, EW, 2>(ta, tb, g, ep, idesc, st);
    return launch_fam<BN, PAIR, EW, 1>(ta, tb, g, ep, idesc, st);
  }
  return launch_fam<BN, PAIR, EW, 0>(ta, tb, g, ep, idesc, st);
}

// Tile shape and schedule.  CTA pairs (256 x 256 tiles, cta_group::2) when there is enough work
// to fill the clusters; single CTAs (128 x 256, or 128 x 128 for narrow outputs) otherwise.
// Stream-K on top of that shape when the last wave of tiles would leave a good part of the SMs
// idle and a tile is long enough (k-blocks) to be worth cutting: the cut costs one partial-tile
// round trip through L2 and exposes one more epilogue.
enum class Shape { kPair256 = 0, kSingle256 = 1, kSingle128 = 2 };
struct Plan {
  Shape shape;
  bool streamk;
};

Plan pick_plan(size_t m_subtiles, size_t N, bool gated, size_t k_blocks, bool have_ws) {
  const Knobs& kn = knobs();
  const size_t sms = (size_t)sm_count();
  Shape sh;
  const size_t tiles_n256 = (N + 255) / 256;
  const size_t pair_tiles = ((m_subtiles + 1) / 2) * tiles_n256;
  if (kn.shape == 0) sh = Shape::kPair256;
  else if (kn.shape == 1 || (kn.shape == 2 && gated)) sh = Shape::kSingle256;
  else if (kn.shape == 2) sh = Shape::kSingle128;
  else if (N <= 128 && !gated) sh = Shape::kSingle128;
  // With a handful of k-blocks a tile is all epilogue: the pair's saving on operand traffic buys
  // nothing and its cluster handshakes cost (measured 63 vs 68 us at 50176 x 1024 x 256).
  else if (k_blocks <= 4) sh = Shape::kSingle256;
  // a pair tile on a half-empty M pair wastes a CTA; need about one wave of clusters -- three
  // quarters of one when K is long, where the pair's halved B traffic outweighs the idle
  // clusters (measured 2567 vs 2152 TOPS at 4096 x 1024 x 28672: 64 pair tiles on 74 clusters)
  else if (m_subtiles >= 2 && (pair_tiles >= sms / 2 || (k_blocks >= 128 && pair_tiles * 4 >= (sms / 2) * 3)))
    sh = Shape::kPair256;
  else sh = Shape::kSingle256;

  bool sk = false;
  if (have_ws && kn.streamk != 0) {
    const size_t bn = sh == Shape::kSingle128 ? 128 : 256;
    const size_t tiles = (sh == Shape::kPair256 ? (m_subtiles + 1) / 2 : m_subtiles) * ((N + bn - 1) / bn);
    const size_t workers = sh == Shape::kPair256 ? sms / 2 : sms;
    const size_t rem = tiles % workers;
    if (kn.streamk == 1) sk = k_blocks >= 2;  // forced (tests): the launch drops it where nothing can be cut
    else sk = rem != 0 && rem * 100 < workers * (size_t)kn.streamk_max_fill && k_blocks >= (size_t)kn.streamk_min_kb &&
              tiles <= workers * 8;
  }
  return {sh, sk};
}

int dispatch(const Plan& plan, const CUtensorMap& ta, const CUtensorMap& tb, Geometry& g, const Epi& ep,
             int a_signed, cudaStream_t st) {
  // tiles whose mainloop (k-blocks x ~0.28 us) is shorter than their epilogue get 16 epilogue warps
  // (16 against 8 warps: bf16 out, K = 2048 76.6 / 88.6 us at 4096 x 10240, K = 4096 54.5 / 53.3 us
  // at 4096 x 4096; f32 out with the zero-point correction, K = 4096: 63 / 74 us for the whole
  // dynamic Linear)
  bool wide_epi = g.num_kb <= 32;
  // ... except 8-bit outputs: at 96 registers per thread (18 warps) the requantising loop spills
  // and reloads through L2; 8 warps at 168 registers measured 51.7 us against 65.7 us on
  // 50176 x 1024 x 256 and 33.4 against 37.8 us on 50176 x 256 x 2304
  if (ep.out_dtype == LQ_S8 || ep.out_dtype == LQ_U8) wide_epi = knobs().q8_epi_warps == 16;
  // tiles that also travel to peer GPUs: their stores take longer to issue
  if ((ep.n_dst > 1 || ep.multicast) && knobs().bcast_epi_warps) wide_epi = knobs().bcast_epi_warps == 16;
  if (knobs().epi_warps) wide_epi = knobs().epi_warps == 16;
  g.streamk = plan.streamk ? 1 : 0;
  switch (plan.shape) {
    case Shape::kPair256:
      return wide_epi ? launch<256, true, 16>(ta, tb, g, ep, make_idesc(a_signed, 256, 256), st)
                      : launch<256, true, 8>(ta, tb, g, ep, make_idesc(a_signed, 256, 256), st);
    case Shape::kSingle256:
      return wide_epi ? launch<256, false, 16>(ta, tb, g, ep, make_idesc(a_signed, 256), st)
                      : launch<256, false, 8>(ta, tb, g, ep, make_idesc(a_signed, 256), st);
    default:
      return launch<128, false, 8>(ta, tb, g, ep, make_idesc(a_signed, 128), st);
  }
}

// Everything a sharded / workspace-carrying call adds to the plain contraction.
struct Extras {
  void* const* outs = nullptr;  // destinations (null: the single `out`)
  int n_dst = 1;
  bool multicast = false;
  size_t col0 = 0;
  void* ws = nullptr;
  size_t ws_bytes = 0;
  int32_t* const* peer_flags = nullptr;
  int n_flags = 0;
  int32_t* signal_counter = nullptr;
  long long wait_budget = 0;  // 0: default
};

int check_workspace(const std::string& w, const Extras& x) {
  if (!x.ws) return LQ_OK;
  if (!aligned16(x.ws)) return fail(LQ_ERR_ALIGNMENT, w + ": workspace must be 16-byte aligned");
  if (x.ws_bytes < lq_gemm_workspace_bytes())
    return fail(LQ_ERR_WORKSPACE, w + ": workspace smaller than lq_gemm_workspace_bytes()");
  if (2 * sm_count() > 2 * kWsMaxCtas) return fail(LQ_ERR_UNSUPPORTED, w + ": more SMs than the workspace layout covers");
  return LQ_OK;
}

int gemm_impl(const char* who, const void* a, int a_signed, const int8_t* b, size_t M, size_t N, size_t K,
              const lq_epilogue_t* e, void* out, size_t ldo, int32_t* status, void* stream, const Extras& x) {
  const std::string w(who);
  if (M == 0 || N == 0) return LQ_OK;
  if (!a || !b) return fail(LQ_ERR_DEVICE, w + ": null pointer");
  if (x.n_dst < 1 || x.n_dst > 8) return fail(LQ_ERR_SHAPE, w + ": between 1 and 8 destinations");
  if (x.outs) {
    for (int i = 0; i < x.n_dst; ++i)
      if (!x.outs[i]) return fail(LQ_ERR_DEVICE, w + ": null destination pointer");
    out = x.outs[0];
  }
  if (!out) return fail(LQ_ERR_DEVICE, w + ": null pointer");
  if (K == 0) return fail(LQ_ERR_SHAPE, w + ": K must be positive");
  if (K % 16 != 0) return fail(LQ_ERR_ALIGNMENT, w + ": K must be a multiple of 16 (pad with zero codes)");
  if (!aligned16(a) || !aligned16(b)) return fail(LQ_ERR_ALIGNMENT, w + ": a and b must be 16-byte aligned");
  if (M > 0x7fffffffu || N > 0x7fffffffu || K > 0x7fffffffu) return fail(LQ_ERR_SHAPE, w + ": extent too large");
  int rc = check_epilogue(e, N, who, true);
  if (rc) return rc;
  if ((rc = check_workspace(w, x))) return rc;
  if (x.n_flags < 0 || x.n_flags > 8) return fail(LQ_ERR_SHAPE, w + ": at most 8 flag words");
  if (x.n_flags > 0 && (!x.ws || !x.peer_flags || !x.signal_counter))
    return fail(LQ_ERR_DEVICE, w + ": signalling needs a workspace, the flag addresses and the step counter");
  const size_t n_out = e->act == LQ_ACT_SILU_GATE ? N / 2 : N;
  if (ldo < x.col0 + n_out) return fail(LQ_ERR_SHAPE, w + ": ldo smaller than column offset + output width");

  Geometry g = {};
  g.conv = 0, g.M = (int)M, g.N = (int)N, g.K = (int)K;
  g.tiles_m = (int)((M + BM - 1) / BM);
  g.num_kb = (int)((K + BK - 1) / BK);
  g.wait_budget = x.wait_budget > 0 ? x.wait_budget : kWaitBudgetCycles;
  const Plan plan = pick_plan((size_t)g.tiles_m, N, e->act == LQ_ACT_SILU_GATE, (size_t)g.num_kb, x.ws != nullptr);
  const int bn = plan.shape == Shape::kSingle128 ? 128 : 256;
  g.tiles_n = (int)((N + bn - 1) / bn);
  CUtensorMap ta, tb;
  if ((rc = encode_2d(&ta, a, M, K, K, BM))) return rc;
  if ((rc = encode_2d(&tb, b, N, K, K, plan.shape == Shape::kPair256 ? 128u : (uint32_t)bn))) return rc;
  Epi ep;
  fill_epi(&ep, e, out, ldo, n_out, status);
  ep.n_dst = x.n_dst, ep.col0 = (long long)x.col0;
  ep.ws = (uint8_t*)x.ws;
  const size_t esz = dtype_size(e->out_dtype);
  ep.vec_ok = ep.vec_ok && ((x.col0 * esz) % 16 == 0);
  if (x.multicast) {
    // multimem stores are whole 16-byte pieces: the output width must tile them exactly
    if (!ep.vec_ok || (n_out * esz) % 16 != 0)
      return fail(LQ_ERR_ALIGNMENT, w + ": multicast output needs 16-byte aligned rows, offset and width");
    ep.multicast = 1;
  }
  for (int i = 1; i < x.n_dst; ++i) {
    ep.more_outs[i - 1] = x.outs[i];
    ep.vec_ok = ep.vec_ok && aligned16(x.outs[i]);
  }
  ep.n_flags = x.n_flags, ep.signal_counter = x.signal_counter;
  for (int i = 0; i < x.n_flags; ++i) {
    if (!x.peer_flags[i]) return fail(LQ_ERR_DEVICE, w + ": null flag address");
    ep.peer_flags[i] = x.peer_flags[i];
  }
  return dispatch(plan, ta, tb, g, ep, a_signed, (cudaStream_t)stream);
}

// One channel group of the convolution.
int conv_group(const void* x, int x_signed, const int8_t* w, const lq_conv_geometry_t& cg, size_t Cg, size_t Kg,
               size_t P, size_t Q, const lq_epilogue_t* e, void* out, int32_t* status, void* ws, size_t ws_bytes,
               void* stream) {
  Geometry g = {};
  g.conv = 1;
  g.P = (int)P, g.Q = (int)Q, g.C = (int)Cg, g.R = (int)cg.R, g.S = (int)cg.S;
  g.pad_h = (int)cg.pad_h, g.pad_w = (int)cg.pad_w, g.stride_h = (int)cg.stride_h, g.stride_w = (int)cg.stride_w;
  g.dil_h = (int)cg.dil_h, g.dil_w = (int)cg.dil_w;
  g.wait_budget = kWaitBudgetCycles;
  // output pixels per tile: tile_w x tile_h <= 128; a TMA box spans at most 256 input positions
  size_t tw = Q < (size_t)BM ? Q : (size_t)BM;
  const size_t tw_cap = 255 / cg.stride_w + 1;
  if (tw > tw_cap) tw = tw_cap;
  size_t th = (size_t)BM / tw;
  if (th > P) th = P;
  const size_t th_cap = 255 / cg.stride_h + 1;
  if (th > th_cap) th = th_cap;
  g.tile_w = (int)tw, g.tile_h = (int)th;
  g.tiles_q = (int)((Q + tw - 1) / tw);
  g.tiles_p = (int)((P + th - 1) / th);
  g.M = (int)(cg.N * P * Q), g.N = (int)Kg, g.K = (int)(cg.R * cg.S * Cg);
  g.tiles_m = (int)cg.N * g.tiles_p * g.tiles_q;
  g.cblocks = (int)((Cg + BK - 1) / BK);
  g.num_kb = (int)(cg.R * cg.S) * g.cblocks;
  Extras xs;
  xs.ws = ws, xs.ws_bytes = ws_bytes;
  int rc = check_workspace("lq_conv2d_nhwc_s8", xs);
  if (rc) return rc;
  const Plan plan = pick_plan((size_t)g.tiles_m, Kg, false, (size_t)g.num_kb, ws != nullptr);
  const int bn = plan.shape == Shape::kSingle128 ? 128 : 256;
  g.tiles_n = (int)((Kg + bn - 1) / bn);
  CUtensorMap ta, tb;
  if ((rc = encode_nhwc(&ta, x, cg.N, cg.H, cg.W, Cg, cg.C, (uint32_t)tw, (uint32_t)th, (uint32_t)cg.stride_w,
                        (uint32_t)cg.stride_h)))
    return rc;
  const size_t kk = cg.R * cg.S * Cg;
  if ((rc = encode_2d(&tb, w, Kg, kk, kk, plan.shape == Shape::kPair256 ? 128u : (uint32_t)bn))) return rc;
  Epi ep;
  fill_epi(&ep, e, out, cg.K, Kg, status);
  ep.ws = (uint8_t*)ws;
  return dispatch(plan, ta, tb, g, ep, x_signed, (cudaStream_t)stream);
}

}  // namespace
}  // namespace lq

using namespace lq;

namespace lq {
void reload_stream_knobs();
void reload_hist_knobs();
}
extern "C" void lq_reload_env(void) {
  knobs_storage().read();
  lq::reload_pdl_knob();
#ifndef LQ_TESTING  // the test-only library holds the contraction alone
  lq::reload_stream_knobs();
  lq::reload_hist_knobs();
#endif
}

extern "C" size_t lq_gemm_workspace_bytes(void) {
  return (size_t)kWsHeaderBytes + (size_t)kWsMaxCtas * kWsSlotBytes;
}

extern "C" int lq_gemm_s8(const void* a, int a_signed, const int8_t* b, size_t M, size_t N, size_t K,
                          const lq_epilogue_t* e, void* out, size_t ldo, int32_t* status,
                          void* stream) {
  return gemm_impl("lq_gemm_s8", a, a_signed, b, M, N, K, e, out, ldo, status, stream, Extras());
}

extern "C" int lq_gemm_s8_ws(const void* a, int a_signed, const int8_t* b, size_t M, size_t N, size_t K,
                             const lq_epilogue_t* e, void* out, size_t ldo, void* workspace,
                             size_t workspace_bytes, int32_t* status, void* stream) {
  Extras x;
  x.ws = workspace, x.ws_bytes = workspace_bytes;
  return gemm_impl("lq_gemm_s8_ws", a, a_signed, b, M, N, K, e, out, ldo, status, stream, x);
}

extern "C" int lq_gemm_s8_bcast(const void* a, int a_signed, const int8_t* b, size_t M, size_t N,
                                size_t K, const lq_epilogue_t* e, void* const* outs, int n_dst,
                                size_t ldo, size_t col0, int32_t* status, void* stream) {
  if (!outs) return fail(LQ_ERR_DEVICE, "lq_gemm_s8_bcast: null pointer");
  Extras x;
  x.outs = outs, x.n_dst = n_dst, x.col0 = col0;
  return gemm_impl("lq_gemm_s8_bcast", a, a_signed, b, M, N, K, e, nullptr, ldo, status, stream, x);
}

extern "C" int lq_gemm_s8_multicast(const void* a, int a_signed, const int8_t* b, size_t M, size_t N,
                                    size_t K, const lq_epilogue_t* e, void* multicast_out, size_t ldo,
                                    size_t col0, int32_t* status, void* stream) {
  Extras x;
  x.multicast = true, x.col0 = col0;
  return gemm_impl("lq_gemm_s8_multicast", a, a_signed, b, M, N, K, e, multicast_out, ldo, status, stream, x);
}

extern "C" int lq_gemm_s8_sharded(const void* a, int a_signed, const int8_t* b, size_t M, size_t N, size_t K,
                                  const lq_epilogue_t* e, void* const* outs, int n_dst, size_t ldo,
                                  size_t col0, int32_t* const* peer_flags, int n_flags,
                                  int32_t* signal_counter, void* workspace, size_t workspace_bytes,
                                  int32_t* status, void* stream) {
  if (!outs) return fail(LQ_ERR_DEVICE, "lq_gemm_s8_sharded: null pointer");
  Extras x;
  x.col0 = col0, x.ws = workspace, x.ws_bytes = workspace_bytes;
  x.peer_flags = peer_flags, x.n_flags = n_flags, x.signal_counter = signal_counter;
  if (n_dst == -1) {  // outs[0] is an NVSwitch multicast address
    x.multicast = true;
    return gemm_impl("lq_gemm_s8_sharded", a, a_signed, b, M, N, K, e, outs[0], ldo, status, stream, x);
  }
  x.outs = outs, x.n_dst = n_dst;
  return gemm_impl("lq_gemm_s8_sharded", a, a_signed, b, M, N, K, e, nullptr, ldo, status, stream, x);
}

extern "C" int lq_conv2d_nhwc_s8_ex(const void* x, int x_signed, const int8_t* w, const lq_conv_geometry_t* cgp,
                                    const lq_epilogue_t* e, void* out, void* workspace, size_t workspace_bytes,
                                    int32_t* status, void* stream) {
  const char* who = "lq_conv2d_nhwc_s8";
  const std::string sw(who);
  if (!cgp) return fail(LQ_ERR_DEVICE, sw + ": null geometry");
  const lq_conv_geometry_t cg = *cgp;
  if (cg.N == 0 || cg.K == 0) return LQ_OK;
  if (!x || !w || !out) return fail(LQ_ERR_DEVICE, sw + ": null pointer");
  if (cg.H == 0 || cg.W == 0 || cg.C == 0 || cg.R == 0 || cg.S == 0) return fail(LQ_ERR_SHAPE, sw + ": zero extent");
  if (cg.stride_h == 0 || cg.stride_w == 0 || cg.dil_h == 0 || cg.dil_w == 0 || cg.groups == 0)
    return fail(LQ_ERR_SHAPE, sw + ": stride, dilation and groups must be positive");
  if (cg.stride_h > 8 || cg.stride_w > 8) return fail(LQ_ERR_UNSUPPORTED, sw + ": stride above 8 (TMA traversal stride)");
  if (cg.C % cg.groups != 0 || cg.K % cg.groups != 0) return fail(LQ_ERR_SHAPE, sw + ": groups must divide C and K");
  const size_t Cg = cg.C / cg.groups, Kg = cg.K / cg.groups;
  if (Cg % 16 != 0) return fail(LQ_ERR_ALIGNMENT, sw + ": channels per group must be a multiple of 16");
  if (!aligned16(x) || !aligned16(w)) return fail(LQ_ERR_ALIGNMENT, sw + ": x and w must be 16-byte aligned");
  const size_t eff_r = (cg.R - 1) * cg.dil_h + 1, eff_s = (cg.S - 1) * cg.dil_w + 1;
  if (cg.P == 0 || cg.Q == 0) return fail(LQ_ERR_SHAPE, sw + ": empty output");
  // every output pixel's window must start inside the padded input: the last rows / columns
  // may hang over the far edge (implicit zero padding there)
  if ((cg.P - 1) * cg.stride_h >= cg.H + cg.pad_h || (cg.Q - 1) * cg.stride_w >= cg.W + cg.pad_w)
    return fail(LQ_ERR_SHAPE, sw + ": output extent larger than the padded input allows");
  if (cg.pad_h >= eff_r + cg.H || cg.pad_w >= eff_s + cg.W) return fail(LQ_ERR_SHAPE, sw + ": padding larger than the input");
  int rc = check_epilogue(e, cg.K, who, false);
  if (rc) return rc;
  // out-of-image taps read code 0, which stands for the value 0.0 only when the zero point is 0;
  // a geometry without any such tap (no padding, no overhang) takes the usual correction term
  const bool reads_outside = cg.pad_h != 0 || cg.pad_w != 0 || (cg.P - 1) * cg.stride_h + eff_r > cg.H ||
                             (cg.Q - 1) * cg.stride_w + eff_s > cg.W;
  if (e->a_zp && reads_outside)
    return fail(LQ_ERR_UNSUPPORTED, sw + ": with implicit padding the activation zero point must be 0 (padding reads code 0)");
  if (e->a_scale_mode != LQ_PER_TENSOR && e->out_dtype != LQ_S32) return fail(LQ_ERR_UNSUPPORTED, sw + ": per-tensor activation scale only");
  if (cg.N * cg.P * cg.Q > 0x7fffffffu) return fail(LQ_ERR_SHAPE, sw + ": too many output pixels");

  if (cg.R == 1 && cg.S == 1 && cg.pad_h == 0 && cg.pad_w == 0 && cg.stride_h == 1 && cg.stride_w == 1 &&
      cg.groups == 1 && cg.P == cg.H && cg.Q == cg.W) {
    // a 1x1 convolution over NHWC pixels is a plain GEMM with M = N*H*W
    Extras xs;
    xs.ws = workspace, xs.ws_bytes = workspace_bytes;
    return gemm_impl(who, x, x_signed, w, cg.N * cg.H * cg.W, cg.K, cg.C, e, out, cg.K, status, stream, xs);
  }
  const size_t esz = dtype_size(e->out_dtype);
  for (size_t gi = 0; gi < cg.groups; ++gi) {
    // group gi: input channels [gi*Cg, ...), filters / output channels [gi*Kg, ...)
    lq_epilogue_t eg = *e;
    if (eg.b_scale) eg.b_scale += gi * Kg;
    if (eg.bias) eg.bias += gi * Kg;
    if (eg.b_rowsum) eg.b_rowsum += gi * Kg;
    rc = conv_group(static_cast<const uint8_t*>(x) + gi * Cg, x_signed, w + gi * Kg * cg.R * cg.S * Cg, cg, Cg, Kg,
                    cg.P, cg.Q, &eg, static_cast<uint8_t*>(out) + gi * Kg * esz, status, workspace, workspace_bytes,
                    stream);
    if (rc) return rc;
  }
  return LQ_OK;
}

extern "C" int lq_conv2d_nhwc_s8(const void* x, int x_signed, const int8_t* w, size_t N, size_t H,
                                 size_t W, size_t C, size_t K, size_t R, size_t S, size_t stride,
                                 size_t pad, const lq_epilogue_t* e, void* out, int32_t* status,
                                 void* stream) {
  if (stride == 0) return fail(LQ_ERR_SHAPE, "lq_conv2d_nhwc_s8: stride must be positive");
  if (H + 2 * pad < R || W + 2 * pad < S) return fail(LQ_ERR_SHAPE, "lq_conv2d_nhwc_s8: filter larger than padded input");
  lq_conv_geometry_t cg;
  cg.N = N, cg.H = H, cg.W = W, cg.C = C, cg.K = K, cg.R = R, cg.S = S;
  cg.stride_h = cg.stride_w = stride, cg.pad_h = cg.pad_w = pad, cg.dil_h = cg.dil_w = 1, cg.groups = 1;
  cg.P = (H + 2 * pad - R) / stride + 1, cg.Q = (W + 2 * pad - S) / stride + 1;
  return lq_conv2d_nhwc_s8_ex(x, x_signed, w, &cg, e, out, nullptr, 0, status, stream);
}

#ifdef LQ_TESTING
// Test-only build: a GEMM whose producer issues no loads and whose waits give up after
// `budget_cycles`, on single-CTA tiles.  Every role leaves its loop when the first wait runs out,
// the status word receives LQ_ERR_TIMEOUT and the kernel returns normally.
extern "C" int lq_test_gemm_wait_expiry(const void* a, const int8_t* b, size_t M, size_t N, size_t K, void* out,
                                        long long budget_cycles, int32_t* status, void* stream) {
  if (!a || !b || !out || !status) return fail(LQ_ERR_DEVICE, "lq_test_gemm_wait_expiry: null pointer");
  if (K % 16 != 0 || M == 0 || N == 0 || K == 0) return fail(LQ_ERR_SHAPE, "lq_test_gemm_wait_expiry: shape");
  Geometry g = {};
  g.M = (int)M, g.N = (int)N, g.K = (int)K;
  g.tiles_m = (int)((M + BM - 1) / BM), g.tiles_n = (int)((N + 255) / 256), g.num_kb = (int)((K + BK - 1) / BK);
  g.wait_budget = budget_cycles, g.test_no_loads = 1;
  CUtensorMap ta, tb;
  int rc;
  if ((rc = encode_2d(&ta, a, M, K, K, BM))) return rc;
  if ((rc = encode_2d(&tb, b, N, K, K, 256u))) return rc;
  lq_epilogue_t e = {};
  e.out_dtype = LQ_S32;
  Epi ep;
  fill_epi(&ep, &e, out, N, N, status);
  return launch<256, false, 8>(ta, tb, g, ep, make_idesc(1, 256), (cudaStream_t)stream);
}
#endif

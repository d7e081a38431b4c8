// Blackwell (sm_100a) primitives in inline PTX: mbarrier, TMA tile loads,
// tensor-memory allocation, tcgen05 MMA / commit / ld / st and the UMMA
// shared-memory and instruction descriptors.
#pragma once
#include <cuda.h>

#include "fm_common.cuh"

namespace fm {
namespace sm100 {

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait: polls the barrier; every 256 polls checks the CTA-wide abort
// flag and a wall-clock budget.  Returns false when the wait was given up
// (the caller unwinds to the common teardown; nothing traps or spins forever).
struct WaitCtx {
  volatile int* abort_flag;  // shared memory
  uint64_t deadline_ns;
};
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& w) {
  if (mbar_try_wait(bar, parity)) return true;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 0u) {
      if (*w.abort_flag) return false;
      if (global_timer_ns() > w.deadline_ns) {
        *w.abort_flag = 1;
        return false;
      }
    }
  }
}

// The same for waits that last a whole work unit (scheduler and epilogue warps): the wait is
// handed to the barrier hardware with a suspend-time hint, so the waiting warp issues next to
// nothing and takes no issue slots from the warps of its scheduler.
__device__ __forceinline__ bool mbar_try_wait_suspended(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_idle(uint32_t bar, uint32_t parity, const WaitCtx& w) {
  for (;;) {
    if (mbar_try_wait_suspended(bar, parity, 20000u)) return true;
    if (*w.abort_flag) return false;
    if (global_timer_ns() > w.deadline_ns) {
      *w.abort_flag = 1;
      return false;
    }
  }
}

// ---------------------------------------------------------------------------
// TMA: 4-D tiled load global -> shared, completion on an mbarrier (no multicast)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* tmap, uint32_t bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// ---------------------------------------------------------------------------
// tensor memory
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// All tcgen05 operations issued so far by this thread arrive (once) on `bar`
// when they complete.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Eight k-steps (K = 128 elements) of D[tmem] (+)= A[smem] * B[smem], both
// operands K-major with 128-byte swizzle, issued from ONE asm block so that
// nothing but two 64-bit adds separates consecutive MMAs.  A_HI / B_HI: distance
// (in 16-byte units) between the two 64-column sub-tiles of the operand.
template <int A_HI, int B_HI>
__device__ __forceinline__ void umma_ss_x8(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc,
                                           uint32_t acc_first) {
  asm volatile(
      "{\n\t.reg .pred p, pt;\n\t.reg .b64 ta, tb;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "add.s64 ta, %1, 2;  add.s64 tb, %2, 2;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t"
      "add.s64 ta, %1, 4;  add.s64 tb, %2, 4;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t"
      "add.s64 ta, %1, 6;  add.s64 tb, %2, 6;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t"
      "add.s64 ta, %1, %5; add.s64 tb, %2, %6;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t"
      "add.s64 ta, %1, %7; add.s64 tb, %2, %8;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t"
      "add.s64 ta, %1, %9; add.s64 tb, %2, %10;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t"
      "add.s64 ta, %1, %11; add.s64 tb, %2, %12;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t}"
      ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(acc_first),
        "n"(A_HI), "n"(B_HI), "n"(A_HI + 2), "n"(B_HI + 2), "n"(A_HI + 4), "n"(B_HI + 4), "n"(A_HI + 6), "n"(B_HI + 6)
      : "memory");
}

// NK k-steps of D[tmem] (+)= A[tmem] * B[smem]: A advances 8 columns (16 bf16)
// and the MN-major B 16 rows (2048 bytes) per step.
template <int NK>
__device__ __forceinline__ void umma_ts_xn(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc,
                                           uint32_t acc_first) {
  static_assert(NK == 4 || NK == 8, "4 or 8 k-steps");
  asm volatile(
      "{\n\t.reg .pred p, pt;\n\t.reg .b64 tb;\n\t.reg .b32 ta;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "add.u32 ta, %1, 8;  add.s64 tb, %2, 128;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], tb, %3, pt;\n\t"
      "add.u32 ta, %1, 16; add.s64 tb, %2, 256;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], tb, %3, pt;\n\t"
      "add.u32 ta, %1, 24; add.s64 tb, %2, 384;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], tb, %3, pt;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b), "r"(idesc), "r"(acc_first)
      : "memory");
  if constexpr (NK == 8) {
    asm volatile(
        "{\n\t.reg .pred pt;\n\t.reg .b64 tb;\n\t.reg .b32 ta;\n\t"
        "setp.eq.b32 pt, 0, 0;\n\t"
        "add.u32 ta, %1, 32; add.s64 tb, %2, 512;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], tb, %3, pt;\n\t"
        "add.u32 ta, %1, 40; add.s64 tb, %2, 640;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], tb, %3, pt;\n\t"
        "add.u32 ta, %1, 48; add.s64 tb, %2, 768;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], tb, %3, pt;\n\t"
        "add.u32 ta, %1, 56; add.s64 tb, %2, 896;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], tb, %3, pt;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b), "r"(idesc)
        : "memory");
  }
}

// Four k-steps (K = 64 elements, one 64-column sub-tile per operand) of the same.
__device__ __forceinline__ void umma_ss_x4(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc,
                                           uint32_t acc_first) {
  asm volatile(
      "{\n\t.reg .pred p, pt;\n\t.reg .b64 ta, tb;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "add.s64 ta, %1, 2;  add.s64 tb, %2, 2;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t"
      "add.s64 ta, %1, 4;  add.s64 tb, %2, 4;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t"
      "add.s64 ta, %1, 6;  add.s64 tb, %2, 6;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t}"
      ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(acc_first)
      : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread
// (thread t of warp w reads TMEM lane 32*(w%4)+t).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
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
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
// One lane of a converged warp is elected; inside the branch the compiler knows
// a single thread is active, so descriptors and addresses stay in uniform
// registers (a plain `lane == 0` test does not give it that guarantee).
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .b32 rx;\n\t.reg .pred px;\n\t"
      "elect.sync rx|px, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, px;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------------------
// descriptors
// ---------------------------------------------------------------------------
// 32-bit instruction descriptor of kind::f16: fp32 accumulate, A/B both bf16
// (or both f16), M x N tile, operand majorness (0 = K-major, 1 = MN-major).
__host__ __device__ constexpr uint32_t make_idesc(bool is_bf16, int M, int N, int a_mn_major, int b_mn_major) {
  return (1u << 4)                                  // D format: f32
         | ((is_bf16 ? 1u : 0u) << 7)               // A format
         | ((is_bf16 ? 1u : 0u) << 10)              // B format
         | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16)
         | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// 64-bit shared-memory matrix descriptor, 128-byte swizzle, sm_100 version.
//   K-major operand (rows of 64 bf16 = 128 B, 8-row atoms of 1024 B):
//     lbo = 1 (unused), sbo = 1024 B between 8-row groups.
//   MN-major operand (128 B of the MN extent contiguous, K rows of 128 B):
//     lbo = bytes between 64-element MN blocks, sbo = 1024 B between 8-row K groups.
__device__ __forceinline__ uint64_t make_sdesc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}

// Block maxima of one row of a 128-column tile (reference: the fused block-score epilogue,
// flashmask/cute/flash_fwd_sm100.py:4256-4371).  `sr` holds the masked raw scores (masked =
// -inf), `rel0` is the first column of the tile relative to the start of the row's document.
// Column j falls into block (rel0 + j) >> log2(BS).
//   * rel0 a multiple of BS: the tile holds 128/BS whole blocks and nothing else contributes
//     to them; their scaled maxima are stored to `dst` (the thread's row of the output; NULL
//     for a row past the end of the sequence) as they are.
//   * otherwise the tile touches 128/BS + 1 blocks and the outer two straddle its
//     neighbours: the scaled maxima are merged (fmax) into this thread's accumulators in
//     shared memory, `acc[(block & 15) * BS_ACC_STRIDE]`, sixteen consecutive blocks of the
//     row in two groups of eight, which the caller merges into `dst` a group at a time.
// Returns the maximum over the whole row of the tile (the row maximum of the online softmax
// is the maximum of the block maxima, so it is not computed a second time).
constexpr int BS_ACC_STRIDE = 256;
// STRADDLE = false compiles the second case out (no document starts given: rel0 is a multiple of 128).
template <int BS, bool STRADDLE>
__device__ __forceinline__ float block_scores(const uint32_t* sr, int rel0, float scale, float* acc, int n_cols,
                                              float* dst) {
  constexpr int NS = 128 / BS;
  constexpr int LOG2 = BS == 32 ? 5 : (BS == 64 ? 6 : 7);
  constexpr int NC = BS == 32 ? 2 : 4;      // independent fmax chains per block (instruction-level parallelism)
  const int base = rel0 >> LOG2;            // arithmetic shift: floor for columns before the document
  const int t = BS - (rel0 & (BS - 1));     // columns of a block at or past t belong to the next block
  if (!STRADDLE || t == BS) {
    float part[NS][NC];
#pragma unroll
    for (int i = 0; i < NS; ++i)
#pragma unroll
      for (int c = 0; c < NC; ++c) part[i][c] = __int_as_float(0xff800000);
#pragma unroll
    for (int j = 0; j < 128; ++j) part[j / BS][j % NC] = fmaxf(part[j / BS][j % NC], __uint_as_float(sr[j]));
    float all = __int_as_float(0xff800000);
#pragma unroll
    for (int i = 0; i < NS; ++i) {
      float m = part[i][0];
#pragma unroll
      for (int c = 1; c < NC; ++c) m = fmaxf(m, part[i][c]);
      all = fmaxf(all, m);
      const int rb = base + i;
      if (dst && rb >= 0 && rb < n_cols) dst[rb] = m * scale;
    }
    return all;
  }
  float part[NS + 1][NC];
#pragma unroll
  for (int i = 0; i <= NS; ++i)
#pragma unroll
    for (int c = 0; c < NC; ++c) part[i][c] = __int_as_float(0xff800000);
#pragma unroll
  for (int j = 0; j < 128; ++j) {
    const float v = __uint_as_float(sr[j]);
    if ((j % BS) >= t) part[j / BS + 1][j % NC] = fmaxf(part[j / BS + 1][j % NC], v);
    else part[j / BS][j % NC] = fmaxf(part[j / BS][j % NC], v);
  }
  float all = __int_as_float(0xff800000);
#pragma unroll
  for (int i = 0; i <= NS; ++i) {
    float m = part[i][0];
#pragma unroll
    for (int c = 1; c < NC; ++c) m = fmaxf(m, part[i][c]);
    all = fmaxf(all, m);
    const int rb = base + i;
    if (dst && rb >= 0 && rb < n_cols) {
      float* a = acc + (rb & 15) * BS_ACC_STRIDE;
      *a = fmaxf(*a, m * scale);
    }
  }
  return all;
}

// host: driver entry point for tensor-map encoding, resolved once
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled();

// [B, S, H, D] tensor (element strides sb, ss, sh; innermost contiguous) as a
// 4-D map (D, H, S, B) with a 64 x 1 x rows x 1 box and 128-byte swizzle.
int make_bshd_tmap(CUtensorMap* out, const void* base, int dtype, int B, int S, int H, int D, int64_t sb,
                   int64_t ss, int64_t sh, int box_rows);

}  // namespace sm100
}  // namespace fm

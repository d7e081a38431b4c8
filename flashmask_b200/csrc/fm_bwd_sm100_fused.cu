// Backward attention as ONE tcgen05 kernel for head dims up to 128: S, dP, dV, dK and dQ of
// a (query block, key tile) pair are each computed once (five GEMMs per pair).
//
// A CTA owns a sequence of UNITS, one 128-key tile of one kv head each (from the dK/dV launch
// table through a global counter, or the unit its block index names).  K and V of the unit
// stay in shared memory; 64-row halves of Q and dO of every q head of the GQA group stream
// through a ring.  TMEM lanes are keys.  Per work item (one 64-query half tile):
//     S^T  = K Q^T              M=128 keys, N=64 queries          (operands from smem)
//     dP^T = V dO^T             M=128, N=64
//     P^T  = exp2(S^T scale - LSE), dS^T = P^T (dP^T - rowsum(O dO))   (compute warpgroups)
//     dV  += P^T dO             A = P^T from TMEM (bf16)
//     dK  += dS^T Q             A = dS^T from shared memory (K-major)
//     dQ^T = K^T dS^T           M=128 head-dim columns, N=64 queries; A = the K tile read
//                               MN-major, B = the same dS^T buffer read MN-major
// dK / dV stay in TMEM for the whole unit and are written once.  dQ^T of an item is drained
// by a fourth warpgroup and added to an fp32 accumulator in global memory with coalesced
// reductions (a warp covers 32 consecutive floats of one query row); a small kernel rounds
// the accumulator to the output type afterwards.  The order of those additions is not
// fixed, so this kernel serves calls that did not ask for deterministic gradients; the
// two-kernel variant (fm_bwd_sm100_persist.cu) has one owner per output element.
//
// TMEM columns: S^T [0,64), dP^T [64,128) (one pair: an item's scores are in registers
// before the next item's score GEMMs are issued), P^T of item parity p [128+32p, +32),
// dQ^T [192,256), dV [256,384), dK [384,512).
//
// Warp roles: 0-3 / 4-7 compute warpgroups (items alternate), 8 TMA producer, 9 UMMA issuer
// (owns TMEM), 10 scheduler + list builder, 11 idle, 12-15 dQ reduction + dK/dV epilogue.
// All waits are bounded.
#include <algorithm>

#include "fm_attn_params.cuh"
#include "fm_sm100.cuh"

namespace fm {

using namespace sm100;

__device__ int g_bwd_fused_status = 0;

struct BwdFusedCfg {
  static constexpr int NSLOT = 3, LIST_MAX = 2048, NTHREADS = 512;
  static constexpr int TILE_BYTES = 128 * 128 * 2;     // 128 rows x 128 cols bf16
  static constexpr int SUB128 = 128 * 128;             // 128-row x 64-col sub-tile (bytes)
  static constexpr int SUB64 = 64 * 128;               // 64-row x 64-col sub-tile (bytes)
  static constexpr int HALF_BYTES = 2 * SUB64;         // one operand of a half tile
  static constexpr int SLOT_BYTES = 2 * HALF_BYTES;    // Q half + dO half
  static constexpr int DS_BYTES = 128 * 128;           // dS^T: 128 keys x 64 queries bf16
  static constexpr int AUX_BYTES = 2048;               // two 64-row x 16-byte statistics operands (see STAT below)
  static constexpr int OFF_STAT = 0;                   // K tile, then V tile
  static constexpr int OFF_RING = OFF_STAT + 2 * TILE_BYTES;
  static constexpr int OFF_DS = OFF_RING + NSLOT * SLOT_BYTES;          // one buffer per item parity
  // STAT: the per-query statistics enter through the GEMMs.  S^T = K Q^T gets one more k-step whose A is a
  // tile of ones and whose B holds, per query, (-c_hi, -c_lo, 0, ...) with c = LSE*log2e / scale_log2 split
  // into two 16-bit parts: the accumulator then already holds S - c, and P = exp2(scale_log2 * (S - c)) needs
  // no per-column value in the compute warps.  dP^T = V dO^T likewise gets (-d_hi, -d_lo) with d = rowsum(O dO).
  // Both operands are K-major without swizzle: 8-row x 16-byte core matrices; the second half of K (columns
  // 8..15) of A reads the ones again, that of B a block of zeros.
  static constexpr int OFF_AUX = OFF_DS + 2 * DS_BYTES;                 // per ring slot: S statistics, dP statistics
  static constexpr int OFF_ONES = OFF_AUX + NSLOT * AUX_BYTES;          // 17 core matrices of ones (2176 bytes)
  static constexpr int OFF_ZEROS = OFF_ONES + 2176;                     // 8 core matrices of zeros (1 KB)
  static constexpr int OFF_LIST = OFF_ZEROS + 1024;                     // two lists of 16-bit entries: units alternate
  static constexpr int OFF_STAGE = OFF_LIST + 2 * LIST_MAX * 2;         // reductions of the unit's K tile (8 x 4 ints)
  static constexpr int EPI_BYTES = 32 * 64;                             // per epilogue warp: 32 rows x 32 bf16 columns
  static constexpr int RROWS = 16;                                      // dQ staging: 16 query rows x 32 floats per buffer,
  static constexpr int RBUF_BYTES = RROWS * 32 * 4;                     // two buffers per warp of the reduction warpgroup
  static constexpr int OFF_EPI = OFF_STAGE + 128;                       // dQ staging; the dK/dV epilogue reuses it
  static constexpr int OFF_INFO = OFF_EPI + 4 * 2 * RBUF_BYTES;         // two unit records of 8 ints
  static constexpr int OFF_BAR = OFF_INFO + 2 * 8 * 4;
  static constexpr int OFF_MISC = OFF_BAR + 32 * 8;
  static constexpr int SMEM = OFF_MISC + 64 + 1024;
  // item-level barriers (phases follow the CTA-wide item counter) ...
  static constexpr int B_RFULL = 0, B_REMPTY = NSLOT, B_GFULL = 2 * NSLOT, B_TFULL = B_GFULL + 2,
                       B_DSFREE = B_TFULL + 2, B_SREAD = B_DSFREE + 2, B_DQFULL = B_SREAD + 1,
                       B_DQFREE = B_DQFULL + 1;
  // ... and unit-level ones (phases follow the unit counter of the CTA)
  static constexpr int B_STAT = B_DQFREE + 1, B_VFREE = B_STAT + 1, B_KFREE = B_VFREE + 1, B_ACC = B_KFREE + 1,
                       B_ACCFREE = B_ACC + 1, B_INFOREADY = B_ACCFREE + 1, B_INFOFREE = B_INFOREADY + 2,
                       B_COORD = B_INFOFREE + 2, B_FETCHGO = B_COORD + 2, B_COUNT = B_FETCHGO + 1;
  static constexpr int FETCH_AHEAD = 16;   // items left in a unit when the next one is claimed
  static_assert(B_COUNT <= 32, "barrier storage");
  static_assert(RBUF_BYTES >= EPI_BYTES && OFF_EPI % 128 == 0, "epilogue staging fits the dQ staging");
  static_assert(OFF_RING % 1024 == 0 && OFF_DS % 1024 == 0 && SLOT_BYTES % 1024 == 0, "swizzled tiles are 1 KB aligned");
  static_assert(SMEM > 120 * 1024 && SMEM <= 227 * 1024, "one CTA per SM (512 TMEM columns)");
};

// Bounded wait that hands the waiting to the barrier hardware (suspend-time hint): a waiting warp issues
// next to nothing, so the issue slots of its scheduler go to the warps that compute.  Same contract as
// mbar_wait: false when the wait was given up (abort flag or wall-clock budget).
__device__ __forceinline__ bool mbar_wait_parked(uint32_t bar, uint32_t parity, const WaitCtx& w) {
  if (mbar_try_wait(bar, parity)) return true;
  for (;;) {
    if (mbar_try_wait_suspended(bar, parity, 4000u)) return true;
    if (*w.abort_flag) return false;
    if (global_timer_ns() > w.deadline_ns) {
      *w.abort_flag = 1;
      return false;
    }
  }
}

__device__ __forceinline__ void fbulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// Barrier over the `n` threads of named barrier `id` that also ANDs a predicate: every thread of the
// group gets the same answer, so a bounded wait that gave up in one warp takes the whole group out of
// its loop together and no warp is left alone at a later barrier.
__device__ __forceinline__ bool group_all(bool ok, int id, int n) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "bar.red.and.pred q, %2, %3, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)ok), "r"(id), "r"(n)
      : "memory");
  return r != 0;
}
// Tiled reduction shared -> global through a 2-D tensor map: the box at (x, y) of the fp32 tensor gets
// the staged box added to it by the copy engine; completion is tracked by this thread's bulk groups.
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* tmap, uint32_t src_smem, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(src_smem), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Shared-memory descriptor of a K-major operand WITHOUT swizzle: 8-row x 16-byte core matrices; `lbo` = bytes
// between the two core matrices of one k-step (K columns 0..7 and 8..15), `sbo` = bytes between 8-row groups.
__device__ __forceinline__ uint64_t make_sdesc_noswz(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}

// Four k-steps (K = 64) of D[tmem] (+)= A[smem] * B[smem]: A K-major (advances 32 bytes per
// step inside its 128-byte rows), B MN-major (advances 16 rows = 2048 bytes per step).
__device__ __forceinline__ void umma_ss_k_mn_x4(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc,
                                                uint32_t acc_first) {
  asm volatile(
      "{\n\t.reg .pred p, pt;\n\t.reg .b64 ta, tb;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "add.s64 ta, %1, 2;  add.s64 tb, %2, 128;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t"
      "add.s64 ta, %1, 4;  add.s64 tb, %2, 256;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t"
      "add.s64 ta, %1, 6;  add.s64 tb, %2, 384;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t}"
      ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc), "r"(acc_first)
      : "memory");
}

// Eight k-steps (K = 128) of D[tmem] = A[smem] * B[smem], both operands MN-major: each step
// advances both by 16 rows (2048 bytes).
__device__ __forceinline__ void umma_ss_mn_mn_x8(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred pf, pt;\n\t.reg .b64 ta, tb;\n\t"
      "setp.ne.b32 pf, 0, 0;\n\t"
      "setp.eq.b32 pt, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pf;\n\t"
      "add.s64 ta, %1, 128; add.s64 tb, %2, 128;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t"
      "add.s64 ta, %1, 256; add.s64 tb, %2, 256;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t"
      "add.s64 ta, %1, 384; add.s64 tb, %2, 384;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t"
      "add.s64 ta, %1, 512; add.s64 tb, %2, 512;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t"
      "add.s64 ta, %1, 640; add.s64 tb, %2, 640;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t"
      "add.s64 ta, %1, 768; add.s64 tb, %2, 768;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t"
      "add.s64 ta, %1, 896; add.s64 tb, %2, 896;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], ta, tb, %3, pt;\n\t}"
      ::"r"(d_tmem), "l"(a), "l"(b), "r"(idesc)
      : "memory");
}

// D: width the head dims are computed at (64 when both fit, else 128); the 64-column variant
// keeps the shared-memory layout and leaves the second 64-column sub-tile of every operand
// unloaded (the dQ^T GEMM then fills TMEM lanes 64..127 from unloaded memory; nothing reads them).
template <bool IS_BF16, int D>
__global__ void __launch_bounds__(512, 1)
bwd_sm100_fused_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                       const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_do,
                       const __grid_constant__ CUtensorMap tm_dq, const AttnKParams p) {
  using Cfg = BwdFusedCfg;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sStat = sbase + Cfg::OFF_STAT, sRing = sbase + Cfg::OFF_RING, sDS = sbase + Cfg::OFF_DS;
  uint16_t* lists = reinterpret_cast<uint16_t*>(smem + Cfg::OFF_LIST);   // entry: item index | tile flags << 12
  volatile int* infos = reinterpret_cast<volatile int*>(smem + Cfg::OFF_INFO);   // [2][8]: b, head, row0, cnt, bh_mask, valid
  const uint32_t bars = sbase + Cfg::OFF_BAR;
  volatile int* misc = reinterpret_cast<volatile int*>(smem + Cfg::OFF_MISC);  // [0] tmem, [4] abort
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };

  const int tid = threadIdx.x;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int lane = tid & 31;
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_do); tma_prefetch_desc(&tm_dq);
  }
  const MaskDesc& md = p.md;
  const int off = p.Sk - p.Sq;
  const int G = p.Hq / p.Hkv;
  const int32_t* table = p.dkdv_order;
  int* sched = p.dkdv_sched;     // [0] next table entry, [1] CTAs done
  const int n_table = p.dkdv_ncta;

  if (tid == 0) misc[4] = 0;
  {
    // constant operands of the statistics k-step: ones (1.0 in the kernel's 16-bit type) and zeros
    const uint32_t one2 = IS_BF16 ? 0x3F803F80u : 0x3C003C00u;
    for (int x = tid; x < 2176 / 4; x += Cfg::NTHREADS) reinterpret_cast<uint32_t*>(smem + Cfg::OFF_ONES)[x] = one2;
    for (int x = tid; x < 1024 / 4; x += Cfg::NTHREADS) reinterpret_cast<uint32_t*>(smem + Cfg::OFF_ZEROS)[x] = 0u;
    fence_proxy_async_smem();
  }
  if (warp == 8 && lane == 0) {
    for (int i = 0; i < Cfg::NSLOT; ++i) { mbar_init(bar(Cfg::B_RFULL + i), 1); mbar_init(bar(Cfg::B_REMPTY + i), 1); }
    for (int h = 0; h < 2; ++h) {
      mbar_init(bar(Cfg::B_GFULL + h), 1); mbar_init(bar(Cfg::B_TFULL + h), 4); mbar_init(bar(Cfg::B_DSFREE + h), 1);
      mbar_init(bar(Cfg::B_INFOREADY + h), 1); mbar_init(bar(Cfg::B_INFOFREE + h), 15);
      mbar_init(bar(Cfg::B_COORD + h), 1);
    }
    mbar_init(bar(Cfg::B_SREAD), 4); mbar_init(bar(Cfg::B_DQFULL), 1); mbar_init(bar(Cfg::B_DQFREE), 4);
    mbar_init(bar(Cfg::B_FETCHGO), 1);
    mbar_init(bar(Cfg::B_STAT), 1); mbar_init(bar(Cfg::B_VFREE), 1); mbar_init(bar(Cfg::B_KFREE), 1);
    mbar_init(bar(Cfg::B_ACC), 1); mbar_init(bar(Cfg::B_ACCFREE), 4);
    fence_mbar_init();
  }
  if (warp == 9) {
    tmem_alloc(sbase + Cfg::OFF_MISC, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = (uint32_t)misc[0];
  WaitCtx wc{misc + 4, global_timer_ns() + 2000000000ull};
  constexpr uint32_t C_S = 0, C_DP = 64, C_P = 128, C_DQ = 192, C_DV = 256, C_DK = 384;

  // 512 threads start with 128 registers each; the compute warpgroups take what the others give up
  if (warp < 8) setmaxnreg_inc<168>();
  else if (warp < 12) setmaxnreg_dec<80>();
  else setmaxnreg_dec<96>();

  if (warp == 10) {
    // =========================== scheduler + list builder ===========================
    int32_t* stage = reinterpret_cast<int32_t*>(smem + Cfg::OFF_STAGE);
    bool ok = true;
    int j = 0;                                    // units published so far
    bool own_unit_taken = false;
    while (ok) {
      const int s = j & 1;
      if (j >= 2) {
        // the record and list of unit j-2 must have been released by every role
        if (lane == 0) ok = mbar_wait_idle(bar(Cfg::B_INFOFREE + s), (uint32_t)((j >> 1) - 1) & 1u, wc);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      if (j >= 1) {
        // a unit is claimed late, when the current one is nearly through: a CTA in a long unit must not
        // sit on work that an idle CTA could take
        if (lane == 0) ok = mbar_wait_idle(bar(Cfg::B_FETCHGO), (uint32_t)(j - 1) & 1u, wc);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      int b, head, row0;
      bool have;
      if (table) {
        int L = 0;
        if (lane == 0) L = atomicAdd(sched, 1);
        L = __shfl_sync(0xffffffffu, L, 0);
        have = L < n_table;
        int2 e = make_int2(0, 0);
        if (have) e = __ldg(reinterpret_cast<const int2*>(table) + L);
        row0 = e.x * 128; head = e.y % p.Hkv; b = e.y / p.Hkv;
      } else {
        have = !own_unit_taken;
        own_unit_taken = true;
        b = blockIdx.z; head = blockIdx.y; row0 = blockIdx.x * 128;
      }
      if (!have) {
        if (lane == 0) {
          infos[s * 8 + 3] = -1; infos[s * 8 + 5] = 0;
          mbar_arrive(bar(Cfg::B_COORD + s)); mbar_arrive(bar(Cfg::B_INFOREADY + s));
        }
        break;
      }
      const int hq0 = head * G;
      const int bh_mask = md.ncols ? ((md.mask_B == 1 ? 0 : b) * md.Hm + hq0 / (p.Hq / md.Hm)) : 0;
      if (lane == 0) {
        // coordinates first: the producer requests the stationary tiles while the list is being built
        infos[s * 8 + 0] = b; infos[s * 8 + 1] = head; infos[s * 8 + 2] = row0; infos[s * 8 + 4] = bh_mask;
        infos[s * 8 + 5] = 1;
        mbar_arrive(bar(Cfg::B_COORD + s));
      }
      uint16_t* list = lists + s * Cfg::LIST_MAX;
      int cnt = 0;
      {
        // 64-query half tiles that see key tile n = row0/128, ascending
        const int n = row0 / 128;
        const int n_half = (p.Sq + 63) / 64;
        const MaskDesc mst = stage_minmax(md, bh_mask, n & ~3, n + 1, stage, 4, lane);
        int lo = 0;
        if (md.causal) lo = max(0, (row0 - off) / 64);
        for (int base = lo; base < n_half; base += 32) {
          const int idx = base + lane;
          uint32_t f = 0;
          if (idx < n_half) f = tile_flags(mst, 0, n, idx * 64, min(idx * 64 + 64, p.Sq), 128);
          const uint32_t bal = __ballot_sync(0xffffffffu, f != 0);
          const int pos = cnt + __popc(bal & ((1u << lane) - 1u));
          if (f && pos < Cfg::LIST_MAX) list[pos] = (uint16_t)((uint32_t)idx | (f << 12));
          cnt += __popc(bal);
        }
      }
      cnt = min(cnt, Cfg::LIST_MAX);
      __syncwarp();
      if (lane == 0) {
        infos[s * 8 + 3] = cnt;                    // 0: nothing visible, the unit's gradients are zero
        mbar_arrive(bar(Cfg::B_INFOREADY + s));   // release: the list and the record are visible to the waiters
      }
      ++j;
    }
  } else if (warp < 8) {
    // =========================== compute warpgroups ===========================
    const int wg = warp >> 2;
    const int r = tid & 127;                     // TMEM lane = key row0 + r
    const uint32_t lane_field = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_field + C_S, tDP = tmem + lane_field + C_DP;
    const uint32_t tP = tmem + lane_field + C_P + 32u * (uint32_t)wg;
    uint8_t* dsrow = smem + Cfg::OFF_DS + wg * Cfg::DS_BYTES + r * 128;
    const float scale_log2 = p.scale_log2;
    bool ok = true;
    int kb = 0;                                  // items of earlier units
    for (int j = 0; ok; ++j) {
      const int s = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait_parked(bar(Cfg::B_INFOREADY + s), (uint32_t)(j >> 1) & 1u, wc));
      if (!ok) break;
      const int cnt = infos[s * 8 + 3];
      if (cnt < 0) break;
      const int b = infos[s * 8 + 0], hk = infos[s * 8 + 1], row0 = infos[s * 8 + 2], bh_mask = infos[s * 8 + 4];
      const uint16_t* list = lists + s * Cfg::LIST_MAX;
      const int K_items = cnt * G;
      if (cnt == 0) {
        // nothing visible: the gradients of this unit are zero
        uint16_t* gk = reinterpret_cast<uint16_t*>(p.dk) + b * p.dk_b + (int64_t)row0 * p.dk_s + hk * p.dk_h;
        uint16_t* gv = reinterpret_cast<uint16_t*>(p.dv) + b * p.dv_b + (int64_t)row0 * p.dv_s + hk * p.dv_h;
        for (int x = tid; x < 128 * 16; x += 256) {
          const int rr = x >> 4, cc = x & 15;
          if (row0 + rr < p.Sk) {
            if (cc * 8 < p.d) *reinterpret_cast<uint4*>(gk + (int64_t)rr * p.dk_s + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
            if (cc * 8 < p.dv_dim) *reinterpret_cast<uint4*>(gv + (int64_t)rr * p.dv_s + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(Cfg::B_INFOFREE + s));
        continue;
      }
      // bounds of this lane's key for the whole unit
      int lts = INT_MAX, lte = INT_MAX, uts = 0, ute = 0;
      {
        const int jj = row0 + r;
        if (jj >= p.Sk) { lts = 0; lte = INT_MAX; }
        else if (md.ncols) {
          const Bounds4 bd = load_bounds(md, md.mask + ((size_t)bh_mask * p.Sk + jj) * md.ncols);
          lts = bd.lts; lte = bd.lte; uts = bd.uts; ute = bd.ute;
        }
      }
      // this warpgroup serves the items whose CTA-wide index kk = kb + k has parity wg
      for (int k = (wg - kb) & 1; k < K_items && ok; k += 2) {
        const int kk = kb + k;
        const uint32_t e = list[k % cnt];
        const int idx = (int)(e & 0xFFFu);
        const uint32_t flags = e >> 12;
        ok = __all_sync(0xffffffffu, mbar_wait_parked(bar(Cfg::B_GFULL + wg), (uint32_t)(kk >> 1) & 1u, wc));
        if (!ok) break;
        tc_fence_after();
        const uint32_t NEG = 0xff800000u;
        // 64 score columns; once they are in registers the score buffers belong to the next item
        uint32_t sr[2][32], dr[2][32];
        tmem_ld32(tS, sr[0]); tmem_ld32(tDP, dr[0]);
        tmem_ld32(tS + 32, sr[1]); tmem_ld32(tDP + 32, dr[1]);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(Cfg::B_SREAD));
        // P^T / dS^T of this parity are free once the GEMMs of item kk-2 have completed
        if (kk >= 2) {
          ok = __all_sync(0xffffffffu, mbar_wait_parked(bar(Cfg::B_DSFREE + wg), (uint32_t)((kk >> 1) - 1) & 1u, wc));
          if (!ok) break;
        }
        // 16 columns (queries) at a time, as passes over independent elements (exp2, then dS, then
        // the packs) so that no instruction waits on its predecessor; each quarter's P^T goes to TMEM
        // and its dS^T to shared memory as soon as it is packed, which keeps few values live
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
          const int hc = qd >> 1, c0 = 16 * (qd & 1);
          const int i0 = idx * 64 + 16 * qd;            // first query of this quarter
          if (flags & ~FM_TF_ACTIVE) {
            // for this key the masked queries are intervals of the 16 columns: one mask word, one bit test per column
            const int a0 = lts - i0, a1 = lte - i0, b0 = uts - i0, b1 = ute - i0;
            const int cz = md.causal ? (row0 + r - off - i0) : 0;         // masked while c < cz
            const uint32_t mbits = (bits_below(a1) & ~bits_below(a0)) | (bits_below(b1) & ~bits_below(b0)) |
                                   bits_below(cz);
#pragma unroll
            for (int c = 0; c < 16; ++c)
              if (mbits & (1u << c)) sr[hc][c0 + c] = NEG;
          }
          // the accumulators already hold S - LSE/scale and dP - rowsum(O dO) (statistics k-step)
          float pe[16], de[16];
#pragma unroll
          for (int c = 0; c < 16; c += 2) {
            float x0, x1;
            mul2(x0, x1, __uint_as_float(sr[hc][c0 + c]), __uint_as_float(sr[hc][c0 + c + 1]), scale_log2, scale_log2);
            pe[c] = fast_exp2(x0); pe[c + 1] = fast_exp2(x1);
          }
#pragma unroll
          for (int c = 0; c < 16; c += 2)
            mul2(de[c], de[c + 1], pe[c], pe[c + 1], __uint_as_float(dr[hc][c0 + c]), __uint_as_float(dr[hc][c0 + c + 1]));
          uint32_t pk1[8], pk2[8];
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            pk1[c] = pack2<IS_BF16>(pe[2 * c], pe[2 * c + 1]);
            pk2[c] = pack2<IS_BF16>(de[2 * c], de[2 * c + 1]);
          }
          tmem_st8(tP + 8 * qd, pk1);
          // dS^T row of this key, queries [16 qd, 16 qd + 16): two 16-byte chunks, 128-byte swizzle
          *reinterpret_cast<uint4*>(dsrow + (((2 * qd) ^ (r & 7)) << 4)) = make_uint4(pk2[0], pk2[1], pk2[2], pk2[3]);
          *reinterpret_cast<uint4*>(dsrow + (((2 * qd + 1) ^ (r & 7)) << 4)) = make_uint4(pk2[4], pk2[5], pk2[6], pk2[7]);
        }
        tc_wait_st();
        fence_proxy_async_smem();   // the dS^T stores become visible to the tensor core's reads
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(Cfg::B_TFULL + wg));
      }
      if (!ok) break;
      if (lane == 0) mbar_arrive(bar(Cfg::B_INFOFREE + s));   // list and record of this unit are no longer read
      kb += K_items;
    }
  } else if (warp == 8) {
    // =========================== producer ===========================
    bool ok = true;
    int kb = 0;
    for (int j = 0; ok; ++j) {
      const int s = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait_parked(bar(Cfg::B_COORD + s), (uint32_t)(j >> 1) & 1u, wc));
      if (!ok) break;
      if (infos[s * 8 + 5] == 0) break;
      const int b = infos[s * 8 + 0], hk = infos[s * 8 + 1], row0 = infos[s * 8 + 2];
      const int hq0 = hk * G;
      const uint16_t* list = lists + s * Cfg::LIST_MAX;
      // V is free once every score GEMM of the previous unit has completed, K once its last dQ^T GEMM has
      if (j > 0) {
        if (lane == 0) ok = mbar_wait_parked(bar(Cfg::B_VFREE), (uint32_t)(j - 1) & 1u, wc);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      if (elect_one()) {
        mbar_arrive_expect_tx(bar(Cfg::B_STAT), 2 * Cfg::TILE_BYTES * D / 128);
        for (int dc = 0; dc < D / 64; ++dc)
          tma_load_4d(sStat + Cfg::TILE_BYTES + dc * Cfg::SUB128, &tm_v, bar(Cfg::B_STAT), dc * 64, hk, row0, b);
      }
      if (j > 0) {
        if (lane == 0) ok = mbar_wait_parked(bar(Cfg::B_KFREE), (uint32_t)(j - 1) & 1u, wc);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      if (elect_one()) {
        for (int dc = 0; dc < D / 64; ++dc)
          tma_load_4d(sStat + dc * Cfg::SUB128, &tm_k, bar(Cfg::B_STAT), dc * 64, hk, row0, b);
      }
      // ... and the items once the list is there
      ok = __all_sync(0xffffffffu, mbar_wait_parked(bar(Cfg::B_INFOREADY + s), (uint32_t)(j >> 1) & 1u, wc));
      if (!ok) break;
      const int cnt = infos[s * 8 + 3];
      const int K_items = cnt * G;
      const int k_go = max(0, K_items - Cfg::FETCH_AHEAD);
      if (K_items == 0 && lane == 0) mbar_arrive(bar(Cfg::B_FETCHGO));
      for (int k = 0; k < K_items && ok; ++k) {
        if (k == k_go && lane == 0) mbar_arrive(bar(Cfg::B_FETCHGO));   // the scheduler may claim the next unit
        const int kk = kb + k;
        const int idx = (int)(list[k % cnt] & 0xFFFu);
        const int slot = kk % Cfg::NSLOT;
        const uint32_t par = ((uint32_t)(kk / Cfg::NSLOT) & 1u) ^ 1u;
        const int hstr = hq0 + k / cnt;
        if (lane == 0) ok = mbar_wait_parked(bar(Cfg::B_REMPTY + slot), par, wc);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (elect_one()) {
          const uint32_t dst = sRing + slot * Cfg::SLOT_BYTES;
          const uint32_t fb = bar(Cfg::B_RFULL + slot);
          mbar_arrive_expect_tx(fb, Cfg::SLOT_BYTES * D / 128 + Cfg::AUX_BYTES);
          for (int dc = 0; dc < D / 64; ++dc) {
            tma_load_4d(dst + dc * Cfg::SUB64, &tm_q, fb, dc * 64, hstr, idx * 64, b);
            tma_load_4d(dst + Cfg::HALF_BYTES + dc * Cfg::SUB64, &tm_do, fb, dc * 64, hstr, idx * 64, b);
          }
          // statistics operands of the 64 queries: 16 bytes per query and array, contiguous in global memory
          const int64_t at = (((int64_t)b * p.Hq + hstr) * p.Sq_r + idx * 64) * 8;
          const uint32_t ax = sbase + Cfg::OFF_AUX + slot * Cfg::AUX_BYTES;
          fbulk_copy_g2s(ax, p.stat_s + at, 1024, fb);
          fbulk_copy_g2s(ax + 1024, p.stat_dp + at, 1024, fb);
        }
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(Cfg::B_INFOFREE + s));
      kb += K_items;
    }
  } else if (warp == 9) {
    // =========================== UMMA issuer 1: the score GEMMs ===========================
    // S^T and dP^T of item kk are issued as soon as the scores of item kk-1 are in registers and
    // the operands of item kk have landed; nothing here waits for the compute warpgroups' results.
    if (elect_one()) {
      constexpr uint32_t idesc_g = make_idesc(IS_BF16, 128, 64, 0, 0);      // S^T, dP^T
      const uint64_t dKk = make_sdesc(sStat, 16, 1024);                     // K tile, K-major (A of S^T)
      const uint64_t dVk = make_sdesc(sStat + Cfg::TILE_BYTES, 16, 1024);   // V tile, K-major (A of dP^T)
      const uint64_t dRk = make_sdesc(sRing, 16, 1024);                     // K-major view of a ring slot
      // 128 rows of ones: 8-row groups 128 bytes apart; the second core matrix of a group is the next group
      const uint64_t dOnes = make_sdesc_noswz(sbase + Cfg::OFF_ONES, 128, 128);
      bool ok = true;
      int kb = 0;
      for (int j = 0; ok; ++j) {
        const int s = j & 1;
        ok = mbar_wait_parked(bar(Cfg::B_INFOREADY + s), (uint32_t)(j >> 1) & 1u, wc);
        if (!ok) break;
        const int cnt = infos[s * 8 + 3];
        if (cnt < 0) break;
        const int K_items = cnt * G;
        mbar_arrive(bar(Cfg::B_INFOFREE + s));     // only the item count is needed here
        ok = mbar_wait_parked(bar(Cfg::B_STAT), (uint32_t)j & 1u, wc);
        if (!ok) break;
        if (K_items == 0) {
          // the stationary tiles of an empty unit have landed and are not used
          mbar_arrive(bar(Cfg::B_VFREE)); mbar_arrive(bar(Cfg::B_KFREE));
          continue;
        }
        for (int k = 0; k < K_items && ok; ++k) {
          const int kk = kb + k;
          const int slot = kk % Cfg::NSLOT, pz = kk & 1;
          if (kk >= 1) ok = mbar_wait_parked(bar(Cfg::B_SREAD), (uint32_t)(kk - 1) & 1u, wc);
          ok = ok && mbar_wait_parked(bar(Cfg::B_RFULL + slot), (uint32_t)(kk / Cfg::NSLOT) & 1u, wc);
          if (!ok) break;
          tc_fence_after();
          const uint64_t dq_ = dRk + (uint64_t)(slot * (Cfg::SLOT_BYTES >> 4));
          const uint64_t do_ = dq_ + (uint64_t)(Cfg::HALF_BYTES >> 4);
          // statistics operands of this slot: B rows 16 bytes apart (8-row groups 128 bytes apart), its second
          // core matrix is the block of zeros further up in shared memory
          const uint32_t sAux = sbase + Cfg::OFF_AUX + slot * Cfg::AUX_BYTES;
          const uint64_t dSs = make_sdesc_noswz(sAux, sbase + Cfg::OFF_ZEROS - sAux, 128);
          const uint64_t dSd = make_sdesc_noswz(sAux + 1024, sbase + Cfg::OFF_ZEROS - (sAux + 1024), 128);
          if constexpr (D == 128) {
            umma_ss_x8<(Cfg::SUB128 >> 4), (Cfg::SUB64 >> 4)>(tmem + C_S, dKk, dq_, idesc_g, 0u);
            umma_ss(tmem + C_S, dOnes, dSs, idesc_g, 1u);
            umma_ss_x8<(Cfg::SUB128 >> 4), (Cfg::SUB64 >> 4)>(tmem + C_DP, dVk, do_, idesc_g, 0u);
            umma_ss(tmem + C_DP, dOnes, dSd, idesc_g, 1u);
          } else {
            umma_ss_x4(tmem + C_S, dKk, dq_, idesc_g, 0u);
            umma_ss(tmem + C_S, dOnes, dSs, idesc_g, 1u);
            umma_ss_x4(tmem + C_DP, dVk, do_, idesc_g, 0u);
            umma_ss(tmem + C_DP, dOnes, dSd, idesc_g, 1u);
          }
          tc_commit(bar(Cfg::B_GFULL + pz));
          if (k == K_items - 1) tc_commit(bar(Cfg::B_VFREE));   // that was the unit's last read of V
        }
        kb += K_items;
      }
    }
    __syncwarp();
  } else if (warp == 11) {
    // =========================== UMMA issuer 2: dV, dK, dQ^T ===========================
    if (elect_one()) {
      constexpr uint32_t idesc_acc = make_idesc(IS_BF16, 128, D, 0, 1);     // dV, dK
      constexpr uint32_t idesc_dq = make_idesc(IS_BF16, 128, 64, 1, 1);     // dQ^T
      const uint64_t dKm = make_sdesc(sStat, Cfg::SUB128, 1024);            // K tile, MN-major (A of dQ^T)
      const uint64_t dRm = make_sdesc(sRing, Cfg::SUB64, 1024);             // MN-major view of a ring slot
      const uint64_t dDk = make_sdesc(sDS, 16, 1024);                       // dS^T, K-major (A of dK)
      const uint64_t dDm = make_sdesc(sDS, Cfg::DS_BYTES, 1024);            // dS^T, MN-major (B of dQ^T)
      bool ok = true;
      int kb = 0, ju = 0;
      for (int j = 0; ok; ++j) {
        const int s = j & 1;
        ok = mbar_wait_parked(bar(Cfg::B_INFOREADY + s), (uint32_t)(j >> 1) & 1u, wc);
        if (!ok) break;
        const int cnt = infos[s * 8 + 3];
        if (cnt < 0) break;
        const int K_items = cnt * G;
        mbar_arrive(bar(Cfg::B_INFOFREE + s));
        if (K_items == 0) continue;                // issuer 1 releases the tiles of an empty unit
        for (int k = 0; k < K_items && ok; ++k) {
          const int kk = kb + k;
          const int slot = kk % Cfg::NSLOT, pz = kk & 1;
          ok = mbar_wait_parked(bar(Cfg::B_TFULL + pz), (uint32_t)(kk >> 1) & 1u, wc);
          if (!ok) break;
          if (k == 0 && ju > 0) {
            // the accumulators still hold the previous unit until its epilogue has read them
            ok = mbar_wait_parked(bar(Cfg::B_ACCFREE), (uint32_t)(ju - 1) & 1u, wc);
            if (!ok) break;
          }
          tc_fence_after();
          const uint64_t dm_q = dRm + (uint64_t)(slot * (Cfg::SLOT_BYTES >> 4));   // Q half, MN-major
          const uint64_t dm_do = dm_q + (uint64_t)(Cfg::HALF_BYTES >> 4);           // dO half, MN-major
          const uint32_t acc_on = k > 0 ? 1u : 0u;
          // dV += P^T dO, dK += dS^T Q; that was the last read of the ring slot
          umma_ts_xn<4>(tmem + C_DV, tmem + C_P + 32u * (uint32_t)pz, dm_do, idesc_acc, acc_on);
          umma_ss_k_mn_x4(tmem + C_DK, dDk + (uint64_t)(pz * (Cfg::DS_BYTES >> 4)), dm_q, idesc_acc, acc_on);
          tc_commit(bar(Cfg::B_REMPTY + slot));
          // dQ^T = K^T dS^T: its buffer is free once the reduction warpgroup has read item kk-1
          if (kk >= 1) {
            ok = mbar_wait_parked(bar(Cfg::B_DQFREE), (uint32_t)(kk - 1) & 1u, wc);
            if (!ok) break;
            tc_fence_after();
          }
          umma_ss_mn_mn_x8(tmem + C_DQ, dKm, dDm + (uint64_t)(pz * (Cfg::DS_BYTES >> 4)), idesc_dq);
          tc_commit(bar(Cfg::B_DQFULL));
          tc_commit(bar(Cfg::B_DSFREE + pz));
          if (k == K_items - 1) { tc_commit(bar(Cfg::B_KFREE)); tc_commit(bar(Cfg::B_ACC)); }
        }
        ++ju;
        kb += K_items;
      }
    }
    __syncwarp();
  } else if (warp >= 12) {
    // =========================== dQ reduction + dK/dV epilogue ===========================
    // Warp 12+e owns TMEM lanes [32e, 32e+32).  dQ^T of an item: lane = head-dim column, 64 columns
    // = the item's queries; a warp adds 32 consecutive floats of one query row per instruction.
    // dK / dV of a unit: 32 columns at a time through a 2 KB staging area of the warp (rows of 64
    // bytes, 16-byte pieces XOR-swizzled by row) so that one store writes 8 rows x 64 contiguous bytes.
    const int ew = warp - 12;
    const uint32_t lane_field = (uint32_t)(ew * 32) << 16;
    uint8_t* wst = smem + Cfg::OFF_EPI + ew * 2 * Cfg::RBUF_BYTES;   // this warp's two staging buffers
    uint8_t* stg = wst;                                              // ... the first also stages dK / dV
    uint32_t rnd = 0;                            // staging rounds of this warp so far (buffer = rnd & 1)
    bool ok = true;
    int ju = 0, kb = 0;
    for (int j = 0; ok; ++j) {
      const int s = j & 1;
      ok = group_all(mbar_wait_idle(bar(Cfg::B_INFOREADY + s), (uint32_t)(j >> 1) & 1u, wc), 2, 128);
      if (!ok) break;
      const int cnt = infos[s * 8 + 3];
      if (cnt < 0) break;
      const int b = infos[s * 8 + 0], head = infos[s * 8 + 1], row0 = infos[s * 8 + 2];
      const uint16_t* list = lists + s * Cfg::LIST_MAX;
      const int K_items = cnt * G;
      // dQ^T of an item: this warp's lanes are 32 head-dim columns, the 64 TMEM columns the item's
      // queries.  16 queries at a time the lane writes its column transposed into a staging buffer
      // ([query][32 columns], conflict-free) and lane 0 hands the buffer to the copy engine, which adds
      // the 16 x 32 box to the fp32 accumulator.  Two buffers per warp: before a buffer is rewritten lane 0
      // waits until every reduction but the latest has read its source.
      for (int k = 0; k < K_items && ok; ++k) {
        const int kk = kb + k;
        ok = group_all(mbar_wait_parked(bar(Cfg::B_DQFULL), (uint32_t)kk & 1u, wc), 2, 128);
        if (!ok) break;
        tc_fence_after();
        const int q0 = (int)(list[k % cnt] & 0xFFFu) * 64;
        const int hq = head * G + k / cnt;
        const int row_base = (b * p.Hq + hq) * p.Sq_r + q0;   // rows past Sq (inside the padding) receive zeros
        uint32_t v[4][16];
#pragma unroll
        for (int r = 0; r < 4; ++r) tmem_ld16(tmem + lane_field + C_DQ + 16 * r, v[r]);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(Cfg::B_DQFREE));
        if (32 * ew < D) {
#pragma unroll
          for (int r = 0; r < 4; ++r) {
            uint8_t* sb = wst + (rnd & 1u) * Cfg::RBUF_BYTES;
            if (lane == 0) bulk_wait_read<1>();
            __syncwarp();
#pragma unroll
            for (int c = 0; c < 16; ++c) reinterpret_cast<uint32_t*>(sb)[c * 32 + lane] = v[r][c];
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              tma_reduce_add_2d(&tm_dq, smem_u32(sb), 32 * ew, row_base + 16 * r);
              bulk_commit();
            }
            ++rnd;
          }
        }
      }
      if (!ok) break;
      kb += K_items;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(Cfg::B_INFOFREE + s));
      if (cnt == 0) continue;                    // the compute warpgroups write the zeros of an empty unit
      // the epilogue stages through this warp's first buffer: its reductions must have read it
      if (lane == 0) bulk_wait_read<0>();
      ok = group_all(mbar_wait_parked(bar(Cfg::B_ACC), (uint32_t)ju & 1u, wc), 2, 128);
      if (!ok) break;
      ++ju;
      tc_fence_after();
      const int rbase = row0 + 32 * ew;
#pragma unroll
      for (int o = 0; o < 2; ++o) {
        // o = 0 dV, o = 1 dK (scaled)
        const uint32_t tA = tmem + lane_field + (o == 0 ? C_DV : C_DK);
        const float mul = o == 0 ? 1.f : p.scale;
        const int width = o == 0 ? p.dv_dim : p.d;   // head dims below 128 end here
        uint16_t* gbase = o == 0 ? reinterpret_cast<uint16_t*>(p.dv) + b * p.dv_b + head * p.dv_h
                                 : reinterpret_cast<uint16_t*>(p.dk) + b * p.dk_b + head * p.dk_h;
        const int64_t ld = o == 0 ? p.dv_s : p.dk_s;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t acc[32];
          tmem_ld32(tA + 32 * c, acc);
          tc_wait_ld();
          if (o == 1 && c == D / 32 - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(Cfg::B_ACCFREE));   // the next unit may overwrite the accumulators
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 v;
            v.x = pack2<IS_BF16>(__uint_as_float(acc[8 * q4 + 0]) * mul, __uint_as_float(acc[8 * q4 + 1]) * mul);
            v.y = pack2<IS_BF16>(__uint_as_float(acc[8 * q4 + 2]) * mul, __uint_as_float(acc[8 * q4 + 3]) * mul);
            v.z = pack2<IS_BF16>(__uint_as_float(acc[8 * q4 + 4]) * mul, __uint_as_float(acc[8 * q4 + 5]) * mul);
            v.w = pack2<IS_BF16>(__uint_as_float(acc[8 * q4 + 6]) * mul, __uint_as_float(acc[8 * q4 + 7]) * mul);
            *reinterpret_cast<uint4*>(stg + lane * 64 + ((q4 ^ ((lane >> 1) & 3)) << 4)) = v;
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int rr = 8 * i + (lane >> 2), piece = lane & 3;
            const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 64 + ((piece ^ ((rr >> 1) & 3)) << 4));
            if (rbase + rr < p.Sk && 32 * c + 8 * piece < width)
              *reinterpret_cast<uint4*>(gbase + (int64_t)(rbase + rr) * ld + 32 * c + 8 * piece) = v;
          }
          __syncwarp();
        }
      }
    }
    if (lane == 0) bulk_wait_all();
  }

  // =========================== teardown ===========================
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (misc[4] != 0) {
    const uint64_t t_end = global_timer_ns() + 200000ull;
    while (global_timer_ns() < t_end) __nanosleep(1000);
    if (tid == 0) atomicExch(&g_bwd_fused_status, FM_ERR_TIMEOUT);
  }
  if (warp == 9) tmem_dealloc(tmem, 512);
  if (table && tid == 0) {
    // the last CTA to leave rewinds the counters for the next launch that uses this table
    __threadfence();
    if (atomicAdd(sched + 1, 1) == (int)(gridDim.x * gridDim.y * gridDim.z) - 1) {
      atomicExch(sched, 0);
      atomicExch(sched + 1, 0);
    }
  }
}

// dq = round(scale * dq_accum): [B, Hq, Sq_r, D] fp32 -> [B, Sq, Hq, d] in the output type.
template <bool IS_BF16, int D>
__global__ void __launch_bounds__(256) bwd_dq_round_kernel(const AttnKParams p) {
  constexpr int CPR = D / 8;                    // 16-byte output chunks per row
  const int64_t n = (int64_t)p.B * p.Hq * p.Sq * CPR;
  for (int64_t x = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; x < n; x += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(x % CPR);
    const int64_t row = x / CPR;                // (b * Hq + h) * Sq + i
    const int i = (int)(row % p.Sq);
    const int64_t bh = row / p.Sq;
    const int h = (int)(bh % p.Hq), b = (int)(bh / p.Hq);
    if (c * 8 >= p.d) continue;
    const float4* src = reinterpret_cast<const float4*>(p.dq_accum + ((bh * p.Sq_r + i) * D + c * 8));
    const float4 a = src[0], g = src[1];
    uint4 v;
    v.x = pack2<IS_BF16>(a.x * p.scale, a.y * p.scale); v.y = pack2<IS_BF16>(a.z * p.scale, a.w * p.scale);
    v.z = pack2<IS_BF16>(g.x * p.scale, g.y * p.scale); v.w = pack2<IS_BF16>(g.z * p.scale, g.w * p.scale);
    uint16_t* dst = reinterpret_cast<uint16_t*>(p.dq) + b * p.dq_b + (int64_t)i * p.dq_s + h * p.dq_h + c * 8;
    *reinterpret_cast<uint4*>(dst) = v;
  }
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
size_t bwd_sm100_fused_accum_bytes(const fm_attn_args* a) {
  const size_t D = (a->d <= 64 && a->dv <= 64) ? 64 : 128;
  const size_t sq_r = (size_t)((a->Sq + 127) / 128) * 128;
  return (size_t)a->B * a->Hq * sq_r * D * sizeof(float);
}

template <bool IS_BF16, int D>
static int launch_bwd_sm100_fused(const AttnKParams& p, const fm_attn_args* a, cudaStream_t s) {
  using Cfg = BwdFusedCfg;
  FM_REQUIRE((a->Sq + 63) / 64 <= Cfg::LIST_MAX, FM_ERR_UNSUPPORTED,
             "backward: Sq=%d exceeds the %d rows this kernel variant indexes", a->Sq, Cfg::LIST_MAX * 64);
  CUtensorMap k128, v128, q64, do64;
  int rc;
#define FM_TMAP(out, ptr, S, H, Dm, st, rows)                                                          \
  if ((rc = make_bshd_tmap(&out, ptr, a->dtype, a->B, S, H, Dm, st[0], st[1], st[2], rows))) return rc;
  FM_TMAP(k128, a->k, a->Sk, a->Hkv, a->d, a->k_stride, 128)
  FM_TMAP(v128, a->v, a->Sk, a->Hkv, a->dv, a->v_stride, 128)
  FM_TMAP(q64, a->q, a->Sq, a->Hq, a->d, a->q_stride, 64)
  FM_TMAP(do64, a->d_o, a->Sq, a->Hq, a->dv, a->do_stride, 64)
#undef FM_TMAP
  // fp32 dQ accumulator as a 2-D tensor [B*Hq*Sq_r rows, D columns], boxes of 16 rows x 32 columns
  CUtensorMap dqmap;
  {
    EncodeTiledFn enc = get_encode_tiled();
    FM_REQUIRE(enc != nullptr, FM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)p.B * p.Hq * p.Sq_r};
    const cuuint64_t strides[1] = {(cuuint64_t)D * 4};
    const cuuint32_t box[2] = {32, (cuuint32_t)Cfg::RROWS};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = enc(&dqmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, p.dq_accum, dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    FM_REQUIRE(r == CUDA_SUCCESS, FM_ERR_CUDA, "cuTensorMapEncodeTiled (dQ accumulator) failed with CUresult %d", (int)r);
  }
  auto kern = bwd_sm100_fused_kernel<IS_BF16, D>;
  FM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
  // (the accumulator was cleared by the preprocess kernel, row by row, unless this call carries earlier sums)
  int dev = 0, n_sm = 0;
  FM_CUDA_TRY(cudaGetDevice(&dev));
  FM_CUDA_TRY(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
  // with a launch table: one persistent CTA per SM (fewer when the table is shorter)
  const dim3 grid = p.dkdv_order ? dim3(std::min(p.dkdv_ncta, n_sm)) : dim3((p.Sk + 127) / 128, p.Hkv, p.B);
  kern<<<grid, Cfg::NTHREADS, Cfg::SMEM, s>>>(k128, v128, q64, do64, dqmap, p);
  FM_CUDA_TRY(cudaGetLastError());
  const int64_t n = (int64_t)p.B * p.Hq * p.Sq * (D / 8);
  const unsigned blocks = (unsigned)std::min<int64_t>((n + 255) / 256, (int64_t)n_sm * 16);
  if (!(p.bwd_flags & FM_BWD_DQ_LEAVE)) {
    bwd_dq_round_kernel<IS_BF16, D><<<blocks, 256, 0, s>>>(p);
    FM_CUDA_TRY(cudaGetLastError());
    count_launches(1);
  }
  count_launches(1);
  return FM_OK;
}

int bwd_sm100_fused_launch(const AttnKParams& p, const fm_attn_args* a, cudaStream_t s) {
  const bool bf = a->dtype == FM_DTYPE_BF16;
  if (a->d <= 64 && a->dv <= 64)
    return bf ? launch_bwd_sm100_fused<true, 64>(p, a, s) : launch_bwd_sm100_fused<false, 64>(p, a, s);
  return bf ? launch_bwd_sm100_fused<true, 128>(p, a, s) : launch_bwd_sm100_fused<false, 128>(p, a, s);
}

int bwd_sm100_fused_status(int* out, bool reset) {
  int v = 0;
  FM_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_bwd_fused_status, sizeof(int)));
  if (reset && v != 0) {
    const int z = 0;
    FM_CUDA_TRY(cudaMemcpyToSymbol(g_bwd_fused_status, &z, sizeof(int)));
  }
  *out = v;
  return FM_OK;
}

}  // namespace fm

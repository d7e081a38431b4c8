// Persistent variant of the tcgen05 forward kernel (d = dv = 128), used when the caller supplies
// a launch table (sparse masks).  Same tiling, tensor-memory layout and tile arithmetic as
// fm_fwd_sm100.cu (the tile body is shared: fm_fwd_sm100_tile.inc); what differs is the control
// flow around a work unit (256 query rows of one (batch, q head)):
//
//   * one CTA per SM walks the launch table through a global counter; a unit is claimed late,
//     when the current one has few K tiles left;
//   * the scheduler warp fetches the next unit, builds its K-tile list into the second list
//     buffer and publishes its coordinates first, so that the producer requests the next Q
//     tiles as soon as the last S = Q K^T of the current unit has completed;
//   * the epilogue stages O through a small per-warp area instead of the Q tiles, so the next
//     unit's Q loads and first score GEMMs run under the epilogue of the current one.
//
// Ring slots, bounds slots and the per-sub-tile S / P / O barriers keep counting over the life
// of the CTA; only the first-tile flags (accumulate off, no rescale) are per unit.
// Warp roles: 0-3 / 4-7 softmax warpgroups, 8 TMA producer, 9 UMMA issuer (owns TMEM),
// 10 scheduler + list builder, 11 idle.  All waits are bounded.
#include <algorithm>

#include <type_traits>

#include "fm_attn_params.cuh"
#include "fm_sm100.cuh"

namespace fm {

using namespace sm100;

__device__ int g_fwd_persist_status = 0;

struct FwdPersistCfg {
  static constexpr int D = 128, DV = 128;
  static constexpr int NSTAGE = 4, NBND = 2, LIST_MAX = 1024, NTHREADS = 384;
  static constexpr int SUB = 128 * 128;                 // bytes of a 128-row x 64-col bf16 sub-tile
  static constexpr int Q_BYTES = 128 * D * 2;
  static constexpr int SLOT_BYTES = 128 * D * 2;
  static constexpr int BND_BYTES = 128 * 4 * 4;
  static constexpr int STAGE_TILES = 64;                // K tiles whose reductions are staged at a time
  static constexpr int EPI_BYTES = 32 * 64;             // per softmax warp: 32 rows x 32 bf16 columns
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_KV = OFF_Q + 2 * Q_BYTES;
  static constexpr int OFF_BND = OFF_KV + NSTAGE * SLOT_BYTES;
  static constexpr int OFF_LIST = OFF_BND + NBND * BND_BYTES;           // two lists: units alternate
  static constexpr int OFF_STAGE = OFF_LIST + 2 * LIST_MAX * 4;
  static constexpr int OFF_EPI = OFF_STAGE + 8 * STAGE_TILES * 4;
  static constexpr int OFF_INFO = OFF_EPI + 8 * EPI_BYTES;              // two unit records of 8 ints
  static constexpr int OFF_BAR = OFF_INFO + 2 * 8 * 4;
  static constexpr int OFF_MISC = OFF_BAR + 32 * 8;
  static constexpr int SMEM = OFF_MISC + 64 + 1024;
  // tile-level barriers (phases follow CTA-wide counters) ...
  static constexpr int B_KVFULL = 0, B_KVEMPTY = NSTAGE, B_SFULL = 2 * NSTAGE, B_PFULL = B_SFULL + 2,
                       B_ODONE = B_PFULL + 2, B_BNDFULL = B_ODONE + 2, B_BNDEMPTY = B_BNDFULL + NBND;
  // ... and unit-level ones (phases follow the unit counter of the CTA)
  static constexpr int B_QFULL = B_BNDEMPTY + NBND, B_QFREE = B_QFULL + 2, B_INFOREADY = B_QFREE + 1,
                       B_INFOFREE = B_INFOREADY + 2, B_COORD = B_INFOFREE + 2, B_FETCHGO = B_COORD + 2,
                       B_COUNT = B_FETCHGO + 1;
  static constexpr int FETCH_AHEAD = 6;                 // K tiles left in a unit when the next one is claimed
  static_assert(B_COUNT <= 32, "barrier storage");
  static_assert(SMEM > 120 * 1024 && SMEM <= 227 * 1024, "one CTA per SM (512 TMEM columns)");
};

__device__ __forceinline__ float neg_inf() { return __int_as_float(0xff800000); }

template <bool IS_BF16>
__global__ void __launch_bounds__(384, 1)
fwd_sm100_persist_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                         const __grid_constant__ CUtensorMap tm_v, const AttnKParams p) {
  using Cfg = FwdPersistCfg;
  constexpr int D = Cfg::D, DV = Cfg::DV;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase + Cfg::OFF_Q, sKV = sbase + Cfg::OFF_KV;
  uint32_t* lists = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_LIST);
  // [2][8]: b, hq, first query row, K tiles (-1: no more units), bh_mask, valid, tiles of sub-tile 0, of sub-tile 1
  volatile int* infos = reinterpret_cast<volatile int*>(smem + Cfg::OFF_INFO);
  const uint32_t bars = sbase + Cfg::OFF_BAR;
  volatile int* misc = reinterpret_cast<volatile int*>(smem + Cfg::OFF_MISC);   // [0] tmem base, [4] abort
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };

  const int tid = threadIdx.x;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int lane = tid & 31;
  if (warp == 8 && lane == 0) { tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); }
  const MaskDesc& md = p.md;
  const int off = p.Sk - p.Sq;
  const int32_t* table = p.fwd_order;
  int* sched = p.fwd_sched;            // [0] next table entry, [1] CTAs that left
  const int n_table = p.fwd_ncta;

  if (tid == 0) misc[4] = 0;
  if (warp == 8 && lane == 0) {
    for (int i = 0; i < Cfg::NSTAGE; ++i) { mbar_init(bar(Cfg::B_KVFULL + i), 1); mbar_init(bar(Cfg::B_KVEMPTY + i), 1); }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(Cfg::B_SFULL + s), 1); mbar_init(bar(Cfg::B_PFULL + s), 128); mbar_init(bar(Cfg::B_ODONE + s), 1);
      mbar_init(bar(Cfg::B_QFULL + s), 1);
      mbar_init(bar(Cfg::B_INFOREADY + s), 1); mbar_init(bar(Cfg::B_INFOFREE + s), 10); mbar_init(bar(Cfg::B_COORD + s), 1);
    }
    for (int i = 0; i < Cfg::NBND; ++i) { mbar_init(bar(Cfg::B_BNDFULL + i), 32); mbar_init(bar(Cfg::B_BNDEMPTY + i), 256); }
    mbar_init(bar(Cfg::B_QFREE), 1);
    mbar_init(bar(Cfg::B_FETCHGO), 1);
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

  if (warp < 8) {
    // =========================== softmax warpgroups ===========================
    setmaxnreg_inc<216>();
    const int s = warp >> 2;
    const int r = tid & 127;                   // row inside the sub-tile == TMEM lane
    const uint32_t lane_field = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_field + 128u * s;
    const uint32_t tP = tS + 64u;
    const uint32_t tO = tmem + lane_field + 256u + 128u * s;
    uint8_t* stg = smem + Cfg::OFF_EPI + warp * Cfg::EPI_BYTES;   // 32 rows x 64 bytes, 16-byte pieces XOR-swizzled
    const float scale_log2 = p.scale_log2;
    constexpr int BLOCK_SCORE = 0; constexpr bool BLOCK_BOS = false;       // the block-score side output is served by the one-unit kernel
    const int bs_rel0 = 0; float* const bs_dst = nullptr; float* const bs_acc = nullptr;
    int n_tot = 0, nbnd = 0;                   // tiles of this sub-tile / bounds slots over the life of the CTA
    bool ok = true;
    for (int j = 0; ok; ++j) {
      const int us = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_INFOREADY + us), (uint32_t)(j >> 1) & 1u, wc));
      if (!ok) break;
      const int cnt = infos[us * 8 + 3];
      if (cnt < 0) break;
      const int b = infos[us * 8 + 0], hq = infos[us * 8 + 1], ms = infos[us * 8 + 2];
      const uint32_t* list = lists + us * Cfg::LIST_MAX;
      const int row = ms + 128 * s + r;
      float m_run = neg_inf(), l_run = 0.f;
      int n_done = 0;                          // tiles of this sub-tile accumulated in this unit
      for (int i = 0; i < cnt && ok; ++i) {
        const uint32_t e = list[i];
        const uint32_t flags = (e >> (16 + 4 * s)) & 0xFu;
        const bool any_bounds = (((e >> 16) | (e >> 20)) & FM_TF_BOUNDS) != 0;
        const int bslot = nbnd % Cfg::NBND;
        const uint32_t bpar = (uint32_t)(nbnd / Cfg::NBND) & 1u;
        if (any_bounds) {
          // every softmax thread passes through the full barrier of a bounds slot before releasing it, so a
          // warpgroup that runs ahead (inactive on these tiles) cannot arrive twice within one phase
          ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_BNDFULL + bslot), bpar, wc));
          if (!ok) break;
        }
        if (flags) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_SFULL + s), (uint32_t)n_tot & 1u, wc));
          if (!ok) break;
#define FM_N_UNIT n_done
#define FM_N_TOT n_tot
#include "fm_fwd_sm100_tile.inc"
#undef FM_N_UNIT
#undef FM_N_TOT
          tc_wait_st();
          tc_fence_before();
          mbar_arrive(bar(Cfg::B_PFULL + s));
          ++n_done;
          ++n_tot;
        }
        if (any_bounds) {
          mbar_arrive(bar(Cfg::B_BNDEMPTY + bslot));
          ++nbnd;
        }
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(Cfg::B_INFOFREE + us));   // list and record of this unit are no longer read
      // ---- epilogue of the unit: O / l -> bf16 -> per-warp staging -> 16-byte stores; LSE ----
      if (n_done > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_ODONE + s), (uint32_t)(n_tot - 1) & 1u, wc));
        if (!ok) break;
        tc_fence_after();
      }
      const float m_fin = (m_run == neg_inf()) ? 0.f : m_run;
      float l_tot = l_run;
      if (p.sink) l_tot += fast_exp2(p.sink[hq] * kLog2e - m_fin);
      const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
      if (row < p.Sq)
        p.lse[((int64_t)b * p.Hq + hq) * p.Sq + row] =
            l_tot > 0.f ? (m_fin + log2f(l_tot)) * kLn2 : (cnt == 0 && p.sink ? p.sink[hq] : neg_inf());
      uint16_t* go = reinterpret_cast<uint16_t*>(p.o) + b * p.o_b + hq * p.o_h;
      const int rbase = ms + 128 * s + 32 * (warp & 3);
#pragma unroll
      for (int c = 0; c < DV / 32; ++c) {
        uint32_t orr[32];
        if (n_done > 0) {
          tmem_ld32(tO + 32 * c, orr);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int x = 0; x < 32; ++x) orr[x] = 0u;
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 v;
          v.x = pack2<IS_BF16>(__uint_as_float(orr[8 * q4 + 0]) * inv, __uint_as_float(orr[8 * q4 + 1]) * inv);
          v.y = pack2<IS_BF16>(__uint_as_float(orr[8 * q4 + 2]) * inv, __uint_as_float(orr[8 * q4 + 3]) * inv);
          v.z = pack2<IS_BF16>(__uint_as_float(orr[8 * q4 + 4]) * inv, __uint_as_float(orr[8 * q4 + 5]) * inv);
          v.w = pack2<IS_BF16>(__uint_as_float(orr[8 * q4 + 6]) * inv, __uint_as_float(orr[8 * q4 + 7]) * inv);
          *reinterpret_cast<uint4*>(stg + lane * 64 + ((q4 ^ ((lane >> 1) & 3)) << 4)) = v;
        }
        __syncwarp();
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const int rr = 8 * x + (lane >> 2), piece = lane & 3;
          const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 64 + ((piece ^ ((rr >> 1) & 3)) << 4));
          if (rbase + rr < p.Sq)
            *reinterpret_cast<uint4*>(go + (int64_t)(rbase + rr) * p.o_s + 32 * c + 8 * piece) = v;
        }
        __syncwarp();
      }
      tc_fence_before();   // the O reads above are ordered before this warpgroup's next arrival on PFULL
    }
  } else {
    setmaxnreg_dec<64>();
    if (warp == 10) {
      // =========================== scheduler + list builder ===========================
      int32_t* stage = reinterpret_cast<int32_t*>(smem + Cfg::OFF_STAGE);
      bool ok = true;
      for (int j = 0; ok; ++j) {
        const int us = j & 1;
        if (j >= 2) {
          // the record and list of unit j-2 must have been released by every role
          if (lane == 0) ok = mbar_wait_idle(bar(Cfg::B_INFOFREE + us), (uint32_t)((j >> 1) - 1) & 1u, wc);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        if (j >= 1) {
          // a unit is claimed late, when the current one is nearly through
          if (lane == 0) ok = mbar_wait_idle(bar(Cfg::B_FETCHGO), (uint32_t)(j - 1) & 1u, wc);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        int L = 0;
        if (lane == 0) L = atomicAdd(sched, 1);
        L = __shfl_sync(0xffffffffu, L, 0);
        if (L >= n_table) {
          if (lane == 0) {
            infos[us * 8 + 3] = -1; infos[us * 8 + 5] = 0;
            mbar_arrive(bar(Cfg::B_COORD + us)); mbar_arrive(bar(Cfg::B_INFOREADY + us));
          }
          break;
        }
        const int2 ent = __ldg(reinterpret_cast<const int2*>(table) + L);
        const int ms = ent.x * 256, hq = ent.y % p.Hq, b = ent.y / p.Hq;
        const int bh_mask = md.ncols ? ((md.mask_B == 1 ? 0 : b) * md.Hm + hq / (p.Hq / md.Hm)) : 0;
        if (lane == 0) {
          // coordinates first: the producer requests the Q tiles while the list is being built
          infos[us * 8 + 0] = b; infos[us * 8 + 1] = hq; infos[us * 8 + 2] = ms; infos[us * 8 + 4] = bh_mask;
          infos[us * 8 + 5] = 1;
          mbar_arrive(bar(Cfg::B_COORD + us));
        }
        // surviving K tiles, right to left, with the flags of both sub-tiles
        uint32_t* list = lists + us * Cfg::LIST_MAX;
        const int nb = (p.Sk + 127) / 128;
        const int me_tile = min(ms + 256, p.Sq);
        int n_hi = nb;
        if (md.causal) n_hi = max(0, min(nb, (me_tile + off + 127) / 128));
        int cnt = 0, c0 = 0, c1 = 0;
        for (int t_hi = n_hi; t_hi > 0;) {
          const int t_lo = (t_hi - 1) & ~(Cfg::STAGE_TILES - 1);
          const MaskDesc mst = stage_minmax(md, bh_mask, t_lo, t_hi, stage, Cfg::STAGE_TILES, lane);
          for (int base = t_hi - 1; base >= t_lo; base -= 32) {
            const int n = base - lane;
            uint32_t f0 = 0, f1 = 0;
            if (n >= t_lo) {
              f0 = tile_flags(mst, 0, n, ms, min(ms + 128, p.Sq), 128);
              if (ms + 128 < p.Sq) f1 = tile_flags(mst, 0, n, ms + 128, min(ms + 256, p.Sq), 128);
            }
            const bool keep = (f0 | f1) != 0;
            const uint32_t bal = __ballot_sync(0xffffffffu, keep);
            const int pos = cnt + __popc(bal & ((1u << lane) - 1u));
            if (keep && pos < Cfg::LIST_MAX) list[pos] = (uint32_t)n | (f0 << 16) | (f1 << 20);
            cnt += __popc(bal);
            c0 += __popc(__ballot_sync(0xffffffffu, f0 != 0));
            c1 += __popc(__ballot_sync(0xffffffffu, f1 != 0));
          }
          __syncwarp();
          t_hi = t_lo;
        }
        __syncwarp();
        if (lane == 0) {
          infos[us * 8 + 3] = min(cnt, Cfg::LIST_MAX); infos[us * 8 + 6] = c0; infos[us * 8 + 7] = c1;
          mbar_arrive(bar(Cfg::B_INFOREADY + us));   // release: the list and the record are visible to the waiters
        }
      }
    } else if (warp == 8) {
      // =========================== TMA / bounds producer ===========================
      int nbnd = 0, kb = 0;                        // bounds slots / ring positions over the life of the CTA
      int jq = -1;                                 // last unit whose Q tiles were requested
      bool ok = true;
      for (int j = 0; ok; ++j) {
        const int us = j & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_COORD + us), (uint32_t)(j >> 1) & 1u, wc));
        if (!ok) break;
        if (infos[us * 8 + 5] == 0) break;
        const int b = infos[us * 8 + 0], hq = infos[us * 8 + 1], ms = infos[us * 8 + 2], bh_mask = infos[us * 8 + 4];
        const int hk = hq / (p.Hq / p.Hkv);
        const uint32_t* list = lists + us * Cfg::LIST_MAX;
        // Q tiles: the buffers are free once every S = Q K^T of the previous unit has completed and its
        // own loads have landed
        if (j > 0) {
          if (lane == 0) {
            ok = mbar_wait(bar(Cfg::B_QFREE), (uint32_t)(j - 1) & 1u, wc);
            ok = ok && mbar_wait(bar(Cfg::B_QFULL + 0), (uint32_t)(j - 1) & 1u, wc);
            ok = ok && mbar_wait(bar(Cfg::B_QFULL + 1), (uint32_t)(j - 1) & 1u, wc);
          }
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        if (elect_one()) {
          for (int s = 0; s < 2; ++s) {
            mbar_arrive_expect_tx(bar(Cfg::B_QFULL + s), Cfg::Q_BYTES);
            for (int dc = 0; dc < D / 64; ++dc)
              tma_load_4d(sQ + s * Cfg::Q_BYTES + dc * Cfg::SUB, &tm_q, bar(Cfg::B_QFULL + s), dc * 64, hq,
                          ms + 128 * s, b);
          }
        }
        jq = j;
        // ... and the K/V tiles once the list is there
        ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_INFOREADY + us), (uint32_t)(j >> 1) & 1u, wc));
        if (!ok) break;
        const int cnt = infos[us * 8 + 3];
        const int i_go = max(0, cnt - Cfg::FETCH_AHEAD);
        if (cnt == 0 && lane == 0) mbar_arrive(bar(Cfg::B_FETCHGO));
        for (int i = 0; i < cnt && ok; ++i) {
          if (i == i_go && lane == 0) mbar_arrive(bar(Cfg::B_FETCHGO));   // the scheduler may claim the next unit
          const uint32_t e = list[i];
          const int j0 = (int)(e & 0xFFFFu) * 128;
          if (elect_one()) {
            for (int kv = 0; kv < 2 && ok; ++kv) {
              const int k = kb + 2 * i + kv, slot = k % Cfg::NSTAGE;
              const uint32_t par = ((uint32_t)(k / Cfg::NSTAGE) & 1u) ^ 1u;
              ok = mbar_wait(bar(Cfg::B_KVEMPTY + slot), par, wc);
              if (!ok) break;
              mbar_arrive_expect_tx(bar(Cfg::B_KVFULL + slot), Cfg::SLOT_BYTES);
              for (int dc = 0; dc < D / 64; ++dc)
                tma_load_4d(sKV + slot * Cfg::SLOT_BYTES + dc * Cfg::SUB, kv == 0 ? &tm_k : &tm_v,
                            bar(Cfg::B_KVFULL + slot), dc * 64, hk, j0, b);
            }
          }
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if ((((e >> 16) | (e >> 20)) & FM_TF_BOUNDS) != 0) {
            const int bslot = nbnd % Cfg::NBND;
            const uint32_t par = ((uint32_t)(nbnd / Cfg::NBND) & 1u) ^ 1u;
            ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_BNDEMPTY + bslot), par, wc));
            if (!ok) break;
            int* dst = reinterpret_cast<int*>(smem + Cfg::OFF_BND + bslot * Cfg::BND_BYTES);
            const int32_t* src = md.mask + ((size_t)bh_mask * p.Sk + j0) * md.ncols;
            stage_bounds(dst, src, 128, min(128, p.Sk - j0), md.ncols, lane);
            mbar_arrive(bar(Cfg::B_BNDFULL + bslot));
            ++nbnd;
          }
        }
        if (!ok) break;
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(Cfg::B_INFOFREE + us));
        kb += 2 * cnt;
      }
      // the Q loads of the last unit must have landed before the CTA leaves
      // (a sub-tile without work never waited for them)
      if (ok && jq >= 0 && lane == 0) {
        mbar_wait(bar(Cfg::B_QFULL + 0), (uint32_t)jq & 1u, wc);
        mbar_wait(bar(Cfg::B_QFULL + 1), (uint32_t)jq & 1u, wc);
      }
    } else if (warp == 9) {
      // =========================== UMMA issuer ===========================
      if (elect_one()) {
        constexpr uint32_t idesc_qk = make_idesc(IS_BF16, 128, 128, 0, 0);
        constexpr uint32_t idesc_pv = make_idesc(IS_BF16, 128, DV, 0, 1);
        int npv_tot[2] = {0, 0};                    // P V products per sub-tile over the life of the CTA
        bool ok = true;
        int kb = 0;
        // descriptors are built once; per MMA only a constant is added to the
        // 14-bit address field (all smem offsets are multiples of 16 bytes)
        const uint64_t dq0 = make_sdesc(sQ, 16, 1024);
        const uint64_t dk0 = make_sdesc(sKV, 16, 1024);
        const uint64_t dv0 = make_sdesc(sKV, Cfg::SUB, 1024);
        for (int j = 0; ok; ++j) {
          const int us = j & 1;
          ok = mbar_wait(bar(Cfg::B_INFOREADY + us), (uint32_t)(j >> 1) & 1u, wc);
          if (!ok) break;
          const int cnt = infos[us * 8 + 3];
          if (cnt < 0) break;
          const uint32_t* list = lists + us * Cfg::LIST_MAX;
          const int cnt_s[2] = {infos[us * 8 + 6], infos[us * 8 + 7]};
          int nqk[2] = {0, 0}, npv[2] = {0, 0};     // per unit
          bool q_ready[2] = {false, false};
          auto issue_qk = [&](auto sub, int i) {
            constexpr int s = decltype(sub)::value;   // compile-time: the per-sub-tile counters stay in registers
            const int k = kb + 2 * i, slot = k % Cfg::NSTAGE;
            ok = ok && mbar_wait(bar(Cfg::B_KVFULL + slot), (uint32_t)(k / Cfg::NSTAGE) & 1u, wc);
            if (ok && !q_ready[s]) { ok = mbar_wait(bar(Cfg::B_QFULL + s), (uint32_t)j & 1u, wc); q_ready[s] = true; }
            if (!ok) return;
            tc_fence_after();
            const uint64_t da = dq0 + (uint64_t)(s * (Cfg::Q_BYTES >> 4));
            const uint64_t db = dk0 + (uint64_t)(slot * (Cfg::SLOT_BYTES >> 4));
            const uint32_t dst = tmem + 128u * s;
            umma_ss_x8<(Cfg::SUB >> 4), (Cfg::SUB >> 4)>(dst, da, db, idesc_qk, 0u);
            tc_commit(bar(Cfg::B_SFULL + s));
            ++nqk[s];
            // after the last S = Q K^T of the unit (both sub-tiles) the Q tiles may be replaced
            if (nqk[0] == cnt_s[0] && nqk[1] == cnt_s[1]) tc_commit(bar(Cfg::B_QFREE));
          };
          auto issue_pv = [&](auto sub, int i) {
            constexpr int s = decltype(sub)::value;
            const int k = kb + 2 * i + 1, slot = k % Cfg::NSTAGE;
            ok = ok && mbar_wait(bar(Cfg::B_KVFULL + slot), (uint32_t)(k / Cfg::NSTAGE) & 1u, wc);
            ok = ok && mbar_wait(bar(Cfg::B_PFULL + s), (uint32_t)npv_tot[s] & 1u, wc);
            if (!ok) return;
            tc_fence_after();
            const uint64_t db = dv0 + (uint64_t)(slot * (Cfg::SLOT_BYTES >> 4));
            const uint32_t dst = tmem + 256u + 128u * s, src = tmem + 128u * s + 64u;
            const uint32_t acc0 = npv[s] > 0 ? 1u : 0u;
            umma_ts_xn<8>(dst, src, db, idesc_pv, acc0);
            tc_commit(bar(Cfg::B_ODONE + s));
            ++npv[s];
            ++npv_tot[s];
          };
          if (cnt == 0) {
            // nothing to compute: the Q tiles of this unit are not used
            mbar_arrive(bar(Cfg::B_QFREE));
            mbar_arrive(bar(Cfg::B_INFOFREE + us));
            continue;
          }
          {
            const uint32_t e = list[0];
            if ((e >> 16) & 0xFu) issue_qk(std::integral_constant<int, 0>{}, 0);
            if ((e >> 20) & 0xFu) issue_qk(std::integral_constant<int, 1>{}, 0);
            if (ok) tc_commit(bar(Cfg::B_KVEMPTY + (kb + 0) % Cfg::NSTAGE));
          }
          for (int i = 0; i < cnt && ok; ++i) {
            const uint32_t e = list[i];
            const uint32_t en = (i + 1 < cnt) ? list[i + 1] : 0u;
            if ((e >> 16) & 0xFu) issue_pv(std::integral_constant<int, 0>{}, i);
            if (ok && ((en >> 16) & 0xFu)) issue_qk(std::integral_constant<int, 0>{}, i + 1);
            if (ok && ((e >> 20) & 0xFu)) issue_pv(std::integral_constant<int, 1>{}, i);
            if (ok && ((en >> 20) & 0xFu)) issue_qk(std::integral_constant<int, 1>{}, i + 1);
            if (!ok) break;
            tc_commit(bar(Cfg::B_KVEMPTY + (kb + 2 * i + 1) % Cfg::NSTAGE));
            if (i + 1 < cnt) tc_commit(bar(Cfg::B_KVEMPTY + (kb + 2 * i + 2) % Cfg::NSTAGE));
          }
          if (ok) mbar_arrive(bar(Cfg::B_INFOFREE + us));   // the list of this unit is no longer read
          kb += 2 * cnt;
        }
      }
      __syncwarp();
    }
  }

  // =========================== teardown ===========================
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (misc[4] != 0) {
    // give copies and MMAs still in flight a bounded time to land before the
    // shared and tensor memory of this CTA are released
    const uint64_t t_end = global_timer_ns() + 200000ull;
    while (global_timer_ns() < t_end) __nanosleep(1000);
    if (tid == 0) atomicExch(&g_fwd_persist_status, FM_ERR_TIMEOUT);
  }
  if (warp == 9) tmem_dealloc(tmem, 512);
  if (tid == 0) {
    // the last CTA to leave rewinds the counters for the next launch that uses this table
    __threadfence();
    if (atomicAdd(sched + 1, 1) == (int)gridDim.x - 1) {
      atomicExch(sched, 0);
      atomicExch(sched + 1, 0);
    }
  }
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
bool fwd_sm100_persist_supported(const fm_attn_args* a) {
  return a->d == 128 && a->dv == 128 && (a->Sk + 127) / 128 <= FwdPersistCfg::LIST_MAX &&
         ((((uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v) & 15) == 0);
}

template <bool IS_BF16>
static int launch_fwd_sm100_persist(const AttnKParams& p, const fm_attn_args* a, cudaStream_t s) {
  using Cfg = FwdPersistCfg;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_bshd_tmap(&tq, a->q, a->dtype, a->B, a->Sq, a->Hq, a->d, a->q_stride[0], a->q_stride[1], a->q_stride[2], 128))) return rc;
  if ((rc = make_bshd_tmap(&tk, a->k, a->dtype, a->B, a->Sk, a->Hkv, a->d, a->k_stride[0], a->k_stride[1], a->k_stride[2], 128))) return rc;
  if ((rc = make_bshd_tmap(&tv, a->v, a->dtype, a->B, a->Sk, a->Hkv, a->dv, a->v_stride[0], a->v_stride[1], a->v_stride[2], 128))) return rc;
  auto kern = fwd_sm100_persist_kernel<IS_BF16>;
  FM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
  int dev = 0, n_sm = 0;
  FM_CUDA_TRY(cudaGetDevice(&dev));
  FM_CUDA_TRY(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
  kern<<<std::min(p.fwd_ncta, n_sm), Cfg::NTHREADS, Cfg::SMEM, s>>>(tq, tk, tv, p);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

int fwd_sm100_persist_launch(const AttnKParams& p, const fm_attn_args* a, cudaStream_t s) {
  return a->dtype == FM_DTYPE_BF16 ? launch_fwd_sm100_persist<true>(p, a, s) : launch_fwd_sm100_persist<false>(p, a, s);
}

int fwd_sm100_persist_status(int* out, bool reset) {
  int v = 0;
  FM_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_fwd_persist_status, sizeof(int)));
  if (reset && v != 0) {
    const int z = 0;
    FM_CUDA_TRY(cudaMemcpyToSymbol(g_fwd_persist_status, &z, sizeof(int)));
  }
  *out = v;
  return FM_OK;
}

}  // namespace fm

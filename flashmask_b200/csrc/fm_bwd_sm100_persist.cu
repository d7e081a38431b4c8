// Persistent variant of the tcgen05 backward kernels (d = dv = 128), used when the caller
// supplies launch tables (sparse masks).  Same two modes, work items, tensor-memory layout and
// item arithmetic as fm_bwd_sm100.cu; what differs is the control flow around a work unit:
//
//   * one CTA per SM walks the launch table through a global counter (units are claimed late,
//     when the current unit is nearly through, so a CTA in a long unit sits on no work);
//   * the scheduler warp fetches the next unit, builds its item list and publishes its
//     coordinates while the current unit is in its main loop; the producer requests the
//     stationary tiles of the next unit as soon as the score GEMMs of the current one are done;
//   * a separate epilogue warpgroup drains the accumulators (TMEM -> registers -> a small
//     per-warp staging area -> 16-byte global stores), so the compute warpgroups go straight
//     from the last item of a unit to the first item of the next one.
//
// Warp roles: 0-3 / 4-7 compute warpgroups, 8 TMA producer, 9 UMMA issuer (owns TMEM),
// 10 scheduler + list builder, 11 idle, 12-15 epilogue.  All waits are bounded.
#include <algorithm>

#include "fm_attn_params.cuh"
#include "fm_sm100.cuh"

namespace fm {

using namespace sm100;

__device__ int g_bwd_persist_status = 0;

constexpr int MODE_DKDV = 0, MODE_DQ = 1;   // as in fm_bwd_sm100.cu

#ifdef FM_TRACE
// Debug build only: timeline of CTA (0,0,0); every tracing thread appends
// (event, item, SM clock) triples to its own lane of the buffer with plain stores.
__device__ int g_ptrace[4 * 3 * 2048];
__device__ __forceinline__ void ptrace_ev(int role, int& n, int ev, int k) {
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && n < 2048) {
    int* t = g_ptrace + (role * 2048 + n) * 3;
    t[0] = ev; t[1] = k; t[2] = (int)clock64();
    ++n;
  }
}
// Phase stamps of the CTAs (x < 64, y = 0, z = 0): one clock value per phase boundary.
__device__ long long g_pprof[2 * 64 * 16];   // [mode][cta][stamp]
// Per-unit log of the UMMA issuer of CTAs 0..7: info ready, stationary ready, first / last accumulate issued, items.
__device__ long long g_unitlog[2 * 8 * 32 * 8];
#define ULOG(j, f, v) do { if (blockIdx.x < 8 && blockIdx.y == 0 && blockIdx.z == 0 && (j) < 32) g_unitlog[((MODE * 8 + blockIdx.x) * 32 + (j)) * 8 + (f)] = (v); } while (0)
#define TRACE_DECL int trace_n = 0;
#define TRACE(role, ev, k) ptrace_ev(role, trace_n, ev, k)
#define PROF(slot) do { if (blockIdx.y == 0 && blockIdx.z == 0 && blockIdx.x < 64) g_pprof[(MODE * 64 + blockIdx.x) * 16 + (slot)] = clock64(); } while (0)
#define PROF_VAL(slot, v) do { if (blockIdx.y == 0 && blockIdx.z == 0 && blockIdx.x < 64) g_pprof[(MODE * 64 + blockIdx.x) * 16 + (slot)] = (v); } while (0)
#else
#define TRACE_DECL
#define TRACE(role, ev, k)
#define PROF(slot)
#define PROF_VAL(slot, v)
#define ULOG(j, f, v)
#endif

struct BwdPersistCfg {
  static constexpr int NSLOT = 4, LIST_MAX = 2048, NTHREADS = 512;
  static constexpr int TILE_BYTES = 128 * 128 * 2;     // 128 rows x 128 cols bf16
  static constexpr int SUB128 = 128 * 128;             // 128-row x 64-col sub-tile (bytes)
  static constexpr int SUB64 = 64 * 128;               // 64-row x 64-col sub-tile (bytes)
  static constexpr int HALF_BYTES = 2 * SUB64;         // one operand of a half tile
  static constexpr int SLOT_BYTES = 2 * HALF_BYTES;    // both operands
  static constexpr int AUX_BYTES = 1024;
  static constexpr int STAGE_TILES = 128;              // K tiles whose reductions are staged at a time
  static constexpr int OFF_STAT = 0;
  static constexpr int OFF_RING = OFF_STAT + 2 * TILE_BYTES;
  static constexpr int OFF_AUX = OFF_RING + NSLOT * SLOT_BYTES;
  static constexpr int OFF_LIST = OFF_AUX + NSLOT * AUX_BYTES;          // two lists of 16-bit entries: units alternate
  static constexpr int OFF_STAGE = OFF_LIST + 2 * LIST_MAX * 2;
  static constexpr int EPI_BYTES = 32 * 64;                             // per epilogue warp: 32 rows x 32 bf16 columns
  static constexpr int OFF_EPI = OFF_STAGE + 8 * STAGE_TILES * 4;
  static constexpr int OFF_INFO = OFF_EPI + 4 * EPI_BYTES;              // two unit records of 8 ints
  static constexpr int OFF_BAR = OFF_INFO + 2 * 8 * 4;
  static constexpr int OFF_MISC = OFF_BAR + 32 * 8;
  static constexpr int SMEM = OFF_MISC + 64 + 1024;
  // item-level barriers (phases follow the CTA-wide item counter) ...
  static constexpr int B_RFULL = 0, B_REMPTY = NSLOT, B_GFULL = 2 * NSLOT, B_TFULL = B_GFULL + 2,
                       B_GREAD = B_TFULL + 2;
  // ... and unit-level ones (phases follow the unit counter of the CTA)
  static constexpr int B_STAT = B_GREAD + 2, B_STATFREE = B_STAT + 1, B_ACC = B_STATFREE + 1,
                       B_ACCFREE = B_ACC + 1, B_INFOREADY = B_ACCFREE + 1, B_INFOFREE = B_INFOREADY + 2,
                       B_COORD = B_INFOFREE + 2, B_FETCHGO = B_COORD + 2, B_COUNT = B_FETCHGO + 1;
  static constexpr int FETCH_AHEAD = 16;   // items left in a unit when the next one is claimed
  static_assert(B_COUNT <= 32, "barrier storage");
  static_assert(SMEM > 120 * 1024 && SMEM <= 227 * 1024, "one CTA per SM (512 TMEM columns)");
};

__device__ __forceinline__ float pbneg_inf() { return __int_as_float(0xff800000); }

__device__ __forceinline__ void pbulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// A CTA works through a sequence of UNITS (one stationary 128-row tile each: a K/V tile in
// MODE_DKDV, a Q/dO tile in MODE_DQ).  Without a launch table it owns exactly the unit its
// block index names.  With one (p.*_order + p.*_sched) the launch is persistent: units are
// fetched from the table through a global counter, and while one unit is in its main loop
// the scheduler warp already fetches the next one and builds its work list, so that entry and
// list build disappear from the critical path of short units.
// D: width the head dims are computed at (64 when both fit, else 128); the 64-column variant keeps
// the shared-memory layout and leaves the second 64-column sub-tile of every operand unloaded.
template <int MODE, bool IS_BF16, int D>
__global__ void __launch_bounds__(512, 1)
bwd_sm100_persist_kernel(const __grid_constant__ CUtensorMap tm_stat1, const __grid_constant__ CUtensorMap tm_stat2,
                 const __grid_constant__ CUtensorMap tm_str1, const __grid_constant__ CUtensorMap tm_str2,
                 const AttnKParams p) {
  using Cfg = BwdPersistCfg;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sStat = sbase + Cfg::OFF_STAT, sRing = sbase + Cfg::OFF_RING;
  uint16_t* lists = reinterpret_cast<uint16_t*>(smem + Cfg::OFF_LIST);   // entry: item index | tile flags << 12
  volatile int* infos = reinterpret_cast<volatile int*>(smem + Cfg::OFF_INFO);   // [2][8]: b, head, row0, cnt, bh_mask, valid
  const uint32_t bars = sbase + Cfg::OFF_BAR;
  volatile int* misc = reinterpret_cast<volatile int*>(smem + Cfg::OFF_MISC);  // [0] tmem, [4] abort
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };

  const int tid = threadIdx.x;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int lane = tid & 31;
  TRACE_DECL
  if (tid == 0) PROF(0);
  // descriptor fetches start before anything else: the first loads wait on them
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&tm_stat1); tma_prefetch_desc(&tm_stat2);
    tma_prefetch_desc(&tm_str1); tma_prefetch_desc(&tm_str2);
  }
  const MaskDesc& md = p.md;
  const int off = p.Sk - p.Sq;
  const int G = p.Hq / p.Hkv;
  const int n_heads = (MODE == MODE_DKDV) ? G : 1;
  const int32_t* table = (MODE == MODE_DKDV) ? p.dkdv_order : p.dq_order;
  int* sched = (MODE == MODE_DKDV) ? p.dkdv_sched : p.dq_sched;     // [0] next table entry, [1] CTAs done
  const int n_table = (MODE == MODE_DKDV) ? p.dkdv_ncta : p.dq_ncta;

  if (tid == 0) misc[4] = 0;
  if (warp == 8 && lane == 0) {
    for (int i = 0; i < Cfg::NSLOT; ++i) {
      mbar_init(bar(Cfg::B_RFULL + i), MODE == MODE_DQ ? 33 : 1);
      mbar_init(bar(Cfg::B_REMPTY + i), 1);
    }
    for (int h = 0; h < 2; ++h) {
      mbar_init(bar(Cfg::B_GFULL + h), 1); mbar_init(bar(Cfg::B_TFULL + h), 4); mbar_init(bar(Cfg::B_GREAD + h), 4);
      mbar_init(bar(Cfg::B_INFOREADY + h), 1); mbar_init(bar(Cfg::B_INFOFREE + h), 14);
      mbar_init(bar(Cfg::B_COORD + h), 1);
    }
    mbar_init(bar(Cfg::B_FETCHGO), 1);
    mbar_init(bar(Cfg::B_STAT), 1); mbar_init(bar(Cfg::B_STATFREE), 1);
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
  if (tid == 0) PROF(1);
  // TMEM columns: score buffers G1_p at 64p, G2_p at 128+64p.
  //   DKDV: P^T_p / dS^T_p (bf16) overlay G2_p at +0 / +32; dV at 256, dK at 384.  G1_p is dead as soon as
  //         its warpgroup has read it, so S^T of item k+2 is issued before item k is finished.
  //   DQ:   dS (bf16) has four own 32-column buffers at 256 (index 2*((k/2)%2) + p), dQ at 384.
  constexpr uint32_t C_G1 = 0, C_G2 = 128, C_T = 256;
  constexpr uint32_t C_ACC1 = (MODE == MODE_DKDV) ? 256 : 384, C_ACC2 = 384;

  // 512 threads start with 128 registers each; the compute warpgroups take what the others give up
  if (warp < 8) setmaxnreg_inc<176>();
  else if (warp < 12) setmaxnreg_dec<80>();
  else setmaxnreg_dec<80>();

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
      // ---- next unit ----
      int b, head, row0;
      bool have;
      if (table) {
        int L = 0;
        if (lane == 0) L = atomicAdd(sched, 1);
        L = __shfl_sync(0xffffffffu, L, 0);
        have = L < n_table;
        int2 e = make_int2(0, 0);
        if (have) e = __ldg(reinterpret_cast<const int2*>(table) + L);
        const int heads = (MODE == MODE_DKDV) ? p.Hkv : p.Hq;
        row0 = e.x * 128; head = e.y % heads; b = e.y / heads;
      } else {
        have = !own_unit_taken;
        own_unit_taken = true;
        if (MODE == MODE_DKDV) { b = blockIdx.z; head = blockIdx.y; row0 = blockIdx.x * 128; }
        else { b = blockIdx.z; head = blockIdx.y; row0 = ((p.Sq + 127) / 128 - 1 - (int)blockIdx.x) * 128; }
      }
      if (!have) {
        if (lane == 0) {
          infos[s * 8 + 3] = -1; infos[s * 8 + 5] = 0;
          mbar_arrive(bar(Cfg::B_COORD + s)); mbar_arrive(bar(Cfg::B_INFOREADY + s));
        }
        break;
      }
      const int hq0 = (MODE == MODE_DKDV) ? head * G : head;
      const int bh_mask = md.ncols ? ((md.mask_B == 1 ? 0 : b) * md.Hm + hq0 / (p.Hq / md.Hm)) : 0;
      if (lane == 0) {
        // coordinates first: the producer requests the stationary tiles while the list is being built
        infos[s * 8 + 0] = b; infos[s * 8 + 1] = head; infos[s * 8 + 2] = row0; infos[s * 8 + 4] = bh_mask;
        infos[s * 8 + 5] = 1;
        mbar_arrive(bar(Cfg::B_COORD + s));
      }
      uint16_t* list = lists + s * Cfg::LIST_MAX;
      int cnt = 0;
      if (MODE == MODE_DKDV) {
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
      } else {
        // 64-key half tiles visible to query tile [row0, row0+128), right to left
        const int me = min(row0 + 128, p.Sq);
        const int n_half = (p.Sk + 63) / 64;
        int hi = n_half;
        if (md.causal) hi = max(0, min(n_half, (me + off + 63) / 64));
        for (int t_hi = (hi + 1) >> 1; t_hi > 0;) {
          const int t_lo = (t_hi - 1) & ~(Cfg::STAGE_TILES - 1);
          const MaskDesc mst = stage_minmax(md, bh_mask, t_lo, t_hi, stage, Cfg::STAGE_TILES, lane);
          for (int base = min(hi, 2 * t_hi) - 1; base >= 2 * t_lo; base -= 32) {
            const int idx = base - lane;
            uint32_t f = 0;
            if (idx >= 2 * t_lo) {
              f = tile_flags(mst, 0, idx >> 1, row0, me, 128);
              if (md.causal && idx * 64 > me - 1 + off) f = 0;
            }
            const uint32_t bal = __ballot_sync(0xffffffffu, f != 0);
            const int pos = cnt + __popc(bal & ((1u << lane) - 1u));
            if (f && pos < Cfg::LIST_MAX) list[pos] = (uint16_t)((uint32_t)idx | (f << 12));
            cnt += __popc(bal);
          }
          __syncwarp();
          t_hi = t_lo;
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
    const int r = tid & 127;                     // TMEM lane
    const uint32_t lane_field = (uint32_t)((warp & 3) * 32) << 16;
    const float scale_log2 = p.scale_log2;
    bool ok = true;
    int kb = 0;                                  // items of earlier units
    for (int j = 0; ok; ++j) {
      const int s = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_INFOREADY + s), (uint32_t)(j >> 1) & 1u, wc));
      if (!ok) break;
      const int cnt = infos[s * 8 + 3];
      if (cnt < 0) break;
      const int b = infos[s * 8 + 0], head = infos[s * 8 + 1], row0 = infos[s * 8 + 2], bh_mask = infos[s * 8 + 4];
      const int hk = (MODE == MODE_DKDV) ? head : head / G;
      const int hq0 = (MODE == MODE_DKDV) ? head * G : head;
      const uint16_t* list = lists + s * Cfg::LIST_MAX;
      const int K_items = cnt * n_heads;
      if (cnt == 0) {
        // nothing visible: the gradients of this unit are zero
        if (MODE == MODE_DKDV) {
          uint16_t* gk = reinterpret_cast<uint16_t*>(p.dk) + b * p.dk_b + (int64_t)row0 * p.dk_s + hk * p.dk_h;
          uint16_t* gv = reinterpret_cast<uint16_t*>(p.dv) + b * p.dv_b + (int64_t)row0 * p.dv_s + hk * p.dv_h;
          for (int x = tid; x < 128 * 16; x += 256) {
            const int rr = x >> 4, cc = x & 15;
            if (row0 + rr < p.Sk) {
              if (cc * 8 < p.d) *reinterpret_cast<uint4*>(gk + (int64_t)rr * p.dk_s + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
              if (cc * 8 < p.dv_dim) *reinterpret_cast<uint4*>(gv + (int64_t)rr * p.dv_s + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
            }
          }
        } else {
          uint16_t* gq = reinterpret_cast<uint16_t*>(p.dq) + b * p.dq_b + (int64_t)row0 * p.dq_s + hq0 * p.dq_h;
          for (int x = tid; x < 128 * 16; x += 256) {
            const int rr = x >> 4, cc = x & 15;
            if (row0 + rr < p.Sq && cc * 8 < p.d)
              *reinterpret_cast<uint4*>(gq + (int64_t)rr * p.dq_s + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(Cfg::B_INFOFREE + s));
        continue;
      }

      // per-lane constants of the unit
      int lts = INT_MAX, lte = INT_MAX, uts = 0, ute = 0;   // DKDV: bounds of key row0 + r
      float lse2_row = 0.f, dps_row = 0.f;                   // DQ: statistics of query row0 + r
      if (MODE == MODE_DKDV) {
        const int jj = row0 + r;
        if (jj >= p.Sk) { lts = 0; lte = INT_MAX; }
        else if (md.ncols) {
          const Bounds4 bd = load_bounds(md, md.mask + ((size_t)bh_mask * p.Sk + jj) * md.ncols);
          lts = bd.lts; lte = bd.lte; uts = bd.uts; ute = bd.ute;
        }
      } else {
        const int i = row0 + r;
        if (i < p.Sq) {
          lse2_row = p.lse_log2[((int64_t)b * p.Hq + hq0) * p.Sq_r + i];
          dps_row = p.dpsum[((int64_t)b * p.Hq + hq0) * p.Sq_r + i];
        }
      }

      // this warpgroup serves the items whose CTA-wide index kk = kb + k has parity wg
      for (int k = (wg - kb) & 1; k < K_items && ok; k += 2) {
        const int kk = kb + k;
        const int pz = wg;
        const uint32_t tG1 = tmem + lane_field + C_G1 + 64u * pz;
        const uint32_t tG2 = tmem + lane_field + C_G2 + 64u * pz;
        const uint32_t e = list[k % cnt];
        const int idx = (int)(e & 0xFFFu);
        const uint32_t flags = e >> 12;
        const int slot = kk % Cfg::NSLOT;
        ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_RFULL + slot), (uint32_t)(kk / Cfg::NSLOT) & 1u, wc));
        if (!ok) break;
        if (r == 0) TRACE(2 + pz, 10, k);   // ring slot observed full
        ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_GFULL + pz), (uint32_t)(kk >> 1) & 1u, wc));
        if (!ok) break;
        if (r == 0) TRACE(2 + pz, 12, k);   // scores observed ready
        tc_fence_after();
        const uint8_t* aux = smem + Cfg::OFF_AUX + slot * Cfg::AUX_BYTES;
        const uint32_t NEG = 0xff800000u;
        // 64 score columns; once they are in registers the score buffers may be
        // overwritten by the next item of this parity (signalled through g_read)
        uint32_t sr[2][32], dr[2][32];
        tmem_ld32(tG1, sr[0]); tmem_ld32(tG2, dr[0]);
        tmem_ld32(tG1 + 32, sr[1]); tmem_ld32(tG2 + 32, dr[1]);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(Cfg::B_GREAD + pz));
        const uint32_t tT = (MODE == MODE_DKDV)
                                ? tG2
                                : tmem + lane_field + C_T + 32u * (uint32_t)((((kk >> 1) & 1) << 1) + pz);
  #include "fm_bwd_sm100_item.inc"
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(Cfg::B_TFULL + pz));
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
      ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_COORD + s), (uint32_t)(j >> 1) & 1u, wc));
      if (!ok) break;
      if (infos[s * 8 + 5] == 0) break;
      const int b = infos[s * 8 + 0], head = infos[s * 8 + 1], row0 = infos[s * 8 + 2], bh_mask = infos[s * 8 + 4];
      const int hk = (MODE == MODE_DKDV) ? head : head / G;
      const int hq0 = (MODE == MODE_DKDV) ? head * G : head;
      const uint16_t* list = lists + s * Cfg::LIST_MAX;
      // stationary tiles: the buffer is free once every score GEMM of the previous unit has completed
      if (j > 0) {
        if (lane == 0) ok = mbar_wait(bar(Cfg::B_STATFREE), (uint32_t)(j - 1) & 1u, wc);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }
      if (elect_one()) {
        mbar_arrive_expect_tx(bar(Cfg::B_STAT), 2 * Cfg::TILE_BYTES * D / 128);
        for (int dc = 0; dc < D / 64; ++dc) {
          tma_load_4d(sStat + dc * Cfg::SUB128, &tm_stat1, bar(Cfg::B_STAT), dc * 64, head, row0, b);
          tma_load_4d(sStat + Cfg::TILE_BYTES + dc * Cfg::SUB128, &tm_stat2, bar(Cfg::B_STAT), dc * 64, head, row0, b);
        }
      }
      // ... and the items once the list is there
      ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_INFOREADY + s), (uint32_t)(j >> 1) & 1u, wc));
      if (!ok) break;
      const int cnt = infos[s * 8 + 3];
      const int K_items = cnt * n_heads;
      const int k_go = max(0, K_items - Cfg::FETCH_AHEAD);
      if (K_items == 0 && lane == 0) mbar_arrive(bar(Cfg::B_FETCHGO));
      for (int k = 0; k < K_items && ok; ++k) {
        if (k == k_go && lane == 0) mbar_arrive(bar(Cfg::B_FETCHGO));   // the scheduler may claim the next unit
        const int kk = kb + k;
        const uint32_t e = list[k % cnt];
        const int idx = (int)(e & 0xFFFu);
        const uint32_t flags = e >> 12;
        const int slot = kk % Cfg::NSLOT;
        const uint32_t par = ((uint32_t)(kk / Cfg::NSLOT) & 1u) ^ 1u;
        const int hstr = (MODE == MODE_DKDV) ? hq0 + k / cnt : hk;
        if (MODE == MODE_DQ) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_REMPTY + slot), par, wc));
        } else {
          if (lane == 0) ok = mbar_wait(bar(Cfg::B_REMPTY + slot), par, wc);
          ok = __all_sync(0xffffffffu, ok);
        }
        if (!ok) break;
        if (lane == 0) TRACE(0, 1, k);    // slot observed empty
        if (elect_one()) {
          const uint32_t dst = sRing + slot * Cfg::SLOT_BYTES;
          const uint32_t fb = bar(Cfg::B_RFULL + slot);
          mbar_arrive_expect_tx(fb, Cfg::SLOT_BYTES * D / 128 + (MODE == MODE_DKDV ? 512 : 0));
          for (int dc = 0; dc < D / 64; ++dc) {
            tma_load_4d(dst + dc * Cfg::SUB64, &tm_str1, fb, dc * 64, hstr, idx * 64, b);
            tma_load_4d(dst + Cfg::HALF_BYTES + dc * Cfg::SUB64, &tm_str2, fb, dc * 64, hstr, idx * 64, b);
          }
          if (MODE == MODE_DKDV) {
            const int64_t at = ((int64_t)b * p.Hq + hstr) * p.Sq_r + idx * 64;
            const uint32_t ax = sbase + Cfg::OFF_AUX + slot * Cfg::AUX_BYTES;
            pbulk_copy_g2s(ax, p.lse_log2 + at, 256, fb);
            pbulk_copy_g2s(ax + 256, p.dpsum + at, 256, fb);
          }
        }
        if (MODE == MODE_DQ) {
          if (flags & FM_TF_BOUNDS) {
            int* dst = reinterpret_cast<int*>(smem + Cfg::OFF_AUX + slot * Cfg::AUX_BYTES);
            const int jh0 = idx * 64;
            const int32_t* src = md.mask + ((size_t)bh_mask * p.Sk + jh0) * md.ncols;
            stage_bounds(dst, src, 64, min(64, p.Sk - jh0), md.ncols, lane);
          }
          mbar_arrive(bar(Cfg::B_RFULL + slot));
        }
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(Cfg::B_INFOFREE + s));
      kb += K_items;
    }
  } else if (warp == 9) {
    // =========================== UMMA issuer ===========================
    if (elect_one()) {
      constexpr uint32_t idesc_g = make_idesc(IS_BF16, 128, 64, 0, 0);
      constexpr uint32_t idesc_acc = make_idesc(IS_BF16, 128, D, 0, 1);
      // descriptors are built once; per MMA only a constant is added to the
      // 14-bit address field (all smem offsets are multiples of 16 bytes)
      const uint64_t dA1 = make_sdesc(sStat, 16, 1024);
      const uint64_t dA2 = make_sdesc(sStat + Cfg::TILE_BYTES, 16, 1024);
      const uint64_t dRk = make_sdesc(sRing, 16, 1024);            // K-major view of a ring slot
      const uint64_t dRm = make_sdesc(sRing, Cfg::SUB64, 1024);    // MN-major view of a ring slot
      bool ok = true;
      int kb = 0, ju = 0;
      // part 1 of the score GEMMs of item kk: the first one (S or S^T) runs as soon as the warpgroup
      // of this parity has READ item kk-2 out of the score buffers
      auto issue_g_early = [&](int kk) {
        const int slot = kk % Cfg::NSLOT, pz = kk & 1;
        if (kk >= 2) ok = ok && mbar_wait(bar(Cfg::B_GREAD + pz), (uint32_t)((kk - 2) >> 1) & 1u, wc);
        TRACE(1, 20, kk);                   // about to wait for the ring slot
        ok = ok && mbar_wait(bar(Cfg::B_RFULL + slot), (uint32_t)(kk / Cfg::NSLOT) & 1u, wc);
        if (!ok) return;
        TRACE(1, 21, kk);                   // ring slot full
        tc_fence_after();
        const uint64_t db1 = dRk + (uint64_t)(slot * (Cfg::SLOT_BYTES >> 4));
        if constexpr (D == 128) umma_ss_x8<(Cfg::SUB128 >> 4), (Cfg::SUB64 >> 4)>(tmem + C_G1 + 64u * pz, dA1, db1, idesc_g, 0u);
        else umma_ss_x4(tmem + C_G1 + 64u * pz, dA1, db1, idesc_g, 0u);
        TRACE(1, 22, kk);                   // G issued
      };
      // part 2: the second score GEMM (dP or dP^T) follows the accumulation MMAs of item kk-2
      // (in DKDV mode it overwrites the buffer that held that item's P^T / dS^T)
      auto issue_g_late = [&](int kk) {
        const int slot = kk % Cfg::NSLOT, pz = kk & 1;
        const uint64_t db2 = dRk + (uint64_t)(slot * (Cfg::SLOT_BYTES >> 4) + (Cfg::HALF_BYTES >> 4));
        if constexpr (D == 128) umma_ss_x8<(Cfg::SUB128 >> 4), (Cfg::SUB64 >> 4)>(tmem + C_G2 + 64u * pz, dA2, db2, idesc_g, 0u);
        else umma_ss_x4(tmem + C_G2 + 64u * pz, dA2, db2, idesc_g, 0u);
        tc_commit(bar(Cfg::B_GFULL + pz));
      };
      for (int j = 0; ok; ++j) {
        const int s = j & 1;
        ULOG(j, 5, clock64());
        ok = mbar_wait(bar(Cfg::B_INFOREADY + s), (uint32_t)(j >> 1) & 1u, wc);
        if (!ok) break;
        ULOG(j, 0, clock64());
        const int cnt = infos[s * 8 + 3];
        if (cnt < 0) break;
        const int K_items = cnt * n_heads;
        mbar_arrive(bar(Cfg::B_INFOFREE + s));     // only the item count is needed here
        ok = mbar_wait(bar(Cfg::B_STAT), (uint32_t)j & 1u, wc);
        if (!ok) break;
        ULOG(j, 1, clock64()); ULOG(j, 4, (long long)K_items);
        if (K_items == 0) {
          // the stationary tiles of an empty unit have landed and are not used
          mbar_arrive(bar(Cfg::B_STATFREE));
          continue;
        }
        if (j == 0) { PROF(2); PROF_VAL(10, (long long)K_items); }
        issue_g_early(kb); if (ok) issue_g_late(kb);
        if (K_items > 1 && ok) { issue_g_early(kb + 1); if (ok) issue_g_late(kb + 1); }
        if (K_items <= 2 && ok) tc_commit(bar(Cfg::B_STATFREE));   // every score GEMM of the unit is issued
        for (int k = 0; k < K_items && ok; ++k) {
          const int kk = kb + k;
          const int slot = kk % Cfg::NSLOT, pz = kk & 1;
          if (k + 2 < K_items) {
            issue_g_early(kk + 2);
            if (!ok) break;
          }
          TRACE(1, 23, kk);                   // about to wait for T
          ok = mbar_wait(bar(Cfg::B_TFULL + pz), (uint32_t)(kk >> 1) & 1u, wc);
          if (!ok) break;
          TRACE(1, 24, kk);                   // T ready
          if (k == 0 && ju > 0) {
            // the accumulators still hold the previous unit until its epilogue has read them
            ok = mbar_wait(bar(Cfg::B_ACCFREE), (uint32_t)(ju - 1) & 1u, wc);
            if (!ok) break;
          }
          tc_fence_after();
          const uint64_t dm1 = dRm + (uint64_t)(slot * (Cfg::SLOT_BYTES >> 4));     // streamed operand 1
          const uint64_t dm2 = dm1 + (uint64_t)(Cfg::HALF_BYTES >> 4);               // streamed operand 2
          const uint32_t acc_on = k > 0 ? 1u : 0u;
          if (MODE == MODE_DKDV) {
            // dV += P^T dO (streamed operand 2), dK += dS^T Q (streamed operand 1)
            const uint32_t t1 = tmem + C_G2 + 64u * pz, t2 = t1 + 32u;
            umma_ts_xn<4>(tmem + C_ACC1, t1, dm2, idesc_acc, acc_on);
            umma_ts_xn<4>(tmem + C_ACC2, t2, dm1, idesc_acc, acc_on);
          } else {
            // dQ += dS K (streamed operand 1)
            const uint32_t t2 = tmem + C_T + 32u * (uint32_t)((((kk >> 1) & 1) << 1) + pz);
            umma_ts_xn<4>(tmem + C_ACC1, t2, dm1, idesc_acc, acc_on);
          }
          tc_commit(bar(Cfg::B_REMPTY + slot));
          TRACE(1, 25, kk);                   // ACC issued
          if (k == 0) ULOG(j, 2, clock64());
          if (k == K_items - 1) ULOG(j, 3, clock64());
          if (k + 2 < K_items) {
            issue_g_late(kk + 2);
            if (k + 3 == K_items) tc_commit(bar(Cfg::B_STATFREE));   // that was the unit's last score GEMM
          }
        }
        if (ok) tc_commit(bar(Cfg::B_ACC));
        if (j == 0) PROF(6);
        ++ju;
        kb += K_items;
      }
    }
    __syncwarp();
  } else if (warp >= 12) {
    // =========================== epilogue warpgroup ===========================
    // Warp 12+e drains TMEM lanes [32e, 32e+32): 32 columns at a time go through a 2 KB staging
    // area of its own (rows of 64 bytes, 16-byte pieces XOR-swizzled by row) so that one store
    // instruction writes 8 rows x 64 contiguous bytes.  The accumulators are released to the next
    // unit as soon as the last columns have been read.
    const int ew = warp - 12;
    const uint32_t lane_field = (uint32_t)(ew * 32) << 16;
    uint8_t* stg = smem + Cfg::OFF_EPI + ew * Cfg::EPI_BYTES;
    constexpr int N_OUT = (MODE == MODE_DKDV) ? 2 : 1;
    bool ok = true;
    int ju = 0;                                  // earlier units that had items (phases of the accumulator barriers)
    for (int j = 0; ok; ++j) {
      const int s = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait_idle(bar(Cfg::B_INFOREADY + s), (uint32_t)(j >> 1) & 1u, wc));
      if (!ok) break;
      const int cnt = infos[s * 8 + 3];
      if (cnt < 0) break;
      const int b = infos[s * 8 + 0], head = infos[s * 8 + 1], row0 = infos[s * 8 + 2];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(Cfg::B_INFOFREE + s));
      if (cnt == 0) continue;                    // the compute warpgroups write the zeros of an empty unit
      ok = __all_sync(0xffffffffu, mbar_wait_idle(bar(Cfg::B_ACC), (uint32_t)ju & 1u, wc));
      if (!ok) break;
      ++ju;
      tc_fence_after();
      const int rbase = row0 + 32 * ew;
      const int rlimit = (MODE == MODE_DKDV) ? p.Sk : p.Sq;
#pragma unroll
      for (int o = 0; o < N_OUT; ++o) {
        // DKDV: o = 0 dV, o = 1 dK (scaled); DQ: dQ (scaled)
        const uint32_t tA = tmem + lane_field + ((MODE == MODE_DKDV && o == 0) ? C_ACC1 : C_ACC2);
        const float mul = (MODE == MODE_DKDV && o == 0) ? 1.f : p.scale;
        const int width = (MODE == MODE_DKDV && o == 0) ? p.dv_dim : p.d;   // head dims below 128 end here
        uint16_t* gbase;
        int64_t ld;
        if (MODE == MODE_DKDV) {
          gbase = o == 0 ? reinterpret_cast<uint16_t*>(p.dv) + b * p.dv_b + head * p.dv_h
                         : reinterpret_cast<uint16_t*>(p.dk) + b * p.dk_b + head * p.dk_h;
          ld = o == 0 ? p.dv_s : p.dk_s;
        } else {
          gbase = reinterpret_cast<uint16_t*>(p.dq) + b * p.dq_b + head * p.dq_h;
          ld = p.dq_s;
        }
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t acc[32];
          tmem_ld32(tA + 32 * c, acc);
          tc_wait_ld();
          if (o == N_OUT - 1 && c == D / 32 - 1) {
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
            if (rbase + rr < rlimit && 32 * c + 8 * piece < width)
              *reinterpret_cast<uint4*>(gbase + (int64_t)(rbase + rr) * ld + 32 * c + 8 * piece) = v;
          }
          __syncwarp();
        }
      }
    }
  }

  // =========================== teardown ===========================
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (tid == 0) PROF(9);
  if (misc[4] != 0) {
    const uint64_t t_end = global_timer_ns() + 200000ull;
    while (global_timer_ns() < t_end) __nanosleep(1000);
    if (tid == 0) atomicExch(&g_bwd_persist_status, FM_ERR_TIMEOUT);
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

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
template <bool IS_BF16, int D>
static int launch_bwd_sm100_persist(const AttnKParams& p, const fm_attn_args* a, cudaStream_t s) {
  using Cfg = BwdPersistCfg;
  FM_REQUIRE((a->Sq + 63) / 64 <= Cfg::LIST_MAX && (a->Sk + 63) / 64 <= Cfg::LIST_MAX, FM_ERR_UNSUPPORTED,
             "backward: Sq=%d / Sk=%d exceed the %d rows this kernel variant indexes", a->Sq, a->Sk,
             Cfg::LIST_MAX * 64);
  CUtensorMap q128, do128, k128, v128, q64, do64, k64, v64;
  int rc;
#define FM_TMAP(out, ptr, S, H, D, st, rows)                                                          \
  if ((rc = make_bshd_tmap(&out, ptr, a->dtype, a->B, S, H, D, st[0], st[1], st[2], rows))) return rc;
  FM_TMAP(k128, a->k, a->Sk, a->Hkv, a->d, a->k_stride, 128)
  FM_TMAP(v128, a->v, a->Sk, a->Hkv, a->dv, a->v_stride, 128)
  FM_TMAP(q64, a->q, a->Sq, a->Hq, a->d, a->q_stride, 64)
  FM_TMAP(do64, a->d_o, a->Sq, a->Hq, a->dv, a->do_stride, 64)
  FM_TMAP(q128, a->q, a->Sq, a->Hq, a->d, a->q_stride, 128)
  FM_TMAP(do128, a->d_o, a->Sq, a->Hq, a->dv, a->do_stride, 128)
  FM_TMAP(k64, a->k, a->Sk, a->Hkv, a->d, a->k_stride, 64)
  FM_TMAP(v64, a->v, a->Sk, a->Hkv, a->dv, a->v_stride, 64)
#undef FM_TMAP
  auto k1 = bwd_sm100_persist_kernel<MODE_DKDV, IS_BF16, D>;
  auto k2 = bwd_sm100_persist_kernel<MODE_DQ, IS_BF16, D>;
  FM_CUDA_TRY(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
  FM_CUDA_TRY(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
  // with a launch table: one persistent CTA per SM (fewer when the table is shorter)
  int dev = 0, n_sm = 0;
  FM_CUDA_TRY(cudaGetDevice(&dev));
  FM_CUDA_TRY(cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev));
  const dim3 g1 = p.dkdv_order ? dim3(std::min(p.dkdv_ncta, n_sm)) : dim3((p.Sk + 127) / 128, p.Hkv, p.B);
  const dim3 g2 = p.dq_order ? dim3(std::min(p.dq_ncta, n_sm)) : dim3((p.Sq + 127) / 128, p.Hq, p.B);
  k1<<<g1, Cfg::NTHREADS, Cfg::SMEM, s>>>(k128, v128, q64, do64, p);
  FM_CUDA_TRY(cudaGetLastError());
  k2<<<g2, Cfg::NTHREADS, Cfg::SMEM, s>>>(q128, do128, k64, v64, p);
  count_launches(2);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

int bwd_sm100_persist_launch(const AttnKParams& p, const fm_attn_args* a, cudaStream_t s) {
  const bool bf = a->dtype == FM_DTYPE_BF16;
  if (a->d <= 64 && a->dv <= 64)
    return bf ? launch_bwd_sm100_persist<true, 64>(p, a, s) : launch_bwd_sm100_persist<false, 64>(p, a, s);
  return bf ? launch_bwd_sm100_persist<true, 128>(p, a, s) : launch_bwd_sm100_persist<false, 128>(p, a, s);
}

#ifdef FM_TRACE
extern "C" __attribute__((visibility("default"))) int fm_debug_ptrace_read(int* out) {
  cudaMemcpyFromSymbol(out, g_ptrace, sizeof(int) * 4 * 3 * 2048);
  cudaMemset(nullptr, 0, 0);
  static int zeros[4 * 3 * 2048];
  cudaMemcpyToSymbol(g_ptrace, zeros, sizeof(zeros));
  return 0;
}
extern "C" __attribute__((visibility("default"))) int fm_debug_unitlog_read(long long* out) {
  return (int)cudaMemcpyFromSymbol(out, g_unitlog, sizeof(long long) * 2 * 8 * 32 * 8);
}
extern "C" __attribute__((visibility("default"))) int fm_debug_pprof_read(long long* out) {
  return (int)cudaMemcpyFromSymbol(out, g_pprof, sizeof(long long) * 2 * 64 * 16);
}
#endif

int bwd_sm100_persist_status(int* out, bool reset) {
  int v = 0;
  FM_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_bwd_persist_status, sizeof(int)));
  if (reset && v != 0) {
    const int z = 0;
    FM_CUDA_TRY(cudaMemcpyToSymbol(g_bwd_persist_status, &z, sizeof(int)));
  }
  *out = v;
  return FM_OK;
}

}  // namespace fm

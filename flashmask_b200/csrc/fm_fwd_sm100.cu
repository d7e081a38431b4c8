// Forward attention on the 5th-generation tensor cores (tcgen05 / UMMA) for
// head dims up to 128: a 64-column and a 128-column variant; smaller head dims
// (multiples of 8) run in the next variant up, the TMA loads filling the
// columns past the end of a head with zeros.  Two more variants serve d = 192 /
// dv = 128 (same plan, 48 KB K tiles, two ring slots) and d = dv = 256 (below).
//
// One CTA owns 256 query rows of one (batch, q head) as two 128-row sub-tiles
// that share every K/V tile.  Warp roles:
//   warps 0-3   softmax of sub-tile 0 (thread t <-> row t, TMEM lane t)
//   warps 4-7   softmax of sub-tile 1
//   warp  8     TMA producer: Q once, then K and V tiles through a 4-slot ring,
//               plus the column bounds of partial tiles (plain loads -> smem)
//   warp  9     UMMA issuer (one elected thread): S_s = Q_s K^T into TMEM,
//               O_s += P_s V with P_s read from TMEM; owns the TMEM allocation
//   warp 10     builds the list of surviving K tiles with per-sub-tile flags
//   warp 11     idle
// TMEM (512 columns): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [384,384+D);
// P_s (bf16, 64 columns) overlays the upper half of S_s.
// Online softmax keeps a stale running maximum and only rescales O when the
// maximum grew by more than 2^8 (the rescale is done by the softmax warps
// themselves).  Every mbarrier wait is bounded: on expiry the CTA raises an
// abort flag, all roles unwind, TMEM is freed and a status word is set.
//
// d = dv = 256: the O accumulator of 128 rows alone needs 256 TMEM columns, so a CTA owns 128 query
// rows and its two "sub-tiles" are the two 128-column halves of V / O for the SAME rows: both
// warpgroups run the softmax of the same scores (S is computed once per warpgroup, in its own
// buffer), warpgroup s accumulates O[:, 128 s : 128 s + 128) = P V[:, 128 s : ...).  One 64 KB Q tile
// and a two-slot ring of 64 KB K / V tiles.  The score GEMM runs twice per tile (6 MMA units for the
// 4 the mathematics needs) in exchange for keeping the plan, the barriers and the tile body above.
#include <type_traits>

#include "fm_attn_params.cuh"
#include "fm_sm100.cuh"

namespace fm {

using namespace sm100;

__device__ int g_fwd_status = 0;

#ifdef FM_TRACE
// Debug build only: clock stamps at the phase boundaries of CTAs (x < 64, y = FM_TRACE_Y, z = 0).
#ifndef FM_TRACE_Y
#define FM_TRACE_Y 0
#endif
__device__ long long g_fprof[64 * 16];
#define FPROF(slot) do { if (blockIdx.y == FM_TRACE_Y && blockIdx.z == 0 && blockIdx.x < 64) g_fprof[blockIdx.x * 16 + (slot)] = clock64(); } while (0)
#define FPROF_VAL(slot, v) do { if (blockIdx.y == FM_TRACE_Y && blockIdx.z == 0 && blockIdx.x < 64) g_fprof[blockIdx.x * 16 + (slot)] = (v); } while (0)
#else
#define FPROF(slot)
#define FPROF_VAL(slot, v)
#endif

// D: width q / k are computed at (64, 128, 192 or 256), DV: width of v / o (64, 128 or 256).
template <int D, int DV = D>
struct FwdSm100Cfg {
  static constexpr bool SPLITV = D == 256;              // sub-tiles are halves of V / O, not of the rows
  static constexpr int ROWS = SPLITV ? 128 : 256;       // query rows per CTA
  static constexpr int DVS = SPLITV ? DV / 2 : DV;      // O columns per warpgroup
  // the 64-column variant doubles the ring depth: its slots are half as large; the 192-column one has room
  // for two slots (one K tile and one V tile in flight) beside its two 48 KB Q sub-tiles
  static constexpr int BM = 128, BN = 128, NSTAGE = (D == 64 ? 8 : (D > 128 ? 2 : 4)), NBND = 2, LIST_MAX = 2048;
  static constexpr int NTHREADS = 384;
  static constexpr int SUB = 128 * 128;                 // bytes of a 128-row x 64-col bf16 sub-tile
  static constexpr int Q_BYTES = BM * D * 2;
  static constexpr int K_BYTES = BN * D * 2, V_BYTES = BN * DV * 2;
  static constexpr int SLOT_BYTES = K_BYTES > V_BYTES ? K_BYTES : V_BYTES;
  static constexpr int BND_BYTES = 128 * 4 * 4;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_KV = OFF_Q + (SPLITV ? 1 : 2) * Q_BYTES;
  // Causal masks: the K and V tiles of the diagonal (the first tile of the list, right to left) are requested at
  // kernel entry into slots 0 and 1, before the list exists, where the ring is deep enough to keep the list
  // build's staging area (64 KB) clear of those two slots.
  static constexpr bool SPEC = NSTAGE >= 4 && NSTAGE * SLOT_BYTES >= 128 * 1024 && 2 * SLOT_BYTES <= 64 * 1024;
  static constexpr int OFF_STAGE = OFF_KV + (SPEC ? 64 * 1024 : 0);
  static constexpr int OFF_BND = OFF_KV + NSTAGE * SLOT_BYTES;
  static constexpr int OFF_LIST = OFF_BND + NBND * BND_BYTES;
  static constexpr int OFF_BAR = OFF_LIST + LIST_MAX * 4;
  static constexpr int OFF_MISC = OFF_BAR + 32 * 8;
  static constexpr int SMEM = OFF_MISC + 64 + 1024;     // + alignment slack
  // block-score variant only: 16 block maxima per softmax thread behind everything else
  static constexpr int OFF_BS = OFF_MISC + 64;
  static constexpr int SMEM_BS = OFF_BS + 16 * BS_ACC_STRIDE * 4 + 1024;
  static_assert(SMEM_BS <= 227 * 1024, "shared memory of the block-score variant");
  // barrier indices
  static constexpr int B_QFULL = 0, B_KVFULL = 2, B_KVEMPTY = 2 + NSTAGE, B_SFULL = 2 + 2 * NSTAGE,
                       B_PFULL = B_SFULL + 2, B_ODONE = B_PFULL + 2, B_BNDFULL = B_ODONE + 2,
                       B_BNDEMPTY = B_BNDFULL + NBND, B_COUNT = B_BNDEMPTY + NBND;
  static_assert((D == 64 && DV == 64) || (D == 128 && DV == 128) || (D == 192 && DV == 128) ||
                    (D == 256 && DV == 256), "head-dim variants");
  static_assert(SMEM_BS <= 227 * 1024 && SMEM <= 227 * 1024, "shared memory");
  static_assert(B_COUNT <= 32, "barrier storage");
  static_assert(OFF_STAGE + LIST_MAX * 8 * 4 <= OFF_BND, "the ring stages the reductions of the list build");
  static_assert(SMEM > 120 * 1024, "one CTA per SM is assumed by the 512-column TMEM allocation");
};

__device__ __forceinline__ float neg_inf() { return __int_as_float(0xff800000); }

// BLOCK_SCORE: 0, or the block size (32 / 64 / 128) of the block-score side output; BLOCK_BOS: document
// starts are given, so a block may straddle two tiles.
template <int D, int DV, bool IS_BF16, int BLOCK_SCORE, bool BLOCK_BOS>
__global__ void __launch_bounds__(384, 1)
fwd_sm100_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const AttnKParams p) {
  using Cfg = FwdSm100Cfg<D, DV>;
  constexpr bool SPLITV = Cfg::SPLITV;
  constexpr int ROWS = Cfg::ROWS, DVS = Cfg::DVS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase + Cfg::OFF_Q, sKV = sbase + Cfg::OFF_KV;
  uint32_t* list = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_LIST);
  const uint32_t bars = sbase + Cfg::OFF_BAR;
  volatile int* misc = reinterpret_cast<volatile int*>(smem + Cfg::OFF_MISC);
  // misc[0] tmem base, [1] cnt, [2] cnt_s0, [3] cnt_s1, [4] abort
  auto bar = [&](int i) { return bars + 8u * (uint32_t)i; };

  const int tid = threadIdx.x;
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int lane = tid & 31;
  if (tid == 0) FPROF(0);
  // descriptor fetches start before anything else: the first loads wait on them
  if (warp == 8 && lane == 0) { tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); }
  const int n_tiles = (p.Sq + ROWS - 1) / ROWS;
  int t = n_tiles - 1 - blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
  if (!SPLITV && p.fwd_order) {
    const OrderedCta c = ordered_cta(p.fwd_order, p.Hq);
    t = c.unit; hq = c.head; b = c.b;
  }
  const int hk = hq / (p.Hq / p.Hkv);
  if (tid == 0) FPROF(8);                    // table entry known
  const MaskDesc& md = p.md;
  const int bh_mask = md.ncols ? ((md.mask_B == 1 ? 0 : b) * md.Hm + hq / (p.Hq / md.Hm)) : 0;
  const int ms = t * ROWS;
  const int off = p.Sk - p.Sq;
  // first K tile right of everything these rows can see, and whether the diagonal tile is loaded ahead of the list
  const int nb = (p.Sk + 127) / 128;
  const int n_hi = md.causal ? max(0, min(nb, (min(ms + ROWS, p.Sq) + off + 127) / 128)) : nb;
  const bool spec = Cfg::SPEC && BLOCK_SCORE == 0 && md.causal && n_hi > 0;

  if (tid == 0) misc[4] = 0;
  if (warp == 8 && lane == 0) {
    mbar_init(bar(Cfg::B_QFULL + 0), 1); mbar_init(bar(Cfg::B_QFULL + 1), 1);
    for (int i = 0; i < Cfg::NSTAGE; ++i) { mbar_init(bar(Cfg::B_KVFULL + i), 1); mbar_init(bar(Cfg::B_KVEMPTY + i), 1); }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(Cfg::B_SFULL + s), 1); mbar_init(bar(Cfg::B_PFULL + s), 128); mbar_init(bar(Cfg::B_ODONE + s), 1);
    }
    for (int i = 0; i < Cfg::NBND; ++i) { mbar_init(bar(Cfg::B_BNDFULL + i), 32); mbar_init(bar(Cfg::B_BNDEMPTY + i), 256); }
    fence_mbar_init();
    // both Q sub-tiles are requested right away: the loads overlap with the
    // list build (rows past the end of the sequence arrive as zeros)
    for (int s = 0; s < (SPLITV ? 1 : 2); ++s) {
      mbar_arrive_expect_tx(bar(Cfg::B_QFULL + s), Cfg::Q_BYTES);
      for (int dc = 0; dc < D / 64; ++dc)
        tma_load_4d(sQ + s * Cfg::Q_BYTES + dc * Cfg::SUB, &tm_q, bar(Cfg::B_QFULL + s), dc * 64, hq,
                    ms + 128 * s, b);
    }
    if (spec) {
      const int j0 = (n_hi - 1) * 128;
      mbar_arrive_expect_tx(bar(Cfg::B_KVFULL + 0), Cfg::K_BYTES);
      for (int dc = 0; dc < D / 64; ++dc)
        tma_load_4d(sKV + dc * Cfg::SUB, &tm_k, bar(Cfg::B_KVFULL + 0), dc * 64, hk, j0, b);
      mbar_arrive_expect_tx(bar(Cfg::B_KVFULL + 1), Cfg::V_BYTES);
      for (int dc = 0; dc < DV / 64; ++dc)
        tma_load_4d(sKV + Cfg::SLOT_BYTES + dc * Cfg::SUB, &tm_v, bar(Cfg::B_KVFULL + 1), dc * 64, hk, j0, b);
    }
  }
  if (warp == 9) {
    tmem_alloc(sbase + Cfg::OFF_MISC, 512);
    tmem_relinquish();
    if (lane == 0) FPROF(12);
  }
  if (warp == 10) {
    // surviving K tiles, right to left, with the flags of both sub-tiles
    int cnt = 0, c0 = 0, c1 = 0;
    // the reductions the classification needs are staged in the (still idle) K/V ring
    const MaskDesc mst = stage_minmax(md, bh_mask, 0, n_hi, reinterpret_cast<int32_t*>(smem + Cfg::OFF_STAGE),
                                      Cfg::LIST_MAX, lane);
    if (lane == 0) FPROF(9);                 // reductions staged
    for (int base = n_hi - 1; base >= 0; base -= 32) {
      const int n = base - lane;
      uint32_t f0 = 0, f1 = 0;
      if (n >= 0) {
        f0 = tile_flags(mst, 0, n, ms, min(ms + 128, p.Sq), 128);
        if (SPLITV) f1 = f0;
        else if (ms + 128 < p.Sq) f1 = tile_flags(mst, 0, n, ms + 128, min(ms + 256, p.Sq), 128);
        if (spec && n == n_hi - 1 && (f0 | f1) == 0) {
          // the diagonal tile is already on its way into slots 0 / 1, so it is the first list entry whatever its
          // class: an invisible one is computed with the element mask (every score masked, P = 0)
          f0 = FM_TF_ACTIVE | FM_TF_CAUSAL | FM_TF_RAGGED | (md.ncols ? FM_TF_BOUNDS : 0u);
          if (ms + 128 < p.Sq) f1 = f0;
        }
      }
      const bool keep = (f0 | f1) != 0;
      const uint32_t bal = __ballot_sync(0xffffffffu, keep);
      const int pos = cnt + __popc(bal & ((1u << lane) - 1u));
      if (keep && pos < Cfg::LIST_MAX) list[pos] = (uint32_t)n | (f0 << 16) | (f1 << 20);
      cnt += __popc(bal);
      c0 += __popc(__ballot_sync(0xffffffffu, f0 != 0));
      c1 += __popc(__ballot_sync(0xffffffffu, f1 != 0));
    }
    if (lane == 0) { misc[1] = min(cnt, Cfg::LIST_MAX); misc[2] = c0; misc[3] = c1; FPROF(10); }
    fence_proxy_async_smem();   // the staging area is handed back to the TMA loads of the ring
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = (uint32_t)misc[0];
  const int cnt = misc[1];
  WaitCtx wc{misc + 4, global_timer_ns() + 2000000000ull};
  if (tid == 0) { FPROF(1); FPROF_VAL(7, (long long)cnt); }
  if (cnt == 0) {
    // nothing visible for these 256 rows: write O = 0 and LSE = -inf (sink
    // present: LSE = sink); the Q loads already in flight are awaited and the
    // tensor memory is returned before leaving
    if (warp == 8 && lane == 0) {
      mbar_wait(bar(Cfg::B_QFULL + 0), 0u, wc);
      if (!SPLITV) mbar_wait(bar(Cfg::B_QFULL + 1), 0u, wc);
    }
    if (warp == 9) tmem_dealloc(tmem, 512);
    uint16_t* go = reinterpret_cast<uint16_t*>(p.o) + b * p.o_b + (int64_t)ms * p.o_s + hq * p.o_h;
    for (int x = tid; x < ROWS * (DV / 8); x += Cfg::NTHREADS) {
      const int rr = x / (DV / 8), cc = x % (DV / 8);
      if (ms + rr < p.Sq && cc * 8 < p.dv_dim)
        *reinterpret_cast<uint4*>(go + (int64_t)rr * p.o_s + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
    const float empty_lse = p.sink ? p.sink[hq] : neg_inf();
    for (int rr = tid; rr < ROWS; rr += Cfg::NTHREADS)
      if (ms + rr < p.Sq) p.lse[((int64_t)b * p.Hq + hq) * p.Sq + ms + rr] = empty_lse;
    return;
  }
  const int cnt_s[2] = {misc[2], misc[3]};

  if (warp < 8) {
    // =========================== softmax warpgroups ===========================
    setmaxnreg_inc<216>();
    const int s = warp >> 2;
    const int r = tid & 127;                   // row inside the sub-tile == TMEM lane
    const int row = ms + (SPLITV ? 0 : 128 * s) + r;
    const uint32_t lane_field = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + lane_field + 128u * s;
    const uint32_t tP = tS + 64u;
    const uint32_t tO = tmem + lane_field + 256u + 128u * s;
    const float scale_log2 = p.scale_log2;
    float m_run = neg_inf(), l_run = 0.f;
    int n_done = 0, nbnd = 0;
    bool ok = true;
    // block-score side output: this thread's row of it, and the first key of the row's document
    // Block scores.  A row whose document starts on a block boundary (always, without block_bos) has
    // every block inside one tile: the maxima are stored straight from registers.  Otherwise a block
    // can straddle two tiles, and the maxima are gathered per thread in shared memory, sixteen
    // consecutive blocks of the row (two groups of eight); a group is merged into global memory once
    // no later tile can touch it: tiles are walked right to left, so its turn comes when a tile lies
    // wholly below it.  The merge (load, fmax, store of 32 contiguous bytes per row) runs BEFORE the
    // thread waits for the scores of the next tile, where its load latency overlaps the tensor pipe.
    float* bs_dst = nullptr;
    float* bs_acc = nullptr;
    int bs_bos = 0, bs_pend_lo = INT_MAX, bs_pend_hi = -1;    // pending groups [lo, hi]; lo > hi: none
    bool bs_vec = false;
    if constexpr (BLOCK_SCORE != 0) {
      // (d = 256: both warpgroups see the same scores; warpgroup 0 writes them)
      if (row < p.Sq && !(SPLITV && s == 1))
        bs_dst = p.block_logit + (((int64_t)b * p.Hq + hq) * p.Sq + row) * p.block_ld;
      if constexpr (BLOCK_BOS) {
        bs_acc = reinterpret_cast<float*>(smem + Cfg::OFF_BS) + tid;
#pragma unroll
        for (int c = 0; c < 16; ++c) bs_acc[c * BS_ACC_STRIDE] = neg_inf();
        if (row < p.Sq) {
          bs_bos = p.block_bos[(int64_t)b * p.Sq + row];
          bs_vec = (reinterpret_cast<uintptr_t>(bs_dst) & 15) == 0;
        }
      }
    }
    auto bs_flush = [&](int g) {
      float* gp = bs_dst + g * 8;
      float* a = bs_acc + (g & 1) * 8 * BS_ACC_STRIDE;
      if (bs_vec && g * 8 + 7 < p.block_cols) {
        float4 o0 = *reinterpret_cast<const float4*>(gp), o1 = *reinterpret_cast<const float4*>(gp + 4);
        o0.x = fmaxf(o0.x, a[0 * BS_ACC_STRIDE]); o0.y = fmaxf(o0.y, a[1 * BS_ACC_STRIDE]);
        o0.z = fmaxf(o0.z, a[2 * BS_ACC_STRIDE]); o0.w = fmaxf(o0.w, a[3 * BS_ACC_STRIDE]);
        o1.x = fmaxf(o1.x, a[4 * BS_ACC_STRIDE]); o1.y = fmaxf(o1.y, a[5 * BS_ACC_STRIDE]);
        o1.z = fmaxf(o1.z, a[6 * BS_ACC_STRIDE]); o1.w = fmaxf(o1.w, a[7 * BS_ACC_STRIDE]);
        *reinterpret_cast<float4*>(gp) = o0;
        *reinterpret_cast<float4*>(gp + 4) = o1;
      } else {
#pragma unroll
        for (int c = 0; c < 8; ++c)
          if (g * 8 + c < p.block_cols) gp[c] = fmaxf(gp[c], a[c * BS_ACC_STRIDE]);
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) a[c * BS_ACC_STRIDE] = neg_inf();
    };
    for (int i = 0; i < cnt && ok; ++i) {
      const uint32_t e = list[i];
      const uint32_t flags = (e >> (16 + 4 * s)) & 0xFu;
      const bool any_bounds = (((e >> 16) | (e >> 20)) & FM_TF_BOUNDS) != 0;
      const int bslot = nbnd % Cfg::NBND;
      const uint32_t bpar = (uint32_t)(nbnd / Cfg::NBND) & 1u;
      if (any_bounds) {
        // every softmax thread passes through the full barrier of a bounds slot
        // before releasing it, so a warpgroup that runs ahead (inactive on these
        // tiles) cannot arrive twice within one phase of the empty barrier
        ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_BNDFULL + bslot), bpar, wc));
        if (!ok) break;
      }
      if (flags) {
        int bs_rel0 = 0;
        if constexpr (BLOCK_SCORE != 0) bs_rel0 = (int)(e & 0xFFFFu) * 128 - bs_bos;
        if constexpr (BLOCK_SCORE != 0 && BLOCK_BOS) {
          constexpr int BS_LOG2 = BLOCK_SCORE == 32 ? 5 : (BLOCK_SCORE == 64 ? 6 : 7);
          if (bs_dst && (bs_rel0 & ((1 << BS_LOG2) - 1)) != 0) {
            // blocks this tile can touch: [base, top]; the groups above them are complete
            const int base = bs_rel0 >> BS_LOG2;
            const int top = base + (128 >> BS_LOG2);
            const int lo_rb = max(base, 0), hi_rb = min(top, p.block_cols - 1);
            if (lo_rb <= hi_rb) {
              const int g_top = hi_rb >> 3, g_bot = lo_rb >> 3;
              for (int g = bs_pend_hi; g >= max(bs_pend_lo, g_top + 1); --g) bs_flush(g);
              bs_pend_hi = min(bs_pend_hi, g_top);
              if (bs_pend_lo > bs_pend_hi) { bs_pend_hi = g_top; bs_pend_lo = g_bot; }
              else bs_pend_lo = min(bs_pend_lo, g_bot);
            }
          }
        }
        ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_SFULL + s), (uint32_t)n_done & 1u, wc));
        if (!ok) break;
        if (tid == 0 && n_done == 0) FPROF(2);
#define FM_N_UNIT n_done
#define FM_N_TOT n_done
#include "fm_fwd_sm100_tile.inc"
#undef FM_N_UNIT
#undef FM_N_TOT
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar(Cfg::B_PFULL + s));
        ++n_done;
      }
      if (any_bounds) {
        mbar_arrive(bar(Cfg::B_BNDEMPTY + bslot));
        ++nbnd;
      }
    }
    if constexpr (BLOCK_SCORE != 0 && BLOCK_BOS) {
      if (ok && bs_dst)
        for (int g = bs_pend_hi; g >= bs_pend_lo; --g) bs_flush(g);
    }
    // ---- epilogue: O / l -> bf16 -> smem staging -> coalesced stores; LSE ----
    if (tid == 0) FPROF(3);
    if (ok && n_done > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_ODONE + s), (uint32_t)(n_done - 1) & 1u, wc));
      tc_fence_after();
    }
    if (tid == 0) FPROF(4);
    if (ok) {
      const float m_fin = (m_run == neg_inf()) ? 0.f : m_run;
      float l_tot = l_run;
      if (p.sink) l_tot += fast_exp2(p.sink[hq] * kLog2e - m_fin);
      const float inv = l_tot > 0.f ? 1.f / l_tot : 0.f;
      uint8_t* stage = smem + Cfg::OFF_Q + (SPLITV ? 0 : s * Cfg::Q_BYTES);   // Q is no longer needed
      constexpr int CH0 = SPLITV ? DVS / 8 : 0;          // d = 256: warpgroup s stages chunks [16 s, 16 s + 16)
#pragma unroll
      for (int c = 0; c < DVS / 32; ++c) {
        uint32_t orr[32];
        if (n_done > 0) {
          tmem_ld32(tO + 32 * c, orr);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) orr[j] = 0u;
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint4 v;
          v.x = pack2<IS_BF16>(__uint_as_float(orr[8 * q4 + 0]) * inv, __uint_as_float(orr[8 * q4 + 1]) * inv);
          v.y = pack2<IS_BF16>(__uint_as_float(orr[8 * q4 + 2]) * inv, __uint_as_float(orr[8 * q4 + 3]) * inv);
          v.z = pack2<IS_BF16>(__uint_as_float(orr[8 * q4 + 4]) * inv, __uint_as_float(orr[8 * q4 + 5]) * inv);
          v.w = pack2<IS_BF16>(__uint_as_float(orr[8 * q4 + 6]) * inv, __uint_as_float(orr[8 * q4 + 7]) * inv);
          const int chunk = CH0 * s + 4 * c + q4;       // 16-byte chunk inside the row
          *reinterpret_cast<uint4*>(stage + r * (DV * 2) + ((chunk ^ (r & (DV / 8 - 1))) << 4)) = v;
        }
      }
      if (row < p.Sq && !(SPLITV && s == 1))
        p.lse[((int64_t)b * p.Hq + hq) * p.Sq + row] = l_tot > 0.f ? (m_fin + log2f(l_tot)) * kLn2 : neg_inf();
      __syncwarp();   // each warp stores the 32 rows it staged itself: no cross-warp dependency
      const int rbase = ms + (SPLITV ? 0 : 128 * s);
      uint16_t* go = reinterpret_cast<uint16_t*>(p.o) + b * p.o_b + (int64_t)rbase * p.o_s + hq * p.o_h;
      constexpr int CH = DV / 8, CHW = DVS / 8;          // chunks per row, chunks this warpgroup staged
      const int wrow = (warp & 3) * 32;
#pragma unroll 4
      for (int idx = lane; idx < 32 * CHW; idx += 32) {
        const int rr = wrow + idx / CHW, cc = CH0 * s + idx % CHW;
        if (rbase + rr < p.Sq && cc * 8 < p.dv_dim) {
          const uint4 v = *reinterpret_cast<const uint4*>(stage + rr * (DV * 2) + ((cc ^ (rr & (CH - 1))) << 4));
          *reinterpret_cast<uint4*>(go + (int64_t)rr * p.o_s + cc * 8) = v;
        }
      }
    }
    if (tid == 0) FPROF(5);
  } else {
    setmaxnreg_dec<64>();
    if (warp == 8) {
      // =========================== TMA / bounds producer ===========================
      int nbnd = 0;
      bool ok = true;
      for (int i = 0; i < cnt && ok; ++i) {
        const uint32_t e = list[i];
        const int j0 = (int)(e & 0xFFFFu) * 128;
        if (!(spec && i == 0) && elect_one()) {       // (the first tile of a causal mask was requested at entry)
          for (int kv = 0; kv < 2 && ok; ++kv) {
            const int k = 2 * i + kv, slot = k % Cfg::NSTAGE;
            const uint32_t par = ((uint32_t)(k / Cfg::NSTAGE) & 1u) ^ 1u;
            ok = mbar_wait(bar(Cfg::B_KVEMPTY + slot), par, wc);
            if (!ok) break;
            mbar_arrive_expect_tx(bar(Cfg::B_KVFULL + slot), kv == 0 ? Cfg::K_BYTES : Cfg::V_BYTES);
            for (int dc = 0; dc < (kv == 0 ? D : DV) / 64; ++dc)
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
      // a sub-tile without work never consumed its Q load: make sure it has landed
      if (ok && lane == 0) { mbar_wait(bar(Cfg::B_QFULL + 0), 0u, wc); if (!SPLITV) mbar_wait(bar(Cfg::B_QFULL + 1), 0u, wc); }
    } else if (warp == 9) {
      // =========================== UMMA issuer ===========================
      if (elect_one()) {
        constexpr uint32_t idesc_qk = make_idesc(IS_BF16, 128, 128, 0, 0);
        constexpr uint32_t idesc_pv = make_idesc(IS_BF16, 128, DVS, 0, 1);
        int npv[2] = {0, 0};
        bool q_ready[2] = {false, false};
        bool ok = true;
        // descriptors are built once; per MMA only a constant is added to the
        // 14-bit address field (all smem offsets are multiples of 16 bytes)
        const uint64_t dq0 = make_sdesc(sQ, 16, 1024);
        const uint64_t dk0 = make_sdesc(sKV, 16, 1024);
        const uint64_t dv0 = make_sdesc(sKV, Cfg::SUB, 1024);
        auto issue_qk = [&](auto sub, int i) {
            constexpr int s = decltype(sub)::value;   // compile-time: the per-sub-tile counters stay in registers
          const int k = 2 * i, slot = k % Cfg::NSTAGE;
          ok = ok && mbar_wait(bar(Cfg::B_KVFULL + slot), (uint32_t)(k / Cfg::NSTAGE) & 1u, wc);
          if (ok && !q_ready[s]) { ok = mbar_wait(bar(Cfg::B_QFULL + (SPLITV ? 0 : s)), 0u, wc); q_ready[s] = true; }
          if (!ok) return;
          tc_fence_after();
          const uint64_t da = dq0 + (uint64_t)(SPLITV ? 0 : s * (Cfg::Q_BYTES >> 4));
          const uint64_t db = dk0 + (uint64_t)(slot * (Cfg::SLOT_BYTES >> 4));
          const uint32_t dst = tmem + 128u * s;
          if constexpr (D == 128) umma_ss_x8<(Cfg::SUB >> 4), (Cfg::SUB >> 4)>(dst, da, db, idesc_qk, 0u);
          else if constexpr (D == 192) {
            // three 64-column sub-tiles of q / k: eight k-steps, then four more on top
            umma_ss_x8<(Cfg::SUB >> 4), (Cfg::SUB >> 4)>(dst, da, db, idesc_qk, 0u);
            umma_ss_x4(dst, da + (uint64_t)(2 * (Cfg::SUB >> 4)), db + (uint64_t)(2 * (Cfg::SUB >> 4)), idesc_qk, 1u);
          } else if constexpr (D == 256) {
            // four 64-column sub-tiles: eight k-steps over the first two, eight over the last two
            umma_ss_x8<(Cfg::SUB >> 4), (Cfg::SUB >> 4)>(dst, da, db, idesc_qk, 0u);
            umma_ss_x8<(Cfg::SUB >> 4), (Cfg::SUB >> 4)>(dst, da + (uint64_t)(2 * (Cfg::SUB >> 4)),
                                                         db + (uint64_t)(2 * (Cfg::SUB >> 4)), idesc_qk, 1u);
          } else umma_ss_x4(dst, da, db, idesc_qk, 0u);
          tc_commit(bar(Cfg::B_SFULL + s));
        };
        auto issue_pv = [&](auto sub, int i) {
            constexpr int s = decltype(sub)::value;
          const int k = 2 * i + 1, slot = k % Cfg::NSTAGE;
          ok = ok && mbar_wait(bar(Cfg::B_KVFULL + slot), (uint32_t)(k / Cfg::NSTAGE) & 1u, wc);
          ok = ok && mbar_wait(bar(Cfg::B_PFULL + s), (uint32_t)npv[s] & 1u, wc);
          if (!ok) return;
          tc_fence_after();
          // (d = 256: warpgroup s owns V columns [128 s, 128 s + 128): sub-tiles 2 s and 2 s + 1 of the V tile)
          const uint64_t db = dv0 + (uint64_t)(slot * (Cfg::SLOT_BYTES >> 4) + (SPLITV ? s * 2 * (Cfg::SUB >> 4) : 0));
          const uint32_t dst = tmem + 256u + 128u * s, src = tmem + 128u * s + 64u;
          const uint32_t acc0 = npv[s] > 0 ? 1u : 0u;
          umma_ts_xn<8>(dst, src, db, idesc_pv, acc0);
          tc_commit(bar(Cfg::B_ODONE + s));
          ++npv[s];
        };
        if (cnt > 0) {
          const uint32_t e = list[0];
          if ((e >> 16) & 0xFu) issue_qk(std::integral_constant<int, 0>{}, 0);
          if ((e >> 20) & 0xFu) issue_qk(std::integral_constant<int, 1>{}, 0);
          if (ok) tc_commit(bar(Cfg::B_KVEMPTY + 0));
        }
        for (int i = 0; i < cnt && ok; ++i) {
          const uint32_t e = list[i];
          const uint32_t en = (i + 1 < cnt) ? list[i + 1] : 0u;
          // the sub-tile whose P is ready first goes first (sub-tile 0 when both or neither are)
          bool one_first = false;
          if (((e >> 16) & 0xFu) && ((e >> 20) & 0xFu))
            one_first = !mbar_try_wait(bar(Cfg::B_PFULL + 0), (uint32_t)npv[0] & 1u) &&
                        mbar_try_wait(bar(Cfg::B_PFULL + 1), (uint32_t)npv[1] & 1u);
          if (one_first) {
            issue_pv(std::integral_constant<int, 1>{}, i);
            if (ok && ((en >> 20) & 0xFu)) issue_qk(std::integral_constant<int, 1>{}, i + 1);
            if (ok) issue_pv(std::integral_constant<int, 0>{}, i);
            if (ok && ((en >> 16) & 0xFu)) issue_qk(std::integral_constant<int, 0>{}, i + 1);
          } else {
            if ((e >> 16) & 0xFu) issue_pv(std::integral_constant<int, 0>{}, i);
            if (ok && ((en >> 16) & 0xFu)) issue_qk(std::integral_constant<int, 0>{}, i + 1);
            if (ok && ((e >> 20) & 0xFu)) issue_pv(std::integral_constant<int, 1>{}, i);
            if (ok && ((en >> 20) & 0xFu)) issue_qk(std::integral_constant<int, 1>{}, i + 1);
          }
          if (!ok) break;
          tc_commit(bar(Cfg::B_KVEMPTY + (2 * i + 1) % Cfg::NSTAGE));
          if (i + 1 < cnt) tc_commit(bar(Cfg::B_KVEMPTY + (2 * i + 2) % Cfg::NSTAGE));
        }
      }
      __syncwarp();
    }
  }

  // =========================== teardown ===========================
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (tid == 0) FPROF(6);
  const bool aborted = misc[4] != 0;
  if (aborted) {
    // give copies and MMAs still in flight a bounded time to land before the
    // shared and tensor memory of this CTA are released
    const uint64_t t_end = global_timer_ns() + 200000ull;
    while (global_timer_ns() < t_end) __nanosleep(1000);
    if (tid == 0) atomicExch(&g_fwd_status, FM_ERR_TIMEOUT);
  }
  if (warp == 9) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
#ifdef FM_TRACE
extern "C" __attribute__((visibility("default"))) int fm_debug_fprof_read(long long* out) {
  return (int)cudaMemcpyFromSymbol(out, g_fprof, sizeof(long long) * 64 * 16);
}
#endif

namespace sm100 {

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

int make_bshd_tmap(CUtensorMap* out, const void* base, int dtype, int B, int S, int H, int D, int64_t sb,
                   int64_t ss, int64_t sh, int box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  FM_REQUIRE(enc != nullptr, FM_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)ss * 2, (cuuint64_t)(sb > 0 ? sb : ss * S) * 2};
  const cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = enc(out, dtype == FM_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                         4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  FM_REQUIRE(r == CUDA_SUCCESS, FM_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return FM_OK;
}

}  // namespace sm100

// One CTA waits on an mbarrier that nothing ever arrives on, with a wall-clock
// budget: exercises the bounded wait and the status word without touching the
// tensor pipe.  The kernel returns normally; the context stays usable.
__global__ void bounded_wait_selftest_kernel(uint64_t budget_ns) {
  __shared__ __align__(8) uint64_t never;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_u32(&never), 1);
    fence_mbar_init();
  }
  __syncthreads();
  WaitCtx wc{&abort_flag, global_timer_ns() + budget_ns};
  const bool ok = mbar_wait(smem_u32(&never), 0u, wc);
  __syncthreads();
  if (threadIdx.x == 0 && !ok) atomicExch(&g_fwd_status, FM_ERR_TIMEOUT);
}

int bounded_wait_selftest_launch(uint64_t budget_ns, cudaStream_t s) {
  bounded_wait_selftest_kernel<<<1, 64, 0, s>>>(budget_ns);
  count_launches(1);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

bool fwd_sm100_supported(const fm_attn_args* a) {
  const bool small = a->d <= 128 && a->dv <= 128 && a->d % 8 == 0 && a->dv % 8 == 0;
  if (!small && !(a->d == 192 && a->dv == 128) && !(a->d == 256 && a->dv == 256)) return false;
  if (((uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v) & 15) return false;
  return true;
}

template <int D, int DV, bool IS_BF16, int BLOCK_SCORE, bool BLOCK_BOS>
static int launch_fwd_sm100(const AttnKParams& p, const fm_attn_args* a, cudaStream_t s) {
  using Cfg = FwdSm100Cfg<D, DV>;
  FM_REQUIRE((a->Sk + 127) / 128 <= Cfg::LIST_MAX, FM_ERR_UNSUPPORTED,
             "forward: Sk=%d exceeds the %d keys this kernel variant indexes", a->Sk, Cfg::LIST_MAX * 128);
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_bshd_tmap(&tq, a->q, a->dtype, a->B, a->Sq, a->Hq, a->d, a->q_stride[0], a->q_stride[1], a->q_stride[2], 128))) return rc;
  if ((rc = make_bshd_tmap(&tk, a->k, a->dtype, a->B, a->Sk, a->Hkv, a->d, a->k_stride[0], a->k_stride[1], a->k_stride[2], 128))) return rc;
  if ((rc = make_bshd_tmap(&tv, a->v, a->dtype, a->B, a->Sk, a->Hkv, a->dv, a->v_stride[0], a->v_stride[1], a->v_stride[2], 128))) return rc;
  auto kern = fwd_sm100_kernel<D, DV, IS_BF16, BLOCK_SCORE, BLOCK_BOS>;
  constexpr int smem_bytes = BLOCK_BOS ? Cfg::SMEM_BS : Cfg::SMEM;
  FM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
  dim3 grid((p.Sq + Cfg::ROWS - 1) / Cfg::ROWS, p.Hq, p.B);
  kern<<<grid, Cfg::NTHREADS, smem_bytes, s>>>(tq, tk, tv, p);
  count_launches(1);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

int fwd_sm100_launch(const AttnKParams& p, const fm_attn_args* a, cudaStream_t s) {
  const bool bf = a->dtype == FM_DTYPE_BF16;
  const bool small = a->d <= 64 && a->dv <= 64;
#define FM_FWD_DISPATCH(BSZ, BOS)                                                                         \
  do {                                                                                                    \
    if (a->d == 256)                                                                                      \
      return bf ? launch_fwd_sm100<256, 256, true, BSZ, BOS>(p, a, s) : launch_fwd_sm100<256, 256, false, BSZ, BOS>(p, a, s); \
    if (a->d == 192)                                                                                      \
      return bf ? launch_fwd_sm100<192, 128, true, BSZ, BOS>(p, a, s) : launch_fwd_sm100<192, 128, false, BSZ, BOS>(p, a, s); \
    if (small)                                                                                            \
      return bf ? launch_fwd_sm100<64, 64, true, BSZ, BOS>(p, a, s) : launch_fwd_sm100<64, 64, false, BSZ, BOS>(p, a, s); \
    return bf ? launch_fwd_sm100<128, 128, true, BSZ, BOS>(p, a, s) : launch_fwd_sm100<128, 128, false, BSZ, BOS>(p, a, s); \
  } while (0)
  if (p.block_logit && p.block_bos) {
    if (p.block_log2 == 5) FM_FWD_DISPATCH(32, true);
    if (p.block_log2 == 6) FM_FWD_DISPATCH(64, true);
    FM_FWD_DISPATCH(128, true);
  }
  if (p.block_logit) {
    if (p.block_log2 == 5) FM_FWD_DISPATCH(32, false);
    if (p.block_log2 == 6) FM_FWD_DISPATCH(64, false);
    FM_FWD_DISPATCH(128, false);
  }
  FM_FWD_DISPATCH(0, false);
#undef FM_FWD_DISPATCH
}

int fwd_sm100_status(int* out, bool reset) {
  int v = 0;
  FM_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_fwd_status, sizeof(int)));
  if (reset && v != 0) {
    const int z = 0;
    FM_CUDA_TRY(cudaMemcpyToSymbol(g_fwd_status, &z, sizeof(int)));
  }
  *out = v;
  return FM_OK;
}

}  // namespace fm

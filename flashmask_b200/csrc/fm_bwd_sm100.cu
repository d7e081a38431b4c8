// Backward attention on the 5th-generation tensor cores (tcgen05 / UMMA) for
// head dims up to 128 (smaller ones, multiples of 8, are computed at width 128:
// the TMA loads fill the columns past the end of a head with zeros and the
// epilogues leave them unwritten) and for d = 192 / dv = 128, as two kernels that
// share one pipeline skeleton:
//
//   MODE_DKDV  one CTA per (128-key tile, kv head, batch).  K and V stay in
//              shared memory; 64-row halves of Q and dO stream through a ring
//              for every q head of the GQA group.  TMEM lanes are keys:
//                S^T = K Q^T, dP^T = V dO^T            (M=128 keys, N=64 queries)
//                dV += P^T dO, dK += dS^T Q             (A from TMEM, M=128, N=128, K=64)
//   MODE_DQ    one CTA per (128-query tile, q head, batch).  Q and dO stay in
//              shared memory; 64-row halves of K and V stream.  TMEM lanes are
//              queries:  S = Q K^T, dP = dO V^T, dQ += dS K.
//
// Work items are the 64-row half tiles that the mask classification keeps; item
// k is computed by softmax warpgroup k%2 out of score buffers k%2, so the
// tensor pipe works on one item while the other warpgroup does exp2 / dS.
// Every output element has exactly one owner CTA and a fixed summation order:
// the gradients are bitwise reproducible and need neither atomics nor fp32
// accumulators in global memory.
//
// Warp roles: 0-3 / 4-7 compute warpgroups, 8 TMA producer, 9 UMMA issuer
// (owns TMEM), 10 item-list builder, 11 idle.  All waits are bounded.
#include "fm_attn_params.cuh"
#include "fm_sm100.cuh"

namespace fm {

using namespace sm100;

__device__ int g_bwd_status = 0;

constexpr int MODE_DKDV = 0, MODE_DQ = 1;

#ifdef FM_TRACE
// Debug build only: timeline of CTA (0,0,0); every tracing thread appends
// (event, item, SM clock) triples to its own lane of the buffer with plain stores.
__device__ int g_trace[4 * 3 * 2048];
__device__ __forceinline__ void trace_ev(int role, int& n, int ev, int k) {
  if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && n < 2048) {
    int* t = g_trace + (role * 2048 + n) * 3;
    t[0] = ev; t[1] = k; t[2] = (int)clock64();
    ++n;
  }
}
// Phase stamps of the CTAs (x < 64, y = 0, z = 0): one clock value per phase boundary.
__device__ long long g_prof[2 * 64 * 16];   // [mode][cta][stamp]
#define TRACE_DECL int trace_n = 0;
#define TRACE(role, ev, k) trace_ev(role, trace_n, ev, k)
#define PROF(slot) do { if (blockIdx.y == 0 && blockIdx.z == 0 && blockIdx.x < 64) g_prof[(MODE * 64 + blockIdx.x) * 16 + (slot)] = clock64(); } while (0)
#define PROF_VAL(slot, v) do { if (blockIdx.y == 0 && blockIdx.z == 0 && blockIdx.x < 64) g_prof[(MODE * 64 + blockIdx.x) * 16 + (slot)] = (v); } while (0)
#else
#define TRACE_DECL
#define TRACE(role, ev, k)
#define PROF(slot)
#define PROF_VAL(slot, v)
#endif

// D: width the d-wide operands (Q, K, dQ, dK) are computed at.  Up to 128 the layout is the one of
// D = 128 (a 64-column variant leaves the second sub-tile of every operand unloaded); D = 192 has
// three 64-column sub-tiles per d-wide operand and a three-slot ring.  The dv-wide operands (V, dO,
// dV) always have room for 128 columns.
template <int D>
struct BwdSm100Cfg {
  static constexpr int W1 = D > 128 ? D : 128;
  static constexpr int NSLOT = D > 128 ? 3 : 4, LIST_MAX = 2048, NTHREADS = 384;
  static constexpr int SUB128 = 128 * 128;             // 128-row x 64-col sub-tile (bytes)
  static constexpr int SUB64 = 64 * 128;               // 64-row x 64-col sub-tile (bytes)
  static constexpr int STAT1_BYTES = 128 * W1 * 2;     // stationary K (dK/dV kernel) or Q (dQ kernel) tile
  static constexpr int STAT2_BYTES = 128 * 128 * 2;    // stationary V or dO tile
  static constexpr int OP1_BYTES = 64 * W1 * 2;        // streamed Q or K half tile
  static constexpr int OP2_BYTES = 64 * 128 * 2;       // streamed dO or V half tile
  static constexpr int SLOT_BYTES = OP1_BYTES + OP2_BYTES;
  static constexpr int AUX_BYTES = 1024;
  static constexpr int OFF_STAT = 0;
  static constexpr int OFF_RING = OFF_STAT + STAT1_BYTES + STAT2_BYTES;
  static constexpr int OFF_AUX = OFF_RING + NSLOT * SLOT_BYTES;
  static constexpr int OFF_LIST = OFF_AUX + NSLOT * AUX_BYTES;
  static constexpr int OFF_BAR = OFF_LIST + LIST_MAX * 4;
  static constexpr int OFF_MISC = OFF_BAR + 32 * 8;
  static constexpr int SMEM = OFF_MISC + 64 + 1024;
  static constexpr int B_STAT = 0, B_RFULL = 1, B_REMPTY = 1 + NSLOT, B_GFULL = 1 + 2 * NSLOT,
                       B_TFULL = B_GFULL + 2, B_GREAD = B_TFULL + 2, B_ACC = B_GREAD + 2, B_COUNT = B_ACC + 1;
  static_assert(B_COUNT <= 32, "barrier storage");
  static_assert(SMEM > 120 * 1024 && SMEM <= 227 * 1024, "one CTA per SM (512 TMEM columns)");
};

// Byte offset of 16-byte chunk `chunk` inside row `r` of an epilogue staging tile: the chunk index is
// XOR-ed with the row so that the lanes of a warp (one row each, same chunk) hit different banks.  Rows of
// 24 chunks (D = 192) swizzle inside groups of eight chunks, rows of 16 chunks over the whole row.
template <bool BIG>
__device__ __forceinline__ int stage_chunk(int chunk, int r) {
  if constexpr (BIG) return ((chunk & ~7) | ((chunk ^ r) & 7)) << 4;
  else return (chunk ^ (r & 15)) << 4;
}

__device__ __forceinline__ float bneg_inf() { return __int_as_float(0xff800000); }

__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// D / DV: widths the head dims are computed at: (64, 64) when both fit, (128, 128) up to 128, and
// (192, 128).  The 64-column variant keeps the shared-memory layout of the 128-column one and simply
// leaves the second 64-column sub-tile of every operand unloaded and unread: half the copies, half
// the tensor work.
//
// At D = 192 the accumulators need 320 (dK 192 + dV 128) of the 512 tensor-memory columns, which
// leaves three 64-column score buffers instead of four: S^T (S) keeps one buffer per item parity, dP^T
// (dP) has a single buffer, and the bf16 operands P^T / dS^T (dS) of an item are written over the
// S^T buffer of that item, which is dead once its warpgroup holds the scores in registers.  The
// issue order then is: accumulation MMAs of item k, S^T of item k+2 (after them in the pipe, so
// the overlay is no longer read), dP^T of item k+2 as soon as the other warpgroup has read dP^T of
// item k+1 out of the single buffer.
template <int MODE, bool IS_BF16, int D, int DV>
__global__ void __launch_bounds__(384, 1)
bwd_sm100_kernel(const __grid_constant__ CUtensorMap tm_stat1, const __grid_constant__ CUtensorMap tm_stat2,
                 const __grid_constant__ CUtensorMap tm_str1, const __grid_constant__ CUtensorMap tm_str2,
                 const AttnKParams p) {
  using Cfg = BwdSm100Cfg<D>;
  constexpr bool BIG = D > 128;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sStat = sbase + Cfg::OFF_STAT, sRing = sbase + Cfg::OFF_RING;
  uint32_t* list = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_LIST);
  const uint32_t bars = sbase + Cfg::OFF_BAR;
  volatile int* misc = reinterpret_cast<volatile int*>(smem + Cfg::OFF_MISC);  // [0] tmem, [1] cnt, [4] abort
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

  // ---- CTA coordinates ----
  int b, hk, hq0, row0;  // row0: first key (DKDV) or first query (DQ) of the stationary tile
  if (MODE == MODE_DKDV) {
    b = blockIdx.z; hk = blockIdx.y; hq0 = hk * G; row0 = blockIdx.x * 128;
  } else {
    const int n_tiles = (p.Sq + 127) / 128;
    b = blockIdx.z; hq0 = blockIdx.y; hk = hq0 / G; row0 = (n_tiles - 1 - (int)blockIdx.x) * 128;
  }
  const int bh_mask = md.ncols ? ((md.mask_B == 1 ? 0 : b) * md.Hm + hq0 / (p.Hq / md.Hm)) : 0;
  const int n_heads = (MODE == MODE_DKDV) ? G : 1;
  if (tid == 0) PROF(15);

  if (tid == 0) misc[4] = 0;
  if (warp == 8 && lane == 0) {
    mbar_init(bar(Cfg::B_STAT), 1);
    for (int i = 0; i < Cfg::NSLOT; ++i) {
      mbar_init(bar(Cfg::B_RFULL + i), MODE == MODE_DQ ? 33 : 1);
      mbar_init(bar(Cfg::B_REMPTY + i), 1);
    }
    for (int h = 0; h < 2; ++h) { mbar_init(bar(Cfg::B_GFULL + h), 1); mbar_init(bar(Cfg::B_TFULL + h), 4); mbar_init(bar(Cfg::B_GREAD + h), 4); }
    mbar_init(bar(Cfg::B_ACC), 1);
    fence_mbar_init();
    // the stationary tiles are requested right away: the loads overlap with the list build
    mbar_arrive_expect_tx(bar(Cfg::B_STAT), (D / 64 + DV / 64) * Cfg::SUB128);
    {
      const int hs = (MODE == MODE_DKDV) ? hk : hq0;
      for (int dc = 0; dc < D / 64; ++dc)
        tma_load_4d(sStat + dc * Cfg::SUB128, &tm_stat1, bar(Cfg::B_STAT), dc * 64, hs, row0, b);
      for (int dc = 0; dc < DV / 64; ++dc)
        tma_load_4d(sStat + Cfg::STAT1_BYTES + dc * Cfg::SUB128, &tm_stat2, bar(Cfg::B_STAT), dc * 64, hs, row0, b);
    }
    PROF(11);
  }
  if (warp == 9) {
    if (lane == 0) PROF(14);
    tmem_alloc(sbase + Cfg::OFF_MISC, 512);
    tmem_relinquish();
    if (lane == 0) PROF(12);
  }
  if (warp == 10) {
    // the reductions the classification needs are staged in the (still idle) operand ring
    int32_t* stage = reinterpret_cast<int32_t*>(smem + Cfg::OFF_RING);
    int cnt = 0;
    if (MODE == MODE_DKDV) {
      // 64-query half tiles that see key tile n = row0/128, ascending
      const int n = row0 / 128;
      const int n_half = (p.Sq + 63) / 64;
      const MaskDesc ms = stage_minmax(md, bh_mask, n & ~3, n + 1, stage, 4, lane);
      int lo = 0;
      if (md.causal) lo = max(0, (row0 - off) / 64);
      for (int base = lo; base < n_half; base += 32) {
        const int idx = base + lane;
        uint32_t f = 0;
        if (idx < n_half) f = tile_flags(ms, 0, n, idx * 64, min(idx * 64 + 64, p.Sq), 128);
        const uint32_t bal = __ballot_sync(0xffffffffu, f != 0);
        const int pos = cnt + __popc(bal & ((1u << lane) - 1u));
        if (f && pos < Cfg::LIST_MAX) list[pos] = (uint32_t)idx | (f << 16);
        cnt += __popc(bal);
      }
    } else {
      // 64-key half tiles visible to query tile [row0, row0+128), right to left
      const int me = min(row0 + 128, p.Sq);
      const int n_half = (p.Sk + 63) / 64;
      int hi = n_half;
      if (md.causal) hi = max(0, min(n_half, (me + off + 63) / 64));
      const MaskDesc ms = stage_minmax(md, bh_mask, 0, (hi + 1) >> 1, stage, Cfg::LIST_MAX, lane);
      for (int base = hi - 1; base >= 0; base -= 32) {
        const int idx = base - lane;
        uint32_t f = 0;
        if (idx >= 0) {
          f = tile_flags(ms, 0, idx >> 1, row0, me, 128);
          if (md.causal && idx * 64 > me - 1 + off) f = 0;
        }
        const uint32_t bal = __ballot_sync(0xffffffffu, f != 0);
        const int pos = cnt + __popc(bal & ((1u << lane) - 1u));
        if (f && pos < Cfg::LIST_MAX) list[pos] = (uint32_t)idx | (f << 16);
        cnt += __popc(bal);
      }
    }
    if (lane == 0) misc[1] = min(cnt, Cfg::LIST_MAX);
    fence_proxy_async_smem();   // the staging area is handed back to the TMA loads of the ring
    if (lane == 0) PROF(13);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = (uint32_t)misc[0];
  const int cnt = misc[1];
  WaitCtx wc{misc + 4, global_timer_ns() + 2000000000ull};
  if (tid == 0) { PROF(1); PROF_VAL(10, (long long)cnt * ((MODE == MODE_DKDV) ? p.Hq / p.Hkv : 1)); }
  if (cnt == 0) {
    // this tile's gradients are all zero: store them; the stationary loads already
    // in flight are awaited and the tensor memory is returned before leaving
    if (warp == 8 && lane == 0) mbar_wait(bar(Cfg::B_STAT), 0u, wc);
    if (warp == 9) tmem_dealloc(tmem, 512);
    if (MODE == MODE_DKDV) {
      uint16_t* gk = reinterpret_cast<uint16_t*>(p.dk) + b * p.dk_b + (int64_t)row0 * p.dk_s + hk * p.dk_h;
      uint16_t* gv = reinterpret_cast<uint16_t*>(p.dv) + b * p.dv_b + (int64_t)row0 * p.dv_s + hk * p.dv_h;
      for (int x = tid; x < 128 * (Cfg::W1 / 8); x += Cfg::NTHREADS) {
        const int rr = x / (Cfg::W1 / 8), cc = x % (Cfg::W1 / 8);
        if (row0 + rr < p.Sk) {
          if (cc * 8 < p.d) *reinterpret_cast<uint4*>(gk + (int64_t)rr * p.dk_s + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
          if (cc * 8 < p.dv_dim) *reinterpret_cast<uint4*>(gv + (int64_t)rr * p.dv_s + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
    } else {
      uint16_t* gq = reinterpret_cast<uint16_t*>(p.dq) + b * p.dq_b + (int64_t)row0 * p.dq_s + hq0 * p.dq_h;
      for (int x = tid; x < 128 * (Cfg::W1 / 8); x += Cfg::NTHREADS) {
        const int rr = x / (Cfg::W1 / 8), cc = x % (Cfg::W1 / 8);
        if (row0 + rr < p.Sq && cc * 8 < p.d)
          *reinterpret_cast<uint4*>(gq + (int64_t)rr * p.dq_s + cc * 8) = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    return;
  }
  const int K_items = cnt * n_heads;
  // TMEM columns: score buffers G1_p at 64p, G2_p at 128+64p.
  //   DKDV: P^T_p / dS^T_p (bf16) overlay G2_p at +0 / +32; dV at 256, dK at 384.  G1_p is dead as soon as
  //         its warpgroup has read it, so S^T of item k+2 is issued before item k is finished.
  //   DQ:   dS (bf16) has four own 32-column buffers at 256 (index 2*((k/2)%2) + p), dQ at 384.
  //   D = 192: G1_p at 64p, one G2 at 128; P^T_p / dS^T_p (dS_p) overlay G1_p at +0 / +32 (+0);
  //         DKDV: dV at 192, dK at 320; DQ: dQ at 192.
  constexpr uint32_t C_G1 = 0, C_G2 = 128, C_T = 256;
  constexpr uint32_t C_ACC1 = BIG ? 192 : ((MODE == MODE_DKDV) ? 256 : 384), C_ACC2 = BIG ? 320 : 384;
  static_assert(!BIG || C_ACC2 + D <= 512, "tensor memory columns");

  if (warp < 8) {
    // =========================== compute warpgroups ===========================
    const int pz = warp >> 2;                    // item parity this warpgroup serves
    const int r = tid & 127;                     // TMEM lane
    const uint32_t lane_field = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tG1 = tmem + lane_field + C_G1 + 64u * pz;
    const uint32_t tG2 = tmem + lane_field + C_G2 + (BIG ? 0u : 64u * pz);
    const float scale_log2 = p.scale_log2;
    bool ok = true;

    // per-lane constants
    int lts = INT_MAX, lte = INT_MAX, uts = 0, ute = 0;   // DKDV: bounds of key row0 + r
    float lse2_row = 0.f, dps_row = 0.f;                   // DQ: statistics of query row0 + r
    if (MODE == MODE_DKDV) {
      const int j = row0 + r;
      if (j >= p.Sk) { lts = 0; lte = INT_MAX; }
      else if (md.ncols) {
        const Bounds4 bd = load_bounds(md, md.mask + ((size_t)bh_mask * p.Sk + j) * md.ncols);
        lts = bd.lts; lte = bd.lte; uts = bd.uts; ute = bd.ute;
      }
    } else {
      const int i = row0 + r;
      if (i < p.Sq) {
        lse2_row = p.lse_log2[((int64_t)b * p.Hq + hq0) * p.Sq_r + i];
        dps_row = p.dpsum[((int64_t)b * p.Hq + hq0) * p.Sq_r + i];
      }
    }

    for (int k = pz; k < K_items && ok; k += 2) {
      const uint32_t e = list[k % cnt];
      const int idx = (int)(e & 0xFFFFu);
      const uint32_t flags = e >> 16;
      const int slot = k % Cfg::NSLOT;
      ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_RFULL + slot), (uint32_t)(k / Cfg::NSLOT) & 1u, wc));
      if (!ok) break;
      if (r == 0) TRACE(2 + pz, 10, k);   // ring slot observed full
      ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_GFULL + pz), (uint32_t)(k >> 1) & 1u, wc));
      if (!ok) break;
      if (r == 0) TRACE(2 + pz, 12, k);   // scores observed ready
      if (tid == 0 && k == 0) PROF(4);
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
      const uint32_t tT = BIG ? tG1
                              : (MODE == MODE_DKDV)
                                    ? tG2
                                    : tmem + lane_field + C_T + 32u * (uint32_t)((((k >> 1) & 1) << 1) + pz);
#include "fm_bwd_sm100_item.inc"
      tc_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0)       mbar_arrive(bar(Cfg::B_TFULL + pz));
    }

    // ---- epilogue ----
    if (ok && K_items > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(bar(Cfg::B_ACC), 0u, wc));
      tc_fence_after();
      if (tid == 0) PROF(7);
    }
    if (ok) {
      if (MODE == MODE_DKDV) {
        // warpgroup 0: dK (scaled) staged in the K tile; warpgroup 1: dV staged in the V tile
        const uint32_t tA = tmem + lane_field + (pz == 0 ? C_ACC2 : C_ACC1);
        const float mul = pz == 0 ? p.scale : 1.f;
        uint8_t* stage = smem + Cfg::OFF_STAT + pz * Cfg::STAT1_BYTES;
        const int pitch = pz == 0 ? Cfg::W1 * 2 : 256;     // bytes per staged row
        const int ncol = pz == 0 ? D : DV;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          if (32 * c >= ncol) break;
          uint32_t orr[32];
          if (K_items > 0) { tmem_ld32(tA + 32 * c, orr); tc_wait_ld(); }
          else {
#pragma unroll
            for (int j = 0; j < 32; ++j) orr[j] = 0u;
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 v;
            v.x = pack2<IS_BF16>(__uint_as_float(orr[8 * q4 + 0]) * mul, __uint_as_float(orr[8 * q4 + 1]) * mul);
            v.y = pack2<IS_BF16>(__uint_as_float(orr[8 * q4 + 2]) * mul, __uint_as_float(orr[8 * q4 + 3]) * mul);
            v.z = pack2<IS_BF16>(__uint_as_float(orr[8 * q4 + 4]) * mul, __uint_as_float(orr[8 * q4 + 5]) * mul);
            v.w = pack2<IS_BF16>(__uint_as_float(orr[8 * q4 + 6]) * mul, __uint_as_float(orr[8 * q4 + 7]) * mul);
            const int chunk = 4 * c + q4;
            *reinterpret_cast<uint4*>(stage + r * pitch + stage_chunk<BIG>(chunk, r)) = v;
          }
        }
        __syncwarp();   // each warp stores the 32 rows it staged itself: no cross-warp dependency
        uint16_t* gout = pz == 0
            ? reinterpret_cast<uint16_t*>(p.dk) + b * p.dk_b + (int64_t)row0 * p.dk_s + hk * p.dk_h
            : reinterpret_cast<uint16_t*>(p.dv) + b * p.dv_b + (int64_t)row0 * p.dv_s + hk * p.dv_h;
        const int64_t ld = pz == 0 ? p.dk_s : p.dv_s;
        const int width = pz == 0 ? p.d : p.dv_dim;   // columns past the head dim hold products of zero fill
        const int wrow = (warp & 3) * 32;
        const int cpr = ncol / 8;                     // 16-byte chunks per row
#pragma unroll 4
        for (int x = lane; x < 32 * cpr; x += 32) {
          const int rr = wrow + x / cpr, cc = x % cpr;
          if (row0 + rr < p.Sk && cc * 8 < width)
            *reinterpret_cast<uint4*>(gout + (int64_t)rr * ld + cc * 8) =
                *reinterpret_cast<const uint4*>(stage + rr * pitch + stage_chunk<BIG>(cc, rr));
        }
      } else {
        // both warpgroups: dQ columns [D/2 pz, D/2 pz + D/2), staged in the Q tile
        const uint32_t tA = tmem + lane_field + C_ACC1 + (uint32_t)(D / 2) * pz;
        uint8_t* stage = smem + Cfg::OFF_STAT;
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          uint32_t orr[32];
          if (K_items > 0) { tmem_ld32(tA + 32 * c, orr); tc_wait_ld(); }
          else {
#pragma unroll
            for (int j = 0; j < 32; ++j) orr[j] = 0u;
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 v;
            v.x = pack2<IS_BF16>(__uint_as_float(orr[8 * q4 + 0]) * p.scale, __uint_as_float(orr[8 * q4 + 1]) * p.scale);
            v.y = pack2<IS_BF16>(__uint_as_float(orr[8 * q4 + 2]) * p.scale, __uint_as_float(orr[8 * q4 + 3]) * p.scale);
            v.z = pack2<IS_BF16>(__uint_as_float(orr[8 * q4 + 4]) * p.scale, __uint_as_float(orr[8 * q4 + 5]) * p.scale);
            v.w = pack2<IS_BF16>(__uint_as_float(orr[8 * q4 + 6]) * p.scale, __uint_as_float(orr[8 * q4 + 7]) * p.scale);
            const int chunk = (D / 16) * pz + 4 * c + q4;
            *reinterpret_cast<uint4*>(stage + r * (Cfg::W1 * 2) + stage_chunk<BIG>(chunk, r)) = v;
          }
        }
        __syncwarp();   // warp-local transpose through the staging tile
        uint16_t* gout = reinterpret_cast<uint16_t*>(p.dq) + b * p.dq_b + (int64_t)row0 * p.dq_s + hq0 * p.dq_h;
        const int wrow = (warp & 3) * 32;
#pragma unroll 4
        for (int x = lane; x < 32 * (D / 16); x += 32) {
          const int rr = wrow + x / (D / 16), cc = (D / 16) * pz + x % (D / 16);
          if (row0 + rr < p.Sq && cc * 8 < p.d)
            *reinterpret_cast<uint4*>(gout + (int64_t)rr * p.dq_s + cc * 8) =
                *reinterpret_cast<const uint4*>(stage + rr * (Cfg::W1 * 2) + stage_chunk<BIG>(cc, rr));
        }
      }
      if (tid == 0) PROF(8);
    }
  } else {
    if (warp == 8) {
      // =========================== producer ===========================
      bool ok = true;
      for (int k = 0; k < K_items && ok; ++k) {
        const uint32_t e = list[k % cnt];
        const int idx = (int)(e & 0xFFFFu);
        const uint32_t flags = e >> 16;
        const int slot = k % Cfg::NSLOT;
        const uint32_t par = ((uint32_t)(k / Cfg::NSLOT) & 1u) ^ 1u;
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
          mbar_arrive_expect_tx(fb, (D / 64 + DV / 64) * Cfg::SUB64 + (MODE == MODE_DKDV ? 512 : 0));
          for (int dc = 0; dc < D / 64; ++dc)
            tma_load_4d(dst + dc * Cfg::SUB64, &tm_str1, fb, dc * 64, hstr, idx * 64, b);
          for (int dc = 0; dc < DV / 64; ++dc)
            tma_load_4d(dst + Cfg::OP1_BYTES + dc * Cfg::SUB64, &tm_str2, fb, dc * 64, hstr, idx * 64, b);
          if (MODE == MODE_DKDV) {
            const int64_t at = ((int64_t)b * p.Hq + hstr) * p.Sq_r + idx * 64;
            const uint32_t ax = sbase + Cfg::OFF_AUX + slot * Cfg::AUX_BYTES;
            bulk_copy_g2s(ax, p.lse_log2 + at, 256, fb);
            bulk_copy_g2s(ax + 256, p.dpsum + at, 256, fb);
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
    } else if (warp == 9) {
      // =========================== UMMA issuer ===========================
      if (K_items > 0 && elect_one()) {
        constexpr uint32_t idesc_g = make_idesc(IS_BF16, 128, 64, 0, 0);
        constexpr uint32_t idesc_acc1 = make_idesc(IS_BF16, 128, D, 0, 1);    // dK / dQ: N = D
        constexpr uint32_t idesc_acc2 = make_idesc(IS_BF16, 128, DV, 0, 1);   // dV: N = DV
        bool ok = mbar_wait(bar(Cfg::B_STAT), 0u, wc);
        PROF(2);
        // descriptors are built once; per MMA only a constant is added to the
        // 14-bit address field (all smem offsets are multiples of 16 bytes)
        const uint64_t dA1 = make_sdesc(sStat, 16, 1024);
        const uint64_t dA2 = make_sdesc(sStat + Cfg::STAT1_BYTES, 16, 1024);
        const uint64_t dRk = make_sdesc(sRing, 16, 1024);            // K-major view of a ring slot
        const uint64_t dRm = make_sdesc(sRing, Cfg::SUB64, 1024);    // MN-major view of a ring slot
        // first score GEMM of item k (S or S^T, D / 16 k-steps); waits for the ring slot
        auto issue_g1 = [&](int k) {
          const int slot = k % Cfg::NSLOT, pz = k & 1;
          TRACE(1, 20, k);                    // about to wait for the ring slot
          ok = ok && mbar_wait(bar(Cfg::B_RFULL + slot), (uint32_t)(k / Cfg::NSLOT) & 1u, wc);
          if (!ok) return;
          TRACE(1, 21, k);                    // ring slot full
          tc_fence_after();
          const uint64_t db1 = dRk + (uint64_t)(slot * (Cfg::SLOT_BYTES >> 4));
          const uint32_t dst = tmem + C_G1 + 64u * pz;
          if constexpr (D >= 128) umma_ss_x8<(Cfg::SUB128 >> 4), (Cfg::SUB64 >> 4)>(dst, dA1, db1, idesc_g, 0u);
          else umma_ss_x4(dst, dA1, db1, idesc_g, 0u);
          if constexpr (D == 192)
            umma_ss_x4(dst, dA1 + (uint64_t)(2 * (Cfg::SUB128 >> 4)), db1 + (uint64_t)(2 * (Cfg::SUB64 >> 4)), idesc_g, 1u);
          TRACE(1, 22, k);                    // G issued
        };
        // second score GEMM (dP or dP^T, DV / 16 k-steps) and the commit that publishes both
        auto issue_g2 = [&](int k) {
          const int slot = k % Cfg::NSLOT, pz = k & 1;
          const uint64_t db2 = dRk + (uint64_t)(slot * (Cfg::SLOT_BYTES >> 4) + (Cfg::OP1_BYTES >> 4));
          const uint32_t dst = tmem + C_G2 + (BIG ? 0u : 64u * pz);
          if constexpr (DV == 128) umma_ss_x8<(Cfg::SUB128 >> 4), (Cfg::SUB64 >> 4)>(dst, dA2, db2, idesc_g, 0u);
          else umma_ss_x4(dst, dA2, db2, idesc_g, 0u);
          tc_commit(bar(Cfg::B_GFULL + pz));
        };
        // accumulation MMAs of item k; their completion frees the ring slot
        auto issue_acc = [&](int k) {
          const int slot = k % Cfg::NSLOT, pz = k & 1;
          const uint64_t dm1 = dRm + (uint64_t)(slot * (Cfg::SLOT_BYTES >> 4));     // streamed operand 1
          const uint64_t dm2 = dm1 + (uint64_t)(Cfg::OP1_BYTES >> 4);                // streamed operand 2
          const uint32_t acc_on = k > 0 ? 1u : 0u;
          if (MODE == MODE_DKDV) {
            // dV += P^T dO (streamed operand 2), dK += dS^T Q (streamed operand 1)
            const uint32_t t1 = tmem + (BIG ? C_G1 : C_G2) + 64u * pz, t2 = t1 + 32u;
            umma_ts_xn<4>(tmem + C_ACC1, t1, dm2, idesc_acc2, acc_on);
            umma_ts_xn<4>(tmem + C_ACC2, t2, dm1, idesc_acc1, acc_on);
          } else {
            // dQ += dS K (streamed operand 1)
            const uint32_t t2 = BIG ? tmem + C_G1 + 64u * pz
                                    : tmem + C_T + 32u * (uint32_t)((((k >> 1) & 1) << 1) + pz);
            umma_ts_xn<4>(tmem + C_ACC1, t2, dm1, idesc_acc1, acc_on);
          }
          tc_commit(bar(Cfg::B_REMPTY + slot));
          TRACE(1, 25, k);                    // ACC issued
        };
        if constexpr (!BIG) {
          // S (S^T) of item k+2 runs as soon as the warpgroup of this parity has READ item k out of the
          // score buffers; dP (dP^T) follows the accumulation MMAs of item k (in DKDV mode it overwrites
          // the buffer that held that item's P^T / dS^T)
          issue_g1(0); PROF(3); if (ok) issue_g2(0);
          if (K_items > 1 && ok) { issue_g1(1); if (ok) issue_g2(1); }
          for (int k = 0; k < K_items && ok; ++k) {
            const int pz = k & 1;
            if (k + 2 < K_items) {
              ok = mbar_wait(bar(Cfg::B_GREAD + pz), (uint32_t)(k >> 1) & 1u, wc);
              if (!ok) break;
              issue_g1(k + 2);
              if (!ok) break;
            }
            TRACE(1, 23, k);                    // about to wait for T
            ok = mbar_wait(bar(Cfg::B_TFULL + pz), (uint32_t)(k >> 1) & 1u, wc);
            if (!ok) break;
            TRACE(1, 24, k);                    // T ready
            tc_fence_after();
            issue_acc(k);
            if (k + 2 < K_items) issue_g2(k + 2);
          }
        } else {
          // one dP (dP^T) buffer: item k+1's may only be issued once item k's has been read
          issue_g1(0); PROF(3); if (ok) issue_g2(0);
          if (K_items > 1 && ok) {
            issue_g1(1);
            ok = ok && mbar_wait(bar(Cfg::B_GREAD + 0), 0u, wc);
            if (ok) issue_g2(1);
          }
          for (int k = 0; k < K_items && ok; ++k) {
            const int pz = k & 1;
            ok = mbar_wait(bar(Cfg::B_TFULL + pz), (uint32_t)(k >> 1) & 1u, wc);
            if (!ok) break;
            tc_fence_after();
            issue_acc(k);
            if (k + 2 < K_items) {
              issue_g1(k + 2);                  // after item k's accumulation MMAs: its overlay is dead
              if (!ok) break;
              ok = mbar_wait(bar(Cfg::B_GREAD + (pz ^ 1)), (uint32_t)((k + 1) >> 1) & 1u, wc);
              if (!ok) break;
              issue_g2(k + 2);
            }
          }
        }
        if (ok) tc_commit(bar(Cfg::B_ACC));
        PROF(6);
      }
      __syncwarp();
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
    if (tid == 0) atomicExch(&g_bwd_status, FM_ERR_TIMEOUT);
  }
  if (warp == 9) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------
// host
// ---------------------------------------------------------------------------
bool bwd_sm100_supported(const fm_attn_args* a) {
  const bool small = a->d <= 128 && a->dv <= 128 && a->d % 8 == 0 && a->dv % 8 == 0;
  if (!small && !(a->d == 192 && a->dv == 128)) return false;
  if (((uintptr_t)a->q | (uintptr_t)a->k | (uintptr_t)a->v | (uintptr_t)a->d_o) & 15) return false;
  return true;
}

template <bool IS_BF16, int D, int DV>
static int launch_bwd_sm100(const AttnKParams& p, const fm_attn_args* a, cudaStream_t s) {
  using Cfg = BwdSm100Cfg<D>;
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
  auto k1 = bwd_sm100_kernel<MODE_DKDV, IS_BF16, D, DV>;
  auto k2 = bwd_sm100_kernel<MODE_DQ, IS_BF16, D, DV>;
  FM_CUDA_TRY(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
  FM_CUDA_TRY(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
  k1<<<dim3((p.Sk + 127) / 128, p.Hkv, p.B), Cfg::NTHREADS, Cfg::SMEM, s>>>(k128, v128, q64, do64, p);
  FM_CUDA_TRY(cudaGetLastError());
  k2<<<dim3((p.Sq + 127) / 128, p.Hq, p.B), Cfg::NTHREADS, Cfg::SMEM, s>>>(q128, do128, k64, v64, p);
  count_launches(2);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

int bwd_sm100_launch(const AttnKParams& p, const fm_attn_args* a, cudaStream_t s) {
  const bool bf = a->dtype == FM_DTYPE_BF16;
  if (a->d > 128) return bf ? launch_bwd_sm100<true, 192, 128>(p, a, s) : launch_bwd_sm100<false, 192, 128>(p, a, s);
  if (a->d <= 64 && a->dv <= 64) return bf ? launch_bwd_sm100<true, 64, 64>(p, a, s) : launch_bwd_sm100<false, 64, 64>(p, a, s);
  return bf ? launch_bwd_sm100<true, 128, 128>(p, a, s) : launch_bwd_sm100<false, 128, 128>(p, a, s);
}

#ifdef FM_TRACE
extern "C" __attribute__((visibility("default"))) int fm_debug_trace_read(int* out) {
  cudaMemcpyFromSymbol(out, g_trace, sizeof(int) * 4 * 3 * 2048);
  cudaMemset(nullptr, 0, 0);
  static int zeros[4 * 3 * 2048];
  cudaMemcpyToSymbol(g_trace, zeros, sizeof(zeros));
  return 0;
}
extern "C" __attribute__((visibility("default"))) int fm_debug_prof_read(long long* out) {
  return (int)cudaMemcpyFromSymbol(out, g_prof, sizeof(long long) * 2 * 64 * 16);
}
#endif

int bwd_sm100_status(int* out, bool reset) {
  int v = 0;
  FM_CUDA_TRY(cudaMemcpyFromSymbol(&v, g_bwd_status, sizeof(int)));
  if (reset && v != 0) {
    const int z = 0;
    FM_CUDA_TRY(cudaMemcpyToSymbol(g_bwd_status, &z, sizeof(int)));
  }
  *out = v;
  return FM_OK;
}

}  // namespace fm

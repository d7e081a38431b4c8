// Backward attention with warp-level tensor-core MMA (mma.sync m16n8k16): the
// general head-dim variant.  Three kernels on one stream:
//   1. preprocess   dPsum = rowsum(O * dO), LSE * log2(e)
//   2. dK/dV        one CTA per (K tile, kv head, batch), loops over the q heads
//                   of the group and the Q tiles that are not skipped
//   3. dQ           one CTA per (Q tile, q head, batch), loops over K tiles
// plus dsink.  Every output element is produced by exactly one thread with a
// fixed summation order, so the gradients are bitwise reproducible; no fp32
// accumulator buffer in global memory and no atomics are needed.
#include "fm_attn_params.cuh"

namespace fm {

template <int ROW_BYTES>
__device__ __forceinline__ uint32_t swz_any(int row, int chunk) {
  if constexpr (ROW_BYTES % 128 == 0) return (uint32_t)row * ROW_BYTES + (uint32_t)((chunk ^ (row & 7)) << 4);
  else if constexpr (ROW_BYTES == 64) return (uint32_t)row * ROW_BYTES + (uint32_t)((chunk ^ ((row >> 1) & 3)) << 4);
  else return (uint32_t)row * ROW_BYTES + (uint32_t)(chunk << 4);
}

template <int ROWS, int COLS, int NTHREADS>
__device__ __forceinline__ void bwd_load_tile_async(uint32_t smem_base, const uint16_t* g, int64_t ld,
                                                    int rows_valid, int cols_valid, int tid) {
  constexpr int CHUNKS = COLS / 8;
  for (int idx = tid; idx < ROWS * CHUNKS; idx += NTHREADS) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const bool ok = r < rows_valid && c * 8 < cols_valid;
    const uint16_t* src = ok ? g + (int64_t)r * ld + c * 8 : g;
    cp_async16(smem_base + swz_any<COLS * 2>(r, c), src, ok);
  }
}

template <int D, int DV, int BR, int BC>
struct BwdMmaCfg {
  static constexpr int NWARP = 8;
  static constexpr int NTHREADS = 256;
  static constexpr int ROW_G = BR / 16;          // warp row groups in phase A
  static constexpr int COL_G = NWARP / ROW_G;    // warp column groups in phase A
  static constexpr int COLS_W = BC / COL_G;      // S columns per warp
  static constexpr int NT_A = COLS_W / 8;
  static constexpr int K_BYTES = BC * D * 2, V_BYTES = BC * DV * 2;
  static constexpr int Q_BYTES = BR * D * 2, DO_BYTES = BR * DV * 2;
  static constexpr int P_BYTES = BR * BC * 2;
  static constexpr int ROWF_BYTES = 2 * BR * 4;  // lse_log2, dpsum
  static constexpr int BND_BYTES = 4 * BC * 4;
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = OFF_K + K_BYTES;
  static constexpr int OFF_Q = OFF_V + V_BYTES;
  static constexpr int OFF_DO = OFF_Q + Q_BYTES;
  static constexpr int OFF_P = OFF_DO + DO_BYTES;
  static constexpr int OFF_DS = OFF_P + P_BYTES;
  static constexpr int OFF_ROWF = OFF_DS + P_BYTES;
  static constexpr int OFF_BND = OFF_ROWF + ROWF_BYTES;
  static constexpr int SMEM = OFF_BND + BND_BYTES;
  static_assert(ROW_G * COL_G == NWARP && COLS_W % 16 == 0, "phase A warp layout");
};

// Phase A: this warp's 16 x COLS_W slab of P and dS, written to smem as bf16.
//   S = Q K^T, dP = dO V^T, P = exp2(S*scale_log2 - lse_log2), dS = P*(dP - dPsum)
template <int D, int DV, int BR, int BC, bool IS_BF16, bool WRITE_P>
__device__ __forceinline__ void phase_a(uint8_t* smem, const AttnKParams& p, int cls, int ms, int j0,
                                        int warp, int lane) {
  using Cfg = BwdMmaCfg<D, DV, BR, BC>;
  const uint32_t sK = smem_u32(smem + Cfg::OFF_K), sV = smem_u32(smem + Cfg::OFF_V);
  const uint32_t sQ = smem_u32(smem + Cfg::OFF_Q), sdO = smem_u32(smem + Cfg::OFF_DO);
  const float* sLse = reinterpret_cast<const float*>(smem + Cfg::OFF_ROWF);
  const float* sDps = sLse + BR;
  const int* sB = reinterpret_cast<const int*>(smem + Cfg::OFF_BND);
  const int wr = warp % Cfg::ROW_G, wc = warp / Cfg::ROW_G;
  const int g = lane >> 2, tq = lane & 3;
  constexpr int NT = Cfg::NT_A;
  float s[NT][4], dp[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) {
    s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    dp[i][0] = dp[i][1] = dp[i][2] = dp[i][3] = 0.f;
  }
  const int row_a = wr * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
  const int col_a = lane >> 4;
  const int brow = wc * Cfg::COLS_W + (lane & 7) + (lane >> 4) * 8;
  const int bcol = (lane >> 3) & 1;
#pragma unroll 4
  for (int kk = 0; kk < D / 16; ++kk) {
    uint32_t a[4];
    ldmatrix_x4(a, sQ + swz_any<D * 2>(row_a, kk * 2 + col_a));
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t bfr[4];
      ldmatrix_x4(bfr, sK + swz_any<D * 2>(brow + np * 16, kk * 2 + bcol));
      mma16816<IS_BF16>(s[2 * np], a, bfr[0], bfr[1]);
      mma16816<IS_BF16>(s[2 * np + 1], a, bfr[2], bfr[3]);
    }
  }
#pragma unroll 4
  for (int kk = 0; kk < DV / 16; ++kk) {
    uint32_t a[4];
    ldmatrix_x4(a, sdO + swz_any<DV * 2>(row_a, kk * 2 + col_a));
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t bfr[4];
      ldmatrix_x4(bfr, sV + swz_any<DV * 2>(brow + np * 16, kk * 2 + bcol));
      mma16816<IS_BF16>(dp[2 * np], a, bfr[0], bfr[1]);
      mma16816<IS_BF16>(dp[2 * np + 1], a, bfr[2], bfr[3]);
    }
  }
  const int off = p.Sk - p.Sq;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int lrow = wr * 16 + g + r * 8;
    const int row = ms + lrow;
    const float lse2 = sLse[lrow], dps = sDps[lrow];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      float pv[2], dsv[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int cl = wc * Cfg::COLS_W + i * 8 + tq * 2 + e;
        bool masked = false;
        if (cls == FM_TILE_PARTIAL) {
          const int lts = sB[cl], lte = sB[BC + cl], uts = sB[2 * BC + cl], ute = sB[3 * BC + cl];
          masked = (row >= lts && row < lte) || (row >= uts && row < ute);
          if (p.md.causal) masked = masked || (j0 + cl > row + off);
        }
        const float pe = masked ? 0.f : fast_exp2(s[i][2 * r + e] * p.scale_log2 - lse2);
        pv[e] = pe;
        dsv[e] = pe * (dp[i][2 * r + e] - dps);
      }
      const int col = wc * Cfg::COLS_W + i * 8 + tq * 2;
      const uint32_t o = swz_any<BC * 2>(lrow, col >> 3) + (col & 7) * 2;
      if (WRITE_P) *reinterpret_cast<uint32_t*>(smem + Cfg::OFF_P + o) = pack2<IS_BF16>(pv[0], pv[1]);
      *reinterpret_cast<uint32_t*>(smem + Cfg::OFF_DS + o) = pack2<IS_BF16>(dsv[0], dsv[1]);
    }
  }
}

// acc[BCT][NT][4] += A^T-style product: OUT[n][c] += sum_m X[m][n] * Y[m][c]
// X is an [BR][BC] smem tile (sP or sdS), Y an [BR][COLS] smem tile (sdO or sQ);
// this warp owns output columns [c0, c0 + NT*8).
template <int BR, int BC, int COLS, int NT, bool IS_BF16>
__device__ __forceinline__ void accum_xT_y(float (&acc)[BC / 16][NT][4], uint32_t sX, uint32_t sY,
                                           int c0, int lane) {
#pragma unroll
  for (int kk = 0; kk < BR / 16; ++kk) {
    uint32_t bfr[NT][2];
    const int yrow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t t4[4];
      ldmatrix_x4_trans(t4, sY + swz_any<COLS * 2>(yrow, c0 / 8 + np * 2 + (lane >> 4)));
      bfr[2 * np][0] = t4[0]; bfr[2 * np][1] = t4[1];
      bfr[2 * np + 1][0] = t4[2]; bfr[2 * np + 1][1] = t4[3];
    }
    if constexpr (NT % 2 == 1) {
      uint32_t t2[2];
      ldmatrix_x2_trans(t2, sY + swz_any<COLS * 2>(yrow, c0 / 8 + (NT - 1)));
      bfr[NT - 1][0] = t2[0]; bfr[NT - 1][1] = t2[1];
    }
#pragma unroll
    for (int i = 0; i < BC / 16; ++i) {
      uint32_t a[4];
      const int xrow = kk * 16 + (lane & 7) + (lane >> 4) * 8;
      ldmatrix_x4_trans(a, sX + swz_any<BC * 2>(xrow, i * 2 + ((lane >> 3) & 1)));
#pragma unroll
      for (int c = 0; c < NT; ++c) mma16816<IS_BF16>(acc[i][c], a, bfr[c][0], bfr[c][1]);
    }
  }
}

// Stage this warp's accumulator slab (rows x its column slice) as bf16 into a
// swizzled smem tile of COLS columns.
template <int ROWT, int NT, int COLS, bool IS_BF16>
__device__ __forceinline__ void stage_acc(uint8_t* tile, const float (&acc)[ROWT][NT][4], int c0,
                                          int lane, float mul) {
  const int g = lane >> 2, tq = lane & 3;
#pragma unroll
  for (int i = 0; i < ROWT; ++i)
#pragma unroll
    for (int c = 0; c < NT; ++c)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int row = i * 16 + g + r * 8, col = c0 + c * 8 + tq * 2;
        *reinterpret_cast<uint32_t*>(tile + swz_any<COLS * 2>(row, col >> 3) + (col & 7) * 2) =
            pack2<IS_BF16>(acc[i][c][2 * r] * mul, acc[i][c][2 * r + 1] * mul);
      }
}

template <int ROWS, int COLS, int NTHREADS>
__device__ __forceinline__ void store_tile(const uint8_t* tile, uint16_t* g, int64_t ld, int rows_valid,
                                           int cols_valid, int tid) {
  constexpr int CH = COLS / 8;
  for (int idx = tid; idx < ROWS * CH; idx += NTHREADS) {
    const int r = idx / CH, c = idx % CH;
    if (r < rows_valid && c * 8 < cols_valid)
      *reinterpret_cast<uint4*>(g + (int64_t)r * ld + c * 8) =
          *reinterpret_cast<const uint4*>(tile + swz_any<COLS * 2>(r, c));
  }
}

__device__ __forceinline__ void stage_bounds(const AttnKParams& p, int bh_mask, int j0, int BC, int* sB,
                                             int tid) {
  if (tid < BC) {
    const int j = j0 + tid;
    Bounds4 bd;
    if (j >= p.Sk) { bd.lts = 0; bd.lte = INT_MAX; bd.uts = 0; bd.ute = 0; }
    else if (p.md.ncols) bd = load_bounds(p.md, p.md.mask + ((size_t)bh_mask * p.Sk + j) * p.md.ncols);
    else { bd.lts = INT_MAX; bd.lte = INT_MAX; bd.uts = 0; bd.ute = 0; }
    sB[tid] = bd.lts; sB[BC + tid] = bd.lte; sB[2 * BC + tid] = bd.uts; sB[3 * BC + tid] = bd.ute;
  }
}

// ---------------------------------------------------------------------------
// dK / dV: K-tile stationary
// ---------------------------------------------------------------------------
template <int D, int DV, int BR, int BC, bool IS_BF16>
__global__ void __launch_bounds__(256) bwd_dkdv_mma_kernel(const AttnKParams p) {
  using Cfg = BwdMmaCfg<D, DV, BR, BC>;
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const MaskDesc& md = p.md;
  const int j0 = n * BC;
  const int off = p.Sk - p.Sq;
  const int n_q_tiles = (p.Sq + BR - 1) / BR;
  const int bh_mask = md.ncols ? ((md.mask_B == 1 ? 0 : b) * md.Hm + (hk * G) / (p.Hq / md.Hm)) : 0;
  const uint32_t sK = smem_u32(smem + Cfg::OFF_K), sV = smem_u32(smem + Cfg::OFF_V);
  const uint32_t sQ = smem_u32(smem + Cfg::OFF_Q), sdO = smem_u32(smem + Cfg::OFF_DO);
  const uint32_t sP = smem_u32(smem + Cfg::OFF_P), sdS = smem_u32(smem + Cfg::OFF_DS);
  float* sLse = reinterpret_cast<float*>(smem + Cfg::OFF_ROWF);
  float* sDps = sLse + BR;
  int* sB = reinterpret_cast<int*>(smem + Cfg::OFF_BND);

  const uint16_t* gk = reinterpret_cast<const uint16_t*>(p.k) + b * p.k_b + (int64_t)j0 * p.k_s + hk * p.k_h;
  const uint16_t* gv = reinterpret_cast<const uint16_t*>(p.v) + b * p.v_b + (int64_t)j0 * p.v_s + hk * p.v_h;
  bwd_load_tile_async<BC, D, 256>(sK, gk, p.k_s, p.Sk - j0, p.d, tid);
  bwd_load_tile_async<BC, DV, 256>(sV, gv, p.v_s, p.Sk - j0, p.dv_dim, tid);
  cp_async_commit();
  stage_bounds(p, bh_mask, j0, BC, sB, tid);

  constexpr int NT_K = D / 64, NT_V = DV / 64;  // n8 tiles of this warp's column slice
  float acc_dk[BC / 16][NT_K][4], acc_dv[BC / 16][NT_V][4];
#pragma unroll
  for (int i = 0; i < BC / 16; ++i) {
#pragma unroll
    for (int c = 0; c < NT_K; ++c) acc_dk[i][c][0] = acc_dk[i][c][1] = acc_dk[i][c][2] = acc_dk[i][c][3] = 0.f;
#pragma unroll
    for (int c = 0; c < NT_V; ++c) acc_dv[i][c][0] = acc_dv[i][c][1] = acc_dv[i][c][2] = acc_dv[i][c][3] = 0.f;
  }

  int m_lo = 0;
  if (md.causal) m_lo = max(0, (j0 - off) / BR);
  for (int gq = 0; gq < G; ++gq) {
    const int hq = hk * G + gq;
    const uint16_t* gQ = reinterpret_cast<const uint16_t*>(p.q) + b * p.q_b + hq * p.q_h;
    const uint16_t* gdO = reinterpret_cast<const uint16_t*>(p.d_o) + b * p.do_b + hq * p.do_h;
    const float* gLse = p.lse_log2 + ((int64_t)b * p.Hq + hq) * p.Sq_r;
    const float* gDps = p.dpsum + ((int64_t)b * p.Hq + hq) * p.Sq_r;
    for (int m = m_lo; m < n_q_tiles; ++m) {
      const int ms = m * BR, me = min(ms + BR, p.Sq);
      const int cls = classify_tile(md, bh_mask, n, ms, me, BC);
      if (cls == FM_TILE_SKIP) continue;
      __syncthreads();  // previous tile's phase B finished with sQ/sdO/sP/sdS
      bwd_load_tile_async<BR, D, 256>(sQ, gQ + (int64_t)ms * p.q_s, p.q_s, me - ms, p.d, tid);
      bwd_load_tile_async<BR, DV, 256>(sdO, gdO + (int64_t)ms * p.do_s, p.do_s, me - ms, p.dv_dim, tid);
      cp_async_commit();
      if (tid < BR) {
        const bool ok = ms + tid < p.Sq;
        sLse[tid] = ok ? gLse[ms + tid] : 0.f;
        sDps[tid] = ok ? gDps[ms + tid] : 0.f;
      }
      cp_async_wait<0>();
      __syncthreads();
      phase_a<D, DV, BR, BC, IS_BF16, true>(smem, p, cls, ms, j0, warp, lane);
      __syncthreads();
      accum_xT_y<BR, BC, DV, NT_V, IS_BF16>(acc_dv, sP, sdO, warp * (DV / 8), lane);
      accum_xT_y<BR, BC, D, NT_K, IS_BF16>(acc_dk, sdS, sQ, warp * (D / 8), lane);
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  stage_acc<BC / 16, NT_K, D, IS_BF16>(smem + Cfg::OFF_K, acc_dk, warp * (D / 8), lane, p.scale);
  stage_acc<BC / 16, NT_V, DV, IS_BF16>(smem + Cfg::OFF_V, acc_dv, warp * (DV / 8), lane, 1.f);
  __syncthreads();
  uint16_t* gdk = reinterpret_cast<uint16_t*>(p.dk) + b * p.dk_b + (int64_t)j0 * p.dk_s + hk * p.dk_h;
  uint16_t* gdv = reinterpret_cast<uint16_t*>(p.dv) + b * p.dv_b + (int64_t)j0 * p.dv_s + hk * p.dv_h;
  store_tile<BC, D, 256>(smem + Cfg::OFF_K, gdk, p.dk_s, p.Sk - j0, p.d, tid);
  store_tile<BC, DV, 256>(smem + Cfg::OFF_V, gdv, p.dv_s, p.Sk - j0, p.dv_dim, tid);
}

// ---------------------------------------------------------------------------
// dQ: Q-tile stationary
// ---------------------------------------------------------------------------
template <int D, int DV, int BR, int BC, bool IS_BF16>
__global__ void __launch_bounds__(256) bwd_dq_mma_kernel(const AttnKParams p) {
  using Cfg = BwdMmaCfg<D, DV, BR, BC>;
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n_q_tiles = (p.Sq + BR - 1) / BR;
  const int m = n_q_tiles - 1 - blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
  const int hk = hq / (p.Hq / p.Hkv);
  const MaskDesc& md = p.md;
  const int bh_mask = md.ncols ? ((md.mask_B == 1 ? 0 : b) * md.Hm + hq / (p.Hq / md.Hm)) : 0;
  const int ms = m * BR, me = min(ms + BR, p.Sq);
  const int off = p.Sk - p.Sq;
  const int nb = (p.Sk + BC - 1) / BC;
  const uint32_t sK = smem_u32(smem + Cfg::OFF_K), sV = smem_u32(smem + Cfg::OFF_V);
  const uint32_t sQ = smem_u32(smem + Cfg::OFF_Q), sdO = smem_u32(smem + Cfg::OFF_DO);
  const uint32_t sdS = smem_u32(smem + Cfg::OFF_DS);
  float* sLse = reinterpret_cast<float*>(smem + Cfg::OFF_ROWF);
  float* sDps = sLse + BR;
  int* sB = reinterpret_cast<int*>(smem + Cfg::OFF_BND);

  const uint16_t* gQ = reinterpret_cast<const uint16_t*>(p.q) + b * p.q_b + (int64_t)ms * p.q_s + hq * p.q_h;
  const uint16_t* gdO = reinterpret_cast<const uint16_t*>(p.d_o) + b * p.do_b + (int64_t)ms * p.do_s + hq * p.do_h;
  const uint16_t* gk = reinterpret_cast<const uint16_t*>(p.k) + b * p.k_b + hk * p.k_h;
  const uint16_t* gv = reinterpret_cast<const uint16_t*>(p.v) + b * p.v_b + hk * p.v_h;
  bwd_load_tile_async<BR, D, 256>(sQ, gQ, p.q_s, me - ms, p.d, tid);
  bwd_load_tile_async<BR, DV, 256>(sdO, gdO, p.do_s, me - ms, p.dv_dim, tid);
  cp_async_commit();
  if (tid < BR) {
    const bool ok = ms + tid < p.Sq;
    sLse[tid] = ok ? p.lse_log2[((int64_t)b * p.Hq + hq) * p.Sq_r + ms + tid] : 0.f;
    sDps[tid] = ok ? p.dpsum[((int64_t)b * p.Hq + hq) * p.Sq_r + ms + tid] : 0.f;
  }

  constexpr int NT_Q = D / 64;
  float acc[BR / 16][NT_Q][4];
#pragma unroll
  for (int i = 0; i < BR / 16; ++i)
#pragma unroll
    for (int c = 0; c < NT_Q; ++c) acc[i][c][0] = acc[i][c][1] = acc[i][c][2] = acc[i][c][3] = 0.f;

  int n_hi = nb;
  if (md.causal) n_hi = max(0, min(nb, (me + off + BC - 1) / BC));
  const int c0 = warp * (D / 8);
  for (int n = n_hi - 1; n >= 0; --n) {
    const int cls = classify_tile(md, bh_mask, n, ms, me, BC);
    if (cls == FM_TILE_SKIP) continue;
    const int j0 = n * BC;
    __syncthreads();
    bwd_load_tile_async<BC, D, 256>(sK, gk + (int64_t)j0 * p.k_s, p.k_s, p.Sk - j0, p.d, tid);
    bwd_load_tile_async<BC, DV, 256>(sV, gv + (int64_t)j0 * p.v_s, p.v_s, p.Sk - j0, p.dv_dim, tid);
    cp_async_commit();
    if (cls == FM_TILE_PARTIAL) stage_bounds(p, bh_mask, j0, BC, sB, tid);
    cp_async_wait<0>();
    __syncthreads();
    phase_a<D, DV, BR, BC, IS_BF16, false>(smem, p, cls, ms, j0, warp, lane);
    __syncthreads();
    // dQ[m][c] += sum_n dS[m][n] K[n][c]
#pragma unroll
    for (int kk = 0; kk < BC / 16; ++kk) {
      uint32_t bfr[NT_Q][2];
      const int krow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int np = 0; np < NT_Q / 2; ++np) {
        uint32_t t4[4];
        ldmatrix_x4_trans(t4, sK + swz_any<D * 2>(krow, c0 / 8 + np * 2 + (lane >> 4)));
        bfr[2 * np][0] = t4[0]; bfr[2 * np][1] = t4[1];
        bfr[2 * np + 1][0] = t4[2]; bfr[2 * np + 1][1] = t4[3];
      }
      if constexpr (NT_Q % 2 == 1) {
        uint32_t t2[2];
        ldmatrix_x2_trans(t2, sK + swz_any<D * 2>(krow, c0 / 8 + (NT_Q - 1)));
        bfr[NT_Q - 1][0] = t2[0]; bfr[NT_Q - 1][1] = t2[1];
      }
#pragma unroll
      for (int i = 0; i < BR / 16; ++i) {
        uint32_t a[4];
        const int arow = i * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldmatrix_x4(a, sdS + swz_any<BC * 2>(arow, kk * 2 + (lane >> 4)));
#pragma unroll
        for (int c = 0; c < NT_Q; ++c) mma16816<IS_BF16>(acc[i][c], a, bfr[c][0], bfr[c][1]);
      }
    }
  }
  cp_async_wait<0>();
  __syncthreads();
  stage_acc<BR / 16, NT_Q, D, IS_BF16>(smem + Cfg::OFF_Q, acc, c0, lane, p.scale);
  __syncthreads();
  uint16_t* gdq = reinterpret_cast<uint16_t*>(p.dq) + b * p.dq_b + (int64_t)ms * p.dq_s + hq * p.dq_h;
  store_tile<BR, D, 256>(smem + Cfg::OFF_Q, gdq, p.dq_s, me - ms, p.d, tid);
}

// ---------------------------------------------------------------------------
// preprocess + dsink
// ---------------------------------------------------------------------------
// dPsum[b,h,i] = sum_c O[b,i,h,c] * dO[b,i,h,c]; lse_log2 = LSE * log2(e) (-inf -> 0).
// LPR lanes share one row (each lane owns 8-element chunks), so a warp covers
// 32 / LPR rows per pass and every lane has a 16-byte load in flight.
template <bool IS_BF16, int LPR>
__global__ void __launch_bounds__(256) bwd_preprocess_kernel(const AttnKParams p) {
  constexpr int RPW = 32 / LPR;                       // rows per warp
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPR, ln = lane % LPR;
  const int row = (blockIdx.x * 8 + warp) * RPW + sub, hq = blockIdx.y, b = blockIdx.z;
  float acc = 0.f, lse2 = 0.f;
  if (row < p.Sq) {
    const uint16_t* o = reinterpret_cast<const uint16_t*>(p.o) + b * p.o_b + (int64_t)row * p.o_s + hq * p.o_h;
    const uint16_t* d_o = reinterpret_cast<const uint16_t*>(p.d_o) + b * p.do_b + (int64_t)row * p.do_s + hq * p.do_h;
    for (int c = ln * 8; c < p.dv_dim; c += LPR * 8) {
      const uint4 a = *reinterpret_cast<const uint4*>(o + c);
      const uint4 g = *reinterpret_cast<const uint4*>(d_o + c);
      const uint32_t av[4] = {a.x, a.y, a.z, a.w}, gv[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 x, y;
        if constexpr (IS_BF16) {
          x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&av[e]));
          y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gv[e]));
        } else {
          x = __half22float2(*reinterpret_cast<const __half2*>(&av[e]));
          y = __half22float2(*reinterpret_cast<const __half2*>(&gv[e]));
        }
        acc += x.x * y.x + x.y * y.y;
      }
    }
    if (ln == 0) {
      const float l = p.lse[((int64_t)b * p.Hq + hq) * p.Sq + row];
      lse2 = (l == -INFINITY) ? 0.f : l * kLog2e;
    }
  }
#pragma unroll
  for (int o2 = LPR / 2; o2; o2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o2);
  if (p.dq_accum && !(p.bwd_flags & FM_BWD_DQ_CARRY) && row < p.Sq_r) {
    // one-kernel backward: this row of the fp32 dQ accumulator starts at zero (the lanes of the row share it)
    const int dacc = (p.d <= 64 && p.dv_dim <= 64) ? 64 : 128;
    float4* z = reinterpret_cast<float4*>(p.dq_accum + (((int64_t)b * p.Hq + hq) * p.Sq_r + row) * dacc);
    for (int c = ln; c < dacc / 4; c += LPR) z[c] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (ln == 0 && row < p.Sq_r) {
    const int64_t at = ((int64_t)b * p.Hq + hq) * p.Sq_r + row;
    p.dpsum[at] = acc;
    p.lse_log2[at] = lse2;
    if (p.stat_s) {
      // the same two values as 16-bit GEMM operands (hi + lo parts, negated): see the one-kernel backward
      const float c = lse2 / p.scale_log2;
      float c_hi, c_lo, d_hi, d_lo;
      if constexpr (IS_BF16) {
        c_hi = __bfloat162float(__float2bfloat16_rn(c)); c_lo = c - c_hi;
        d_hi = __bfloat162float(__float2bfloat16_rn(acc)); d_lo = acc - d_hi;
      } else {
        c_hi = __half2float(__float2half_rn(c)); c_lo = c - c_hi;
        d_hi = __half2float(__float2half_rn(acc)); d_lo = acc - d_hi;
      }
      *reinterpret_cast<uint4*>(p.stat_s + at * 8) = make_uint4(pack2<IS_BF16>(-c_hi, -c_lo), 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(p.stat_dp + at * 8) = make_uint4(pack2<IS_BF16>(-d_hi, -d_lo), 0u, 0u, 0u);
    }
  }
}

// dsink[h] = - sum_{b,i} exp2(sink*log2e - lse_log2) * dPsum, fixed-order reduce.
__global__ void __launch_bounds__(256) bwd_dsink_kernel(const AttnKParams p) {
  const int hq = blockIdx.x;
  const float s2 = p.sink[hq] * kLog2e;
  float acc = 0.f;
  for (int b = 0; b < p.B; ++b) {
    const float* l = p.lse_log2 + ((int64_t)b * p.Hq + hq) * p.Sq_r;
    const float* dps = p.dpsum + ((int64_t)b * p.Hq + hq) * p.Sq_r;
    for (int i = threadIdx.x; i < p.Sq; i += 256) acc += exp2f(s2 - l[i]) * dps[i];
  }
  __shared__ float red[8];
#pragma unroll
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < 8; ++w) s += red[w];
    p.dsink[hq] = -s;
  }
}

template <int D, int DV, int BR, int BC>
static int launch_bwd(const AttnKParams& p, int dtype, cudaStream_t s) {
  using Cfg = BwdMmaCfg<D, DV, BR, BC>;
  const int nb = (p.Sk + BC - 1) / BC, tq = (p.Sq + BR - 1) / BR;
  if (dtype == FM_DTYPE_BF16) {
    auto k1 = bwd_dkdv_mma_kernel<D, DV, BR, BC, true>;
    auto k2 = bwd_dq_mma_kernel<D, DV, BR, BC, true>;
    FM_CUDA_TRY(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
    FM_CUDA_TRY(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
    k1<<<dim3(nb, p.Hkv, p.B), 256, Cfg::SMEM, s>>>(p);
    k2<<<dim3(tq, p.Hq, p.B), 256, Cfg::SMEM, s>>>(p);
    count_launches(2);
  } else {
    auto k1 = bwd_dkdv_mma_kernel<D, DV, BR, BC, false>;
    auto k2 = bwd_dq_mma_kernel<D, DV, BR, BC, false>;
    FM_CUDA_TRY(cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
    FM_CUDA_TRY(cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
    k1<<<dim3(nb, p.Hkv, p.B), 256, Cfg::SMEM, s>>>(p);
    k2<<<dim3(tq, p.Hq, p.B), 256, Cfg::SMEM, s>>>(p);
    count_launches(2);
  }
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

int bwd_mma_tile_shape(int d, int dv, int* tile_m, int* tile_n) {
  if (d <= 128 && dv <= 128) { *tile_m = 64; *tile_n = 64; return FM_OK; }
  if (d == 192 && dv == 128) { *tile_m = 64; *tile_n = 64; return FM_OK; }
  if (d == 256 && dv == 256) { *tile_m = 64; *tile_n = 64; return FM_OK; }
  if ((d == 512 || d == 576) && dv == 512) { *tile_m = 64; *tile_n = 32; return FM_OK; }
  return FM_ERR_UNSUPPORTED;
}

template <int LPR>
static void launch_preprocess(const AttnKParams& p, int dtype, cudaStream_t s) {
  constexpr int rows_per_block = 8 * (32 / LPR);
  dim3 grid((p.Sq_r + rows_per_block - 1) / rows_per_block, p.Hq, p.B);
  if (dtype == FM_DTYPE_BF16) bwd_preprocess_kernel<true, LPR><<<grid, 256, 0, s>>>(p);
  else bwd_preprocess_kernel<false, LPR><<<grid, 256, 0, s>>>(p);
  count_launches(1);
}

int bwd_preprocess_launch(const AttnKParams& p, int dtype, cudaStream_t s) {
  const int chunks = p.dv_dim / 8;
  if (chunks <= 8) launch_preprocess<8>(p, dtype, s);
  else if (chunks <= 16) launch_preprocess<16>(p, dtype, s);
  else launch_preprocess<32>(p, dtype, s);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

int bwd_dsink_launch(const AttnKParams& p, cudaStream_t s) {
  bwd_dsink_kernel<<<p.Hq, 256, 0, s>>>(p);
  count_launches(1);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

int bwd_mma_launch(const AttnKParams& p, int dtype, cudaStream_t s) {
  const int d = p.d, dv = p.dv_dim;
  if (d <= 64 && dv <= 64) return launch_bwd<64, 64, 64, 64>(p, dtype, s);
  if (d <= 128 && dv <= 128) return launch_bwd<128, 128, 64, 64>(p, dtype, s);
  if (d == 192 && dv == 128) return launch_bwd<192, 128, 64, 64>(p, dtype, s);
  if (d == 256 && dv == 256) return launch_bwd<256, 256, 64, 64>(p, dtype, s);
  if ((d == 512 || d == 576) && dv == 512) return launch_bwd<576, 512, 64, 32>(p, dtype, s);
  set_error("backward: unsupported head dims (d=%d, dv=%d)", d, dv);
  return FM_ERR_UNSUPPORTED;
}

}  // namespace fm

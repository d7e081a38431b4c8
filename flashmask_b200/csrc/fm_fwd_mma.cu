// Forward attention with warp-level tensor-core MMA (mma.sync m16n8k16):
// the general head-dim variant (d in {64,128,192,256,576}, dv in
// {64,128,256,512}).  One CTA owns BR query rows of one (batch, q head) and
// walks the K tiles that the mask preprocessing did not classify as skipped;
// partial tiles get the element mask from the column bounds staged in shared
// memory, unmasked tiles skip all mask arithmetic.
#include "fm_attn_params.cuh"

namespace fm {

template <int D, int DV, int BR, int BC, int NSPLIT, bool IS_BF16>
struct FwdMmaCfg {
  static constexpr int ROW_WARPS = BR / 16;
  static constexpr int NWARP = ROW_WARPS * NSPLIT;
  static constexpr int NTHREADS = NWARP * 32;
  static constexpr int Q_BYTES = BR * D * 2;
  static constexpr int K_BYTES = BC * D * 2;
  static constexpr int V_BYTES = BC * DV * 2;
  static constexpr int BND_BYTES = 4 * BC * 4;
  static constexpr int SMEM = Q_BYTES + K_BYTES + V_BYTES + BND_BYTES;
  static constexpr int DV_W = DV / NSPLIT;  // output columns per warp
  static constexpr bool Q_IN_REGS = (D <= 128);
};

// Copy ROWS x COLS (elements, COLS*2 bytes per row) from global (row stride
// `ld` elements) into a swizzled smem tile, zero-filling rows >= rows_valid and
// columns >= cols_valid.
template <int ROWS, int COLS, int NTHREADS>
__device__ __forceinline__ void load_tile_async(uint32_t smem_base, const uint16_t* g, int64_t ld,
                                                int rows_valid, int cols_valid, int tid) {
  constexpr int CHUNKS = COLS / 8;
  for (int idx = tid; idx < ROWS * CHUNKS; idx += NTHREADS) {
    const int r = idx / CHUNKS, c = idx % CHUNKS;
    const bool ok = r < rows_valid && c * 8 < cols_valid;
    const uint16_t* src = ok ? g + (int64_t)r * ld + c * 8 : g;
    cp_async16(smem_base + swz<COLS * 2>(r, c), src, ok);
  }
}

template <int D, int DV, int BR, int BC, int NSPLIT, bool IS_BF16>
__global__ void __launch_bounds__(FwdMmaCfg<D, DV, BR, BC, NSPLIT, IS_BF16>::NTHREADS)
fwd_mma_kernel(const AttnKParams p) {
  using Cfg = FwdMmaCfg<D, DV, BR, BC, NSPLIT, IS_BF16>;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK = sQ + Cfg::Q_BYTES;
  const uint32_t sV = sK + Cfg::K_BYTES;
  int* sB = reinterpret_cast<int*>(smem + Cfg::Q_BYTES + Cfg::K_BYTES + Cfg::V_BYTES);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wr = warp % Cfg::ROW_WARPS, ws = warp / Cfg::ROW_WARPS;
  const int g = lane >> 2, tq = lane & 3;
  const int n_q_tiles = (p.Sq + BR - 1) / BR;
  const int t = n_q_tiles - 1 - blockIdx.x;  // heaviest causal tiles first
  const int hq = blockIdx.y, b = blockIdx.z;
  const int hk = hq / (p.Hq / p.Hkv);
  const MaskDesc& md = p.md;
  const int bh_mask = md.ncols ? ((md.mask_B == 1 ? 0 : b) * md.Hm + hq / (p.Hq / md.Hm)) : 0;
  const int ms = t * BR, me = min(ms + BR, p.Sq);
  const int off = p.Sk - p.Sq;
  const int nb = (p.Sk + BC - 1) / BC;

  const uint16_t* gq = reinterpret_cast<const uint16_t*>(p.q) + b * p.q_b + (int64_t)ms * p.q_s + hq * p.q_h;
  const uint16_t* gk = reinterpret_cast<const uint16_t*>(p.k) + b * p.k_b + hk * p.k_h;
  const uint16_t* gv = reinterpret_cast<const uint16_t*>(p.v) + b * p.v_b + hk * p.v_h;

  load_tile_async<BR, D, Cfg::NTHREADS>(sQ, gq, p.q_s, me - ms, p.d, tid);
  cp_async_commit();

  int n_hi = nb;
  if (md.causal) n_hi = max(0, min(nb, (me + off + BC - 1) / BC));

  constexpr int NT_S = BC / 8;          // n8 tiles of S per warp row-slab
  constexpr int NT_O = Cfg::DV_W / 8;   // n8 tiles of O per warp
  float o_acc[NT_O][4];
#pragma unroll
  for (int i = 0; i < NT_O; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
  float m_i[2] = {-INFINITY, -INFINITY}, l_i[2] = {0.f, 0.f};

  uint32_t q_frag[Cfg::Q_IN_REGS ? D / 16 : 1][4];
  bool q_loaded = false;

  const int row_a = wr * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;  // ldmatrix A row
  const int col_a = (lane >> 4);                                    // chunk offset (0/1)

  for (int n = n_hi - 1; n >= 0; --n) {
    const int cls = classify_tile(md, bh_mask, n, ms, me, BC);
    if (cls == FM_TILE_SKIP) continue;
    __syncthreads();  // all warps finished reading the previous K/V tile
    const int j0 = n * BC;
    load_tile_async<BC, D, Cfg::NTHREADS>(sK, gk + (int64_t)j0 * p.k_s, p.k_s, p.Sk - j0, p.d, tid);
    load_tile_async<BC, DV, Cfg::NTHREADS>(sV, gv + (int64_t)j0 * p.v_s, p.v_s, p.Sk - j0, p.dv_dim, tid);
    cp_async_commit();
    if (cls == FM_TILE_PARTIAL && tid < BC) {
      const int j = j0 + tid;
      Bounds4 bd;
      if (j >= p.Sk) { bd.lts = 0; bd.lte = INT_MAX; bd.uts = 0; bd.ute = 0; }
      else if (md.ncols) bd = load_bounds(md, md.mask + ((size_t)bh_mask * p.Sk + j) * md.ncols);
      else { bd.lts = INT_MAX; bd.lte = INT_MAX; bd.uts = 0; bd.ute = 0; }
      sB[tid] = bd.lts; sB[BC + tid] = bd.lte; sB[2 * BC + tid] = bd.uts; sB[3 * BC + tid] = bd.ute;
    }
    cp_async_wait<0>();
    __syncthreads();

    if (Cfg::Q_IN_REGS && !q_loaded) {
#pragma unroll
      for (int kk = 0; kk < (Cfg::Q_IN_REGS ? D / 16 : 1); ++kk)
        ldmatrix_x4(q_frag[kk], sQ + swz<D * 2>(row_a, kk * 2 + col_a));
      q_loaded = true;
    }

    // ---- S = Q K^T --------------------------------------------------------
    float s[NT_S][4];
#pragma unroll
    for (int i = 0; i < NT_S; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a[4];
      if constexpr (Cfg::Q_IN_REGS) {
        a[0] = q_frag[kk][0]; a[1] = q_frag[kk][1]; a[2] = q_frag[kk][2]; a[3] = q_frag[kk][3];
      } else {
        ldmatrix_x4(a, sQ + swz<D * 2>(row_a, kk * 2 + col_a));
      }
#pragma unroll
      for (int np = 0; np < NT_S / 2; ++np) {
        uint32_t bfr[4];
        const int krow = np * 16 + (lane & 7) + (lane >> 4) * 8;
        ldmatrix_x4(bfr, sK + swz<D * 2>(krow, kk * 2 + ((lane >> 3) & 1)));
        mma16816<IS_BF16>(s[2 * np], a, bfr[0], bfr[1]);
        mma16816<IS_BF16>(s[2 * np + 1], a, bfr[2], bfr[3]);
      }
    }

    // ---- scale, mask ------------------------------------------------------
    const int r0 = ms + wr * 16 + g;  // global row of c0/c1; c2/c3 are r0 + 8
    if (cls == FM_TILE_PARTIAL) {
#pragma unroll
      for (int i = 0; i < NT_S; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int cl = i * 8 + tq * 2 + (e & 1);
          const int row = r0 + (e >> 1) * 8;
          const int lts = sB[cl], lte = sB[BC + cl], uts = sB[2 * BC + cl], ute = sB[3 * BC + cl];
          bool masked = (row >= lts && row < lte) || (row >= uts && row < ute);
          if (md.causal) masked = masked || (j0 + cl > row + off);
          s[i][e] = masked ? -INFINITY : s[i][e] * p.scale_log2;
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < NT_S; ++i) {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[i][e] *= p.scale_log2;
      }
    }

    // ---- optional block-score side output ---------------------------------
    // Per (row, block of key columns) maximum of the masked, scaled scores, merged into
    // block_logit with fmax (reference: flashmask/cute/flash_fwd_sm100.py:4256-4371).  A quad of
    // lanes shares two rows; its lane 0 owns them in every tile, so the merge needs no atomics.
    // One warp per row slab writes (the others hold the same scores).
    if (p.block_logit != nullptr && ws == 0) {
      constexpr int NSLOT = BC / 32 + 1;     // blocks a tile can touch at the smallest block size
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int row = r0 + r * 8;
        const int bos = p.block_bos ? p.block_bos[(int64_t)b * p.Sq + min(row, p.Sq - 1)] : 0;
        const int rel0 = j0 - bos;
        const int base = rel0 >> p.block_log2;               // arithmetic shift: floor
        float* dst = p.block_logit + (((int64_t)b * p.Hq + hq) * p.Sq + row) * p.block_ld;
#pragma unroll
        for (int k = 0; k < NSLOT; ++k) {
          const int blk = base + k;
          float mx = -INFINITY;
#pragma unroll
          for (int i = 0; i < NT_S; ++i) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int cl = i * 8 + tq * 2 + e;
              if (((rel0 + cl) >> p.block_log2) == blk) mx = fmaxf(mx, s[i][2 * r + e]);
            }
          }
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
          mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
          // the scores are in log2 units here: back to softmax_scale * q.k
          if (tq == 0 && row < p.Sq && blk >= 0 && blk < p.block_cols) dst[blk] = fmaxf(dst[blk], mx * kLn2);
        }
      }
    }

    // ---- online softmax ---------------------------------------------------
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < NT_S; ++i) mx = fmaxf(mx, fmaxf(s[i][2 * r], s[i][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m_i[r], mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = fast_exp2(m_i[r] - m_use);
      m_i[r] = m_new;
      float rs = 0.f;
#pragma unroll
      for (int i = 0; i < NT_S; ++i) {
        s[i][2 * r] = fast_exp2(s[i][2 * r] - m_use);
        s[i][2 * r + 1] = fast_exp2(s[i][2 * r + 1] - m_use);
        rs += s[i][2 * r] + s[i][2 * r + 1];
      }
      l_i[r] = l_i[r] * alpha + rs;
#pragma unroll
      for (int i = 0; i < NT_O; ++i) { o_acc[i][2 * r] *= alpha; o_acc[i][2 * r + 1] *= alpha; }
    }

    // ---- O += P V ---------------------------------------------------------
#pragma unroll
    for (int kk = 0; kk < BC / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack2<IS_BF16>(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack2<IS_BF16>(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack2<IS_BF16>(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack2<IS_BF16>(s[2 * kk + 1][2], s[2 * kk + 1][3]);
      const int vrow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int np = 0; np < NT_O / 2; ++np) {
        uint32_t bfr[4];
        const int chunk = (ws * Cfg::DV_W) / 8 + np * 2 + (lane >> 4);
        ldmatrix_x4_trans(bfr, sV + swz<DV * 2>(vrow, chunk));
        mma16816<IS_BF16>(o_acc[2 * np], a, bfr[0], bfr[1]);
        mma16816<IS_BF16>(o_acc[2 * np + 1], a, bfr[2], bfr[3]);
      }
    }
  }

  // ---- epilogue -------------------------------------------------------------
  cp_async_wait<0>();
  __syncthreads();  // K/V reads and the Q load are complete: sQ is reused for O
  const float sink_log2 = p.sink ? p.sink[hq] * kLog2e : 0.f;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float l = l_i[r];
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const float m_fin = (m_i[r] == -INFINITY) ? 0.f : m_i[r];
    if (p.sink) l += fast_exp2(sink_log2 - m_fin);
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const int row = ms + wr * 16 + g + r * 8;
    if (ws == 0 && tq == 0 && row < p.Sq)
      p.lse[((int64_t)b * p.Hq + hq) * p.Sq + row] = l > 0.f ? (m_fin + log2f(l)) * kLn2 : -INFINITY;
    const int lrow = wr * 16 + g + r * 8;
#pragma unroll
    for (int i = 0; i < NT_O; ++i) {
      const int col = ws * Cfg::DV_W + i * 8 + tq * 2;
      const uint32_t v = pack2<IS_BF16>(o_acc[i][2 * r] * inv, o_acc[i][2 * r + 1] * inv);
      *reinterpret_cast<uint32_t*>(smem + swz<DV * 2>(lrow, col >> 3) + (col & 7) * 2) = v;
    }
  }
  __syncthreads();
  uint16_t* go = reinterpret_cast<uint16_t*>(p.o) + b * p.o_b + (int64_t)ms * p.o_s + hq * p.o_h;
  constexpr int OCH = DV / 8;
  for (int idx = tid; idx < BR * OCH; idx += Cfg::NTHREADS) {
    const int r = idx / OCH, c = idx % OCH;
    if (ms + r < p.Sq && c * 8 < p.dv_dim) {
      const uint4 v = *reinterpret_cast<const uint4*>(smem + swz<DV * 2>(r, c));
      *reinterpret_cast<uint4*>(go + (int64_t)r * p.o_s + c * 8) = v;
    }
  }
}

template <int D, int DV, int BR, int BC, int NSPLIT>
static int launch_fwd(const AttnKParams& p, int dtype, cudaStream_t s) {
  using CfgB = FwdMmaCfg<D, DV, BR, BC, NSPLIT, true>;
  dim3 grid((p.Sq + BR - 1) / BR, p.Hq, p.B);
  if (dtype == FM_DTYPE_BF16) {
    auto kern = fwd_mma_kernel<D, DV, BR, BC, NSPLIT, true>;
    FM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, CfgB::SMEM));
    kern<<<grid, CfgB::NTHREADS, CfgB::SMEM, s>>>(p);
    count_launches(1);
  } else {
    auto kern = fwd_mma_kernel<D, DV, BR, BC, NSPLIT, false>;
    FM_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, CfgB::SMEM));
    kern<<<grid, CfgB::NTHREADS, CfgB::SMEM, s>>>(p);
    count_launches(1);
  }
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

// Head-dim bucket -> (BR, BC).  The smem tile is the padded bucket; the true
// d / dv only bound the global loads and stores.
int fwd_mma_tile_shape(int d, int dv, int* tile_m, int* tile_n) {
  if (d <= 64 && dv <= 64) { *tile_m = 128; *tile_n = 64; return FM_OK; }
  if (d <= 128 && dv <= 128) { *tile_m = 128; *tile_n = 64; return FM_OK; }
  if (d == 192 && dv == 128) { *tile_m = 128; *tile_n = 64; return FM_OK; }
  if (d == 256 && dv == 256) { *tile_m = 64; *tile_n = 64; return FM_OK; }
  if ((d == 512 || d == 576) && dv == 512) { *tile_m = 64; *tile_n = 32; return FM_OK; }
  return FM_ERR_UNSUPPORTED;
}

int fwd_mma_launch(const AttnKParams& p, int dtype, cudaStream_t s) {
  const int d = p.d, dv = p.dv_dim;
  if (d <= 64 && dv <= 64) return launch_fwd<64, 64, 128, 64, 1>(p, dtype, s);
  if (d <= 128 && dv <= 128) return launch_fwd<128, 128, 128, 64, 1>(p, dtype, s);
  if (d == 192 && dv == 128) return launch_fwd<192, 128, 128, 64, 1>(p, dtype, s);
  if (d == 256 && dv == 256) return launch_fwd<256, 256, 64, 64, 1>(p, dtype, s);
  if ((d == 512 || d == 576) && dv == 512) return launch_fwd<576, 512, 64, 32, 2>(p, dtype, s);
  set_error("forward: unsupported head dims (d=%d, dv=%d)", d, dv);
  return FM_ERR_UNSUPPORTED;
}

}  // namespace fm

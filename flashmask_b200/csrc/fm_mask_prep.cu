// Mask preprocessing: per-K-tile min/max of every bound column in ONE pass,
// then (Q tile, K tile) classification + surviving-tile counts, and the exact
// unmasked-pair count used as the work measure.  Integer, HBM-bound work:
// coalesced vector loads, one warp per K tile / per Q tile.
#include "fm_common.cuh"

namespace fm {

// One warp reduces the tile_n * NCOLS contiguous int32 of one K tile.  Because
// 32 % NCOLS == 0 every lane only ever sees bound column (lane % NCOLS).
template <int NCOLS>
__global__ void __launch_bounds__(128) scan_minmax_kernel(const int32_t* __restrict__ mask,
                                                         int32_t* __restrict__ minmax, int BHm,
                                                         int Sk, int tile_n, int nb, int nblk_pad,
                                                         int causal) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 4 + warp;
  const int bh = blockIdx.y;
  if (n >= nblk_pad) return;
  int vmax = 0, vmin = INT_MAX;
  if (n < nb) {
    const int col0 = n * tile_n;
    const int cols = min(tile_n, Sk - col0);
    const int32_t* src = mask + ((size_t)bh * Sk + col0) * NCOLS;
    const int total = cols * NCOLS;
    for (int e = lane; e < total; e += 32) {
      const int v = __ldg(src + e);
      vmax = max(vmax, v);
      vmin = min(vmin, v);
    }
#pragma unroll
    for (int o = 16; o >= NCOLS; o >>= 1) {
      vmax = max(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
      vmin = min(vmin, __shfl_xor_sync(0xffffffffu, vmin, o));
    }
  } else {
    vmin = 0;  // pad entries read as 0 in both reductions
  }
  if (lane < NCOLS) {
    // bound carried by mask column `lane`
    int slot_max;
    if (NCOLS == 1) slot_max = FM_MM_LTS_MAX;
    else if (NCOLS == 2) slot_max = lane == 0 ? FM_MM_LTS_MAX : (causal ? FM_MM_LTE_MAX : FM_MM_UTE_MAX);
    else slot_max = 2 * lane;
    const size_t slot = (size_t)BHm * nblk_pad;
    const size_t at = (size_t)bh * nblk_pad + n;
    minmax[slot_max * slot + at] = vmax;
    minmax[(slot_max + 1) * slot + at] = vmin;
  }
}

// One warp per Q tile: class of every K tile (optional) and the number of
// surviving tiles.
__global__ void __launch_bounds__(128) classify_kernel(MaskDesc md, int tile_m, int tile_n, int tq,
                                                      int nb, int32_t* __restrict__ valid_cnt,
                                                      int8_t* __restrict__ tile_class) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  const int bh = blockIdx.y;
  if (t >= tq) return;
  const int ms = t * tile_m, me = min(ms + tile_m, md.Sq);
  int cnt = 0;
  for (int n = lane; n < nb; n += 32) {
    const int c = classify_tile(md, bh, n, ms, me, tile_n);
    cnt += c != FM_TILE_SKIP;
    if (tile_class) tile_class[((size_t)bh * tq + t) * nb + n] = (int8_t)c;
  }
#pragma unroll
  for (int o = 16; o; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if (lane == 0 && valid_cnt) valid_cnt[(size_t)bh * tq + t] = cnt;
}

__global__ void __launch_bounds__(256) count_visible_kernel(MaskDesc md, int64_t* __restrict__ out) {
  const int bh = blockIdx.x;
  const int Sq = md.Sq, Sk = md.Sk, off = Sk - Sq;
  long long acc = 0;
  for (int j = threadIdx.x; j < Sk; j += blockDim.x) {
    Bounds4 b = load_bounds(md, md.mask + ((size_t)bh * Sk + j) * md.ncols);
    int lo1 = min(max(b.lts, 0), Sq), hi1 = min(max(b.lte, 0), Sq);
    int lo2 = min(max(b.uts, 0), Sq), hi2 = min(max(b.ute, 0), Sq);
    if (md.causal) { lo2 = 0; hi2 = min(max(j - off, 0), Sq); }
    hi1 = max(hi1, lo1); hi2 = max(hi2, lo2);
    const int inter = max(0, min(hi1, hi2) - max(lo1, lo2));
    acc += Sq - ((hi1 - lo1) + (hi2 - lo2) - inter);
  }
  __shared__ long long red[8];
#pragma unroll
  for (int o = 16; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    long long s = 0;
    for (int w = 0; w < 8; ++w) s += red[w];
    out[bh] = s;
  }
}

}  // namespace fm

using namespace fm;

extern "C" int fm_mask_nblk_pad(int Sk, int tile_n) {
  if (tile_n <= 0) return 0;
  return (int)((((unsigned)(Sk + tile_n - 1) / (unsigned)tile_n) + 3u) & 0xfffffffcu);
}

extern "C" int fm_mask_prepare(const int32_t* mask, int B, int Hm, int Sq, int Sk, int ncols,
                               int causal, int tile_m, int tile_n, int32_t* minmax,
                               int32_t* valid_cnt, int8_t* tile_class, void* stream) {
  FM_REQUIRE(B > 0 && Hm > 0 && Sq > 0 && Sk > 0, FM_ERR_INVALID_ARGUMENT,
             "fm_mask_prepare: B/Hm/Sq/Sk must be positive");
  FM_REQUIRE(tile_m > 0 && tile_n > 0, FM_ERR_INVALID_ARGUMENT, "fm_mask_prepare: bad tile shape");
  FM_REQUIRE(ncols == 0 || ncols == 1 || ncols == 2 || ncols == 4, FM_ERR_INVALID_ARGUMENT,
             "fm_mask_prepare: ncols must be 0, 1, 2 or 4 (got %d)", ncols);
  FM_REQUIRE(!(ncols == 1 && !causal), FM_ERR_INVALID_ARGUMENT,
             "fm_mask_prepare: a 1-column mask is only defined with causal=1");
  FM_REQUIRE(!(ncols == 4 && causal), FM_ERR_INVALID_ARGUMENT,
             "fm_mask_prepare: a 4-column mask is only defined with causal=0");
  FM_REQUIRE(ncols == 0 || (mask && minmax), FM_ERR_INVALID_ARGUMENT,
             "fm_mask_prepare: mask/minmax pointers are NULL");
  cudaStream_t s = (cudaStream_t)stream;
  const int nb = (Sk + tile_n - 1) / tile_n;
  const int pad = fm_mask_nblk_pad(Sk, tile_n);
  const int BHm = B * Hm;
  if (ncols) {
    dim3 grid((pad + 3) / 4, BHm);
    if (ncols == 1) scan_minmax_kernel<1><<<grid, 128, 0, s>>>(mask, minmax, BHm, Sk, tile_n, nb, pad, causal);
    else if (ncols == 2) scan_minmax_kernel<2><<<grid, 128, 0, s>>>(mask, minmax, BHm, Sk, tile_n, nb, pad, causal);
    else scan_minmax_kernel<4><<<grid, 128, 0, s>>>(mask, minmax, BHm, Sk, tile_n, nb, pad, causal);
    FM_CUDA_TRY(cudaGetLastError());
  }
  if (valid_cnt || tile_class) {
    MaskDesc md{mask, minmax, ncols, causal, Hm, B, pad, BHm, Sq, Sk};
    const int tq = (Sq + tile_m - 1) / tile_m;
    dim3 grid((tq + 3) / 4, BHm);
    classify_kernel<<<grid, 128, 0, s>>>(md, tile_m, tile_n, tq, nb, valid_cnt, tile_class);
    FM_CUDA_TRY(cudaGetLastError());
  }
  return FM_OK;
}

extern "C" int fm_mask_count_visible(const int32_t* mask, int B, int Hm, int Sq, int Sk, int ncols,
                                     int causal, int64_t* out, void* stream) {
  FM_REQUIRE(mask && out && (ncols == 1 || ncols == 2 || ncols == 4), FM_ERR_INVALID_ARGUMENT,
             "fm_mask_count_visible: needs a mask with 1, 2 or 4 columns");
  MaskDesc md{mask, nullptr, ncols, causal, Hm, B, 0, B * Hm, Sq, Sk};
  count_visible_kernel<<<B * Hm, 256, 0, (cudaStream_t)stream>>>(md, out);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

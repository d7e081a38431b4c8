// Mask preprocessing: per-K-tile min/max of every bound column in ONE pass,
// then (Q tile, K tile) classification + surviving-tile counts, and the exact
// unmasked-pair count used as the work measure.  Integer, HBM-bound work:
// coalesced vector loads, one warp per K tile / per Q tile.
#include <algorithm>
#include <cstdlib>

#include "fm_attn_params.cuh"

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

// Longest-work-first launch table of one kernel, built by ONE CTA of 1024 threads.
//   1. work of every unit (axis 0: a block of `block_rows` query rows -> K tiles it keeps;
//      axis 1: a K tile -> `block_rows`-row query blocks it keeps), one warp per unit;
//   2. units are dealt into FM_ORDER_BUCKETS work classes relative to the heaviest unit and
//      ordered by (class, index): heaviest class first, index order inside a class;
//   3. the launch table lists, class by class, every repeat (heads sharing the mask head,
//      batches sharing a broadcast mask) of the class's units, repeat-major: CTAs next to
//      each other in dispatch order work on neighbouring tiles of the same head, as in the
//      index order, so operands shared between neighbouring tiles still meet in L2.
// smem: work[E], order[E], hist/start[FM_ORDER_BUCKETS + 1], red[32], class[E] bytes.
constexpr int FM_ORDER_BUCKETS = 8;
constexpr int FM_PERSIST_MAX_ITEMS = 96;

__global__ void __launch_bounds__(1024) launch_order_kernel(MaskDesc md_in, int tile_n, OrderJobs jobs, int n_classes,
                                                            int stage_ints, int work_off) {
  const OrderJob& jb = jobs.job[blockIdx.x];   // one CTA per table
  const int axis = jb.axis, block_rows = jb.block_rows, n_units = jb.n_units, n_other = jb.n_other;
  const int rep_h = jb.rep_h, rep_b = jb.rep_b, heads = jb.heads, item_mult = jb.item_mult;
  int32_t* __restrict__ out = jb.out;
  extern __shared__ int32_t sm_all[];
  // the per-tile reductions of the whole mask are staged in shared memory first (when they fit):
  // classifying a unit then costs no global round trip
  MaskDesc md = md_in;
  if (stage_ints) {
    const int row4 = (md.BHm * md.nblk_pad) >> 2;                      // int4 per reduction
    const uint32_t which = md.ncols == 1 ? 0x03u : (md.ncols == 4 ? 0xFFu : (md.causal ? 0x0Fu : 0xC3u));
    for (int w = 0; w < 8; ++w) {
      if (!(which >> w & 1u)) continue;
      const int4* src = reinterpret_cast<const int4*>(md_in.minmax) + (size_t)w * row4;
      int4* dst = reinterpret_cast<int4*>(sm_all) + (size_t)w * row4;
      for (int i = threadIdx.x; i < row4; i += 1024) dst[i] = __ldg(src + i);
    }
    md.minmax = sm_all;
    __syncthreads();
  }
  int32_t* sm = sm_all + work_off;
  const int E = md.BHm * n_units;
  int32_t* swork = sm;
  int32_t* sorder = sm + E;
  int32_t* sstart = sm + 2 * E;           // [FM_ORDER_BUCKETS + 1]
  int32_t* sred = sstart + FM_ORDER_BUCKETS + 1;  // [32]
  uint8_t* sclass = reinterpret_cast<uint8_t*>(sred + 32);  // [E]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_cta = E * rep_h * rep_b;
  int2* table = reinterpret_cast<int2*>(out);
  int32_t* gwork = out + 2 * (size_t)n_cta;
  int32_t* gorder = gwork + E;
  if (tid < 4) gorder[E + tid] = 0;   // counters of the persistent kernels that walk this table

  for (int e = warp; e < E; e += 32) {
    const int bh = e / n_units, u = e % n_units;
    int cnt = 0;
    if (axis == 0) {
      const int ms = u * block_rows, me = min(ms + block_rows, md.Sq);
      for (int n = lane; n < n_other; n += 32) cnt += tile_flags(md, bh, n, ms, me, tile_n) != 0;
    } else {
      for (int t = lane; t < n_other; t += 32) {
        const int ms = t * block_rows, me = min(ms + block_rows, md.Sq);
        cnt += tile_flags(md, bh, u, ms, me, tile_n) != 0;
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    if (lane == 0) { swork[e] = cnt; gwork[e] = cnt; }
  }
  if (tid <= FM_ORDER_BUCKETS) sstart[tid] = 0;
  __syncthreads();

  int mx = 0;
  long long total = 0;
  for (int e = tid; e < E; e += 1024) { mx = max(mx, swork[e]); total += swork[e]; }
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    total += __shfl_xor_sync(0xffffffffu, total, o);
  }
  __shared__ long long stot[32];
  if (lane == 0) { sred[warp] = mx; stot[warp] = total; }
  __syncthreads();
  mx = 0;
  total = 0;
  for (int w = 0; w < 32; ++w) { mx = max(mx, sred[w]); total += stot[w]; }
  // [E+2]: 1 while a unit averages at most FM_PERSIST_MAX_ITEMS work items, the range in which the
  // persistent backward variant (which hides the per-unit prologue and epilogue at a slightly slower
  // main loop) was measured faster; information for the host, the kernels do not read it
  if (tid == 0) gorder[E + 2] = total * item_mult <= (long long)FM_PERSIST_MAX_ITEMS * E ? 1 : 0;
  for (int e = tid; e < E; e += 1024) {
    const int k = (int)(((long long)(mx - swork[e]) * n_classes) / (mx + 1));  // 0 = heaviest class
    sclass[e] = (uint8_t)k;
    atomicAdd(&sstart[k + 1], 1);
  }
  __syncthreads();
  if (tid == 0)
    for (int k = 0; k < FM_ORDER_BUCKETS; ++k) sstart[k + 1] += sstart[k];
  __syncthreads();
  for (int e = tid; e < E; e += 1024) {
    const int k = sclass[e];
    int before = 0;
    for (int j = 0; j < e; ++j) before += sclass[j] == k;
    const int r = sstart[k] + before;
    sorder[r] = e;
    gorder[r] = e;
  }
  __syncthreads();

  const int rep = rep_h * rep_b;
  for (int L = tid; L < n_cta; L += 1024) {
    int k = 0;
    while (L >= rep * sstart[k + 1]) ++k;
    const int size = sstart[k + 1] - sstart[k];
    const int l = L - rep * sstart[k];
    const int rr = l / size;
    const int id = sorder[sstart[k] + l % size];
    const int unit = id % n_units;
    const int head = (id / n_units) % md.Hm * rep_h + rr % rep_h;
    const int b = md.mask_B == 1 ? rr / rep_h : id / (n_units * md.Hm);
    table[L] = make_int2(unit, b * heads + head);
  }
}

}  // namespace fm

using namespace fm;

int fm::launch_order_build(const MaskDesc& md, int tile_n, const OrderJobs& jobs, int n_jobs, cudaStream_t s) {
  size_t smem = 0;
  for (int i = 0; i < n_jobs; ++i) {
    const size_t E = (size_t)md.BHm * jobs.job[i].n_units;
    smem = std::max(smem, sizeof(int32_t) * (2 * E + FM_ORDER_BUCKETS + 1 + 32) + E);
  }
  int n_classes = FM_ORDER_BUCKETS;
  if (const int e = option_order_classes()) n_classes = std::min(FM_ORDER_BUCKETS, std::max(1, e));
  // staging area for the reductions: 8 x BHm x nblk_pad ints, only when that stays small
  const size_t stage_ints = 8 * (size_t)md.BHm * md.nblk_pad;
  const int staged = (stage_ints * 4 + smem <= 96 * 1024 && (reinterpret_cast<uintptr_t>(md.minmax) & 15) == 0)
                         ? (int)stage_ints : 0;
  smem += (size_t)staged * 4;
  if (smem > 48 * 1024)
    FM_CUDA_TRY(cudaFuncSetAttribute(launch_order_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
  launch_order_kernel<<<n_jobs, 1024, smem, s>>>(md, tile_n, jobs, n_classes, staged, staged);
  count_launches(1);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

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
    count_launches(1);
    FM_CUDA_TRY(cudaGetLastError());
  }
  if (valid_cnt || tile_class) {
    MaskDesc md{mask, minmax, ncols, causal, Hm, B, pad, BHm, Sq, Sk};
    const int tq = (Sq + tile_m - 1) / tile_m;
    dim3 grid((tq + 3) / 4, BHm);
    classify_kernel<<<grid, 128, 0, s>>>(md, tile_m, tile_n, tq, nb, valid_cnt, tile_class);
    count_launches(1);
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
  count_launches(1);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

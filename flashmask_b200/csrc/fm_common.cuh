// Shared device/host helpers for the flashmask_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <climits>
#include <cstdio>

#include "flashmask_b200.h"

namespace fm {

// ---------------------------------------------------------------------------
// error plumbing (host)
// ---------------------------------------------------------------------------
void set_error(const char* fmt, ...);
// Every host function that launches kernels reports how many (fm_launch_count sums them).
void count_launches(int n);
int cuda_fail(cudaError_t e, const char* what);

#define FM_CUDA_TRY(expr)                                     \
  do {                                                        \
    cudaError_t _e = (expr);                                  \
    if (_e != cudaSuccess) return ::fm::cuda_fail(_e, #expr); \
  } while (0)

#define FM_REQUIRE(cond, code, ...)     \
  do {                                  \
    if (!(cond)) {                      \
      ::fm::set_error(__VA_ARGS__);     \
      return (code);                    \
    }                                   \
  } while (0)

// ---------------------------------------------------------------------------
// mask geometry shared by all attention kernels
// ---------------------------------------------------------------------------
struct MaskDesc {
  const int32_t* mask;    // [mask_B, Hm, Sk, ncols] or nullptr
  const int32_t* minmax;  // [8, mask_B*Hm, nblk_pad] or nullptr
  int ncols;              // 0 | 1 | 2 | 4
  int causal;
  int Hm, mask_B, nblk_pad, BHm;
  int Sq, Sk;
};

// Column bounds normalised to two masked row intervals [lts,lte) U [uts,ute).
struct Bounds4 {
  int lts, lte, uts, ute;
};

__device__ __forceinline__ Bounds4 load_bounds(const MaskDesc& md, const int32_t* col_ptr) {
  // col_ptr points at the first int of column j.
  Bounds4 b;
  b.lts = INT_MAX; b.lte = INT_MAX; b.uts = 0; b.ute = 0;
  if (md.ncols == 1) {
    b.lts = col_ptr[0];
  } else if (md.ncols == 2) {
    int2 v = *reinterpret_cast<const int2*>(col_ptr);
    b.lts = v.x;
    if (md.causal) b.lte = v.y; else b.ute = v.y;
  } else if (md.ncols == 4) {
    int4 v = *reinterpret_cast<const int4*>(col_ptr);
    b.lts = v.x; b.lte = v.y; b.uts = v.z; b.ute = v.w;
  }
  return b;
}

// Tile flags of rows [ms, me) against K tile n, from the per-tile reductions.
// 0 = skipped (every element masked by the bounds or by causal geometry), else
// bit 0 set plus the element masks the tile still needs:
//   FM_TF_BOUNDS  some column bound may cut through the tile
//   FM_TF_CAUSAL  the causal diagonal crosses the tile
//   FM_TF_RAGGED  the tile hangs over the end of the key sequence
constexpr uint32_t FM_TF_ACTIVE = 1, FM_TF_BOUNDS = 2, FM_TF_CAUSAL = 4, FM_TF_RAGGED = 8;

__device__ __forceinline__ uint32_t tile_flags(const MaskDesc& md, int bh_mask, int n, int ms, int me,
                                               int tile_n) {
  const int ns = n * tile_n;
  const int ne = min(ns + tile_n, md.Sk);
  const int off = md.Sk - md.Sq;
  uint32_t flags = FM_TF_ACTIVE | (ne < ns + tile_n ? FM_TF_RAGGED : 0u);
  if (md.causal) {
    if (ns > (me - 1 + off)) return 0;               // entirely in the future
    if (!((ne - 1) <= (ms + off))) flags |= FM_TF_CAUSAL;
  }
  if (md.ncols) {
    const int32_t* mm = md.minmax + (size_t)bh_mask * md.nblk_pad + n;
    const size_t slot = (size_t)md.BHm * md.nblk_pad;
    const int lts_max = mm[FM_MM_LTS_MAX * slot], lts_min = mm[FM_MM_LTS_MIN * slot];
    bool fully, part;
    if (md.ncols == 4) {
      const int lte_max = mm[FM_MM_LTE_MAX * slot], lte_min = mm[FM_MM_LTE_MIN * slot];
      const int uts_max = mm[FM_MM_UTS_MAX * slot], uts_min = mm[FM_MM_UTS_MIN * slot];
      const int ute_max = mm[FM_MM_UTE_MAX * slot], ute_min = mm[FM_MM_UTE_MIN * slot];
      fully = (ms >= lts_max && me <= lte_min) || (ms >= uts_max && me <= ute_min);
      part = (ms < lte_max && me > lts_min) || (ms < ute_max && me > uts_min);
    } else if (md.ncols == 2 && md.causal) {
      const int lte_max = mm[FM_MM_LTE_MAX * slot], lte_min = mm[FM_MM_LTE_MIN * slot];
      fully = ms >= lts_max && me <= lte_min;
      part = ms < lte_max && me > lts_min;
    } else if (md.ncols == 2) {
      const int ute_max = mm[FM_MM_UTE_MAX * slot], ute_min = mm[FM_MM_UTE_MIN * slot];
      fully = ms >= lts_max || me <= ute_min;
      part = me > lts_min || ms < ute_max;
    } else {
      fully = ms >= lts_max;
      part = me > lts_min;
    }
    if (fully) return 0;
    if (part) flags |= FM_TF_BOUNDS;
  }
  return flags;
}

// One warp copies the per-K-tile reductions of tiles [n_lo, n_hi) of mask row `bh` into
// shared memory with all its global loads in flight at once, and returns a descriptor
// whose tile_flags(staged, 0, n, ...) reads them from there.  Walking a tile list with
// tile_flags on the global copy costs one dependent global round trip per 32 tiles; this
// way the whole range costs one.  n_lo is a multiple of 4 (16-byte loads; every row of
// `minmax` is padded to a multiple of 4 tiles and 16-byte aligned), `stage` holds
// 8 * cap ints with cap a multiple of 4 and >= n_hi - n_lo.
__device__ __forceinline__ MaskDesc stage_minmax(const MaskDesc& md, int bh, int n_lo, int n_hi,
                                                 int32_t* stage, int cap, int lane) {
  MaskDesc s = md;
  if (!md.ncols) return s;
  const size_t slot = (size_t)md.BHm * md.nblk_pad;
  const int32_t* src = md.minmax + (size_t)bh * md.nblk_pad + n_lo;
  const int n4 = (n_hi - n_lo + 3) >> 2;
  // reductions the mask carries: LTS always, LTE for causal 2-column and 4-column masks,
  // UTS for 4-column, UTE for non-causal 2-column and 4-column
  const uint32_t which = md.ncols == 1 ? 0x03u : (md.ncols == 4 ? 0xFFu : (md.causal ? 0x0Fu : 0xC3u));
  for (int base = 0; base < n4; base += 32) {
    const int i = base + lane;
    int4 v[8];
#pragma unroll
    for (int w = 0; w < 8; ++w)
      if ((which >> w & 1u) && i < n4) v[w] = __ldg(reinterpret_cast<const int4*>(src + w * slot) + i);
#pragma unroll
    for (int w = 0; w < 8; ++w)
      if ((which >> w & 1u) && i < n4) reinterpret_cast<int4*>(stage + w * cap)[i] = v[w];
  }
  __syncwarp();
  s.minmax = stage - n_lo;
  s.BHm = 1;
  s.nblk_pad = cap;
  return s;
}

// One warp copies the row bounds of `cols` key columns (cols * ncols ints; cols is 64 or 128)
// into shared memory, zero past `valid_cols` (a ragged last tile).  Every load is issued before
// the first store, so the copy costs one global round trip however many bounds a column has.
__device__ __forceinline__ void stage_bounds(int* dst, const int32_t* src, int cols, int valid_cols, int ncols,
                                             int lane) {
  const int n = cols * ncols;
  if (valid_cols == cols && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    const int n4 = n >> 2;                      // <= 128 vectors: at most 4 per lane
    int4 v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (lane + 32 * i < n4) v[i] = __ldg(reinterpret_cast<const int4*>(src) + lane + 32 * i);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (lane + 32 * i < n4) reinterpret_cast<int4*>(dst)[lane + 32 * i] = v[i];
  } else {
    const int valid = valid_cols * ncols;
    int v[16];                                  // <= 512 ints: at most 16 per lane
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int x = lane + 32 * i;
      v[i] = (x < valid) ? __ldg(src + x) : 0;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (lane + 32 * i < n) dst[lane + 32 * i] = v[i];
  }
}

// Three-way class of the same tile: skipped / partial (needs an element mask) / unmasked.
__device__ __forceinline__ int classify_tile(const MaskDesc& md, int bh_mask, int n, int ms, int me,
                                             int tile_n) {
  const uint32_t f = tile_flags(md, bh_mask, n, ms, me, tile_n);
  return f == 0 ? FM_TILE_SKIP : ((f & ~FM_TF_ACTIVE) ? FM_TILE_PARTIAL : FM_TILE_FULL);
}

// ---------------------------------------------------------------------------
// small PTX wrappers used by the warp-MMA kernels
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool pred) {
  const int sz = pred ? 16 : 0;  // src-size 0 => zero fill
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n"
               : "=r"(r[0]), "=r"(r[1])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n"
               : "=r"(r[0]), "=r"(r[1])
               : "r"(addr));
}

// D(16x8,f32) += A(16x16) * B(16x8); IS_BF16 selects bf16 / f16 operands.
template <bool IS_BF16>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  if constexpr (IS_BF16) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

template <bool IS_BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (IS_BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}

// Bits [0, x) of a 32-bit word set (x <= 0: none, x >= 32: all).
__device__ __forceinline__ uint32_t bits_below(int x) {
  return __funnelshift_lc(0xffffffffu, 0u, (uint32_t)max(x, 0));
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// Two fp32 lanes per instruction (sm_100 packed arithmetic): (x0, x1) = (a0, a1) * b + c and (a0, a1) += (b0, b1).
// They halve the issue slots the softmax spends on scaling the scores and on the row sums.
__device__ __forceinline__ void fma2_scalar(float& x0, float& x1, float a0, float a1, float b, float c) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(x0), "=f"(x1) : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
// max(a, b, c) in one instruction (sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ void mul2(float& x0, float& x1, float a0, float a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 ra, ra, rb;\n\t"
      "mov.b64 {%0, %1}, ra;\n\t}"
      : "=f"(x0), "=f"(x1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ void add2(float& a0, float& a1, float b0, float b1) {
  asm("{\n\t.reg .b64 ra, rb;\n\t"
      "mov.b64 ra, {%0, %1};\n\tmov.b64 rb, {%2, %3};\n\t"
      "add.rn.f32x2 ra, ra, rb;\n\t"
      "mov.b64 {%0, %1}, ra;\n\t}"
      : "+f"(a0), "+f"(a1) : "f"(b0), "f"(b1));
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows hold
// ROW_BYTES bytes (ROW_BYTES/16 a multiple of 8): XOR swizzle on the low 3 bits
// so that ldmatrix over 8 consecutive rows is bank-conflict free.
template <int ROW_BYTES>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  return (uint32_t)row * ROW_BYTES + (uint32_t)((chunk ^ (row & 7)) << 4);
}

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

}  // namespace fm

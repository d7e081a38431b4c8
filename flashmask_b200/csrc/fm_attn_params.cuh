// Kernel-side parameter block shared by the attention kernels.
#pragma once
#include "fm_common.cuh"

namespace fm {

struct AttnKParams {
  const void* q; const void* k; const void* v;
  void* o; float* lse; const float* sink;
  const void* d_o; void* dq; void* dk; void* dv; float* dsink;
  float* dpsum;     // [B,Hq,Sq_r] fp32 workspace: rowsum(O * dO)
  float* lse_log2;  // [B,Hq,Sq_r] fp32 workspace: LSE * log2(e), -inf -> 0
  float* dq_accum;  // [B,Hq,Sq_r,64|128] fp32 workspace (one-kernel backward: dQ summed by reductions)
  // one-kernel backward only: the row statistics as 16-bit GEMM operands, [B,Hq,Sq_r,8] each:
  // (-c_hi, -c_lo, 0 x 6) with c = LSE*log2e / scale_log2, and (-d_hi, -d_lo, 0 x 6) with d = rowsum(O dO)
  uint16_t* stat_s; uint16_t* stat_dp;
  int bwd_flags;    // FM_BWD_DQ_CARRY: the accumulator holds earlier sums; FM_BWD_DQ_LEAVE: dq is not written
  int64_t q_b, q_s, q_h, k_b, k_s, k_h, v_b, v_s, v_h, o_b, o_s, o_h;
  int64_t do_b, do_s, do_h, dq_b, dq_s, dq_h, dk_b, dk_s, dk_h, dv_b, dv_s, dv_h;
  int B, Sq, Sk, Hq, Hkv, d, dv_dim;
  int Sq_r;  // Sq rounded up to the row tile, stride of the per-row workspaces
  float scale, scale_log2;
  MaskDesc md;
  // optional longest-work-first launch orders (unit ids over (mask_b, mask_h, unit)); nullptr = index order
  const int32_t* fwd_order; const int32_t* dq_order; const int32_t* dkdv_order;
  // state behind a backward table: [0] next table entry, [1] CTAs that left, [2] 1 when the persistent
  // variant runs on this table, 0 when the one-unit-per-CTA variant does (written by the table builder)
  int* dq_sched; int* dkdv_sched;
  int dq_ncta, dkdv_ncta;   // entries of the tables
  // optional side output of the forward: per (query row, block of key columns) the maximum of the
  // masked, scaled scores, combined into block_logit[b][head][row][block] with fmax; block ids are
  // relative to block_bos[b][row] (the first key of the row's document) when that is given
  float* block_logit; const int32_t* block_bos;
  int block_log2, block_cols, block_ld;   // log2(block size), ceil(Sk / block size), row stride
};

// CTA coordinates under a launch order: the CTAs of a launch are numbered in
// dispatch order L = x + gx*(y + gy*z) and table[L] = (unit, b * heads + head).
struct OrderedCta { int b, head, unit; };
__device__ __forceinline__ OrderedCta ordered_cta(const int32_t* table, int heads) {
  const unsigned L = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  const int2 e = __ldg(reinterpret_cast<const int2*>(table) + L);
  OrderedCta c;
  c.unit = e.x; c.head = e.y % heads; c.b = e.y / heads;
  return c;
}

// Units a launch table may cover (one CTA builds it, the unit work staged in shared memory).
constexpr int FM_ORDER_MAX_UNITS = 4096;
// One table to build: the ordered axis (0 rows / 1 key tiles), rows per unit, units, extent of the
// other axis, repeats, heads of the kernel, work items per unit of work, destination.
struct OrderJob { int axis, block_rows, n_units, n_other, rep_h, rep_b, heads, item_mult; int32_t* out; };
struct OrderJobs { OrderJob job[3]; };
// Builds up to three tables in one launch (one CTA each).
int launch_order_build(const MaskDesc& md, int tile_n, const OrderJobs& jobs, int n_jobs, cudaStream_t s);
// Work classes requested through the environment when the library was loaded (0: the default).
int option_order_classes();

}  // namespace fm

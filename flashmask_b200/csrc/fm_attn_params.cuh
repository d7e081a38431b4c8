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
  float* dq_accum;  // [B,Hq,Sq_r,d_r] fp32 workspace (atomic dQ path)
  int64_t q_b, q_s, q_h, k_b, k_s, k_h, v_b, v_s, v_h, o_b, o_s, o_h;
  int64_t do_b, do_s, do_h, dq_b, dq_s, dq_h, dk_b, dk_s, dk_h, dv_b, dv_s, dv_h;
  int B, Sq, Sk, Hq, Hkv, d, dv_dim;
  int Sq_r;  // Sq rounded up to the row tile, stride of the per-row workspaces
  float scale, scale_log2;
  MaskDesc md;
};

int fill_kparams(const fm_attn_args* a, AttnKParams* p, bool backward);

}  // namespace fm

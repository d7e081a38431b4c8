// extern "C" entry points: argument validation, kernel-variant selection,
// workspace carving.  No allocation, no host synchronisation.
#include <atomic>
#include <cstdarg>
#include <cstdlib>
#include <cstring>

#include "fm_attn_params.cuh"

namespace fm {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

static std::atomic<unsigned long long> g_launches{0};
void count_launches(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) at %s", (int)e, cudaGetErrorString(e), what);
  return FM_ERR_CUDA;
}

// implemented in the kernel translation units
int fwd_mma_tile_shape(int d, int dv, int* tile_m, int* tile_n);
int fwd_mma_launch(const AttnKParams& p, int dtype, cudaStream_t s);
int bwd_mma_tile_shape(int d, int dv, int* tile_m, int* tile_n);
int bwd_mma_launch(const AttnKParams& p, int dtype, cudaStream_t s);
int bwd_preprocess_launch(const AttnKParams& p, int dtype, cudaStream_t s);
int bwd_dsink_launch(const AttnKParams& p, cudaStream_t s);
bool fwd_sm100_supported(const fm_attn_args* a);
int fwd_sm100_launch(const AttnKParams& p, const fm_attn_args* a, cudaStream_t s);
bool bwd_sm100_supported(const fm_attn_args* a);
int bwd_sm100_launch(const AttnKParams& p, const fm_attn_args* a, cudaStream_t s);
int bwd_sm100_persist_launch(const AttnKParams& p, const fm_attn_args* a, cudaStream_t s);
int bwd_sm100_fused_launch(const AttnKParams& p, const fm_attn_args* a, cudaStream_t s);
int bwd_sm100_fused_status(int* out, bool reset);
size_t bwd_sm100_fused_accum_bytes(const fm_attn_args* a);
int bwd_sm100_persist_status(int* out, bool reset);
size_t bwd_sm100_workspace_bytes(const fm_attn_args* a);

int fwd_sm100_status(int* out, bool reset);
int bwd_sm100_status(int* out, bool reset);
int bounded_wait_selftest_launch(uint64_t budget_ns, cudaStream_t s);

static inline int round_up(int x, int m) { return (x + m - 1) / m * m; }

// A/B switches, read from the environment ONCE when the library is loaded (and again only when
// the host asks through fm_reload_options): no entry point touches the environment per call.
//   FLASHMASK_B200_FWD=mma       forward on the warp-MMA kernels for every head dim
//   FLASHMASK_B200_BWD=mma       backward on the warp-MMA kernels for every head dim
//   FLASHMASK_B200_BWD=split     tcgen05 backward as two kernels (dK/dV + dQ) even when the call
//                                did not ask for deterministic gradients
//   FLASHMASK_B200_PERSIST=0     tcgen05 backward: one unit per CTA even with launch tables
//   FLASHMASK_B200_CLASSES=n     work classes of the launch tables (1..8)
struct Options { bool fwd_mma, bwd_mma, bwd_split, bwd_persist; int order_classes; };
static Options read_options() {
  Options o{false, false, false, true, 0};
  if (const char* e = getenv("FLASHMASK_B200_FWD")) o.fwd_mma = strcmp(e, "mma") == 0;
  if (const char* e = getenv("FLASHMASK_B200_BWD")) { o.bwd_mma = strcmp(e, "mma") == 0; o.bwd_split = strcmp(e, "split") == 0; }
  if (const char* e = getenv("FLASHMASK_B200_PERSIST")) o.bwd_persist = !(e[0] == '0' && e[1] == 0);
  if (const char* e = getenv("FLASHMASK_B200_CLASSES")) o.order_classes = atoi(e);
  return o;
}
static Options g_opt = read_options();
int option_order_classes() { return g_opt.order_classes; }

// Kernel variant of the forward for (d, dv): the tcgen05 kernels cover head dims up to
// 128 (multiples of 8); FLASHMASK_B200_FWD=mma forces the warp-MMA variant (A/B runs).
static bool fwd_uses_sm100(int d, int dv) {
  const bool small = d <= 128 && dv <= 128 && d % 8 == 0 && dv % 8 == 0;
  if (!small && !(d == 192 && dv == 128) && !(d == 256 && dv == 256)) return false;
  return !g_opt.fwd_mma;
}

static bool stride_ok(const int64_t* s) { return s[0] % 8 == 0 && s[1] % 8 == 0 && s[2] % 8 == 0; }

static int validate_common(const fm_attn_args* a, const char* who) {
  FM_REQUIRE(a != nullptr, FM_ERR_INVALID_ARGUMENT, "%s: args is NULL", who);
  FM_REQUIRE(a->B > 0 && a->Sq > 0 && a->Sk > 0 && a->Hq > 0 && a->Hkv > 0, FM_ERR_INVALID_ARGUMENT,
             "%s: B/Sq/Sk/Hq/Hkv must be positive", who);
  FM_REQUIRE(a->Hq % a->Hkv == 0, FM_ERR_INVALID_ARGUMENT, "%s: Hq (%d) must be a multiple of Hkv (%d)",
             who, a->Hq, a->Hkv);
  FM_REQUIRE(a->d > 0 && a->dv > 0 && a->d % 8 == 0 && a->dv % 8 == 0, FM_ERR_INVALID_ARGUMENT,
             "%s: head dims must be positive multiples of 8 (d=%d, dv=%d)", who, a->d, a->dv);
  FM_REQUIRE(a->dtype == FM_DTYPE_BF16 || a->dtype == FM_DTYPE_FP16, FM_ERR_INVALID_ARGUMENT,
             "%s: dtype must be FM_DTYPE_BF16 or FM_DTYPE_FP16", who);
  FM_REQUIRE(a->q && a->k && a->v && a->o && a->lse, FM_ERR_INVALID_ARGUMENT,
             "%s: q/k/v/o/lse must not be NULL", who);
  FM_REQUIRE(stride_ok(a->q_stride) && stride_ok(a->k_stride) && stride_ok(a->v_stride) &&
                 stride_ok(a->o_stride),
             FM_ERR_INVALID_ARGUMENT, "%s: strides must be multiples of 8 elements (16-byte rows)", who);
  FM_REQUIRE(a->ncols == 0 || a->ncols == 1 || a->ncols == 2 || a->ncols == 4, FM_ERR_INVALID_ARGUMENT,
             "%s: ncols must be 0, 1, 2 or 4", who);
  if (a->ncols) {
    FM_REQUIRE(a->mask && a->minmax, FM_ERR_INVALID_ARGUMENT, "%s: mask given but mask/minmax is NULL", who);
    FM_REQUIRE(((uintptr_t)a->minmax & 15) == 0, FM_ERR_INVALID_ARGUMENT, "%s: minmax must be 16-byte aligned", who);
    FM_REQUIRE(a->Hm == 1 || a->Hm == a->Hkv, FM_ERR_INVALID_ARGUMENT,
               "%s: mask heads (%d) must be 1 or Hkv", who, a->Hm);
    FM_REQUIRE(a->mask_B == a->B || a->mask_B == 1, FM_ERR_INVALID_ARGUMENT,
               "%s: mask batch (%d) must be B or 1", who, a->mask_B);
    FM_REQUIRE(!(a->ncols == 1 && !a->causal) && !(a->ncols == 4 && a->causal), FM_ERR_INVALID_ARGUMENT,
               "%s: ncols=%d is not defined for causal=%d", who, a->ncols, a->causal);
  }
  return FM_OK;
}

int fill_kparams(const fm_attn_args* a, AttnKParams* p, bool backward) {
  memset(p, 0, sizeof(*p));
  p->q = a->q; p->k = a->k; p->v = a->v; p->o = a->o; p->lse = a->lse; p->sink = a->sink;
  p->q_b = a->q_stride[0]; p->q_s = a->q_stride[1]; p->q_h = a->q_stride[2];
  p->k_b = a->k_stride[0]; p->k_s = a->k_stride[1]; p->k_h = a->k_stride[2];
  p->v_b = a->v_stride[0]; p->v_s = a->v_stride[1]; p->v_h = a->v_stride[2];
  p->o_b = a->o_stride[0]; p->o_s = a->o_stride[1]; p->o_h = a->o_stride[2];
  p->B = a->B; p->Sq = a->Sq; p->Sk = a->Sk; p->Hq = a->Hq; p->Hkv = a->Hkv;
  p->d = a->d; p->dv_dim = a->dv;
  p->Sq_r = round_up(a->Sq, 128);
  p->scale = a->softmax_scale;
  p->scale_log2 = a->softmax_scale * kLog2e;
  p->md.mask = a->ncols ? a->mask : nullptr;
  p->md.minmax = a->ncols ? a->minmax : nullptr;
  p->md.ncols = a->ncols; p->md.causal = a->causal; p->md.Hm = a->ncols ? a->Hm : 1;
  p->md.mask_B = a->ncols ? a->mask_B : 1;
  p->md.nblk_pad = fm_mask_nblk_pad(a->Sk, a->tile_n > 0 ? a->tile_n : 64);
  p->md.BHm = p->md.mask_B * p->md.Hm;
  p->md.Sq = a->Sq; p->md.Sk = a->Sk;
  if (a->ncols) { p->fwd_order = a->fwd_order; p->dq_order = a->dq_order; p->dkdv_order = a->dkdv_order; }
  if (backward) {
    p->d_o = a->d_o; p->dq = a->dq; p->dk = a->dk; p->dv = a->dv_out; p->dsink = a->dsink;
    p->do_b = a->do_stride[0]; p->do_s = a->do_stride[1]; p->do_h = a->do_stride[2];
    p->dq_b = a->dq_stride[0]; p->dq_s = a->dq_stride[1]; p->dq_h = a->dq_stride[2];
    p->dk_b = a->dk_stride[0]; p->dk_s = a->dk_stride[1]; p->dk_h = a->dk_stride[2];
    p->dv_b = a->dv_stride[0]; p->dv_s = a->dv_stride[1]; p->dv_h = a->dv_stride[2];
  }
  return FM_OK;
}

}  // namespace fm

using namespace fm;

extern "C" const char* fm_version(void) { return "flashmask_b200 0.1.0 sm_100a"; }
extern "C" const char* fm_last_error(void) { return g_err; }

extern "C" unsigned long long fm_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int fm_reload_options(void) {
  g_opt = read_options();
  return FM_OK;
}

static bool bwd_uses_sm100(int d, int dv) {
  const bool small = d <= 128 && dv <= 128 && d % 8 == 0 && dv % 8 == 0;
  if (!small && !(d == 192 && dv == 128)) return false;
  return !g_opt.bwd_mma;
}

// The one-kernel backward (five GEMMs per tile pair, dQ summed into an fp32 accumulator in an order
// that is not fixed) serves the tcgen05 head dims whenever the call does not ask for deterministic
// gradients; the two-kernel variant gives every output element one owner and a fixed order.
// Measured on 8K-128K masks it is 5-22 % faster at d = dv = 64 and d = dv = 128; head dims that only
// partly fill a 64-column box measured slower (d = 96: +25 %), so they keep the two-kernel variant.
static bool bwd_uses_fused(const fm_attn_args* a) {
  const bool exact = a->d == a->dv && (a->d == 64 || a->d == 128);
  return bwd_uses_sm100(a->d, a->dv) && exact && !a->deterministic && !g_opt.bwd_split;
}

// preprocess -> main kernels of the selected variant -> dsink, on one stream
static int run_bwd_kernels(const fm_attn_args* a, const AttnKParams& p, cudaStream_t s) {
  int rc = bwd_preprocess_launch(p, a->dtype, s);
  if (rc != FM_OK) return rc;
  if (bwd_uses_sm100(a->d, a->dv)) {
    FM_REQUIRE(bwd_sm100_supported(a), FM_ERR_INVALID_ARGUMENT, "backward: q/k/v/d_o must be 16-byte aligned");
    if (p.dq_accum) {
      rc = bwd_sm100_fused_launch(p, a, s);
      if (rc != FM_OK) return rc;
      if (a->sink) rc = bwd_dsink_launch(p, s);
      return rc;
    }
    // With launch tables (a mask tensor) the persistent variant walks them; without, one unit per CTA.
    // Measured on six 8K-32K masks the persistent variant is 3-14 % faster where units are short
    // (documents, windows) and 3-5 % slower where every unit is hundreds of items long (its main loop
    // is slightly slower; the table records in [E+2] which side of that line a mask is on).
    // FLASHMASK_B200_PERSIST=0 keeps the one-unit-per-CTA variant.
    // (Without tables the persistent kernels also work, one unit per CTA, bitwise the same; measured on dense
    // masks they are 5-12 % slower than the one-unit kernels, which is why both exist.)
    const bool persist = p.dq_order && p.dkdv_order && g_opt.bwd_persist && a->d <= 128;   // 192 / 128: one-unit kernels only
    rc = persist ? bwd_sm100_persist_launch(p, a, s) : bwd_sm100_launch(p, a, s);
  } else {
    rc = bwd_mma_launch(p, a->dtype, s);
  }
  if (rc != FM_OK) return rc;
  if (a->sink) rc = bwd_dsink_launch(p, s);
  return rc;
}

extern "C" int fm_fwd_tile_shape(int d, int dv, int* tile_m, int* tile_n) {
  FM_REQUIRE(tile_m && tile_n, FM_ERR_INVALID_ARGUMENT, "fm_fwd_tile_shape: NULL output");
  if (fwd_uses_sm100(d, dv)) { *tile_m = 128; *tile_n = 128; return FM_OK; }
  int rc = fwd_mma_tile_shape(d, dv, tile_m, tile_n);
  if (rc != FM_OK) set_error("fm_fwd_tile_shape: unsupported head dims (d=%d, dv=%d)", d, dv);
  return rc;
}

extern "C" int fm_bwd_tile_shape(int d, int dv, int* tile_m, int* tile_n) {
  FM_REQUIRE(tile_m && tile_n, FM_ERR_INVALID_ARGUMENT, "fm_bwd_tile_shape: NULL output");
  if (bwd_uses_sm100(d, dv)) { *tile_m = 64; *tile_n = 128; return FM_OK; }
  int rc = bwd_mma_tile_shape(d, dv, tile_m, tile_n);
  if (rc != FM_OK) set_error("fm_bwd_tile_shape: unsupported head dims (d=%d, dv=%d)", d, dv);
  return rc;
}

// Side output of the forward (fm_fwd_block_score); block_logit == nullptr: none.
struct BlockScore { float* block_logit; const int32_t* block_bos; int block_size, block_ld; };

static int fwd_impl(const fm_attn_args* a, const BlockScore& bs, void* stream) {
  int rc = validate_common(a, "fm_fwd");
  if (rc != FM_OK) return rc;
  int tm, tn;
  rc = fm_fwd_tile_shape(a->d, a->dv, &tm, &tn);
  if (rc != FM_OK) return rc;
  FM_REQUIRE(a->ncols == 0 || a->tile_n == tn, FM_ERR_INVALID_ARGUMENT,
             "fm_fwd: minmax was prepared for tile_n=%d, this variant needs %d", a->tile_n, tn);
  AttnKParams p;
  fill_kparams(a, &p, false);
  p.md.nblk_pad = fm_mask_nblk_pad(a->Sk, tn);
  if (bs.block_logit) {
    FM_REQUIRE(bs.block_size == 32 || bs.block_size == 64 || bs.block_size == 128, FM_ERR_UNSUPPORTED,
               "fm_fwd_block_score: block_size must be 32, 64 or 128 (got %d)", bs.block_size);
    p.block_cols = (a->Sk + bs.block_size - 1) / bs.block_size;
    FM_REQUIRE(bs.block_ld >= p.block_cols, FM_ERR_INVALID_ARGUMENT,
               "fm_fwd_block_score: block_logit has %d blocks per row, ceil(Sk / block_size) = %d are needed",
               bs.block_ld, p.block_cols);
    p.block_logit = bs.block_logit; p.block_bos = bs.block_bos; p.block_ld = bs.block_ld;
    p.block_log2 = bs.block_size == 32 ? 5 : (bs.block_size == 64 ? 6 : 7);
    // the tcgen05 kernels have compile-time variants for it; the warp-MMA kernels (head dims 256 and up,
    // or FLASHMASK_B200_FWD=mma) a run-time branch
    if (fwd_uses_sm100(a->d, a->dv) && fwd_sm100_supported(a)) return fwd_sm100_launch(p, a, (cudaStream_t)stream);
    FM_REQUIRE(!fwd_uses_sm100(a->d, a->dv), FM_ERR_INVALID_ARGUMENT, "fm_fwd_block_score: q/k/v must be 16-byte aligned");
    return fwd_mma_launch(p, a->dtype, (cudaStream_t)stream);
  }
  if (fwd_uses_sm100(a->d, a->dv) && fwd_sm100_supported(a)) return fwd_sm100_launch(p, a, (cudaStream_t)stream);
  FM_REQUIRE(!fwd_uses_sm100(a->d, a->dv), FM_ERR_INVALID_ARGUMENT,
             "fm_fwd: q/k/v must be 16-byte aligned");
  return fwd_mma_launch(p, a->dtype, (cudaStream_t)stream);
}

extern "C" int fm_fwd(const fm_attn_args* a, void* stream) { return fwd_impl(a, BlockScore{}, stream); }

extern "C" int fm_fwd_block_score(const fm_attn_args* a, float* block_logit, int block_size, int block_ld,
                                  const int32_t* block_bos, void* stream) {
  FM_REQUIRE(block_logit != nullptr, FM_ERR_INVALID_ARGUMENT, "fm_fwd_block_score: block_logit is NULL");
  return fwd_impl(a, BlockScore{block_logit, block_bos, block_size, block_ld}, stream);
}

// Geometry of a launch order: the ordered axis, rows per unit, the block the work is
// counted in, and how often a unit repeats (heads per mask head, batches per mask batch).
// Only the tcgen05 variants read an order.
struct OrderGeom { int axis, block_rows, n_units, n_other, heads, rep_h, rep_b; int64_t E, n_cta; };
static bool order_geometry_any(const fm_attn_args* a, int which, OrderGeom* g) {
  if (!a || a->ncols == 0 || a->Sq <= 0 || a->Sk <= 0 || a->B <= 0 || a->Hq <= 0 || a->Hkv <= 0) return false;
  if (!(a->Hm == 1 || a->Hm == a->Hkv) || !(a->mask_B == 1 || a->mask_B == a->B) || a->Hq % a->Hkv) return false;
  const int nk = (a->Sk + 127) / 128;
  // (the 256-column forward owns 128 rows per CTA and takes no table; the 192-column backward runs the
  // one-unit kernels, which take none either)
  if (which == FM_ORDER_FWD) {
    if (!fwd_uses_sm100(a->d, a->dv) || a->d > 192) return false;
    *g = OrderGeom{0, 256, (a->Sq + 255) / 256, nk, a->Hq};
  } else if (which == FM_ORDER_BWD_DQ) {
    if (!bwd_uses_sm100(a->d, a->dv) || a->d > 128) return false;
    *g = OrderGeom{0, 128, (a->Sq + 127) / 128, nk, a->Hq};
  } else if (which == FM_ORDER_BWD_DKDV) {
    if (!bwd_uses_sm100(a->d, a->dv) || a->d > 128) return false;
    *g = OrderGeom{1, 64, nk, (a->Sq + 63) / 64, a->Hkv};
  } else {
    return false;
  }
  g->rep_h = g->heads / a->Hm;
  g->rep_b = a->B / a->mask_B;
  g->E = (int64_t)a->mask_B * a->Hm * g->n_units;
  g->n_cta = g->E * g->rep_h * g->rep_b;
  return g->E <= FM_ORDER_MAX_UNITS && g->n_cta < (1ll << 30);
}

static bool order_geometry(const fm_attn_args* a, int which, OrderGeom* g) {
  if (!order_geometry_any(a, which, g)) return false;
  // The backward kernels walk their table persistently (the next unit is fetched and its list
  // built while the current one is in its main loop), so a table never costs them a dependent
  // load on the critical path; the forward reads its entry at CTA start and gains wherever CTAs
  // differ in work.  All three are built whenever the geometry allows.
  return true;
}

extern "C" int64_t fm_launch_order_ints(const fm_attn_args* a, int which) {
  OrderGeom g;
  if (!order_geometry(a, which, &g)) return 0;
  return 2 * g.n_cta + 2 * g.E + 4;
}

// The counters of the persistent kernels live behind the table and the two unit arrays.
static void attach_bwd_tables(const fm_attn_args* a, AttnKParams* p) {
  OrderGeom g;
  p->dq_sched = p->dkdv_sched = nullptr;
  p->dq_ncta = p->dkdv_ncta = 0;
  if (p->dq_order && order_geometry_any(a, FM_ORDER_BWD_DQ, &g)) {
    p->dq_ncta = (int)g.n_cta;
    p->dq_sched = const_cast<int*>(p->dq_order) + 2 * g.n_cta + 2 * g.E;
  } else {
    p->dq_order = nullptr;
  }
  if (p->dkdv_order && order_geometry_any(a, FM_ORDER_BWD_DKDV, &g)) {
    p->dkdv_ncta = (int)g.n_cta;
    p->dkdv_sched = const_cast<int*>(p->dkdv_order) + 2 * g.n_cta + 2 * g.E;
  } else {
    p->dkdv_order = nullptr;
  }
}

static OrderJob order_job(const fm_attn_args* a, int which, const OrderGeom& g, int32_t* out) {
  // work items per unit of work: two 64-key halves per K tile (dQ), one per q head of the group (dK/dV)
  const int item_mult = which == FM_ORDER_BWD_DQ ? 2 : (which == FM_ORDER_BWD_DKDV ? a->Hq / a->Hkv : 1);
  return OrderJob{g.axis, g.block_rows, g.n_units, g.n_other, g.rep_h, g.rep_b, g.heads, item_mult, out};
}

extern "C" int fm_launch_order(const fm_attn_args* a, int which, int32_t* out, void* stream) {
  int32_t* outs[3] = {nullptr, nullptr, nullptr};
  FM_REQUIRE(which >= 0 && which < 3, FM_ERR_INVALID_ARGUMENT, "fm_launch_order: unknown kernel %d", which);
  FM_REQUIRE(out != nullptr, FM_ERR_INVALID_ARGUMENT, "fm_launch_order: NULL argument");
  outs[which] = out;
  return fm_launch_orders(a, outs[0], outs[1], outs[2], stream);
}

extern "C" int fm_launch_orders(const fm_attn_args* a, int32_t* out_fwd, int32_t* out_dq, int32_t* out_dkdv,
                                void* stream) {
  FM_REQUIRE(a && (out_fwd || out_dq || out_dkdv), FM_ERR_INVALID_ARGUMENT, "fm_launch_orders: NULL argument");
  FM_REQUIRE(a->minmax && a->tile_n == 128, FM_ERR_INVALID_ARGUMENT,
             "fm_launch_orders: minmax must be prepared with tile_n = 128");
  int32_t* outs[3] = {out_fwd, out_dq, out_dkdv};
  OrderJobs jobs;
  int n = 0;
  for (int which = 0; which < 3; ++which) {
    if (!outs[which]) continue;
    OrderGeom g;
    FM_REQUIRE(order_geometry(a, which, &g), FM_ERR_UNSUPPORTED,
               "fm_launch_orders: no order for kernel %d with this variant / mask (fm_launch_order_ints returned 0)",
               which);
    FM_REQUIRE(((uintptr_t)outs[which] & 7) == 0, FM_ERR_INVALID_ARGUMENT, "fm_launch_orders: out must be 8-byte aligned");
    jobs.job[n++] = order_job(a, which, g, outs[which]);
  }
  MaskDesc md{a->mask, a->minmax, a->ncols, a->causal, a->Hm, a->mask_B, fm_mask_nblk_pad(a->Sk, 128),
              a->mask_B * a->Hm, a->Sq, a->Sk};
  return launch_order_build(md, 128, jobs, n, (cudaStream_t)stream);
}

// Workspace layout: rowsum(O dO) and LSE*log2e, one float each per (batch, q head, padded row),
// then (one-kernel backward only) the fp32 dQ accumulator, 256-byte aligned.
static size_t bwd_row_stat_bytes(const fm_attn_args* a) {
  const size_t rows = (size_t)a->B * a->Hq * round_up(a->Sq, 128);
  return (2 * rows * sizeof(float) + 255) & ~(size_t)255;
}

// One-kernel backward: the statistics once more as 16-bit GEMM operands, 2 x 16 bytes per row.
static size_t bwd_stat_operand_bytes(const fm_attn_args* a) {
  return (size_t)a->B * a->Hq * round_up(a->Sq, 128) * 32;
}

extern "C" size_t fm_bwd_workspace_bytes(const fm_attn_args* a) {
  if (!a || a->B <= 0 || a->Hq <= 0 || a->Sq <= 0) return 0;
  return bwd_row_stat_bytes(a) +
         (bwd_uses_fused(a) ? bwd_sm100_fused_accum_bytes(a) + bwd_stat_operand_bytes(a) : 0);
}

extern "C" int fm_bwd_accumulates(const fm_attn_args* a) {
  return (a && a->d > 0 && a->dv > 0 && bwd_uses_fused(a)) ? 1 : 0;
}

extern "C" int fm_bwd(const fm_attn_args* a, void* stream) {
  int rc = validate_common(a, "fm_bwd");
  if (rc != FM_OK) return rc;
  FM_REQUIRE(a->d_o && a->dq && a->dk && a->dv_out, FM_ERR_INVALID_ARGUMENT,
             "fm_bwd: d_o/dq/dk/dv must not be NULL");
  FM_REQUIRE(stride_ok(a->do_stride) && stride_ok(a->dq_stride) && stride_ok(a->dk_stride) &&
                 stride_ok(a->dv_stride),
             FM_ERR_INVALID_ARGUMENT, "fm_bwd: strides must be multiples of 8 elements");
  FM_REQUIRE(!(a->sink && !a->dsink), FM_ERR_INVALID_ARGUMENT, "fm_bwd: sink given but dsink is NULL");
  int tm, tn;
  rc = fm_bwd_tile_shape(a->d, a->dv, &tm, &tn);
  if (rc != FM_OK) return rc;
  FM_REQUIRE(a->ncols == 0 || a->tile_n == tn, FM_ERR_INVALID_ARGUMENT,
             "fm_bwd: minmax was prepared for tile_n=%d, this variant needs %d", a->tile_n, tn);
  const size_t need = fm_bwd_workspace_bytes(a);
  FM_REQUIRE(a->workspace && a->workspace_bytes >= need, FM_ERR_WORKSPACE,
             "fm_bwd: workspace too small (%zu bytes given, %zu needed)", a->workspace_bytes, need);
  FM_REQUIRE(((uintptr_t)a->workspace & 255) == 0, FM_ERR_WORKSPACE, "fm_bwd: workspace must be 256-byte aligned");
  AttnKParams p;
  fill_kparams(a, &p, true);
  p.md.nblk_pad = fm_mask_nblk_pad(a->Sk, tn);
  const size_t rows = (size_t)a->B * a->Hq * p.Sq_r;
  p.dpsum = reinterpret_cast<float*>(a->workspace);
  p.lse_log2 = p.dpsum + rows;
  if (bwd_uses_fused(a)) {
    uint8_t* w = reinterpret_cast<uint8_t*>(a->workspace) + bwd_row_stat_bytes(a);
    p.dq_accum = reinterpret_cast<float*>(w);
    p.stat_s = reinterpret_cast<uint16_t*>(w + bwd_sm100_fused_accum_bytes(a));
    p.stat_dp = p.stat_s + (size_t)a->B * a->Hq * p.Sq_r * 8;
    p.bwd_flags = a->bwd_flags;
  }
  cudaStream_t s = (cudaStream_t)stream;
  attach_bwd_tables(a, &p);
  return run_bwd_kernels(a, p, s);
}

extern "C" int fm_kernel_status(int* status, int reset) {
  FM_REQUIRE(status != nullptr, FM_ERR_INVALID_ARGUMENT, "fm_kernel_status: NULL output");
  int f = 0, bw = 0;
  int rc = fwd_sm100_status(&f, reset != 0);
  if (rc != FM_OK) return rc;
  rc = bwd_sm100_status(&bw, reset != 0);
  if (rc != FM_OK) return rc;
  int bp = 0, bf = 0;
  rc = bwd_sm100_persist_status(&bp, reset != 0);
  if (rc != FM_OK) return rc;
  rc = bwd_sm100_fused_status(&bf, reset != 0);
  *status = f ? f : (bw ? bw : (bp ? bp : bf));
  return rc;
}

extern "C" int fm_selftest_bounded_wait(int budget_us, void* stream) {
  FM_REQUIRE(budget_us > 0 && budget_us <= 1000000, FM_ERR_INVALID_ARGUMENT,
             "fm_selftest_bounded_wait: budget must be in (0, 1 s]");
  return bounded_wait_selftest_launch((uint64_t)budget_us * 1000ull, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------
// Backward for callers that must not allocate
// ---------------------------------------------------------------------------
// Row-statistics scratch of the backward (rowsum(O*dO) and LSE*log2(e), one
// float each per (batch, q head, padded query row)) held in the library image
// instead of a caller workspace.  Every GPU that loads the library carries
// these 8 MiB until the process exits.
#define FM_STATIC_SCRATCH_ROWS (1 << 20)
static __device__ __align__(256) float g_bwd_row_scratch[2 * FM_STATIC_SCRATCH_ROWS];

// Device address of the array above, per device ordinal.  In host code the
// array's name is only a handle; the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
static float* g_bwd_row_scratch_addr[64] = {nullptr};

static int static_scratch_for_current_device(float** out) {
  int dev = -1;
  FM_CUDA_TRY(cudaGetDevice(&dev));
  FM_REQUIRE(dev >= 0 && dev < 64, FM_ERR_UNSUPPORTED, "fm_bwd_static_scratch: device ordinal %d not supported", dev);
  if (g_bwd_row_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    FM_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_bwd_row_scratch));
    FM_REQUIRE(ptr != nullptr, FM_ERR_CUDA, "fm_bwd_static_scratch: cudaGetSymbolAddress returned NULL");
    g_bwd_row_scratch_addr[dev] = static_cast<float*>(ptr);
  }
  *out = g_bwd_row_scratch_addr[dev];
  return FM_OK;
}

extern "C" int fm_bwd_static_scratch(const fm_attn_args* a, void* stream) {
  int rc = validate_common(a, "fm_bwd_static_scratch");
  if (rc != FM_OK) return rc;
  FM_REQUIRE(a->d_o && a->dq && a->dk && a->dv_out, FM_ERR_INVALID_ARGUMENT,
             "fm_bwd_static_scratch: d_o/dq/dk/dv must not be NULL");
  FM_REQUIRE(stride_ok(a->do_stride) && stride_ok(a->dq_stride) && stride_ok(a->dk_stride) &&
                 stride_ok(a->dv_stride),
             FM_ERR_INVALID_ARGUMENT, "fm_bwd_static_scratch: strides must be multiples of 8 elements");
  FM_REQUIRE(!(a->sink && !a->dsink), FM_ERR_INVALID_ARGUMENT,
             "fm_bwd_static_scratch: sink given but dsink is NULL");
  int tm, tn;
  rc = fm_bwd_tile_shape(a->d, a->dv, &tm, &tn);
  if (rc != FM_OK) return rc;
  FM_REQUIRE(a->ncols == 0 || a->tile_n == tn, FM_ERR_INVALID_ARGUMENT,
             "fm_bwd_static_scratch: minmax was prepared for tile_n=%d, this variant needs %d", a->tile_n, tn);
  const size_t rows = (size_t)a->B * a->Hq * round_up(a->Sq, 128);
  FM_REQUIRE(rows <= (size_t)FM_STATIC_SCRATCH_ROWS, FM_ERR_WORKSPACE,
             "fm_bwd_static_scratch: B*Hq*roundup(Sq,128) = %zu rows exceeds the built-in scratch of %d rows; "
             "use fm_bwd with a caller workspace",
             rows, FM_STATIC_SCRATCH_ROWS);
  float* scratch = nullptr;
  rc = static_scratch_for_current_device(&scratch);
  if (rc != FM_OK) return rc;
  AttnKParams p;
  fill_kparams(a, &p, true);
  p.md.nblk_pad = fm_mask_nblk_pad(a->Sk, tn);
  // Both halves are fully rewritten by the preprocess kernel for every row the
  // later kernels read, so nothing left by an earlier call has to be cleared.
  p.dpsum = scratch;
  p.lse_log2 = scratch + rows;
  attach_bwd_tables(a, &p);
  return run_bwd_kernels(a, p, (cudaStream_t)stream);
}

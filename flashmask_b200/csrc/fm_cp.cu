// Context-parallel support kernels and the host-side partitioner.
//
//  * workload per balance chunk from the surviving-tile counts
//  * key-axis rerank of the mask into rank order, row-bound localisation
//  * visible-pair count per key shard (which remote shards a rank needs)
//  * forward partial merge by log-sum-exp, fp32 accumulate / cast helpers
//  * fixed-order fp32 reduction of bf16 dK/dV partials
//  * LPT heap partition (host C++)
// All integer / elementwise work is HBM-bound: flat grids, 16-byte accesses
// where the layout allows.
#include <algorithm>
#include <queue>
#include <vector>

#include "fm_common.cuh"

namespace fm {

// workload[h, c] = sum over batch and over the 128-row blocks of chunk c of the
// number of K blocks that are not fully masked.  out[h, c] = {workload, c}.
__global__ void cp_chunk_workload_kernel(const int32_t* __restrict__ valid_cnt, int B, int Hm, int Tq,
                                         int blocks_per_chunk, int n_chunks, int32_t* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int h = blockIdx.y;
  if (c >= n_chunks) return;
  int acc = 0;
  for (int b = 0; b < B; ++b) {
    const int32_t* src = valid_cnt + ((size_t)b * Hm + h) * Tq + (size_t)c * blocks_per_chunk;
    for (int t = 0; t < blocks_per_chunk; ++t)
      if (c * blocks_per_chunk + t < Tq) acc += src[t];
  }
  out[((size_t)h * n_chunks + c) * 2 + 0] = acc;
  out[((size_t)h * n_chunks + c) * 2 + 1] = c;
}

// out[b,h,s_out,:] = in[b,h, chunk_idx[s_out / C] * C + s_out % C, :]; rows that
// map past S are left untouched.
__global__ void cp_rerank_kernel(const int32_t* __restrict__ in, const int32_t* __restrict__ chunk_idx,
                                 int32_t* __restrict__ out, int BH, int S, int D, int n_chunks, int C) {
  const int64_t total = (int64_t)BH * n_chunks * C * D;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int d = (int)(i % D);
  const int64_t s_out = (i / D) % ((int64_t)n_chunks * C);
  const int64_t bh = i / D / ((int64_t)n_chunks * C);
  const int64_t src_s = (int64_t)chunk_idx[s_out / C] * C + s_out % C;
  if (src_s >= S) return;
  out[i] = in[(bh * S + src_s) * D + d];
}

// Row bound v (global row index) -> position in the concatenation of this
// rank's chunks: max over local chunks k of clamp(v - chunk[k]*C, 0, C) (+ k*C
// when positive).
__global__ void cp_localize_kernel(const int32_t* __restrict__ in, const int32_t* __restrict__ chunk_idx,
                                   int32_t* __restrict__ out, int64_t n, int n_local, int C) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int v = in[i];
  int best = 0;
  for (int k = 0; k < n_local; ++k) {
    int loc = v - chunk_idx[k] * C;
    loc = max(loc, 0);
    loc = min(loc, C);
    if (loc > 0) loc += k * C;
    if (k == 0 || loc > best) best = loc;
  }
  out[i] = best;
}

// visible[(b*Hm+h), shard] = number of unmasked (row, column) pairs with the
// column inside key shard `shard` (columns [shard*S_shard, (shard+1)*S_shard)).
__global__ void __launch_bounds__(256) cp_shard_visible_kernel(MaskDesc md, int S_shard, int n_shards,
                                                              int64_t* __restrict__ out) {
  const int shard = blockIdx.x, bh = blockIdx.y;
  const int Sq = md.Sq, Sk = md.Sk, off = Sk - Sq;
  long long acc = 0;
  const int j_end = min(Sk, (shard + 1) * S_shard);
  for (int j = shard * S_shard + threadIdx.x; j < j_end; j += blockDim.x) {
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
    out[(size_t)bh * n_shards + shard] = s;
  }
}

template <bool IS_BF16>
__device__ __forceinline__ float2 unpack2(uint32_t v) {
  if constexpr (IS_BF16) return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
  else return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

// Running merge of forward partials: (acc, lse_run) <- merge with (o_s, lse_s)
//   new = logaddexp(lse_run, lse_s); acc = acc*exp(lse_run-new) + o_s*exp(lse_s-new)
// acc [B,S,H,dv] fp32, o_s [B,S,H,dv] 16-bit, lse [B,H,S] fp32.  One warp per row.
template <bool IS_BF16>
__global__ void __launch_bounds__(256) cp_merge_kernel(float* __restrict__ acc, float* __restrict__ lse_run,
                                                      const uint16_t* __restrict__ o_s,
                                                      const float* __restrict__ lse_s, int B, int S, int H,
                                                      int dv, int first) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;  // (b, s, h)
  if (row >= (int64_t)B * S * H) return;
  const int h = (int)(row % H);
  const int64_t bs = row / H;
  const int s = (int)(bs % S);
  const int b = (int)(bs / S);
  const int64_t li = ((int64_t)b * H + h) * S + s;
  const float ls = lse_s[li];
  float wa, ws, ln;
  if (first) { wa = 0.f; ws = 1.f; ln = ls; }
  else {
    const float lr = lse_run[li];
    const float mx = fmaxf(lr, ls);
    if (mx == -INFINITY) { wa = 0.f; ws = 0.f; ln = -INFINITY; }
    else {
      const float ea = __expf(lr - mx), es = __expf(ls - mx);
      ln = mx + __logf(ea + es);
      wa = __expf(lr - ln); ws = __expf(ls - ln);
    }
  }
  float* a = acc + row * dv;
  const uint16_t* o = o_s + row * dv;
  for (int c = lane * 4; c < dv; c += 128) {
    const uint2 raw = *reinterpret_cast<const uint2*>(o + c);
    const float2 x = unpack2<IS_BF16>(raw.x), y = unpack2<IS_BF16>(raw.y);
    float4 av = first ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(a + c);
    av.x = av.x * wa + x.x * ws; av.y = av.y * wa + x.y * ws;
    av.z = av.z * wa + y.x * ws; av.w = av.w * wa + y.y * ws;
    *reinterpret_cast<float4*>(a + c) = av;
  }
  if (lane == 0) lse_run[li] = ln;
}

// Merge of exactly two forward partials straight into the 16-bit output:
//   lse = logaddexp(lse_a, lse_b); out = o_a*exp(lse_a-lse) + o_b*exp(lse_b-lse), rounded once.
// One warp per (b, s, h) row; reads two 16-bit rows, writes one (no fp32 accumulator round trip).
template <bool IS_BF16>
__global__ void __launch_bounds__(256) cp_merge_two_kernel(const uint16_t* o_a, const float* __restrict__ lse_a,
                                                          const uint16_t* __restrict__ o_b, const float* __restrict__ lse_b,
                                                          uint16_t* out, float* __restrict__ lse_out,
                                                          int B, int S, int H, int dv) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 8 + warp;  // (b, s, h)
  if (row >= (int64_t)B * S * H) return;
  const int h = (int)(row % H);
  const int64_t bs = row / H;
  const int s = (int)(bs % S);
  const int b = (int)(bs / S);
  const int64_t li = ((int64_t)b * H + h) * S + s;
  const float la = lse_a[li], lb = lse_b[li];
  const float mx = fmaxf(la, lb);
  float wa = 0.f, wb = 0.f, ln = -INFINITY;
  if (mx != -INFINITY) {
    const float ea = __expf(la - mx), eb = __expf(lb - mx);
    ln = mx + __logf(ea + eb);
    wa = __expf(la - ln); wb = __expf(lb - ln);
  }
  const uint16_t* pa = o_a + row * dv;
  const uint16_t* pb = o_b + row * dv;
  uint16_t* po = out + row * dv;
  for (int c = lane * 8; c < dv; c += 256) {
    const uint4 ra = *reinterpret_cast<const uint4*>(pa + c), rb = *reinterpret_cast<const uint4*>(pb + c);
    const uint32_t av[4] = {ra.x, ra.y, ra.z, ra.w}, bv[4] = {rb.x, rb.y, rb.z, rb.w};
    uint32_t ov[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x = unpack2<IS_BF16>(av[e]), y = unpack2<IS_BF16>(bv[e]);
      ov[e] = pack2<IS_BF16>(x.x * wa + y.x * wb, x.y * wa + y.y * wb);
    }
    *reinterpret_cast<uint4*>(po + c) = make_uint4(ov[0], ov[1], ov[2], ov[3]);
  }
  if (lane == 0) lse_out[li] = ln;
}

template <bool IS_BF16>
__global__ void cp_add_kernel(float* __restrict__ acc, const uint16_t* __restrict__ x, int64_t n, int first) {
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  const uint2 raw = *reinterpret_cast<const uint2*>(x + i);
  const float2 p = unpack2<IS_BF16>(raw.x), q = unpack2<IS_BF16>(raw.y);
  float4 a = first ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(acc + i);
  a.x += p.x; a.y += p.y; a.z += q.x; a.w += q.y;
  *reinterpret_cast<float4*>(acc + i) = a;
}

template <bool IS_BF16>
__global__ void cp_cast_kernel(const float* __restrict__ acc, uint16_t* __restrict__ out, int64_t n) {
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  const float4 a = *reinterpret_cast<const float4*>(acc + i);
  uint2 r;
  r.x = pack2<IS_BF16>(a.x, a.y);
  r.y = pack2<IS_BF16>(a.z, a.w);
  *reinterpret_cast<uint2*>(out + i) = r;
}

struct PartialPtrs {
  const uint16_t* p[64];
};

// out = round(sum_i fp32(partial_i)), summed in index order: deterministic.
template <bool IS_BF16>
__global__ void cp_reduce_partials_kernel(PartialPtrs ptrs, int n_parts, uint16_t* __restrict__ out, int64_t n) {
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int k = 0; k < n_parts; ++k) {
    const uint2 raw = *reinterpret_cast<const uint2*>(ptrs.p[k] + i);
    const float2 x = unpack2<IS_BF16>(raw.x), y = unpack2<IS_BF16>(raw.y);
    a.x += x.x; a.y += x.y; a.z += y.x; a.w += y.y;
  }
  uint2 r;
  r.x = pack2<IS_BF16>(a.x, a.y);
  r.y = pack2<IS_BF16>(a.z, a.w);
  *reinterpret_cast<uint2*>(out + i) = r;
}

}  // namespace fm

using namespace fm;

extern "C" int fm_cp_chunk_workload(const int32_t* valid_cnt, int B, int Hm, int Tq, int blocks_per_chunk,
                                    int32_t* out, void* stream) {
  FM_REQUIRE(valid_cnt && out && B > 0 && Hm > 0 && Tq > 0 && blocks_per_chunk > 0, FM_ERR_INVALID_ARGUMENT,
             "fm_cp_chunk_workload: bad arguments");
  const int n_chunks = (Tq + blocks_per_chunk - 1) / blocks_per_chunk;
  cp_chunk_workload_kernel<<<dim3((n_chunks + 127) / 128, Hm), 128, 0, (cudaStream_t)stream>>>(
      valid_cnt, B, Hm, Tq, blocks_per_chunk, n_chunks, out);
  count_launches(1);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

extern "C" int fm_cp_rerank(const int32_t* mask, const int32_t* chunk_idx, int32_t* out, int B, int H, int S,
                            int D, int n_chunks, int chunk_size, void* stream) {
  FM_REQUIRE(mask && chunk_idx && out && B > 0 && H > 0 && S > 0 && D > 0 && n_chunks > 0 && chunk_size > 0,
             FM_ERR_INVALID_ARGUMENT, "fm_cp_rerank: bad arguments");
  const int64_t total = (int64_t)B * H * n_chunks * chunk_size * D;
  cp_rerank_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(mask, chunk_idx, out, B * H, S,
                                                                                      D, n_chunks, chunk_size);
  count_launches(1);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

extern "C" int fm_cp_localize(const int32_t* mask, const int32_t* local_chunk_idx, int32_t* out, int64_t n,
                              int n_local, int chunk_size, void* stream) {
  FM_REQUIRE(mask && local_chunk_idx && out && n > 0 && n_local > 0 && chunk_size > 0, FM_ERR_INVALID_ARGUMENT,
             "fm_cp_localize: bad arguments");
  cp_localize_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(mask, local_chunk_idx, out, n,
                                                                                    n_local, chunk_size);
  count_launches(1);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

extern "C" int fm_cp_shard_visible(const int32_t* mask, int B, int Hm, int Sq, int Sk, int ncols, int causal,
                                   int n_shards, int64_t* out, void* stream) {
  FM_REQUIRE(mask && out && n_shards > 0 && Sk % n_shards == 0 && (ncols == 1 || ncols == 2 || ncols == 4),
             FM_ERR_INVALID_ARGUMENT, "fm_cp_shard_visible: Sk must be a multiple of the shard count");
  MaskDesc md{mask, nullptr, ncols, causal, Hm, B, 0, B * Hm, Sq, Sk};
  cp_shard_visible_kernel<<<dim3(n_shards, B * Hm), 256, 0, (cudaStream_t)stream>>>(md, Sk / n_shards, n_shards, out);
  count_launches(1);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

extern "C" int fm_cp_merge_partial(float* acc, float* lse_run, const void* o_s, const float* lse_s, int B, int S,
                                   int H, int dv, int dtype, int first, void* stream) {
  FM_REQUIRE(acc && lse_run && o_s && lse_s && dv % 4 == 0, FM_ERR_INVALID_ARGUMENT, "fm_cp_merge_partial: bad arguments");
  const int64_t rows = (int64_t)B * S * H;
  const unsigned grid = (unsigned)((rows + 7) / 8);
  if (dtype == FM_DTYPE_BF16)
    cp_merge_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(acc, lse_run, (const uint16_t*)o_s, lse_s, B, S, H, dv, first);
  else
    cp_merge_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(acc, lse_run, (const uint16_t*)o_s, lse_s, B, S, H, dv, first);
  count_launches(1);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

extern "C" int fm_cp_merge_two(const void* o_a, const float* lse_a, const void* o_b, const float* lse_b, void* out,
                               float* lse_out, int B, int S, int H, int dv, int dtype, void* stream) {
  FM_REQUIRE(o_a && lse_a && o_b && lse_b && out && lse_out && dv % 8 == 0, FM_ERR_INVALID_ARGUMENT,
             "fm_cp_merge_two: bad arguments (dv must be a multiple of 8)");
  const int64_t rows = (int64_t)B * S * H;
  const unsigned grid = (unsigned)((rows + 7) / 8);
  if (dtype == FM_DTYPE_BF16)
    cp_merge_two_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)o_a, lse_a, (const uint16_t*)o_b, lse_b,
                                                                      (uint16_t*)out, lse_out, B, S, H, dv);
  else
    cp_merge_two_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>((const uint16_t*)o_a, lse_a, (const uint16_t*)o_b, lse_b,
                                                                       (uint16_t*)out, lse_out, B, S, H, dv);
  count_launches(1);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

extern "C" int fm_cp_accumulate(float* acc, const void* x, int64_t n, int dtype, int first, void* stream) {
  FM_REQUIRE(acc && x && n > 0 && n % 4 == 0, FM_ERR_INVALID_ARGUMENT, "fm_cp_accumulate: n must be a multiple of 4");
  const unsigned grid = (unsigned)((n / 4 + 255) / 256);
  if (dtype == FM_DTYPE_BF16) cp_add_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(acc, (const uint16_t*)x, n, first);
  else cp_add_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(acc, (const uint16_t*)x, n, first);
  count_launches(1);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

extern "C" int fm_cp_cast(const float* acc, void* out, int64_t n, int dtype, void* stream) {
  FM_REQUIRE(acc && out && n > 0 && n % 4 == 0, FM_ERR_INVALID_ARGUMENT, "fm_cp_cast: n must be a multiple of 4");
  const unsigned grid = (unsigned)((n / 4 + 255) / 256);
  if (dtype == FM_DTYPE_BF16) cp_cast_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(acc, (uint16_t*)out, n);
  else cp_cast_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(acc, (uint16_t*)out, n);
  count_launches(1);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

extern "C" int fm_cp_reduce_partials(const void* const* parts, int n_parts, void* out, int64_t n, int dtype,
                                     void* stream) {
  FM_REQUIRE(parts && out && n_parts > 0 && n_parts <= 64 && n > 0 && n % 4 == 0, FM_ERR_INVALID_ARGUMENT,
             "fm_cp_reduce_partials: 1..64 partials, n a multiple of 4");
  PartialPtrs pp;
  for (int i = 0; i < n_parts; ++i) {
    FM_REQUIRE(parts[i] != nullptr, FM_ERR_INVALID_ARGUMENT, "fm_cp_reduce_partials: partial %d is NULL", i);
    pp.p[i] = (const uint16_t*)parts[i];
  }
  const unsigned grid = (unsigned)((n / 4 + 255) / 256);
  if (dtype == FM_DTYPE_BF16)
    cp_reduce_partials_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(pp, n_parts, (uint16_t*)out, n);
  else
    cp_reduce_partials_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(pp, n_parts, (uint16_t*)out, n);
  count_launches(1);
  FM_CUDA_TRY(cudaGetLastError());
  return FM_OK;
}

// Longest-processing-time heap partition with a per-bucket capacity of N / M
// tasks: tasks in weight-descending order (stable), each to the lightest
// bucket that still has room, or to the lightest bucket when all are full.
// bucket_of[t] receives the bucket of task t (input order).  Host pointers.
extern "C" int fm_cp_partition_heap(const int32_t* weights, int n, int n_buckets, int32_t* bucket_of) {
  FM_REQUIRE(weights && bucket_of && n >= 0 && n_buckets > 0, FM_ERR_INVALID_ARGUMENT,
             "fm_cp_partition_heap: bad arguments");
  const int cap = n / n_buckets;
  std::vector<int> order(n);
  for (int i = 0; i < n; ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return weights[a] > weights[b]; });
  typedef std::pair<long long, int> Item;  // (load, bucket): smallest first
  std::priority_queue<Item, std::vector<Item>, std::greater<Item>> heap;
  std::vector<long long> load(n_buckets, 0);
  std::vector<int> count(n_buckets, 0);
  for (int j = 0; j < n_buckets; ++j) heap.push(Item(0, j));
  std::vector<Item> parked;
  for (int t : order) {
    parked.clear();
    bool placed = false;
    while (!heap.empty()) {
      Item it = heap.top();
      heap.pop();
      if (count[it.second] < cap) {
        bucket_of[t] = it.second;
        load[it.second] += weights[t];
        count[it.second] += 1;
        heap.push(Item(load[it.second], it.second));
        placed = true;
        break;
      }
      parked.push_back(it);
    }
    for (const Item& it : parked) heap.push(it);
    if (!placed) {
      Item it = heap.top();
      heap.pop();
      bucket_of[t] = it.second;
      load[it.second] += weights[t];
      count[it.second] += 1;
      heap.push(Item(load[it.second], it.second));
    }
  }
  return FM_OK;
}

// Iterative pairwise / triple optimal repartition ("IPO") of weighted balance
// chunks over context-parallel ranks: n chunks, m ranks, every rank gets exactly
// k = n/m chunks, minimise the heaviest rank.
//
// Restates the algorithm of the reference's solver
// (flashmask/cp_balance/csrc/cp_balance_fast.hpp:416-581 and the sub-solvers at
// :118-414) decision for decision, so that the assignment — not only its
// maximum load — is the same:
//   1. LPT start: chunks by (weight desc, index asc), each to the lightest rank
//      that still has room (lowest rank on ties).
//   2. repeat: take the heaviest rank, re-split its 2k chunks with every other
//      rank exactly (meet in the middle for k <= 10, branch and bound above),
//      apply the partner that lowers the maximum most; when no pair helps and
//      k <= 8, re-split the heaviest rank with two partners (3-way branch and
//      bound against "strictly below the current maximum").
//   3. stop at the lower bound max(ceil(total/m), heaviest chunk), when a round
//      changes nothing, or after the round budget.
// Host code only; no device work.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <vector>

#include "flashmask_b200.h"
#include "fm_common.cuh"

namespace {

constexpr int kIpoMaxChunks = 512;   // callers fall back to the heap partition above this
constexpr int kIpoMaxRanks = 32;
constexpr int kIpoMaxPerRankOpt = 16;  // above this only the LPT start is returned
constexpr int kPairMax = 2 * kIpoMaxPerRankOpt + 2;
constexpr int kTripleMax = 3 * 8 + 2;

// order[] <- 0..n-1 sorted by (w desc, index asc): a strict total order, so any
// sorting algorithm gives the same permutation.
void order_heaviest_first(const int* w, int n, int* order) {
  for (int i = 0; i < n; ++i) order[i] = i;
  std::sort(order, order + n, [w](int a, int b) { return w[a] != w[b] ? w[a] > w[b] : a < b; });
}

// ---------------------------------------------------------------------------
// Depth-first search: can the items (sorted heaviest first) be dealt into G
// groups of exactly `per` items with every group sum <= limit?  Items are
// placed in order; the first feasible leaf wins, so the visiting order of the
// groups is part of the result.
// ---------------------------------------------------------------------------
template <int G>
struct EqualDealSearch {
  int n = 0, per = 0, limit = 0;
  const int* w = nullptr;       // sorted weights
  const int* tail = nullptr;    // tail[i] = sum of w[i..n)
  int sum[G] = {}, cnt[G] = {};
  int* where = nullptr;         // group of each sorted position
  long long visited = 0, budget = 0;

  bool place(int pos) {
    if (++visited > budget) return false;  // once exhausted every frame unwinds as "no"
    if (pos == n) return true;
    const int left = n - pos, cur = w[pos];
    int room = 0, open = 0, last = -1;
    for (int g = 0; g < G; ++g) {
      if (cnt[g] >= per) continue;
      if (G == 3) {
        // the `need` lightest remaining items are the least this group can still take
        const int need = per - cnt[g], from = n - need;
        if (from < pos) {
          if (left < need || tail[pos] + sum[g] > limit) return false;
        } else if (tail[from] + sum[g] > limit) {
          return false;
        }
      }
      room += limit - sum[g];
      ++open;
      last = g;
    }
    if (tail[pos] > room) return false;
    if (open == 1) {
      if (left != per - cnt[last] || tail[pos] + sum[last] > limit) return false;
      for (int p = pos; p < n; ++p) where[p] = last;
      return true;
    }
    // an item equal to its predecessor never goes to an earlier group than it did
    const int first = (pos > 0 && w[pos] == w[pos - 1]) ? where[pos - 1] : 0;
    int tried_sum[G], tried_cnt[G], tried = 0;
    for (int g = first; g < G; ++g) {
      if (cnt[g] >= per || sum[g] + cur > limit) continue;
      if (G == 2) {
        // two groups in the same state are interchangeable: only group 0 is explored
        if (g == 1 && sum[0] == sum[1] && cnt[0] == cnt[1]) continue;
      } else {
        bool same = false;
        for (int s = 0; s < tried; ++s) same = same || (tried_sum[s] == sum[g] && tried_cnt[s] == cnt[g]);
        if (same) continue;
        tried_sum[tried] = sum[g];
        tried_cnt[tried] = cnt[g];
        ++tried;
      }
      sum[g] += cur; ++cnt[g]; where[pos] = g;
      if (place(pos + 1)) return true;
      --cnt[g]; sum[g] -= cur;
    }
    return false;
  }

  bool run(int new_limit, long long node_budget) {
    limit = new_limit;
    budget = node_budget;
    visited = 0;
    for (int g = 0; g < G; ++g) sum[g] = cnt[g] = 0;
    return place(0);
  }
};

struct PairSplit {
  int heavier = 0;              // the larger of the two sums
  bool first[kPairMax] = {};    // item t goes to the first rank of the pair
};

// Exact equal-cardinality 2-way split of 2k items, k <= 10: enumerate the
// subsets of the second half grouped by size and ordered by sum, then for each
// subset of the first half look up the complement closest to half the total.
PairSplit split_pair_meet_in_middle(const int* item, int n_items) {
  const int k = n_items / 2, nb = n_items - k;
  int total = 0;
  for (int i = 0; i < n_items; ++i) total += item[i];
  struct Half { int sum; uint16_t pick; };
  static thread_local std::vector<Half> by_size[kIpoMaxPerRankOpt + 1];
  for (int s = 0; s <= nb; ++s) by_size[s].clear();
  for (int pick = 0; pick < (1 << nb); ++pick) {
    int s = 0;
    for (int i = 0; i < nb; ++i) s += (pick >> i & 1) ? item[k + i] : 0;
    by_size[__builtin_popcount(pick)].push_back(Half{s, static_cast<uint16_t>(pick)});
  }
  // ordered by sum only; which of several equal sums comes first follows std::sort
  for (int s = 0; s <= nb; ++s)
    std::sort(by_size[s].begin(), by_size[s].end(), [](const Half& a, const Half& b) { return a.sum < b.sum; });

  int best = total;
  uint32_t best_a = 0, best_b = 0;
  for (int pa = 0; pa < (1 << k); ++pa) {
    const int need = k - __builtin_popcount(pa);
    if (need < 0 || need > nb || by_size[need].empty()) continue;
    int sa = 0;
    for (int i = 0; i < k; ++i) sa += (pa >> i & 1) ? item[i] : 0;
    const std::vector<Half>& cand = by_size[need];
    const int want = (total + 1) / 2 - sa;
    const int at = static_cast<int>(std::lower_bound(cand.begin(), cand.end(), want,
                                                     [](const Half& h, int v) { return h.sum < v; }) - cand.begin());
    for (int c = at - 1; c <= at; ++c) {
      if (c < 0 || c >= static_cast<int>(cand.size())) continue;
      const int s0 = sa + cand[c].sum, worse = std::max(s0, total - s0);
      if (worse < best) { best = worse; best_a = pa; best_b = cand[c].pick; }
    }
  }
  PairSplit r;
  r.heavier = best;
  for (int i = 0; i < k; ++i) r.first[i] = best_a >> i & 1;
  for (int i = 0; i < nb; ++i) r.first[k + i] = best_b >> i & 1;
  return r;
}

// The same split for k > 10: LPT upper bound, then bisection on the limit with
// the depth-first search (500k nodes per probe; an exhausted probe counts as
// infeasible).
PairSplit split_pair_search(const int* item, int n_items) {
  const int k = n_items / 2;
  int order[kPairMax], w[kPairMax], tail[kPairMax + 1], where[kPairMax];
  order_heaviest_first(item, n_items, order);
  int total = 0;
  for (int i = 0; i < n_items; ++i) { w[i] = item[order[i]]; total += w[i]; }
  tail[n_items] = 0;
  for (int i = n_items - 1; i >= 0; --i) tail[i] = tail[i + 1] + w[i];
  // the floor uses the FIRST item as given, not the heaviest one
  const int floor_ = std::max((total + 1) / 2, item[0]);

  PairSplit best;
  int s[2] = {0, 0}, c[2] = {0, 0};
  for (int i = 0; i < n_items; ++i) {
    const int g = c[0] >= k ? 1 : c[1] >= k ? 0 : (s[0] <= s[1] ? 0 : 1);
    s[g] += w[i]; ++c[g];
    best.first[order[i]] = g == 0;
  }
  best.heavier = std::max(s[0], s[1]);
  if (best.heavier == floor_) return best;

  EqualDealSearch<2> dfs;
  dfs.n = n_items; dfs.per = k; dfs.w = w; dfs.tail = tail; dfs.where = where;
  for (int lo = floor_, hi = best.heavier - 1; lo <= hi;) {
    const int mid = (lo + hi) / 2;
    if (dfs.run(mid, 500000)) {
      best.heavier = mid;
      for (int i = 0; i < n_items; ++i) best.first[order[i]] = where[i] == 0;
      hi = mid - 1;
    } else {
      lo = mid + 1;
    }
  }
  return best;
}

PairSplit split_pair(const int* item, int n_items) {
  return n_items / 2 <= 10 ? split_pair_meet_in_middle(item, n_items) : split_pair_search(item, n_items);
}

struct TripleSplit {
  int heaviest = 0;             // limit + 1 when no split within the limit was found
  int group[kTripleMax] = {};
};

// 3k items into 3 groups of k with every sum <= limit (2M-node budget).
TripleSplit split_triple_within(const int* item, int n_items, int limit) {
  const int k = n_items / 3;
  int order[kTripleMax], w[kTripleMax], tail[kTripleMax + 1], where[kTripleMax];
  order_heaviest_first(item, n_items, order);
  int total = 0;
  for (int i = 0; i < n_items; ++i) { w[i] = item[order[i]]; total += w[i]; }
  tail[n_items] = 0;
  for (int i = n_items - 1; i >= 0; --i) tail[i] = tail[i + 1] + w[i];
  TripleSplit r;
  r.heaviest = limit + 1;
  if (limit < std::max((total + 2) / 3, w[0])) return r;
  EqualDealSearch<3> dfs;
  dfs.n = n_items; dfs.per = k; dfs.w = w; dfs.tail = tail; dfs.where = where;
  if (dfs.run(limit, 2000000)) {
    int s[3] = {0, 0, 0};
    for (int i = 0; i < n_items; ++i) { s[where[i]] += w[i]; r.group[order[i]] = where[i]; }
    r.heaviest = std::max(s[0], std::max(s[1], s[2]));
  }
  return r;
}

struct RankTable {
  int m, k;
  const int* w;
  std::vector<int> chunk;   // [m][k]
  std::vector<int> load, count;
  RankTable(int m_, int k_, const int* w_) : m(m_), k(k_), w(w_), chunk(size_t(m_) * k_), load(m_, 0), count(m_, 0) {}
  int* row(int r) { return chunk.data() + size_t(r) * k; }
  void clear(int r) { load[r] = 0; count[r] = 0; }
  void give(int r, int c) { row(r)[count[r]++] = c; load[r] += w[c]; }
  int heaviest(int* which) const {  // first rank holding the maximum
    int best = 0, at = 0;
    for (int r = 0; r < m; ++r)
      if (load[r] > best) { best = load[r]; at = r; }
    *which = at;
    return best;
  }
};

// One pass of "re-split the heaviest rank with its best partner" until no pair helps.
bool improve_by_pairs(RankTable& t, int floor_) {
  bool any = false;
  for (;;) {
    int heavy;
    const int top = t.heaviest(&heavy);
    if (top <= floor_) break;
    // largest and second largest load among the other ranks
    int o1 = 0, o1_at = -1, o2 = 0;
    for (int r = 0; r < t.m; ++r) {
      if (r == heavy) continue;
      if (t.load[r] > o1) { o2 = o1; o1 = t.load[r]; o1_at = r; }
      else if (t.load[r] > o2) o2 = t.load[r];
    }
    int partner = -1, reach = top;
    PairSplit chosen;
    int item[kPairMax];
    for (int r = 0; r < t.m; ++r) {
      if (r == heavy) continue;
      for (int i = 0; i < t.k; ++i) { item[i] = t.w[t.row(heavy)[i]]; item[t.k + i] = t.w[t.row(r)[i]]; }
      PairSplit s = split_pair(item, 2 * t.k);
      const int after = std::max(r == o1_at ? o2 : o1, s.heavier);
      if (after < reach) { reach = after; partner = r; chosen = s; }
    }
    if (partner < 0) break;
    int pool[kPairMax];
    for (int i = 0; i < t.k; ++i) { pool[i] = t.row(heavy)[i]; pool[t.k + i] = t.row(partner)[i]; }
    t.clear(heavy);
    t.clear(partner);
    for (int i = 0; i < 2 * t.k; ++i) t.give(chosen.first[i] ? heavy : partner, pool[i]);
    any = true;
  }
  return any;
}

// Re-split the heaviest rank with two partners (lightest partners first); the
// first triple that gets strictly below the current maximum is applied.
// Returns 1 when applied, 0 when nothing helped, -1 when already at the floor.
int improve_by_triples(RankTable& t, int floor_) {
  int heavy;
  const int top = t.heaviest(&heavy);
  if (top <= floor_) return -1;
  int others[kIpoMaxRanks], no = 0;
  for (int r = 0; r < t.m; ++r)
    if (r != heavy) others[no++] = r;
  std::sort(others, others + no, [&t](int a, int b) { return t.load[a] != t.load[b] ? t.load[a] < t.load[b] : a < b; });
  for (int a = 0; a < no; ++a) {
    for (int b = a + 1; b < no; ++b) {
      const int p1 = others[a], p2 = others[b];
      int rest = 0;  // heaviest rank outside the triple
      for (int q = no - 1; q >= 0; --q)
        if (q != a && q != b) { rest = t.load[others[q]]; break; }
      if (rest >= top) continue;
      int biggest = 0;
      for (int i = 0; i < t.k; ++i)
        biggest = std::max(biggest, std::max(t.w[t.row(heavy)[i]], std::max(t.w[t.row(p1)[i]], t.w[t.row(p2)[i]])));
      const int tri = t.load[heavy] + t.load[p1] + t.load[p2];
      if (std::max(rest, std::max((tri + 2) / 3, biggest)) >= top) continue;
      int item[kTripleMax], pool[kTripleMax], n3 = 0;
      const int member[3] = {heavy, p1, p2};
      for (int g = 0; g < 3; ++g)
        for (int i = 0; i < t.k; ++i) { pool[n3] = t.row(member[g])[i]; item[n3] = t.w[pool[n3]]; ++n3; }
      TripleSplit s = split_triple_within(item, n3, top - 1);
      if (std::max(rest, s.heaviest) >= top) continue;
      for (int g = 0; g < 3; ++g) t.clear(member[g]);
      for (int i = 0; i < n3; ++i) t.give(member[s.group[i]], pool[i]);
      return 1;
    }
  }
  return 0;
}

}  // namespace

extern "C" int fm_cp_partition_ipo(const int32_t* weights, int n, int n_buckets, int32_t* assign,
                                   int64_t* max_load) {
  FM_REQUIRE(weights && assign && n > 0 && n_buckets > 0, FM_ERR_INVALID_ARGUMENT, "fm_cp_partition_ipo: bad arguments");
  FM_REQUIRE(n % n_buckets == 0, FM_ERR_INVALID_ARGUMENT,
             "fm_cp_partition_ipo: the number of chunks must be a multiple of the number of buckets");
  FM_REQUIRE(n <= kIpoMaxChunks && n_buckets <= kIpoMaxRanks, FM_ERR_UNSUPPORTED,
             "fm_cp_partition_ipo: at most 512 chunks and 32 buckets (use fm_cp_partition_heap beyond)");
  for (int i = 0; i < n; ++i)
    FM_REQUIRE(weights[i] >= 0, FM_ERR_INVALID_ARGUMENT, "fm_cp_partition_ipo: negative weight");
  const int m = n_buckets, k = n / m;
  RankTable t(m, k, weights);

  std::vector<int> order(n);
  order_heaviest_first(weights, n, order.data());
  long long total = 0;
  for (int i = 0; i < n; ++i) {
    int to = -1;
    for (int r = 0; r < m; ++r)
      if (t.count[r] < k && (to < 0 || t.load[r] < t.load[to])) to = r;
    t.give(to, order[i]);
    total += weights[i];
  }
  FM_REQUIRE(total <= 0x3fffffff, FM_ERR_INVALID_ARGUMENT, "fm_cp_partition_ipo: total weight exceeds 2^30");

  if (k <= kIpoMaxPerRankOpt) {
    const int floor_ = std::max(static_cast<int>((total + m - 1) / m), weights[order[0]]);
    const int rounds = k <= 10 ? 200 : (k <= 14 ? 50 : 20);
    for (int round = 0; round < rounds; ++round) {
      bool changed = improve_by_pairs(t, floor_);
      if (m >= 3 && k <= 8) {
        const int r3 = improve_by_triples(t, floor_);
        if (r3 < 0) break;
        changed = changed || r3 > 0;
      }
      if (!changed) break;
    }
  }
  std::memcpy(assign, t.chunk.data(), sizeof(int32_t) * size_t(n));
  if (max_load) {
    int at;
    *max_load = t.heaviest(&at);
  }
  return FM_OK;
}

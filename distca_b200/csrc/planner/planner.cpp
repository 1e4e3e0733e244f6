// Linear layout, item model and the greedy balancer of the CAD planner (see planner.h).
// Behaviour follows the reference's Python planner: sequential fill with head/tail pairs
// (distca/planner/planner.py:190-271), dummy documents (:58-131), shard-length lists (:276-328), FLOPs and
// bytes-per-FLOP priority (:366-402), middle cuts (:404-495), most-starved-first rebalancing (:627-731).
#include "planner.h"

#include <algorithm>
#include <cmath>
#include <limits>
#include <numeric>
#include <stdexcept>
#include <string>

namespace dca {
namespace planner {

static inline double chunk_flops(double q, double kv) {
  // sum over the q queries of the number of keys each one sees: q*kv - q*(q-1)/2
  return q * kv - std::floor(q * (q - 1.0) / 2.0);
}

double Item::flops() const {
  double f = 0.0;
  if (head.len() > 0) f += chunk_flops(head.len(), head.b);
  if (tail.len() > 0) f += chunk_flops(tail.len(), tail.b);
  return f;
}

// Tile pairs the attention kernels visit for a chunk: query tile i (rows [i*T, min((i+1)*T, q))) sees the keys
// [0, kv - q + min((i+1)*T, q)), i.e. ceil(.../T) key tiles; the diagonal tile counts whole.
static inline double chunk_tile_pairs(int q, int kv, int T) {
  if (q <= 0) return 0.0;
  const long nq = (q + T - 1) / T;
  const long base_tiles = ((long)(kv - q) + T - 1) / T;          // ceil((kv - q) / T)
  // tiles i < nq - 1 are full: (i + 1) + ceil((kv - q) / T) key tiles each; the last one reaches kv
  const double full = (double)(nq - 1) * nq / 2.0 + (double)(nq - 1) * base_tiles;
  return full + (double)(((long)kv + T - 1) / T);
}

double CostModel::chunk_ms(int q, int kv) const {
  if (q <= 0) return 0.0;
  const double nq = (double)((q + tile - 1) / tile);
  return ms_per_tile_pair * chunk_tile_pairs(q, kv, tile) + ms_per_q_tile * nq + ms_per_task;
}

double PlannerOptions::item_cost(const Item& it) const {
  if (!cost.enabled) {
    const int chunks = (it.head.len() > 0) + (it.tail.len() > 0);
    return it.flops() + (chunks ? per_task_overhead_flops : 0.0);
  }
  return cost.chunk_ms(it.head.len(), it.head.b) + cost.chunk_ms(it.tail.len(), it.tail.b);
}

double PlannerOptions::marginal_cost(const Item& it) const {
  // one token off the head's end and one off the tail's start: doc_len + 1 query-key pairs
  if (!cost.enabled) return it.doc_len + 1.0;
  const double t = (double)cost.tile;
  return cost.ms_per_tile_pair * (it.doc_len + 1.0) / (t * t) + 2.0 * cost.ms_per_q_tile / t;
}

// ---------------------------------------------------------------------------------------------
// linear layout
// ---------------------------------------------------------------------------------------------
namespace {

struct Filler {
  long per_rank;
  int world;
  std::vector<long> budget;
  std::vector<long> used;
  int cur = 0;
  std::vector<Item> items;
  int next_doc = 0;

  Filler(long tokens_per_rank, int w) : per_rank(tokens_per_rank), world(w), budget(w, tokens_per_rank), used(w, 0) {}

  void place_document(int len) {
    const int doc = next_doc++;
    long remaining = len;
    int prefix = 0;        // tokens already placed from the front
    int suffix_end = len;  // end of what is left at the back
    while (remaining > 0) {
      while (cur < world && budget[cur] == 0) ++cur;
      if (cur >= world) {
        long total = 0;
        for (long b : budget) total += b;
        throw std::runtime_error("documents do not fit the linear layout: document " + std::to_string(doc) +
                                 " of " + std::to_string(len) + " tokens has " + std::to_string(remaining) +
                                 " left, " + std::to_string(world) + " ranks x " + std::to_string(per_rank) +
                                 " tokens, free " + std::to_string(total));
      }
      const long chunk = std::min(remaining, budget[cur]);
      Item it;
      it.doc = doc;
      it.doc_len = len;
      it.src = it.dst = cur;
      it.head_row0 = (int)used[cur];
      if (remaining == len && chunk == len) {
        it.head = {0, len};
        it.tail = {len, len};
        it.tail_row0 = it.head_row0 + len;
      } else {
        const int qh = (int)(chunk / 2);
        const int qt = (int)(chunk - qh);
        it.head = {prefix, prefix + qh};
        it.tail = {suffix_end - qt, suffix_end};
        it.tail_row0 = it.head_row0 + qh;
        prefix += qh;
        suffix_end -= qt;
      }
      items.push_back(it);
      budget[cur] -= chunk;
      used[cur] += chunk;
      remaining -= chunk;
    }
  }

  void place_dummy(int len) {
    // a lone short document owns the next rank that is still empty
    while (cur < world && used[cur] != 0) ++cur;
    if (cur >= world) throw std::runtime_error("no empty rank left for a dummy document");
    const int doc = next_doc++;
    Item it;
    it.doc = doc;
    it.doc_len = len;
    it.src = it.dst = cur;
    it.head = {0, len};
    it.tail = {len, len};
    it.head_row0 = 0;
    it.tail_row0 = len;
    items.push_back(it);
    used[cur] = len;
    budget[cur] = 0;
    ++cur;
  }
};

}  // namespace

std::vector<Item> batch_to_items(const std::vector<std::vector<int>>& batches, long tokens_per_rank, int world) {
  Filler f(tokens_per_rank, world);
  for (const auto& b : batches)
    for (int len : b)
      if (len > 0) f.place_document(len);
  return f.items;
}

std::vector<Item> batch_to_items_with_dummy(const std::vector<std::vector<int>>& batches, long tokens_per_rank,
                                            int world) {
  Filler f(tokens_per_rank, world);
  for (const auto& b : batches) {
    if (b.size() == 1 && b[0] > 0 && b[0] < tokens_per_rank) {
      // make sure a partially filled rank is closed before the dummy takes the next empty one
      if (f.cur < world && f.used[f.cur] != 0 && f.budget[f.cur] != 0) {
        f.budget[f.cur] = 0;
      }
      f.place_dummy(b[0]);
    } else {
      for (int len : b)
        if (len > 0) f.place_document(len);
    }
  }
  return f.items;
}

std::vector<Item> items_fixed_layout(const std::vector<std::vector<int>>& docs_per_rank) {
  std::vector<Item> items;
  int doc = 0;
  for (size_t r = 0; r < docs_per_rank.size(); ++r) {
    int row = 0;
    for (int len : docs_per_rank[r]) {
      if (len <= 0) continue;
      Item it;
      it.doc = doc++;
      it.doc_len = len;
      it.src = it.dst = (int)r;
      it.head = {0, len};
      it.tail = {len, len};
      it.head_row0 = row;
      it.tail_row0 = row + len;
      row += len;
      items.push_back(it);
    }
  }
  return items;
}

std::vector<std::vector<int>> cp_list_to_mlp_list(const std::vector<std::vector<int>>& cp_list, int world,
                                                  long tokens_per_rank) {
  std::vector<std::vector<int>> out(world);
  std::vector<Item> items;
  try {
    items = batch_to_items(cp_list, tokens_per_rank, world);
  } catch (const std::runtime_error&) {
    // more tokens than capacity: lay out what fits (extra documents are dropped)
    Filler f(tokens_per_rank, world);
    for (const auto& b : cp_list)
      for (int len : b) {
        long free_total = 0;
        for (long x : f.budget) free_total += x;
        if (len > 0 && len <= free_total) f.place_document(len);
      }
    items = f.items;
  }
  for (const auto& it : items) {
    if (it.whole()) {
      out[it.src].push_back(it.head.len());
    } else {
      out[it.src].push_back(it.head.len());
      out[it.src].push_back(it.tail.len());
    }
  }
  return out;
}

// ---------------------------------------------------------------------------------------------
// balancing
// ---------------------------------------------------------------------------------------------
namespace {

// Cut `m` tokens off the end of the head and the start of the tail of `it` (in place) and return
// them as a new item on server `dst`.
Item cut_middle(Item& it, int m, int dst) {
  if (it.whole()) {
    const int L = it.head.len();
    const int qh = (L + 1) / 2;
    const int a = it.head.a;
    it.tail = {a + qh, a + L};
    it.tail_row0 = it.head_row0 + qh;
    it.head = {a, a + qh};
  }
  Item moved = it;
  moved.dst = dst;
  moved.head = {it.head.b - m, it.head.b};
  moved.head_row0 = it.head_row0 + (it.head.len() - m);
  moved.tail = {it.tail.a, it.tail.a + m};
  moved.tail_row0 = it.tail_row0;
  it.head.b -= m;
  it.tail.a += m;
  it.tail_row0 += m;
  return moved;
}

}  // namespace

// Baseline placement without balancing decisions: every document of at least `min_len` tokens is
// cut into 2 * world equal chunks and server k gets chunk k from the front and chunk k from the
// back (the head-tail pairing that equalises causal work), like per-document context parallelism
// with an all-gather of K/V; shorter documents stay with their owner.
std::vector<Item> per_document_cp(const std::vector<Item>& layout, int world, int min_len) {
  std::vector<Item> out;
  for (const Item& src_item : layout) {
    if (world <= 1 || !src_item.whole() || src_item.doc_len < min_len || src_item.head.len() < 2 * world) {
      out.push_back(src_item);
      continue;
    }
    Item rest = src_item;
    const int m = rest.head.len() / (2 * world);
    for (int k = world - 1; k >= 1; --k) out.push_back(cut_middle(rest, m, (src_item.src + k) % world));
    out.push_back(rest);   // outermost head and tail chunk stay on the owner
  }
  return out;
}

// Legacy policy ("water filling"): only the single most expensive document is cut; its middle is
// handed out to the other servers, each getting what it lacks to reach the mean, the outermost part
// stays with the owner. Cheap to compute and enough when one document dominates the batch; with
// several long documents the general balancer below does better.
std::vector<Item> water_fill(const std::vector<Item>& layout, const PlannerOptions& opt) {
  std::vector<Item> items = layout;
  const int W = opt.world;
  if (items.empty() || W <= 1) return items;
  size_t big = 0;
  for (size_t i = 1; i < items.size(); ++i)
    if (items[i].flops() > items[big].flops()) big = i;
  std::vector<double> load(W, 0.0);
  double total = 0.0;
  for (size_t i = 0; i < items.size(); ++i) {
    total += items[i].flops();
    if (i != big) load[items[i].dst] += items[i].flops();
  }
  const double mean = total / W;
  std::vector<int> order;
  for (int r = 0; r < W; ++r)
    if (r != items[big].dst) order.push_back(r);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return load[a] < load[b]; });
  for (int r : order) {
    const double lack = mean - load[r];
    if (lack <= 0) continue;
    Item& it = items[big];
    // never give away so much that the owner itself falls below the mean
    const double spare = it.flops() + load[it.dst] - mean;
    const double give = std::min(lack, spare);
    if (give <= 0) break;
    const int limit = it.whole() ? it.head.len() / 2 : std::min(it.head.len(), it.tail.len());
    int m = (int)(give / (it.doc_len + 1.0));
    if (m > limit) m = limit;
    if (m <= 0) continue;
    const Item piece = cut_middle(it, m, r);
    load[r] += piece.flops();
    items.push_back(piece);  // invalidates `it`
  }
  std::vector<Item> out;
  for (const auto& it : items)
    if (it.head.len() + it.tail.len() > 0) out.push_back(it);
  return out;
}

std::vector<Item> balance(const std::vector<Item>& items_in, const PlannerOptions& opt) {
  std::vector<Item> items = items_in;
  const int W = opt.world;
  // Everything below is in the units of opt.item_cost(): predicted milliseconds with the cost model,
  // query-key pairs without it.
  std::vector<double> load(W, 0.0);
  std::vector<double> item_flops(items.size());
  for (size_t i = 0; i < items.size(); ++i) {
    item_flops[i] = opt.item_cost(items[i]);
    load[items[i].dst] += item_flops[i];
  }
  const double total = std::accumulate(load.begin(), load.end(), 0.0);
  const double avg = total / W;
  const double threshold = avg * opt.tolerance;
  // every server's target: an equal share, or a share in proportion to its measured speed
  std::vector<double> target(W, avg);
  if ((int)opt.speed.size() == W) {
    double ssum = 0.0;
    for (double v : opt.speed) ssum += v > 0 ? v : 0.0;
    if (ssum > 0)
      for (int r = 0; r < W; ++r) target[r] = total * (opt.speed[r] > 0 ? opt.speed[r] : 0.0) / ssum;
  }
  std::vector<double> surplus(W);
  for (int r = 0; r < W; ++r) surplus[r] = load[r] - target[r];

  std::vector<int> recipients;
  for (int r = 0; r < W; ++r)
    if (surplus[r] < 0) recipients.push_back(r);
  std::stable_sort(recipients.begin(), recipients.end(), [&](int a, int b) { return surplus[a] < surplus[b]; });

  // One transfer of at most `need` cost units to `rcv`, taken from the cheapest (bytes per unit of cost)
  // item among the servers `donor_ok` admits. Returns the cost moved (0 = nothing movable).
  auto transfer = [&](int rcv, double need, auto donor_ok) -> double {
    int best = -1;
    double best_prio = std::numeric_limits<double>::infinity();
    double best_max = 0.0;
    for (size_t i = 0; i < items.size(); ++i) {
      const Item& it = items[i];
      const int d = it.dst;
      if (d == rcv || surplus[d] <= 0 || item_flops[i] <= 0 || !donor_ok(d)) continue;
      const double movable = std::min({surplus[d], need, item_flops[i]});
      if (movable <= 0) continue;
      const double q_tokens = movable / opt.marginal_cost(it);
      const double bytes = q_tokens * opt.dims.q_row_bytes + 2.0 * (it.doc_len + 1.0) * opt.dims.kv_row_bytes;
      const double prio = bytes / movable;
      if (prio < best_prio) {
        best_prio = prio;
        best = (int)i;
        best_max = movable;
      }
    }
    if (best < 0) return 0.0;
    const int donor = items[best].dst;
    if (best_max >= item_flops[best]) {
      const double moved = item_flops[best];
      items[best].dst = rcv;
      surplus[donor] -= moved;
      surplus[rcv] += moved;
      return moved;
    }
    Item& it = items[best];
    const int limit = it.whole() ? it.head.len() / 2 : std::min(it.head.len(), it.tail.len());
    int m = (int)(best_max / opt.marginal_cost(it));
    if (opt.cost.enabled && m > opt.cost.tile) m = m / opt.cost.tile * opt.cost.tile;   // cut on tile boundaries
    if (m > limit) m = limit;
    if (m <= 0) return 0.0;
    const double before = item_flops[best];
    const Item piece = cut_middle(it, m, rcv);
    const double after = opt.item_cost(it);
    const double gained = opt.item_cost(piece);
    item_flops[best] = after;
    surplus[donor] -= (before - after);
    surplus[rcv] += gained;
    items.push_back(piece);  // invalidates `it`
    item_flops.push_back(gained);
    return gained;
  };

  // Phase 1: feed every under-loaded server, most starved first, until it is within the tolerance.
  for (int rcv : recipients) {
    double need = -surplus[rcv];
    while (need > threshold) {
      const double moved = transfer(rcv, need, [](int) { return true; });
      if (moved <= 0) break;
      need -= moved;
    }
  }
  // Phase 2: phase 1 stops when the receivers are satisfied, which can leave one donor well above the
  // mean while several receivers each sit a little below it. Drain the most loaded server into the
  // least loaded one until no server is more than the tolerance above the mean.
  for (int guard = 0; guard < 8 * W; ++guard) {
    const int d = (int)(std::max_element(surplus.begin(), surplus.end()) - surplus.begin());
    const int r = (int)(std::min_element(surplus.begin(), surplus.end()) - surplus.begin());
    if (surplus[d] <= threshold || surplus[r] >= 0 || d == r) break;
    const double want = std::min(surplus[d], -surplus[r]);
    if (transfer(r, want, [d](int x) { return x == d; }) <= 0) break;
  }
  std::vector<Item> out;
  out.reserve(items.size());
  for (const auto& it : items)
    if (it.head.len() + it.tail.len() > 0) out.push_back(it);
  return out;
}

// ---------------------------------------------------------------------------------------------
// time model
// ---------------------------------------------------------------------------------------------
double TimeModel::attn_ms_for(double q, double kv) const {
  if (attn_len.empty()) return chunk_flops(q, kv) * 1e-9;
  // cost of a whole causal document of length L, interpolated linearly in L^2, extrapolated
  // quadratically; a chunk (q, kv) costs whole(kv) - whole(kv - q).
  auto whole = [&](double L) -> double {
    if (L <= 0) return 0.0;
    const size_t n = attn_len.size();
    const double x = L * L;
    if (L <= attn_len.front()) return attn_ms.front() * x / (attn_len.front() * attn_len.front());
    if (L >= attn_len.back()) return attn_ms.back() * x / (attn_len.back() * attn_len.back());
    size_t hi = 1;
    while (hi < n && attn_len[hi] < L) ++hi;
    const double x0 = attn_len[hi - 1] * attn_len[hi - 1], x1 = attn_len[hi] * attn_len[hi];
    const double t = (x - x0) / (x1 - x0);
    return attn_ms[hi - 1] + t * (attn_ms[hi] - attn_ms[hi - 1]);
  };
  return whole(kv) - whole(kv - q);
}

}  // namespace planner
}  // namespace dca

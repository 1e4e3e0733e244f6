// Stage 3 of the CAD planner: turn balanced items into the tables the runtime executes
// (see planner.h). Also the reference-style all-to-all byte matrices and the step simulator.
#include <algorithm>
#include <cmath>
#include <limits>
#include <map>
#include <numeric>
#include <stdexcept>

#include "planner.h"

namespace dca {
namespace planner {

namespace {

struct Chunk {
  int doc, a, b;       // query token range of the document
  int owner, owner_row0;
};

double max_over_mean(const std::vector<double>& v) {
  if (v.empty()) return 1.0;
  const double mx = *std::max_element(v.begin(), v.end());
  const double mean = std::accumulate(v.begin(), v.end(), 0.0) / v.size();
  return mean > 0 ? mx / mean : 1.0;
}

}  // namespace

Plan compile_plan(const std::vector<Item>& layout_items, const std::vector<Item>& balanced,
                  const PlannerOptions& opt) {
  const int W = opt.world;
  Plan plan;
  plan.world = W;
  plan.tolerance_used = opt.tolerance;
  plan.items = balanced;
  plan.ranks.resize(W);
  plan.flops_before.assign(W, 0.0);
  plan.flops_after.assign(W, 0.0);
  plan.cost_after.assign(W, 0.0);
  for (const auto& it : layout_items) plan.flops_before[it.dst] += it.flops();

  // ---- owner side: local layout (rows -> document ranges) ----
  for (const auto& it : layout_items) {
    RankPlan& rp = plan.ranks[it.src];
    if (it.head.len() > 0) rp.layout.push_back({it.doc, it.head.a, it.head.b, it.head_row0});
    if (it.tail.len() > 0) rp.layout.push_back({it.doc, it.tail.a, it.tail.b, it.tail_row0});
  }
  for (auto& rp : plan.ranks) {
    std::sort(rp.layout.begin(), rp.layout.end(), [](const Segment& x, const Segment& y) { return x.row0 < y.row0; });
    long n = 0;
    for (const auto& s : rp.layout) n = std::max<long>(n, s.row0 + (s.b - s.a));
    rp.num_tokens = n;
    rp.q_dst_rank.assign(n, -1);
    rp.q_dst_row.assign(n, -1);
    rp.send_bytes.assign(W, 0);
  }

  // ---- server side: chunks grouped by document, ordered by position ----
  std::vector<std::vector<Chunk>> per_server(W);
  for (const auto& it : balanced) {
    plan.flops_after[it.dst] += it.flops();
    plan.cost_after[it.dst] += opt.item_cost(it);
    if (it.head.len() > 0) per_server[it.dst].push_back({it.doc, it.head.a, it.head.b, it.src, it.head_row0});
    if (it.tail.len() > 0) per_server[it.dst].push_back({it.doc, it.tail.a, it.tail.b, it.src, it.tail_row0});
  }
  // context of (server, doc): keys [0, ctx_len)
  std::vector<std::map<int, std::pair<int, int>>> ctx(W);  // doc -> (k_row0, ctx_len)
  for (int s = 0; s < W; ++s) {
    auto& chunks = per_server[s];
    std::sort(chunks.begin(), chunks.end(), [](const Chunk& x, const Chunk& y) {
      return x.doc != y.doc ? x.doc < y.doc : x.a < y.a;
    });
    // merge chunks that are adjacent both in the document and in the owner's buffer
    std::vector<Chunk> merged;
    for (const auto& c : chunks) {
      if (!merged.empty()) {
        Chunk& m = merged.back();
        if (m.doc == c.doc && m.b == c.a && m.owner == c.owner && m.owner_row0 + (m.b - m.a) == c.owner_row0) {
          m.b = c.b;
          continue;
        }
      }
      merged.push_back(c);
    }
    chunks.swap(merged);
    RankPlan& rp = plan.ranks[s];
    long qrow = 0, krow = 0;
    for (const auto& c : chunks) {
      auto& e = ctx[s][c.doc];
      e.second = std::max(e.second, c.b);
    }
    for (auto& kv : ctx[s]) {
      kv.second.first = (int)krow;
      krow += kv.second.second;
    }
    for (const auto& c : chunks) {
      Task t;
      t.doc = c.doc;
      t.q_a = c.a;
      t.q_b = c.b;
      t.q_row0 = (int)qrow;
      t.k_row0 = ctx[s][c.doc].first;
      t.kv_len = c.b;
      t.owner = c.owner;
      t.owner_row0 = c.owner_row0;
      rp.tasks.push_back(t);
      RankPlan& own = plan.ranks[c.owner];
      for (int i = 0; i < c.b - c.a; ++i) {
        own.q_dst_rank[c.owner_row0 + i] = s;
        own.q_dst_row[c.owner_row0 + i] = (int)qrow + i;
      }
      own.send_bytes[s] += (int64_t)(c.b - c.a) * opt.dims.q_row_bytes;
      qrow += c.b - c.a;
    }
    rp.q_rows = qrow;
    rp.kv_rows = krow;
    rp.flops = plan.flops_after[s];
    if ((opt.max_q_rows > 0 && qrow > opt.max_q_rows) || (opt.max_kv_rows > 0 && krow > opt.max_kv_rows))
      plan.fits = false;
  }

  // ---- K/V fan-out: every owner segment goes to every server whose context of that document reaches it ----
  std::vector<std::vector<std::vector<std::pair<int, int>>>> copies(W);  // [owner][row] -> (server, k_row)
  for (int r = 0; r < W; ++r) copies[r].resize(plan.ranks[r].num_tokens);
  for (int r = 0; r < W; ++r) {
    for (const auto& seg : plan.ranks[r].layout) {
      for (int s = 0; s < W; ++s) {
        auto f = ctx[s].find(seg.doc);
        if (f == ctx[s].end()) continue;
        const int k_row0 = f->second.first, ctx_len = f->second.second;
        const int end = std::min(seg.b, ctx_len);
        if (end <= seg.a) continue;
        for (int t = seg.a; t < end; ++t)
          copies[r][seg.row0 + (t - seg.a)].push_back({s, k_row0 + t});
        plan.ranks[r].send_bytes[s] += (int64_t)(end - seg.a) * 2 * opt.dims.kv_row_bytes;
      }
    }
  }
  for (int r = 0; r < W; ++r) {
    RankPlan& rp = plan.ranks[r];
    size_t mc = 0;
    for (const auto& c : copies[r]) mc = std::max(mc, c.size());
    rp.max_copies = (int)mc;
  }
  // one common slot count keeps the owner-side gradient buffers the same shape everywhere
  int global_copies = 1;
  for (const auto& rp : plan.ranks) global_copies = std::max(global_copies, rp.max_copies);
  for (int r = 0; r < W; ++r) {
    RankPlan& rp = plan.ranks[r];
    rp.max_copies = global_copies;
    rp.kv_dst_rank.assign((size_t)rp.num_tokens * global_copies, -1);
    rp.kv_dst_row.assign((size_t)rp.num_tokens * global_copies, -1);
    for (long t = 0; t < rp.num_tokens; ++t)
      for (size_t c = 0; c < copies[r][t].size(); ++c) {
        rp.kv_dst_rank[t * global_copies + c] = copies[r][t][c].first;
        rp.kv_dst_row[t * global_copies + c] = copies[r][t][c].second;
      }
  }
  // ---- context segments on each server: which owner rows (and which of its slots) a run came from ----
  for (int r = 0; r < W; ++r) {
    for (const auto& seg : plan.ranks[r].layout) {
      const int n = seg.b - seg.a;
      int i = 0;
      while (i < n) {
        // runs with the same copy list structure: walk per slot
        const auto& cl = copies[r][seg.row0 + i];
        int j = i + 1;
        while (j < n && copies[r][seg.row0 + j].size() == cl.size()) {
          bool same = true;
          for (size_t c = 0; c < cl.size(); ++c)
            if (copies[r][seg.row0 + j][c].first != cl[c].first) { same = false; break; }
          if (!same) break;
          ++j;
        }
        for (size_t c = 0; c < cl.size(); ++c) {
          ContextSegment cs;
          cs.k_row0 = cl[c].second;
          cs.n = j - i;
          cs.owner = r;
          cs.owner_row0 = seg.row0 + i;
          cs.slot = (int)c;
          plan.ranks[cl[c].first].ctx_segments.push_back(cs);
        }
        i = j;
      }
    }
  }
  plan.imbalance_before = max_over_mean(plan.flops_before);
  plan.imbalance_after = max_over_mean(plan.flops_after);
  {
    // cost of every server against ITS share of the total (equal shares unless speeds are given)
    double total = 0.0, ssum = 0.0;
    for (double c : plan.cost_after) total += c;
    const bool weighted = (int)opt.speed.size() == W;
    for (int r = 0; r < W; ++r) ssum += weighted ? std::max(opt.speed[r], 0.0) : 1.0;
    double worst = 0.0;
    for (int r = 0; r < W; ++r) {
      const double share = total * (weighted ? std::max(opt.speed[r], 0.0) : 1.0) / (ssum > 0 ? ssum : 1.0);
      if (share > 0) worst = std::max(worst, plan.cost_after[r] / share);
    }
    plan.cost_imbalance_after = total > 0 ? worst : 1.0;
  }
  return plan;
}

static Plan plan_from_layout(const std::vector<Item>& layout, const PlannerOptions& opt_in);

Plan plan_batch(const std::vector<std::vector<int>>& batches, const PlannerOptions& opt_in, bool with_dummy) {
  const std::vector<Item> layout = with_dummy
                                       ? batch_to_items_with_dummy(batches, opt_in.tokens_per_rank, opt_in.world)
                                       : batch_to_items(batches, opt_in.tokens_per_rank, opt_in.world);
  return plan_from_layout(layout, opt_in);
}

Plan plan_fixed(const std::vector<std::vector<int>>& docs_per_rank, const PlannerOptions& opt_in) {
  if ((int)docs_per_rank.size() != opt_in.world)
    throw std::runtime_error("plan_fixed: one document list per rank is required");
  return plan_from_layout(items_fixed_layout(docs_per_rank), opt_in);
}

Plan plan_fixed_cp(const std::vector<std::vector<int>>& docs_per_rank, const PlannerOptions& opt, int min_len) {
  if ((int)docs_per_rank.size() != opt.world)
    throw std::runtime_error("plan_fixed_cp: one document list per rank is required");
  const std::vector<Item> layout = items_fixed_layout(docs_per_rank);
  Plan plan = compile_plan(layout, per_document_cp(layout, opt.world, min_len), opt);
  plan.tolerance_used = -1.0;   // no balancer involved
  return plan;
}

Plan plan_fixed_water_fill(const std::vector<std::vector<int>>& docs_per_rank, const PlannerOptions& opt) {
  if ((int)docs_per_rank.size() != opt.world)
    throw std::runtime_error("plan_fixed_water_fill: one document list per rank is required");
  const std::vector<Item> layout = items_fixed_layout(docs_per_rank);
  Plan plan = compile_plan(layout, water_fill(layout, opt), opt);
  plan.tolerance_used = -2.0;   // no tolerance involved
  return plan;
}

static Plan plan_from_layout(const std::vector<Item>& layout, const PlannerOptions& opt_in) {
  PlannerOptions opt = opt_in;
  // tolerance ladder: the requested value first, then looser and looser until the arena fits
  std::vector<double> ladder = {opt_in.tolerance};
  for (double t : {0.05, 0.1, 0.15, 0.2, 0.3, 0.4, 0.5, 0.6, 0.7, 0.8, 0.9, 1.0})
    if (t > opt_in.tolerance) ladder.push_back(t);
  Plan last;
  for (double tol : ladder) {
    opt.tolerance = tol;
    last = compile_plan(layout, balance(layout, opt), opt);
    if (last.fits) return last;
  }
  // nothing moved at all (every rank serves itself); reports fits=false if even that overflows
  last = compile_plan(layout, layout, opt);
  last.tolerance_used = std::numeric_limits<double>::infinity();
  return last;
}

// ---------------------------------------------------------------------------------------------
Fa2aMatrices fa2a_matrices(const Plan& plan, const ModelDims& dims) {
  const int W = plan.world;
  Fa2aMatrices m;
  m.world = W;
  m.send_disp.assign((size_t)W * W, 0);
  m.transfer_sz.assign((size_t)W * W, 0);
  m.recv_disp.assign((size_t)W * W, 0);
  m.recv_transfer_sz.assign((size_t)W * W, 0);
  for (int i = 0; i < W; ++i)
    for (int j = 0; j < W; ++j) m.transfer_sz[(size_t)i * W + j] = (uint64_t)plan.ranks[i].send_bytes[j];
  for (int i = 0; i < W; ++i) {
    uint64_t acc = 0;
    for (int j = 0; j < W; ++j) {
      m.send_disp[(size_t)i * W + j] = acc;
      acc += m.transfer_sz[(size_t)i * W + j];
    }
    m.max_send = std::max(m.max_send, acc);
  }
  for (int j = 0; j < W; ++j) {
    uint64_t acc = 0;
    for (int i = 0; i < W; ++i) {
      m.recv_disp[(size_t)i * W + j] = acc;
      acc += m.transfer_sz[(size_t)i * W + j];
      m.recv_transfer_sz[(size_t)j * W + i] = m.transfer_sz[(size_t)i * W + j];
    }
    m.max_recv = std::max(m.max_recv, acc);
  }
  (void)dims;
  return m;
}

SimResult simulate(const Plan& plan, const TimeModel& tm, const ModelDims& dims) {
  const int W = plan.world;
  SimResult r;
  r.attn_ms.assign(W, 0.0);
  r.linear_ms.assign(W, 0.0);
  r.comm_ms.assign(W, 0.0);
  for (int s = 0; s < W; ++s) {
    for (const auto& t : plan.ranks[s].tasks) r.attn_ms[s] += tm.attn_ms_for(t.q_b - t.q_a, t.kv_len);
    r.linear_ms[s] = tm.linear_ms_per_token * plan.ranks[s].num_tokens;
    int64_t out = 0, in = 0;
    for (int j = 0; j < W; ++j) {
      if (j != s) out += plan.ranks[s].send_bytes[j];
      if (j != s) in += plan.ranks[j].send_bytes[s];
    }
    r.comm_ms[s] = (double)std::max(out, in) / (tm.link_gbytes_per_s * 1e6);
  }
  (void)dims;
  double worst = 0.0;
  for (int s = 0; s < W; ++s) worst = std::max(worst, r.attn_ms[s] + r.linear_ms[s]);
  r.step_ms = worst;
  r.imbalance = max_over_mean(r.attn_ms);
  return r;
}

}  // namespace planner
}  // namespace dca

// Host-side core-attention-disaggregation (CAD) planner.
//
// Input: the documents of one (micro-)batch. Output: which rank runs core attention for which
// token range of which document, balanced by attention cost, plus every table the runtime needs
// to move Q/K/V rows to the attention servers and results back.
//
// Concepts
//   * linear layout : ranks are filled with tokens in order; a document that does not fit is cut
//     and every cut piece is stored as a (head, tail) pair taken symmetrically from the front and
//     the back of what is left of the document, so each piece has a balanced causal workload.
//   * item          : a head/tail pair (or a whole document) with an owner rank (where the tokens
//     live) and a server rank (where its core attention runs).
//   * balancing     : most-starved server first, take work from over-loaded servers, cheapest
//     bytes-per-FLOP item first, cutting items from the middle (end of head + start of tail) so the
//     moved part is again a balanced pair.
//   * context       : on a server, the K/V rows [0, ctx_len) of one document, stored once and shared
//     by all query shards of that document on that server.
//
// The behaviour follows the reference planner (distca/planner/planner.py:58-328, 366-495, 627-801)
// and metadata compiler (distca/runtime/compute_metadata.py:368-734); the data layout is this
// repository's own (direct peer stores to row addresses instead of per-peer byte segments).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace dca {
namespace planner {

struct Range {
  int a = 0, b = 0;  // [a, b) in document token coordinates
  int len() const { return b - a; }
};

// A contiguous run of one document's tokens in a rank's local token buffer.
struct Segment {
  int doc;
  int a, b;   // token range of the document
  int row0;   // first local row
};

struct Item {
  int doc = 0;
  int doc_len = 0;
  int src = 0;       // owner of the tokens
  int dst = 0;       // attention server
  Range head, tail;  // tail.len() == 0 for an uncut document held as one range
  int head_row0 = 0; // local row of head.a on `src`
  int tail_row0 = 0; // local row of tail.a on `src`
  bool whole() const { return tail.len() == 0; }
  double flops() const;
};

struct ModelDims {
  int q_row_bytes = 8192;    // bytes of one token's Q row on one tensor-parallel rank
  int kv_row_bytes = 2048;   // bytes of one token's K row (V is the same)
};

// Profiled cost of core attention (forward + backward) in milliseconds, tile-granular like the kernels:
// a chunk of q queries whose last one sees kv keys costs
//     ms_per_tile_pair * (128 x 128 query-key tile pairs the kernels visit, diagonal tiles counted whole)
//   + ms_per_q_tile    * (128-row query tiles: pipeline fill, statistics, epilogue per tile)
//   + ms_per_task      (once per chunk).
// The constants come from the attention micro-benchmarks of this repository's kernels (see
// distca_b200/planner/__init__.py::default_cost_model). With `enabled` false the balancer counts query-key
// pairs, as the reference does (distca/planner/planner.py:366-378); its time model is a table over document
// lengths used by its simulator only (distca/timemodule/compute.py:75-118).
struct CostModel {
  bool enabled = false;
  int tile = 128;
  double ms_per_tile_pair = 0.0;
  double ms_per_q_tile = 0.0;
  double ms_per_task = 0.0;
  double chunk_ms(int q, int kv) const;
};

struct PlannerOptions {
  int world = 1;                 // attention-server ranks
  long tokens_per_rank = 0;      // capacity of the linear layout
  double tolerance = 0.1;        // stop feeding a server once it is within avg * tolerance
  ModelDims dims;
  long max_q_rows = 0;           // arena capacity per server in rows (0 = unlimited)
  long max_kv_rows = 0;
  double per_task_overhead_flops = 0.0;  // fixed cost charged per chunk when balancing by query-key pairs
  CostModel cost;                        // balance predicted milliseconds instead of query-key pairs
  // Relative speed of every server (empty = all equal): server r is given the share speed[r] / sum(speed) of
  // the work. The runtime feeds back measured / predicted attention time here (GPUs under a power cap do
  // not all run at the same clock).
  std::vector<double> speed;
  // cost of an item under these options: milliseconds (cost model) or query-key pairs
  double item_cost(const Item& it) const;
  // cost of moving one more token from the end of the head AND the start of the tail of `it`
  double marginal_cost(const Item& it) const;
};

// One core-attention task on a server (rows are in the server's receive arena).
struct Task {
  int doc;
  int q_a, q_b;        // query token range of the document
  int q_row0;          // first row in the server's Q region
  int k_row0;          // first row of the document context in the server's K/V region
  int kv_len;          // keys visible to the last query = q_b
  int owner;           // rank that owns the query tokens
  int owner_row0;      // their first row in the owner's local token buffer
};

// A run of context rows on a server that came from one owner (used to return dK/dV).
struct ContextSegment {
  int k_row0;          // first row in the server's K/V region
  int n;               // rows
  int owner;
  int owner_row0;      // first row in the owner's local buffer
  int slot;            // which of the owner's copy slots this server writes
};

struct RankPlan {
  // ---- as owner of tokens (tables have one entry per local token) ----
  long num_tokens = 0;
  std::vector<Segment> layout;          // local rows -> document ranges (for positions / labels)
  std::vector<int32_t> q_dst_rank, q_dst_row;      // [T]
  int max_copies = 0;
  std::vector<int32_t> kv_dst_rank, kv_dst_row;    // [T * max_copies], -1 = unused
  // ---- as attention server ----
  std::vector<Task> tasks;
  std::vector<ContextSegment> ctx_segments;
  long q_rows = 0, kv_rows = 0;         // arena rows in use
  double flops = 0.0;                   // planned attention cost
  // ---- traffic (bytes this rank sends to each peer in the forward dispatch) ----
  std::vector<int64_t> send_bytes;      // [world]
};

struct Plan {
  int world = 0;
  double tolerance_used = 0.0;
  std::vector<Item> items;              // after balancing
  std::vector<RankPlan> ranks;
  std::vector<double> flops_before, flops_after;
  double imbalance_before = 0.0, imbalance_after = 0.0;  // max / mean of query-key pairs
  std::vector<double> cost_after;       // what the balancer balanced: predicted ms (cost model) or pairs, per server
  double cost_imbalance_after = 0.0;    // max over servers of cost / (that server's share of the total)
  bool fits = true;                     // arena capacity respected
};

// ---- stage 1: linear layout ----
// Sequential fill of `world` ranks with `tokens_per_rank` tokens each. Throws std::runtime_error when
// the documents do not fit.
std::vector<Item> batch_to_items(const std::vector<std::vector<int>>& batches, long tokens_per_rank,
                                 int world);
// Same, but a batch that is a single document shorter than the rank budget is pinned alone on the
// next empty rank (pipeline stages that run a dummy forward).
std::vector<Item> batch_to_items_with_dummy(const std::vector<std::vector<int>>& batches,
                                            long tokens_per_rank, int world);
// Documents that are already placed: rank r owns exactly docs_per_rank[r], whole, in order (a rank
// may own nothing, e.g. a pipeline stage in a bubble that only serves attention).
std::vector<Item> items_fixed_layout(const std::vector<std::vector<int>>& docs_per_rank);
// documents per sequence -> shard lengths per rank (head and tail of a cut piece count separately)
std::vector<std::vector<int>> cp_list_to_mlp_list(const std::vector<std::vector<int>>& cp_list,
                                                  int world, long tokens_per_rank);

// ---- stage 2: balancing ----
std::vector<Item> balance(const std::vector<Item>& items, const PlannerOptions& opt);

// Legacy policy: cut only the most expensive document and fill the other servers up to the mean.
std::vector<Item> water_fill(const std::vector<Item>& layout, const PlannerOptions& opt);
// Baseline: per-document context parallelism (no balancing, see planner.cpp).
std::vector<Item> per_document_cp(const std::vector<Item>& layout, int world, int min_len);

// ---- stage 3: tables ----
Plan compile_plan(const std::vector<Item>& layout_items, const std::vector<Item>& balanced,
                  const PlannerOptions& opt);

// All stages; raises the tolerance (0.05 ... 1.0, then "no move") until the plan fits the arena.
Plan plan_batch(const std::vector<std::vector<int>>& batches, const PlannerOptions& opt,
                bool with_dummy = false);
// Same with the fixed per-rank placement of items_fixed_layout().
Plan plan_fixed(const std::vector<std::vector<int>>& docs_per_rank, const PlannerOptions& opt);
// Fixed placement with the per-document context-parallel baseline instead of the balancer.
Plan plan_fixed_cp(const std::vector<std::vector<int>>& docs_per_rank, const PlannerOptions& opt, int min_len);
// Fixed placement with the legacy water-filling policy.
Plan plan_fixed_water_fill(const std::vector<std::vector<int>>& docs_per_rank, const PlannerOptions& opt);

// ---- reference-style all-to-all matrices (for the fa2a micro-benchmark and compatibility) ----
// send_disp[i][j], transfer_sz[i][j], recv_disp[i][j] in bytes, row-major [world, world]:
// rank i's segment for rank j is [Q rows | K rows | V rows].
struct Fa2aMatrices {
  int world = 0;
  std::vector<uint64_t> send_disp, transfer_sz, recv_disp, recv_transfer_sz;
  uint64_t max_send = 0, max_recv = 0;
};
Fa2aMatrices fa2a_matrices(const Plan& plan, const ModelDims& dims);

// ---- time model + simulator ----
struct TimeModel {
  // attention: piecewise-linear in kv_len^2-space table of (L, ms for a whole causal document of L)
  std::vector<double> attn_len, attn_ms;
  double linear_ms_per_token = 0.0;    // everything that is not core attention, per token per layer
  double link_gbytes_per_s = 770.0;
  double attn_ms_for(double q, double kv) const;   // cost of one chunk
};
struct SimResult {
  std::vector<double> attn_ms, linear_ms, comm_ms;
  double step_ms = 0.0, imbalance = 0.0;
};
SimResult simulate(const Plan& plan, const TimeModel& tm, const ModelDims& dims);

}  // namespace planner
}  // namespace dca

// pybind11 bindings of the CAD planner: module ``distca_b200._planner``.
// Heavy calls release the GIL so a Python thread can plan step N+1 while step N runs.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "planner.h"

namespace py = pybind11;
using namespace dca::planner;

template <typename T>
static py::array_t<T> to_numpy(const std::vector<T>& v) {
  py::array_t<T> a(v.size());
  if (!v.empty()) std::memcpy(a.mutable_data(), v.data(), v.size() * sizeof(T));
  return a;
}

static py::array_t<int32_t> tasks_to_numpy(const std::vector<Task>& t) {
  py::array_t<int32_t> a({(py::ssize_t)t.size(), (py::ssize_t)8});
  auto m = a.mutable_unchecked<2>();
  for (py::ssize_t i = 0; i < (py::ssize_t)t.size(); ++i) {
    m(i, 0) = t[i].doc; m(i, 1) = t[i].q_a; m(i, 2) = t[i].q_b; m(i, 3) = t[i].q_row0;
    m(i, 4) = t[i].k_row0; m(i, 5) = t[i].kv_len; m(i, 6) = t[i].owner; m(i, 7) = t[i].owner_row0;
  }
  return a;
}

static py::array_t<int32_t> ctxseg_to_numpy(const std::vector<ContextSegment>& t) {
  py::array_t<int32_t> a({(py::ssize_t)t.size(), (py::ssize_t)5});
  auto m = a.mutable_unchecked<2>();
  for (py::ssize_t i = 0; i < (py::ssize_t)t.size(); ++i) {
    m(i, 0) = t[i].k_row0; m(i, 1) = t[i].n; m(i, 2) = t[i].owner; m(i, 3) = t[i].owner_row0; m(i, 4) = t[i].slot;
  }
  return a;
}

static py::array_t<int32_t> layout_to_numpy(const std::vector<Segment>& t) {
  py::array_t<int32_t> a({(py::ssize_t)t.size(), (py::ssize_t)4});
  auto m = a.mutable_unchecked<2>();
  for (py::ssize_t i = 0; i < (py::ssize_t)t.size(); ++i) {
    m(i, 0) = t[i].doc; m(i, 1) = t[i].a; m(i, 2) = t[i].b; m(i, 3) = t[i].row0;
  }
  return a;
}

static py::list items_to_list(const std::vector<Item>& items) {
  py::list out;
  for (const auto& it : items) {
    py::dict d;
    d["doc"] = it.doc; d["doc_len"] = it.doc_len; d["src"] = it.src; d["dst"] = it.dst;
    d["head"] = py::make_tuple(it.head.a, it.head.b);
    d["tail"] = py::make_tuple(it.tail.a, it.tail.b);
    d["head_row0"] = it.head_row0; d["tail_row0"] = it.tail_row0;
    d["flops"] = it.flops();
    out.append(d);
  }
  return out;
}

PYBIND11_MODULE(_planner, m) {
  m.doc() = "C++ CAD planner: linear layout, balancing, dispatch tables, simulator";

  py::class_<ModelDims>(m, "ModelDims")
      .def(py::init<>())
      .def_readwrite("q_row_bytes", &ModelDims::q_row_bytes)
      .def_readwrite("kv_row_bytes", &ModelDims::kv_row_bytes);

  py::class_<CostModel>(m, "CostModel")
      .def(py::init<>())
      .def_readwrite("enabled", &CostModel::enabled)
      .def_readwrite("tile", &CostModel::tile)
      .def_readwrite("ms_per_tile_pair", &CostModel::ms_per_tile_pair)
      .def_readwrite("ms_per_q_tile", &CostModel::ms_per_q_tile)
      .def_readwrite("ms_per_task", &CostModel::ms_per_task)
      .def("chunk_ms", &CostModel::chunk_ms);

  py::class_<PlannerOptions>(m, "PlannerOptions")
      .def(py::init<>())
      .def_readwrite("world", &PlannerOptions::world)
      .def_readwrite("tokens_per_rank", &PlannerOptions::tokens_per_rank)
      .def_readwrite("tolerance", &PlannerOptions::tolerance)
      .def_readwrite("dims", &PlannerOptions::dims)
      .def_readwrite("max_q_rows", &PlannerOptions::max_q_rows)
      .def_readwrite("max_kv_rows", &PlannerOptions::max_kv_rows)
      .def_readwrite("per_task_overhead_flops", &PlannerOptions::per_task_overhead_flops)
      .def_readwrite("cost", &PlannerOptions::cost)
      .def_readwrite("speed", &PlannerOptions::speed);

  py::class_<RankPlan>(m, "RankPlan")
      .def_readonly("num_tokens", &RankPlan::num_tokens)
      .def_readonly("max_copies", &RankPlan::max_copies)
      .def_readonly("q_rows", &RankPlan::q_rows)
      .def_readonly("kv_rows", &RankPlan::kv_rows)
      .def_readonly("flops", &RankPlan::flops)
      .def_property_readonly("layout", [](const RankPlan& r) { return layout_to_numpy(r.layout); })
      .def_property_readonly("q_dst_rank", [](const RankPlan& r) { return to_numpy(r.q_dst_rank); })
      .def_property_readonly("q_dst_row", [](const RankPlan& r) { return to_numpy(r.q_dst_row); })
      .def_property_readonly("kv_dst_rank", [](const RankPlan& r) { return to_numpy(r.kv_dst_rank); })
      .def_property_readonly("kv_dst_row", [](const RankPlan& r) { return to_numpy(r.kv_dst_row); })
      .def_property_readonly("tasks", [](const RankPlan& r) { return tasks_to_numpy(r.tasks); })
      .def_property_readonly("ctx_segments", [](const RankPlan& r) { return ctxseg_to_numpy(r.ctx_segments); })
      .def_property_readonly("send_bytes", [](const RankPlan& r) { return to_numpy(r.send_bytes); });

  py::class_<Plan>(m, "Plan")
      .def_readonly("world", &Plan::world)
      .def_readonly("tolerance_used", &Plan::tolerance_used)
      .def_readonly("flops_before", &Plan::flops_before)
      .def_readonly("flops_after", &Plan::flops_after)
      .def_readonly("imbalance_before", &Plan::imbalance_before)
      .def_readonly("imbalance_after", &Plan::imbalance_after)
      .def_readonly("cost_after", &Plan::cost_after)
      .def_readonly("cost_imbalance_after", &Plan::cost_imbalance_after)
      .def_readonly("fits", &Plan::fits)
      .def_property_readonly("items", [](const Plan& p) { return items_to_list(p.items); })
      .def("rank", [](const Plan& p, int r) -> const RankPlan& { return p.ranks.at(r); },
           py::return_value_policy::reference_internal);

  py::class_<Fa2aMatrices>(m, "Fa2aMatrices")
      .def_readonly("world", &Fa2aMatrices::world)
      .def_readonly("max_send", &Fa2aMatrices::max_send)
      .def_readonly("max_recv", &Fa2aMatrices::max_recv)
      .def_property_readonly("send_disp", [](const Fa2aMatrices& f) { return to_numpy(f.send_disp); })
      .def_property_readonly("transfer_sz", [](const Fa2aMatrices& f) { return to_numpy(f.transfer_sz); })
      .def_property_readonly("recv_disp", [](const Fa2aMatrices& f) { return to_numpy(f.recv_disp); })
      .def_property_readonly("recv_transfer_sz", [](const Fa2aMatrices& f) { return to_numpy(f.recv_transfer_sz); });

  py::class_<TimeModel>(m, "TimeModel")
      .def(py::init<>())
      .def_readwrite("attn_len", &TimeModel::attn_len)
      .def_readwrite("attn_ms", &TimeModel::attn_ms)
      .def_readwrite("linear_ms_per_token", &TimeModel::linear_ms_per_token)
      .def_readwrite("link_gbytes_per_s", &TimeModel::link_gbytes_per_s)
      .def("attn_ms_for", &TimeModel::attn_ms_for);

  py::class_<SimResult>(m, "SimResult")
      .def_readonly("attn_ms", &SimResult::attn_ms)
      .def_readonly("linear_ms", &SimResult::linear_ms)
      .def_readonly("comm_ms", &SimResult::comm_ms)
      .def_readonly("step_ms", &SimResult::step_ms)
      .def_readonly("imbalance", &SimResult::imbalance);

  m.def("batch_to_items", [](const std::vector<std::vector<int>>& b, long tpr, int world) {
    return items_to_list(batch_to_items(b, tpr, world));
  });
  m.def("batch_to_items_with_dummy", [](const std::vector<std::vector<int>>& b, long tpr, int world) {
    return items_to_list(batch_to_items_with_dummy(b, tpr, world));
  });
  m.def("cp_list_to_mlp_list", &cp_list_to_mlp_list);
  m.def("plan_batch", &plan_batch, py::arg("batches"), py::arg("options"), py::arg("with_dummy") = false,
        py::call_guard<py::gil_scoped_release>());
  m.def("plan_fixed_cp", &plan_fixed_cp, py::arg("docs_per_rank"), py::arg("options"), py::arg("min_len"),
        "Per-document context-parallel baseline placement (no balancing) for documents already on their ranks.",
        py::call_guard<py::gil_scoped_release>());
  m.def("plan_fixed_water_fill", &plan_fixed_water_fill, py::arg("docs_per_rank"), py::arg("options"),
        "Legacy policy: only the most expensive document is cut and spread (water filling).",
        py::call_guard<py::gil_scoped_release>());
  m.def("plan_fixed", &plan_fixed, py::arg("docs_per_rank"), py::arg("options"),
        py::call_guard<py::gil_scoped_release>());
  m.def("balance_only", [](const std::vector<std::vector<int>>& b, const PlannerOptions& opt) {
    auto layout = batch_to_items(b, opt.tokens_per_rank, opt.world);
    return items_to_list(balance(layout, opt));
  });
  m.def("fa2a_matrices", &fa2a_matrices);
  m.def("simulate", &simulate, py::call_guard<py::gil_scoped_release>());
}

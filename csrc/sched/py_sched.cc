// pybind11 surface of the host scheduler: numpy int64 matrices in, plans out.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <chrono>
#include <cstring>

#include "plan.h"

namespace py = pybind11;
using namespace fastb;

namespace {

using I64Array = py::array_t<int64_t, py::array::c_style | py::array::forcecast>;

Matrix to_matrix(const I64Array& a) {
  if (a.ndim() != 2 || a.shape(0) != a.shape(1)) throw std::invalid_argument("traffic matrix must be square int64[n, n]");
  return Matrix(static_cast<int>(a.shape(0)), a.data());
}
I64Array from_matrix(const Matrix& m) {
  I64Array a({m.n, m.n});
  std::copy(m.v.begin(), m.v.end(), a.mutable_data());
  return a;
}
py::dict stage_list(const Decomposition& d) {
  py::dict r;
  py::list st;
  for (const Stage& s : d.stages) st.append(py::make_tuple(s.weight, s.to));
  r["stages"] = st;
  r["line_sum"] = d.line_sum;
  r["scale"] = d.scale;
  r["padded"] = from_matrix(d.padded);
  r["padding"] = from_matrix(d.padding);
  return r;
}

// Work items as one int64[k, 10] array: src_off, dst_off, bytes, dst_rank, src_buf, dst_buf,
// wait_kind, signal_kind, stage, wait_stage.
py::dict program_dict(const RankProgram& g) {
  py::dict d;
  I64Array items({static_cast<py::ssize_t>(g.items.size()), static_cast<py::ssize_t>(10)});
  int64_t* q = items.mutable_data();
  for (const WorkItem& w : g.items) {
    *q++ = w.src_off; *q++ = w.dst_off; *q++ = w.bytes; *q++ = w.dst_rank; *q++ = w.src_buf; *q++ = w.dst_buf;
    *q++ = w.wait_kind; *q++ = w.signal_kind; *q++ = w.stage; *q++ = w.wait_stage;
  }
  d["rank"] = g.rank;
  d["items"] = items;
  d["expect_output_bytes"] = g.expect_output_bytes;
  d["expect_balance_bytes"] = g.expect_balance_bytes;
  d["expect_rail_bytes"] = g.expect_rail_bytes;
  d["input_bytes"] = g.buffers_bytes.input_units;
  d["output_bytes"] = g.buffers_bytes.output_units;
  d["balance_bytes"] = g.buffers_bytes.balance_units;
  d["rail_bytes"] = g.buffers_bytes.rail_units;
  return d;
}

}  // namespace

PYBIND11_MODULE(_sched, m) {
  m.doc() = "Host scheduler: doubly-stochastic padding, BvN stages, hierarchical plans, cost model";

  py::enum_<PlanKind>(m, "PlanKind")
      .value("STAGED", PlanKind::kStaged).value("SINGLE_BURST", PlanKind::kSingleBurst)
      .value("FANOUT", PlanKind::kFanout).value("SPREAD_OUT", PlanKind::kSpreadOut);
  py::enum_<MatchPolicy>(m, "MatchPolicy").value("FIRST_FIT", MatchPolicy::kFirstFit).value("BOTTLENECK", MatchPolicy::kBottleneck);
  py::enum_<ScalePolicy>(m, "ScalePolicy")
      .value("NONE", ScalePolicy::kNone).value("LIMIT_MAX_SUM", ScalePolicy::kLimitMaxSum)
      .value("ALWAYS", ScalePolicy::kAlways).value("ALPHA_BETA", ScalePolicy::kAlphaBeta);

  py::class_<LinkModel>(m, "LinkModel")
      .def(py::init([](double a, double b) { return LinkModel{a, b}; }), py::arg("alpha_us") = 0.0, py::arg("beta_us_per_mb") = 0.0)
      .def_readwrite("alpha_us", &LinkModel::alpha_us).def_readwrite("beta_us_per_mb", &LinkModel::beta_us_per_mb);
  m.def("nvlink_model", &nvlink_model, py::arg("gbytes_per_s") = 900.0, py::arg("alpha_us") = 2.0);
  m.def("gbps_model", &gbps_model);
  m.def("hybrid_cube_mesh_links", &hybrid_cube_mesh_links);

  m.def("decompose", [](const I64Array& a, MatchPolicy pol, int64_t scale) {
    Decomposition d = decompose(to_matrix(a), pol, scale);
    py::dict r = stage_list(d);
    r["exact"] = verify_decomposition(d);
    return r;
  }, py::arg("matrix"), py::arg("policy") = MatchPolicy::kFirstFit, py::arg("scale") = 1);
  m.def("decompose_time_us", [](const I64Array& a, MatchPolicy pol, int reps) {
    Matrix mm = to_matrix(a);
    auto t0 = std::chrono::steady_clock::now();
    size_t sink = 0;
    for (int r = 0; r < reps; ++r) sink += decompose(mm, pol, 1).stages.size();
    auto t1 = std::chrono::steady_clock::now();
    (void)sink;
    return std::chrono::duration<double, std::micro>(t1 - t0).count() / reps;
  }, py::arg("matrix"), py::arg("policy") = MatchPolicy::kFirstFit, py::arg("reps") = 100);
  m.def("choose_scale", [](const I64Array& a, int gpus, ScalePolicy sp, LinkModel inter, LinkModel intra, double mbpu) {
    return choose_scale(to_matrix(a), gpus, sp, inter, intra, mbpu);
  });
  m.def("matrix_hash", [](const I64Array& a) { return to_matrix(a).hash(); });

  py::class_<Plan>(m, "Plan")
      .def_property_readonly("servers", [](const Plan& p) { return p.topo.servers; })
      .def_property_readonly("gpus", [](const Plan& p) { return p.topo.gpus; })
      .def_property_readonly("kind", [](const Plan& p) { return p.opt.kind; })
      .def_property_readonly("only_rank", [](const Plan& p) { return p.opt.only_rank; })
      .def_property_readonly("rail_tail_start", [](const Plan& p) { return p.rail_tail_start; })
      .def_property_readonly("transpose", [](const Plan& p) { return p.opt.transpose; })
      .def_property_readonly("num_stages", [](const Plan& p) { return p.num_stages; })
      .def_property_readonly("num_ops", [](const Plan& p) { return p.ops.size(); })
      .def_property_readonly("matrix", [](const Plan& p) { return from_matrix(p.matrix); })
      .def_property_readonly("server_matrix", [](const Plan& p) { return from_matrix(p.server_matrix); })
      .def_property_readonly("matrix_hash", [](const Plan& p) { return p.matrix_hash; })
      .def_property_readonly("decomposition", [](const Plan& p) { return stage_list(p.decomp); })
      .def_property_readonly("in_disp", [](const Plan& p) {
        const int n = p.matrix.n; I64Array a({n, n}); std::copy(p.in_disp.begin(), p.in_disp.end(), a.mutable_data()); return a; })
      .def_property_readonly("out_disp", [](const Plan& p) {
        const int n = p.matrix.n; I64Array a({n, n}); std::copy(p.out_disp.begin(), p.out_disp.end(), a.mutable_data()); return a; })
      .def_property_readonly("buffers", [](const Plan& p) {
        // int64[n, 4]: input, output, balance, rail units per rank
        I64Array a({static_cast<py::ssize_t>(p.buffers.size()), static_cast<py::ssize_t>(4)});
        int64_t* q = a.mutable_data();
        for (const RankBuffers& b : p.buffers) { *q++ = b.input_units; *q++ = b.output_units; *q++ = b.balance_units; *q++ = b.rail_units; }
        return a; })
      .def_property_readonly("ops", [](const Plan& p) {
        // int64[k, 12]: phase, stage, src_rank, dst_rank, src_buf, dst_buf, src_off, dst_off, len, origin, final, pair_off
        I64Array a({static_cast<py::ssize_t>(p.ops.size()), static_cast<py::ssize_t>(12)});
        int64_t* q = a.mutable_data();
        for (const Op& o : p.ops) {
          *q++ = static_cast<int>(o.phase); *q++ = o.stage; *q++ = o.src_rank; *q++ = o.dst_rank; *q++ = static_cast<int>(o.src_buf);
          *q++ = static_cast<int>(o.dst_buf); *q++ = o.src_off; *q++ = o.dst_off; *q++ = o.len; *q++ = o.origin; *q++ = o.final_dst; *q++ = o.pair_off;
        }
        return a; })
      .def("validate", &validate_plan)
      .def("tampered", [](const Plan& p, int64_t op, const std::string& field, int64_t value) {
        // A copy with one op damaged, for tests of the validator and of the executors' checks.
        Plan q = p;
        if (op < 0 || op >= static_cast<int64_t>(q.ops.size())) throw std::out_of_range("tampered: op index");
        Op& o = q.ops[static_cast<size_t>(op)];
        if (field == "drop") q.ops.erase(q.ops.begin() + op);
        else if (field == "duplicate") q.ops.push_back(o);
        else if (field == "len") o.len = value;
        else if (field == "src_off") o.src_off = value;
        else if (field == "dst_off") o.dst_off = value;
        else if (field == "pair_off") o.pair_off = value;
        else if (field == "src_rank") o.src_rank = static_cast<int32_t>(value);
        else if (field == "dst_rank") o.dst_rank = static_cast<int32_t>(value);
        else if (field == "stage") o.stage = static_cast<int32_t>(value);
        else throw std::invalid_argument("tampered: field");
        return q; }, py::arg("op"), py::arg("field"), py::arg("value") = 0)
      .def("delivered_matrix", [](const Plan& p) { return from_matrix(delivered_matrix(p)); })
      .def("stage_matrix", [](const Plan& p, int k) { return from_matrix(stage_matrix(p, k)); })
      .def("to_json", &plan_to_json, py::arg("include_ops") = true)
      .def("to_bytes", [](const Plan& p) { auto b = plan_to_bytes(p); return py::bytes(reinterpret_cast<const char*>(b.data()), b.size()); })
      .def_static("from_bytes", [](const py::bytes& s) { std::string t = s; return plan_from_bytes(std::vector<uint8_t>(t.begin(), t.end())); })
      .def("cost", [](const Plan& p, LinkModel inter, LinkModel intra, double mbpu, const std::string& topo, std::vector<int> links) {
        CostModel cm{inter, intra, mbpu};
        if (topo == "full_mesh") cm.intra_topology = IntraTopology::kFullMesh;
        else if (topo == "ring") cm.intra_topology = IntraTopology::kRing;
        else if (topo == "hybrid_cube_mesh") { cm.intra_topology = IntraTopology::kLinkGraph; cm.links = hybrid_cube_mesh_links(); }
        else if (topo == "links") { cm.intra_topology = IntraTopology::kLinkGraph; cm.links = std::move(links); }
        else if (topo != "switch") throw std::invalid_argument("intra_topology: switch | full_mesh | ring | hybrid_cube_mesh | links");
        PlanCost c = model_cost(p, cm);
        py::dict d;
        d["total_us"] = c.total_us; d["balance_us"] = c.balance_us; d["inter_us"] = c.inter_us; d["exposed_intra_us"] = c.exposed_intra_us;
        d["lower_bound_us"] = c.lower_bound_us; d["spread_out_us"] = c.spread_out_us; d["chunked_total_us"] = c.chunked_total_us;
        d["balance_per_stage_total_us"] = c.balance_per_stage_total_us; d["stage_balance_us"] = c.stage_balance_us;
        d["stage_inter_us"] = c.stage_inter_us; d["stage_redistribute_us"] = c.stage_redistribute_us;
        return d; }, py::arg("inter"), py::arg("intra"), py::arg("mb_per_unit") = 1.0, py::arg("intra_topology") = "switch",
           py::arg("links") = std::vector<int>())
      .def("lower", [](const Plan& p, int rank, int unit_bytes, int64_t chunk_bytes, int64_t rail_segment_bytes, int max_rail_slots) {
        LowerOptions lo; lo.unit_bytes = unit_bytes; lo.chunk_bytes = chunk_bytes; lo.rail_segment_bytes = rail_segment_bytes; lo.max_rail_slots = max_rail_slots;
        return program_dict(lower_for_rank(p, rank, lo)); }, py::arg("rank"), py::arg("unit_bytes") = 1, py::arg("chunk_bytes") = 1 << 20,
           py::arg("rail_segment_bytes") = 0, py::arg("max_rail_slots") = 4096)
      .def("run_threads", [](const Plan& p, std::vector<py::array_t<uint8_t, py::array::c_style>> ins, int unit_bytes, int64_t chunk_bytes,
                             int workers, int epochs, double timeout_s, int absent_rank, int withhold_rank, int64_t withhold_item,
                             int64_t rail_segment_bytes) {
        const int n = p.matrix.n;
        if (static_cast<int>(ins.size()) != n) throw std::invalid_argument("need one input array per rank");
        std::vector<const uint8_t*> ip;
        for (int r = 0; r < n; ++r) {
          if (ins[r].size() < p.buffers[r].input_units * unit_bytes) throw std::invalid_argument("input smaller than the plan needs");
          ip.push_back(ins[r].data());
        }
        HostRunOptions o; o.unit_bytes = unit_bytes; o.chunk_bytes = chunk_bytes; o.workers = workers; o.epochs = epochs; o.timeout_s = timeout_s;
        o.absent_rank = absent_rank; o.withhold_rank = withhold_rank; o.withhold_item = withhold_item; o.rail_segment_bytes = rail_segment_bytes;
        HostRunResult res;
        { py::gil_scoped_release nogil; res = run_on_host_threads(p, o, ip); }
        py::dict d;
        d["ok"] = res.ok;
        d["failure"] = py::make_tuple(res.failure.rank, res.failure.site, res.failure.detail, res.failure.seen, res.failure.want);
        py::list outs;
        for (auto& v : res.outputs) { py::array_t<uint8_t> a(static_cast<py::ssize_t>(v.size())); std::memcpy(a.mutable_data(), v.data(), v.size()); outs.append(a); }
        d["outputs"] = outs;
        return d; }, py::arg("inputs"), py::arg("unit_bytes") = 1, py::arg("chunk_bytes") = 4096, py::arg("workers") = 3, py::arg("epochs") = 2,
           py::arg("timeout_s") = 2.0, py::arg("absent_rank") = -1, py::arg("withhold_rank") = -1, py::arg("withhold_item") = -1,
           py::arg("rail_segment_bytes") = 0)
      .def("execute_on_host", [](const Plan& p, int unit_bytes, std::vector<py::array_t<uint8_t, py::array::c_style>> ins,
                                 std::vector<py::array_t<uint8_t, py::array::c_style>> outs, int64_t drop_op) {
        const int n = p.matrix.n;
        if (static_cast<int>(ins.size()) != n || static_cast<int>(outs.size()) != n) throw std::invalid_argument("need one input and one output array per rank");
        std::vector<const uint8_t*> ip; std::vector<uint8_t*> op;
        for (int r = 0; r < n; ++r) {
          if (ins[r].size() < p.buffers[r].input_units * unit_bytes || outs[r].size() < p.buffers[r].output_units * unit_bytes)
            throw std::invalid_argument("buffer smaller than the plan needs");
          ip.push_back(ins[r].data()); op.push_back(outs[r].mutable_data());
        }
        return execute_on_host(p, unit_bytes, ip, op, drop_op); }, py::arg("unit_bytes"), py::arg("inputs"), py::arg("outputs"), py::arg("drop_op") = -1);

  m.def("build_plan", [](const I64Array& a, int servers, int gpus, PlanKind kind, MatchPolicy match, ScalePolicy sp, int64_t scale,
                         int64_t split_align, bool transpose, LinkModel inter, LinkModel intra, double mbpu, bool balance_alpha_beta, int only_rank) {
    PlanOptions o; o.kind = kind; o.match = match; o.scale_policy = sp; o.scale = scale; o.split_align = split_align; o.transpose = transpose;
    o.inter = inter; o.intra = intra; o.mb_per_unit = mbpu; o.balance_alpha_beta = balance_alpha_beta; o.only_rank = only_rank;
    return build_plan(to_matrix(a), Topology{servers, gpus}, o);
  }, py::arg("matrix"), py::arg("servers"), py::arg("gpus"), py::arg("kind") = PlanKind::kStaged, py::arg("match") = MatchPolicy::kFirstFit,
     py::arg("scale_policy") = ScalePolicy::kNone, py::arg("scale") = 0, py::arg("split_align") = 1, py::arg("transpose") = false,
     py::arg("inter") = LinkModel{0.7, 22.0}, py::arg("intra") = LinkModel{0.1, 1.2}, py::arg("mb_per_unit") = 1.0,
     py::arg("balance_alpha_beta") = false, py::arg("only_rank") = -1);
  m.def("select_plan", [](const I64Array& a, int servers, int gpus, std::vector<PlanKind> kinds, LinkModel inter, LinkModel intra, double mbpu,
                          MatchPolicy match, ScalePolicy sp, int64_t split_align, bool transpose, bool balance_alpha_beta) {
    PlanOptions o; o.match = match; o.scale_policy = sp; o.split_align = split_align; o.transpose = transpose;
    o.inter = inter; o.intra = intra; o.mb_per_unit = mbpu; o.balance_alpha_beta = balance_alpha_beta;
    PlanChoice c = select_plan(to_matrix(a), Topology{servers, gpus}, o, CostModel{inter, intra, mbpu}, kinds);
    py::list table;
    for (auto& kv : c.modeled_us) table.append(py::make_tuple(kv.first, kv.second));
    return py::make_tuple(std::move(c.plan), table);
  }, py::arg("matrix"), py::arg("servers"), py::arg("gpus"), py::arg("kinds"), py::arg("inter"), py::arg("intra"), py::arg("mb_per_unit") = 1.0,
     py::arg("match") = MatchPolicy::kFirstFit, py::arg("scale_policy") = ScalePolicy::kNone, py::arg("split_align") = 1,
     py::arg("transpose") = false, py::arg("balance_alpha_beta") = false);
  m.def("build_plan_time_us", [](const I64Array& a, int servers, int gpus, int reps) {
    Matrix mm = to_matrix(a);
    auto t0 = std::chrono::steady_clock::now();
    size_t sink = 0;
    for (int r = 0; r < reps; ++r) sink += build_plan(mm, Topology{servers, gpus}, PlanOptions{}).ops.size();
    auto t1 = std::chrono::steady_clock::now();
    (void)sink;
    return std::chrono::duration<double, std::micro>(t1 - t0).count() / reps;
  });

  m.def("workload_uniform", [](int n, int64_t mx, uint64_t seed, bool zd) { return from_matrix(workload_uniform(n, mx, seed, zd)); },
        py::arg("n"), py::arg("max_entry"), py::arg("seed"), py::arg("zero_diag") = false);
  m.def("workload_balanced", [](int n, int64_t e, bool zd) { return from_matrix(workload_balanced(n, e, zd)); }, py::arg("n"), py::arg("entry"), py::arg("zero_diag") = false);
  m.def("workload_zipf_rows", [](int n, double s, int64_t total, uint64_t seed, int64_t q) { return from_matrix(workload_zipf_rows(n, s, total, seed, q)); },
        py::arg("n"), py::arg("s"), py::arg("row_total"), py::arg("seed"), py::arg("quantum") = 1);
  m.def("workload_zipf_entries", [](int n, double s, int64_t mx, uint64_t seed) { return from_matrix(workload_zipf_entries(n, s, mx, seed)); });
}

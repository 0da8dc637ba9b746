// fastb-sim: CPU-only simulator and plan checker.
//
// Sub-commands (all print one JSON object per line):
//   plan      build + validate a plan for one seeded matrix and report stages / modeled time
//   verify    random matrices over a range of dimensions; decomposition must be exact
//   grid      modeled speed-up over spread-out for a servers x gpus grid
//   skew      modeled speed-up vs Zipf skew
//   size      modeled speed-up vs transfer size with and without coarsening
//   fabric    modeled speed-up and exposed intra-server share vs intra-server link speed
//   topology  modeled speed-up under each intra-server fabric model
//   overhead  scheduler time and staging memory relative to the payload, per cluster size
// Covers the reference simulator's drivers (simulation/test.cpp:15-60 DecompositionTester,
// :73-116 run, :119-264 grid, :346-498 fabric, :501-592 skew, :595-684 size).
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>

#include "../sched/plan.h"

using namespace fastb;

namespace {
struct Args {
  std::map<std::string, std::string> kv;
  double num(const char* k, double d) const { auto it = kv.find(k); return it == kv.end() ? d : std::atof(it->second.c_str()); }
  long long integer(const char* k, long long d) const { auto it = kv.find(k); return it == kv.end() ? d : std::atoll(it->second.c_str()); }
  std::string str(const char* k, const char* d) const { auto it = kv.find(k); return it == kv.end() ? d : it->second; }
};
Args parse(int argc, char** argv) {
  Args a;
  for (int i = 2; i < argc; ++i) {
    std::string s = argv[i];
    if (s.rfind("--", 0) != 0) continue;
    size_t eq = s.find('=');
    if (eq == std::string::npos) a.kv[s.substr(2)] = (i + 1 < argc && argv[i + 1][0] != '-') ? argv[++i] : "1";
    else a.kv[s.substr(2, eq - 2)] = s.substr(eq + 1);
  }
  return a;
}
double now_us() { return std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now().time_since_epoch()).count(); }

Matrix make_workload(const Args& a, int n, uint64_t seed) {
  const std::string w = a.str("workload", "zipf");
  if (w == "uniform") return workload_uniform(n, a.integer("max-entry", 10000), seed, a.integer("zero-diag", 0));
  if (w == "balanced") return workload_balanced(n, a.integer("entry", 1 << 20), a.integer("zero-diag", 1));
  if (w == "zipf-entries") return workload_zipf_entries(n, a.num("skew", 0.8), a.integer("max-entry", 10000), seed);
  return workload_zipf_rows(n, a.num("skew", 1.2), a.integer("row-bytes", 256ll << 20), seed, a.integer("quantum", 1));
}
PlanKind kind_of(const std::string& s) {
  if (s == "burst") return PlanKind::kSingleBurst;
  if (s == "fanout") return PlanKind::kFanout;
  if (s == "spreadout") return PlanKind::kSpreadOut;
  return PlanKind::kStaged;
}
CostModel cost_of(const Args& a, int servers) {
  CostModel cm;
  if (servers == 1 || a.integer("flat", 0)) {
    cm.inter = cm.intra = nvlink_model(a.num("nvlink-gbs", 900.0), a.num("alpha-us", 2.0));
  } else {
    cm.inter = gbps_model(a.num("inter-gbps", 400.0), a.num("inter-alpha-us", 0.7));
    cm.intra = nvlink_model(a.num("nvlink-gbs", 900.0), a.num("intra-alpha-us", 0.1));
  }
  cm.mb_per_unit = a.num("mb-per-unit", 1e-6);  // default unit = 1 byte
  const std::string topo = a.str("intra-topology", "switch");
  if (topo == "full_mesh") cm.intra_topology = IntraTopology::kFullMesh;
  else if (topo == "ring") cm.intra_topology = IntraTopology::kRing;
  else if (topo == "hybrid_cube_mesh") { cm.intra_topology = IntraTopology::kLinkGraph; cm.links = hybrid_cube_mesh_links(); }
  return cm;
}

int cmd_plan(const Args& a) {
  const int S = static_cast<int>(a.integer("servers", 8)), G = static_cast<int>(a.integer("gpus", 1));
  const int n = S * G;
  Matrix m = make_workload(a, n, static_cast<uint64_t>(a.integer("seed", 1)));
  PlanOptions o;
  o.kind = kind_of(a.str("kind", "staged"));
  o.match = a.str("match", "first") == "bottleneck" ? MatchPolicy::kBottleneck : MatchPolicy::kFirstFit;
  o.split_align = a.integer("align", 1);
  o.scale = a.integer("scale", 0);
  o.transpose = a.integer("transpose", 0);
  const bool pick = a.str("kind", "staged") == "auto";  // let the cost model choose among the kinds
  const double t0 = now_us();
  Plan p;
  if (pick) {
    std::vector<PlanKind> cand = {PlanKind::kFanout, PlanKind::kStaged};
    if (G > 1) cand.push_back(PlanKind::kSingleBurst);
    PlanChoice ch = select_plan(m, Topology{S, G}, o, cost_of(a, S), cand);
    for (auto& kv : ch.modeled_us)
      std::printf("{\"cmd\":\"plan\",\"candidate\":%d,\"modeled_us\":%.3f}\n", static_cast<int>(kv.first), kv.second);
    p = std::move(ch.plan);
    o.kind = p.opt.kind;
  } else {
    p = build_plan(m, Topology{S, G}, o);
  }
  const double t1 = now_us();
  const std::string err = validate_plan(p);
  const bool exact = delivered_matrix(p) == p.matrix;
  // The stages must add up to the matrix exactly: re-sum every stage's real traffic.
  Matrix acc(n);
  for (const Op& q : p.ops)
    if (q.src_buf == Buf::kInput) acc.at(q.origin, q.final_dst) += q.len;
  const bool stages_sum = acc == p.matrix;
  PlanCost c = model_cost(p, cost_of(a, S));
  std::printf("{\"cmd\":\"plan\",\"kind\":%d,\"servers\":%d,\"gpus\":%d,\"stages\":%d,\"ops\":%zu,\"valid\":%s,\"error\":\"%s\",\"delivered_exact\":%s,"
              "\"stages_sum_to_matrix\":%s,\"decomposition_exact\":%s,\"line_sum\":%lld,\"max_line_sum_input\":%lld,\"scheduler_us\":%.2f,"
              "\"modeled_us\":%.3f,\"modeled_chunked_us\":%.3f,\"modeled_balance_per_stage_us\":%.3f,\"lower_bound_us\":%.3f,\"spread_out_us\":%.3f,\"speedup_vs_spread_out\":%.4f,\"bound_fraction\":%.4f}\n",
              static_cast<int>(o.kind), S, G, p.num_stages, p.ops.size(), err.empty() ? "true" : "false", err.c_str(), exact ? "true" : "false",
              stages_sum ? "true" : "false", (o.kind != PlanKind::kStaged || verify_decomposition(p.decomp)) ? "true" : "false",
              static_cast<long long>(p.decomp.line_sum), static_cast<long long>(p.matrix.max_line_sum()), t1 - t0, c.total_us, c.chunked_total_us,
              c.balance_per_stage_total_us, c.lower_bound_us, c.spread_out_us, c.total_us > 0 ? c.spread_out_us / c.total_us : 0.0,
              c.total_us > 0 ? c.lower_bound_us / c.total_us : 0.0);
  if (a.integer("dump", 0)) std::printf("%s\n", plan_to_json(p, a.integer("dump", 0) > 1).c_str());
  return err.empty() && exact && stages_sum ? 0 : 1;
}

int cmd_verify(const Args& a) {
  const int lo = static_cast<int>(a.integer("min-dim", 2)), hi = static_cast<int>(a.integer("max-dim", 64));
  const int reps = static_cast<int>(a.integer("reps", 5));
  int bad = 0;
  for (int n = lo; n <= hi; n = n < 16 ? n + 1 : n * 2) {
    double us = 0; size_t stages = 0;
    for (int r = 0; r < reps; ++r) {
      Matrix m = workload_uniform(n, a.integer("max-entry", 10000), 1000 * n + r, false);
      const double t0 = now_us();
      Decomposition d = decompose(m, MatchPolicy::kFirstFit, 1);
      us += now_us() - t0;
      stages += d.stages.size();
      if (!verify_decomposition(d)) ++bad;
    }
    std::printf("{\"cmd\":\"verify\",\"dim\":%d,\"mean_stages\":%.1f,\"mean_us\":%.2f,\"bound_stages\":%d}\n", n,
                static_cast<double>(stages) / reps, us / reps, n * n - 2 * n + 2);
  }
  std::printf("{\"cmd\":\"verify\",\"failures\":%d}\n", bad);
  return bad ? 1 : 0;
}

double speedup(const Matrix& m, int S, int G, const CostModel& cm, ScalePolicy sp, double* exposed = nullptr, double* sched_us = nullptr) {
  PlanOptions o;
  o.scale_policy = sp; o.inter = cm.inter; o.intra = cm.intra; o.mb_per_unit = cm.mb_per_unit;
  const double t0 = now_us();
  Plan p = build_plan(m, Topology{S, G}, o);
  if (sched_us) *sched_us = now_us() - t0;
  PlanCost c = model_cost(p, cm);
  if (exposed) *exposed = c.total_us > 0 ? c.exposed_intra_us / c.total_us : 0;
  return c.total_us > 0 ? c.spread_out_us / c.total_us : 0;
}

int cmd_grid(const Args& a) {
  for (int S : {2, 4, 8, 16, 32, 64})
    for (int G : {2, 4, 8, 16}) {
      if (S * G > a.integer("max-ranks", 512)) continue;
      CostModel cm = cost_of(a, S); cm.mb_per_unit = a.num("mb-per-unit", 1.0);
      double sp = 0, us = 0; const int reps = static_cast<int>(a.integer("reps", 3));
      for (int r = 0; r < reps; ++r) { double u; sp += speedup(workload_uniform(S * G, 10000, 17 * S + G + r, false), S, G, cm, ScalePolicy::kNone, nullptr, &u); us += u; }
      std::printf("{\"cmd\":\"grid\",\"servers\":%d,\"gpus\":%d,\"speedup\":%.3f,\"scheduler_ms\":%.3f}\n", S, G, sp / reps, us / reps / 1e3);
    }
  return 0;
}
int cmd_skew(const Args& a) {
  const int S = static_cast<int>(a.integer("servers", 16)), G = static_cast<int>(a.integer("gpus", 8));
  CostModel cm = cost_of(a, S); cm.mb_per_unit = a.num("mb-per-unit", 1.0);
  for (double s : {0.1, 0.3, 0.5, 0.7, 0.8, 0.9, 0.99}) {
    double sp = speedup(workload_zipf_entries(S * G, s, 10000, 5), S, G, cm, ScalePolicy::kNone);
    std::printf("{\"cmd\":\"skew\",\"servers\":%d,\"gpus\":%d,\"skew\":%.2f,\"speedup\":%.3f}\n", S, G, s, sp);
  }
  return 0;
}
int cmd_size(const Args& a) {
  const int S = static_cast<int>(a.integer("servers", 16)), G = static_cast<int>(a.integer("gpus", 8));
  Matrix m = workload_uniform(S * G, 10000, 9, false);
  for (double mbpu : {1e-7, 1e-6, 1e-5, 1e-4, 1e-3, 1e-2, 1e-1, 1.0}) {
    CostModel cm = cost_of(a, S); cm.mb_per_unit = mbpu;
    std::printf("{\"cmd\":\"size\",\"mb_per_unit\":%g,\"no_scale\":%.3f,\"alpha_beta_scale\":%.3f,\"always_scale\":%.3f}\n", mbpu,
                speedup(m, S, G, cm, ScalePolicy::kNone), speedup(m, S, G, cm, ScalePolicy::kAlphaBeta), speedup(m, S, G, cm, ScalePolicy::kAlways));
  }
  return 0;
}
// Modeled speed-up over spread-out for each intra-server fabric model (the reference's
// topology_benchmark, simulation/test.cpp:266-343), 8 GPUs per server.
int cmd_topology(const Args& a) {
  const int G = 8;
  const char* names[] = {"switch", "full_mesh", "ring", "hybrid_cube_mesh"};
  for (int S : {2, 4, 8, 16}) {
    Matrix m = workload_uniform(S * G, 10000, 21 + S, false);
    Plan p = build_plan(m, Topology{S, G}, PlanOptions{});
    for (int t = 0; t < 4; ++t) {
      CostModel cm;
      cm.inter = gbps_model(a.num("inter-gbps", 100.0), 0.7);
      cm.intra = gbps_model(a.num("intra-gbps", 400.0), 0.1);
      cm.mb_per_unit = a.num("mb-per-unit", 1.0);
      cm.intra_topology = static_cast<IntraTopology>(t);
      if (t == 3) cm.links = hybrid_cube_mesh_links();
      PlanCost c = model_cost(p, cm);
      std::printf("{\"cmd\":\"topology\",\"servers\":%d,\"fabric\":\"%s\",\"modeled_us\":%.1f,\"speedup\":%.3f,\"exposed_intra_share\":%.4f}\n", S, names[t], c.total_us,
                  c.total_us > 0 ? c.spread_out_us / c.total_us : 0.0, c.total_us > 0 ? c.exposed_intra_us / c.total_us : 0.0);
    }
  }
  return 0;
}

// Scheduler cost and staging memory against the plain send/receive buffers, per cluster size
// (the reference's overhead test, amd/test_alltoall.cpp:2750-2823).
int cmd_overhead(const Args& a) {
  const int G = static_cast<int>(a.integer("gpus", 8));
  for (int S = 2; S <= static_cast<int>(a.integer("max-servers", 8)); ++S) {
    Matrix m = workload_uniform(S * G, a.integer("max-entry", 10000), 40 + S, false);
    const int reps = static_cast<int>(a.integer("reps", 20));
    const double t0 = now_us();
    size_t ops = 0;
    Plan p;
    for (int r = 0; r < reps; ++r) { p = build_plan(m, Topology{S, G}, PlanOptions{}); ops += p.ops.size(); }
    const double us = (now_us() - t0) / reps;
    int64_t payload = 0, staging = 0;
    for (const RankBuffers& b : p.buffers) { payload += b.input_units + b.output_units; staging += b.balance_units + b.rail_units; }
    std::printf("{\"cmd\":\"overhead\",\"servers\":%d,\"gpus\":%d,\"scheduler_us\":%.1f,\"stages\":%d,\"ops\":%zu,\"staging_over_payload\":%.4f}\n", S, G, us,
                p.num_stages, p.ops.size(), payload ? static_cast<double>(staging) / static_cast<double>(payload) : 0.0);
    (void)ops;
  }
  return 0;
}
int cmd_fabric(const Args& a) {
  const int S = static_cast<int>(a.integer("servers", 16)), G = static_cast<int>(a.integer("gpus", 8));
  Matrix m = workload_uniform(S * G, 10000, 11, false);
  for (double tbps : {1.0, 2.0, 4.0, 8.0, 16.0}) {
    CostModel cm; cm.inter = gbps_model(a.num("inter-gbps", 100.0), 0.7); cm.intra = gbps_model(tbps * 1000.0, 0.1); cm.mb_per_unit = a.num("mb-per-unit", 1.0);
    double exposed = 0; double sp = speedup(m, S, G, cm, ScalePolicy::kNone, &exposed);
    std::printf("{\"cmd\":\"fabric\",\"intra_tbps\":%.0f,\"speedup\":%.3f,\"exposed_intra_share\":%.4f}\n", tbps, sp, exposed);
  }
  return 0;
}
}  // namespace

int main(int argc, char** argv) {
  if (argc < 2) {
    std::fprintf(stderr, "usage: fastb-sim {plan|verify|grid|skew|size|fabric|topology|overhead} [--key value ...]\n");
    return 2;
  }
  Args a = parse(argc, argv);
  const std::string c = argv[1];
  try {
    if (c == "plan") return cmd_plan(a);
    if (c == "verify") return cmd_verify(a);
    if (c == "grid") return cmd_grid(a);
    if (c == "skew") return cmd_skew(a);
    if (c == "size") return cmd_size(a);
    if (c == "fabric") return cmd_fabric(a);
    if (c == "overhead") return cmd_overhead(a);
    if (c == "topology") return cmd_topology(a);
  } catch (const std::exception& e) {
    std::fprintf(stderr, "fastb-sim: %s\n", e.what());
    return 1;
  }
  std::fprintf(stderr, "unknown command %s\n", c.c_str());
  return 2;
}

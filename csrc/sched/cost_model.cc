// Alpha-beta cost model of a plan, and the baselines it is compared against.
#include <algorithm>

#include "plan.h"

namespace fastb {

LinkModel nvlink_model(double gbytes_per_s, double alpha_us) {
  // 1 MB (1e6 bytes) at X GB/s takes 1e3 / X microseconds.
  return LinkModel{alpha_us, 1e3 / gbytes_per_s};
}
LinkModel gbps_model(double gbit_per_s, double alpha_us) { return LinkModel{alpha_us, 8e3 / gbit_per_s}; }

namespace {
// Ring-offset ("spread-out") time of a dense dim x dim transfer matrix on one link class: round d
// costs the slowest of its transfers (simulation/scheduler/config.cpp:61-80 semantics).
double spread_out_time(const std::vector<int64_t>& m, int dim, LinkModel l, double mbpu) {
  double t = 0;
  for (int d = 0; d < dim; ++d) {
    int64_t mx = 0;
    for (int j = 0; j < dim; ++j) mx = std::max(mx, m[static_cast<size_t>(j) * dim + (j + d) % dim]);
    if (mx) t += l.alpha_us + static_cast<double>(mx) * l.beta_us_per_mb * mbpu;
  }
  return t;
}
double full_mesh_time(const std::vector<int64_t>& m, int dim, LinkModel l, double mbpu) {
  int64_t mx = 0;
  for (int i = 0; i < dim; ++i)
    for (int j = 0; j < dim; ++j)
      if (i != j) mx = std::max(mx, m[static_cast<size_t>(i) * dim + j]);
  return mx ? l.alpha_us + static_cast<double>(mx) * l.beta_us_per_mb * mbpu : 0.0;
}

// Offsets 1 .. (dim-1)/2 travel forward, the rest backward; an offset of h hops pays h times its
// slowest transfer; the two directions use different links and overlap.
double ring_time(const std::vector<int64_t>& m, int dim, LinkModel l, double mbpu) {
  double fwd = 0, rev = 0;
  for (int d = 1; d < dim; ++d) {
    int64_t mx = 0;
    for (int j = 0; j < dim; ++j) mx = std::max(mx, m[static_cast<size_t>(j) * dim + (j + d) % dim]);
    if (!mx) continue;
    const bool forward = d <= (dim - 1) / 2;
    const int hops = forward ? d : dim - d;
    (forward ? fwd : rev) += (l.alpha_us + static_cast<double>(mx) * l.beta_us_per_mb * mbpu) * hops;
  }
  return std::max(fwd, rev);
}

// Phase 1: all directly linked pairs at once (a pair with k links moves k times faster).
// Phase 2: every unlinked pair relays through the neighbour with the widest path; the relays that
// feed one destination share its links, so their second hops add up.
double link_graph_time(const std::vector<int64_t>& m, int dim, const std::vector<int>& links, LinkModel l, double mbpu) {
  if (static_cast<int>(links.size()) != dim * dim) return spread_out_time(m, dim, l, mbpu);
  auto mult = [&](int i, int j) { return links[static_cast<size_t>(i) * dim + j]; };
  double direct = 0, relay = 0;
  for (int i = 0; i < dim; ++i)
    for (int j = 0; j < dim; ++j) {
      const int64_t x = m[static_cast<size_t>(i) * dim + j];
      if (i == j || !x || !mult(i, j)) continue;
      direct = std::max(direct, l.alpha_us + static_cast<double>(x) * l.beta_us_per_mb * mbpu / mult(i, j));
    }
  for (int j = 0; j < dim; ++j) {
    double first = 0, second = 0;
    bool any = false;
    for (int i = 0; i < dim; ++i) {
      const int64_t x = m[static_cast<size_t>(i) * dim + j];
      if (i == j || !x || mult(i, j)) continue;
      int best = -1, width = 0;
      for (int r = 0; r < dim; ++r) {
        const int w = std::min(mult(i, r), mult(r, j));
        if (w > width) { width = w; best = r; }
      }
      if (best < 0) return spread_out_time(m, dim, l, mbpu);  // disconnected description: fall back
      any = true;
      first = std::max(first, static_cast<double>(x) * l.beta_us_per_mb * mbpu / mult(i, best));
      second += static_cast<double>(x) * l.beta_us_per_mb * mbpu / mult(best, j);
    }
    if (any) relay = std::max(relay, 2 * l.alpha_us + first + second);
  }
  return direct + relay;
}

double intra_time(const std::vector<int64_t>& m, int dim, const CostModel& cm) {
  switch (cm.intra_topology) {
    case IntraTopology::kFullMesh: return full_mesh_time(m, dim, cm.intra, cm.mb_per_unit);
    case IntraTopology::kRing: return ring_time(m, dim, cm.intra, cm.mb_per_unit);
    case IntraTopology::kLinkGraph: return link_graph_time(m, dim, cm.links, cm.intra, cm.mb_per_unit);
    default: return spread_out_time(m, dim, cm.intra, cm.mb_per_unit);
  }
}
}  // namespace

std::vector<int> hybrid_cube_mesh_links() {
  std::vector<int> l(64, 0);
  auto set = [&](int a, int b, int k) { l[a * 8 + b] = k; l[b * 8 + a] = k; };
  const int dbl[][2] = {{0, 1}, {0, 2}, {2, 3}, {1, 4}, {3, 6}, {4, 5}, {5, 7}, {6, 7}};
  const int sgl[][2] = {{0, 3}, {1, 2}, {1, 3}, {0, 5}, {2, 7}, {4, 6}, {4, 7}, {5, 6}};
  for (auto& p : dbl) set(p[0], p[1], 2);
  for (auto& p : sgl) set(p[0], p[1], 1);
  return l;
}

PlanCost model_cost(const Plan& p, const CostModel& cm) {
  const int n = p.matrix.n, S = p.topo.servers, G = p.topo.gpus;
  const double mb = cm.mb_per_unit;
  PlanCost c;
  const bool flat_direct = p.opt.kind == PlanKind::kFanout || p.opt.kind == PlanKind::kSpreadOut;

  // Baseline: n rounds, round i pairs j -> (j+i)%n; a round is as slow as its slowest pair.
  for (int i = 0; i < n; ++i) {
    double worst = 0;
    for (int j = 0; j < n; ++j) {
      const int col = (j + i) % n;
      const int64_t x = p.matrix.at(j, col);
      if (!x) continue;
      const LinkModel& l = (j / G == col / G) ? cm.intra : cm.inter;
      worst = std::max(worst, l.alpha_us + static_cast<double>(x) * l.beta_us_per_mb * mb);
    }
    c.spread_out_us += worst;
  }
  // Lower bound: the busiest inter-server port (each GPU owns one), or the busiest port at all
  // when there is a single tier.
  {
    int64_t worst_inter = 0, worst_any = 0;
    for (int s = 0; s < S; ++s) {
      int64_t out = 0, in = 0;
      for (int i = 0; i < G; ++i)
        for (int q = 0; q < n; ++q) {
          if (q / G == s) continue;
          out += p.matrix.at(s * G + i, q);
          in += p.matrix.at(q, s * G + i);
        }
      worst_inter = std::max(worst_inter, (std::max(out, in) + G - 1) / G);
    }
    for (int r = 0; r < n; ++r) {
      int64_t out = p.matrix.row_sum(r) - p.matrix.at(r, r), in = p.matrix.col_sum(r) - p.matrix.at(r, r);
      worst_any = std::max(worst_any, std::max(out, in));
    }
    c.lower_bound_us = S > 1 ? static_cast<double>(worst_inter) * cm.inter.beta_us_per_mb * mb
                             : static_cast<double>(worst_any) * cm.intra.beta_us_per_mb * mb;
  }

  if (flat_direct) {
    if (p.opt.kind == PlanKind::kSpreadOut) {
      c.total_us = c.spread_out_us;
    } else {
      // Fan-out: all pairs in flight at once; the busiest port bounds it, one latency paid.
      int64_t worst = 0;
      for (int r = 0; r < n; ++r) worst = std::max({worst, p.matrix.row_sum(r), p.matrix.col_sum(r)});
      const LinkModel& l = S > 1 ? cm.inter : cm.intra;
      c.total_us = l.alpha_us + static_cast<double>(worst) * l.beta_us_per_mb * mb;
    }
    c.inter_us = c.total_us;
    c.chunked_total_us = c.total_us;
    return c;
  }

  // Balance: per server, one spread-out pass per destination server; servers run in parallel.
  const int K = p.num_stages;
  std::vector<std::vector<int64_t>> bal(static_cast<size_t>(S) * S, std::vector<int64_t>());
  std::vector<std::vector<int64_t>> intrinsic(S, std::vector<int64_t>(static_cast<size_t>(G) * G, 0));
  std::vector<std::vector<int64_t>> redis(static_cast<size_t>(std::max(K, 1)) * S, std::vector<int64_t>());
  std::vector<int64_t> stage_max(std::max(K, 1), 0);
  for (const Op& o : p.ops) {
    const int s = o.src_rank / G, i = o.src_rank % G, j = o.dst_rank % G;
    switch (o.phase) {
      case Phase::kBalance: {
        auto& m = bal[static_cast<size_t>(s) * S + o.final_dst / G];
        if (m.empty()) m.assign(static_cast<size_t>(G) * G, 0);
        m[static_cast<size_t>(i) * G + j] += o.len;
        break;
      }
      case Phase::kIntrinsic: intrinsic[s][static_cast<size_t>(i) * G + j] += o.len; break;
      case Phase::kRedistribute: {
        auto& m = redis[static_cast<size_t>(o.stage) * S + s];
        if (m.empty()) m.assign(static_cast<size_t>(G) * G, 0);
        m[static_cast<size_t>(i) * G + j] += o.len;
        break;
      }
      case Phase::kRail: break;
    }
  }
  // Per stage, the time is set by the most loaded rail: sum real units per (stage, src rank).
  {
    std::vector<int64_t> per(static_cast<size_t>(std::max(K, 1)) * n, 0);
    for (const Op& o : p.ops)
      if (o.phase == Phase::kRail) per[static_cast<size_t>(o.stage) * n + o.src_rank] += o.len;
    for (int k = 0; k < K; ++k)
      for (int r = 0; r < n; ++r) stage_max[k] = std::max(stage_max[k], per[static_cast<size_t>(k) * n + r]);
  }
  for (int s = 0; s < S; ++s) {
    double t = 0;
    for (int d = 0; d < S; ++d) {
      const auto& m = bal[static_cast<size_t>(s) * S + d];
      if (!m.empty()) t += intra_time(m, G, cm);
    }
    c.balance_us = std::max(c.balance_us, t);
  }
  double intrinsic_us = 0;
  for (int s = 0; s < S; ++s) intrinsic_us = std::max(intrinsic_us, intra_time(intrinsic[s], G, cm));

  c.stage_inter_us.assign(K, 0);
  c.stage_redistribute_us.assign(K, 0);
  for (int k = 0; k < K; ++k) {
    if (stage_max[k]) c.stage_inter_us[k] = cm.inter.alpha_us + static_cast<double>(stage_max[k]) * cm.inter.beta_us_per_mb * mb;
    for (int s = 0; s < S; ++s) {
      const auto& m = redis[static_cast<size_t>(k) * S + s];
      if (!m.empty()) c.stage_redistribute_us[k] = std::max(c.stage_redistribute_us[k], intra_time(m, G, cm));
    }
    c.inter_us += c.stage_inter_us[k];
  }
  double t = c.balance_us;
  if (K == 0) {
    t += intrinsic_us;
  } else {
    t += std::max(c.stage_inter_us[0], intrinsic_us);
    for (int k = 1; k < K; ++k) t += std::max(c.stage_inter_us[k], c.stage_redistribute_us[k - 1]);
    t += c.stage_redistribute_us[K - 1];
  }
  c.total_us = t;
  c.exposed_intra_us = t - c.inter_us;
  {
    // Balance per stage: a rail piece whose origin is not the rail GPU was relayed by the balance
    // phase, so the provenance of stage k's rail ops is exactly the balancing stage k needs.
    std::vector<std::vector<int64_t>> sbal(static_cast<size_t>(std::max(K, 1)) * S, std::vector<int64_t>());
    for (const Op& o : p.ops) {
      if (o.phase != Phase::kRail || o.origin == o.src_rank || o.stage < 0 || o.stage >= K) continue;
      auto& m = sbal[static_cast<size_t>(o.stage) * S + o.src_rank / G];
      if (m.empty()) m.assign(static_cast<size_t>(G) * G, 0);
      m[static_cast<size_t>(o.origin % G) * G + o.src_rank % G] += o.len;
    }
    auto bal_time = [&](int k, int s) { const auto& m = sbal[static_cast<size_t>(k) * S + s]; return m.empty() ? 0.0 : intra_time(m, G, cm); };
    auto red_time = [&](int k, int s) { const auto& m = redis[static_cast<size_t>(k) * S + s]; return m.empty() ? 0.0 : intra_time(m, G, cm); };
    c.stage_balance_us.assign(K, 0);
    for (int k = 0; k < K; ++k)
      for (int s = 0; s < S; ++s) c.stage_balance_us[k] = std::max(c.stage_balance_us[k], bal_time(k, s));
    double tv = K > 0 ? c.stage_balance_us[0] : 0.0;
    if (K == 0) tv += intrinsic_us;
    for (int k = 0; k < K; ++k) {
      // While stage k is on the wire each server forwards stage k - 1 and prepares stage k + 1
      // (after the last preparation: the traffic that never leaves the server).
      double intra = 0;
      for (int s = 0; s < S; ++s) {
        const double fwd_prev = k > 0 ? red_time(k - 1, s) : 0.0;
        const double next = k + 1 < K ? bal_time(k + 1, s) : intra_time(intrinsic[s], G, cm);
        intra = std::max(intra, fwd_prev + next);
      }
      tv += std::max(intra, c.stage_inter_us[k]);
    }
    if (K > 0) tv += c.stage_redistribute_us[K - 1];
    c.balance_per_stage_total_us = tv;
  }
  {
    // Two resources, pieces of fraction f of a stage: the NIC runs the stages back to back (stage k
    // ends at A_k); the intra-server fabric forwards stage k from the moment its first piece has
    // landed and the previous forward is done, and ends no earlier than one piece after A_k.
    const double f = std::min(1.0, std::max(cm.rail_segment_fraction, 1e-6));
    double a_prev = c.balance_us, fwd = c.balance_us + intrinsic_us, a = c.balance_us;
    for (int k = 0; k < K; ++k) {
      a = a_prev + c.stage_inter_us[k];
      const double r = c.stage_redistribute_us[k];
      if (r > 0) fwd = std::max(std::max(fwd, a_prev + f * c.stage_inter_us[k]) + r, a + f * r);
      a_prev = a;
    }
    c.chunked_total_us = std::max(a, fwd);
  }
  return c;
}

PlanChoice select_plan(const Matrix& traffic, Topology topo, const PlanOptions& base, const CostModel& cm,
                       const std::vector<PlanKind>& candidates) {
  if (candidates.empty()) throw std::invalid_argument("select_plan: no candidate kinds");
  PlanChoice best;
  bool have = false;
  std::vector<std::pair<PlanKind, double>> table;
  for (PlanKind k : candidates) {
    PlanOptions o = base;
    o.kind = k;
    Plan p = build_plan(traffic, topo, o);
    PlanCost c = model_cost(p, cm);
    table.emplace_back(k, c.total_us);
    if (!have || c.total_us < best.cost.total_us) {
      best.plan = std::move(p);
      best.cost = std::move(c);
      have = true;
    }
  }
  best.modeled_us = std::move(table);
  return best;
}

}  // namespace fastb

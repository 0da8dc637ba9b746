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
}  // namespace

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
      if (!m.empty()) t += spread_out_time(m, G, cm.intra, mb);
    }
    c.balance_us = std::max(c.balance_us, t);
  }
  double intrinsic_us = 0;
  for (int s = 0; s < S; ++s) intrinsic_us = std::max(intrinsic_us, spread_out_time(intrinsic[s], G, cm.intra, mb));

  c.stage_inter_us.assign(K, 0);
  c.stage_redistribute_us.assign(K, 0);
  for (int k = 0; k < K; ++k) {
    if (stage_max[k]) c.stage_inter_us[k] = cm.inter.alpha_us + static_cast<double>(stage_max[k]) * cm.inter.beta_us_per_mb * mb;
    for (int s = 0; s < S; ++s) {
      const auto& m = redis[static_cast<size_t>(k) * S + s];
      if (!m.empty()) c.stage_redistribute_us[k] = std::max(c.stage_redistribute_us[k], spread_out_time(m, G, cm.intra, mb));
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
  return c;
}

}  // namespace fastb

// Minimal C++ use of the scheduler library: plan a skewed all-to-all(v) for 2 servers x 4 GPUs,
// check the plan, look at its cost under a link model and lower it for one rank.
//   cmake -S . -B build/cmake && cmake --build build/cmake --target plan_example && build/cmake/plan_example
#include <cstdio>

#include "plan.h"

int main() {
  using namespace fastb;
  const Topology topo{2, 4};
  const Matrix traffic = workload_zipf_rows(topo.servers * topo.gpus, /*skew=*/1.2, /*row_total=*/64 << 20, /*seed=*/7, /*quantum=*/16);

  PlanOptions opt;                 // staged plan: balance, permutation stages, redistribution
  opt.split_align = 16;            // cut pieces on 16-unit boundaries (units are bytes here)
  const Plan plan = build_plan(traffic, topo, opt);
  const std::string err = validate_plan(plan);
  if (!err.empty()) { std::printf("invalid plan: %s\n", err.c_str()); return 1; }

  CostModel cm;                    // 400 GbE between servers, NVLink inside
  cm.inter = gbps_model(400.0, 0.7);
  cm.intra = nvlink_model(900.0, 0.1);
  cm.mb_per_unit = 1e-6;
  const PlanCost cost = model_cost(plan, cm);
  std::printf("stages %d, ops %zu, modeled %.1f us (bound %.1f us, spread-out %.1f us)\n", plan.num_stages, plan.ops.size(), cost.total_us,
              cost.lower_bound_us, cost.spread_out_us);

  // Let the cost model choose between the fan-out and the staged plan for a small message.
  const Matrix small = workload_zipf_rows(8, 1.2, 64 << 10, 7, 16);
  const PlanChoice pick = select_plan(small, topo, opt, cm, {PlanKind::kFanout, PlanKind::kStaged});
  std::printf("64 KiB rows: kind %d chosen (%.1f us)\n", static_cast<int>(pick.plan.opt.kind), pick.cost.total_us);

  LowerOptions lo;                 // work list of rank 0: one item = one CTA's copy
  lo.unit_bytes = 1;
  lo.chunk_bytes = 1 << 20;
  const RankProgram prog = lower_for_rank(plan, 0, lo);
  std::printf("rank 0: %zu work items, expects %lld output bytes\n", prog.items.size(), static_cast<long long>(prog.expect_output_bytes));
  return delivered_matrix(plan) == plan.matrix ? 0 : 1;
}

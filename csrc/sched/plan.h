// Staged transfer plan for an all-to-all(v) on a (servers x gpus_per_server) cluster.
//
// The plan is a flat list of byte-range moves ("ops"). Each op carries its provenance (which
// origin->final pair of the traffic matrix it belongs to, and where inside that pair's segment),
// so a plan can be validated, replayed on host buffers, lowered to per-GPU work lists, costed,
// and serialised without any other state.
//
// Capability parity with the reference's GlobalScheduler / LocalScheduler
// (nvidia/src/fast_alltoall/alltoall_global_scheduler.cc:243-443 flash_scheduler,
//  :649-886 ablation; alltoall_local_scheduler.cc:129-275 prepare/balance/restore;
//  buffer planning :888-1107; per-GPU lowering :1181-1821; block split :1109-1150;
//  chunk pipeline :1152-1178), without the fixed-size 20 MB result struct and its
//  GPU_NUM_PER_SERVER / MAX_SERVER_NUM / MAX_TRANSFER_STEP_NUM caps.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "decompose.h"
#include "matrix.h"

namespace fastb {

enum class Buf : uint8_t {
  kInput = 0,    // caller's send buffer (segments ordered by destination rank)
  kOutput = 1,   // caller's receive buffer (segments ordered by source rank)
  kBalance = 2,  // staging on a same-server GPU that relays part of a heavier GPU's load
  kRail = 3,     // staging on the rail GPU of the destination server, before redistribution
};

enum class Phase : uint8_t {
  kBalance = 0,       // intra-server: heavy GPU -> light GPU, before any inter-server stage
  kIntrinsic = 1,     // intra-server traffic that never leaves the server (or a direct flat op)
  kRail = 2,          // inter-server stage: GPU i of server s -> GPU i of server perm(s)
  kRedistribute = 3,  // intra-server: rail GPU -> true destination GPU
};

struct Op {
  Phase phase;
  Buf src_buf, dst_buf;
  int32_t stage;     // rail / redistribute / staged-direct: stage index; otherwise -1
  int32_t src_rank, dst_rank;
  int32_t origin, final_dst;  // the matrix pair this piece belongs to
  int64_t src_off, dst_off;   // units, relative to the named buffer of the named rank
  int64_t len;                // units
  int64_t pair_off;           // units, offset inside the origin->final segment
};

enum class PlanKind : int {
  kStaged = 0,     // balance + BvN permutation stages + redistribute (FAST)
  kSingleBurst = 1,// balance + one burst per destination server + redistribute (the "FLASH-A" ablation)
  kFanout = 2,     // every pair at once, straight into the output (NCCL-group-like)
  kSpreadOut = 3,  // n-1 ring-offset rounds
};

struct Topology {
  int servers = 1;
  int gpus = 1;  // per server
  int ranks() const { return servers * gpus; }
};

struct PlanOptions {
  PlanKind kind = PlanKind::kStaged;
  MatchPolicy match = MatchPolicy::kFirstFit;
  ScalePolicy scale_policy = ScalePolicy::kNone;
  int64_t scale = 0;        // explicit coarsening divisor; 0 = derive from scale_policy
  int64_t split_align = 1;  // units; pieces are only cut at multiples of this inside a segment
  bool transpose = false;   // plan the reverse collective (combine / backward all-to-all)
  // >= 0: keep only the ops this rank sends or receives (buffer sizes, offsets and stages are those
  // of the full plan). What one rank needs to lower and run its part; the op list of a full plan
  // grows with the cube of the server count (the reference's per-GPU view is schedule_this_gpu,
  // alltoall_global_scheduler.cc:1512-1821).
  int only_rank = -1;
  // Skip the balancing of a (server, server) tile whose transfer is latency-dominated: when the
  // beta cost of balancing + redistributing it is less than twice its alpha cost (the reference
  // simulator's check_balance_dispatch, simulation/scheduler/local.cpp:187-216). Uses `intra`.
  bool balance_alpha_beta = false;
  LinkModel inter{0.7, 22.0};  // used by ScalePolicy::kAlphaBeta only
  LinkModel intra{0.1, 1.2};
  double mb_per_unit = 1.0;
};

struct RankBuffers {
  int64_t input_units = 0, output_units = 0, balance_units = 0, rail_units = 0;
};

struct Plan {
  Topology topo;
  PlanOptions opt;
  Matrix matrix;           // as planned (already transposed if opt.transpose)
  Matrix server_matrix;    // S x S, per-rail load after balancing (ceil(tile_sum / gpus))
  Decomposition decomp;    // of server_matrix (empty for kFanout / kSpreadOut)
  int32_t num_stages = 0;  // number of distinct stage indices used by ops
  std::vector<int64_t> in_disp, out_disp;  // n x n: offset of segment [r][peer] in r's input / output
  std::vector<RankBuffers> buffers;        // per rank
  // Per rank: offset (units) in the rail staging from which the regions are no longer laid out in
  // stage order. Alignment can leave a few units behind a stage budget; they are shipped with the
  // pair's last stage but staged after everything else. Equal to rail_units when there is no such tail.
  std::vector<int64_t> rail_tail_start;
  std::vector<Op> ops;                     // global list, grouped by phase then stage
  uint64_t matrix_hash = 0;
};

Plan build_plan(const Matrix& traffic, Topology topo, const PlanOptions& opt = {});

// ---- validation -----------------------------------------------------------------------------
// Checks every op against buffer bounds, that each stage's rail ops form a partial permutation at
// server level (one peer server per server per stage), that every unit of every pair reaches the
// final output exactly once, and that staged data is forwarded completely. Returns an empty
// string when the plan is sound, else the first problem found.
std::string validate_plan(const Plan& p);

// Sum over ops that write final output, per (origin, final) pair: must equal the matrix.
Matrix delivered_matrix(const Plan& p);
// Real (non-phantom) units moved by inter-server stage k at GPU-pair granularity.
Matrix stage_matrix(const Plan& p, int stage);

// Replays the plan on host memory. inputs[r] / outputs[r] are byte buffers of
// input_units*unit_bytes / output_units*unit_bytes. `drop_op` (>=0) withholds one op, which is
// how tests model a lost message. Returns the number of output bytes written.
int64_t execute_on_host(const Plan& p, int unit_bytes, const std::vector<const uint8_t*>& inputs,
                        const std::vector<uint8_t*>& outputs, int64_t drop_op = -1);

// ---- cost model -----------------------------------------------------------------------------
// How the GPUs of one server reach each other (simulation/scheduler/config.cpp:61-179 has one
// hand-written cost function per fabric; here one routine is driven by this description).
enum class IntraTopology : int {
  kSwitch = 0,     // one port per GPU into a switch: ring-offset rounds, a round costs its slowest pair
  kFullMesh = 1,   // a dedicated link per pair: everything in flight at once
  kRing = 2,       // bidirectional ring: a transfer takes the shorter way, paying every hop
  kLinkGraph = 3,  // arbitrary point-to-point links (multiplicity matrix); unlinked pairs relay over one hop
};
struct CostModel {
  LinkModel inter{0.7, 22.0};  // defaults: 400 GbE class NIC (the reference simulator's ETHER400)
  LinkModel intra{0.1, 1.2};   // defaults: the reference simulator's B100 entry
  double mb_per_unit = 1.0;
  IntraTopology intra_topology = IntraTopology::kSwitch;
  std::vector<int> links;      // kLinkGraph: gpus x gpus link multiplicities (0 = no direct link)
  double rail_segment_fraction = 1.0 / 16;  // piece size over stage size for PlanCost::chunked_total_us
};
// Link multiplicities of the 8-GPU hybrid cube mesh (6 links per GPU, the fabric the reference's
// intra_transfer_hybrid_cude_mesh hard-codes).
std::vector<int> hybrid_cube_mesh_links();
struct PlanCost {
  double total_us = 0, balance_us = 0, inter_us = 0, exposed_intra_us = 0;
  double lower_bound_us = 0;   // busiest port (or busiest server NIC set) at full rate
  double spread_out_us = 0;    // ring-offset baseline on the same matrix
  std::vector<double> stage_inter_us, stage_redistribute_us;
  // The same plan executed with chunk-level readiness (LowerOptions::rail_segment_bytes): the
  // redistribution of a stage follows its inter-server transfer piece by piece instead of waiting
  // for the whole stage. Equal to total_us for plans without redistribution.
  double chunked_total_us = 0;
  // The same plan with the balancing spread over the stages instead of done up front (the reference
  // simulator's first pipeline variant, simulation/scheduler/global.cpp:404-529): before stage k's
  // inter-server transfer only the units stage k ships are balanced, and that balancing shares the
  // intra-server fabric with the redistribution of stage k - 1, both hidden under the inter-server
  // transfer that runs at that time. stage_balance_us[k] is the slowest server's balancing for stage k.
  double balance_per_stage_total_us = 0;
  std::vector<double> stage_balance_us;
};
// Pipeline model: balance, then stage k's inter-server transfer overlaps stage k-1's
// redistribution (simulation/scheduler/global.cpp:237-402 pipeline2). For one server per GPU
// (flat NVSwitch domain) every stage is charged to the `inter` link.
PlanCost model_cost(const Plan& p, const CostModel& cm);
// Builds one plan per candidate kind and keeps the one the cost model says finishes first (ties go
// to the earlier candidate). This is the staged-versus-fan-out switch: permutation stages pay one
// alpha each and win when the slow tier is bandwidth-bound and skewed; a single fan-out wins for
// small messages. With the kAlphaBeta scale policy in `base`, staged candidates are coarsened first.
struct PlanChoice {
  Plan plan;
  PlanCost cost;
  std::vector<std::pair<PlanKind, double>> modeled_us;  // every candidate, in the order given
};
PlanChoice select_plan(const Matrix& traffic, Topology topo, const PlanOptions& base, const CostModel& cm,
                       const std::vector<PlanKind>& candidates);
// Link model for one NVLink-5 port: alpha in us, bandwidth in GB/s.
LinkModel nvlink_model(double gbytes_per_s = 900.0, double alpha_us = 2.0);
LinkModel gbps_model(double gbit_per_s, double alpha_us);

// ---- lowering ---------------------------------------------------------------------------------
// A work item is what one CTA copies in one go.
struct WorkItem {
  int64_t src_off, dst_off, bytes;  // bytes, relative to buffer bases
  int32_t dst_rank;
  uint8_t src_buf, dst_buf;
  uint8_t wait_kind;    // 0 none, 1 wait for balance arrivals, 2 wait for rail arrivals of wait_stage
  uint8_t signal_kind;  // 1 balance counter, 2 rail counter of `stage`, 3 output counter
  int32_t stage, wait_stage;
};
struct RankProgram {
  int rank = 0;
  std::vector<WorkItem> items;              // execution order
  int64_t expect_output_bytes = 0;          // bytes that land in this rank's output
  int64_t expect_balance_bytes = 0;         // bytes that land in this rank's balance staging
  std::vector<int64_t> expect_rail_bytes;   // per stage: bytes that land in this rank's rail staging
  RankBuffers buffers_bytes;
};
struct LowerOptions {
  int unit_bytes = 1;
  int64_t chunk_bytes = 1 << 20;  // upper size of a work item
  int64_t min_chunk_bytes = 64 << 10;
  int max_chunks_per_op = 1 << 16;
  // > 0: the rail staging gets one arrival counter per this many bytes, and a forwarder waits only
  // for the pieces it reads (chunk-level readiness inside a stage). 0: one counter per stage. The
  // program then has `expect_rail_bytes.size()` counters instead of one per stage; work items name
  // them in `stage` / `wait_stage`. Pieces are coarsened until no rank needs more than
  // `max_rail_slots` counters (the size of the device signal block).
  int64_t rail_segment_bytes = 0;
  int max_rail_slots = 4096;
};
RankProgram lower_for_rank(const Plan& p, int rank, const LowerOptions& lo);

// ---- threaded host twin of the device executor ----------------------------------------------------
// Runs the lowered work lists of all ranks with `workers` threads per rank (the kernel's CTAs) for
// `epochs` consecutive collectives over the same signal words, with the device protocol's ready
// epochs, byte counters, bounded waits and counter clearing (host_threads.cc). Faults are made on
// the host: a rank that never enters, or one work item whose arrival is never counted.
struct HostRunOptions {
  int unit_bytes = 1;
  int64_t chunk_bytes = 4096;
  int64_t rail_segment_bytes = 0;  // see LowerOptions
  int workers = 3;
  int epochs = 2;
  double timeout_s = 2.0;
  int absent_rank = -1;
  int withhold_rank = -1;
  int64_t withhold_item = -1;
};
struct HostRunFailure {
  int rank = -1, site = 0;       // site: 1 entry-ready, 2 balance arrivals, 3 rail arrivals, 4 output arrivals
  int64_t detail = 0;
  uint64_t seen = 0, want = 0;
};
struct HostRunResult {
  bool ok = false;
  HostRunFailure failure;
  std::vector<std::vector<uint8_t>> outputs;  // of the last collective
};
HostRunResult run_on_host_threads(const Plan& p, const HostRunOptions& o, const std::vector<const uint8_t*>& inputs);

// ---- serialisation ------------------------------------------------------------------------------
std::string plan_to_json(const Plan& p, bool include_ops = true);
std::vector<uint8_t> plan_to_bytes(const Plan& p);
Plan plan_from_bytes(const std::vector<uint8_t>& blob);

// ---- workloads ------------------------------------------------------------------------------------
// Deterministic generators (splitmix64 stream; same output on every platform and from Python).
Matrix workload_uniform(int n, int64_t max_entry, uint64_t seed, bool zero_diag);
Matrix workload_balanced(int n, int64_t entry, bool zero_diag);
// Row i spreads `row_total` over the other ranks with weights 1/k^s assigned along a seeded
// random permutation of destinations; rounding remainders go to the heaviest destination so each
// row sums exactly; entries are multiples of `quantum`.
Matrix workload_zipf_rows(int n, double s, int64_t row_total, uint64_t seed, int64_t quantum = 1);
// Entries drawn i.i.d. from a Zipf(s) law over {1..max_entry} (the reference testers' generator,
// simulation/test.cpp:686-722), diagonal kept.
Matrix workload_zipf_entries(int n, double s, int64_t max_entry, uint64_t seed);

}  // namespace fastb

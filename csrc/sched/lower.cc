// Lowering of a global plan to the work list of one GPU.
//
// The reference lowers to per-GPU parameter blocks and splits every peer transfer evenly over the
// CTAs (alltoall_global_scheduler.cc:1109-1150) and into <=16 chunks of >=32 MiB with cumulative
// ready thresholds (:1152-1178). Here one chunk IS one CTA work item, chunks of concurrent ops are
// interleaved so that every peer of a slot is in flight at once, and ordering between phases is
// carried by byte counters (balance / per-stage rail / output) instead of per-block flags.
#include <algorithm>

#include "plan.h"

namespace fastb {

RankProgram lower_for_rank(const Plan& p, int rank, const LowerOptions& lo) {
  const int n = p.matrix.n;
  if (rank < 0 || rank >= n) throw std::invalid_argument("lower_for_rank: rank out of range");
  if (lo.unit_bytes < 1 || lo.chunk_bytes < 1) throw std::invalid_argument("lower_for_rank: bad options");
  RankProgram prog;
  prog.rank = rank;
  const int K = p.num_stages;
  prog.expect_rail_bytes.assign(K, 0);
  const int64_t ub = lo.unit_bytes;
  const RankBuffers& b = p.buffers[rank];
  prog.buffers_bytes = RankBuffers{b.input_units * ub, b.output_units * ub, b.balance_units * ub, b.rail_units * ub};

  // slot 0: balance | slot 1: rail 0, intrinsic, un-staged direct ops | slot k+1: rail k (+ staged
  // direct ops of round k) and redistribution of stage k-1 | last slot: final redistribution.
  std::vector<std::vector<const Op*>> push_slot(K + 3), fwd_slot(K + 3);
  for (const Op& o : p.ops) {
    if (o.dst_rank == rank) {
      const int64_t bytes = o.len * ub;
      if (o.dst_buf == Buf::kOutput) prog.expect_output_bytes += bytes;
      else if (o.dst_buf == Buf::kBalance) prog.expect_balance_bytes += bytes;
      else prog.expect_rail_bytes[o.stage] += bytes;
    }
    if (o.src_rank != rank) continue;
    switch (o.phase) {
      case Phase::kBalance: push_slot[0].push_back(&o); break;
      case Phase::kIntrinsic: push_slot[o.stage < 0 ? 1 : 1 + o.stage].push_back(&o); break;
      case Phase::kRail: push_slot[1 + o.stage].push_back(&o); break;
      case Phase::kRedistribute: fwd_slot[2 + o.stage].push_back(&o); break;
    }
  }
  auto chunk_of = [&](int64_t bytes) {
    int64_t c = lo.chunk_bytes;
    if (bytes / c > lo.max_chunks_per_op) c = (bytes + lo.max_chunks_per_op - 1) / lo.max_chunks_per_op;
    c = (c + 15) / 16 * 16;
    return c;
  };
  auto emit_interleaved = [&](const std::vector<const Op*>& ops) {
    // Proportional interleave: chunk j of an op with c chunks gets key (j + 1/2) / c and chunks are
    // issued in key order, so every op of the slot advances at a rate proportional to its size
    // and all of them finish together (equal ops degenerate to plain round-robin). A heavy pair
    // is then in flight from the first chunk on instead of trailing alone at the end.
    struct Slice { double key; size_t op; int64_t begin, bytes; };
    std::vector<Slice> slices;
    for (size_t k = 0; k < ops.size(); ++k) {
      const int64_t total = ops[k]->len * ub;
      const int64_t c = chunk_of(total);
      const int64_t pieces = (total + c - 1) / c;
      for (int64_t j = 0; j < pieces; ++j)
        slices.push_back(Slice{(static_cast<double>(j) + 0.5) / static_cast<double>(pieces), k, j * c, std::min(c, total - j * c)});
    }
    std::stable_sort(slices.begin(), slices.end(), [](const Slice& x, const Slice& y) { return x.key < y.key; });
    for (const Slice& sl : slices) {
      const Op& o = *ops[sl.op];
      WorkItem w{};
      w.src_off = o.src_off * ub + sl.begin;
      w.dst_off = o.dst_off * ub + sl.begin;
      w.bytes = sl.bytes;
      w.dst_rank = o.dst_rank;
      w.src_buf = static_cast<uint8_t>(o.src_buf);
      w.dst_buf = static_cast<uint8_t>(o.dst_buf);
      w.wait_kind = o.src_buf == Buf::kBalance ? 1 : o.src_buf == Buf::kRail ? 2 : 0;
      w.signal_kind = o.dst_buf == Buf::kBalance ? 1 : o.dst_buf == Buf::kRail ? 2 : 3;
      w.stage = o.stage;
      w.wait_stage = o.src_buf == Buf::kRail ? o.stage : -1;
      prog.items.push_back(w);
    }
  };
  for (int s = 0; s < K + 3; ++s) {
    emit_interleaved(push_slot[s]);
    emit_interleaved(fwd_slot[s]);
  }
  return prog;
}

}  // namespace fastb

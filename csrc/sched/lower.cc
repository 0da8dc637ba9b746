// Lowering of a global plan to the work list of one GPU.
//
// The reference lowers to per-GPU parameter blocks and splits every peer transfer evenly over the
// CTAs (alltoall_global_scheduler.cc:1109-1150) and into <=16 chunks of >=32 MiB with cumulative
// ready thresholds (:1152-1178). Here one chunk IS one CTA work item, chunks of concurrent ops are
// interleaved so that every peer of a slot is in flight at once, and ordering between phases is
// carried by byte counters (balance / per-stage rail / output) instead of per-block flags.
#include <algorithm>
#include <cstdint>

#include "plan.h"

namespace fastb {

namespace {

// Arrival counters of the rail staging. Without segments there is one per stage (slot = stage).
// With segments a rank's rail staging is cut into pieces of `seg` bytes by absolute offset and a
// piece of stage k gets the counter `offset / seg + k`, so that a forwarder waits only for the
// pieces it reads (the reference's cumulative chunk_ready_threshold,
// alltoall_global_scheduler.cc:1152-1178, without its assumption that chunks arrive in order).
// Adding the stage index keeps the counters of neighbouring stages apart even where their regions
// share a `seg`-sized window: a forward of stage k must never wait for bytes of a later stage,
// whose pushes come after it in the work lists (that would be a cycle between ranks). This relies
// on the regions lying in stage order, which holds up to Plan::rail_tail_start; what is staged
// behind it (remainders of aligned cuts, a few units per pair) gets one counter per stage instead.
// The numbering needs nothing but per-rank sizes, so a one-rank view of the plan lowers exactly
// like the full plan.
struct RailSlots {
  int64_t seg = 0, ub = 1;    // segment bytes (0 = one slot per stage); unit bytes
  int K = 0;
  const Plan* plan = nullptr;
  std::vector<int> count;     // [rank] counters of the rank

  bool in_tail(int owner, int64_t byte_off) const { return seg > 0 && byte_off >= plan->rail_tail_start[owner] * ub; }
  int ordered_slots(int owner) const { return static_cast<int>((plan->buffers[owner].rail_units * ub + seg - 1) / seg) + K; }
  int slot(int owner, int stage, int64_t byte_off) const {
    if (seg <= 0) return stage;
    return in_tail(owner, byte_off) ? ordered_slots(owner) + stage : static_cast<int>(byte_off / seg) + stage;
  }
  // End (bytes, exclusive) of the piece that contains byte_off; tail pieces are not cut.
  int64_t piece_end(int owner, int64_t byte_off) const {
    if (seg <= 0 || in_tail(owner, byte_off)) return INT64_MAX;
    return std::min((byte_off / seg + 1) * seg, plan->rail_tail_start[owner] * ub);
  }
};

RailSlots make_slots(const Plan& p, const LowerOptions& lo_opt) {
  RailSlots rs;
  const int n = p.matrix.n, K = p.num_stages;
  rs.plan = &p; rs.K = K; rs.ub = lo_opt.unit_bytes;
  rs.count.assign(n, K);
  if (lo_opt.rail_segment_bytes <= 0 || K == 0) return rs;
  int64_t widest = 0;
  for (int r = 0; r < n; ++r) widest = std::max(widest, p.buffers[r].rail_units * lo_opt.unit_bytes);
  if (widest == 0) return rs;  // nothing is staged (flat plans): nothing to segment
  rs.seg = (std::max<int64_t>(lo_opt.rail_segment_bytes, 16) + 15) / 16 * 16;
  // Every rank must fit the signal block: coarsen until the largest staging area does (never
  // below one counter per stage, plus one per stage for the tail).
  const int64_t room = std::max<int64_t>(lo_opt.max_rail_slots - 2 * K, 1);
  while ((widest + rs.seg - 1) / rs.seg > room && rs.seg < widest) rs.seg *= 2;
  for (int r = 0; r < n; ++r) rs.count[r] = rs.ordered_slots(r) + K;
  return rs;
}

}  // namespace

RankProgram lower_for_rank(const Plan& p, int rank, const LowerOptions& lo) {
  const int n = p.matrix.n;
  if (rank < 0 || rank >= n) throw std::invalid_argument("lower_for_rank: rank out of range");
  if (lo.unit_bytes < 1 || lo.chunk_bytes < 1) throw std::invalid_argument("lower_for_rank: bad options");
  RankProgram prog;
  prog.rank = rank;
  const int K = p.num_stages;
  const int64_t ub = lo.unit_bytes;
  const RailSlots slots = make_slots(p, lo);
  prog.expect_rail_bytes.assign(slots.count[rank], 0);
  const RankBuffers& b = p.buffers[rank];
  prog.buffers_bytes = RankBuffers{b.input_units * ub, b.output_units * ub, b.balance_units * ub, b.rail_units * ub};

  // A piece is the part of an op that signals (rail push) or waits for (forward) one rail slot.
  struct Piece { const Op* op; int64_t begin, bytes; int signal_slot, wait_slot; };
  auto pieces_of = [&](const Op& o, std::vector<Piece>& out) {
    const int64_t total = o.len * ub;
    const bool to_rail = o.dst_buf == Buf::kRail, from_rail = o.src_buf == Buf::kRail;
    if (slots.seg <= 0 || (!to_rail && !from_rail)) {
      out.push_back(Piece{&o, 0, total, o.stage, from_rail ? o.stage : -1});
      return;
    }
    // Cut where the rail-side offset crosses a piece boundary (a forward reads rail, a push writes it).
    const int owner = to_rail ? o.dst_rank : o.src_rank;
    const int64_t rail0 = (to_rail ? o.dst_off : o.src_off) * ub;
    int64_t done = 0;
    while (done < total) {
      const int64_t at = rail0 + done;
      const int64_t take = std::min(total - done, slots.piece_end(owner, at) - at);
      const int s = slots.slot(owner, o.stage, at);
      out.push_back(Piece{&o, done, take, to_rail ? s : o.stage, from_rail ? s : -1});
      done += take;
    }
  };

  // slot 0: balance | slot 1: rail 0, intrinsic, un-staged direct ops | slot k+1: rail k (+ staged
  // direct ops of round k) and redistribution of stage k-1 | last slot: final redistribution.
  std::vector<std::vector<Piece>> push_slot(K + 3), fwd_slot(K + 3);
  std::vector<Piece> tmp;
  for (const Op& o : p.ops) {
    if (o.dst_rank == rank) {
      const int64_t bytes = o.len * ub;
      if (o.dst_buf == Buf::kOutput) prog.expect_output_bytes += bytes;
      else if (o.dst_buf == Buf::kBalance) prog.expect_balance_bytes += bytes;
      else {
        tmp.clear();
        pieces_of(o, tmp);
        for (const Piece& pc : tmp) prog.expect_rail_bytes[pc.signal_slot] += pc.bytes;
      }
    }
    if (o.src_rank != rank) continue;
    std::vector<Piece>* dst = nullptr;
    switch (o.phase) {
      case Phase::kBalance: dst = &push_slot[0]; break;
      case Phase::kIntrinsic: dst = &push_slot[o.stage < 0 ? 1 : 1 + o.stage]; break;
      case Phase::kRail: dst = &push_slot[1 + o.stage]; break;
      case Phase::kRedistribute: dst = &fwd_slot[2 + o.stage]; break;
    }
    pieces_of(o, *dst);
  }
  auto chunk_of = [&](int64_t bytes) {
    int64_t c = lo.chunk_bytes;
    if (bytes / c > lo.max_chunks_per_op) c = (bytes + lo.max_chunks_per_op - 1) / lo.max_chunks_per_op;
    c = (c + 15) / 16 * 16;
    return c;
  };
  auto emit_interleaved = [&](const std::vector<Piece>& pcs) {
    // Proportional interleave: chunk j of a piece with c chunks gets key (j + 1/2) / c and chunks are
    // issued in key order, so every transfer of the slot advances at a rate proportional to its size
    // and all of them finish together (equal ones degenerate to plain round-robin). A heavy pair
    // is then in flight from the first chunk on instead of trailing alone at the end.
    struct Slice { double key; size_t pc; int64_t begin, bytes; };
    std::vector<Slice> slices;
    for (size_t k = 0; k < pcs.size(); ++k) {
      const int64_t total = pcs[k].bytes;
      const int64_t c = chunk_of(total);
      const int64_t pieces = (total + c - 1) / c;
      for (int64_t j = 0; j < pieces; ++j)
        slices.push_back(Slice{(static_cast<double>(j) + 0.5) / static_cast<double>(pieces), k, j * c, std::min(c, total - j * c)});
    }
    std::stable_sort(slices.begin(), slices.end(), [](const Slice& x, const Slice& y) { return x.key < y.key; });
    for (const Slice& sl : slices) {
      const Piece& pc = pcs[sl.pc];
      const Op& o = *pc.op;
      WorkItem w{};
      w.src_off = o.src_off * ub + pc.begin + sl.begin;
      w.dst_off = o.dst_off * ub + pc.begin + sl.begin;
      w.bytes = sl.bytes;
      w.dst_rank = o.dst_rank;
      w.src_buf = static_cast<uint8_t>(o.src_buf);
      w.dst_buf = static_cast<uint8_t>(o.dst_buf);
      w.wait_kind = o.src_buf == Buf::kBalance ? 1 : o.src_buf == Buf::kRail ? 2 : 0;
      w.signal_kind = o.dst_buf == Buf::kBalance ? 1 : o.dst_buf == Buf::kRail ? 2 : 3;
      w.stage = pc.signal_slot;
      w.wait_stage = pc.wait_slot;
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

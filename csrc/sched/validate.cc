// Plan validation and host replay (the CPU oracle for every executor).
#include <algorithm>
#include <cstring>
#include <sstream>

#include "plan.h"

namespace fastb {

namespace {
int64_t buf_units(const RankBuffers& b, Buf k) {
  switch (k) {
    case Buf::kInput: return b.input_units;
    case Buf::kOutput: return b.output_units;
    case Buf::kBalance: return b.balance_units;
    default: return b.rail_units;
  }
}
using Interval = std::pair<int64_t, int64_t>;  // [begin, end)

// Empty string if `iv` tiles [0, total) exactly once.
std::string tiles_exactly(std::vector<Interval>& iv, int64_t total) {
  std::sort(iv.begin(), iv.end());
  int64_t pos = 0;
  for (const Interval& x : iv) {
    if (x.first != pos) return x.first < pos ? "overlap" : "gap";
    pos = x.second;
  }
  return pos == total ? "" : "short";
}
}  // namespace

std::string validate_plan(const Plan& p) {
  const int n = p.matrix.n, G = p.topo.gpus, S = p.topo.servers;
  std::ostringstream err;
  // Structure first (a plan may come from a file): everything below indexes by these sizes.
  if (n < 0 || G < 1 || S < 1 || static_cast<int64_t>(S) * G != n) return "topology does not match the matrix";
  if (static_cast<int>(p.buffers.size()) != n) return "buffers: wrong rank count";
  if (p.in_disp.size() != static_cast<size_t>(n) * n || p.out_disp.size() != static_cast<size_t>(n) * n) return "displacement tables: wrong size";
  if (p.matrix.v.size() != static_cast<size_t>(n) * n) return "matrix: wrong size";
  if (p.num_stages < 0) return "negative stage count";
  // A decomposition of an S x S matrix has at most S^2 - 2S + 2 stages, the spread-out kind n rounds;
  // anything far beyond is a damaged header, and tables are sized by this count later on.
  if (static_cast<int64_t>(p.num_stages) > static_cast<int64_t>(S) * S + n + 2) return "stage count out of range";
  {  // no buffer of any rank can hold more than the whole traffic (sizes feed offset arithmetic later on)
    int64_t total = 0;
    for (int64_t x : p.matrix.v) {
      if (x < 0 || x > (int64_t{1} << 50)) return "matrix entry out of range";
      total += x;
      if (total > (int64_t{1} << 56)) return "matrix total out of range";
    }
    for (const RankBuffers& b : p.buffers)
      for (int64_t u : {b.input_units, b.output_units, b.balance_units, b.rail_units})
        if (u < 0 || u > total) return "buffer size out of range";
  }
  if (p.rail_tail_start.size() != static_cast<size_t>(n)) return "rail tail table: wrong size";
  for (int r = 0; r < n; ++r)
    if (p.rail_tail_start[r] < 0 || p.rail_tail_start[r] > p.buffers[r].rail_units) return "rail tail outside the staging area";
  const int only = p.opt.only_rank;  // >= 0: a one-rank view, only that rank's deliveries and staging can be complete
  if (only >= n) return "only_rank out of range";
  // Flat tables instead of maps: validation runs on every new plan, and a 512-rank plan has millions of ops.
  std::vector<std::vector<Interval>> delivered(static_cast<size_t>(n) * n);  // origin * n + final -> segment intervals
  std::vector<std::vector<Interval>> staged_w(static_cast<size_t>(n) * 2), staged_r(static_cast<size_t>(n) * 2);  // rank * 2 + (rail ? 1 : 0)
  const size_t stage_cells = p.opt.kind == PlanKind::kStaged ? static_cast<size_t>(std::max(p.num_stages, 0)) * S : 0;
  std::vector<int> stage_to(stage_cells, -1), stage_from(stage_cells, -1);   // stage * S + server -> peer server
  auto staging_slot = [](int rank, Buf b) { return static_cast<size_t>(rank) * 2 + (b == Buf::kRail ? 1 : 0); };

  for (size_t k = 0; k < p.ops.size(); ++k) {
    const Op& o = p.ops[k];
    auto bad = [&](const char* what) { err << "op " << k << ": " << what; return err.str(); };
    if (o.len <= 0) return bad("non-positive length");
    if (only >= 0 && o.src_rank != only && o.dst_rank != only) return bad("op of another rank in a one-rank view");
    if (static_cast<unsigned>(o.phase) > 3u || static_cast<unsigned>(o.src_buf) > 3u || static_cast<unsigned>(o.dst_buf) > 3u) return bad("unknown phase or buffer");
    if (o.src_rank < 0 || o.src_rank >= n || o.dst_rank < 0 || o.dst_rank >= n) return bad("rank out of range");
    if (o.origin < 0 || o.origin >= n || o.final_dst < 0 || o.final_dst >= n) return bad("pair out of range");
    if (o.src_off < 0 || o.src_off + o.len > buf_units(p.buffers[o.src_rank], o.src_buf)) return bad("source range outside its buffer");
    if (o.dst_off < 0 || o.dst_off + o.len > buf_units(p.buffers[o.dst_rank], o.dst_buf)) return bad("destination range outside its buffer");
    if (o.pair_off < 0 || o.pair_off + o.len > p.matrix.at(o.origin, o.final_dst)) return bad("piece outside its pair segment");
    if (o.src_buf == Buf::kOutput || o.dst_buf == Buf::kInput) return bad("reads output or writes input");
    // The lowering files ops by stage: none outside [-1, num_stages), staged phases never -1.
    if (o.stage < -1 || o.stage >= p.num_stages) return bad("stage out of range");
    if (o.stage < 0 && (o.phase == Phase::kRail || o.phase == Phase::kRedistribute)) return bad("stage out of range");
    if ((o.src_buf == Buf::kRail || o.dst_buf == Buf::kRail) && o.stage < 0) return bad("rail staging used outside a stage");
    const int ss = o.src_rank / G, ds = o.dst_rank / G;
    if (o.phase != Phase::kRail && p.opt.kind != PlanKind::kFanout && p.opt.kind != PlanKind::kSpreadOut && ss != ds)
      return bad("intra-server phase crosses servers");
    if (o.phase == Phase::kRail) {
      if (ss == ds) return bad("rail op inside one server");
      if (o.src_rank % G != o.dst_rank % G) return bad("rail op is not rail-aligned");
      if (o.stage < 0 || o.stage >= p.num_stages) return bad("stage out of range");
      if (p.opt.kind == PlanKind::kStaged) {
        int& to = stage_to[static_cast<size_t>(o.stage) * S + ss];
        int& from = stage_from[static_cast<size_t>(o.stage) * S + ds];
        if (to >= 0 && to != ds) return bad("server sends to two servers in one stage");
        if (from >= 0 && from != ss) return bad("server receives from two servers in one stage");
        to = ds; from = ss;
      }
    }
    if (o.src_buf == Buf::kInput) {
      if (o.src_rank != o.origin) return bad("input read on a rank that is not the origin");
      if (o.src_off != p.in_disp[static_cast<size_t>(o.origin) * n + o.final_dst] + o.pair_off) return bad("input offset does not match the pair segment");
    } else {
      staged_r[staging_slot(o.src_rank, o.src_buf)].push_back({o.src_off, o.src_off + o.len});
    }
    if (o.dst_buf == Buf::kOutput) {
      if (o.dst_rank != o.final_dst) return bad("output written on a rank that is not the final destination");
      if (o.dst_off != p.out_disp[static_cast<size_t>(o.final_dst) * n + o.origin] + o.pair_off) return bad("output offset does not match the pair segment");
      delivered[static_cast<size_t>(o.origin) * n + o.final_dst].push_back({o.pair_off, o.pair_off + o.len});
    } else {
      staged_w[staging_slot(o.dst_rank, o.dst_buf)].push_back({o.dst_off, o.dst_off + o.len});
    }
  }
  {  // up to rail_tail_start the regions of a rank's rail staging follow the stage order
    std::vector<std::vector<std::pair<int64_t, int>>> by_off(n);
    for (const Op& o : p.ops)
      if (o.dst_buf == Buf::kRail && o.dst_off < p.rail_tail_start[o.dst_rank]) by_off[o.dst_rank].push_back({o.dst_off, o.stage});
    for (int r = 0; r < n; ++r) {
      std::sort(by_off[r].begin(), by_off[r].end());
      for (size_t k = 1; k < by_off[r].size(); ++k)
        if (by_off[r][k].second < by_off[r][k - 1].second) { err << "rank " << r << ": rail staging is not in stage order before its tail"; return err.str(); }
    }
  }
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < n; ++j) {
      if (only >= 0 && j != only) continue;
      std::string r = tiles_exactly(delivered[static_cast<size_t>(i) * n + j], p.matrix.at(i, j));
      if (!r.empty()) { err << "pair " << i << "->" << j << ": delivery has a " << r; return err.str(); }
    }
  for (int r = 0; r < n; ++r)
    for (Buf b : {Buf::kBalance, Buf::kRail}) {
      if (only >= 0 && r != only) continue;
      std::vector<Interval>&w = staged_w[staging_slot(r, b)], &rd = staged_r[staging_slot(r, b)];
      std::string a = tiles_exactly(w, buf_units(p.buffers[r], b));
      if (!a.empty()) { err << "rank " << r << " staging " << static_cast<int>(b) << ": writes have a " << a; return err.str(); }
      // Reads may split a written piece, but together they must cover the same bytes once.
      a = tiles_exactly(rd, buf_units(p.buffers[r], b));
      if (!a.empty()) { err << "rank " << r << " staging " << static_cast<int>(b) << ": forwards have a " << a; return err.str(); }
    }
  return "";
}

int64_t execute_on_host(const Plan& p, int unit_bytes, const std::vector<const uint8_t*>& inputs,
                        const std::vector<uint8_t*>& outputs, int64_t drop_op) {
  const int n = p.matrix.n;
  if (static_cast<int>(inputs.size()) != n || static_cast<int>(outputs.size()) != n)
    throw std::invalid_argument("execute_on_host: one input and one output buffer per rank");
  std::vector<std::vector<uint8_t>> bal(n), rail(n);
  for (int r = 0; r < n; ++r) {
    bal[r].resize(static_cast<size_t>(p.buffers[r].balance_units) * unit_bytes);
    rail[r].resize(static_cast<size_t>(p.buffers[r].rail_units) * unit_bytes);
  }
  auto base = [&](int r, Buf b, bool write) -> uint8_t* {
    switch (b) {
      case Buf::kInput: return write ? nullptr : const_cast<uint8_t*>(inputs[r]);
      case Buf::kOutput: return outputs[r];
      case Buf::kBalance: return bal[r].data();
      default: return rail[r].data();
    }
  };
  int64_t written = 0;
  for (size_t k = 0; k < p.ops.size(); ++k) {
    if (static_cast<int64_t>(k) == drop_op) continue;
    const Op& o = p.ops[k];
    const uint8_t* s = base(o.src_rank, o.src_buf, false) + o.src_off * unit_bytes;
    uint8_t* d = base(o.dst_rank, o.dst_buf, true) + o.dst_off * unit_bytes;
    std::memcpy(d, s, static_cast<size_t>(o.len) * unit_bytes);
    if (o.dst_buf == Buf::kOutput) written += o.len * unit_bytes;
  }
  return written;
}

}  // namespace fastb

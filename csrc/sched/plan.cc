#include "plan.h"

#include <algorithm>
#include <deque>
#include <stdexcept>

namespace fastb {

namespace {

struct Piece {
  int origin_local, final_local;
  int64_t pair_off, len;
  Buf buf;
  int64_t off;  // units, inside `buf` of the GPU currently holding the piece
};

// Largest cut <= want that keeps the remainder of `p` aligned inside its segment, or the whole
// piece when want covers it.
int64_t aligned_cut(const Piece& p, int64_t want, int64_t align) {
  if (want >= p.len) return p.len;
  if (align <= 1) return want;
  const int64_t end = (p.pair_off + want) / align * align;  // absolute cut position in the segment
  return end > p.pair_off ? end - p.pair_off : 0;
}

}  // namespace

Plan build_plan(const Matrix& traffic, Topology topo, const PlanOptions& opt) {
  traffic.check_non_negative();
  if (topo.servers < 1 || topo.gpus < 1 || topo.ranks() != traffic.n)
    throw std::invalid_argument("build_plan: servers * gpus must equal the matrix dimension");
  if (opt.split_align < 1) throw std::invalid_argument("build_plan: split_align must be >= 1");

  Plan p;
  p.topo = topo;
  p.opt = opt;
  p.matrix = opt.transpose ? traffic.transposed() : traffic;
  p.matrix_hash = p.matrix.hash();
  const Matrix& M = p.matrix;
  const int n = M.n, S = topo.servers, G = topo.gpus;

  p.in_disp.assign(static_cast<size_t>(n) * n, 0);
  p.out_disp.assign(static_cast<size_t>(n) * n, 0);
  p.buffers.assign(n, RankBuffers{});
  for (int r = 0; r < n; ++r) {
    int64_t a = 0, b = 0;
    for (int q = 0; q < n; ++q) {
      p.in_disp[static_cast<size_t>(r) * n + q] = a;
      a += M.at(r, q);
      p.out_disp[static_cast<size_t>(r) * n + q] = b;
      b += M.at(q, r);
    }
    p.buffers[r].input_units = a;
    p.buffers[r].output_units = b;
  }
  auto in_at = [&](int r, int d) { return p.in_disp[static_cast<size_t>(r) * n + d]; };
  auto out_at = [&](int r, int s) { return p.out_disp[static_cast<size_t>(r) * n + s]; };
  const int only = opt.only_rank;
  if (only >= n) throw std::invalid_argument("build_plan: only_rank out of range");
  auto keep = [only](int src, int dst) { return only < 0 || src == only || dst == only; };
  auto direct = [&](int r, int d, int stage) {
    if (M.at(r, d) == 0 || !keep(r, d)) return;
    p.ops.push_back(Op{Phase::kIntrinsic, Buf::kInput, Buf::kOutput, stage, r, d, r, d, in_at(r, d),
                       out_at(d, r), M.at(r, d), 0});
  };

  p.server_matrix = Matrix(S);

  if (opt.kind == PlanKind::kFanout) {
    for (int step = 0; step < n; ++step)
      for (int r = 0; r < n; ++r) direct(r, (r + step) % n, -1);
    p.num_stages = 0;
    p.rail_tail_start.assign(n, 0);
    return p;
  }
  if (opt.kind == PlanKind::kSpreadOut) {
    for (int step = 0; step < n; ++step)
      for (int r = 0; r < n; ++r) direct(r, (r + step) % n, step);
    p.num_stages = n;
    p.rail_tail_start.assign(n, 0);
    return p;
  }

  // ---- balance: equalise the per-GPU load of every (src server, dst server) tile -------------
  // hold[(s*S+t)*G+i] = pieces GPU i of server s will put on its rail toward server t.
  std::vector<std::deque<Piece>> hold(static_cast<size_t>(S) * S * G);
  auto hold_at = [&](int s, int t, int i) -> std::deque<Piece>& { return hold[(static_cast<size_t>(s) * S + t) * G + i]; };

  for (int s = 0; s < S; ++s) {
    for (int t = 0; t < S; ++t) {
      if (s == t) continue;
      std::vector<int64_t> load(G, 0);
      int64_t sum = 0;
      for (int i = 0; i < G; ++i) {
        for (int j = 0; j < G; ++j) {
          const int64_t x = M.at(s * G + i, t * G + j);
          if (x == 0) continue;
          hold_at(s, t, i).push_back(Piece{i, j, 0, x, Buf::kInput, in_at(s * G + i, t * G + j)});
          load[i] += x;
        }
        sum += load[i];
      }
      const int64_t target = (sum + G - 1) / G;
      bool balance = G > 1;
      if (balance && opt.balance_alpha_beta) {
        double alpha = opt.intra.alpha_us;
        double beta = static_cast<double>(*std::max_element(load.begin(), load.end())) * opt.intra.beta_us_per_mb * opt.mb_per_unit;
        for (int d = 0; d < G; ++d) {
          int64_t mx = 0;
          for (int j = 0; j < G; ++j) mx = std::max(mx, M.at(s * G + j, t * G + (j + d) % G));
          if (mx) { alpha += opt.intra.alpha_us; beta += static_cast<double>(mx) * opt.intra.beta_us_per_mb * opt.mb_per_unit; }
        }
        balance = !(beta / alpha < 2.0);
      }
      for (int big = 0; big < G && balance; ++big) {
        for (int small = 0; small < G && load[big] > target; ++small) {
          if (small == big || load[small] >= target) continue;
          auto& src = hold_at(s, t, big);
          // Walk the heavy GPU's own pieces (only data still in its input buffer can be relayed).
          for (size_t k = 0; k < src.size() && load[big] > target && load[small] < target;) {
            Piece& pc = src[k];
            if (pc.buf != Buf::kInput) { ++k; continue; }
            const int64_t want = std::min(load[big] - target, target - load[small]);
            const int64_t mv = aligned_cut(pc, want, opt.split_align);
            if (mv == 0) { ++k; continue; }
            const int dst_rank = s * G + small, src_rank = s * G + big;
            int64_t& cursor = p.buffers[dst_rank].balance_units;
            if (keep(src_rank, dst_rank))
              p.ops.push_back(Op{Phase::kBalance, Buf::kInput, Buf::kBalance, -1, src_rank, dst_rank,
                                 src_rank, t * G + pc.final_local, pc.off, cursor, mv, pc.pair_off});
            hold_at(s, t, small).push_back(Piece{pc.origin_local, pc.final_local, pc.pair_off, mv, Buf::kBalance, cursor});
            cursor += mv;
            load[big] -= mv;
            load[small] += mv;
            if (mv == pc.len) {
              src.erase(src.begin() + static_cast<std::ptrdiff_t>(k));
            } else {
              pc.pair_off += mv; pc.off += mv; pc.len -= mv;
              ++k;
            }
          }
        }
      }
      p.server_matrix.at(s, t) = *std::max_element(load.begin(), load.end());
    }
  }

  // ---- intra-server traffic ---------------------------------------------------------------------
  for (int s = 0; s < S; ++s)
    for (int step = 0; step < G; ++step)
      for (int i = 0; i < G; ++i) direct(s * G + i, s * G + (i + step) % G, -1);

  // ---- inter-server stages ----------------------------------------------------------------------
  std::vector<Stage> stages;
  if (opt.kind == PlanKind::kStaged) {
    int64_t scale = opt.scale > 0 ? opt.scale
                                  : choose_scale(p.server_matrix, G, opt.scale_policy, opt.inter, opt.intra, opt.mb_per_unit);
    if (scale < 1) scale = 1;
    p.decomp = decompose(p.server_matrix, opt.match, scale);
    stages = p.decomp.stages;
  } else {  // kSingleBurst: every server pair at once, unlimited budget
    Stage all;
    all.weight = -1;
    stages.push_back(all);
  }

  std::vector<int> last_stage_of_pair(static_cast<size_t>(S) * S, -1);
  
  const int K = static_cast<int>(stages.size());
  // Rail and redistribution ops are collected per stage and concatenated at the end, so that the
  // final list is [balance][intrinsic][rail 0][redis 0][rail 1][redis 1]...
  std::vector<std::vector<Op>> rail_of_stage(K), redis_of_stage(K);

  auto emit_rail = [&](int k, int s, int t, int i, int64_t budget) {
    auto& q = hold_at(s, t, i);
    if (q.empty()) return;
    const int src_rank = s * G + i, dst_rank = t * G + i;
    std::vector<Op>& rail = rail_of_stage[k];
    std::vector<Op>& redis = redis_of_stage[k];
    while (!q.empty() && budget != 0) {
      Piece& pc = q.front();
      const int64_t take = budget < 0 ? pc.len : aligned_cut(pc, budget, opt.split_align);
      if (take == 0) break;
      const int origin = s * G + pc.origin_local, fin = t * G + pc.final_local;
      if (pc.final_local == i) {
        if (keep(src_rank, dst_rank))
          rail.push_back(Op{Phase::kRail, pc.buf, Buf::kOutput, k, src_rank, dst_rank, origin, fin, pc.off,
                            out_at(fin, origin) + pc.pair_off, take, pc.pair_off});
      } else {
        int64_t& cursor = p.buffers[dst_rank].rail_units;
        if (keep(src_rank, dst_rank))
          rail.push_back(Op{Phase::kRail, pc.buf, Buf::kRail, k, src_rank, dst_rank, origin, fin, pc.off, cursor,
                            take, pc.pair_off});
        if (keep(dst_rank, fin))
          redis.push_back(Op{Phase::kRedistribute, Buf::kRail, Buf::kOutput, k, dst_rank, fin, origin, fin, cursor,
                             out_at(fin, origin) + pc.pair_off, take, pc.pair_off});
        cursor += take;
      }
      if (budget > 0) budget -= take;
      if (take == pc.len) q.pop_front();
      else { pc.pair_off += take; pc.off += take; pc.len -= take; }
    }
  };

  for (int k = 0; k < K; ++k) {
    for (int s = 0; s < S; ++s) {
      if (opt.kind == PlanKind::kStaged) {
        const int t = stages[k].to[s];
        if (t == s) continue;
        last_stage_of_pair[static_cast<size_t>(s) * S + t] = k;
        for (int i = 0; i < G; ++i) emit_rail(k, s, t, i, stages[k].weight);
      } else {
        for (int step = 1; step < S; ++step) {
          const int t = (s + step) % S;
          for (int i = 0; i < G; ++i) emit_rail(k, s, t, i, -1);
        }
      }
    }
  }
  p.rail_tail_start.resize(n);
  for (int r = 0; r < n; ++r) p.rail_tail_start[r] = p.buffers[r].rail_units;  // up to here regions follow the stage order
  // Alignment can leave a few units behind a stage budget; ship them with the pair's last stage.
  if (opt.kind == PlanKind::kStaged) {
    for (int s = 0; s < S; ++s)
      for (int t = 0; t < S; ++t) {
        if (s == t) continue;
        for (int i = 0; i < G; ++i) {
          if (hold_at(s, t, i).empty()) continue;
          const int k = last_stage_of_pair[static_cast<size_t>(s) * S + t];
          if (k < 0) throw std::logic_error("build_plan: traffic left without a stage");
          emit_rail(k, s, t, i, -1);
        }
      }
  }
  size_t total = p.ops.size();
  for (int k = 0; k < K; ++k) total += rail_of_stage[k].size() + redis_of_stage[k].size();
  p.ops.reserve(total);
  for (int k = 0; k < K; ++k) {
    p.ops.insert(p.ops.end(), rail_of_stage[k].begin(), rail_of_stage[k].end());
    p.ops.insert(p.ops.end(), redis_of_stage[k].begin(), redis_of_stage[k].end());
    std::vector<Op>().swap(rail_of_stage[k]);
    std::vector<Op>().swap(redis_of_stage[k]);
  }
  p.num_stages = K;
  return p;
}

Matrix delivered_matrix(const Plan& p) {
  Matrix d(p.matrix.n);
  for (const Op& o : p.ops)
    if (o.dst_buf == Buf::kOutput) d.at(o.origin, o.final_dst) += o.len;
  return d;
}

Matrix stage_matrix(const Plan& p, int stage) {
  Matrix d(p.matrix.n);
  for (const Op& o : p.ops)
    if (o.stage == stage && (o.phase == Phase::kRail || (o.phase == Phase::kIntrinsic && o.stage >= 0)))
      d.at(o.src_rank, o.dst_rank) += o.len;
  return d;
}

}  // namespace fastb

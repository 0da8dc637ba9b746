// Native self-check of the scheduler library (no Python, no GPU): random matrices over a range of
// topologies; every plan must validate, deliver the matrix exactly, survive a binary round trip
// and replay bit-exactly on host buffers. Exit code 0 = all good. Mirrors the role of the
// reference's DecompositionTester (simulation/test.cpp:15-60) for the whole planner.
#include <cstdio>
#include <cstring>
#include <vector>

#include "../kernels/tile_walker.h"
#include "../runtime/range_allocator.h"
#include "plan.h"

using namespace fastb;

static int failures = 0;
#define CHECK(cond, ...)                                   \
  do {                                                     \
    if (!(cond)) { ++failures; std::printf("FAIL %s:%d: ", __FILE__, __LINE__); std::printf(__VA_ARGS__); std::printf("\n"); } \
  } while (0)

static void replay_check(const Plan& p, int unit_bytes, uint64_t seed) {
  const int n = p.matrix.n;
  std::vector<std::vector<uint8_t>> in(n), out(n);
  std::vector<const uint8_t*> ip;
  std::vector<uint8_t*> op;
  uint64_t x = seed * 0x9e3779b97f4a7c15ull + 1;
  for (int r = 0; r < n; ++r) {
    in[r].resize(static_cast<size_t>(p.buffers[r].input_units) * unit_bytes);
    out[r].assign(static_cast<size_t>(p.buffers[r].output_units) * unit_bytes, 0xEE);
    for (auto& b : in[r]) { x = x * 6364136223846793005ull + 1442695040888963407ull; b = static_cast<uint8_t>(x >> 56); }
    ip.push_back(in[r].data());
    op.push_back(out[r].data());
  }
  const int64_t written = execute_on_host(p, unit_bytes, ip, op);
  CHECK(written == p.matrix.total() * unit_bytes, "replay wrote %lld bytes, matrix has %lld", static_cast<long long>(written), static_cast<long long>(p.matrix.total() * unit_bytes));
  for (int d = 0; d < n; ++d)
    for (int s = 0; s < n; ++s) {
      const int64_t len = p.matrix.at(s, d) * unit_bytes;
      const uint8_t* a = in[s].data() + p.in_disp[static_cast<size_t>(s) * n + d] * unit_bytes;
      const uint8_t* b = out[d].data() + p.out_disp[static_cast<size_t>(d) * n + s] * unit_bytes;
      CHECK(len == 0 || std::memcmp(a, b, static_cast<size_t>(len)) == 0, "segment %d->%d differs", s, d);
    }
}

// The symmetric-heap allocator: deterministic offsets, alignment, coalescing, exhaustion.
static void allocator_check() {
  RangeAllocator a(1 << 20), b(1 << 20);
  std::vector<size_t> offs;
  uint64_t x = 12345;
  for (int i = 0; i < 2000; ++i) {
    x = x * 6364136223846793005ull + 1442695040888963407ull;
    if (offs.empty() || (x >> 60) < 10) {
      const size_t sz = (x >> 20) % 5000;
      try {
        const size_t oa = a.alloc(sz), ob = b.alloc(sz);
        CHECK(oa == ob && oa % 256 == 0, "allocator offsets differ or are unaligned");
        offs.push_back(oa);
      } catch (const std::runtime_error&) {
        bool threw = false;
        try { b.alloc(sz); } catch (const std::runtime_error&) { threw = true; }
        CHECK(threw, "exhaustion must be deterministic");
      }
    } else {
      const size_t k = (x >> 30) % offs.size();
      a.free(offs[k]); b.free(offs[k]);
      offs.erase(offs.begin() + static_cast<std::ptrdiff_t>(k));
    }
    CHECK(a.in_use() == b.in_use() && a.live_blocks() == offs.size(), "allocator bookkeeping");
  }
  for (size_t o : offs) { a.free(o); b.free(o); }
  CHECK(a.pristine() && b.pristine(), "free list must coalesce back to one block");
  bool threw = false;
  try { a.free(512); } catch (const std::invalid_argument&) { threw = true; }
  CHECK(threw, "freeing an unknown offset must be refused");
  threw = false;
  try { a.alloc((1 << 20) + 1); } catch (const std::runtime_error&) { threw = true; }
  CHECK(threw, "over-capacity request must be refused");
}

// The grouped GEMMs' tile enumeration: every role of every CTA steps its own walker by the grid
// stride; together they must visit every tile of every group exactly once, in bands, with the
// right reduction length, and stop after the last tile.
template <int TILE_M>
static void walker_check() {
  using fastb::gemm::TileCoord;
  using fastb::gemm::TileWalker;
  uint64_t x = 0x9e3779b97f4a7c15ull + TILE_M;
  auto rnd = [&](int m) { x ^= x << 13; x ^= x >> 7; x ^= x << 17; return static_cast<int>(x % static_cast<uint64_t>(m)); };
  for (int trial = 0; trial < 400; ++trial) {
    const int G = 1 + rnd(9), tiles_n = 1 + rnd(7), fixed_m = 1 + rnd(5), stride = 1 + rnd(40);
    const bool wgrad = trial % 3 == 2;
    const int band_rows = trial % 4 == 0 ? 0 : TILE_M * (1 + rnd(6));
    std::vector<int> off(G + 1, 0);
    for (int g = 0; g < G; ++g) off[g + 1] = off[g] + (rnd(4) == 0 ? 0 : TILE_M * (1 + rnd(40)));  // empty groups included
    const int red_len = 64 * (1 + rnd(8));
    long long want = 0;
    std::vector<long long> first(G + 1, 0);
    for (int g = 0; g < G; ++g) { first[g] = want; want += static_cast<long long>(wgrad ? fixed_m : (off[g + 1] - off[g]) / TILE_M) * tiles_n; }
    std::vector<int> seen(static_cast<size_t>(want), 0);
    for (int cta = 0; cta < stride; ++cta) {
      TileWalker<TILE_M> w{off.data(), G, tiles_n, fixed_m, red_len, wgrad, band_rows};
      TileCoord c{};
      int tile = cta;
      for (; w.locate(tile, c); tile += stride) {
        const int mt = wgrad ? fixed_m : (off[c.g + 1] - off[c.g]) / TILE_M;
        CHECK(c.g >= 0 && c.g < G && c.m_idx >= 0 && c.m_idx < mt && c.n_idx >= 0 && c.n_idx < tiles_n, "walker: coordinate out of range");
        CHECK(c.row0 == off[c.g], "walker: row0");
        CHECK(c.red_blocks == (wgrad ? (off[c.g + 1] - off[c.g]) / 64 : red_len / 64), "walker: reduction length");
        const long long id = first[c.g] + static_cast<long long>(c.m_idx) * tiles_n + c.n_idx;
        CHECK(id >= 0 && id < want, "walker: tile id");
        if (id >= 0 && id < want) ++seen[static_cast<size_t>(id)];
        // Band order: tiles of a band come before tiles of the next band of the same group.
        const int kb = (band_rows > 0 ? band_rows : fastb::gemm::kDefaultBandRows) / TILE_M > 1 ? (band_rows > 0 ? band_rows : fastb::gemm::kDefaultBandRows) / TILE_M : 1;
        const long long local = tile - first[c.g];
        CHECK(c.m_idx / kb == local / (static_cast<long long>(kb) * tiles_n), "walker: band order");
      }
      CHECK(tile >= want, "walker: stopped early");
    }
    for (long long i = 0; i < want; ++i) CHECK(seen[static_cast<size_t>(i)] == 1, "walker: tile %lld visited %d times", i, seen[static_cast<size_t>(i)]);
  }
}

int main() {
  allocator_check();
  walker_check<128>();
  walker_check<256>();
  const int topo[][2] = {{1, 1}, {1, 4}, {4, 1}, {2, 2}, {2, 4}, {3, 3}, {8, 1}, {4, 2}};
  const PlanKind kinds[] = {PlanKind::kStaged, PlanKind::kSingleBurst, PlanKind::kFanout, PlanKind::kSpreadOut};
  int plans = 0;
  for (auto& t : topo) {
    const int S = t[0], G = t[1], n = S * G;
    for (uint64_t seed = 0; seed < 6; ++seed) {
      Matrix m = seed % 3 == 2 && n > 1 ? workload_zipf_rows(n, 1.2, 50000, seed, 4) : workload_uniform(n, 400, seed * 7 + n, seed % 2 == 1);
      Decomposition d = decompose(m, seed % 2 ? MatchPolicy::kBottleneck : MatchPolicy::kFirstFit, 1);
      CHECK(verify_decomposition(d), "decomposition not exact (n=%d seed=%llu)", n, static_cast<unsigned long long>(seed));
      CHECK(d.line_sum == m.max_line_sum(), "line sum mismatch");
      for (PlanKind k : kinds)
        for (int64_t align : {int64_t{1}, int64_t{16}}) {
          PlanOptions o;
          o.kind = k; o.split_align = align; o.transpose = seed % 2 == 0;
          Plan p = build_plan(m, Topology{S, G}, o);
          const std::string err = validate_plan(p);
          CHECK(err.empty(), "invalid plan S=%d G=%d kind=%d: %s", S, G, static_cast<int>(k), err.c_str());
          CHECK(delivered_matrix(p) == p.matrix, "delivery differs from the matrix");
          Plan q = plan_from_bytes(plan_to_bytes(p));
          CHECK(validate_plan(q).empty() && q.ops.size() == p.ops.size() && q.matrix_hash == p.matrix_hash, "binary round trip");
          replay_check(p, 3, seed);
          for (int r = 0; r < n; ++r) {
            LowerOptions lo; lo.unit_bytes = 2; lo.chunk_bytes = 256;
            RankProgram g = lower_for_rank(p, r, lo);
            int64_t sent = 0;
            for (const WorkItem& w : g.items) sent += w.bytes;
            int64_t want = 0;
            for (const Op& op : p.ops) if (op.src_rank == r) want += op.len * 2;
            CHECK(sent == want, "lowering lost bytes on rank %d", r);
            CHECK(g.expect_output_bytes == p.matrix.col_sum(r) * 2, "expected output bytes on rank %d", r);
          }
          ++plans;
        }
    }
  }
  {  // the selector returns the cheapest candidate under the model and lists all of them
    Matrix m = workload_zipf_rows(16, 1.2, 1 << 26, 3, 16);
    CostModel cm; cm.mb_per_unit = 1e-6;
    PlanChoice ch = select_plan(m, Topology{4, 4}, PlanOptions{}, cm, {PlanKind::kFanout, PlanKind::kStaged, PlanKind::kSingleBurst});
    CHECK(ch.modeled_us.size() == 3, "selector table size");
    double best = ch.modeled_us[0].second;
    for (auto& kv : ch.modeled_us) best = std::min(best, kv.second);
    CHECK(ch.cost.total_us == best && validate_plan(ch.plan).empty() && delivered_matrix(ch.plan) == ch.plan.matrix, "selector choice");
    ++plans;
  }
  std::printf("{\"selfcheck\":\"sched\",\"plans\":%d,\"failures\":%d}\n", plans, failures);
  return failures ? 1 : 0;
}

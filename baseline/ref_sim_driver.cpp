// Driver around the UNMODIFIED reference simulator sources (simulation/algorithm, simulation/scheduler):
// reads "servers gpus inter_alpha inter_beta intra_alpha intra_beta mb_per_unit" and the n*n matrix
// from stdin, runs the reference's own SDSM + Birkhoff decomposition and its pipeline / pipeline2 / pipeline3 cost models,
// and prints one JSON line. Built by baseline/build_ref_sim.sh with
// `-include cstring -include cstdint` (the reference omits those headers); nothing of the
// reference is copied into this repository.
#include <chrono>
#include <cstdio>
#include <vector>

#include "algorithm/all2all.h"
#include "scheduler/config.h"
#include "scheduler/global.h"
#include "scheduler/local.h"

int main() {
  unsigned S, G;
  double ia, ib, ja, jb, mbpu;
  if (scanf("%u %u %lf %lf %lf %lf %lf", &S, &G, &ia, &ib, &ja, &jb, &mbpu) != 7) return 2;
  const unsigned n = S * G;
  std::vector<uint> m(static_cast<size_t>(n) * n);
  for (auto& x : m) if (scanf("%u", &x) != 1) return 2;
  struct link_info_t inter = {0, ia, ib}, intra = {0, ja, jb};
  std::vector<LocalScheduler*> locals;
  for (unsigned s = 0; s < S; ++s) locals.push_back(new LocalScheduler(m.data() + static_cast<size_t>(s) * G * n, G, S, s, intra));
  GlobalScheduler gs(S, G, locals, inter, intra, false, mbpu);
  // Server matrix as the reference builds it, for its own decomposition.
  std::vector<uint> sm(static_cast<size_t>(S) * S);
  for (unsigned s = 0; s < S; ++s) for (unsigned t = 0; t < S; ++t) sm[s * S + t] = locals[s]->server2server_data[t];
  Matrix mat;
  mat.copy(sm.data(), S);
  FastAll2All a2a(&mat, G);
  auto t0 = std::chrono::steady_clock::now();
  a2a.to_scaled_doubly_stochastic_matrix();
  a2a.decompose();
  auto t1 = std::chrono::steady_clock::now();
  unsigned long long freq_sum = 0;
  for (auto& p : a2a.p_sets) freq_sum += p.get_freq();
  const bool exact = a2a.verify_decomposition();
  struct pipeline_result_t r = gs.pipeline2(mbpu);
  // pipeline3 = pipeline2 with a pluggable intra-server fabric cost; it consumes the schedulers'
  // state, so each call gets a fresh set.
  auto with_fabric = [&](intra_transfer_topo_fn fn) {
    std::vector<LocalScheduler*> ls;
    for (unsigned s = 0; s < S; ++s) ls.push_back(new LocalScheduler(m.data() + static_cast<size_t>(s) * G * n, G, S, s, intra));
    GlobalScheduler g3(S, G, ls, inter, intra, false, mbpu);
    return g3.pipeline3(mbpu, fn).t;
  };
  const double full_mesh = with_fabric(&intra_transfer_full_mesh);
  const double ring2 = G == 8 ? with_fabric(&intra_transfer_2ring) : -1.0;
  const double cube = G == 8 ? with_fabric(&intra_transfer_hybrid_cude_mesh) : -1.0;
  // pipeline = the first variant: balance per stage instead of once up front. Fresh schedulers again.
  double pipeline1 = -1.0;
  {
    std::vector<LocalScheduler*> ls;
    for (unsigned s = 0; s < S; ++s) ls.push_back(new LocalScheduler(m.data() + static_cast<size_t>(s) * G * n, G, S, s, intra));
    GlobalScheduler g1(S, G, ls, inter, intra, false, mbpu);
    pipeline1 = g1.pipeline(mbpu).t;
  }
  const double spread = spread_out_baseline(m.data(), S, G, inter, intra, mbpu);
  printf("{\"stages\":%zu,\"freq_sum\":%llu,\"exact\":%s,\"decompose_us\":%.2f,\"pipeline2_us\":%.4f,\"spread_out_us\":%.4f,"
         "\"pipeline1_us\":%.4f,\"pipeline3_full_mesh_us\":%.4f,\"pipeline3_2ring_us\":%.4f,\"pipeline3_hybrid_cube_mesh_us\":%.4f}\n", a2a.p_sets.size(), freq_sum,
         exact ? "true" : "false", std::chrono::duration<double, std::micro>(t1 - t0).count(), r.t, spread, pipeline1, full_mesh, ring2, cube);
  return 0;
}

// Race check of the executor protocol: runs the threaded host twin (host_threads.cc) over a set
// of topologies and plan kinds, several workers per rank and several collectives in a row, and
// compares every output with the sequential replay. Meant to be built with -fsanitize=thread
// (build/fastb-twin-tsan): ThreadSanitizer then reports any payload access that is not ordered by
// the protocol's release / acquire pairs. Also runs without the sanitizer as a plain stress test.
#include <cstdio>
#include <cstdlib>

#include "plan.h"

using namespace fastb;

int main(int argc, char** argv) {
  const int rounds = argc > 1 ? std::atoi(argv[1]) : 2;
  const int topo[][2] = {{4, 1}, {8, 1}, {2, 2}, {2, 4}, {3, 2}, {1, 4}};
  const PlanKind kinds[] = {PlanKind::kStaged, PlanKind::kSingleBurst, PlanKind::kFanout, PlanKind::kSpreadOut};
  int runs = 0, failures = 0;
  for (int round = 0; round < rounds; ++round)
    for (auto& t : topo)
      for (PlanKind k : kinds) {
        const int S = t[0], G = t[1], n = S * G;
        Matrix m = (round + n) % 2 ? workload_zipf_rows(n, 1.2, 20000, 17 * round + n, 4) : workload_uniform(n, 300, 31 * round + n, round % 2 == 1);
        PlanOptions po; po.kind = k; po.split_align = round % 2 ? 4 : 1; po.transpose = round % 2 == 1;
        Plan p = build_plan(m, Topology{S, G}, po);
        const int unit = 3;
        std::vector<std::vector<uint8_t>> in(n), want(n);
        std::vector<const uint8_t*> ip; std::vector<uint8_t*> wp;
        uint64_t x = 88172645463325252ull + runs;
        for (int r = 0; r < n; ++r) {
          in[r].resize(static_cast<size_t>(p.buffers[r].input_units) * unit);
          for (auto& b : in[r]) { x ^= x << 13; x ^= x >> 7; x ^= x << 17; b = static_cast<uint8_t>(x); }
          want[r].assign(static_cast<size_t>(p.buffers[r].output_units) * unit, 0);
          ip.push_back(in[r].data()); wp.push_back(want[r].data());
        }
        execute_on_host(p, unit, ip, wp);
        HostRunOptions o; o.unit_bytes = unit; o.chunk_bytes = 192; o.workers = 2 + runs % 3; o.epochs = 3; o.timeout_s = 20.0;
        o.rail_segment_bytes = runs % 2 ? 256 : 0;  // every other run: one arrival counter per 256 bytes of rail staging
        HostRunResult res = run_on_host_threads(p, o, ip);
        ++runs;
        bool same = res.ok;
        for (int r = 0; r < n && same; ++r) same = res.outputs[r] == want[r];
        if (!same) {
          ++failures;
          std::printf("FAIL S=%d G=%d kind=%d round=%d: ok=%d rank=%d site=%d\n", S, G, static_cast<int>(k), round, res.ok ? 1 : 0, res.failure.rank, res.failure.site);
        }
      }
  std::printf("{\"twin_check\":\"a2a protocol\",\"runs\":%d,\"failures\":%d}\n", runs, failures);
  return failures ? 1 : 0;
}

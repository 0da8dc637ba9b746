// Mutation fuzzer of the plan file format: every damaged blob must either fail to parse, fail
// validation, or be a sound plan that lowers, costs and prints without touching memory it does
// not own. Meant for the AddressSanitizer build (-DFASTB_ASAN=ON); also runs plain.
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include "plan.h"
using namespace fastb;
int main(int argc, char** argv) {
  const int rounds = argc > 1 ? std::atoi(argv[1]) : 3000;
  uint64_t x = 12345;
  auto rnd = [&]() { x ^= x << 13; x ^= x >> 7; x ^= x << 17; return x; };
  int parsed = 0, valid = 0, threw = 0;
  for (int base = 0; base < 6; ++base) {
    const int S = 1 + base % 4, G = 1 + (base * 7) % 4;
    Matrix m = workload_uniform(S * G, 200, base, false);
    PlanOptions o; o.split_align = base % 2 ? 4 : 1; o.kind = static_cast<PlanKind>(base % 4);
    Plan p = build_plan(m, Topology{S, G}, o);
    std::vector<uint8_t> blob = plan_to_bytes(p);
    for (int t = 0; t < rounds; ++t) {
      std::vector<uint8_t> b = blob;
      const int edits = 1 + rnd() % 3;
      for (int e = 0; e < edits; ++e) {
        const size_t pos = rnd() % b.size();
        switch (rnd() % 4) {
          case 0: b[pos] ^= static_cast<uint8_t>(1u << (rnd() % 8)); break;
          case 1: { int64_t v = static_cast<int64_t>(rnd()); if (pos + 8 <= b.size()) std::memcpy(&b[pos], &v, 8); break; }
          case 2: { int32_t v = static_cast<int32_t>(rnd() % 11) - 5; if (pos + 4 <= b.size()) std::memcpy(&b[pos], &v, 4); break; }
          default: b.resize(pos); break;
        }
        if (b.empty()) break;
      }
      try {
        Plan q = plan_from_bytes(b);
        ++parsed;
        if (validate_plan(q).empty()) {
          ++valid;
          LowerOptions lo; lo.unit_bytes = 2; lo.chunk_bytes = 64; lo.rail_segment_bytes = t % 2 ? 48 : 0;
          for (int r = 0; r < q.matrix.n; ++r) (void)lower_for_rank(q, r, lo);
          (void)delivered_matrix(q);
          CostModel cm; (void)model_cost(q, cm);
          (void)plan_to_json(q, true);
        }
      } catch (const std::exception&) { ++threw; }
    }
  }
  std::printf("{\"fuzz\":\"plan blobs\",\"parsed\":%d,\"valid\":%d,\"rejected_at_parse\":%d}\n", parsed, valid, threw);
  return 0;
}

// Seeded traffic-matrix generators shared by the simulator, the tests and the benches.
#include <algorithm>
#include <cmath>
#include <numeric>

#include "plan.h"

namespace fastb {

namespace {
struct SplitMix64 {
  uint64_t s;
  explicit SplitMix64(uint64_t seed) : s(seed) {}
  uint64_t next() {
    uint64_t z = (s += 0x9e3779b97f4a7c15ull);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
  }
  double unit() { return static_cast<double>(next() >> 11) * (1.0 / 9007199254740992.0); }
  uint64_t below(uint64_t m) { return m ? next() % m : 0; }
};
}  // namespace

Matrix workload_uniform(int n, int64_t max_entry, uint64_t seed, bool zero_diag) {
  Matrix m(n);
  SplitMix64 g(seed);
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < n; ++j) {
      int64_t x = static_cast<int64_t>(g.below(static_cast<uint64_t>(max_entry) + 1));
      m.at(i, j) = (zero_diag && i == j) ? 0 : x;
    }
  return m;
}

Matrix workload_balanced(int n, int64_t entry, bool zero_diag) {
  Matrix m(n);
  for (int i = 0; i < n; ++i)
    for (int j = 0; j < n; ++j) m.at(i, j) = (zero_diag && i == j) ? 0 : entry;
  return m;
}

Matrix workload_zipf_rows(int n, double s, int64_t row_total, uint64_t seed, int64_t quantum) {
  Matrix m(n);
  if (n < 2) return m;
  if (quantum < 1) quantum = 1;
  SplitMix64 g(seed);
  std::vector<double> w(n - 1);
  double wsum = 0;
  for (int k = 0; k < n - 1; ++k) { w[k] = 1.0 / std::pow(static_cast<double>(k + 1), s); wsum += w[k]; }
  for (int i = 0; i < n; ++i) {
    std::vector<int> dst;
    for (int j = 0; j < n; ++j) if (j != i) dst.push_back(j);
    for (int k = n - 2; k > 0; --k) std::swap(dst[k], dst[g.below(static_cast<uint64_t>(k) + 1)]);
    int64_t used = 0;
    for (int k = 0; k < n - 1; ++k) {
      int64_t x = static_cast<int64_t>(static_cast<double>(row_total) * (w[k] / wsum)) / quantum * quantum;
      m.at(i, dst[k]) = x;
      used += x;
    }
    m.at(i, dst[0]) += row_total - used;  // heaviest destination absorbs the rounding remainder
  }
  return m;
}

Matrix workload_zipf_entries(int n, double s, int64_t max_entry, uint64_t seed) {
  // Inverse-CDF sampling on the exact discrete law (tabulated once; max_entry is small).
  Matrix m(n);
  SplitMix64 g(seed);
  std::vector<double> cdf(static_cast<size_t>(max_entry));
  double acc = 0;
  for (int64_t k = 1; k <= max_entry; ++k) { acc += 1.0 / std::pow(static_cast<double>(k), s); cdf[k - 1] = acc; }
  for (auto& x : m.v) {
    const double u = g.unit() * acc;
    x = static_cast<int64_t>(std::lower_bound(cdf.begin(), cdf.end(), u) - cdf.begin()) + 1;
  }
  return m;
}

}  // namespace fastb

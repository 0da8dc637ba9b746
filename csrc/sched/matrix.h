// Dense square traffic matrix of signed 64-bit entries (units or bytes).
//
// Entry (i, j) is the amount rank i sends to rank j; rank = server * gpus_per_server + local.
// Covers what the reference's Matrix struct provides (nvidia/src/fast_alltoall/alltoall_matrix.cc:14-263:
// get/set/add/sub, ceil-divide "scale", max row/column sum, doubly-stochastic test) as a small
// value type over one flat vector, with no bounds logging and no heap churn per call.
#pragma once
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

namespace fastb {

struct Matrix {
  int n = 0;
  std::vector<int64_t> v;

  Matrix() = default;
  explicit Matrix(int dim) : n(dim), v(static_cast<size_t>(dim) * dim, 0) {}
  Matrix(int dim, const int64_t* data) : n(dim), v(data, data + static_cast<size_t>(dim) * dim) {}

  int64_t& at(int i, int j) { return v[static_cast<size_t>(i) * n + j]; }
  int64_t at(int i, int j) const { return v[static_cast<size_t>(i) * n + j]; }

  int64_t row_sum(int i) const {
    int64_t s = 0;
    for (int j = 0; j < n; ++j) s += at(i, j);
    return s;
  }
  int64_t col_sum(int j) const {
    int64_t s = 0;
    for (int i = 0; i < n; ++i) s += at(i, j);
    return s;
  }
  int64_t total() const {
    int64_t s = 0;
    for (int64_t x : v) s += x;
    return s;
  }
  // Largest row or column sum: the per-port lower bound of any schedule, in matrix units.
  int64_t max_line_sum() const {
    int64_t m = 0;
    for (int i = 0; i < n; ++i) {
      int64_t r = row_sum(i), c = col_sum(i);
      if (r > m) m = r;
      if (c > m) m = c;
    }
    return m;
  }
  // True when every row and every column sums to the same value.
  bool is_doubly_stochastic() const {
    int64_t m = max_line_sum();
    for (int i = 0; i < n; ++i)
      if (row_sum(i) != m || col_sum(i) != m) return false;
    return true;
  }
  Matrix transposed() const {
    Matrix t(n);
    for (int i = 0; i < n; ++i)
      for (int j = 0; j < n; ++j) t.at(j, i) = at(i, j);
    return t;
  }
  // Ceil-divide every entry (the coarsening step of alpha-beta scaling).
  Matrix ceil_div(int64_t f) const {
    Matrix r(n);
    for (size_t k = 0; k < v.size(); ++k) r.v[k] = (v[k] + f - 1) / f;
    return r;
  }
  bool operator==(const Matrix& o) const { return n == o.n && v == o.v; }
  void check_non_negative() const {
    for (int64_t x : v)
      if (x < 0) throw std::invalid_argument("traffic matrix has a negative entry");
  }
  // FNV-1a over the entries; identical matrices on every rank give identical hashes, so ranks
  // can compare hashes before trusting that they planned the same collective.
  uint64_t hash() const {
    uint64_t h = 1469598103934665603ull ^ static_cast<uint64_t>(n);
    for (int64_t x : v) {
      uint64_t u = static_cast<uint64_t>(x);
      for (int b = 0; b < 8; ++b) {
        h ^= (u >> (8 * b)) & 0xff;
        h *= 1099511628211ull;
      }
    }
    return h;
  }
};

}  // namespace fastb

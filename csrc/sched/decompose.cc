#include "decompose.h"

#include <algorithm>
#include <stdexcept>

namespace fastb {

Matrix pad_to_doubly_stochastic(Matrix& m) {
  const int n = m.n;
  Matrix pad(n);
  const int64_t target = m.max_line_sum();
  std::vector<int64_t> rdef(n), cdef(n);
  for (int i = 0; i < n; ++i) {
    rdef[i] = target - m.row_sum(i);
    cdef[i] = target - m.col_sum(i);
  }
  // North-west-corner fill: total row deficit == total column deficit, so two cursors meet at
  // the end and at most 2n-1 entries are touched.
  int i = 0, j = 0;
  while (i < n && j < n) {
    if (rdef[i] == 0) { ++i; continue; }
    if (cdef[j] == 0) { ++j; continue; }
    const int64_t d = std::min(rdef[i], cdef[j]);
    pad.at(i, j) += d;
    m.at(i, j) += d;
    rdef[i] -= d;
    cdef[j] -= d;
  }
  return pad;
}

namespace {

// Bipartite matching over the positive entries of a matrix, rows on the left.
class Matcher {
 public:
  explicit Matcher(int n) : n_(n), words_((n + 63) / 64), adj_(static_cast<size_t>(n) * words_, 0),
                            row_to_col_(n, -1), col_to_row_(n, -1), seen_(words_) {}

  void set_edges(const Matrix& m, int64_t threshold) {
    std::fill(adj_.begin(), adj_.end(), 0);
    for (int i = 0; i < n_; ++i)
      for (int j = 0; j < n_; ++j)
        if (m.at(i, j) >= threshold && m.at(i, j) > 0) adj_[i * words_ + (j >> 6)] |= 1ull << (j & 63);
  }
  void remove_edge(int i, int j) { adj_[i * words_ + (j >> 6)] &= ~(1ull << (j & 63)); }
  void unmatch_row(int i) {
    int j = row_to_col_[i];
    if (j >= 0) { col_to_row_[j] = -1; row_to_col_[i] = -1; }
  }
  void clear_matching() {
    std::fill(row_to_col_.begin(), row_to_col_.end(), -1);
    std::fill(col_to_row_.begin(), col_to_row_.end(), -1);
  }
  // Augments every unmatched row; returns the matching size.
  int solve() {
    int size = 0;
    for (int i = 0; i < n_; ++i) {
      if (row_to_col_[i] >= 0) { ++size; continue; }
      std::fill(seen_.begin(), seen_.end(), 0);
      if (augment(i)) ++size;
    }
    return size;
  }
  const std::vector<int>& row_to_col() const { return row_to_col_; }

 private:
  bool augment(int i) {
    const uint64_t* row = &adj_[static_cast<size_t>(i) * words_];
    // First pass: a free column reachable directly.
    for (int w = 0; w < words_; ++w) {
      uint64_t cand = row[w] & ~seen_[w];
      while (cand) {
        int j = (w << 6) + __builtin_ctzll(cand);
        cand &= cand - 1;
        if (col_to_row_[j] < 0) {
          seen_[w] |= 1ull << (j & 63);
          col_to_row_[j] = i;
          row_to_col_[i] = j;
          return true;
        }
      }
    }
    for (int w = 0; w < words_; ++w) {
      uint64_t cand = row[w] & ~seen_[w];
      while (cand) {
        int j = (w << 6) + __builtin_ctzll(cand);
        cand &= cand - 1;
        if (seen_[w] & (1ull << (j & 63))) continue;
        seen_[w] |= 1ull << (j & 63);
        if (augment(col_to_row_[j])) {
          col_to_row_[j] = i;
          row_to_col_[i] = j;
          return true;
        }
        cand &= ~seen_[w];
      }
    }
    return false;
  }

  int n_, words_;
  std::vector<uint64_t> adj_;
  std::vector<int> row_to_col_, col_to_row_;
  std::vector<uint64_t> seen_;
};

}  // namespace

std::vector<Stage> bvn_decompose(Matrix m, MatchPolicy policy) {
  const int n = m.n;
  std::vector<Stage> stages;
  if (n == 0) return stages;
  if (!m.is_doubly_stochastic()) throw std::invalid_argument("bvn_decompose: matrix is not doubly stochastic");
  int64_t remaining = m.row_sum(0);
  Matcher matcher(n);
  if (policy == MatchPolicy::kFirstFit) matcher.set_edges(m, 1);

  while (remaining > 0) {
    if (policy == MatchPolicy::kBottleneck) {
      // Largest threshold t such that the entries >= t still contain a perfect matching.
      std::vector<int64_t> vals;
      for (int64_t x : m.v) if (x > 0) vals.push_back(x);
      std::sort(vals.begin(), vals.end());
      vals.erase(std::unique(vals.begin(), vals.end()), vals.end());
      size_t lo = 0, hi = vals.size() - 1;  // vals[lo] always feasible (Birkhoff)
      while (lo < hi) {
        size_t mid = (lo + hi + 1) / 2;
        matcher.set_edges(m, vals[mid]);
        matcher.clear_matching();
        if (matcher.solve() == n) lo = mid; else hi = mid - 1;
      }
      matcher.set_edges(m, vals[lo]);
      matcher.clear_matching();
    }
    if (matcher.solve() != n) throw std::logic_error("bvn_decompose: no perfect matching on a doubly-stochastic matrix");
    Stage st;
    st.to = matcher.row_to_col();
    int64_t w = m.at(0, st.to[0]);
    for (int i = 1; i < n; ++i) w = std::min(w, m.at(i, st.to[i]));
    st.weight = w;
    for (int i = 0; i < n; ++i) {
      int64_t& e = m.at(i, st.to[i]);
      e -= w;
      if (e == 0 && policy == MatchPolicy::kFirstFit) {
        // Only rows whose matched entry vanished need a new partner next round.
        matcher.remove_edge(i, st.to[i]);
        matcher.unmatch_row(i);
      }
    }
    remaining -= w;
    stages.push_back(std::move(st));
  }
  std::stable_sort(stages.begin(), stages.end(),
                   [](const Stage& a, const Stage& b) { return a.weight > b.weight; });
  return stages;
}

Decomposition decompose(const Matrix& input, MatchPolicy policy, int64_t scale) {
  input.check_non_negative();
  if (scale < 1) throw std::invalid_argument("decompose: scale must be >= 1");
  Decomposition d;
  d.scale = scale;
  d.padded = scale == 1 ? input : input.ceil_div(scale);
  d.padding = pad_to_doubly_stochastic(d.padded);
  d.line_sum = d.padded.n ? d.padded.row_sum(0) : 0;
  d.stages = bvn_decompose(d.padded, policy);
  for (Stage& s : d.stages) s.weight *= scale;
  return d;
}

bool verify_decomposition(const Decomposition& d) {
  const int n = d.padded.n;
  Matrix acc(n);
  for (const Stage& s : d.stages) {
    if (static_cast<int>(s.to.size()) != n || s.weight <= 0 || s.weight % d.scale) return false;
    std::vector<char> hit(n, 0);
    for (int i = 0; i < n; ++i) {
      int j = s.to[i];
      if (j < 0 || j >= n || hit[j]) return false;
      hit[j] = 1;
      acc.at(i, j) += s.weight / d.scale;
    }
  }
  return acc == d.padded;
}

int64_t choose_scale(const Matrix& sm, int gpus, ScalePolicy policy, LinkModel inter, LinkModel intra,
                     double mb_per_unit) {
  if (policy == ScalePolicy::kNone) return 1;
  const int s = sm.n;
  auto ok = [&](int64_t f) {
    const int64_t max_sum = sm.ceil_div(f).max_line_sum();
    switch (policy) {
      case ScalePolicy::kLimitMaxSum: return max_sum <= 100;
      case ScalePolicy::kAlways: return max_sum <= s;
      case ScalePolicy::kAlphaBeta: {
        if (max_sum <= s) return true;
        double a = inter.alpha_us * s * s + intra.alpha_us * s * s * gpus;
        double b = inter.beta_us_per_mb * static_cast<double>(max_sum) * static_cast<double>(f) * mb_per_unit;
        return a / b < 0.1;
      }
      default: return true;
    }
  };
  // The predicates are monotone in f on the grid {1, 3, 5, ...}; bisect for the smallest hit.
  int64_t lo = 0, hi = (1000000 - 1) / 2;  // f = 1 + 2k
  if (!ok(1 + 2 * hi)) return -1;
  while (lo < hi) {
    int64_t mid = (lo + hi) / 2;
    if (ok(1 + 2 * mid)) hi = mid; else lo = mid + 1;
  }
  return 1 + 2 * lo;
}

}  // namespace fastb

// Doubly-stochastic padding and Birkhoff-von-Neumann decomposition into permutation stages.
//
// Behaviour matches the reference's FastAll2All
// (nvidia/src/fast_alltoall/alltoall_algorithm.cc:29-57 padding, :80-197 decomposition,
//  :59-78 ordering by weight, :205-223 verification; simulation/algorithm/all2all.cpp:26-257
//  including the ceil-divide coarsening and its three predicates), rebuilt around bitset
// adjacency and an incrementally repaired matching so that an 8x8 plan costs microseconds.
#pragma once
#include <cstdint>
#include <vector>

#include "matrix.h"

namespace fastb {

// One permutation stage: row i talks to column to[i] for `weight` units.
struct Stage {
  std::vector<int> to;
  int64_t weight = 0;
};

enum class MatchPolicy : int {
  kFirstFit = 0,    // any perfect matching, repaired incrementally (what the reference computes)
  kBottleneck = 1,  // perfect matching whose smallest entry is largest: fewer, fatter stages
};

struct Decomposition {
  Matrix padded;              // input + phantom padding; every line sums to line_sum
  Matrix padding;             // phantom part only (never transferred)
  int64_t line_sum = 0;       // max row/column sum of the input == sum of stage weights
  int64_t scale = 1;          // coarsening divisor used (1 = exact units)
  std::vector<Stage> stages;  // sorted by weight, heaviest first
};

// Adds phantom traffic until every row and column sums to max_line_sum(). Returns the padding.
Matrix pad_to_doubly_stochastic(Matrix& m);

// Decomposes a doubly-stochastic matrix. Throws std::logic_error if no perfect matching exists
// (cannot happen for a valid input; the reference indexes out of range in that case).
std::vector<Stage> bvn_decompose(Matrix m, MatchPolicy policy = MatchPolicy::kFirstFit);

// pad + decompose (+ optional coarsening by `scale`: entries are ceil-divided first, and the
// stage weights are multiplied back, so stages still cover the input).
Decomposition decompose(const Matrix& input, MatchPolicy policy = MatchPolicy::kFirstFit,
                        int64_t scale = 1);

// Sum of weight * permutation over all stages == padded matrix * scale? (exactness check)
bool verify_decomposition(const Decomposition& d);

// Coarsening predicates of the reference simulator (simulation/algorithm/all2all.cpp:203-221).
struct LinkModel {
  double alpha_us = 0.0;      // per-message latency
  double beta_us_per_mb = 0;  // inverse bandwidth
};
enum class ScalePolicy : int { kNone = 0, kLimitMaxSum = 1, kAlways = 2, kAlphaBeta = 3 };

// Smallest divisor in [1, 1e6] (odd steps of 2 like the reference's search grid) whose
// ceil-divided matrix satisfies the predicate; returns 1 when policy is kNone, -1 if none does.
int64_t choose_scale(const Matrix& server_matrix, int gpus_per_server, ScalePolicy policy,
                     LinkModel inter, LinkModel intra, double mb_per_unit);

}  // namespace fastb

// Algorithm generators: each one emits a step program (program.h) for one
// collective algorithm.  `count` follows the reference call signatures:
//   allgather      : elements contributed by each rank      (in n,   out P*n)
//   reduce_scatter : elements received by each rank         (in P*n, out n)
//   allreduce      : total vector length                    (in N,   out N)
//   alltoall       : elements exchanged per rank pair       (in P*n, out P*n)
//   gather / bcast / reduce (building blocks): see each generator
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "program.h"

namespace chb {

struct AlgoSpec {
  std::string coll;   // "allgather" | "reduce_scatter" | "allreduce" | "alltoall" | ...
  std::string algo;   // e.g. "radix_batch", "ring", "recursive_doubling"
  int P = 1;
  int k = 2;          // radix
  int b = 1;          // group size (hierarchical) or batch (store-and-forward variants)
  int64_t count = 0;
  int aux = 0;        // algorithm specific (root, ranks per node, single_phase_recv ...)
};

// Throws std::runtime_error with a message naming the violated precondition
// (for example P % b != 0, or count % P != 0 for the hierarchical allreduce).
Builder build_algorithm(const AlgoSpec& s);

// Names accepted for `algo` per collective.
std::vector<std::string> list_algorithms(const std::string& coll);

// ---- schedule arithmetic shared by several generators -------------------------
int64_t ipow(int64_t base, int exp);
// Number of radix-k phases needed to span b slots: how often b-1 can be
// integer-divided by k before it reaches zero.
int num_phases(int b, int k);

// Radix-k recursive exchange over n ranks (fold of the n - k^log leftover
// ranks, per-phase neighbours, per-phase owned ranges).
struct Recexch {
  int n = 0, k = 2, p_of_k = 1, log = 0, rem = 0, T = 0;
  Recexch(int n, int k);
  bool participates(int rank) const;
  int partner(int rank) const;                 // for a folded-out rank: who absorbs it
  std::vector<int> folded_into(int rank) const;  // for a participant: ranks it absorbs
  int step2rank(int rank) const;               // -1 if folded out
  int orig(int step2) const;                   // inverse of step2rank; orig(-1) = -1
  std::vector<int> neighbours(int rank, int phase) const;  // k-1 (or fewer) original ranks
  // Interval of original ranks owned by `rank` when phase `phase` starts
  // (phase = log means everything).
  void range(int rank, int phase, int* offset, int* count) const;
};

}  // namespace chb

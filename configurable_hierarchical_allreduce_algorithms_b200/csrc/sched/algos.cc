// Algorithm registry: (collective, algorithm name) -> generator.
#include "algos.h"

#include <stdexcept>

namespace chb {

// gen_chiara.cc
Builder gen_ag_radix_batch(int P, int64_t n, int k, int b);
Builder gen_rs_radix_batch(int P, int64_t n, int k, int b);
Builder gen_ar_radix_batch(int P, int64_t N, int k, int b);
void emit_ag_radix_batch(Builder& B, int P, int64_t n, int k, int b, int IB, int64_t IO);
Builder gen_phase(const std::string& name, int P, int64_t c, int k, int b);
// gen_baselines.cc
Builder gen_ar_recursive_doubling(int P, int64_t N);
Builder gen_ar_ring(int P, int64_t N);
Builder gen_ar_rabenseifner(int P, int64_t N);
Builder gen_ar_k_rsag(int P, int64_t N, int k);
Builder gen_ar_recursive_multiplying(int P, int64_t N, int k);
Builder gen_ar_recexch(int P, int64_t N, int k);
Builder gen_ar_smp(int P, int64_t N, int ranks_per_node);
Builder gen_rs_pairwise(int P, int64_t n);
Builder gen_rs_ring(int P, int64_t n);
Builder gen_rs_recursive_halving(int P, int64_t n);
void emit_rs_recursive_halving(Builder& B, int P, int64_t n, int dbuf, int64_t doff);
Builder gen_rs_recursive_doubling(int P, int64_t n);
Builder gen_rs_radix(int P, int64_t n, int k);
Builder gen_ag_kbruck(int P, int64_t n, int k);
Builder gen_ag_ring(int P, int64_t n);
Builder gen_ag_recursive_doubling(int P, int64_t n);
Builder gen_ag_linear(int P, int64_t n);
Builder gen_gather_knomial(int P, int64_t n, int k, int root);
Builder gen_grouped(const std::string& coll, const std::string& flat_algo, int P, int64_t count, int k, int b, bool lanes);
// gen_tuna.cc
Builder gen_rs_tuna(int P, int64_t n, int r, int b);
void emit_rs_tuna(Builder& B, int P, int64_t n, int r, int b, int dbuf, int64_t doff);
Builder gen_a2a_tuna(int P, int64_t n, int r, int b);
Builder gen_a2a_linear(int P, int64_t n);

namespace {

// Allreduce = some reduce-scatter into a scratch block, then the hierarchical
// allgather reading that block.  Mirrors the reference's earlier allreduce
// variants:
//   testing/custom_implementations/work_dir/all_reduce/all_reduce_semi_custom_0_1.cpp:159-193
//     (recursive-halving reduce-scatter + hierarchical allgather)
//   testing/custom_implementations/work_dir/all_reduce/all_reduce_custom_0_1.cpp:658-692,
//   all_reduce_custom_0_2.cpp:49-663
//     (store-and-forward reduce-scatter + hierarchical allgather)
Builder gen_ar_semi(int P, int64_t N, int k, int b) {
  if (N % P != 0) throw std::runtime_error("all_reduce_semi_radix_batch: count must be a multiple of the number of ranks");
  int64_t n = N / P;
  Builder B(P, N, N, "all_reduce_semi_radix_batch");
  int R = B.tmp(n);
  emit_rs_recursive_halving(B, P, n, R, 0);
  emit_ag_radix_batch(B, P, n, k, b, R, 0);
  return B;
}

Builder gen_ar_custom(int P, int64_t N, int k, int b) {
  if (N % P != 0) throw std::runtime_error("all_reduce_custom: count must be a multiple of the number of ranks");
  int64_t n = N / P;
  Builder B(P, N, N, "all_reduce_custom");
  int R = B.tmp(n);
  // the store-and-forward reduce-scatter uses k as its radix and b as its batch
  emit_rs_tuna(B, P, n, k, b, R, 0);
  // the allgather half needs a group size that divides P: use the largest
  // divisor of P not above b
  int bb = b < 1 ? 1 : (b > P ? P : b);
  while (P % bb != 0) --bb;
  emit_ag_radix_batch(B, P, n, k, bb, R, 0);
  return B;
}

}  // namespace

std::vector<std::string> list_algorithms(const std::string& coll) {
  if (coll == "allreduce")
    return {"radix_batch", "semi_radix_batch", "custom", "recursive_doubling", "ring",
            "reduce_scatter_allgather", "k_reduce_scatter_allgather", "recursive_multiplying",
            "recursive_exchange", "inter_reduce_exchange_bcast"};
  if (coll == "reduce_scatter")
    return {"radix_batch", "pairwise", "ring", "recursive_halving", "recursive_doubling", "radix",
            "radix_block", "k_nomial"};
  if (coll == "allgather")
    return {"radix_batch", "k_brucks", "ring", "recursive_doubling", "linear"};
  if (coll == "alltoall") return {"tuna", "linear"};
  if (coll == "gather") return {"k_nomial"};
  if (coll == "phase")
    return {"intra_gather_k_nomial", "inter_allgather_linear", "intra_allgather_k_brucks",
            "intra_reduce_scatter_radix_batch", "inter_reduce_linear", "intra_scatter_radix_batch"};
  return {};
}

Builder build_algorithm(const AlgoSpec& s) {
  if (s.P < 1) throw std::runtime_error("number of ranks must be >= 1");
  if (s.count < 0) throw std::runtime_error("count must be >= 0");
  const std::string& c = s.coll;
  const std::string& a = s.algo;
  if (c == "allreduce") {
    if (a == "radix_batch") return gen_ar_radix_batch(s.P, s.count, s.k, s.b);
    if (a == "semi_radix_batch") return gen_ar_semi(s.P, s.count, s.k, s.b);
    if (a == "custom") return gen_ar_custom(s.P, s.count, s.k, s.b);
    if (a == "recursive_doubling") return gen_ar_recursive_doubling(s.P, s.count);
    if (a == "ring") return gen_ar_ring(s.P, s.count);
    if (a == "reduce_scatter_allgather") return gen_ar_rabenseifner(s.P, s.count);
    if (a == "k_reduce_scatter_allgather") return gen_ar_k_rsag(s.P, s.count, s.k);
    if (a == "recursive_multiplying") return gen_ar_recursive_multiplying(s.P, s.count, s.k);
    if (a == "recursive_exchange") return gen_ar_recexch(s.P, s.count, s.k);
    if (a == "inter_reduce_exchange_bcast") return gen_ar_smp(s.P, s.count, s.aux > 0 ? s.aux : (s.b > 0 ? s.b : 1));
  } else if (c == "reduce_scatter") {
    if (a == "radix_batch") return gen_rs_radix_batch(s.P, s.count, s.k, s.b);
    if (a == "pairwise") return gen_rs_pairwise(s.P, s.count);
    if (a == "ring") return gen_rs_ring(s.P, s.count);
    if (a == "recursive_halving") return gen_rs_recursive_halving(s.P, s.count);
    if (a == "recursive_doubling") return gen_rs_recursive_doubling(s.P, s.count);
    if (a == "radix") return gen_rs_radix(s.P, s.count, s.k);
    if (a == "radix_block") return gen_rs_tuna(s.P, s.count, s.k, s.b);
    // k-nomial recursive halving (tuna_based_outdated/reduce_scatter_k_nomial.cpp:25-217): the same radix-k
    // neighbour sets and halving ranges as "radix"; only the way leftover ranks are folded differs
    if (a == "k_nomial") return gen_rs_radix(s.P, s.count, s.k);
  } else if (c == "allgather") {
    if (a == "radix_batch") return gen_ag_radix_batch(s.P, s.count, s.k, s.b);
    if (a == "k_brucks") return gen_ag_kbruck(s.P, s.count, s.k);
    if (a == "ring") return gen_ag_ring(s.P, s.count);
    if (a == "recursive_doubling") return gen_ag_recursive_doubling(s.P, s.count);
    if (a == "linear") return gen_ag_linear(s.P, s.count);
  } else if (c == "alltoall") {
    if (a == "tuna") return gen_a2a_tuna(s.P, s.count, s.k, s.b);
    if (a == "linear") return gen_a2a_linear(s.P, s.count);
  } else if (c == "gather") {
    if (a == "k_nomial") return gen_gather_knomial(s.P, s.count, s.k, s.aux);
  } else if (c == "phase") {
    return gen_phase(a, s.P, s.count, s.k, s.b);
  }
  // phases as stand-alone collectives on sub-communicators: "intra_<flat algorithm>" runs it inside
  // every group of b consecutive ranks, "inter_<flat algorithm>" along every lane of stride b
  if (a.rfind("intra_", 0) == 0) return gen_grouped(c, a.substr(6), s.P, s.count, s.k, s.b, false);
  if (a.rfind("inter_", 0) == 0 && a != "inter_reduce_exchange_bcast") return gen_grouped(c, a.substr(6), s.P, s.count, s.k, s.b, true);
  throw std::runtime_error("unknown collective/algorithm: " + c + "/" + a);
}

}  // namespace chb

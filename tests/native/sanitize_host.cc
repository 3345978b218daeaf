// Host-side exercise of the schedule compiler for sanitizer builds: every
// registered algorithm is generated, lowered, verified, simulated under a
// random interleaving and executed with one thread per rank, and the result is
// compared with the definition of the collective.  Built by the test suite
// with -fsanitize=address,undefined and, for the threaded executor, with
// -fsanitize=thread; a finding of either makes the process exit non-zero.
//
// Usage: sanitize_host [threads-only]
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "sched/algos.h"
#include "sched/ll_plan.h"
#include "sched/program.h"
#include "sched/types.h"

using namespace chb;

namespace {

int32_t value(int rank, int64_t i) { return (int32_t)((rank * 131 + i * 7 + 3) % 1009); }

// Expected output of the rank with index `me` inside the (sub-)communicator `members`;
// returns false when this rank's output is unspecified.
bool expect(const std::string& coll, const std::vector<int>& members, int me, int64_t in_elems, int64_t out_elems,
            int root, std::vector<int32_t>& e) {
  const int P = (int)members.size();
  e.assign(out_elems, 0);
  if (coll == "allreduce") {
    for (int64_t i = 0; i < out_elems; ++i)
      for (int q : members) e[i] += value(q, i);
  } else if (coll == "reduce_scatter") {
    for (int64_t i = 0; i < out_elems; ++i)
      for (int q : members) e[i] += value(q, (int64_t)me * out_elems + i);
  } else if (coll == "allgather" || coll == "gather") {
    if (coll == "gather" && me != root) return false;
    for (int q = 0; q < P; ++q)
      for (int64_t i = 0; i < in_elems; ++i) e[q * in_elems + i] = value(members[q], i);
  } else if (coll == "alltoall") {
    const int64_t n = in_elems / P;
    for (int q = 0; q < P; ++q)
      for (int64_t i = 0; i < n; ++i) e[q * n + i] = value(members[q], (int64_t)me * n + i);
  } else {
    return false;
  }
  return true;
}

// The ranks that rank r communicates with: everybody, its group of b consecutive ranks
// ("intra_<algo>") or its lane of stride b ("inter_<algo>").
std::vector<int> members_of(const AlgoSpec& s, int r, int* me) {
  std::vector<int> m;
  if (s.algo.rfind("intra_", 0) == 0) {
    for (int j = 0; j < s.b; ++j) m.push_back(r / s.b * s.b + j);
    *me = r % s.b;
  } else if (s.algo.rfind("inter_", 0) == 0 && s.algo != "inter_reduce_exchange_bcast") {
    for (int j = 0; j < s.P / s.b; ++j) m.push_back(r % s.b + j * s.b);
    *me = r / s.b;
  } else {
    for (int j = 0; j < s.P; ++j) m.push_back(j);
    *me = r;
  }
  return m;
}

int g_cases = 0, g_fail = 0;

void fail(const std::string& what, const AlgoSpec& s, const std::string& detail) {
  ++g_fail;
  std::fprintf(stderr, "FAIL %s: %s/%s P=%d k=%d b=%d count=%lld %s\n", what.c_str(), s.coll.c_str(), s.algo.c_str(),
               s.P, s.k, s.b, (long long)s.count, detail.c_str());
}

void run_case(const AlgoSpec& s, bool threads_only) {
  Builder B(1, 0, 0, "");
  try {
    B = build_algorithm(s);
  } catch (const std::runtime_error&) {
    return;   // a violated precondition (b does not divide P, ...) is reported, not executed
  }
  for (int variant = 0; variant < 2; ++variant) {
    LowerOpts o;
    o.in_symmetric = o.out_symmetric = (variant == 1);
    Program p = B.lower(o);
    ++g_cases;
    std::string err;
    if (!threads_only && verify(p, &err) != 0) fail("verify", s, err);
    std::vector<std::vector<int32_t>> in(s.P), out(s.P);
    std::vector<void*> ip(s.P), op(s.P);
    for (int r = 0; r < s.P; ++r) {
      in[r].resize(p.in_elems > 0 ? p.in_elems : 1);
      out[r].assign(p.out_elems > 0 ? p.out_elems : 1, -1);
      for (int64_t i = 0; i < p.in_elems; ++i) in[r][i] = value(r, i);
      ip[r] = in[r].data();
      op[r] = out[r].data();
    }
    auto check = [&](const char* what) {
      std::vector<int32_t> e;
      for (int r = 0; r < s.P; ++r) {
        int me = 0;
        const std::vector<int> members = members_of(s, r, &me);
        if (!expect(s.coll, members, me, p.in_elems, p.out_elems, s.aux, e)) continue;
        if (std::memcmp(e.data(), out[r].data(), sizeof(int32_t) * p.out_elems) != 0) {
          fail(what, s, "wrong result on rank " + std::to_string(r));
          return;
        }
      }
    };
    if (!threads_only) {
      for (uint64_t seed = 1; seed <= 2; ++seed) {
        for (auto& v : out) std::fill(v.begin(), v.end(), -1);
        if (simulate(p, DT_I32, OP_SUM, ip.data(), op.data(), seed * 7919u + variant, &err) != 0) fail("simulate", s, err);
        else check("simulate");
      }
    }
    // the push form of the same program (plan tables + line-by-line execution, two launches on the two inbox
    // halves) for the collectives the executor accepts
    if (!threads_only && variant == 1 &&
        (s.coll == "allreduce" || s.coll == "reduce_scatter" || s.coll == "allgather" || s.coll == "alltoall")) {
      for (auto& v : out) std::fill(v.begin(), v.end(), -1);
      if (simulate_ll(p, DT_I32, OP_SUM, ip.data(), op.data(), 17u, 3, LL_FAULT_NONE, 2, &err) != 0) fail("simulate_ll", s, err);
      else check("simulate_ll");
    }
    for (auto& v : out) std::fill(v.begin(), v.end(), -1);
    double sec = 0;
    if (run_threads(p, DT_I32, OP_SUM, ip.data(), op.data(), 2, &sec) != 0) fail("run_threads", s, "wait expired");
    else check("run_threads");
  }
}

}  // namespace

int main(int argc, char** argv) {
  const bool threads_only = argc > 1 && !std::strcmp(argv[1], "threads-only");
  const char* colls[] = {"allreduce", "reduce_scatter", "allgather", "alltoall", "gather", "phase"};   // phases: memory safety only
  const int Ps_full[] = {1, 2, 3, 4, 6, 8, 12};
  const int Ps_thr[] = {2, 4, 6};
  const int* Ps = threads_only ? Ps_thr : Ps_full;
  const int nP = threads_only ? 3 : 7;
  for (const char* coll : colls) {
    std::vector<std::string> algos = list_algorithms(coll);
    if (std::string(coll) != "alltoall" && std::string(coll) != "gather" && std::string(coll) != "phase") {
      algos.push_back("intra_ring");
      algos.push_back("inter_ring");
    }
    for (const std::string& algo : algos) {
      for (int pi = 0; pi < nP; ++pi) {
        const int P = Ps[pi];
        for (int k = 2; k <= 4; ++k) {
          for (int b = 1; b <= P; ++b) {
            if (P % b) continue;
            if (threads_only && !(k == 2 || b == 2)) continue;
            AlgoSpec s;
            s.coll = coll;
            s.algo = algo;
            s.P = P;
            s.k = k;
            s.b = b;
            s.aux = 0;
            // allreduce counts are totals (a multiple of P), the others are per block; 5 keeps ragged tails in play
            s.count = std::string(coll) == "allreduce" ? (int64_t)P * 5 : 5;
            run_case(s, threads_only);
          }
        }
      }
    }
  }
  std::printf("%d programs, %d failures\n", g_cases, g_fail);
  return g_fail ? 1 : 0;
}

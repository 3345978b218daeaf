// Flat (non-hierarchical) comparison algorithms as pull step programs.
//
// Behaviour reproduced (not code) from the reference's re-implementations of
// MPICH's algorithms:
//   allreduce      testing/mpich_implementations/all_reduce/allreduce_recursive_doubling.cpp:4-102
//                  .../allreduce_ring.cpp:3-104
//                  .../allreduce_reduce_scatter_allgather.cpp:3-174        (Rabenseifner)
//                  .../allreduce_k_reduce_scatter_allgather.cpp:257-540    (radix-k RS + AG)
//                  .../allreduce_recursive_multiplying.cpp:3-177
//                  .../allreduce_recexch.cpp:188-448
//                  .../allreduce_inter_reduce_exchange_bcast.cpp:6-116     (node-hierarchical)
//   reduce-scatter testing/mpich_implementations/reduce_scatter/reduce_scatter_pairwise.cpp:4-74
//                  .../reduce_scatter_recursive_halving.cpp:7-153
//                  .../reduce_scatter_recursive_doubling.cpp:10-177
//                  .../reduce_scatter_radix.cpp:204-377
//   allgather      testing/custom_implementations/work_dir/all_gather/outdated_versions/
//                  all_gather_0_1_alpha.cpp:36-113 (k-nomial gather), :220-313 (radix-k Bruck)
//
// A two-sided exchange "send my vector, receive yours, reduce" becomes
// new = mine op yours on both sides; because each side reads the other's
// vector while producing its own, full-vector exchanges ping-pong between two
// scratch vectors, while halving exchanges (disjoint kept/sent ranges) run in
// place.
#include <algorithm>
#include <stdexcept>

#include "algos.h"

namespace chb {
namespace {

// Per-rank "where does my current vector live" tracker for full-vector
// exchange algorithms.
struct Cur {
  std::vector<int> buf;
  int A, Bb;
  Cur(int P, int A_, int B_) : buf(P, L_IN), A(A_), Bb(B_) {}
  int next(int r) const { return buf[r] == A ? Bb : A; }
};

struct Pof2Fold {
  int P, pof2, rem;
  explicit Pof2Fold(int P_) : P(P_) {
    pof2 = 1;
    while (pof2 * 2 <= P) pof2 *= 2;
    rem = P - pof2;
  }
  int newrank(int r) const { return r < 2 * rem ? (r % 2 == 0 ? -1 : r / 2) : r - rem; }
  int real(int nr) const { return nr < rem ? nr * 2 + 1 : nr + rem; }
};

std::vector<Src> sorted_sources(std::vector<Src> v) {
  std::sort(v.begin(), v.end(), [](const Src& a, const Src& b) { return a.peer < b.peer; });
  return v;
}

// split `count` into `parts` near-equal contiguous blocks, larger ones first
void split_blocks(int64_t count, int parts, std::vector<int64_t>& off, std::vector<int64_t>& cnt) {
  off.assign(parts + 1, 0);
  cnt.assign(parts, 0);
  for (int i = 0; i < parts; ++i) {
    cnt[i] = count / parts + (i < count % parts ? 1 : 0);
    off[i + 1] = off[i] + cnt[i];
  }
}

}  // namespace

// ============================ allreduce: recursive doubling ==========================
Builder gen_ar_recursive_doubling(int P, int64_t N) {
  Builder B(P, N, N, "allreduce_recursive_doubling");
  if (P == 1) { B.copy(0, L_OUT, 0, 0, L_IN, 0, N); return B; }
  Pof2Fold f(P);
  int TA = B.tmp(N), TB = B.tmp(N);
  Cur cur(P, TA, TB);
  for (int r = 1; r < 2 * f.rem; r += 2) {
    B.reduce(r, TA, 0, {Src{r - 1, L_IN, 0}, Src{r, L_IN, 0}}, N, false);
    cur.buf[r] = TA;
  }
  int nrounds = 0;
  for (int m = 1; m < f.pof2; m <<= 1) ++nrounds;
  int round = 0;
  for (int mask = 1; mask < f.pof2; mask <<= 1, ++round) {
    bool last = (round == nrounds - 1);
    std::vector<int> nxt(P);
    for (int r = 0; r < P; ++r) {
      int nr = f.newrank(r);
      if (nr < 0) continue;
      int dst = f.real(nr ^ mask);
      int d = last ? (int)L_OUT : cur.next(r);
      // lower rank's operand first (keeps the order for non-commutative use)
      std::vector<Src> s = sorted_sources({Src{r, cur.buf[r], 0}, Src{dst, cur.buf[dst], 0}});
      B.reduce(r, d, 0, s, N, false, last ? OPF_FINAL : 0);
      nxt[r] = d;
    }
    for (int r = 0; r < P; ++r)
      if (f.newrank(r) >= 0) cur.buf[r] = nxt[r];
  }
  if (nrounds == 0)  // pof2 == 1 cannot happen for P >= 2, kept for completeness
    for (int r = 0; r < P; ++r)
      if (f.newrank(r) >= 0) B.copy(r, L_OUT, 0, r, cur.buf[r], 0, N);
  for (int r = 0; r < 2 * f.rem; r += 2) B.copy(r, L_OUT, 0, r + 1, L_OUT, 0, N);
  return B;
}

// ============================ ring pieces =============================================
// Reduce-scatter half of the ring on `cnt/off` chunks, working in `WB` (buffer
// that ends up holding the fully reduced chunk r at rank r).
static void ring_rs(Builder& B, int P, int WB, const std::vector<int64_t>& off,
                    const std::vector<int64_t>& cnt) {
  for (int i = 0; i < P - 1; ++i)
    for (int r = 0; r < P; ++r) {
      int left = (r - 1 + P) % P;
      int c = ((r - 2 - i) % P + P) % P;
      std::vector<Src> s;
      s.push_back(i == 0 ? Src{left, L_IN, off[c]} : Src{left, WB, off[c]});
      s.push_back(Src{r, L_IN, off[c]});
      B.reduce(r, WB, off[c], s, cnt[c], false, i == P - 2 ? OPF_FINAL : 0);
    }
}
static void ring_ag(Builder& B, int P, int WB, const std::vector<int64_t>& off,
                    const std::vector<int64_t>& cnt, bool first_from_in) {
  for (int i = 0; i < P - 1; ++i)
    for (int r = 0; r < P; ++r) {
      int left = (r - 1 + P) % P;
      int c = ((r - 1 - i) % P + P) % P;
      if (i == 0 && first_from_in) B.copy(r, WB, off[c], left, L_IN, 0, cnt[c]);
      else B.copy(r, WB, off[c], left, WB, off[c], cnt[c]);
    }
}

Builder gen_ar_ring(int P, int64_t N) {
  Builder B(P, N, N, "allreduce_ring");
  if (P == 1) { B.copy(0, L_OUT, 0, 0, L_IN, 0, N); return B; }
  // chunks of ceil(N/P) with a short (possibly empty) tail
  int64_t c = (N + P - 1) / P;
  std::vector<int64_t> off(P + 1), cnt(P);
  for (int i = 0; i < P; ++i) {
    off[i] = std::min<int64_t>((int64_t)i * c, N);
    cnt[i] = std::max<int64_t>(0, std::min<int64_t>(c, N - (int64_t)i * c));
  }
  off[P] = N;
  ring_rs(B, P, L_OUT, off, cnt);
  ring_ag(B, P, L_OUT, off, cnt, false);
  return B;
}

// ============================ allreduce: Rabenseifner ================================
Builder gen_ar_rabenseifner(int P, int64_t N) {
  Builder B(P, N, N, "allreduce_reduce_scatter_allgather");
  if (P == 1) { B.copy(0, L_OUT, 0, 0, L_IN, 0, N); return B; }
  Pof2Fold f(P);
  if (N < f.pof2) throw std::runtime_error("allreduce_reduce_scatter_allgather: count must be >= the largest power of two <= ranks");
  int ACC = B.tmp(N);
  std::vector<int> cur(P, L_IN);
  for (int r = 1; r < 2 * f.rem; r += 2) {
    B.reduce(r, ACC, 0, {Src{r - 1, L_IN, 0}, Src{r, L_IN, 0}}, N, false);
    cur[r] = ACC;
  }
  std::vector<int64_t> off, cnt;
  split_blocks(N, f.pof2, off, cnt);
  std::vector<int> lo(P, 0), hi(P, f.pof2);
  int steps = 0;
  for (int m = 1; m < f.pof2; m <<= 1) ++steps;
  // recursive halving with distance doubling
  int step = 0;
  std::vector<std::vector<std::pair<int, int>>> hist(P);  // ranges before each step
  for (int mask = 1; mask < f.pof2; mask <<= 1, ++step) {
    bool last = step == steps - 1;
    std::vector<int> nxt = cur;
    for (int r = 0; r < P; ++r) {
      int nr = f.newrank(r);
      if (nr < 0) continue;
      int nd = nr ^ mask, dst = f.real(nd);
      hist[r].emplace_back(lo[r], hi[r]);
      int mid = lo[r] + (hi[r] - lo[r]) / 2;
      int klo = nr < nd ? lo[r] : mid, khi = nr < nd ? mid : hi[r];
      int d = last ? (int)L_OUT : ACC;
      std::vector<Src> s;
      bool acc = false;
      if (cur[r] == ACC && d == ACC) acc = true;
      else s.push_back(Src{r, cur[r], off[klo]});
      s.push_back(Src{dst, cur[dst], off[klo]});
      B.reduce(r, d, off[klo], s, off[khi] - off[klo], acc, last ? OPF_FINAL : 0);
      lo[r] = klo;
      hi[r] = khi;
      nxt[r] = d;
    }
    cur = nxt;
  }
  // recursive doubling allgather, distance halving, everything in OUT
  for (int mask = f.pof2 >> 1, s = steps - 1; mask > 0; mask >>= 1, --s)
    for (int r = 0; r < P; ++r) {
      int nr = f.newrank(r);
      if (nr < 0) continue;
      int dst = f.real(nr ^ mask);
      // after this step I own the range I had before RS step s; fetch the
      // partner's part of it
      int plo = hist[r][s].first, phi = hist[r][s].second;
      int mid = plo + (phi - plo) / 2;
      bool lower = (nr < (nr ^ mask));
      int flo = lower ? mid : plo, fhi = lower ? phi : mid;
      B.copy(r, L_OUT, off[flo], dst, L_OUT, off[flo], off[fhi] - off[flo]);
    }
  for (int r = 0; r < 2 * f.rem; r += 2) B.copy(r, L_OUT, 0, r + 1, L_OUT, 0, N);
  return B;
}

// ============================ allreduce: radix-k RS + AG =============================
// Radix-k recursive exchange: reduce-scatter with the nearest neighbours first, so that a rank ends up with
// the block whose index is its digit-reversed rank, then the allgather in the opposite order.  Phases,
// block sizes (count / k^log each, the last block takes the remainder) and the order in which a rank adds its
// neighbours' contributions follow the reference
// (testing/mpich_implementations/all_reduce/allreduce_k_reduce_scatter_allgather.cpp:330-470), which makes
// float results identical to its results bit for bit.
Builder gen_ar_k_rsag(int P, int64_t N, int k) {
  Builder B(P, N, N, "allreduce_k_reduce_scatter_allgather");
  if (P == 1) { B.copy(0, L_OUT, 0, 0, L_IN, 0, N); return B; }
  Recexch rx(P, k);
  const int K = rx.k, L = rx.log, pk = rx.p_of_k;
  std::vector<int64_t> off(pk + 1);
  for (int i = 0; i < pk; ++i) off[i] = (int64_t)i * (N / pk);
  off[pk] = N;
  int ACC = B.tmp(N);
  std::vector<int> cur(P, L_IN);
  for (int r = 0; r < P; ++r) {
    std::vector<int> fl = rx.folded_into(r);
    if (fl.empty()) continue;
    std::vector<Src> s{Src{r, L_IN, 0}};                 // own data first, then the folded ranks in receive order
    for (int q : fl) s.push_back(Src{q, L_IN, 0});
    B.reduce(r, ACC, 0, s, N, false);
    cur[r] = ACC;
  }
  auto reversed = [&](int v) {                           // digit 0 becomes the most significant digit
    int out = 0;
    for (int i = 0; i < L; ++i) { out = out * K + v % K; v /= K; }
    return out;
  };
  // blocks owned by rank r once the phases of digits 0 .. L-1-level are done
  auto owned = [&](int r, int level, int* lo, int* hi) {
    int64_t pw = ipow(K, level);
    *lo = (int)(reversed(rx.step2rank(r)) / pw * pw);
    *hi = (int)(*lo + pw);
  };
  for (int ph = 0; ph < L; ++ph) {
    std::vector<int> nxt = cur;
    const bool last = ph == L - 1;
    for (int r = 0; r < P; ++r) {
      if (!rx.participates(r)) continue;
      int lo, hi;
      owned(r, L - 1 - ph, &lo, &hi);
      int d = last ? (int)L_OUT : ACC;
      std::vector<Src> s;
      bool acc = (cur[r] == ACC && d == ACC);
      if (!acc) s.push_back(Src{r, cur[r], off[lo]});
      for (int q : rx.neighbours(r, ph)) s.push_back(Src{q, cur[q], off[lo]});
      B.reduce(r, d, off[lo], s, off[hi] - off[lo], acc, last ? OPF_FINAL : 0);
      nxt[r] = d;
    }
    cur = nxt;
  }
  if (L == 0)
    for (int r = 0; r < P; ++r)
      if (rx.participates(r)) B.copy(r, L_OUT, 0, r, cur[r], 0, N);
  for (int ph = L - 1; ph >= 0; --ph)
    for (int r = 0; r < P; ++r) {
      if (!rx.participates(r)) continue;
      for (int q : rx.neighbours(r, ph)) {
        int lo, hi;
        owned(q, L - 1 - ph, &lo, &hi);
        B.copy(r, L_OUT, off[lo], q, L_OUT, off[lo], off[hi] - off[lo]);
      }
    }
  for (int r = 0; r < P; ++r)
    if (!rx.participates(r)) B.copy(r, L_OUT, 0, rx.partner(r), L_OUT, 0, N);
  return B;
}

// ============================ allreduce: full-vector radix-k ========================
// fold_mode 0: ranks >= k^log fold onto rank % k^log (recursive multiplying)
// fold_mode 1: recursive-exchange fold in groups of k (recexch)
static Builder gen_ar_fullvec(int P, int64_t N, int k, int fold_mode, const char* name) {
  Builder B(P, N, N, name);
  if (P == 1) { B.copy(0, L_OUT, 0, 0, L_IN, 0, N); return B; }
  if (k < 2) throw std::runtime_error("radix must be >= 2");
  int TA = B.tmp(N), TB = B.tmp(N);
  Cur cur(P, TA, TB);
  Recexch rx(P, k);
  int keff = rx.k, pofk = rx.p_of_k, log = rx.log;
  if (fold_mode == 0) {
    // recursive multiplying keeps the radix it is given, also beyond the number of ranks (everything then folds
    // onto the ranks below k^log), allreduce_recursive_multiplying.cpp:9-12
    keff = k;
    pofk = 1;
    log = 0;
    while ((int64_t)pofk * k <= P) { pofk *= k; ++log; }
  }
  auto participates = [&](int r) { return fold_mode == 0 ? r < pofk : rx.participates(r); };
  auto folded = [&](int r) {
    std::vector<int> v;
    if (fold_mode == 0) { for (int q = r + pofk; q < P; q += pofk) v.push_back(q); }
    else v = rx.folded_into(r);
    return v;
  };
  auto partner = [&](int r) { return fold_mode == 0 ? r % pofk : rx.partner(r); };
  auto neigh = [&](int r, int p) {
    if (fold_mode == 1) return rx.neighbours(r, p);
    std::vector<int> v;
    int64_t pw = ipow(keff, p);
    int digit = (int)((r / pw) % keff);
    for (int d = 0; d < keff; ++d)
      if (d != digit) v.push_back((int)(r + (d - digit) * pw));
    return v;
  };
  for (int r = 0; r < P; ++r) {
    if (!participates(r)) continue;
    std::vector<int> fl = folded(r);
    if (fl.empty()) continue;
    // the reference adds the folded ranks' data in the order it receives them: recursive exchange starts from its
    // own data (allreduce_recexch.cpp:283-296), recursive multiplying chains the senders in rank order and adds
    // its own data last (allreduce_recursive_multiplying.cpp:57-76)
    std::vector<Src> s;
    if (fold_mode == 1) s.push_back(Src{r, L_IN, 0});
    for (int q : fl) s.push_back(Src{q, L_IN, 0});
    if (fold_mode == 0) s.push_back(Src{r, L_IN, 0});
    B.reduce(r, TA, 0, s, N, false);
    cur.buf[r] = TA;
  }
  for (int p = 0; p < log; ++p) {
    bool last = p == log - 1;
    std::vector<int> nxt(P, 0);
    for (int r = 0; r < P; ++r) {
      if (!participates(r)) continue;
      int d = last ? (int)L_OUT : cur.next(r);
      std::vector<Src> s{Src{r, cur.buf[r], 0}};
      for (int q : neigh(r, p)) s.push_back(Src{q, cur.buf[q], 0});
      B.reduce(r, d, 0, sorted_sources(s), N, false, last ? OPF_FINAL : 0);
      nxt[r] = d;
    }
    for (int r = 0; r < P; ++r)
      if (participates(r)) cur.buf[r] = nxt[r];
  }
  if (log == 0)
    for (int r = 0; r < P; ++r)
      if (participates(r)) B.copy(r, L_OUT, 0, r, cur.buf[r], 0, N);
  for (int r = 0; r < P; ++r)
    if (!participates(r)) B.copy(r, L_OUT, 0, partner(r), L_OUT, 0, N);
  return B;
}
Builder gen_ar_recursive_multiplying(int P, int64_t N, int k) {
  return gen_ar_fullvec(P, N, k, 0, "allreduce_recursive_multiplying");
}
Builder gen_ar_recexch(int P, int64_t N, int k) {
  return gen_ar_fullvec(P, N, k, 1, "allreduce_recursive_exchange");
}

// ============================ allreduce: node-hierarchical ==========================
// Local reduce to the first rank of each node, recursive doubling between the
// node leaders, local broadcast.
Builder gen_ar_smp(int P, int64_t N, int ranks_per_node) {
  if (ranks_per_node < 1) throw std::runtime_error("ranks per node must be >= 1");
  Builder B(P, N, N, "allreduce_inter_reduce_exchange_bcast");
  int nodes = (P + ranks_per_node - 1) / ranks_per_node;
  int TA = B.tmp(N), TB = B.tmp(N);
  std::vector<int> leader(nodes);
  std::vector<int> cur(P, L_IN);
  for (int nd = 0; nd < nodes; ++nd) {
    int lead = nd * ranks_per_node;
    leader[nd] = lead;
    std::vector<Src> s;
    for (int r = lead; r < std::min(P, lead + ranks_per_node); ++r) s.push_back(Src{r, L_IN, 0});
    int d = nodes == 1 ? (int)L_OUT : TA;
    B.reduce(lead, d, 0, s, N, false, nodes == 1 ? OPF_FINAL : 0);
    cur[lead] = d;
  }
  if (nodes > 1) {
    Pof2Fold f(nodes);
    auto nextbuf = [&](int r) { return cur[r] == TA ? TB : TA; };
    for (int i = 1; i < 2 * f.rem; i += 2) {
      int r = leader[i], q = leader[i - 1];
      int d = nextbuf(r);
      B.reduce(r, d, 0, {Src{q, cur[q], 0}, Src{r, cur[r], 0}}, N, false);
      cur[r] = d;
    }
    int steps = 0;
    for (int m = 1; m < f.pof2; m <<= 1) ++steps;
    int step = 0;
    for (int mask = 1; mask < f.pof2; mask <<= 1, ++step) {
      bool last = step == steps - 1;
      std::vector<int> nxt = cur;
      for (int i = 0; i < nodes; ++i) {
        int nr = f.newrank(i);
        if (nr < 0) continue;
        int r = leader[i], q = leader[f.real(nr ^ mask)];
        int d = last ? (int)L_OUT : nextbuf(r);
        B.reduce(r, d, 0, sorted_sources({Src{r, cur[r], 0}, Src{q, cur[q], 0}}), N, false, last ? OPF_FINAL : 0);
        nxt[r] = d;
      }
      cur = nxt;
    }
    if (steps == 0)
      for (int i = 0; i < nodes; ++i)
        if (f.newrank(i) >= 0) B.copy(leader[i], L_OUT, 0, leader[i], cur[leader[i]], 0, N);
    for (int i = 0; i < 2 * f.rem; i += 2) B.copy(leader[i], L_OUT, 0, leader[i + 1], L_OUT, 0, N);
  }
  for (int r = 0; r < P; ++r) {
    int lead = r / ranks_per_node * ranks_per_node;
    if (r != lead) B.copy(r, L_OUT, 0, lead, L_OUT, 0, N);
  }
  return B;
}

// ============================ reduce-scatter baselines ==============================
Builder gen_rs_pairwise(int P, int64_t n) {
  Builder B(P, (int64_t)P * n, n, "reduce_scatter_pairwise");
  for (int r = 0; r < P; ++r) B.copy(r, L_OUT, 0, r, L_IN, (int64_t)r * n, n);
  for (int i = 1; i < P; ++i)
    for (int r = 0; r < P; ++r) {
      int src = (r - i + P) % P;
      B.reduce(r, L_OUT, 0, {Src{src, L_IN, (int64_t)r * n}}, n, true, i == P - 1 ? OPF_FINAL : 0);
    }
  return B;
}

Builder gen_rs_ring(int P, int64_t n) {
  Builder B(P, (int64_t)P * n, n, "reduce_scatter_ring");
  if (P == 1) { B.copy(0, L_OUT, 0, 0, L_IN, 0, n); return B; }
  int ACC = B.tmp((int64_t)P * n);
  for (int i = 0; i < P - 1; ++i)
    for (int r = 0; r < P; ++r) {
      int left = (r - 1 + P) % P;
      int c = ((r - 2 - i) % P + P) % P;
      bool last = i == P - 2;  // then c == r
      std::vector<Src> s;
      s.push_back(i == 0 ? Src{left, L_IN, (int64_t)c * n} : Src{left, ACC, (int64_t)c * n});
      s.push_back(Src{r, L_IN, (int64_t)c * n});
      if (last) B.reduce(r, L_OUT, 0, s, n, false, OPF_FINAL);
      else B.reduce(r, ACC, (int64_t)c * n, s, n, false);
    }
  return B;
}

// Result block of rank r lands in (dbuf, doff) so that callers can chain an
// allgather after it.
void emit_rs_recursive_halving(Builder& B, int P, int64_t n, int dbuf, int64_t doff) {
  if (P == 1) { B.copy(0, dbuf, doff, 0, L_IN, 0, n); return; }
  Pof2Fold f(P);
  const int64_t N = (int64_t)P * n;
  int ACC = B.tmp(N);
  std::vector<int> cur(P, L_IN);
  for (int r = 1; r < 2 * f.rem; r += 2) {
    B.reduce(r, ACC, 0, {Src{r - 1, L_IN, 0}, Src{r, L_IN, 0}}, N, false);
    cur[r] = ACC;
  }
  // block ranges per new rank: folded pairs own two original blocks
  std::vector<int64_t> off(f.pof2 + 1, 0);
  for (int i = 0; i < f.pof2; ++i) off[i + 1] = off[i] + (i < f.rem ? 2 : 1) * n;
  std::vector<int> lo(P, 0), hi(P, f.pof2);
  for (int mask = f.pof2 >> 1; mask > 0; mask >>= 1) {
    std::vector<int> nxt = cur;
    for (int r = 0; r < P; ++r) {
      int nr = f.newrank(r);
      if (nr < 0) continue;
      int nd = nr ^ mask, dst = f.real(nd);
      int mid = lo[r] + (hi[r] - lo[r]) / 2;
      int klo = nr < nd ? lo[r] : mid, khi = nr < nd ? mid : hi[r];
      std::vector<Src> s;
      bool acc = cur[r] == ACC;
      if (!acc) s.push_back(Src{r, L_IN, off[klo]});
      s.push_back(Src{dst, cur[dst], off[klo]});
      B.reduce(r, ACC, off[klo], s, off[khi] - off[klo], acc, mask == 1 ? OPF_FINAL : 0);
      lo[r] = klo;
      hi[r] = khi;
      nxt[r] = ACC;
    }
    cur = nxt;
  }
  for (int r = 0; r < P; ++r) {
    int nr = f.newrank(r);
    if (nr >= 0) B.copy(r, dbuf, doff, r, cur[r], (int64_t)r * n, n);
    else B.copy(r, dbuf, doff, r + 1, ACC, (int64_t)r * n, n);  // handed back by the odd partner
  }
}

Builder gen_rs_recursive_halving(int P, int64_t n) {
  Builder B(P, (int64_t)P * n, n, "reduce_scatter_recursive_halving");
  emit_rs_recursive_halving(B, P, n, L_OUT, 0);
  return B;
}

Builder gen_rs_recursive_doubling(int P, int64_t n) {
  Builder B(P, (int64_t)P * n, n, "reduce_scatter_recursive_doubling");
  if (P == 1) { B.copy(0, L_OUT, 0, 0, L_IN, 0, n); return B; }
  const int64_t N = (int64_t)P * n;
  int TA = B.tmp(N), TB = B.tmp(N);
  Cur cur(P, TA, TB);
  int nst = 0;
  for (int m = 1; m < P; m <<= 1) ++nst;
  int stage = 0;
  for (int mask = 1; mask < P; mask <<= 1, ++stage) {
    bool last = stage == nst - 1;
    std::vector<int> nxt(P);
    for (int r = 0; r < P; ++r) {
      int dst = r ^ mask;
      int my_root = (r >> stage) << stage;
      int dst_root = (dst >> stage) << stage;
      int big_root = (r >> (stage + 1)) << (stage + 1);  // subtree after this stage
      int big_end = std::min(P, big_root + 2 * mask);
      // who supplies the partner subtree's partial sums
      int src = -1;
      int completed = std::max(0, std::min(P, dst_root + mask) - dst_root);  // existing members
      if (dst < P) src = dst;
      else if (completed > 0) src = dst_root + (r - my_root) % completed;  // forwarded data, fetched directly
      int d = cur.next(r);
      nxt[r] = d;
      // blocks still needed afterwards: everything outside the merged subtree, plus my own
      auto emit = [&](int blo, int bhi, int dbuf, int64_t doff) {
        if (bhi <= blo) return;
        std::vector<Src> s{Src{r, cur.buf[r], (int64_t)blo * n}};
        if (src >= 0) s.push_back(Src{src, cur.buf[src], (int64_t)blo * n});
        if (dst_root < my_root) std::swap(s.front(), s.back());
        B.reduce(r, dbuf, doff, s, (int64_t)(bhi - blo) * n, false, last ? OPF_FINAL : 0);
      };
      if (last) { emit(r, r + 1, L_OUT, 0); continue; }
      emit(0, big_root, d, 0);
      emit(big_end, P, d, (int64_t)big_end * n);
      emit(r, r + 1, d, (int64_t)r * n);
    }
    for (int r = 0; r < P; ++r) cur.buf[r] = nxt[r];
  }
  return B;
}

// radix-k recursive exchange reduce-scatter over the whole communicator
Builder gen_rs_radix(int P, int64_t n, int k) {
  Builder B(P, (int64_t)P * n, n, "reduce_scatter_radix");
  if (P == 1) { B.copy(0, L_OUT, 0, 0, L_IN, 0, n); return B; }
  Recexch rx(P, k);
  const int64_t N = (int64_t)P * n;
  int ACC = B.tmp(N);
  std::vector<int> cur(P, L_IN);
  for (int r = 0; r < P; ++r) {
    std::vector<int> fl = rx.folded_into(r);
    if (fl.empty()) continue;
    std::vector<Src> s{Src{r, L_IN, 0}};
    for (int q : fl) s.push_back(Src{q, L_IN, 0});
    B.reduce(r, ACC, 0, s, N, false);
    cur[r] = ACC;
  }
  for (int p = rx.log - 1; p >= 0; --p) {
    std::vector<int> nxt = cur;
    for (int r = 0; r < P; ++r) {
      if (!rx.participates(r)) continue;
      int off, cnt;
      rx.range(r, p, &off, &cnt);
      std::vector<Src> s;
      bool acc = cur[r] == ACC;
      if (!acc) s.push_back(Src{r, L_IN, (int64_t)off * n});
      for (int q : rx.neighbours(r, p)) s.push_back(Src{q, cur[q], (int64_t)off * n});
      B.reduce(r, ACC, (int64_t)off * n, s, (int64_t)cnt * n, acc, p == 0 ? OPF_FINAL : 0);
      nxt[r] = ACC;
    }
    cur = nxt;
  }
  for (int r = 0; r < P; ++r) {
    if (rx.participates(r)) B.copy(r, L_OUT, 0, r, cur[r], (int64_t)r * n, n);
    else B.copy(r, L_OUT, 0, rx.partner(r), ACC, (int64_t)r * n, n);
  }
  return B;
}

// ============================ allgather baselines ===================================
// radix-k Bruck over the whole communicator, blocks written to final positions
Builder gen_ag_kbruck(int P, int64_t n, int k) {
  if (k < 2) throw std::runtime_error("radix must be >= 2");
  Builder B(P, n, (int64_t)P * n, "allgather_k_brucks");
  for (int r = 0; r < P; ++r) B.copy(r, L_OUT, (int64_t)r * n, r, L_IN, 0, n);
  int L = num_phases(P, k);
  for (int i = 0; i < L; ++i) {
    int64_t delta = ipow(k, i);
    for (int r = 0; r < P; ++r)
      for (int j = 1; j < k; ++j) {
        if (j * delta >= P) break;
        int src = (int)((r + j * delta) % P);
        int len = (int)std::min<int64_t>(delta, P - j * delta);
        // src holds blocks src, src+1, ... (mod P); its own block is read from its input
        B.copy(r, L_OUT, (int64_t)src * n, src, L_IN, 0, n);
        int q = 1;
        while (q < len) {
          int blk = (src + q) % P;
          int run = std::min(len - q, P - blk);
          B.copy(r, L_OUT, (int64_t)blk * n, src, L_OUT, (int64_t)blk * n, (int64_t)run * n);
          q += run;
        }
      }
  }
  return B;
}

Builder gen_ag_ring(int P, int64_t n) {
  Builder B(P, n, (int64_t)P * n, "allgather_ring");
  std::vector<int64_t> off(P + 1), cnt(P, n);
  for (int i = 0; i <= P; ++i) off[i] = (int64_t)i * n;
  for (int r = 0; r < P; ++r) B.copy(r, L_OUT, off[r], r, L_IN, 0, n);
  ring_ag(B, P, L_OUT, off, cnt, true);
  return B;
}

Builder gen_ag_recursive_doubling(int P, int64_t n) {
  if (P & (P - 1)) throw std::runtime_error("allgather_recursive_doubling needs a power-of-two number of ranks");
  Builder B(P, n, (int64_t)P * n, "allgather_recursive_doubling");
  for (int r = 0; r < P; ++r) B.copy(r, L_OUT, (int64_t)r * n, r, L_IN, 0, n);
  for (int mask = 1; mask < P; mask <<= 1)
    for (int r = 0; r < P; ++r) {
      int dst = r ^ mask;
      int root = dst & ~(mask - 1);
      if (mask == 1) B.copy(r, L_OUT, (int64_t)dst * n, dst, L_IN, 0, n);
      else B.copy(r, L_OUT, (int64_t)root * n, dst, L_OUT, (int64_t)root * n, (int64_t)mask * n);
    }
  return B;
}

// flat linear exchange: every rank fetches every block from its owner
Builder gen_ag_linear(int P, int64_t n) {
  Builder B(P, n, (int64_t)P * n, "allgather_linear");
  for (int r = 0; r < P; ++r)
    for (int i = 0; i < P; ++i) {
      int q = (r + i) % P;
      B.copy(r, L_OUT, (int64_t)q * n, q, L_IN, 0, n);
    }
  return B;
}

// k-nomial gather of one block per rank to `root` (building block kept by the
// reference next to the Bruck baseline); out = P*n at the root, untouched elsewhere.
Builder gen_gather_knomial(int P, int64_t n, int k, int root) {
  if (k < 2) throw std::runtime_error("radix must be >= 2");
  if (root < 0 || root >= P) throw std::runtime_error("root out of range");
  Builder B(P, n, (int64_t)P * n, "gather_k_nomial");
  int KG = B.tmp((int64_t)P * n);
  int L = num_phases(P, k);
  for (int p = 0; p < L; ++p) {
    int64_t delta = ipow(k, p), gsz = delta * k;
    for (int64_t x = 0; x < P; x += gsz) {
      int parent = (int)((x + root) % P);
      for (int j = 1; j < k; ++j) {
        int64_t c = x + j * delta;
        if (c >= P) break;
        int64_t len = std::min<int64_t>(delta, P - c);
        int child = (int)((c + root) % P);
        B.copy(parent, KG, c * n, child, L_IN, 0, n);
        if (len > 1) B.copy(parent, KG, (c + 1) * n, child, KG, (c + 1) * n, (len - 1) * n);
      }
    }
  }
  // un-rotate at the root
  B.copy(root, L_OUT, (int64_t)root * n, root, L_IN, 0, n);
  if (P - root - 1 > 0) B.copy(root, L_OUT, (int64_t)(root + 1) * n, root, KG, n, (int64_t)(P - root - 1) * n);
  if (root > 0) B.copy(root, L_OUT, 0, root, KG, (int64_t)(P - root) * n, (int64_t)root * n);
  return B;
}

}  // namespace chb

// ============================ building blocks on sub-groups =========================
// The reference keeps the phases of its hierarchical collectives as stand-alone
// functions over the whole communicator with the group structure inside
// (intra_allgather_k_brucks, inter_allgather_linear:
//  testing/custom_implementations/work_dir/all_gather/outdated_versions/intra_allgather_k_brucks.cpp:22-256,
//  inter_allgather_linear.cpp:12-55; intra_reduce_scatter_radix_batch, inter_reduce_linear,
//  intra_scatter_radix_batch: work_dir/reduce_scatter/intra_reduce_scatter_radix.cpp:208-541,
//  inter_linear_reduce.cpp:11-73, intra_scatter_radix_batch.cpp:11-110).
// Here a phase is a flat algorithm embedded once per group of b consecutive
// ranks ("intra") or once per lane of equal in-group slot ("inter"):
//   intra: collective among ranks g*b .. g*b+b-1       (sub-communicator size b)
//   inter: collective among ranks r, r+b, r+2b, ...     (sub-communicator size P/b)
namespace chb {
Builder build_algorithm(const AlgoSpec& s);

Builder gen_grouped(const std::string& coll, const std::string& flat_algo, int P, int64_t count, int k, int b,
                    bool lanes) {
  if (b < 1 || P % b) throw std::runtime_error("group size b must divide the number of ranks");
  const int sub_p = lanes ? P / b : b;
  AlgoSpec ss;
  ss.coll = coll;
  ss.algo = flat_algo;
  ss.P = sub_p;
  ss.k = k;
  ss.b = 1;
  ss.count = count;
  Builder sub = build_algorithm(ss);
  // same buffer lengths as the sub-program; every rank belongs to exactly one sub-communicator
  int64_t in_e = coll == "allgather" ? count : (coll == "allreduce" ? count : count * sub_p);
  int64_t out_e = coll == "allgather" ? count * sub_p : count;
  Builder B(P, in_e, out_e, std::string(lanes ? "inter_" : "intra_") + coll + "_" + flat_algo);
  int tmp_base = -1;
  const int nsub = P / sub_p;
  for (int g = 0; g < nsub; ++g) {
    std::vector<int> map(sub_p);
    for (int i = 0; i < sub_p; ++i) map[i] = lanes ? i * b + g : g * b + i;
    tmp_base = B.embed(sub, map, tmp_base);
  }
  return B;
}
}  // namespace chb

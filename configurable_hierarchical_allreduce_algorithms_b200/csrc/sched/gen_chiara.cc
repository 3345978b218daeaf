// Hierarchical radix-k / group-b collectives (allgather, reduce-scatter,
// allreduce) as pull step programs.
//
// Behaviour reproduced (not code): the three-phase hierarchy of
//   testing/custom_implementations/work_dir/all_gather/all_gather_radix_batch_1_0.cpp:37-377
//   testing/custom_implementations/work_dir/reduce_scatter/reduce_scatter_radix_batch.cpp:200-653
//   testing/custom_implementations/work_dir/all_reduce/all_reduce_radix_batch.cpp:202-788
// Ranks form G = P/b contiguous groups of b; a radix-k algorithm runs inside
// each group, a flat exchange runs between groups along lanes of equal
// in-group slot, and a second radix-k algorithm runs inside each group.
//
// Differences that follow from the pull formulation on a switch:
//   * the k-1 neighbour exchanges of one round are one multi-source step,
//   * every block is written straight to its final position, so the
//     un-rotation after the k-nomial gather and the rotation after the k-ary
//     Bruck rounds disappear into the addressing,
//   * the S stages of the intra-group phases are independent and end up in
//     the same rounds,
//   * a folded-out slot's partial result is fetched from the slot that
//     absorbed it instead of being handed back first.
#include <algorithm>
#include <stdexcept>

#include "algos.h"

namespace chb {

int64_t ipow(int64_t base, int exp) {
  int64_t r = 1;
  while (exp-- > 0) r *= base;
  return r;
}

int num_phases(int b, int k) {
  int L = 0;
  for (int x = b - 1; x > 0; x /= k) ++L;
  return L;
}

// ------------------------------- Recexch ------------------------------------------
Recexch::Recexch(int n_, int k_) : n(n_), k(k_) {
  if (n < 1) throw std::runtime_error("recexch: need at least one rank");
  if (k < 2) throw std::runtime_error("recexch: radix must be >= 2");
  if (n < k) k = std::max(n, 2);
  p_of_k = 1;
  log = 0;
  while ((int64_t)p_of_k * k <= n) { p_of_k *= k; ++log; }
  rem = n - p_of_k;
  T = (int)((int64_t)rem * k / (k - 1));
}
bool Recexch::participates(int r) const { return !(r < T && r % k != k - 1); }
int Recexch::partner(int r) const {
  int p = r + (k - 1 - r % k);
  return p > T - 1 ? T : p;
}
std::vector<int> Recexch::folded_into(int r) const {
  std::vector<int> v;
  if (r < T) {
    if (r % k == k - 1)
      for (int j = 1; j < k; ++j) v.push_back(r - j);
  } else if (r == T && T % k != 0) {
    for (int j = 1; j <= T % k; ++j) v.push_back(T - j);
  }
  return v;
}
int Recexch::step2rank(int r) const {
  if (r < T) return (r % k == k - 1) ? r / k : -1;
  return r - rem;
}
int Recexch::orig(int s) const {
  if (s < 0) return -1;
  return s < rem / (k - 1) ? s * k + (k - 1) : s + rem;
}
std::vector<int> Recexch::neighbours(int r, int phase) const {
  std::vector<int> v;
  int s = step2rank(r);
  if (s < 0) return v;
  int64_t pw = ipow(k, phase);
  int digit = (int)((s / pw) % k);
  for (int d = 0; d < k; ++d) {
    if (d == digit) continue;
    int64_t t = s + (int64_t)(d - digit) * pw;
    if (t >= 0 && t < p_of_k) v.push_back(orig((int)t));
  }
  return v;
}
void Recexch::range(int r, int phase, int* offset, int* count) const {
  int s = step2rank(r);
  int64_t pw = ipow(k, phase);
  int lo = (int)(s / pw * pw) - 1;
  int hi = (int)(lo + pw);
  *offset = orig(lo) + 1;
  *count = orig(hi) - orig(lo);
}

namespace {

struct Geo {
  int P, b, G, S, U, L, k;
  int64_t n;
  Geo(int P_, int b_, int k_, int64_t n_) : P(P_), b(b_), k(k_), n(n_) {
    if (b < 1) throw std::runtime_error("group size b must be >= 1");
    if (k < 2) throw std::runtime_error("radix k must be >= 2");
    if (P % b != 0) throw std::runtime_error("group size b must divide the number of ranks");
    G = P / b;
    S = G / b;
    U = G % b;
    L = num_phases(b, k);
  }
  int rank_of(int g, int slot) const { return g * b + slot; }
  int nstages() const { return S + (U ? 1 : 0); }
  // number of populated chunks (destination / source groups) in stage s
  int stage_width(int s) const { return s < S ? b : U; }
};

// Emit copies of the slot set { (first + q) % b : 0 <= q < len, slot < limit }
// as at most a few contiguous runs; f(slot_begin, run_len) is called per run.
template <class F>
void cyclic_runs(int first, int len, int b, int limit, F f) {
  int q = 0;
  while (q < len) {
    int slot = (first + q) % b;
    int run = std::min(len - q, b - slot);  // until wrap
    // clip [slot, slot+run) to [0, limit)
    int lo = slot, hi = std::min(slot + run, limit);
    if (hi > lo) f(lo, hi - lo);
    q += run;
  }
}

// ---- allgather phase 1: k-nomial gather of the group's b blocks to the slot
// g % b, kept in normalised order in KG (position x = distance from the root).
// The root's own block stays in IN.
void ag_knomial_gather(Builder& B, const Geo& g, int KG, int IB, int64_t IO) {
  for (int grp = 0; grp < g.G; ++grp) {
    int root_local = grp % g.b;
    for (int p = 0; p < g.L; ++p) {
      int64_t delta = ipow(g.k, p), gsz = delta * g.k;
      for (int x = 0; x < g.b; x += (int)gsz) {  // subtree roots of this phase
        int parent = g.rank_of(grp, (x + root_local) % g.b);
        for (int j = 1; j < g.k; ++j) {
          int64_t c = x + j * delta;
          if (c >= g.b) break;
          int64_t len = std::min<int64_t>(delta, g.b - c);
          int child = g.rank_of(grp, (int)((c + root_local) % g.b));
          B.copy(parent, KG, c * g.n, child, IB, IO, g.n);
          if (len > 1) B.copy(parent, KG, (c + 1) * g.n, child, KG, (c + 1) * g.n, (len - 1) * g.n);
        }
      }
    }
  }
}

// Copy group `grp`'s chunk (b blocks, group order) from its root's gather
// buffer into `dst_rank`'s OUT at the final position, un-rotating on the fly.
void ag_fetch_chunk_from_root(Builder& B, const Geo& g, int KG, int grp, int dst_rank, int IB, int64_t IO) {
  int root_local = grp % g.b;
  int root = g.rank_of(grp, root_local);
  int64_t base = (int64_t)grp * g.b * g.n;
  // normalised x = 0 -> slot root_local, from the root's IN
  B.copy(dst_rank, L_OUT, base + root_local * g.n, root, IB, IO, g.n);
  // x in [1, b-root_local) -> slots root_local+1 .. b-1
  int64_t run1 = g.b - root_local - 1;
  if (run1 > 0) B.copy(dst_rank, L_OUT, base + (root_local + 1) * g.n, root, KG, g.n, run1 * g.n);
  // x in [b-root_local, b) -> slots 0 .. root_local-1
  if (root_local > 0)
    B.copy(dst_rank, L_OUT, base, root, KG, (int64_t)(g.b - root_local) * g.n, (int64_t)root_local * g.n);
}

// ---- allgather phase 3: k-ary Bruck rounds inside every group, one stage per
// block of b source groups, writing each chunk to its final OUT position.
// chunk_elems = elements per group chunk (b*n).
void ag_kbruck_stages(Builder& B, const Geo& g, int64_t chunk_elems) {
  if (g.b == 1) return;
  for (int grp = 0; grp < g.G; ++grp)
    for (int s = 0; s < g.nstages(); ++s) {
      int width = g.stage_width(s);
      for (int i = 0; i < g.L; ++i) {
        int64_t delta = ipow(g.k, i);
        for (int r = 0; r < g.b; ++r) {
          int me = g.rank_of(grp, r);
          for (int j = 1; j < g.k; ++j) {
            if (j * delta >= g.b) break;
            int src_slot = (int)((r + j * delta) % g.b);
            int len = (int)std::min<int64_t>(delta, g.b - j * delta);
            int src = g.rank_of(grp, src_slot);
            cyclic_runs(src_slot, len, g.b, width, [&](int slot, int run) {
              int64_t off = ((int64_t)s * g.b + slot) * chunk_elems;
              B.copy(me, L_OUT, off, src, L_OUT, off, (int64_t)run * chunk_elems);
            });
          }
        }
      }
    }
}

// ---- reduce-scatter fold + phase 1: radix-k recursive exchange inside every
// group on chunks of chunk_elems, all stages.  On return cur_buf[slot] names
// the logical buffer holding slot's partial sums (IN when nothing was done),
// and holder[slot] the slot whose buffer holds the partial for chunk `slot`.
struct RsIntra {
  std::vector<int> cur_buf;  // per slot: L_IN or ACC
  std::vector<int> holder;   // per slot
};

RsIntra rs_intra(Builder& B, const Geo& g, int ACC, int64_t chunk_elems) {
  RsIntra out;
  out.cur_buf.assign(g.b, L_IN);
  out.holder.resize(g.b);
  Recexch rx(g.b, g.k);
  const int64_t total = (int64_t)g.P / g.b * chunk_elems;  // whole input (G chunks)
  // fold: a slot that does not take part hands its whole input to a partner
  for (int grp = 0; grp < g.G; ++grp)
    for (int slot = 0; slot < g.b; ++slot) {
      std::vector<int> f = rx.folded_into(slot);
      if (f.empty()) continue;
      std::vector<Src> srcs{Src{g.rank_of(grp, slot), L_IN, 0}};
      for (int q : f) srcs.push_back(Src{g.rank_of(grp, q), L_IN, 0});
      B.reduce(g.rank_of(grp, slot), ACC, 0, srcs, total, false);
    }
  for (int slot = 0; slot < g.b; ++slot)
    if (!rx.folded_into(slot).empty()) out.cur_buf[slot] = ACC;
  // exchange phases
  for (int p = rx.log - 1; p >= 0; --p) {
    for (int grp = 0; grp < g.G; ++grp)
      for (int slot = 0; slot < g.b; ++slot) {
        if (!rx.participates(slot)) continue;
        int off, cnt;
        rx.range(slot, p, &off, &cnt);
        std::vector<int> nb = rx.neighbours(slot, p);
        int me = g.rank_of(grp, slot);
        for (int s = 0; s < g.nstages(); ++s) {
          int width = g.stage_width(s);
          int lo = off, hi = std::min(off + cnt, width);
          if (hi <= lo) continue;
          int64_t eoff = ((int64_t)s * g.b + lo) * chunk_elems;
          int64_t ecnt = (int64_t)(hi - lo) * chunk_elems;
          std::vector<Src> srcs;
          bool acc = (out.cur_buf[slot] == ACC);
          if (!acc) srcs.push_back(Src{me, L_IN, eoff});
          for (int q : nb) srcs.push_back(Src{g.rank_of(grp, q), out.cur_buf[q], eoff});
          B.reduce(me, ACC, eoff, srcs, ecnt, acc);
        }
      }
    for (int slot = 0; slot < g.b; ++slot)
      if (rx.participates(slot)) out.cur_buf[slot] = ACC;
  }
  for (int slot = 0; slot < g.b; ++slot) {
    if (rx.participates(slot)) {
      int off, cnt;
      rx.range(slot, 0, &off, &cnt);
      for (int q = off; q < off + cnt; ++q) out.holder[q] = slot;
    }
  }
  return out;
}

// ---- inter-group linear reduce along lanes: the lane root of destination
// group d sums the G partial chunks (its own group's included) in one pass.
void rs_lane_reduce(Builder& B, const Geo& g, const RsIntra& ri, int dst_buf, bool dst_is_out_chunk,
                    int64_t chunk_elems, uint32_t flags) {
  for (int d = 0; d < g.G; ++d) {
    int lane = d % g.b;
    int root = g.rank_of(d, lane);
    int h = ri.holder[lane];
    std::vector<Src> srcs;
    // own group first, then the others in group order (the order the reference
    // posts its receives in)
    srcs.push_back(Src{g.rank_of(d, h), ri.cur_buf[h], (int64_t)d * chunk_elems});
    for (int q = 0; q < g.G; ++q)
      if (q != d) srcs.push_back(Src{g.rank_of(q, h), ri.cur_buf[h], (int64_t)d * chunk_elems});
    B.reduce(root, dst_buf, dst_is_out_chunk ? (int64_t)d * chunk_elems : 0, srcs, chunk_elems, false, flags);
  }
}

// ---- k-nomial scatter inside every group from the rotating root (slot grp % b), whose b blocks sit
// in `src_buf` in slot order: every rank ends with its own block in OUT; SC (b*n per rank,
// normalised order) carries the runs that a subtree root hands on.  Children pull their run.
void rs_knomial_scatter(Builder& B, const Geo& g, int src_buf, int SC) {
  const int64_t n = g.n;
  for (int grp = 0; grp < g.G; ++grp) {
    int root_local = grp % g.b;
    int root = g.rank_of(grp, root_local);
    B.copy(root, L_OUT, 0, root, src_buf, (int64_t)root_local * n, n);
    for (int p = g.L - 1; p >= 0; --p) {
      int64_t delta = ipow(g.k, p), gsz = delta * g.k;
      for (int64_t x = 0; x < g.b; x += gsz) {
        int64_t block_end = std::min<int64_t>(x + gsz, g.b);
        int parent = g.rank_of(grp, (int)((x + root_local) % g.b));
        for (int j = 1; j < g.k; ++j) {
          int64_t c = x + j * delta;
          if (c >= block_end) break;
          int64_t len = std::min<int64_t>(delta, block_end - c);
          int child = g.rank_of(grp, (int)((c + root_local) % g.b));
          if (x == 0) {
            // parent is the root: blocks live in src_buf in slot order
            int slot = (int)((c + root_local) % g.b);
            B.copy(child, L_OUT, 0, root, src_buf, (int64_t)slot * n, n);
            if (len > 1)
              cyclic_runs((int)((c + 1 + root_local) % g.b), (int)len - 1, g.b, g.b, [&](int s0, int run) {
                int64_t xpos = ((s0 - root_local + g.b) % g.b);
                B.copy(child, SC, xpos * n, root, src_buf, (int64_t)s0 * n, (int64_t)run * n);
              });
          } else {
            B.copy(child, L_OUT, 0, parent, SC, c * n, n);
            if (len > 1) B.copy(child, SC, (c + 1) * n, parent, SC, (c + 1) * n, (len - 1) * n);
          }
        }
      }
    }
  }
}

}  // namespace

// =============================== allgather ======================================
// Emits the three allgather phases; every rank's own block is read from
// (IB, IO) so that the allreduce variants can chain it after a reduce-scatter.
void emit_ag_radix_batch(Builder& B, int P, int64_t n, int k, int b, int IB, int64_t IO) {
  Geo g(P, b, k, n);
  int KG = g.b > 1 ? B.tmp((int64_t)g.b * n) : -1;
  // phase 1
  if (g.b > 1) ag_knomial_gather(B, g, KG, IB, IO);
  // phase 2: every member of lane (grp % b) fetches grp's chunk from its root
  for (int grp = 0; grp < g.G; ++grp) {
    int lane = grp % g.b;
    for (int q = 0; q < g.G; ++q) {
      int dst = g.rank_of(q, lane);
      if (g.b > 1) ag_fetch_chunk_from_root(B, g, KG, grp, dst, IB, IO);
      else B.copy(dst, L_OUT, (int64_t)grp * n, g.rank_of(grp, 0), IB, IO, n);
    }
  }
  // phase 3
  ag_kbruck_stages(B, g, (int64_t)g.b * n);
}

Builder gen_ag_radix_batch(int P, int64_t n, int k, int b) {
  Builder B(P, n, (int64_t)P * n, "allgather_radix_batch");
  emit_ag_radix_batch(B, P, n, k, b, L_IN, 0);
  return B;
}

// =============================== reduce-scatter =================================
Builder gen_rs_radix_batch(int P, int64_t n, int k, int b) {
  Geo g(P, b, k, n);
  Builder B(P, (int64_t)P * n, n, "reduce_scatter_radix_batch");
  const int64_t chunk = (int64_t)g.b * n;
  if (g.b == 1) {
    // flat: every rank sums its block over all ranks in one pass
    RsIntra ri;
    ri.cur_buf.assign(1, L_IN);
    ri.holder.assign(1, 0);
    rs_lane_reduce(B, g, ri, L_OUT, false, chunk, OPF_FINAL);
    return B;
  }
  int ACC = B.tmp((int64_t)P * n);
  int RED = B.tmp(chunk);
  int SC = B.tmp(chunk);
  RsIntra ri = rs_intra(B, g, ACC, chunk);
  rs_lane_reduce(B, g, ri, RED, false, chunk, OPF_FINAL);
  // phase 3: k-nomial scatter from the rotating root, children pull their run
  rs_knomial_scatter(B, g, RED, SC);
  return B;
}

// =============================== allreduce ======================================
Builder gen_ar_radix_batch(int P, int64_t N, int k, int b) {
  if (N % P != 0) throw std::runtime_error("allreduce_radix_batch: count must be a multiple of the number of ranks");
  int64_t n = N / P;
  Geo g(P, b, k, n);
  Builder B(P, N, N, "all_reduce_radix_batch");
  const int64_t chunk = (int64_t)g.b * n;
  RsIntra ri;
  if (g.b == 1) {
    ri.cur_buf.assign(1, L_IN);
    ri.holder.assign(1, 0);
  } else {
    int ACC = B.tmp(N);
    ri = rs_intra(B, g, ACC, chunk);
  }
  // inter-group reduce: the lane root of group d produces chunk d of the result
  rs_lane_reduce(B, g, ri, L_OUT, true, chunk, OPF_FINAL);
  // inter-group broadcast along lanes
  for (int d = 0; d < g.G; ++d) {
    int lane = d % g.b, root = g.rank_of(d, lane);
    for (int q = 0; q < g.G; ++q)
      if (q != d) B.copy(g.rank_of(q, lane), L_OUT, (int64_t)d * chunk, root, L_OUT, (int64_t)d * chunk, chunk);
  }
  // intra-group k-ary Bruck per stage
  ag_kbruck_stages(B, g, chunk);
  return B;
}

// =============================== stand-alone phases ==============================
// The reference keeps the phases of its hierarchical collectives as functions of their own, with
// their own buffer layouts, to test them one at a time:
//   testing/custom_implementations/work_dir/all_gather/outdated_versions/all_gather_0_3_beta.cpp:36 (intra_gather_k_nomial),
//   :141 (intra_allgather_k_brucks), :377 (inter_allgather_linear);
//   testing/custom_implementations/work_dir/reduce_scatter/intra_reduce_scatter_radix.cpp:208-541,
//   .../inter_linear_reduce.cpp:11-73, .../intra_scatter_radix_batch.cpp:11-110.
// Here each is a program with the same inputs and outputs (c = elements per block or chunk):
//   intra_gather_k_nomial            in c            out b*c        group root: the group's blocks in slot order
//   inter_allgather_linear           in b*c          out T*b*c      entry s: the chunk of group s*b + lane, from its lane root
//   intra_allgather_k_brucks         in T*c          out G*c        stage s: block s of every slot, in slot order
//   intra_reduce_scatter_radix_batch in P*c          out T*b*c      entry s: chunk of group s*b + slot summed over my group
//   inter_reduce_linear              in T*b*c        out b*c        lane root of group d: entry d/b summed over the lane
//   intra_scatter_radix_batch        in b*c          out c          block `slot` of the group root's input
// with T = ceil(G / b) stages; entries without a source (the last stage when G % b != 0) stay untouched.
Builder gen_phase(const std::string& name, int P, int64_t c, int k, int b) {
  Geo g(P, b, k, c);
  const int T = g.nstages();
  const int64_t chunk = (int64_t)g.b * c;
  if (name == "intra_gather_k_nomial") {
    Builder B(P, c, chunk, name);
    if (g.b == 1) {
      for (int r = 0; r < P; ++r) B.copy(r, L_OUT, 0, r, L_IN, 0, c);
      return B;
    }
    int KG = B.tmp(chunk);
    ag_knomial_gather(B, g, KG, L_IN, 0);
    for (int grp = 0; grp < g.G; ++grp) {   // the root un-rotates once (own block from its input)
      int root_local = grp % g.b, root = g.rank_of(grp, root_local);
      B.copy(root, L_OUT, (int64_t)root_local * c, root, L_IN, 0, c);
      int64_t run1 = g.b - root_local - 1;
      if (run1 > 0) B.copy(root, L_OUT, (int64_t)(root_local + 1) * c, root, KG, c, run1 * c);
      if (root_local > 0) B.copy(root, L_OUT, 0, root, KG, (int64_t)(g.b - root_local) * c, (int64_t)root_local * c);
    }
    return B;
  }
  if (name == "inter_allgather_linear") {
    Builder B(P, chunk, (int64_t)T * chunk, name);
    for (int d = 0; d < g.G; ++d) {
      int lane = d % g.b, root = g.rank_of(d, lane);
      for (int q = 0; q < g.G; ++q) B.copy(g.rank_of(q, lane), L_OUT, (int64_t)(d / g.b) * chunk, root, L_IN, 0, chunk);
    }
    return B;
  }
  if (name == "intra_allgather_k_brucks") {
    Builder B(P, (int64_t)T * c, (int64_t)g.G * c, name);
    Geo gc(P, b, k, c);
    for (int grp = 0; grp < g.G; ++grp)
      for (int s = 0; s < T; ++s)
        for (int slot = 0; slot < g.stage_width(s); ++slot) {
          int me = g.rank_of(grp, slot);
          B.copy(me, L_OUT, ((int64_t)s * g.b + slot) * c, me, L_IN, (int64_t)s * c, c);
        }
    ag_kbruck_stages(B, gc, c);
    return B;
  }
  if (name == "intra_reduce_scatter_radix_batch") {
    Builder B(P, (int64_t)P * c, (int64_t)T * chunk, name);
    if (g.b == 1) {
      for (int r = 0; r < P; ++r) B.copy(r, L_OUT, 0, r, L_IN, 0, (int64_t)P * c);
      return B;
    }
    int ACC = B.tmp((int64_t)P * c);
    RsIntra ri = rs_intra(B, g, ACC, chunk);
    for (int grp = 0; grp < g.G; ++grp)
      for (int slot = 0; slot < g.b; ++slot) {
        int h = ri.holder[slot];
        for (int s = 0; s < T; ++s) {
          int d = s * g.b + slot;
          if (d >= g.G) continue;
          B.copy(g.rank_of(grp, slot), L_OUT, (int64_t)s * chunk, g.rank_of(grp, h), ri.cur_buf[h], (int64_t)d * chunk, chunk);
        }
      }
    return B;
  }
  if (name == "inter_reduce_linear") {
    Builder B(P, (int64_t)T * chunk, chunk, name);
    for (int d = 0; d < g.G; ++d) {
      int lane = d % g.b, root = g.rank_of(d, lane);
      std::vector<Src> srcs{Src{root, L_IN, (int64_t)(d / g.b) * chunk}};     // own contribution first, like the reference
      for (int q = 0; q < g.G; ++q)
        if (q != d) srcs.push_back(Src{g.rank_of(q, lane), L_IN, (int64_t)(d / g.b) * chunk});
      B.reduce(root, L_OUT, 0, srcs, chunk, false, OPF_FINAL);
    }
    return B;
  }
  if (name == "intra_scatter_radix_batch") {
    Builder B(P, chunk, c, name);
    if (g.b == 1) {
      for (int r = 0; r < P; ++r) B.copy(r, L_OUT, 0, r, L_IN, 0, c);
      return B;
    }
    int SC = B.tmp(chunk);
    rs_knomial_scatter(B, g, L_IN, SC);
    return B;
  }
  throw std::runtime_error("unknown phase: " + name);
}

}  // namespace chb

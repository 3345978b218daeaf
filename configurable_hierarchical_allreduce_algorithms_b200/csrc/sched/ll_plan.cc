#include "ll_plan.h"

#include <algorithm>
#include <cstring>
#include <random>

namespace chb {

std::vector<char> make_ll_blob(const Program& p, int esz, LPHeader* hout) {
  const int P = p.P, T = p.nrounds;
  std::vector<LPLevel> levels((size_t)P * T);
  std::vector<LPStep> steps;
  std::vector<LPSrc> srcs;
  std::vector<std::vector<LPSend>> sends_of((size_t)P * T);
  std::vector<long long> inbox(P, 0);
  LPHeader h{};
  // steps in (rank, level) order; every remote source gets its inbox slot and its owner a send
  for (int r = 0; r < P; ++r)
    for (int t = 0; t < T; ++t) {
      LPLevel& lv = levels[(size_t)r * T + t];
      lv.step_begin = (int)steps.size();
      long long pre = 0;
      for (int oi : p.rr[r][t].ops) {
        const Op& o = p.ops[oi];
        LPStep s{};
        s.dst_off = o.dst_off;
        s.count = o.count;
        s.dst_buf = o.dst_buf;
        s.flags = o.flags | (o.acc ? 0x100u : 0u);
        s.src_begin = (int)srcs.size();
        s.nsrc = (int)o.srcs.size();
        s.line_prefix = pre;
        const long long nl = ll_lines_of(o.count, esz);
        pre += nl;
        for (const Src& x : o.srcs) {
          LPSrc d{x.off, -1, x.peer, x.buf};
          if (x.peer != r) {
            d.inbox_line = inbox[r];
            inbox[r] += nl;
            sends_of[(size_t)x.peer * T + t].push_back(LPSend{x.off, o.count, d.inbox_line, 0, r, x.buf});
          }
          srcs.push_back(d);
        }
        steps.push_back(s);
      }
      lv.step_end = (int)steps.size();
      lv.step_lines = pre;
    }
  // forwarding: a send of level t + 1 whose source lies inside the destination of ONE step of level t (same
  // buffer, offset difference a whole number of lines) is issued by that step's threads instead
  std::vector<std::vector<LPFwd>> fwd_of(steps.size());
  for (int r = 0; r < P; ++r)
    for (int t = 0; t + 1 < T; ++t) {
      const LPLevel& lv = levels[(size_t)r * T + t];
      std::vector<LPSend>& next = sends_of[(size_t)r * T + t + 1];
      std::vector<LPSend> keep;
      for (const LPSend& sd : next) {
        bool done = false;
        for (int si = lv.step_begin; si < lv.step_end && !done; ++si) {
          const LPStep& st = steps[(size_t)si];
          if (st.dst_buf != sd.src_buf || sd.src_off < st.dst_off || sd.src_off + sd.count > st.dst_off + st.count) continue;
          const long long delta = (sd.src_off - st.dst_off) * esz;
          if (delta % 8) continue;
          fwd_of[(size_t)si].push_back(LPFwd{delta / 8, ll_lines_of(sd.count, esz), sd.inbox_line, sd.dst_rank, 0});
          done = true;
        }
        if (!done) keep.push_back(sd);
      }
      next.swap(keep);
    }
  // Every sender starts with the receiver after itself and goes round from there (pushes of a level and
  // forwards of a step alike): at any moment the P senders aim at P different receivers, instead of all
  // filling receiver 0's inbox first, then receiver 1's, ... with one ingress link busy and the others idle.
  auto after = [P](int sender, int dst) { return (dst - sender - 1 + P) % P; };
  std::vector<LPFwd> fwds;
  {
    size_t si = 0;
    for (int r = 0; r < P; ++r)
      for (int t = 0; t < T; ++t) {
        const LPLevel& lv = levels[(size_t)r * T + t];
        for (si = (size_t)lv.step_begin; si < (size_t)lv.step_end; ++si) {
          std::stable_sort(fwd_of[si].begin(), fwd_of[si].end(),
                           [&](const LPFwd& a, const LPFwd& b) { return after(r, a.dst_rank) < after(r, b.dst_rank); });
          steps[si].fwd_begin = (int)fwds.size();
          steps[si].nfwd = (int)fwd_of[si].size();
          for (const LPFwd& f : fwd_of[si]) fwds.push_back(f);
        }
        std::vector<LPSend>& sd = sends_of[(size_t)r * T + t];
        std::stable_sort(sd.begin(), sd.end(),
                         [&](const LPSend& a, const LPSend& b) { return after(r, a.dst_rank) < after(r, b.dst_rank); });
      }
  }
  std::vector<LPSend> sends;
  for (int r = 0; r < P; ++r)
    for (int t = 0; t < T; ++t) {
      LPLevel& lv = levels[(size_t)r * T + t];
      lv.send_begin = (int)sends.size();
      long long pre = 0;
      for (LPSend s : sends_of[(size_t)r * T + t]) {
        s.line_prefix = pre;
        pre += ll_lines_of(s.count, esz);
        sends.push_back(s);
      }
      lv.send_end = (int)sends.size();
      lv.send_lines = pre;
      h.max_level_lines = std::max(h.max_level_lines, lv.send_lines + lv.step_lines);
    }
  // barriers: before level t only if it reads local memory written since the last barrier, or overwrites local
  // memory read or written since then (the caller's input is never written; inbox lines carry their own flags).
  // Two accesses of ONE thread need no barrier, program order is enough: thread g of a rank owns the lines
  // g, g + threads, ... of every phase, so an access at byte off * esz + (line - prefix) * 8 of a buffer belongs to
  // the same thread in both phases, whatever the number of threads, exactly when off * esz - prefix * 8 (the
  // `shift` below) is the same for both; equal shifts also make the line boundaries coincide.
  struct Reg { int buf; long long lo, hi, shift; };
  auto hits = [](const std::vector<Reg>& a, const Reg& x) {
    for (const Reg& y : a)
      if (y.buf == x.buf && x.lo < y.hi && y.lo < x.hi && y.shift != x.shift) return true;
    return false;
  };
  for (int r = 0; r < P; ++r) {
    std::vector<Reg> wr, rd;
    for (int t = 0; t < T; ++t) {
      LPLevel& lv = levels[(size_t)r * T + t];
      std::vector<Reg> reads, writes;
      for (int si = lv.step_begin; si < lv.step_end; ++si) {
        const LPStep& st = steps[(size_t)si];
        const Reg d{st.dst_buf, st.dst_off, st.dst_off + st.count, st.dst_off * esz - st.line_prefix * 8};
        writes.push_back(d);
        if (st.flags & 0x100u) reads.push_back(d);
        for (int j = 0; j < st.nsrc; ++j) {
          const LPSrc& x = srcs[(size_t)st.src_begin + j];
          if (x.inbox_line < 0) reads.push_back(Reg{x.buf, x.off, x.off + st.count, x.off * esz - st.line_prefix * 8});
        }
      }
      for (int i = lv.send_begin; i < lv.send_end; ++i) {
        const LPSend& sd = sends[(size_t)i];
        reads.push_back(Reg{sd.src_buf, sd.src_off, sd.src_off + sd.count, sd.src_off * esz - sd.line_prefix * 8});
      }
      bool need = false;
      for (const Reg& x : reads) need = need || hits(wr, x);
      for (const Reg& x : writes) need = need || hits(wr, x) || hits(rd, x);
      lv.barrier_before = (t > 0 && need) ? 1 : 0;
      lv.all_copy = lv.step_end > lv.step_begin ? 1 : 0;
      for (int si = lv.step_begin; si < lv.step_end; ++si) {
        const LPStep& st = steps[(size_t)si];
        if (st.nsrc != 1 || (st.flags & (0x100u | OPF_FINAL)) || srcs[(size_t)st.src_begin].inbox_line < 0) lv.all_copy = 0;
      }
      if (lv.barrier_before) { wr.clear(); rd.clear(); }
      wr.insert(wr.end(), writes.begin(), writes.end());
      rd.insert(rd.end(), reads.begin(), reads.end());
    }
  }
  h.P = P;
  h.nlevels = T;
  h.nsteps = (int)steps.size();
  h.nsrcs = (int)srcs.size();
  h.nsends = (int)sends.size();
  h.esz = esz;
  for (int r = 0; r < P; ++r) h.inbox_lines = std::max(h.inbox_lines, inbox[r]);
  // every rank's own entries, for executors that keep them close (shared memory on the GPU)
  std::vector<LPRank> ranks((size_t)P);
  for (int r = 0; r < P && T > 0; ++r) {
    LPRank& R = ranks[(size_t)r];
    const LPLevel& first = levels[(size_t)r * T];
    const LPLevel& last = levels[(size_t)r * T + T - 1];
    R.step0 = first.step_begin;
    R.nstep = last.step_end - first.step_begin;
    R.send0 = first.send_begin;
    R.nsend = last.send_end - first.send_begin;
    R.src0 = R.nstep ? steps[(size_t)R.step0].src_begin : 0;
    R.fwd0 = R.nstep ? steps[(size_t)R.step0].fwd_begin : 0;
    for (int i = 0; i < R.nstep; ++i) {
      R.nsrc += steps[(size_t)(R.step0 + i)].nsrc;
      R.nfwd += steps[(size_t)(R.step0 + i)].nfwd;
    }
    const long long bytes = (long long)T * sizeof(LPLevel) + (long long)R.nstep * sizeof(LPStep) + (long long)R.nsrc * sizeof(LPSrc) +
                            (long long)R.nsend * sizeof(LPSend) + (long long)R.nfwd * sizeof(LPFwd);
    h.rank_table_bytes = std::max(h.rank_table_bytes, bytes);
  }
  auto al = [](size_t x) { return (x + 15) / 16 * 16; };
  size_t off = (size_t)kLPRanksOffset;
  h.off_ranks = (long long)off;  off = al(off + ranks.size() * sizeof(LPRank));
  h.off_levels = (long long)off; off = al(off + levels.size() * sizeof(LPLevel));
  h.off_steps = (long long)off;  off = al(off + steps.size() * sizeof(LPStep));
  h.off_srcs = (long long)off;   off = al(off + srcs.size() * sizeof(LPSrc));
  h.off_sends = (long long)off;  off = al(off + sends.size() * sizeof(LPSend));
  h.off_fwds = (long long)off;   off = al(off + fwds.size() * sizeof(LPFwd));
  std::vector<char> blob(off, 0);
  std::memcpy(blob.data(), &h, sizeof(h));
  auto put = [&](long long o, const void* src, size_t n) { if (n) std::memcpy(blob.data() + o, src, n); };
  put(h.off_ranks, ranks.data(), ranks.size() * sizeof(LPRank));
  put(h.off_levels, levels.data(), levels.size() * sizeof(LPLevel));
  put(h.off_steps, steps.data(), steps.size() * sizeof(LPStep));
  put(h.off_srcs, srcs.data(), srcs.size() * sizeof(LPSrc));
  put(h.off_sends, sends.data(), sends.size() * sizeof(LPSend));
  put(h.off_fwds, fwds.data(), fwds.size() * sizeof(LPFwd));
  *hout = h;
  return blob;
}

long long ll_inbox_lines(const Program& p, int esz) {
  long long worst = 0;
  std::vector<long long> inbox(p.P, 0);
  for (const Op& o : p.ops)
    for (const Src& x : o.srcs)
      if (x.peer != o.rank) inbox[o.rank] += ll_lines_of(o.count, esz);
  for (long long v : inbox) worst = std::max(worst, v);
  return worst;
}

// ================================ host execution of the tables ================================
namespace {

template <typename T>
inline T apply_ll(int op, T a, T b) {
  switch (op) {
    case OP_SUM: return a + b;
    case OP_MAX: return a > b ? a : b;
    case OP_MIN: return a < b ? a : b;
    case OP_PROD: return a * b;
  }
  return a;
}

template <typename Item>
int find_item(const Item* items, int begin, int end, long long gl) {
  int lo = begin, hi = end - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (items[mid].line_prefix <= gl) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

struct Line { unsigned char b[8]; };

// 8 payload bytes at byte offset off of a block of nbytes bytes (missing bytes read as zero)
Line load_line(const char* base, long long off, long long nbytes) {
  Line v{};
  for (int i = 0; i < 8 && off + i < nbytes; ++i) v.b[i] = (unsigned char)base[off + i];
  return v;
}
void store_line(char* base, long long off, long long nbytes, const Line& v) {
  for (int i = 0; i < 8 && off + i < nbytes; ++i) base[off + i] = (char)v.b[i];
}

template <typename T>
int simulate_ll_t(const Program& p, int rop, void* const* in, void* const* out, uint64_t seed, int TT,
                  int fault, int launches, std::string* err) {
  constexpr int PE = (int)(8 / sizeof(T));
  LPHeader h{};
  const std::vector<char> blob = make_ll_blob(p, (int)sizeof(T), &h);
  const int P = h.P, NL = h.nlevels;
  const LPLevel* levels = reinterpret_cast<const LPLevel*>(blob.data() + h.off_levels);
  const LPStep* steps = reinterpret_cast<const LPStep*>(blob.data() + h.off_steps);
  const LPSrc* srcs = reinterpret_cast<const LPSrc*>(blob.data() + h.off_srcs);
  const LPSend* sends = reinterpret_cast<const LPSend*>(blob.data() + h.off_sends);
  const LPFwd* fwds = reinterpret_cast<const LPFwd*>(blob.data() + h.off_fwds);
  std::vector<std::vector<T>> work(P);
  // Inbox: two halves that alternate by launch parity, like on the GPU.  tag = number of the launch that wrote the
  // line, plus one (the flag a reader of that launch waits for); a line is overwritten without asking, so a sender
  // that is two launches ahead of a reader destroys a line that was never read, which `unread` catches.
  const size_t NLN = (size_t)h.inbox_lines;
  std::vector<std::vector<Line>> inbox(P);
  std::vector<std::vector<int>> tag(P);
  std::vector<std::vector<unsigned char>> unread(P);
  for (int r = 0; r < P; ++r) {
    work[r].resize((size_t)p.work_elems);
    if (!work[r].empty()) std::memset(work[r].data(), 0xFF, work[r].size() * sizeof(T));
    inbox[r].assign(2 * NLN, Line{});
    tag[r].assign(2 * NLN, 0);
    unread[r].assign(2 * NLN, 0);
  }
  auto base = [&](int rank, int buf) -> char* {
    switch (buf) {
      case P_IN: return (char*)in[rank];
      case P_OUT: return (char*)out[rank];
      default: return (char*)work[rank].data();
    }
  };
  auto deliver = [&](int dst, long long line, const Line& v, int launch) -> bool {
    if (dst < 0 || dst >= P || line < 0 || line >= h.inbox_lines) return false;
    const size_t at = (size_t)(launch & 1) * NLN + (size_t)line;
    if (unread[dst][at]) return false;            // written twice in one launch, or overwritten before it was read
    inbox[dst][at] = v;
    tag[dst][at] = launch + 1;
    unread[dst][at] = 1;
    return true;
  };
  // one virtual thread: where it is in its rank's levels
  struct Thr { int rank, v, level = 0, phase = 0, launch = 0; long long gl = 0; int passed = 0; bool arrived = false, done = false, at_end = false; };
  std::vector<Thr> th;
  for (int r = 0; r < P; ++r)
    for (int v = 0; v < TT; ++v) { Thr t; t.rank = r; t.v = v; t.gl = v; th.push_back(t); }
  std::vector<long long> arrivals(P, 0), finished(P, 0);
  std::string why;
  // advance thread t by one unit (a barrier, or one line); 1 progressed, 0 blocked, -1 error
  auto advance = [&](Thr& t) -> int {
    const int r = t.rank;
    while (true) {
      if (t.level >= NL) {
        // end of a launch: the next kernel of this rank starts when every thread of this one has returned
        if (!t.at_end) { t.at_end = true; ++finished[r]; }
        if (t.launch + 1 >= launches) { t.done = true; return 1; }
        if (finished[r] < (long long)TT * (t.launch + 1)) {
          why = "rank " + std::to_string(r) + " waits for the end of its launch " + std::to_string(t.launch);
          return 0;
        }
        t.at_end = false;
        ++t.launch;
        t.level = 0;
        t.phase = 0;
        return 1;
      }
      const LPLevel& L = levels[(size_t)r * NL + t.level];
      if (t.phase == 0) {
        const bool barrier = L.barrier_before && fault != LL_FAULT_NO_BARRIERS;
        if (barrier) {
          if (!t.arrived) { t.arrived = true; ++arrivals[r]; }
          if (arrivals[r] < (long long)TT * (t.passed + 1)) {
            why = "rank " + std::to_string(r) + " waits at the barrier before level " + std::to_string(t.level);
            return 0;
          }
          t.arrived = false;
          ++t.passed;
        }
        t.phase = 1;
        t.gl = t.v;
        if (barrier) return 1;
      }
      if (t.phase == 1) {
        if (t.gl >= L.send_lines) { t.phase = 2; t.gl = t.v; continue; }
        const LPSend& S = sends[find_item(sends, L.send_begin, L.send_end, t.gl)];
        const long long l = t.gl - S.line_prefix;
        const Line v = load_line(base(r, S.src_buf) + S.src_off * (long long)sizeof(T), l * 8, S.count * (long long)sizeof(T));
        if (!deliver(S.dst_rank, S.inbox_line + l, v, t.launch)) {
          why = "a line pushed by rank " + std::to_string(r) + " in launch " + std::to_string(t.launch) + " meets an unread line in the inbox of rank " + std::to_string(S.dst_rank);
          return -1;
        }
        t.gl += TT;
        return 1;
      }
      if (t.gl >= L.step_lines) { ++t.level; t.phase = 0; continue; }
      const LPStep& st = steps[find_item(steps, L.step_begin, L.step_end, t.gl)];
      const long long l = t.gl - st.line_prefix;
      const long long nbytes = st.count * (long long)sizeof(T);
      for (int j = 0; j < st.nsrc; ++j) {
        const LPSrc& sc = srcs[(size_t)st.src_begin + j];
        if (sc.inbox_line >= 0 && tag[r][(size_t)(t.launch & 1) * NLN + (size_t)(sc.inbox_line + l)] != t.launch + 1) {
          why = "rank " + std::to_string(r) + " level " + std::to_string(t.level) + " waits for line " + std::to_string(l) +
                " from rank " + std::to_string(sc.peer);
          return 0;
        }
      }
      char* dst = base(r, st.dst_buf) + st.dst_off * (long long)sizeof(T);
      const bool acc = (st.flags & 0x100u) != 0;
      T a[PE];
      bool have = false;
      Line v{};
      auto take = [&](const Line& x) {
        T e[PE];
        std::memcpy(e, x.b, 8);
        for (int i = 0; i < PE; ++i) a[i] = have ? apply_ll<T>(rop, a[i], e[i]) : e[i];
        have = true;
      };
      if (acc) take(load_line(dst, l * 8, nbytes));
      for (int j = 0; j < st.nsrc; ++j) {
        const LPSrc& sc = srcs[(size_t)st.src_begin + j];
        if (sc.inbox_line >= 0) {
          const size_t at = (size_t)(t.launch & 1) * NLN + (size_t)(sc.inbox_line + l);
          v = inbox[r][at];
          unread[r][at] = 0;
        } else {
          v = load_line(base(r, sc.buf) + sc.off * (long long)sizeof(T), l * 8, nbytes);
        }
        take(v);
      }
      if (acc || st.nsrc > 1) std::memcpy(v.b, a, 8);
      store_line(dst, l * 8, nbytes, v);
      const int nfwd = fault == LL_FAULT_DROP_A_FORWARD && st.nfwd > 0 ? st.nfwd - 1 : st.nfwd;
      for (int f = 0; f < nfwd; ++f) {
        const LPFwd& F = fwds[(size_t)st.fwd_begin + f];
        const long long lf = l - F.line_begin;
        if (lf >= 0 && lf < F.nlines && !deliver(F.dst_rank, F.inbox_line + lf, v, t.launch)) {
          why = "a line forwarded by rank " + std::to_string(r) + " in launch " + std::to_string(t.launch) + " meets an unread line in the inbox of rank " + std::to_string(F.dst_rank);
          return -1;
        }
      }
      t.gl += TT;
      return 1;
    }
  };
  std::mt19937_64 rng(seed);
  size_t remaining = th.size();
  while (remaining > 0) {
    const size_t n = th.size();
    const size_t start = (size_t)(rng() % n);
    bool moved = false;
    for (size_t i = 0; i < n && !moved; ++i) {
      Thr& t = th[(start + i) % n];
      if (t.done) continue;
      int burst = 1 + (int)(rng() % 4);
      while (burst-- > 0 && !t.done) {
        const int rc = advance(t);
        if (rc < 0) { if (err) *err = why; return -1; }
        if (rc == 0) break;
        moved = true;
        if (t.done) --remaining;
      }
    }
    if (!moved) {
      if (err) *err = "deadlock: " + why;
      return -1;
    }
  }
  return 0;
}

}  // namespace

int simulate_ll(const Program& p, int dtype, int op, void* const* in, void* const* out, uint64_t seed,
                int nthreads, int fault, int launches, std::string* err) {
  if (launches < 1 || launches > 64) { if (err) *err = "simulate_ll: 1 to 64 launches"; return -2; }
  if (nthreads < 1 || nthreads > 4096) { if (err) *err = "simulate_ll: 1 to 4096 threads per rank"; return -2; }
  if ((p.reads_peer_in && !p.in_symmetric) || (p.reads_peer_out && !p.out_symmetric)) {
    if (err) *err = "simulate_ll: the push form wants a program lowered without staging copies";
    return -2;
  }
  switch (dtype) {
    case DT_F32: return simulate_ll_t<float>(p, op, in, out, seed, nthreads, fault, launches, err);
    case DT_F64: return simulate_ll_t<double>(p, op, in, out, seed, nthreads, fault, launches, err);
    case DT_I32: return simulate_ll_t<int32_t>(p, op, in, out, seed, nthreads, fault, launches, err);
    case DT_I64: return simulate_ll_t<int64_t>(p, op, in, out, seed, nthreads, fault, launches, err);
    case DT_U8: return simulate_ll_t<uint8_t>(p, op, in, out, seed, nthreads, fault, launches, err);
  }
  if (err) *err = "simulate_ll: unsupported dtype on the host";
  return -2;
}

}  // namespace chb

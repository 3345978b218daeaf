// Builder, lowering (buffer placement, dependency analysis, round assignment),
// host simulator and static verifier for step programs.  See program.h.
#include "program.h"

#include <algorithm>
#include <cstring>
#include <map>
#include <random>
#include <sstream>
#include <stdexcept>

namespace chb {

int dtype_size(int dt) {
  switch (dt) {
    case DT_F32: return 4;
    case DT_BF16: return 2;
    case DT_F16: return 2;
    case DT_I32: return 4;
    case DT_F64: return 8;
    case DT_I64: return 8;
    case DT_U8: return 1;
  }
  return 0;
}

Builder::Builder(int P, int64_t in_elems, int64_t out_elems, std::string name)
    : P_(P), in_elems_(in_elems), out_elems_(out_elems), name_(std::move(name)) {}

int Builder::tmp(int64_t elems) {
  tmp_elems_.push_back(elems);
  return L_TMP0 + (int)tmp_elems_.size() - 1;
}

void Builder::copy(int rank, int dbuf, int64_t doff, int speer, int sbuf, int64_t soff,
                   int64_t count, uint32_t flags) {
  if (count <= 0) return;
  reduce(rank, dbuf, doff, {Src{speer, sbuf, soff}}, count, false, flags);
}

void Builder::reduce(int rank, int dbuf, int64_t doff, const std::vector<Src>& srcs,
                     int64_t count, bool acc, uint32_t flags) {
  if (count <= 0) return;
  if (srcs.empty()) return;
  auto size_of = [&](int buf) -> int64_t {
    if (buf == L_IN) return in_elems_;
    if (buf == L_OUT) return out_elems_;
    int i = buf - L_TMP0;
    if (i < 0 || i >= (int)tmp_elems_.size()) throw std::runtime_error("bad buffer id");
    return tmp_elems_[i];
  };
  if (rank < 0 || rank >= P_) throw std::runtime_error(name_ + ": executing rank out of range");
  if (dbuf == L_IN) throw std::runtime_error(name_ + ": step writes the input buffer");
  if (doff < 0 || doff + count > size_of(dbuf))
    throw std::runtime_error(name_ + ": destination range out of bounds");
  for (const Src& s : srcs) {
    if (s.peer < 0 || s.peer >= P_) throw std::runtime_error(name_ + ": peer out of range");
    if (s.off < 0 || s.off + count > size_of(s.buf))
      throw std::runtime_error(name_ + ": source range out of bounds");
  }
  Op op;
  op.rank = rank;
  op.dst_buf = dbuf;
  op.dst_off = doff;
  op.count = count;
  op.acc = acc;
  op.flags = flags;
  op.fence = fence_;
  op.srcs = srcs;
  ops_.push_back(std::move(op));
}

int Builder::embed(const Builder& sub, const std::vector<int>& rank_map, int tmp_base) {
  if ((int)rank_map.size() != sub.P_) throw std::runtime_error(name_ + ": rank map does not match the embedded program");
  if (sub.in_elems_ > in_elems_ || sub.out_elems_ > out_elems_)
    throw std::runtime_error(name_ + ": embedded program needs larger buffers");
  if (tmp_base < 0) {
    tmp_base = L_TMP0 + (int)tmp_elems_.size();
    for (int64_t e : sub.tmp_elems_) tmp_elems_.push_back(e);
  }
  auto map_buf = [&](int b) { return b < L_TMP0 ? b : tmp_base + (b - L_TMP0); };
  const int32_t fence0 = fence_;
  int32_t maxf = 0;
  for (const Op& o : sub.ops_) {
    Op q = o;
    q.rank = rank_map[o.rank];
    q.dst_buf = map_buf(o.dst_buf);
    q.fence = fence0 + o.fence;
    maxf = std::max(maxf, o.fence);
    for (Src& s : q.srcs) { s.peer = rank_map[s.peer]; s.buf = map_buf(s.buf); }
    ops_.push_back(std::move(q));
  }
  embed_fence_span_ = std::max(embed_fence_span_, maxf);
  return tmp_base;
}

namespace {

struct Access {
  int64_t off, cnt;
  int32_t level;
  int32_t exec_rank;
  bool write;
  bool arrival = false;   // the owner's "my input is final" point, not a step (see lower(), part 4)
};

inline bool overlap(int64_t a, int64_t an, int64_t b, int64_t bn) {
  return a < b + bn && b < a + an;
}

inline int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

}  // namespace

Program Builder::lower(const LowerOpts& o) const {
  Program p;
  p.name = name_;
  p.P = P_;
  p.in_elems = in_elems_;
  p.out_elems = out_elems_;
  p.in_symmetric = o.in_symmetric;
  p.out_symmetric = o.out_symmetric;

  // ---- 1. which caller buffers do peers read? --------------------------------
  bool rin = false, rout = false;
  std::vector<int64_t> in_lo(P_, INT64_MAX), in_hi(P_, -1);
  for (const Op& op : ops_)
    for (const Src& s : op.srcs)
      if (s.peer != op.rank) {
        if (s.buf == L_IN) {
          rin = true;
          in_lo[s.peer] = std::min(in_lo[s.peer], s.off);
          in_hi[s.peer] = std::max(in_hi[s.peer], s.off + op.count);
        }
        if (s.buf == L_OUT) rout = true;
      }
  p.reads_peer_in = rin;
  p.reads_peer_out = rout;
  const bool stage_in = (rin && !o.in_symmetric) || o.in_place;
  const bool stage_out = rout && !o.out_symmetric;

  // ---- 2. scratch layout -------------------------------------------------------
  const int64_t A = 64;  // elements; keeps every region 16-byte aligned for any dtype
  int64_t cur = 0;
  std::vector<int64_t> tmp_off(tmp_elems_.size());
  for (size_t i = 0; i < tmp_elems_.size(); ++i) {
    tmp_off[i] = cur;
    cur += align_up(tmp_elems_[i], A);
  }
  int64_t ins_off = -1, outs_off = -1;
  if (stage_in) { ins_off = cur; cur += align_up(in_elems_, A); }
  if (stage_out) { outs_off = cur; cur += align_up(out_elems_, A); }
  p.work_elems = cur;

  // ---- 3. physical ops ---------------------------------------------------------
  std::vector<Op>& ops = p.ops;
  ops.reserve(ops_.size() + 2 * P_);
  if (stage_in)
    for (int r = 0; r < P_; ++r) {
      if (o.in_place) { in_lo[r] = 0; in_hi[r] = in_elems_; }
      if (in_hi[r] < 0) continue;
      Op s;
      s.rank = r;
      s.dst_buf = P_WORK;
      s.dst_off = ins_off + in_lo[r];
      s.count = in_hi[r] - in_lo[r];
      s.flags = OPF_STAGE;
      s.fence = ops_.empty() ? 0 : ops_.front().fence;
      s.srcs = {Src{r, P_IN, in_lo[r]}};
      ops.push_back(std::move(s));
    }
  int32_t max_fence = 0;
  for (const Op& l : ops_) {
    Op q = l;
    max_fence = std::max(max_fence, l.fence);
    if (l.dst_buf == L_OUT) {
      if (stage_out) { q.dst_buf = P_WORK; q.dst_off = outs_off + l.dst_off; }
      else q.dst_buf = P_OUT;
    } else {
      q.dst_buf = P_WORK;
      q.dst_off = tmp_off[l.dst_buf - L_TMP0] + l.dst_off;
    }
    for (Src& s : q.srcs) {
      if (s.buf == L_IN) {
        if (stage_in && (s.peer != l.rank || o.in_place)) { s.buf = P_WORK; s.off += ins_off; }
        else s.buf = P_IN;
      } else if (s.buf == L_OUT) {
        if (stage_out) { s.buf = P_WORK; s.off += outs_off; }
        else s.buf = P_OUT;
      } else {
        s.off += tmp_off[s.buf - L_TMP0];
        s.buf = P_WORK;
      }
    }
    ops.push_back(std::move(q));
  }
  if (stage_out)
    for (int r = 0; r < P_; ++r) {
      Op s;
      s.rank = r;
      s.dst_buf = P_OUT;
      s.dst_off = 0;
      s.count = out_elems_;
      s.flags = OPF_STAGE;
      s.fence = max_fence;
      s.srcs = {Src{r, P_WORK, outs_off}};
      ops.push_back(std::move(s));
    }

  // Fence groups must be visited in order.  Generators emit them in order; only
  // embedded sub-programs (independent rank sets, each restarting at the current
  // fence) interleave them, and for those a stable sort by fence keeps every
  // sub-program's own order.
  std::stable_sort(ops.begin(), ops.end(), [](const Op& a, const Op& b) { return a.fence < b.fence; });

  // ---- 4. dependency analysis and round assignment ----------------------------
  // history[(owner rank, phys buf)] -> accesses so far
  std::vector<std::vector<Access>> hist((size_t)P_ * 3);
  auto H = [&](int rank, int buf) -> std::vector<Access>& { return hist[(size_t)rank * 3 + buf]; };
  struct XDep { int32_t waiter, round, peer, need; };
  std::vector<XDep> xdeps;
  // Entry handshake.  A caller input that peers pull directly (in_symmetric, not staged) is produced by
  // whatever the owner's stream ran before this collective, so a reader must not touch it before the
  // owner has entered the collective.  The owner's entry is modelled as a write of the input by the
  // owner in round 0: every peer that reads it lands in round >= 1 with a wait on (owner, 0), and the
  // owner's round 0 (possibly without steps) signals those readers.  The owner's own reads are not
  // delayed.  Staged inputs need none of this: the staging copy is a step of the owner.
  // (In the two-sided original a message cannot leave before the sender's call began:
  //  testing/custom_implementations/work_dir/all_reduce/all_reduce_radix_batch.cpp:353-364.)
  if (rin && !stage_in)
    for (int r = 0; r < P_; ++r)
      if (in_hi[r] >= 0) {
        Access a{in_lo[r], in_hi[r] - in_lo[r], 0, r, true};
        a.arrival = true;
        H(r, P_IN).push_back(a);
      }
  int32_t cur_fence = INT32_MIN, fence_floor = 0, max_level = -1;
  for (Op& op : ops) {
    if (op.fence != cur_fence) {
      if (cur_fence != INT32_MIN) fence_floor = max_level + 1;
      cur_fence = op.fence;
    }
    int32_t lvl = fence_floor;
    std::vector<std::pair<int32_t, int32_t>> deps;  // (exec_rank, level)
    auto scan = [&](int owner, int buf, int64_t off, int64_t cnt, bool i_write) {
      for (const Access& a : H(owner, buf)) {
        if (!overlap(a.off, a.cnt, off, cnt)) continue;
        if (!i_write && !a.write) continue;  // read after read
        if (a.arrival && a.exec_rank == op.rank) continue;  // the owner itself is past its own entry
        lvl = std::max(lvl, a.level + 1);
        if (a.exec_rank != op.rank) deps.emplace_back(a.exec_rank, a.level);
      }
    };
    for (const Src& s : op.srcs) scan(s.peer, s.buf, s.off, op.count, false);
    scan(op.rank, op.dst_buf, op.dst_off, op.count, true);
    op.level = lvl;
    max_level = std::max(max_level, lvl);
    for (auto& d : deps) xdeps.push_back(XDep{op.rank, lvl, d.first, d.second});
    for (const Src& s : op.srcs)
      H(s.peer, s.buf).push_back(Access{s.off, op.count, lvl, op.rank, false});
    H(op.rank, op.dst_buf).push_back(Access{op.dst_off, op.count, lvl, op.rank, true});
  }
  p.nrounds = std::max(1, max_level + 1);

  // ---- 5. per-rank rounds, waits, signals --------------------------------------
  p.rr.assign(P_, std::vector<RankRound>(p.nrounds));
  for (size_t i = 0; i < ops.size(); ++i) p.rr[ops[i].rank][ops[i].level].ops.push_back((int32_t)i);
  // need[waiter][round][peer] = max round of peer required
  std::vector<std::map<int64_t, int32_t>> need(P_);
  for (const XDep& d : xdeps) {
    int64_t key = (int64_t)d.round * P_ + d.peer;
    auto it = need[d.waiter].find(key);
    if (it == need[d.waiter].end()) need[d.waiter][key] = d.need;
    else it->second = std::max(it->second, d.need);
  }
  for (int r = 0; r < P_; ++r) {
    std::vector<int32_t> known(P_, -1);
    for (auto& kv : need[r]) {  // ordered by round, then peer
      int32_t round = (int32_t)(kv.first / P_), peer = (int32_t)(kv.first % P_);
      if (o.global_rounds) continue;
      if (kv.second <= known[peer]) continue;
      known[peer] = kv.second;
      p.rr[r][round].waits.push_back(Wait{peer, kv.second});
    }
  }
  if (o.global_rounds) {
    for (int r = 0; r < P_; ++r)
      for (int t = 1; t < p.nrounds; ++t)
        for (int q = 0; q < P_; ++q)
          if (q != r) p.rr[r][t].waits.push_back(Wait{q, t - 1});
  }
  // exit waits: peers that read this rank's caller buffers directly
  p.exit_waits.assign(P_, {});
  {
    std::vector<std::vector<int32_t>> ex(P_, std::vector<int32_t>(P_, -1));
    for (const Op& op : ops)
      for (const Src& s : op.srcs)
        if (s.peer != op.rank && (s.buf == P_IN || s.buf == P_OUT))
          ex[s.peer][op.rank] = std::max(ex[s.peer][op.rank], op.level);
    for (int a = 0; a < P_; ++a)
      for (int b = 0; b < P_; ++b)
        if (ex[a][b] >= 0) p.exit_waits[a].push_back(Wait{b, ex[a][b]});
  }
  // signals mirror waits
  auto add_signal = [&](int from, int round, int to) {
    auto& v = p.rr[from][round].signals;
    if (std::find(v.begin(), v.end(), to) == v.end()) v.push_back(to);
  };
  for (int r = 0; r < P_; ++r) {
    for (int t = 0; t < p.nrounds; ++t)
      for (const Wait& w : p.rr[r][t].waits) add_signal(w.peer, w.need, r);
    for (const Wait& w : p.exit_waits[r]) add_signal(w.peer, w.need, r);
  }
  // the last round always notifies everybody: it is the "previous call is
  // over" token the next call waits for before it touches scratch again.
  for (int r = 0; r < P_; ++r)
    for (int q = 0; q < P_; ++q)
      if (q != r) add_signal(r, p.nrounds - 1, q);

  // ---- 6. statistics -------------------------------------------------------------
  std::vector<int64_t> per_rank(P_, 0);
  for (const Op& op : ops) {
    p.stats.max_nsrc = std::max<int64_t>(p.stats.max_nsrc, (int64_t)op.srcs.size() + (op.acc ? 1 : 0));
    for (const Src& s : op.srcs) {
      if (s.peer != op.rank) {
        p.stats.remote_msgs++;
        p.stats.remote_elems += op.count;
        per_rank[op.rank] += op.count;
      } else {
        p.stats.local_elems += op.count;
      }
    }
  }
  for (int r = 0; r < P_; ++r) p.stats.max_rank_remote_elems = std::max(p.stats.max_rank_remote_elems, per_rank[r]);
  return p;
}

// =============================== simulator ======================================
namespace {

template <typename T>
inline T apply(int op, T a, T b) {
  switch (op) {
    case OP_SUM: return a + b;
    case OP_MAX: return a > b ? a : b;
    case OP_MIN: return a < b ? a : b;
    case OP_PROD: return a * b;
  }
  return a;
}

template <typename T>
int simulate_t(const Program& p, int rop, void* const* in, void* const* out, uint64_t seed,
               std::string* err) {
  const int P = p.P;
  std::vector<std::vector<T>> work(P);
  for (int r = 0; r < P; ++r) {
    work[r].resize((size_t)p.work_elems);
    // poison scratch so that reads of never-written scratch show up
    if (!work[r].empty()) std::memset(work[r].data(), 0xFF, work[r].size() * sizeof(T));
  }
  auto ptr = [&](int rank, int buf, int64_t off) -> T* {
    switch (buf) {
      case P_IN: return (T*)in[rank] + off;
      case P_OUT: return (T*)out[rank] + off;
      default: return work[rank].data() + off;
    }
  };
  // Inputs that peers pull directly are only final once their owner has entered the collective: until a
  // rank starts its round 0 its input holds poison here, so a schedule that lets a peer read too early
  // produces a wrong result instead of passing by luck.
  bool late_inputs = false;
  for (const Op& op : p.ops)
    for (const Src& s : op.srcs) late_inputs |= (s.peer != op.rank && s.buf == P_IN);
  std::vector<std::vector<T>> held(late_inputs ? P : 0);
  for (int r = 0; r < (int)held.size(); ++r) {
    held[r].assign((T*)in[r], (T*)in[r] + p.in_elems);
    std::memset(in[r], 0xEE, (size_t)p.in_elems * sizeof(T));
  }
  std::vector<int> next(P, 0);  // next round to execute; completed = next-1
  std::mt19937_64 rng(seed);
  std::vector<T> tmp;
  int remaining = P;
  while (remaining > 0) {
    std::vector<int> ready;
    for (int r = 0; r < P; ++r) {
      if (next[r] >= p.nrounds) continue;
      bool ok = true;
      for (const Wait& w : p.rr[r][next[r]].waits)
        if (next[w.peer] - 1 < w.need) { ok = false; break; }
      if (ok) ready.push_back(r);
    }
    if (ready.empty()) {
      for (int q = 0; q < (int)held.size(); ++q)
        if (next[q] == 0) std::memcpy(in[q], held[q].data(), (size_t)p.in_elems * sizeof(T));
      if (err) *err = "deadlock: no rank can start its next round";
      return -1;
    }
    int r = ready[rng() % ready.size()];
    if (late_inputs && next[r] == 0) std::memcpy(in[r], held[r].data(), (size_t)p.in_elems * sizeof(T));
    std::vector<int32_t> order = p.rr[r][next[r]].ops;
    std::shuffle(order.begin(), order.end(), rng);
    for (int32_t oi : order) {
      const Op& op = p.ops[oi];
      tmp.assign((size_t)op.count, T());
      size_t first = 0;
      if (op.acc) {
        std::memcpy(tmp.data(), ptr(op.rank, op.dst_buf, op.dst_off), op.count * sizeof(T));
      } else {
        const Src& s = op.srcs[0];
        std::memcpy(tmp.data(), ptr(s.peer, s.buf, s.off), op.count * sizeof(T));
        first = 1;
      }
      for (size_t si = first; si < op.srcs.size(); ++si) {
        const Src& s = op.srcs[si];
        const T* sp = ptr(s.peer, s.buf, s.off);
        for (int64_t i = 0; i < op.count; ++i) tmp[i] = apply<T>(rop, tmp[i], sp[i]);
      }
      std::memcpy(ptr(op.rank, op.dst_buf, op.dst_off), tmp.data(), op.count * sizeof(T));
    }
    if (++next[r] >= p.nrounds) --remaining;
  }
  return 0;
}

}  // namespace

int simulate(const Program& p, int dtype, int op, void* const* in, void* const* out,
             uint64_t seed, std::string* err) {
  switch (dtype) {
    case DT_F32: return simulate_t<float>(p, op, in, out, seed, err);
    case DT_F64: return simulate_t<double>(p, op, in, out, seed, err);
    case DT_I32: return simulate_t<int32_t>(p, op, in, out, seed, err);
    case DT_I64: return simulate_t<int64_t>(p, op, in, out, seed, err);
    case DT_U8: return simulate_t<uint8_t>(p, op, in, out, seed, err);
  }
  if (err) *err = "simulate: unsupported dtype on the host";
  return -2;
}

// =============================== verifier =======================================
int verify(const Program& p, std::string* err) {
  const int P = p.P, R = p.nrounds;
  int bad = 0;
  std::ostringstream msg;
  // vector clocks: vc[r][t][a] = highest round of a known complete when r starts round t
  std::vector<std::vector<std::vector<int32_t>>> vc(
      P, std::vector<std::vector<int32_t>>(R + 1, std::vector<int32_t>(P, -1)));
  // (waits only point to strictly earlier rounds, so one ascending sweep suffices)
  for (int t = 0; t < R; ++t)
      for (int r = 0; r < P; ++r) {
        auto& v = vc[r][t];
        if (t > 0) {
          v = vc[r][t - 1];
          v[r] = t - 1;
        }
        for (const Wait& w : p.rr[r][t].waits) {
          if (w.need >= t) { ++bad; msg << "wait on a non-earlier round; "; continue; }
          v[w.peer] = std::max(v[w.peer], w.need);
          // everything the peer knew when it started round need+1 ... conservatively
          // what it knew when it started round `need`
          const auto& pv = vc[w.peer][w.need];
          for (int a = 0; a < P; ++a) v[a] = std::max(v[a], pv[a]);
        }
      }
  struct Acc { int64_t off, cnt; int32_t level, exec; bool write; int idx; };
  std::vector<std::vector<Acc>> hist((size_t)P * 3);
  for (size_t i = 0; i < p.ops.size(); ++i) {
    const Op& op = p.ops[i];
    auto check = [&](int owner, int buf, int64_t off, int64_t cnt, bool i_write) {
      for (const Acc& a : hist[(size_t)owner * 3 + buf]) {
        if (!overlap(a.off, a.cnt, off, cnt)) continue;
        if (!i_write && !a.write) continue;
        if (a.level >= op.level) {
          ++bad;
          msg << "ops " << a.idx << " and " << i << " conflict within round " << op.level << "; ";
        } else if (a.exec != op.rank && vc[op.rank][op.level][a.exec] < a.level) {
          ++bad;
          msg << "op " << i << " (rank " << op.rank << ", round " << op.level
              << ") not ordered after op " << a.idx << " (rank " << a.exec << ", round " << a.level << "); ";
        }
      }
    };
    for (const Src& s : op.srcs) check(s.peer, s.buf, s.off, op.count, false);
    check(op.rank, op.dst_buf, op.dst_off, op.count, true);
    for (const Src& s : op.srcs)
      hist[(size_t)s.peer * 3 + s.buf].push_back(Acc{s.off, op.count, op.level, op.rank, false, (int)i});
    hist[(size_t)op.rank * 3 + op.dst_buf].push_back(Acc{op.dst_off, op.count, op.level, op.rank, true, (int)i});
    // peer-visible only through WORK unless the caller buffers are symmetric
    for (const Src& s : op.srcs)
      if (s.peer != op.rank) {
        if (s.buf == P_IN && !p.in_symmetric) { ++bad; msg << "op " << i << " reads a private input; "; }
        // a peer's input is only final once that peer has entered the collective (completed its round 0)
        if (s.buf == P_IN && p.in_symmetric && vc[op.rank][op.level][s.peer] < 0) {
          ++bad;
          msg << "op " << i << " (rank " << op.rank << ", round " << op.level << ") reads the input of rank " << s.peer
              << " before that rank is known to have entered; ";
        }
        if (s.buf == P_OUT && !p.out_symmetric) { ++bad; msg << "op " << i << " reads a private output; "; }
      }
  }
  if (err) *err = msg.str();
  return bad;
}

}  // namespace chb

// =============================== threaded host executor =========================
// One OS thread per rank, real concurrency: a rank publishes the index of the
// last round it completed (release), waiters spin on it (acquire).  This is the
// host-memory counterpart of the GPU interpreter (same waits, same signals) and
// the closest analogue of the reference's execution model, where every rank is a
// process and message matching orders the rounds.
#include <atomic>
#include <chrono>
#include <thread>

namespace chb {
namespace {

template <typename T>
void run_rank(const Program& p, int rank, int rop, void* const* in, void* const* out, std::vector<T>* work,
              std::atomic<int>* done, std::atomic<bool>* failed, const std::vector<T>* late_input, int delay_ms) {
  if (late_input) {
    // this rank enters late, and its input only becomes final when it enters
    std::this_thread::sleep_for(std::chrono::milliseconds(delay_ms));
    std::memcpy(in[rank], late_input->data(), late_input->size() * sizeof(T));
  }
  auto ptr = [&](int r, int buf, int64_t off) -> T* {
    switch (buf) {
      case P_IN: return (T*)in[r] + off;
      case P_OUT: return (T*)out[r] + off;
      default: return work[r].data() + off;
    }
  };
  for (int t = 0; t < p.nrounds; ++t) {
    for (const Wait& w : p.rr[rank][t].waits) {
      auto t0 = std::chrono::steady_clock::now();
      while (done[w.peer].load(std::memory_order_acquire) < w.need) {
        if (failed->load(std::memory_order_relaxed)) return;
        if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(20)) { failed->store(true); return; }
        std::this_thread::yield();
      }
    }
    for (int32_t oi : p.rr[rank][t].ops) {
      const Op& op = p.ops[oi];
      T* dst = ptr(op.rank, op.dst_buf, op.dst_off);
      size_t first = 0;
      if (!op.acc) {
        const Src& s = op.srcs[0];
        const T* sp = ptr(s.peer, s.buf, s.off);
        if (sp != dst) std::memmove(dst, sp, (size_t)op.count * sizeof(T));
        first = 1;
      }
      for (size_t si = first; si < op.srcs.size(); ++si) {
        const Src& s = op.srcs[si];
        const T* sp = ptr(s.peer, s.buf, s.off);
        switch (rop) {
          case OP_SUM: for (int64_t i = 0; i < op.count; ++i) dst[i] = dst[i] + sp[i]; break;
          case OP_MAX: for (int64_t i = 0; i < op.count; ++i) dst[i] = dst[i] > sp[i] ? dst[i] : sp[i]; break;
          case OP_MIN: for (int64_t i = 0; i < op.count; ++i) dst[i] = dst[i] < sp[i] ? dst[i] : sp[i]; break;
          default: for (int64_t i = 0; i < op.count; ++i) dst[i] = dst[i] * sp[i]; break;
        }
      }
    }
    done[rank].store(t, std::memory_order_release);
  }
  // peers that read this rank's caller buffers must be done before it returns
  for (const Wait& w : p.exit_waits[rank])
    while (done[w.peer].load(std::memory_order_acquire) < w.need) {
      if (failed->load(std::memory_order_relaxed)) return;
      std::this_thread::yield();
    }
}

template <typename T>
int run_threads_t(const Program& p, int rop, void* const* in, void* const* out, int iters, double* seconds,
                  int late_rank, int delay_ms) {
  const int P = p.P;
  std::vector<T> held;
  if (late_rank >= 0 && late_rank < P) held.assign((T*)in[late_rank], (T*)in[late_rank] + p.in_elems);
  std::vector<std::vector<T>> work(P);
  for (auto& w : work) w.resize((size_t)std::max<int64_t>(p.work_elems, 1));
  std::atomic<bool> failed{false};
  double total = 0;
  for (int it = 0; it < iters; ++it) {
    std::vector<std::atomic<int>> done(P);
    for (auto& d : done) d.store(-1);
    auto t0 = std::chrono::steady_clock::now();
    std::vector<std::thread> th;
    if (!held.empty()) std::memset(in[late_rank], 0xEE, held.size() * sizeof(T));
    for (int r = 0; r < P; ++r)
      th.emplace_back(run_rank<T>, std::cref(p), r, rop, in, out, work.data(), done.data(), &failed,
                      (!held.empty() && r == late_rank) ? &held : nullptr, delay_ms);
    for (auto& t : th) t.join();
    total += std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (failed.load()) return -1;
  }
  if (seconds) *seconds = total / std::max(1, iters);
  return 0;
}

}  // namespace

// Note on reduction order: a non-accumulating step combines into dst starting
// from its first source, i.e. ((s0 op s1) op s2) ..., like the simulator.
int run_threads(const Program& p, int dtype, int op, void* const* in, void* const* out, int iters, double* seconds,
                int late_rank, int delay_ms) {
  switch (dtype) {
    case DT_F32: return run_threads_t<float>(p, op, in, out, iters, seconds, late_rank, delay_ms);
    case DT_F64: return run_threads_t<double>(p, op, in, out, iters, seconds, late_rank, delay_ms);
    case DT_I32: return run_threads_t<int32_t>(p, op, in, out, iters, seconds, late_rank, delay_ms);
    case DT_I64: return run_threads_t<int64_t>(p, op, in, out, iters, seconds, late_rank, delay_ms);
  }
  return -2;
}

}  // namespace chb

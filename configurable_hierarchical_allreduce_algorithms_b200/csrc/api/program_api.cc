// C ABI for step programs (chb.h, "programs" section).
#include <cstdio>
#include <cstring>
#include <exception>
#include <string>

#include "../sched/ll_plan.h"
#include "../sched/algos.h"
#include "../sched/program.h"
#include "chb.h"
#include "program_handle.h"

#include <stdexcept>
#include <vector>

namespace chb { Builder gen_a2av_tuna(int P, const std::vector<int64_t>& counts, int r, int b); }

namespace {
void set_err(char* err, int errlen, const std::string& s) {
  if (!err || errlen <= 0) return;
  std::snprintf(err, (size_t)errlen, "%s", s.c_str());
}
}  // namespace

extern "C" {

chb_program_t* chb_program_create(const char* coll, const char* algo, int P, int k, int b,
                                  int64_t count, int aux, int in_symmetric, int out_symmetric,
                                  char* err, int errlen) {
  try {
    chb::AlgoSpec s;
    s.coll = coll ? coll : "";
    s.algo = algo ? algo : "";
    s.P = P;
    s.k = k;
    s.b = b;
    s.count = count;
    s.aux = aux;
    chb::Builder B = chb::build_algorithm(s);
    chb::LowerOpts o;
    o.in_symmetric = (in_symmetric & 1) != 0;
    o.in_place = (in_symmetric & 2) != 0;  // bit 1: input aliases output
    o.out_symmetric = out_symmetric != 0;
    auto* p = new chb_program;
    p->prog = B.lower(o);
    return p;
  } catch (const std::exception& e) {
    set_err(err, errlen, e.what());
    return nullptr;
  }
}

chb_program_t* chb_program_create_alltoallv(int P, int r, int b, const int64_t* counts, char* err, int errlen) {
  try {
    if (!counts || P < 1) throw std::runtime_error("alltoallv needs a P x P count matrix");
    std::vector<int64_t> c(counts, counts + (size_t)P * P);
    chb::Builder B = chb::gen_a2av_tuna(P, c, r, b);
    auto* p = new chb_program;
    p->prog = B.lower(chb::LowerOpts{});
    return p;
  } catch (const std::exception& e) {
    set_err(err, errlen, e.what());
    return nullptr;
  }
}

void chb_program_destroy(chb_program_t* p) { delete p; }

int chb_program_info(const chb_program_t* p, int64_t* info, int n) {
  if (!p || !info) return CHB_ERR_ARG;
  int64_t v[CHB_INFO_COUNT_] = {0};
  const chb::Program& g = p->prog;
  int64_t nsrcs = 0, nwaits = 0, nsig = 0, nexit = 0;
  for (const auto& op : g.ops) nsrcs += (int64_t)op.srcs.size();
  for (const auto& rr : g.rr)
    for (const auto& r : rr) { nwaits += (int64_t)r.waits.size(); nsig += (int64_t)r.signals.size(); }
  for (const auto& e : g.exit_waits) nexit += (int64_t)e.size();
  v[CHB_INFO_P] = g.P;
  v[CHB_INFO_NROUNDS] = g.nrounds;
  v[CHB_INFO_IN_ELEMS] = g.in_elems;
  v[CHB_INFO_OUT_ELEMS] = g.out_elems;
  v[CHB_INFO_WORK_ELEMS] = g.work_elems;
  v[CHB_INFO_NOPS] = (int64_t)g.ops.size();
  v[CHB_INFO_REMOTE_MSGS] = g.stats.remote_msgs;
  v[CHB_INFO_REMOTE_ELEMS] = g.stats.remote_elems;
  v[CHB_INFO_MAX_RANK_REMOTE_ELEMS] = g.stats.max_rank_remote_elems;
  v[CHB_INFO_LOCAL_ELEMS] = g.stats.local_elems;
  v[CHB_INFO_MAX_NSRC] = g.stats.max_nsrc;
  v[CHB_INFO_READS_PEER_IN] = g.reads_peer_in;
  v[CHB_INFO_READS_PEER_OUT] = g.reads_peer_out;
  v[CHB_INFO_NSRCS] = nsrcs;
  v[CHB_INFO_NWAITS] = nwaits;
  v[CHB_INFO_NEXIT_WAITS] = nexit;
  v[CHB_INFO_NSIGNALS] = nsig;
  for (int i = 0; i < n && i < CHB_INFO_COUNT_; ++i) info[i] = v[i];
  return CHB_SUCCESS;
}

const char* chb_program_name(const chb_program_t* p) { return p ? p->prog.name.c_str() : ""; }

int chb_program_verify(const chb_program_t* p, char* err, int errlen) {
  if (!p) return -1;
  std::string e;
  int bad = chb::verify(p->prog, &e);
  if (bad) set_err(err, errlen, e);
  return bad;
}

int chb_program_simulate(const chb_program_t* p, int dtype, int op, void* const* in,
                         void* const* out, uint64_t seed, char* err, int errlen) {
  if (!p) return CHB_ERR_ARG;
  std::string e;
  int rc = chb::simulate(p->prog, dtype, op, in, out, seed, &e);
  if (rc) { set_err(err, errlen, e); return rc == -1 ? CHB_ERR_TIMEOUT : CHB_ERR_ARG; }
  return CHB_SUCCESS;
}

long long chb_program_ll_lines(const chb_program_t* p, int esz) {
  if (!p || esz < 1) return -1;
  return chb::ll_inbox_lines(p->prog, esz);
}

int chb_program_ll_info(const chb_program_t* p, int esz, long long* info, int n) {
  if (!p || !info || esz < 1) return CHB_ERR_ARG;
  chb::LPHeader h{};
  std::vector<char> blob = chb::make_ll_blob(p->prog, esz, &h);
  const chb::LPLevel* lv = reinterpret_cast<const chb::LPLevel*>(blob.data() + h.off_levels);
  long long barriers = 0;
  for (long long i = 0; i < (long long)h.P * h.nlevels; ++i) barriers += lv[i].barrier_before;
  long long forwarded = 0;
  const chb::LPStep* st = reinterpret_cast<const chb::LPStep*>(blob.data() + h.off_steps);
  for (int i = 0; i < h.nsteps; ++i) forwarded += st[i].nfwd;
  const long long v[7] = {h.nlevels, h.nsends, forwarded, barriers, h.inbox_lines, h.max_level_lines, h.rank_table_bytes};
  for (int i = 0; i < n && i < 7; ++i) info[i] = v[i];
  return CHB_SUCCESS;
}

int chb_program_simulate_ll(const chb_program_t* p, int dtype, int op, void* const* in, void* const* out,
                            uint64_t seed, int nthreads, int fault, int launches, char* err, int errlen) {
  if (!p || !in || !out || fault < 0 || fault > 2) return CHB_ERR_ARG;
  std::string e;
  int rc = chb::simulate_ll(p->prog, dtype, op, in, out, seed, nthreads, fault, launches, &e);
  if (rc) { set_err(err, errlen, e); return rc == -1 ? CHB_ERR_TIMEOUT : CHB_ERR_ARG; }
  return CHB_SUCCESS;
}

int chb_program_run_threads(const chb_program_t* p, int dtype, int op, void* const* in, void* const* out,
                            int iters, double* seconds) {
  if (!p || !in || !out) return CHB_ERR_ARG;
  int rc = chb::run_threads(p->prog, dtype, op, in, out, iters, seconds);
  return rc == 0 ? CHB_SUCCESS : (rc == -1 ? CHB_ERR_TIMEOUT : CHB_ERR_ARG);
}

int chb_program_run_threads_late(const chb_program_t* p, int dtype, int op, void* const* in, void* const* out,
                                 int late_rank, int delay_ms) {
  if (!p || !in || !out || late_rank < 0 || late_rank >= p->prog.P) return CHB_ERR_ARG;
  int rc = chb::run_threads(p->prog, dtype, op, in, out, 1, nullptr, late_rank, delay_ms);
  return rc == 0 ? CHB_SUCCESS : (rc == -1 ? CHB_ERR_TIMEOUT : CHB_ERR_ARG);
}

int chb_program_export(const chb_program_t* p, int64_t* ops, int64_t* srcs, int64_t* waits,
                       int64_t* exit_waits, int64_t* signals) {
  if (!p) return CHB_ERR_ARG;
  const chb::Program& g = p->prog;
  int64_t sb = 0;
  for (size_t i = 0; i < g.ops.size(); ++i) {
    const chb::Op& o = g.ops[i];
    if (ops) {
      int64_t* r = ops + i * 8;
      r[0] = o.rank; r[1] = o.level; r[2] = o.dst_buf; r[3] = o.dst_off; r[4] = o.count;
      r[5] = o.acc ? 1 : 0; r[6] = sb; r[7] = (int64_t)o.srcs.size();
    }
    for (const chb::Src& s : o.srcs) {
      if (srcs) { srcs[sb * 3] = s.peer; srcs[sb * 3 + 1] = s.buf; srcs[sb * 3 + 2] = s.off; }
      ++sb;
    }
  }
  int64_t w = 0, sg = 0, ew = 0;
  for (int r = 0; r < g.P; ++r) {
    for (int t = 0; t < g.nrounds; ++t) {
      for (const chb::Wait& x : g.rr[r][t].waits) {
        if (waits) { waits[w * 4] = r; waits[w * 4 + 1] = t; waits[w * 4 + 2] = x.peer; waits[w * 4 + 3] = x.need; }
        ++w;
      }
      for (int32_t q : g.rr[r][t].signals) {
        if (signals) { signals[sg * 3] = r; signals[sg * 3 + 1] = t; signals[sg * 3 + 2] = q; }
        ++sg;
      }
    }
    for (const chb::Wait& x : g.exit_waits[r]) {
      if (exit_waits) { exit_waits[ew * 3] = r; exit_waits[ew * 3 + 1] = x.peer; exit_waits[ew * 3 + 2] = x.need; }
      ++ew;
    }
  }
  return CHB_SUCCESS;
}

int chb_list_algorithms(const char* coll, char* out, int outlen) {
  std::string s;
  for (const std::string& a : chb::list_algorithms(coll ? coll : "")) {
    if (!s.empty()) s += ",";
    s += a;
  }
  if (out && outlen > 0) std::snprintf(out, (size_t)outlen, "%s", s.c_str());
  return (int)s.size();
}

int chb_dtype_size(int dtype) { return chb::dtype_size(dtype); }
const char* chb_version(void) { return "chb-b200 0.1"; }

}  // extern "C"

// Step-program IR for configurable collectives.
//
// A collective algorithm is compiled once, for a given (collective, algorithm,
// P, k, b, count), into a *step program*: for every rank a list of pull steps
//
//     dst[off : off+count]  =  (dst op)  src_0 op src_1 op ... op src_{m-1}
//
// where dst is always a buffer of the executing rank and every src is a
// buffer region of the executing rank or of a peer.  A message of a two-sided
// algorithm (sender region -> receiver region, optionally followed by a local
// reduction) is one such step executed by the receiver; the k-1 neighbour
// exchanges of one radix-k round collapse into one multi-source step.
//
// Generators emit steps in a serially correct order against *logical*
// buffers (IN, OUT, numbered temporaries).  lower() then
//   1. places temporaries in the per-rank symmetric scratch (WORK),
//   2. stages IN / OUT through WORK when peers read them and the caller's
//      buffers are not peer-visible,
//   3. derives dependencies from region overlap (RAW, WAW, WAR), assigns every
//      step a round (longest dependency path) and
//   4. turns cross-rank dependencies into per-round (peer, round) waits and
//      matching signals.
// The same lowered program drives the CPU simulator, the gloo executor and the
// persistent GPU interpreter kernel.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "types.h"

namespace chb {

enum LogicalBuf : int32_t { L_IN = 0, L_OUT = 1, L_TMP0 = 2 };
enum PhysBuf : int32_t { P_IN = 0, P_OUT = 1, P_WORK = 2 };

enum OpFlags : uint32_t {
  OPF_NONE = 0,
  OPF_STAGE = 1,      // staging copy inserted by lower()
  OPF_FINAL = 2,      // produces final values of the reduction (scale point)
};

struct Src {
  int32_t peer;
  int32_t buf;
  int64_t off;
};

struct Op {
  int32_t rank = 0;       // executing rank (owner of dst)
  int32_t dst_buf = 0;
  int64_t dst_off = 0;
  int64_t count = 0;
  bool acc = false;       // dst participates as the first operand
  uint32_t flags = 0;
  int32_t fence = 0;      // generator-imposed minimum round ordering group
  int32_t level = -1;     // round, filled by lower()
  std::vector<Src> srcs;
};

struct Wait {
  int32_t peer;
  int32_t need;           // peer must have completed this round
};

struct RankRound {
  std::vector<int32_t> ops;       // indices into Program::ops
  std::vector<Wait> waits;        // to satisfy before the round starts
  std::vector<int32_t> signals;   // peers to notify when the round is complete
};

struct ProgramStats {
  int64_t remote_msgs = 0;        // number of (step, remote source) pairs
  int64_t remote_elems = 0;       // elements pulled from peers, all ranks
  int64_t max_rank_remote_elems = 0;
  int64_t local_elems = 0;        // elements read locally, all ranks
  int64_t max_nsrc = 0;
};

struct Program {
  std::string name;
  int P = 0;
  int64_t in_elems = 0, out_elems = 0, work_elems = 0;
  int nrounds = 0;
  bool in_symmetric = false, out_symmetric = false;
  bool reads_peer_in = false, reads_peer_out = false;
  std::vector<Op> ops;                          // physical buffers, level set
  std::vector<std::vector<RankRound>> rr;       // [rank][round]
  std::vector<std::vector<Wait>> exit_waits;    // [rank]
  ProgramStats stats;
};

struct LowerOpts {
  bool in_symmetric = false;    // peers may read the caller's input buffer
  bool out_symmetric = false;   // peers may read the caller's output buffer
  bool global_rounds = false;   // every wait becomes "all ranks" (debug aid)
  bool in_place = false;        // input and output alias: every read of IN goes through a scratch copy
};

class Builder {
 public:
  Builder(int P, int64_t in_elems, int64_t out_elems, std::string name);
  int P() const { return P_; }
  // New per-rank temporary of `elems` elements; returns its logical id.
  int tmp(int64_t elems);
  // dst = src (single source).
  void copy(int rank, int dbuf, int64_t doff, int speer, int sbuf, int64_t soff,
            int64_t count, uint32_t flags = 0);
  // dst = [dst op] src_0 op ... ; sources are combined left to right.
  void reduce(int rank, int dbuf, int64_t doff, const std::vector<Src>& srcs,
              int64_t count, bool acc, uint32_t flags = 0);
  // Everything emitted after fence() is scheduled in a later round than
  // everything emitted before it (models a global MPI_Waitall boundary).
  void fence() { ++fence_; }
  // Append all steps of `sub` (a program over rank_map.size() ranks with the same
  // input / output lengths) with sub-rank i executed by rank rank_map[i]; used to
  // run one flat algorithm independently inside every group or along every lane.
  // tmp_base < 0 allocates fresh temporaries and returns their first id, so that
  // further embeddings of the same sub-program can share them.
  int embed(const Builder& sub, const std::vector<int>& rank_map, int tmp_base = -1);
  Program lower(const LowerOpts& o) const;

 private:
  int P_;
  int64_t in_elems_, out_elems_;
  std::string name_;
  std::vector<int64_t> tmp_elems_;
  std::vector<Op> ops_;
  int32_t fence_ = 0;
  int32_t embed_fence_span_ = 0;   // largest fence offset used by embedded programs
};

// ---- reduction / element types shared by simulator, C API and kernels ----

// Run a lowered program on host memory for all P ranks in one process.
// in[r] / out[r] point at rank r's buffers.  Ranks advance one round at a
// time in a pseudo-random order (seed) that honours only the program's own
// waits, so a missing dependency shows up as a wrong result.
// Returns 0, or a negative code (-1 deadlock, -2 bad argument).
int simulate(const Program& p, int dtype, int op, void* const* in, void* const* out,
             uint64_t seed, std::string* err);

// Execute a lowered program with one host thread per rank (real concurrency,
// release / acquire on per-rank round counters); `iters` repetitions, mean wall
// seconds per repetition in *seconds.  Returns 0, -1 on a wait that expired, -2
// for an unsupported dtype.  A step whose first source aliases its destination
// is handled (in-place copies are skipped).
// late_rank >= 0: that rank's thread starts delay_ms late and its input holds poison until it does (an
// input that peers pull directly is only final once its owner has entered the collective).
int run_threads(const Program& p, int dtype, int op, void* const* in, void* const* out, int iters,
                double* seconds, int late_rank = -1, int delay_ms = 0);

// Static check: within one round no region is written by one step and read
// or written by another (on any rank); and every cross-round cross-rank
// hazard is covered by a wait chain.  Returns number of violations.
int verify(const Program& p, std::string* err);

}  // namespace chb

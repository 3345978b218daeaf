// The flagged-line (push) form of a lowered step program, as flat tables: what kernels/llprog.cu executes on the
// GPU and what simulate_ll() below executes on host memory.
//
// Every remote source of a step becomes a message that its OWNER pushes, as 16-byte lines {data, flag, data, flag},
// into a slot of the reader's inbox reserved for that (step, source) pair.  Level t of a rank (t = round of the
// lowered program): 1. push every region of mine that a peer's step of level t reads; 2. execute my steps of
// level t (local sources loaded, remote ones awaited in the inbox, combined left to right, stored once).  A send
// of level t + 1 whose source lies inside the destination of one of my steps of level t is forwarded line by line
// by the threads of that step instead; a rank-local barrier separates two levels only where the later one reads
// or overwrites local memory that the earlier ones wrote or read.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "program.h"

namespace chb {

// all_copy: every step of the level stores one remote source unchanged (an allgather round): the executor then
// takes several lines of a thread at once
struct LPLevel { int step_begin, step_end, send_begin, send_end; long long step_lines, send_lines; int barrier_before, all_copy; };
struct LPStep { long long dst_off, count, line_prefix; int dst_buf, nsrc, src_begin; unsigned flags; int fwd_begin, nfwd; };
// lines [line_begin, line_begin + nlines) of a step's result go to inbox_line.. of dst_rank as they are produced
struct LPFwd { long long line_begin, nlines, inbox_line; int dst_rank, pad; };
struct LPSrc { long long off, inbox_line; int peer, buf; };          // inbox_line < 0: local source
struct LPSend { long long src_off, count, inbox_line, line_prefix; int dst_rank, src_buf; };
// the entries of one rank are contiguous in every table: [first, first + n)
struct LPRank { int step0, nstep, src0, nsrc, send0, nsend, fwd0, nfwd; };
struct LPHeader {
  int P, nlevels, nsteps, nsrcs, nsends, esz;
  long long off_ranks, off_levels, off_steps, off_srcs, off_sends, off_fwds;
  long long max_level_lines;     // busiest (rank, level): lines pushed + lines executed
  long long inbox_lines;         // lines needed in the fullest inbox
  long long rank_table_bytes;    // bytes of the largest rank's own entries (levels, steps, sources, sends, forwards)
};
// LPRank[P] follows the header at this fixed offset, so that a rank can fetch its ranges and the header together
constexpr long long kLPRanksOffset = 128;
static_assert(sizeof(LPHeader) <= kLPRanksOffset, "the rank table starts right after the header");

inline long long ll_lines_of(long long count, int esz) { return (count * esz + 7) / 8; }

// Flatten a lowered program into the tables above for elements of esz bytes.  Layout of the result: LPHeader, LPRank[P]
// at kLPRanksOffset, then at the header's offsets LPLevel[P * nlevels] (rank-major), LPStep[], LPSrc[], LPSend[], LPFwd[].
std::vector<char> make_ll_blob(const Program& p, int esz, LPHeader* hout);

// Lines the fullest inbox needs (without building the tables).
long long ll_inbox_lines(const Program& p, int esz);

// Run the push form on host memory the way the kernel does, line by line: every rank is `nthreads` virtual
// threads, thread v owning lines v, v + nthreads, ... of every level's push and step phases; a thread stops at a
// line whose remote source has not arrived and at a barrier that its rank has not completed, and the scheduler
// picks the next thread to advance at random (seed).  Nothing but the tables orders the threads, so a message
// that nobody sends shows up as a deadlock (-1, err says which rank waits for which peer) and a dropped barrier
// or a wrong forward as a wrong result in some interleavings.  Returns 0, -1, or -2 for a bad argument.
// fault (for the tests of this simulator itself: does it notice a broken plan?): LL_FAULT_NO_BARRIERS ignores the
// plan's barriers, LL_FAULT_DROP_A_FORWARD leaves out the last forward of every step.
enum { LL_FAULT_NONE = 0, LL_FAULT_NO_BARRIERS = 1, LL_FAULT_DROP_A_FORWARD = 2 };
// launches > 1 runs the program that many times back to back on the same buffers: every rank starts its next
// launch as soon as its own previous one has returned (stream order), nothing else holds a rank back, and the
// inbox halves alternate by launch parity as on the GPU.  A sender that gets two launches ahead of a reader then
// overwrites a line that was never read, which ends the run with -1: that is the case the executor excludes by
// accepting only collectives in which every rank's result depends on every rank's input.
int simulate_ll(const Program& p, int dtype, int op, void* const* in, void* const* out, uint64_t seed,
                int nthreads, int fault, int launches, std::string* err);

}  // namespace chb

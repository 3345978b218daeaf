// Persistent step-program interpreter: one launch executes a whole collective.
//
// A compiled program (csrc/sched/program.h) is flattened into a device blob;
// every rank walks its rounds: wait for the (peer, round) pairs the round
// depends on, run the round's pull steps with all CTAs of the rank, meet at
// the rank-local barrier, then release the peers that wait for this round.
// A step reads up to kMaxSrc regions (local or peer, 16-byte vectors through
// the owner's L2), combines them in fp32 (or the native integer / double
// type) and stores the result once; this is where the reference's
// MPI_Isend/Irecv/Waitall + MPI_Reduce_local loops end up
// (testing/custom_implementations/work_dir/all_reduce/all_reduce_radix_batch.cpp:339-368,
//  501-539, 552-569, 591-646).
//
// With World::nlocal == P (all ranks emulated on one GPU) blockIdx.y selects
// the rank and the launch is cooperative, so that ranks which wait for each
// other are guaranteed to be co-resident.
#include <cstdio>
#include <cstring>
#include <vector>

#include "../api/chb.h"
#include "../api/program_handle.h"
#include "../symm/comm.h"
#include "common.cuh"

namespace chb {

constexpr int kInterpThreads = 512;
constexpr int kMaxSrc = 40;              // sources per step (incl. the accumulate operand)
constexpr long long kSmallStepElems = 16 << 10;  // steps below this many elements are run whole, by one CTA

struct DevStep { long long dst_off; long long count; int dst_buf; int nsrc; int src_begin; unsigned flags; };
struct DevSrc { long long off; int peer; int buf; };
struct DevWait { int peer; int need; };
// order[ord_begin ..): the round's steps, the nbig large ones first (big_tot / big_max: their total and largest count)
struct DevRound { int step_begin, step_end, wait_begin, wait_end, sig_begin, sig_end, ord_begin, nbig; long long big_tot, big_max; };
struct DevHeader {
  int P, nrounds, nsteps, nsrcs, nwaits, nsigs;
  long long off_rounds, off_steps, off_srcs, off_waits, off_sigs, off_exit, off_order;
  long long limit[3];   // elements of the caller input, caller output and scratch (for range checks)
};
// The entries of one rank are contiguous in every table: [first, first + n).  DevRank[P] follows the header at a
// fixed offset, so that a rank fetches its ranges together with the header.
struct DevRank { int step0, nstep, src0, nsrc, wait0, nwait, sig0, nsig, ord0, nord, exit0, nexit; };
constexpr long long kDevRanksOffset = 128;
static_assert(sizeof(DevHeader) <= kDevRanksOffset, "the rank table starts right after the header");
constexpr long long kInterpSmemTables = 40 << 10;   // bytes of table entries a CTA keeps in shared memory

struct IoTable {
  const char* in[kMaxRanks];
  char* out[kMaxRanks];
};

// Every range a program touches lies inside the buffer it names: checked once per program before
// its schedule is uploaded, so that a generator bug cannot turn into a stray peer access.
static bool ranges_ok(const Program& p, std::string* why) {
  const int64_t lim[3] = {p.in_elems, p.out_elems, p.work_elems};
  for (size_t i = 0; i < p.ops.size(); ++i) {
    const Op& o = p.ops[i];
    bool ok = o.rank >= 0 && o.rank < p.P && o.dst_buf >= 0 && o.dst_buf <= 2 && o.count >= 0 && o.dst_off >= 0 &&
              o.dst_off + o.count <= lim[o.dst_buf];
    for (const Src& x : o.srcs)
      ok = ok && x.peer >= 0 && x.peer < p.P && x.buf >= 0 && x.buf <= 2 && x.off >= 0 && x.off + o.count <= lim[x.buf];
    if (!ok) {
      *why = "step " + std::to_string(i) + " of " + p.name + " addresses memory outside its buffer";
      return false;
    }
  }
  return true;
}

static std::vector<char> make_blob(const Program& p, long long* rank_table_bytes) {
  DevHeader h{};
  h.P = p.P;
  h.nrounds = p.nrounds;
  h.limit[0] = p.in_elems;
  h.limit[1] = p.out_elems;
  h.limit[2] = p.work_elems;
  std::vector<DevRound> rounds((size_t)p.P * p.nrounds);
  std::vector<DevStep> steps;
  std::vector<DevSrc> srcs;
  std::vector<DevWait> waits;
  std::vector<int> sigs;
  std::vector<int> order;
  std::vector<int> exits((size_t)p.P * 2);
  for (int r = 0; r < p.P; ++r)
    for (int t = 0; t < p.nrounds; ++t) {
      const RankRound& rr = p.rr[r][t];
      DevRound& d = rounds[(size_t)r * p.nrounds + t];
      d.step_begin = (int)steps.size();
      for (int oi : rr.ops) {
        const Op& o = p.ops[oi];
        DevStep s{};
        s.dst_off = o.dst_off;
        s.count = o.count;
        s.dst_buf = o.dst_buf;
        s.flags = o.flags | (o.acc ? 0x100u : 0u);
        s.src_begin = (int)srcs.size();
        s.nsrc = (int)o.srcs.size();
        for (const Src& x : o.srcs) srcs.push_back(DevSrc{x.off, x.peer, x.buf});
        steps.push_back(s);
      }
      d.step_end = (int)steps.size();
      // what the tile scheduler needs, worked out here once instead of by one thread per round and launch
      d.ord_begin = (int)order.size();
      for (int pass = 0; pass < 2; ++pass)
        for (int si = d.step_begin; si < d.step_end; ++si) {
          const bool big = steps[(size_t)si].count >= kSmallStepElems;
          if (big != (pass == 0)) continue;
          order.push_back(si);
          if (big) {
            ++d.nbig;
            d.big_tot += steps[(size_t)si].count;
            d.big_max = std::max<long long>(d.big_max, steps[(size_t)si].count);
          }
        }
      d.wait_begin = (int)waits.size();
      for (const Wait& w : rr.waits) waits.push_back(DevWait{w.peer, w.need});
      d.wait_end = (int)waits.size();
      d.sig_begin = (int)sigs.size();
      for (int q : rr.signals) sigs.push_back(q);
      d.sig_end = (int)sigs.size();
    }
  for (int r = 0; r < p.P; ++r) {
    exits[2 * r] = (int)waits.size();
    for (const Wait& w : p.exit_waits[r]) waits.push_back(DevWait{w.peer, w.need});
    exits[2 * r + 1] = (int)waits.size();
  }
  h.nsteps = (int)steps.size();
  h.nsrcs = (int)srcs.size();
  h.nwaits = (int)waits.size();
  h.nsigs = (int)sigs.size();
  std::vector<DevRank> ranks((size_t)p.P);
  long long worst = 0;
  for (int r = 0; r < p.P && p.nrounds > 0; ++r) {
    DevRank& R = ranks[(size_t)r];
    const DevRound& first = rounds[(size_t)r * p.nrounds];
    const DevRound& last = rounds[(size_t)r * p.nrounds + p.nrounds - 1];
    R.step0 = first.step_begin;  R.nstep = last.step_end - first.step_begin;
    R.wait0 = first.wait_begin;  R.nwait = last.wait_end - first.wait_begin;
    R.sig0 = first.sig_begin;    R.nsig = last.sig_end - first.sig_begin;
    R.ord0 = first.ord_begin;    R.nord = R.nstep;
    R.src0 = R.nstep ? steps[(size_t)R.step0].src_begin : 0;
    for (int i = 0; i < R.nstep; ++i) R.nsrc += steps[(size_t)(R.step0 + i)].nsrc;
    R.exit0 = exits[2 * (size_t)r];
    R.nexit = exits[2 * (size_t)r + 1] - exits[2 * (size_t)r];
    const long long bytes = (long long)p.nrounds * sizeof(DevRound) + (long long)R.nstep * sizeof(DevStep) +
                            (long long)R.nsrc * sizeof(DevSrc) + (long long)(R.nwait + R.nexit) * sizeof(DevWait) +
                            (long long)(R.nsig + R.nord) * sizeof(int);
    worst = std::max(worst, bytes);
  }
  if (rank_table_bytes) *rank_table_bytes = worst;
  auto al = [](size_t x) { return (x + 15) / 16 * 16; };
  size_t off = (size_t)kDevRanksOffset;
  off = al(off + ranks.size() * sizeof(DevRank));
  h.off_rounds = (long long)off; off = al(off + rounds.size() * sizeof(DevRound));
  h.off_steps = (long long)off;  off = al(off + steps.size() * sizeof(DevStep));
  h.off_srcs = (long long)off;   off = al(off + srcs.size() * sizeof(DevSrc));
  h.off_waits = (long long)off;  off = al(off + waits.size() * sizeof(DevWait));
  h.off_sigs = (long long)off;   off = al(off + sigs.size() * sizeof(int));
  h.off_exit = (long long)off;   off = al(off + exits.size() * sizeof(int));
  h.off_order = (long long)off;  off = al(off + order.size() * sizeof(int));
  std::vector<char> blob(off, 0);
  std::memcpy(blob.data(), &h, sizeof(h));
  auto put = [&](long long o, const void* src, size_t n) { if (n) std::memcpy(blob.data() + o, src, n); };
  put(kDevRanksOffset, ranks.data(), ranks.size() * sizeof(DevRank));
  put(h.off_rounds, rounds.data(), rounds.size() * sizeof(DevRound));
  put(h.off_steps, steps.data(), steps.size() * sizeof(DevStep));
  put(h.off_srcs, srcs.data(), srcs.size() * sizeof(DevSrc));
  put(h.off_waits, waits.data(), waits.size() * sizeof(DevWait));
  put(h.off_sigs, sigs.data(), sigs.size() * sizeof(int));
  put(h.off_exit, exits.data(), exits.size() * sizeof(int));
  put(h.off_order, order.data(), order.size() * sizeof(int));
  return blob;
}

// ------------------------------------------------------------------ one step (or one tile of it)
// Elements [e0, e0 + cnt) of step `st`, strided over `nparts` CTAs of which this one is `part`.
// Sources are combined left to right (the order in which the reference receives and reduces), but
// their loads are issued kSrcGroup sources at a time and two vectors deep, so that every thread keeps
// 128 bytes of NVLink round trips in flight whether a step has one remote source or P-1 of them.
constexpr int kSrcGroup = 2;

// 256-bit reduce loop over vectors [j0, nw) strided by TT: G sources x UW vectors in flight per thread.
// (not inlined: each variant gets a register allocation of its own instead of inflating the interpreter's)
template <typename T, int G, int UW>
__device__ __noinline__ void reduce_loop32(const char* const* s_ptr, char* dst, int nsrc, long long j0, long long nw,
                                              long long TT, int op, bool do_scale, float scale) {
  using Acc = typename Elem<T>::Acc;
  constexpr int VE = Elem<T>::kPerVec;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  for (; j0 < nw; j0 += TT * UW) {
    Acc a[UW][2][VE];
    for (int s = 0; s < nsrc; s += G) {
      uint4 x[G][UW][2];
#pragma unroll
      for (int gi = 0; gi < G; ++gi) {
        if (s + gi < nsrc) {
          const char* p0 = s_ptr[s + gi];
#pragma unroll
          for (int u = 0; u < UW; ++u) {
            const long long j = j0 + (long long)u * TT;
            if (j < nw) ld32_cg(p0 + j * 32, x[gi][u][0], x[gi][u][1]);
            else x[gi][u][0] = x[gi][u][1] = zero;
          }
        }
      }
#pragma unroll
      for (int gi = 0; gi < G; ++gi) {
        if (s + gi < nsrc) {
          if (gi == 0 && s == 0) {
#pragma unroll
            for (int u = 0; u < UW; ++u) { vec_to_acc<T>(x[0][u][0], a[u][0]); vec_to_acc<T>(x[0][u][1], a[u][1]); }
          } else {
#pragma unroll
            for (int u = 0; u < UW; ++u) { vec_combine<T>(op, x[gi][u][0], a[u][0]); vec_combine<T>(op, x[gi][u][1], a[u][1]); }
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < UW; ++u) {
      const long long j = j0 + (long long)u * TT;
      if (j < nw) {
        if (do_scale) { acc_scale<T>(a[u][0], scale); acc_scale<T>(a[u][1], scale); }
        st32(dst + j * 32, acc_to_vec<T>(a[u][0]), acc_to_vec<T>(a[u][1]));
      }
    }
  }
}

template <typename T>
__device__ __forceinline__ void run_step(const DevStep& st, const DevSrc* __restrict__ srcs, const World& w,
                                         const IoTable& io, int rank, long long e0, long long cnt,
                                         unsigned part, unsigned nparts,
                                         int op, float scale, const char** s_ptr, int* s_meta, const long long* limit) {
  using Acc = typename Elem<T>::Acc;
  constexpr int VE = Elem<T>::kPerVec;
  constexpr int G = kSrcGroup;
  const int tid = threadIdx.x;
  const bool acc = (st.flags & 0x100u) != 0;
  const int nsrc = st.nsrc + (acc ? 1 : 0);
  __syncthreads();  // previous step's readers of s_ptr are done
  if (tid < nsrc || tid == kMaxSrc) {
    if (tid == kMaxSrc) {
      char* base = st.dst_buf == 0 ? const_cast<char*>(io.in[rank]) : (st.dst_buf == 1 ? io.out[rank] : w.work[rank]);
      s_ptr[kMaxSrc] = base + (st.dst_off + e0) * (long long)sizeof(T);
    } else if (acc && tid == 0) {
      char* base = st.dst_buf == 1 ? io.out[rank] : w.work[rank];
      s_ptr[0] = base + (st.dst_off + e0) * (long long)sizeof(T);
    } else {
      const DevSrc s = srcs[st.src_begin + tid - (acc ? 1 : 0)];
      const char* base = s.buf == 0 ? io.in[s.peer] : (s.buf == 1 ? io.out[s.peer] : w.work[s.peer]);
      s_ptr[tid] = base + (s.off + e0) * (long long)sizeof(T);
    }
  }
#ifdef CHB_CHECK_BOUNDS
  // checked build: the same range test as on the host, on the values the kernel actually uses
  if (tid == 0) {
    bool ok = e0 >= 0 && cnt >= 0 && e0 + cnt <= st.count && st.dst_off >= 0 && st.dst_off + st.count <= limit[st.dst_buf];
    for (int j = 0; j < st.nsrc; ++j) {
      const DevSrc s = srcs[st.src_begin + j];
      ok = ok && s.off >= 0 && s.off + st.count <= limit[s.buf] && s.peer >= 0 && s.peer < w.P;
    }
    s_meta[0] = ok ? 0 : -1;
    if (!ok) record_timeout(w.ctrl[rank], ST_OUT_OF_RANGE, rank, -1, -1, (unsigned long long)st.dst_off, (unsigned long long)st.count);
  }
  __syncthreads();
  if (s_meta[0] < 0) return;
#endif
  __syncthreads();
  // widest vector every pointer allows (every thread works it out from the shared table: no second barrier)
  unsigned long long m = (unsigned long long)s_ptr[kMaxSrc];
  for (int i = 0; i < nsrc; ++i) m |= (unsigned long long)s_ptr[i];
  const int align_level = (m & 31ull) == 0ull ? 2 : ((m & 15ull) == 0ull ? 1 : 0);
  const bool aligned = align_level != 0;
  char* dst = const_cast<char*>(s_ptr[kMaxSrc]);
  const bool do_scale = (st.flags & OPF_FINAL) && scale != 1.0f;
  const long long count = cnt;
  const long long nvec = aligned ? count / VE : 0;
  const long long TT = (long long)nparts * blockDim.x;
  const long long g = (long long)part * blockDim.x + tid;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  long long i0 = g;
  if (align_level == 2) {
    // 256-bit accesses on pairs of vectors; a last odd vector is left to the 128-bit loop
    const long long nw = nvec / 2;
    long long j0 = g;
    if (nsrc == 1 && !do_scale) {
      // plain copy (gather / broadcast steps, staging): no arithmetic, full tiles with twice the bytes in flight
      constexpr int UC = 4;
      const char* p = s_ptr[0] + j0 * 32;
      char* d = dst + j0 * 32;
      const long long stride = TT * 32;
      for (; j0 + (long long)(UC - 1) * TT < nw; j0 += TT * UC) {
        uint4 lo[UC], hi[UC];
#pragma unroll
        for (int u = 0; u < UC; ++u) ld32_cg(p + u * stride, lo[u], hi[u]);
#pragma unroll
        for (int u = 0; u < UC; ++u) st32(d + u * stride, lo[u], hi[u]);
        p += UC * stride;
        d += UC * stride;
      }
    }
    // a tile with at most one vector per thread is bound by the depth of its chain of round trips: four sources at
    // a time; longer tiles by bytes in flight: two sources, two vectors deep (the same 128 bytes per thread)
    if (nw <= TT) reduce_loop32<T, 4, 1>(s_ptr, dst, nsrc, j0, nw, TT, op, do_scale, scale);
    else reduce_loop32<T, kSrcGroup, 2>(s_ptr, dst, nsrc, j0, nw, TT, op, do_scale, scale);
    i0 = nw * 2 + g;
  }
  constexpr int U = 2;
  for (; i0 < nvec; i0 += TT * U) {
    Acc a[U][VE];
    for (int s = 0; s < nsrc; s += G) {
      uint4 x[G][U];
#pragma unroll
      for (int gi = 0; gi < G; ++gi) {
        if (s + gi < nsrc) {
          const char* p0 = s_ptr[s + gi];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const long long i = i0 + (long long)u * TT;
            x[gi][u] = (i < nvec) ? ld16_cg(p0 + i * 16) : zero;
          }
        }
      }
#pragma unroll
      for (int gi = 0; gi < G; ++gi) {
        if (s + gi < nsrc) {
          if (gi == 0 && s == 0) {
#pragma unroll
            for (int u = 0; u < U; ++u) vec_to_acc<T>(x[0][u], a[u]);
          } else {
#pragma unroll
            for (int u = 0; u < U; ++u) vec_combine<T>(op, x[gi][u], a[u]);
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = i0 + (long long)u * TT;
      if (i < nvec) {
        if (do_scale) acc_scale<T>(a[u], scale);
        st16(dst + i * 16, acc_to_vec<T>(a[u]));
      }
    }
  }
  // scalar tail (or the whole step when some pointer is not 16-byte aligned)
  for (long long e = nvec * VE + g; e < count; e += TT) {
    Acc a = Elem<T>::up(reinterpret_cast<const T*>(s_ptr[0])[e]);
    for (int s = 1; s < nsrc; ++s)
      a = combine<Acc>(op, a, Elem<T>::up(__ldcg(reinterpret_cast<const T*>(s_ptr[s]) + e)));
    if (do_scale) a = (Acc)(a * scale);
    reinterpret_cast<T*>(dst)[e] = Elem<T>::down(a);
  }
}

// ------------------------------------------------------------------ the kernel
// Large steps of one round are independent of each other.  They are cut into tiles and the tiles are
// dealt to the CTAs row by row: tile j of every large step, then tile j + 1 of every large step, with
// the step order rotated by the rank.  All sources of a round are therefore pulled at the same time
// (the k-1 neighbour exchanges and the lanes of one round run concurrently, where the reference posts
// them one after the other: testing/custom_implementations/work_dir/all_reduce/all_reduce_radix_batch.cpp:343-364),
// and at any moment the P readers of one round are spread over P different owners instead of all
// reading from the owner that comes first in the schedule.
constexpr long long kTileGrain = 16 << 10;        // tiles are multiples of this (keeps 32-byte alignment for every type)
constexpr long long kTileMin = 16 << 10, kTileMax = 1 << 20;   // 16 KiB = one 32-byte vector per thread of a CTA

// This rank's own table entries move into shared memory: a round then finds its waits, steps, sources and signals
// there instead of through a chain of dependent global loads (about ten of them per launch of a two-round program).
// One word per thread and table first, all loads issued before any store, so that the tables arrive together;
// loops take what is left of a long table.  The tables keep their global indices: each returned pointer is moved
// back by the index of the rank's first entry.  Round waits and exit waits sit in two places of one global table
// and become two tables here.  (Not inlined: the interpreter's own register allocation stays as it is.)  The
// caller synchronises the CTA before the first use.
struct RankTables {
  const DevRound* rounds;
  const DevStep* steps;
  const DevSrc* srcs;
  const DevWait* waits;
  const DevWait* exit_waits;
  const int* sigs;
  const int* order;
  int n_exit;
};
__device__ __noinline__ RankTables tables_to_smem(const char* __restrict__ blob, const DevHeader* h, int rank, unsigned char* smem) {
  const int tid = threadIdx.x;
  const int nrounds = h->nrounds;
  const DevRank R = reinterpret_cast<const DevRank*>(blob + kDevRanksOffset)[rank];
  constexpr int NT = 7;
  const unsigned* g[NT] = {
      reinterpret_cast<const unsigned*>(reinterpret_cast<const DevRound*>(blob + h->off_rounds) + (size_t)rank * nrounds),
      reinterpret_cast<const unsigned*>(reinterpret_cast<const DevStep*>(blob + h->off_steps) + R.step0),
      reinterpret_cast<const unsigned*>(reinterpret_cast<const DevSrc*>(blob + h->off_srcs) + R.src0),
      reinterpret_cast<const unsigned*>(reinterpret_cast<const DevWait*>(blob + h->off_waits) + R.wait0),
      reinterpret_cast<const unsigned*>(reinterpret_cast<const DevWait*>(blob + h->off_waits) + R.exit0),
      reinterpret_cast<const unsigned*>(reinterpret_cast<const int*>(blob + h->off_sigs) + R.sig0),
      reinterpret_cast<const unsigned*>(reinterpret_cast<const int*>(blob + h->off_order) + R.ord0)};
  const int words[NT] = {nrounds * (int)(sizeof(DevRound) / 4), R.nstep * (int)(sizeof(DevStep) / 4),
                         R.nsrc * (int)(sizeof(DevSrc) / 4), R.nwait * (int)(sizeof(DevWait) / 4),
                         R.nexit * (int)(sizeof(DevWait) / 4), R.nsig, R.nord};
  unsigned* s[NT];
  s[0] = reinterpret_cast<unsigned*>(smem);
#pragma unroll
  for (int k = 1; k < NT; ++k) s[k] = s[k - 1] + ((words[k - 1] + 1) & ~1);     // 8-byte aligned starts
  unsigned first[NT];
#pragma unroll
  for (int k = 0; k < NT; ++k) first[k] = tid < words[k] ? g[k][tid] : 0u;
#pragma unroll
  for (int k = 0; k < NT; ++k)
    if (tid < words[k]) s[k][tid] = first[k];
#pragma unroll
  for (int k = 0; k < NT; ++k)
    for (int i = tid + (int)blockDim.x; i < words[k]; i += (int)blockDim.x) s[k][i] = g[k][i];
  RankTables t;
  t.rounds = reinterpret_cast<const DevRound*>(s[0]);
  t.steps = reinterpret_cast<const DevStep*>(s[1]) - R.step0;
  t.srcs = reinterpret_cast<const DevSrc*>(s[2]) - R.src0;
  t.waits = reinterpret_cast<const DevWait*>(s[3]) - R.wait0;
  t.exit_waits = reinterpret_cast<const DevWait*>(s[4]);
  t.sigs = reinterpret_cast<const int*>(s[5]) - R.sig0;
  t.order = reinterpret_cast<const int*>(s[6]) - R.ord0;
  t.n_exit = R.nexit;
  return t;
}

template <typename T>
__global__ void __launch_bounds__(kInterpThreads, 1)
interp_kernel(World w, const char* __restrict__ blob, IoTable io, int op, float scale, int tables_in_smem) {
  extern __shared__ __align__(16) unsigned char interp_tables[];
  const int rank = w.rank0 + (int)blockIdx.y;
  const unsigned nct = gridDim.x, cta = blockIdx.x;
  const int tid = threadIdx.x;
  Ctrl* c = w.ctrl[rank];
  // the epoch and the abort word are asked for first, so that they travel while the tables are fetched
  unsigned long long epoch_first = 0ull;
  unsigned abort_first = 0u;
  if (tid == 0) { epoch_first = ld_volatile_u64(&c->epoch); abort_first = ld_volatile_u32(&c->abort); }
  const DevHeader* h = reinterpret_cast<const DevHeader*>(blob);
  const DevRound* rounds = reinterpret_cast<const DevRound*>(blob + h->off_rounds) + (size_t)rank * h->nrounds;
  const DevStep* steps = reinterpret_cast<const DevStep*>(blob + h->off_steps);
  const DevSrc* srcs = reinterpret_cast<const DevSrc*>(blob + h->off_srcs);
  const DevWait* waits = reinterpret_cast<const DevWait*>(blob + h->off_waits);
  const int* sigs = reinterpret_cast<const int*>(blob + h->off_sigs);
  const int* exits = reinterpret_cast<const int*>(blob + h->off_exit);
  const int* order = reinterpret_cast<const int*>(blob + h->off_order);
  const int P = h->P, nrounds = h->nrounds;
  const DevWait* exit_waits = nullptr;   // this rank's exit waits; looked up in the global table when left null
  int n_exit = -1;
  if (tables_in_smem) {
    const RankTables tb = tables_to_smem(blob, h, rank, interp_tables);
    rounds = tb.rounds;
    steps = tb.steps;
    srcs = tb.srcs;
    waits = tb.waits;
    sigs = tb.sigs;
    order = tb.order;
    exit_waits = tb.exit_waits;
    n_exit = tb.n_exit;
  }

  __shared__ unsigned long long s_base;
  __shared__ int s_ok;
  __shared__ const char* s_ptr[kMaxSrc + 1];
  __shared__ int s_meta[4];
  if (tid == 0) {
    s_base = epoch_first;
    s_ok = abort_first ? 0 : 1;
  }
  __syncthreads();
  const unsigned long long base = s_base;
  unsigned gen = 0;
  // every peer has left the previous launch (its last round signals everybody)
  if (tid < P && tid != rank)
    if (!wait_flag_ge(&w.sig[rank][tid], base, c, w.timeout_ns, ST_TIMEOUT_ENTRY, rank, -1, tid)) s_ok = 0;
  __syncthreads();
  bool ok = s_ok != 0;

  for (int t = 0; t < nrounds && ok; ++t) {
    const DevRound R = rounds[t];
    for (int i = R.wait_begin + tid; i < R.wait_end; i += blockDim.x) {
      const DevWait wt = waits[i];
      if (!wait_flag_ge(&w.sig[rank][wt.peer], base + (unsigned long long)wt.need + 1ull, c, w.timeout_ns,
                        ST_TIMEOUT_ROUND, rank, t, wt.peer))
        s_ok = 0;
    }
    __syncthreads();
    ok = s_ok != 0;
    if (!ok) break;
    unsigned long long* tr = w.trace[rank];
    if (tr && cta == 0 && tid == 0 && t < w.trace_rounds) tr[2 * t] = globaltimer_ns();   // waits of round t satisfied
    const int nst = R.step_end - R.step_begin;
    if (nst > 0) {
      // Tile size: every CTA gets the same number m of tiles (one, unless that tile would exceed kTileMax), each as
      // large as that allows: the shortest chain of dependent round trips per CTA and the most bytes in flight per
      // thread, and no CTA left with one tile more than the others.  A large step is cut into q = nct * m / nb tiles.
      const int nb = R.nbig, nsmall = nst - nb;
      const long long grain_e = kTileGrain / (long long)sizeof(T), max_e = kTileMax / (long long)sizeof(T);
      long long te = kTileMin / (long long)sizeof(T);
      if (nb > 0) {
        long long m = (R.big_max * nb + (long long)nct * max_e - 1) / ((long long)nct * max_e);
        if (m < 1) m = 1;
        long long q = (long long)nct * m / nb;
        if (q < 1) q = 1;
        long long t = (R.big_max + q - 1) / q;
        t = (t + grain_e - 1) / grain_e * grain_e;
        if (t > te) te = t;
      }
      const long long rows = nb ? (R.big_max + te - 1) / te : 0;
      const long long nitems = (long long)nsmall + rows * nb;
      // work items of this round: the small steps (one CTA each), then the tiles of the large steps
      for (long long v = cta; v < nitems; v += nct) {
        int sidx;
        long long e0 = 0;
        if (v < nsmall) {
          sidx = order[R.ord_begin + nb + (int)v];
        } else {
          const long long u = v - nsmall;
          sidx = order[R.ord_begin + (int)((u % nb + rank) % nb)];
          e0 = (u / nb) * te;
        }
        const DevStep st = steps[sidx];
        if (e0 >= st.count) continue;
        long long cnt = st.count - e0;
        if (v >= nsmall && cnt > te) cnt = te;
        run_step<T>(st, srcs, w, io, rank, e0, cnt, 0u, 1u, op, scale, s_ptr, s_meta, h->limit);
      }
      ok = rank_barrier(c, nct, gen, w.timeout_ns, rank, t);
      if (!ok) break;
    }
    // (a round without steps only announces that this rank has entered: nothing to wait for)
    if (tr && cta == 0 && tid == 0 && t < w.trace_rounds) tr[2 * t + 1] = globaltimer_ns();  // round t complete on this rank
    if (cta == 0) {
      const int n = R.sig_end - R.sig_begin;
      for (int i = tid; i < n; i += blockDim.x) {
        __threadfence_system();
        st_release_sys(&w.sig[sigs[R.sig_begin + i]][rank], base + (unsigned long long)t + 1ull);
      }
    }
  }
  // peers that read this rank's caller buffers directly must be done with them
  if (ok) {
    if (n_exit < 0) {
      exit_waits = waits + exits[2 * rank];
      n_exit = exits[2 * rank + 1] - exits[2 * rank];
    }
    for (int i = tid; i < n_exit; i += blockDim.x) {
      const DevWait wt = exit_waits[i];
      wait_flag_ge(&w.sig[rank][wt.peer], base + (unsigned long long)wt.need + 1ull, c, w.timeout_ns,
                   ST_TIMEOUT_EXIT, rank, nrounds, wt.peer);
    }
  }
  rank_exit(c, nct, [&](Ctrl* cc) { cc->epoch = base + (unsigned long long)nrounds; });
}

// A world of one rank has no peers: a program is then a list of local copies.
// Large ones run on this lean kernel instead of the interpreter, whose register
// footprint allows one CTA per SM only; here eight resident 256-thread CTAs per SM
// with 256-bit accesses keep enough bytes in flight to fill HBM.  Bookkeeping (epoch, launch counter) is the
// interpreter's, so the two can be mixed freely on one communicator.
constexpr int kCopyThreads = 256;
constexpr int kCopyUnroll = 4;
constexpr int kCopyCtasPerSm = 16;   // two waves of eight resident CTAs: measured best for 1 GiB (6.46 TB/s read + write)

// nvec: number of 32-byte vectors; src / dst 32-byte aligned.
__global__ void __launch_bounds__(kCopyThreads)
local_copy_kernel(Ctrl* c, const char* __restrict__ src, char* __restrict__ dst, long long nvec, int nrounds) {
  const long long tile = (long long)kCopyThreads * kCopyUnroll;
  const long long ntiles = (nvec + tile - 1) / tile;
  for (long long t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const long long i0 = t * tile + threadIdx.x;
    uint4 lo[kCopyUnroll], hi[kCopyUnroll];
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) {
      const long long i = i0 + (long long)u * kCopyThreads;
      if (i < nvec) ld32_cg(src + i * 32, lo[u], hi[u]);
    }
#pragma unroll
    for (int u = 0; u < kCopyUnroll; ++u) {
      const long long i = i0 + (long long)u * kCopyThreads;
      if (i < nvec) st32(dst + i * 32, lo[u], hi[u]);
    }
  }
  rank_exit(c, gridDim.x, [&](Ctrl* cc) { cc->epoch = cc->epoch + (unsigned long long)nrounds; });
}

typedef void (*InterpFn)(World, const char*, IoTable, int, float, int);

static InterpFn pick_kernel(int dtype) {
  switch (dtype) {
    case DT_F32: return interp_kernel<float>;
    case DT_BF16: return interp_kernel<__nv_bfloat16>;
    case DT_F16: return interp_kernel<__half>;
    case DT_I32: return interp_kernel<int32_t>;
    case DT_F64: return interp_kernel<double>;
    case DT_I64: return interp_kernel<int64_t>;
    case DT_U8: return interp_kernel<uint8_t>;
  }
  return nullptr;
}

}  // namespace chb

using namespace chb;

extern "C" {

// Upload (once) and return the device blob of a program for this communicator.
static int get_blob(chb_comm* c, const chb_program* p, void** out) {
  auto it = c->blobs.find(p->uid);
  if (it != c->blobs.end()) { *out = it->second; return CHB_SUCCESS; }
  if (p->prog.stats.max_nsrc > kMaxSrc) { c->last_error = "program has a step with too many sources"; return CHB_ERR_UNSUPPORTED; }
  if (!ranges_ok(p->prog, &c->last_error)) return CHB_ERR_ARG;
  long long table_bytes = 0;
  std::vector<char> blob = make_blob(p->prog, &table_bytes);
  void* d = nullptr;
  if (cudaMalloc(&d, blob.size()) != cudaSuccess) { c->last_error = "cudaMalloc(program blob) failed"; return CHB_ERR_NO_MEM; }
  if (cudaMemcpy(d, blob.data(), blob.size(), cudaMemcpyHostToDevice) != cudaSuccess) {
    cudaFree(d);
    c->last_error = "cudaMemcpy(program blob) failed";
    return CHB_ERR_CUDA;
  }
  c->blobs[p->uid] = d;
  c->blob_table_bytes[p->uid] = table_bytes;
  *out = d;
  return CHB_SUCCESS;
}

int chb_program_prepare(chb_comm* c, const chb_program* p) {
  if (!c || !p) return CHB_ERR_ARG;
  void* d;
  return get_blob(c, p, &d);
}

void chb_program_release(chb_comm* c, const chb_program* p) {
  if (!c) return;
  if (!p) return;
  auto it = c->blobs.find(p->uid);
  if (it != c->blobs.end()) { cudaFree(it->second); c->blobs.erase(it); c->blob_table_bytes.erase(p->uid); }
  for (auto jt = c->ll_blobs.lower_bound(p->uid * 16u); jt != c->ll_blobs.end() && jt->first < (p->uid + 1) * 16u;) {
    cudaFree(jt->second.first);
    jt = c->ll_blobs.erase(jt);
  }
}

// Launch a compiled program.  in / out hold one pointer per local rank
// (nlocal entries).  A caller buffer that lies inside the rank's symmetric
// heap is peer-visible at the same offset on every rank; the program must
// have been compiled with in_symmetric / out_symmetric only if that holds.
int chb_run_program(chb_comm* c, const chb_program* p, int dtype, int op, const void* const* in,
                    void* const* out, float scale, int nctas, cudaStream_t stream) {
  if (!c || !p || !in || !out) return CHB_ERR_ARG;
  const Program& g = p->prog;
  if (g.P != c->P) { c->last_error = "program was compiled for a different number of ranks"; return CHB_ERR_ARG; }
  InterpFn fn = pick_kernel(dtype);
  if (!fn) return CHB_ERR_ARG;
  const size_t esz = (size_t)dtype_size(dtype);
  if ((size_t)g.work_elems * esz > c->scratch_bytes) {
    c->last_error = "program needs more symmetric scratch than the communicator has";
    return CHB_ERR_NO_MEM;
  }
  if (op == OP_PROD && (dtype == DT_U8)) return CHB_ERR_OP;
  if (c->P == 1 && c->nlocal == 1 && scale == 1.0f && g.ops.size() == 1 && g.nrounds == 1) {
    // single rank: the whole collective is one local copy
    const Op& o = g.ops[0];
    const long long bytes = o.count * (long long)esz;
    if (!o.acc && o.srcs.size() == 1 && o.srcs[0].buf == P_IN && o.dst_buf == P_OUT && bytes >= (1 << 20) && bytes % 32 == 0) {
      const char* sp = (const char*)in[0] + o.srcs[0].off * (long long)esz;
      char* dp = (char*)out[0] + o.dst_off * (long long)esz;
      if ((((uintptr_t)sp | (uintptr_t)dp) & 31u) == 0 && sp != dp) {
        const long long nvec = bytes / 32;
        const long long tiles = (nvec + kCopyThreads * kCopyUnroll - 1) / (kCopyThreads * kCopyUnroll);
        long long blocks = (long long)c->sm_count * kCopyCtasPerSm;
        if (blocks > tiles) blocks = tiles;
        local_copy_kernel<<<(unsigned)blocks, kCopyThreads, 0, stream>>>(c->ctrl, sp, dp, nvec, g.nrounds);
        if (cudaGetLastError() != cudaSuccess) { c->last_error = "copy launch failed"; return CHB_ERR_CUDA; }
        return CHB_SUCCESS;
      }
    }
  }
  void* blob;
  int rc = get_blob(c, p, &blob);
  if (rc) return rc;
  IoTable io{};
  for (int q = 0; q < c->P; ++q) { io.in[q] = nullptr; io.out[q] = nullptr; }
  for (int l = 0; l < c->nlocal; ++l) {
    io.in[c->rank + l] = (const char*)in[l];
    io.out[c->rank + l] = (char*)out[l];
  }
  if (c->nlocal == 1) {
    // peers' caller buffers: same offset inside their heaps
    if (g.reads_peer_in && g.in_symmetric) {
      for (int q = 0; q < c->P; ++q) {
        char* t = c->translate(in[0], c->rank, q);
        if (!t) { c->last_error = "input is not inside the symmetric heap"; return CHB_ERR_ARG; }
        io.in[q] = t;
      }
    }
    if (g.reads_peer_out && g.out_symmetric) {
      for (int q = 0; q < c->P; ++q) {
        char* t = c->translate(out[0], c->rank, q);
        if (!t) { c->last_error = "output is not inside the symmetric heap"; return CHB_ERR_ARG; }
        io.out[q] = t;
      }
    }
  }
  int per_rank_budget = c->max_ctas / (c->nlocal > 0 ? c->nlocal : 1);
  if (per_rank_budget < 1) per_rank_budget = 1;
  if (nctas <= 0) {
    // enough CTAs to keep NVLink busy for large steps, one for latency-bound programs
    long long bytes = (long long)std::max(g.in_elems, g.out_elems) * (long long)esz;
    // NVLink wants about 2 MB in flight per GPU (rate x loaded latency) and a thread keeps 128 bytes in flight:
    // bandwidth-bound sizes take (nearly) every SM, one CTA each
    nctas = bytes <= (64 << 10) ? 1 : (bytes <= (1 << 20) ? 32 : (bytes <= (4 << 20) ? 64 : 128));
    // a single-rank world only copies locally: HBM-bound, wants every SM
    if (c->P == 1 && bytes > (16 << 20)) nctas = per_rank_budget;
  }
  if (nctas > per_rank_budget) nctas = per_rank_budget;
  dim3 grid((unsigned)nctas, (unsigned)c->nlocal, 1), block(kInterpThreads, 1, 1);
  World w = c->world;
  const char* blobp = (const char*)blob;
  // a rank's own table entries go to shared memory when they fit what every kernel may have without opting in
  const long long table_bytes = c->blob_table_bytes[p->uid];
  int in_smem = table_bytes > 0 && table_bytes + 64 <= kInterpSmemTables && tables_in_smem_wanted() ? 1 : 0;
  const size_t smem = in_smem ? (size_t)table_bytes + 64 : 0;      // + the padding between the tables
  void* args[] = {&w, &blobp, &io, &op, &scale, &in_smem};
  cudaError_t e;
  if (c->nlocal > 1 || nctas > 1) e = cudaLaunchCooperativeKernel((const void*)fn, grid, block, args, smem, stream);
  else e = cudaLaunchKernel((const void*)fn, grid, block, args, smem, stream);
  if (e != cudaSuccess) {
    c->last_error = std::string("interp launch failed: ") + cudaGetErrorString(e);
    return CHB_ERR_CUDA;
  }
  return CHB_SUCCESS;
}

}  // extern "C"

// Step programs executed with flagged lines: the latency-bound way to run ANY schedule.
//
// The pull interpreter (interp.cu) pays, per round, a grid barrier, a release
// store, an acquire poll and a load round trip over NVLink.  Here every remote
// source of a step becomes a message that its OWNER pushes, as 16-byte lines
// {data, flag, data, flag}, into a slot of the reader's inbox reserved for that
// (step, source) pair; the reader polls its own memory until the line carries
// the flag of this launch.  A round then costs one NVLink traversal and no
// cross-GPU barrier, whatever the algorithm: the radix-k / group-b shapes, the
// recursive-doubling and Rabenseifner baselines and the rest can be compared in
// the regime where the number of rounds decides (the regime of the reference's
// published wins, testing/plots/all_reduce/results_custom_polaris.csv).
//
// Level t of a rank (t = round of the lowered program):
//   1. push: every region of mine that a peer's step of level t reads goes to
//      that peer's inbox.  It was written by my own steps of levels < t.
//   2. execute my steps of level t: local sources are loaded, remote ones are
//      polled in the inbox, combined left to right, stored once.
// Steps of one level never conflict (the lowering guarantees it), so 1 and 2 of
// the same level need no ordering.
//
// Levels overlap line by line.  When a region that a peer reads at level t + 1
// lies inside the destination of one of my steps of level t, the thread that
// produces a line of that step forwards it to the peer at once, from registers:
// the peer's next round starts on line c as soon as line c of this round
// exists, not when the round is complete (the reference waits for whole rounds:
// MPI_Waitall at testing/custom_implementations/work_dir/all_reduce/all_reduce_radix_batch.cpp:622).
// A rank-local barrier separates two levels only where the later one reads or
// overwrites local memory that the earlier one wrote or read; for the flat
// two-round allreduce, for instance, none is left.
// Owners push from inside their own launch, so an input is never read before
// its owner's stream has produced it, and nobody reads a peer's buffers: no
// entry handshake, no exit waits, no staging of caller buffers.
//
// Flags are launch sequence numbers shared with the one-shot kernels (ll.cu);
// the two inbox halves alternate by launch parity.  That is sound for
// collectives in which every rank's result depends on every rank's input
// (allreduce, reduce-scatter, allgather, all-to-all): a rank can finish launch n only after
// every peer has entered launch n, so nobody is ever two launches ahead.
#include <algorithm>
#include <cstring>
#include <vector>

#include "../api/chb.h"
#include "../api/program_handle.h"
#include "../sched/ll_plan.h"
#include "../symm/comm.h"
#include "common.cuh"
#include "ll_lines.cuh"

namespace chb {

constexpr int kLPThreads = 512;
constexpr long long kLPSmemTables = 40 << 10;   // bytes of table entries a CTA keeps in shared memory
constexpr int kLPMaxCtas = 128;   // an explicit request may go this far; the default stops at 64

struct LPIo {
  const char* in[kMaxRanks];
  char* out[kMaxRanks];
};

// Index of the item in [begin, end) whose line range holds global line gl (prefixes ascend from 0).
template <typename Item>
__device__ __forceinline__ int find_item(const Item* items, int begin, int end, long long gl) {
  int lo = begin, hi = end - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (items[mid].line_prefix <= gl) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

template <typename T>
__global__ void __launch_bounds__(kLPThreads, 1)
llprog_kernel(World w, const char* __restrict__ blob, LPIo io, int op, float scale, long long lines_per_src,
              int tables_in_smem) {
  using Acc = typename Elem<T>::Acc;
  constexpr int PE = (int)(8 / sizeof(T));     // elements per line
  extern __shared__ __align__(16) unsigned char lp_tables[];
  const int rank = w.rank0 + (int)blockIdx.y;
  const unsigned nct = gridDim.x;
  Ctrl* c = w.ctrl[rank];
  // the launch number and the abort word are asked for first, so that they travel while the tables are fetched
  unsigned long long seq_first = 0ull;
  int abort_first = 0;
  if (threadIdx.x == 0) { seq_first = ld_volatile_u64(&c->ll_seq); abort_first = ld_volatile_u32(&c->abort); }
  const LPHeader* h = reinterpret_cast<const LPHeader*>(blob);
  const int nlevels = h->nlevels;
  const LPLevel* levels = reinterpret_cast<const LPLevel*>(blob + h->off_levels) + (size_t)rank * nlevels;
  const LPStep* steps = reinterpret_cast<const LPStep*>(blob + h->off_steps);
  const LPSrc* srcs = reinterpret_cast<const LPSrc*>(blob + h->off_srcs);
  const LPSend* sends = reinterpret_cast<const LPSend*>(blob + h->off_sends);
  const LPFwd* fwds = reinterpret_cast<const LPFwd*>(blob + h->off_fwds);
  if (tables_in_smem) {
    // This rank's own table entries move into shared memory: every lookup below (which send or step owns a line,
    // its sources, its forwards) is then a shared-memory access instead of a chain of dependent global loads,
    // which is most of the time of a small message.  One 8-byte word per thread and table first, all loads issued
    // before any store, so the five tables arrive together; loops take what is left of a long table.
    const LPRank R = reinterpret_cast<const LPRank*>(blob + kLPRanksOffset)[rank];
    const unsigned long long* g[5] = {
        reinterpret_cast<const unsigned long long*>(levels), reinterpret_cast<const unsigned long long*>(steps + R.step0),
        reinterpret_cast<const unsigned long long*>(srcs + R.src0), reinterpret_cast<const unsigned long long*>(sends + R.send0),
        reinterpret_cast<const unsigned long long*>(fwds + R.fwd0)};
    const int words[5] = {nlevels * (int)(sizeof(LPLevel) / 8), R.nstep * (int)(sizeof(LPStep) / 8), R.nsrc * (int)(sizeof(LPSrc) / 8),
                          R.nsend * (int)(sizeof(LPSend) / 8), R.nfwd * (int)(sizeof(LPFwd) / 8)};
    unsigned long long* s[5];
    s[0] = reinterpret_cast<unsigned long long*>(lp_tables);
#pragma unroll
    for (int k = 1; k < 5; ++k) s[k] = s[k - 1] + words[k - 1];
    unsigned long long first[5];
#pragma unroll
    for (int k = 0; k < 5; ++k) first[k] = (int)threadIdx.x < words[k] ? g[k][threadIdx.x] : 0ull;
#pragma unroll
    for (int k = 0; k < 5; ++k)
      if ((int)threadIdx.x < words[k]) s[k][threadIdx.x] = first[k];
#pragma unroll
    for (int k = 0; k < 5; ++k)
      for (int i = (int)threadIdx.x + (int)blockDim.x; i < words[k]; i += (int)blockDim.x) s[k][i] = g[k][i];
    // the tables keep their global indices: each pointer is moved back by the index of the rank's first entry
    levels = reinterpret_cast<const LPLevel*>(s[0]);
    steps = reinterpret_cast<const LPStep*>(s[1]) - R.step0;
    srcs = reinterpret_cast<const LPSrc*>(s[2]) - R.src0;
    sends = reinterpret_cast<const LPSend*>(s[3]) - R.send0;
    fwds = reinterpret_cast<const LPFwd*>(s[4]) - R.fwd0;
  }
  __shared__ unsigned long long s_seq;
  __shared__ int s_abort;
  if (threadIdx.x == 0) { s_seq = seq_first; s_abort = abort_first; }
  __syncthreads();
  const unsigned long long seq = s_seq;
  bool dead = s_abort != 0;                 // this thread does no more work (an expired wait, or an aborted rank)
  const unsigned flag = (unsigned)(seq % 0xFFFFFFFFull) + 1u;
  const long long half = (long long)(seq & 1ull) * w.P * lines_per_src;
  const long long TT = (long long)nct * blockDim.x;
  const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const bool do_scale = scale != 1.0f;
  const char* my_in = io.in[rank];
  char* my_out = io.out[rank];
  char* my_work = w.work[rank];
  const char* inbox = w.ll[rank] + half * 16;
  unsigned gen = 0;

  for (int t = 0; t < nlevels; ++t) {
    const LPLevel L = levels[t];
    // a level that touches local memory of the levels before it starts only when those are complete on this rank;
    // all threads take part in the barrier, also those that have given up, and an aborted rank leaves here together
    if (L.barrier_before && !rank_barrier(c, nct, gen, w.timeout_ns, rank, t)) break;
    // per-level stamps of the first thread (the counterpart of the interpreter's per-round trace): when it starts
    // the level and when its own share of the level is done
    unsigned long long* tr = w.trace[rank];
    const bool stamp = tr && gtid == 0 && t < w.trace_rounds;
    if (stamp) tr[2 * t] = globaltimer_ns();
    // ---- 1. push what peers' steps of this level read from me (and no step of mine has forwarded already):
    // four lines of a thread at a time, all payload loads issued before the first store
    {
      int cur = -1;
      LPSend S{};
      long long end = 0;
      for (long long gl0 = gtid; gl0 < L.send_lines && !dead; gl0 += kLineGroup * TT) {
        const char* from[kLineGroup];
        char* to[kLineGroup];
        long long at[kLineGroup], len[kLineGroup];
#pragma unroll
        for (int u = 0; u < kLineGroup; ++u) {
          const long long gl = gl0 + u * TT;
          from[u] = nullptr;
          to[u] = nullptr;
          at[u] = len[u] = 0;
          if (gl < L.send_lines) {
            if (cur < 0 || gl >= end) {
              cur = find_item(sends, L.send_begin, L.send_end, gl);
              S = sends[cur];
              end = S.line_prefix + (S.count * (long long)sizeof(T) + 7) / 8;
            }
            const long long l = gl - S.line_prefix;
            from[u] = (S.src_buf == 0 ? my_in : (S.src_buf == 1 ? my_out : my_work)) + S.src_off * (long long)sizeof(T);
            at[u] = l * 8;
            len[u] = S.count * (long long)sizeof(T);
            to[u] = w.ll[S.dst_rank] + (half + S.inbox_line + l) * 16;
          }
        }
        uint2 v[kLineGroup];
#pragma unroll
        for (int u = 0; u < kLineGroup; ++u) v[u] = from[u] ? load_payload(from[u], at[u], len[u]) : make_uint2(0u, 0u);
#pragma unroll
        for (int u = 0; u < kLineGroup; ++u)
          if (to[u]) st_line(to[u], v[u].x, v[u].y, flag);
      }
    }
    // ---- 2. my steps of this level
    int cur = -1;
    LPStep st{};
    long long end = 0;
    // a level of plain copies (an allgather round): four lines of a thread at a time, their inbox lines read together
    for (long long gl0 = gtid; L.all_copy && gl0 < L.step_lines && !dead; gl0 += kLineGroup * TT) {
      const char* line[kLineGroup];
      int peer[kLineGroup], item[kLineGroup];
      long long at[kLineGroup];
      uint2 x[kLineGroup];
#pragma unroll
      for (int u = 0; u < kLineGroup; ++u) {
        const long long gl = gl0 + u * TT;
        line[u] = nullptr;
        peer[u] = -1;
        item[u] = 0;
        at[u] = 0;
        x[u] = make_uint2(0u, 0u);
        if (gl < L.step_lines) {
          if (cur < 0 || gl >= end) {
            cur = find_item(steps, L.step_begin, L.step_end, gl);
            st = steps[cur];
            end = st.line_prefix + (st.count * (long long)sizeof(T) + 7) / 8;
          }
          const LPSrc sc = srcs[st.src_begin];
          item[u] = cur;
          at[u] = gl - st.line_prefix;
          peer[u] = sc.peer;
          line[u] = inbox + (sc.inbox_line + at[u]) * 16;
        }
      }
      if (!poll_lines(line, peer, flag, x, c, w.timeout_ns, rank, gl0)) { dead = true; break; }
#pragma unroll
      for (int u = 0; u < kLineGroup; ++u) {
        if (line[u] == nullptr) continue;
        const LPStep s2 = steps[item[u]];
        char* dst = (s2.dst_buf == 1 ? my_out : my_work) + s2.dst_off * (long long)sizeof(T);
        store_payload(dst, at[u] * 8, s2.count * (long long)sizeof(T), x[u]);
        for (int f = 0; f < s2.nfwd; ++f) {
          const LPFwd F = fwds[s2.fwd_begin + f];
          const long long lf = at[u] - F.line_begin;
          if (lf >= 0 && lf < F.nlines) st_line(w.ll[F.dst_rank] + (half + F.inbox_line + lf) * 16, x[u].x, x[u].y, flag);
        }
      }
    }
    for (long long gl = gtid; !L.all_copy && gl < L.step_lines && !dead; gl += TT) {
      if (cur < 0 || gl >= end) {
        cur = find_item(steps, L.step_begin, L.step_end, gl);
        st = steps[cur];
        end = st.line_prefix + (st.count * (long long)sizeof(T) + 7) / 8;
      }
      const long long l = gl - st.line_prefix;
      const long long nbytes = st.count * (long long)sizeof(T);
      char* dst = (st.dst_buf == 1 ? my_out : my_work) + st.dst_off * (long long)sizeof(T);
      const bool acc = (st.flags & 0x100u) != 0;
      Acc a[PE];
      uint2 v = make_uint2(0u, 0u);
      bool have = false;
      if (acc) { payload_to_acc<T>(load_payload(dst, l * 8, nbytes), a); have = true; }
      // sources four at a time: their table entries are loaded together, their lines are read together (one
      // memory latency for the group instead of one per source), then combined left to right; a line that has
      // not arrived yet is polled on its own
      for (int j0 = 0; j0 < st.nsrc && !dead; j0 += kLineGroup) {
        const char* line[kLineGroup];
        int peer[kLineGroup];
        uint2 x[kLineGroup];
#pragma unroll
        for (int jj = 0; jj < kLineGroup; ++jj) {
          line[jj] = nullptr;
          peer[jj] = -1;
          x[jj] = make_uint2(0u, 0u);
          if (j0 + jj < st.nsrc) {
            const LPSrc sc = srcs[st.src_begin + j0 + jj];
            peer[jj] = sc.peer;
            if (sc.inbox_line >= 0) {
              line[jj] = inbox + (sc.inbox_line + l) * 16;
            } else {
              const char* base = (sc.buf == 0 ? my_in : (sc.buf == 1 ? my_out : my_work)) + sc.off * (long long)sizeof(T);
              x[jj] = load_payload(base, l * 8, nbytes);
            }
          }
        }
        if (!poll_lines(line, peer, flag, x, c, w.timeout_ns, rank, l)) { dead = true; break; }
#pragma unroll
        for (int jj = 0; jj < kLineGroup; ++jj) {
          if (j0 + jj < st.nsrc) {
            v = x[jj];
            if (!have) { payload_to_acc<T>(v, a); have = true; }
            else payload_combine<T>(op, v, a);
          }
        }
      }
      if (dead) break;
      // a plain copy keeps the payload's bits; everything else goes through the accumulator type
      if (acc || st.nsrc > 1 || (do_scale && (st.flags & OPF_FINAL)))
        v = acc_to_payload<T>(a, scale, do_scale && (st.flags & OPF_FINAL));
      store_payload(dst, l * 8, nbytes, v);
      // the next level's readers of this line get it now, from registers
      // (table entries four at a time, so that their loads overlap instead of queueing behind the stores)
      for (int f0 = 0; f0 < st.nfwd; f0 += kLineGroup) {
        char* to[kLineGroup];
#pragma unroll
        for (int i = 0; i < kLineGroup; ++i) {
          to[i] = nullptr;
          if (f0 + i < st.nfwd) {
            const LPFwd F = fwds[st.fwd_begin + f0 + i];
            const long long lf = l - F.line_begin;
            if (lf >= 0 && lf < F.nlines) to[i] = w.ll[F.dst_rank] + (half + F.inbox_line + lf) * 16;
          }
        }
#pragma unroll
        for (int i = 0; i < kLineGroup; ++i)
          if (to[i] != nullptr) st_line(to[i], v.x, v.y, flag);
      }
    }
    if (stamp) tr[2 * t + 1] = globaltimer_ns();
  }
  rank_exit(c, nct, [&](Ctrl* cc) { cc->ll_seq = seq + 1ull; });
}

typedef void (*LPFn)(World, const char*, LPIo, int, float, long long, int);
static LPFn pick_lp(int dtype) {
  switch (dtype) {
    case DT_F32: return llprog_kernel<float>;
    case DT_BF16: return llprog_kernel<__nv_bfloat16>;
    case DT_F16: return llprog_kernel<__half>;
    case DT_I32: return llprog_kernel<int32_t>;
    case DT_F64: return llprog_kernel<double>;
    case DT_I64: return llprog_kernel<int64_t>;
    case DT_U8: return llprog_kernel<uint8_t>;
  }
  return nullptr;
}

}  // namespace chb

using namespace chb;

extern "C" {

// Run a compiled program with flagged lines (see the head of this file).  The program must have been
// lowered with in_symmetric and out_symmetric set (no staging copies are wanted: nobody reads a peer's
// buffers here, so the caller's buffers may live anywhere), for a collective in which every rank's
// result depends on every rank's input.  in / out: one pointer per local rank.
// Returns CHB_ERR_COUNT when the messages do not fit the inbox.
int chb_run_program_ll(chb_comm* c, const chb_program* p, int dtype, int op, const void* const* in,
                       void* const* out, float scale, int nctas, cudaStream_t stream) {
  if (!c || !p || !in || !out) return CHB_ERR_ARG;
  const Program& g = p->prog;
  if (g.P != c->P) { c->last_error = "program was compiled for a different number of ranks"; return CHB_ERR_ARG; }
  LPFn fn = pick_lp(dtype);
  if (!fn) return CHB_ERR_ARG;
  const int esz = dtype_size(dtype);
  if (op == OP_PROD && dtype == DT_U8) return CHB_ERR_OP;
  if ((g.reads_peer_in && !g.in_symmetric) || (g.reads_peer_out && !g.out_symmetric)) {
    c->last_error = "flagged-line execution wants a program lowered without staging copies";
    return CHB_ERR_ARG;
  }
  if ((size_t)g.work_elems * (size_t)esz > c->scratch_bytes) {
    c->last_error = "program needs more scratch than the communicator has";
    return CHB_ERR_NO_MEM;
  }
  const uint64_t key = p->uid * 16u + (uint64_t)esz;
  void* blob = nullptr;
  LPHeader hd{};
  auto it = c->ll_blobs.find(key);
  if (it != c->ll_blobs.end()) {
    blob = it->second.first;
    hd.max_level_lines = it->second.second.first;
    hd.rank_table_bytes = it->second.second.second;
  } else {
    std::vector<char> host = make_ll_blob(g, esz, &hd);
    if (hd.inbox_lines > (long long)c->P * (long long)c->ll_lines_per_src) {
      c->last_error = "messages of this program exceed the flagged-line inbox";
      return CHB_ERR_COUNT;
    }
    if (cudaMalloc(&blob, host.size()) != cudaSuccess) { c->last_error = "cudaMalloc(program lines) failed"; return CHB_ERR_NO_MEM; }
    if (cudaMemcpy(blob, host.data(), host.size(), cudaMemcpyHostToDevice) != cudaSuccess) {
      cudaFree(blob);
      c->last_error = "cudaMemcpy(program lines) failed";
      return CHB_ERR_CUDA;
    }
    c->ll_blobs[key] = {blob, {hd.max_level_lines, hd.rank_table_bytes}};
  }
  LPIo io{};
  for (int l = 0; l < c->nlocal; ++l) {
    io.in[c->rank + l] = (const char*)in[l];
    io.out[c->rank + l] = (char*)out[l];
  }
  int budget = c->max_ctas / (c->nlocal > 0 ? c->nlocal : 1);
  if (budget < 1) budget = 1;
  if (nctas <= 0) {
    // about four lines per thread in the busiest level
    nctas = (int)((hd.max_level_lines + kLPThreads * 4 - 1) / (kLPThreads * 4));
    if (nctas > 64) nctas = 64;
  }
  if (nctas > kLPMaxCtas) nctas = kLPMaxCtas;
  if (nctas > budget) nctas = budget;
  if (nctas < 1) nctas = 1;
  dim3 grid((unsigned)nctas, (unsigned)c->nlocal, 1), block(kLPThreads, 1, 1);
  World w = c->world;
  const char* bp = (const char*)blob;
  long long lps = (long long)c->ll_lines_per_src;
  // a rank's own table entries go to shared memory when they fit what every kernel may have without opting in
  int in_smem = hd.rank_table_bytes > 0 && hd.rank_table_bytes <= kLPSmemTables && tables_in_smem_wanted() ? 1 : 0;
  const size_t smem = in_smem ? (size_t)hd.rank_table_bytes : 0;
  void* args[] = {&w, &bp, &io, &op, &scale, &lps, &in_smem};
  cudaError_t e;
  if (c->nlocal > 1 || nctas > 1) e = cudaLaunchCooperativeKernel((const void*)fn, grid, block, args, smem, stream);
  else e = cudaLaunchKernel((const void*)fn, grid, block, args, smem, stream);
  if (e != cudaSuccess) { c->last_error = std::string("flagged-line program launch failed: ") + cudaGetErrorString(e); return CHB_ERR_CUDA; }
  return CHB_SUCCESS;
}

}  // extern "C"

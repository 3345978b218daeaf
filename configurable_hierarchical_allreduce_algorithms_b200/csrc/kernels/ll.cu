// One-shot collectives for latency-bound sizes: every rank pushes its data
// straight into the peers' inboxes as 16-byte lines {data, flag, data, flag}
// and every rank polls its own (local) inbox, so a whole allreduce /
// reduce-scatter / allgather costs one launch and one NVLink traversal, with
// no barrier at all.  The flag is the launch sequence number, never reset;
// two inbox halves alternate by launch parity, which is enough because a rank
// can run at most one launch ahead of the slowest peer (it needs that peer's
// lines of the current launch to finish it).
//
// This is the large-radix / single-round end of the design space the
// reference explores with k >= b (one phase, every peer at once:
// testing/custom_implementations/work_dir/all_reduce/all_reduce_radix_batch.cpp:339-368
// with nphases == 1), taken to its limit on a full-bandwidth switch.
// Sums run in rank order 0..P-1 on every rank, so all ranks obtain
// bit-identical results.
#include <cstdio>

#include "../api/chb.h"
#include "../symm/comm.h"
#include "common.cuh"
#include "ll_lines.cuh"

namespace chb {

constexpr int kLLThreads = 512;
enum { LL_AR = 0, LL_RS = 1, LL_AG = 2 };

struct LLIo {
  const char* in[kMaxRanks];
  char* out[kMaxRanks];
};

// nbytes: payload bytes each rank sends to one peer (AR: whole vector; RS / AG: one block)
template <typename T, int MODE>
__global__ void __launch_bounds__(kLLThreads, 1)
ll_kernel(World w, LLIo io, long long nbytes, int op, float scale, long long lines_per_src) {
  using Acc = typename Elem<T>::Acc;
  const int rank = w.rank0 + (int)blockIdx.y;
  const int P = w.P;
  const unsigned nct = gridDim.x;
  Ctrl* c = w.ctrl[rank];
  __shared__ unsigned long long s_seq;
  __shared__ int s_abort;
  if (threadIdx.x == 0) { s_seq = ld_volatile_u64(&c->ll_seq); s_abort = ld_volatile_u32(&c->abort); }
  __syncthreads();
  const unsigned long long seq = s_seq;
  const bool dead = s_abort != 0;
  const unsigned flag = (unsigned)(seq % 0xFFFFFFFFull) + 1u;
  const long long half = (long long)(seq & 1ull) * P;
  const long long nlines = (nbytes + 7) / 8;
  const long long TT = (long long)nct * blockDim.x;
  const char* in = io.in[rank];
  char* out = io.out[rank];
  const bool do_scale = scale != 1.0f;

  const long long l0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  // ---- push all my lines to every peer first, so that they travel together
  for (long long l = l0; l < nlines && !dead; l += TT) {
    uint2 mine = make_uint2(0u, 0u);
    if (MODE != LL_RS) mine = load_payload(in, l * 8, nbytes);
    for (int i = 1; i < P; ++i) {
      const int p = (rank + i) % P;
      uint2 v = (MODE == LL_RS) ? load_payload(in + (long long)p * nbytes, l * 8, nbytes) : mine;
      st_line(w.ll[p] + ((half + rank) * lines_per_src + l) * 16, v.x, v.y, flag);
    }
  }
  // ---- collect the peers' lines from my inbox, combining in rank order
  for (long long l = l0; l < nlines && !dead; l += TT) {
    const uint2 mine = load_payload(in + (MODE == LL_RS ? (long long)rank * nbytes : 0ll), l * 8, nbytes);
    Acc a[8 / sizeof(T)];
    bool have = false, failed = false;
    for (int p0 = 0; p0 < P && !failed; p0 += kLineGroup) {
      const char* line[kLineGroup];
      int peer[kLineGroup];
      uint2 v[kLineGroup];
#pragma unroll
      for (int i = 0; i < kLineGroup; ++i) {
        const int p = p0 + i;
        peer[i] = p;
        v[i] = mine;
        line[i] = (p < P && p != rank) ? w.ll[rank] + ((half + p) * lines_per_src + l) * 16 : nullptr;
      }
      if (!poll_lines(line, peer, flag, v, c, w.timeout_ns, rank, l)) { failed = true; break; }
#pragma unroll
      for (int i = 0; i < kLineGroup; ++i) {
        const int p = p0 + i;
        if (p >= P) continue;
        if (MODE == LL_AG) {
          store_payload(out + (long long)p * nbytes, l * 8, nbytes, v[i]);
        } else {
          if (!have) { payload_to_acc<T>(v[i], a); have = true; }
          else payload_combine<T>(op, v[i], a);
        }
      }
    }
    if (failed) break;
    if (MODE != LL_AG) store_payload(out, l * 8, nbytes, acc_to_payload<T>(a, scale, do_scale));
  }
  rank_exit(c, nct, [&](Ctrl* cc) { cc->ll_seq = seq + 1ull; });
}

// Two-shot allreduce with flagged lines: rank r first receives everybody's
// slice r (lines in the lower half of each source slot), reduces it in rank
// order, then pushes the reduced slice to everybody (upper half of its slot).
// Bytes on the wire per rank: 2 * 2 * (P-1)/P * vector (the factor 2 is the
// flag overhead), against 2 * (P-1) * vector for the one-shot form, and still
// no barrier.  slice_bytes: bytes of one slice (vector = P slices, the last
// one may be shorter: total_bytes).
template <typename T>
__global__ void __launch_bounds__(kLLThreads, 1)
ll2_kernel(World w, LLIo io, long long total_bytes, long long slice_bytes, int op, float scale,
           long long lines_per_src) {
  using Acc = typename Elem<T>::Acc;
  const int rank = w.rank0 + (int)blockIdx.y;
  const int P = w.P;
  const unsigned nct = gridDim.x;
  Ctrl* c = w.ctrl[rank];
  __shared__ unsigned long long s_seq;
  __shared__ int s_abort;
  if (threadIdx.x == 0) { s_seq = ld_volatile_u64(&c->ll_seq); s_abort = ld_volatile_u32(&c->abort); }
  __syncthreads();
  const unsigned long long seq = s_seq;
  const bool dead = s_abort != 0;
  const unsigned flag = (unsigned)(seq % 0xFFFFFFFFull) + 1u;
  const long long half = (long long)(seq & 1ull) * P;
  const long long upper = lines_per_src / 2;   // first line of the broadcast half of a slot
  const long long TT = (long long)nct * blockDim.x;
  const long long l0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const char* in = io.in[rank];
  char* out = io.out[rank];
  const bool do_scale = scale != 1.0f;
  auto slice_len = [&](int p) {
    long long lo = (long long)p * slice_bytes;
    long long n = total_bytes - lo;
    return n < 0 ? 0ll : (n > slice_bytes ? slice_bytes : n);
  };
  const long long max_lines = (slice_bytes + 7) / 8;
  // phase A: scatter my contribution to every slice owner
  for (long long l = l0; l < max_lines && !dead; l += TT)
    for (int i = 1; i < P; ++i) {
      const int p = (rank + i) % P;
      const long long n = slice_len(p);
      if (l * 8 < n) {
        const uint2 v = load_payload(in + (long long)p * slice_bytes, l * 8, n);
        st_line(w.ll[p] + ((half + rank) * lines_per_src + l) * 16, v.x, v.y, flag);
      }
    }
  // phase B: reduce my slice in rank order, store it and push it to everybody
  const long long mine_n = slice_len(rank);
  bool failed = false;
  for (long long l = l0; l * 8 < mine_n && !dead && !failed; l += TT) {
    Acc a[8 / sizeof(T)];
    const uint2 mine = load_payload(in + (long long)rank * slice_bytes, l * 8, mine_n);
    for (int p0 = 0; p0 < P && !failed; p0 += kLineGroup) {
      const char* line[kLineGroup];
      int peer[kLineGroup];
      uint2 v[kLineGroup];
#pragma unroll
      for (int i = 0; i < kLineGroup; ++i) {
        const int p = p0 + i;
        peer[i] = p;
        v[i] = mine;
        line[i] = (p < P && p != rank) ? w.ll[rank] + ((half + p) * lines_per_src + l) * 16 : nullptr;
      }
      if (!poll_lines(line, peer, flag, v, c, w.timeout_ns, rank, l)) { failed = true; break; }
#pragma unroll
      for (int i = 0; i < kLineGroup; ++i) {
        const int p = p0 + i;
        if (p >= P) continue;
        if (p == 0) payload_to_acc<T>(v[i], a);
        else payload_combine<T>(op, v[i], a);
      }
    }
    if (failed) break;
    const uint2 r = acc_to_payload<T>(a, scale, do_scale);
    store_payload(out + (long long)rank * slice_bytes, l * 8, mine_n, r);
    for (int i = 1; i < P; ++i) {
      const int p = (rank + i) % P;
      st_line(w.ll[p] + ((half + rank) * lines_per_src + upper + l) * 16, r.x, r.y, flag);
    }
  }
  // phase C: collect the other reduced slices
  for (long long l = l0; l < max_lines && !dead && !failed; l += TT)
    for (int i0 = 1; i0 < P && !failed; i0 += kLineGroup) {
      const char* line[kLineGroup];
      int peer[kLineGroup];
      uint2 v[kLineGroup];
#pragma unroll
      for (int i = 0; i < kLineGroup; ++i) {
        const int p = (rank + i0 + i) % P;
        peer[i] = p;
        v[i] = make_uint2(0u, 0u);
        line[i] = (i0 + i < P && l * 8 < slice_len(p)) ? w.ll[rank] + ((half + p) * lines_per_src + upper + l) * 16 : nullptr;
      }
      if (!poll_lines(line, peer, flag, v, c, w.timeout_ns, rank, l)) { failed = true; break; }
#pragma unroll
      for (int i = 0; i < kLineGroup; ++i)
        if (line[i] != nullptr) store_payload(out + (long long)peer[i] * slice_bytes, l * 8, slice_len(peer[i]), v[i]);
    }
  rank_exit(c, nct, [&](Ctrl* cc) { cc->ll_seq = seq + 1ull; });
}

typedef void (*LL2Fn)(World, LLIo, long long, long long, int, float, long long);
static LL2Fn pick_ll2(int dtype) {
  switch (dtype) {
    case DT_F32: return ll2_kernel<float>;
    case DT_BF16: return ll2_kernel<__nv_bfloat16>;
    case DT_F16: return ll2_kernel<__half>;
    case DT_I32: return ll2_kernel<int32_t>;
    case DT_F64: return ll2_kernel<double>;
    case DT_I64: return ll2_kernel<int64_t>;
    case DT_U8: return ll2_kernel<uint8_t>;
  }
  return nullptr;
}

typedef void (*LLFn)(World, LLIo, long long, int, float, long long);

template <int MODE>
static LLFn pick_ll(int dtype) {
  switch (dtype) {
    case DT_F32: return ll_kernel<float, MODE>;
    case DT_BF16: return ll_kernel<__nv_bfloat16, MODE>;
    case DT_F16: return ll_kernel<__half, MODE>;
    case DT_I32: return ll_kernel<int32_t, MODE>;
    case DT_F64: return ll_kernel<double, MODE>;
    case DT_I64: return ll_kernel<int64_t, MODE>;
    case DT_U8: return ll_kernel<uint8_t, MODE>;
  }
  return nullptr;
}

}  // namespace chb

using namespace chb;

extern "C" {

// Largest payload (bytes per rank pair) the inbox can take.
long long chb_ll_max_bytes(const chb_comm* c) { return c ? (long long)c->ll_lines_per_src * 8 : 0; }

// Largest vector (bytes) the two-shot flagged-line allreduce can take.
long long chb_ll2_max_bytes(const chb_comm* c) {
  return c ? (long long)(c->ll_lines_per_src / 2) * 8 * c->P : 0;
}

// mode: 0 allreduce (count = vector length), 1 reduce-scatter (count = elements
// per rank; in holds P*count), 2 allgather (count = elements per rank; out holds
// P*count), 3 two-shot allreduce (count = vector length).
// in / out: one pointer per local rank, 8-byte aligned.
int chb_ll_collective(chb_comm* c, int mode, int dtype, int op, const void* const* in, void* const* out,
                      long long count, float scale, int nctas, cudaStream_t stream) {
  if (!c || !in || !out || count < 0) return CHB_ERR_ARG;
  const long long nbytes = count * (long long)dtype_size(dtype);
  const bool two_shot = mode == 3;
  long long slice_bytes = 0;
  if (two_shot) {
    slice_bytes = ((nbytes + c->P - 1) / c->P + 7) / 8 * 8;
    if (nbytes > chb_ll2_max_bytes(c)) { c->last_error = "message exceeds the flagged-line inbox"; return CHB_ERR_COUNT; }
  } else if (nbytes > chb_ll_max_bytes(c)) {
    c->last_error = "message exceeds the flagged-line inbox";
    return CHB_ERR_COUNT;
  }
  LLFn fn = mode == LL_AR ? pick_ll<LL_AR>(dtype) : mode == LL_RS ? pick_ll<LL_RS>(dtype) : mode == LL_AG ? pick_ll<LL_AG>(dtype) : nullptr;
  LL2Fn fn2 = two_shot ? pick_ll2(dtype) : nullptr;
  if (!fn && !fn2) return CHB_ERR_ARG;
  LLIo io{};
  for (int l = 0; l < c->nlocal; ++l) {
    if ((((uintptr_t)in[l]) | ((uintptr_t)out[l])) & 7u) { c->last_error = "flagged-line path needs 8-byte aligned buffers"; return CHB_ERR_ARG; }
    io.in[c->rank + l] = (const char*)in[l];
    io.out[c->rank + l] = (char*)out[l];
  }
  if (nbytes == 0) return CHB_SUCCESS;
  const long long nlines = ((two_shot ? slice_bytes : nbytes) + 7) / 8;
  int budget = c->max_ctas / (c->nlocal > 0 ? c->nlocal : 1);
  if (budget < 1) budget = 1;
  if (nctas <= 0) {
    nctas = (int)((nlines + kLLThreads - 1) / kLLThreads);
    if (nctas > 32) nctas = 32;
  }
  if (nctas > 64) nctas = 64;
  if (nctas > budget) nctas = budget;
  if (nctas < 1) nctas = 1;
  dim3 grid((unsigned)nctas, (unsigned)c->nlocal, 1), block(kLLThreads, 1, 1);
  World w = c->world;
  long long lps = (long long)c->ll_lines_per_src;
  long long nb = nbytes;
  void* args1[] = {&w, &io, &nb, &op, &scale, &lps};
  void* args2[] = {&w, &io, &nb, &slice_bytes, &op, &scale, &lps};
  const void* f = two_shot ? (const void*)fn2 : (const void*)fn;
  void** args = two_shot ? args2 : args1;
  cudaError_t e;
  if (c->nlocal > 1) e = cudaLaunchCooperativeKernel(f, grid, block, args, 0, stream);
  else e = cudaLaunchKernel(f, grid, block, args, 0, stream);
  if (e != cudaSuccess) { c->last_error = std::string("ll launch failed: ") + cudaGetErrorString(e); return CHB_ERR_CUDA; }
  return CHB_SUCCESS;
}

}  // extern "C"

// Communicator life cycle, cudaIpc helpers, the stand-alone bounded barrier and
// the status word (chb.h, "communicators" section).
#include <cstdio>
#include <cstring>
#include <string>

#include "../api/chb.h"
#include "../boot/bootstrap.h"
#include "comm.h"
#include "vmm.h"

using namespace chb;

namespace {

__global__ void barrier_kernel(World w, unsigned long long timeout_ns_override) {
  // One CTA per local rank.  Thread q tells peer q "I arrived" and waits for
  // peer q's arrival; values are launch sequence numbers, never reset.
  const int rank = w.rank0 + (int)blockIdx.y;
  Ctrl* c = w.ctrl[rank];
  __shared__ unsigned long long s_seq;
  if (threadIdx.x == 0) s_seq = ld_volatile_u64(&c->bar_seq) + 1ull;
  __syncthreads();
  const unsigned long long seq = s_seq;
  const unsigned long long tmo = timeout_ns_override ? timeout_ns_override : w.timeout_ns;
  const int q = threadIdx.x;
  if (q < w.P && q != rank && !ld_volatile_u32(&c->abort)) {
    __threadfence_system();
    st_release_sys(&w.sig[q][kSigBarrierBase + rank], seq);
    wait_flag_ge(&w.sig[rank][kSigBarrierBase + q], seq, c, tmo, ST_TIMEOUT_BARRIER, rank, -1, q);
  }
  __syncthreads();
  if (threadIdx.x == 0) { c->bar_seq = seq; c->status[6] += 1ull; }
}

__global__ void reset_ctrl_kernel(Ctrl* c, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    c[i].bar_count = 0;
    c[i].exit_count = 0;
    c[i].abort = 0;
    for (int k = 0; k < 6; ++k) c[i].status[k] = 0;
  }
}

size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace

extern "C" {

const char* chb_comm_last_error(const chb_comm* c) { return c ? c->last_error.c_str() : "null communicator"; }

// Layout of one rank's heap for the given region sizes; returns total bytes.
// ll_bytes is the flagged-line payload capacity per rank pair.
size_t chb_heap_bytes(int P, size_t ll_payload_bytes, size_t scratch_bytes, size_t user_bytes) {
  size_t sig = round_up(sizeof(unsigned long long) * kSigSlots, 4096);
  size_t lines = (ll_payload_bytes + 7) / 8;
  size_t ll = round_up(2ull * (size_t)P * lines * 16, 4096);
  return sig + ll + round_up(scratch_bytes, 4096) + round_up(user_bytes, 4096);
}

// heap_ptrs: P peer-mapped base pointers of equally laid out heaps (for an
// emulated world: P slices of one local allocation).  mc_ptr: multicast alias
// of the local heap or NULL.  The heaps must be zero-filled before the first
// collective (chb_comm_create clears the local ones).
chb_comm* chb_comm_create(int rank, int P, int nlocal, void* const* heap_ptrs, void* mc_ptr,
                          size_t ll_payload_bytes, size_t scratch_bytes, size_t user_bytes,
                          char* err, int errlen) {
  auto fail = [&](const std::string& m) -> chb_comm* {
    if (err && errlen > 0) std::snprintf(err, (size_t)errlen, "%s", m.c_str());
    return nullptr;
  };
  if (P < 1 || P > kMaxRanks) return fail("number of ranks must be between 1 and 16");
  if (!(nlocal == 1 || nlocal == P)) return fail("nlocal must be 1 or P");
  if (rank < 0 || rank + nlocal > P) return fail("rank out of range");
  chb_comm* c = new chb_comm;
  c->P = P;
  c->rank = rank;
  c->nlocal = nlocal;
  if (cudaGetDevice(&c->device) != cudaSuccess) { delete c; return fail("no CUDA device"); }
  cudaDeviceProp prop;
  cudaGetDeviceProperties(&prop, c->device);
  c->sm_count = prop.multiProcessorCount;
  c->max_ctas = prop.multiProcessorCount;  // every kernel here fits one 512-thread CTA per SM
  c->sig_bytes = round_up(sizeof(unsigned long long) * kSigSlots, 4096);
  c->ll_lines_per_src = (ll_payload_bytes + 7) / 8;
  c->ll_bytes = round_up(2ull * (size_t)P * c->ll_lines_per_src * 16, 4096);
  c->scratch_bytes = round_up(scratch_bytes, 4096);
  c->user_bytes = round_up(user_bytes, 4096);
  c->heap_bytes = c->sig_bytes + c->ll_bytes + c->scratch_bytes + c->user_bytes;
  c->heap.resize(P);
  for (int p = 0; p < P; ++p) {
    c->heap[p] = (char*)heap_ptrs[p];
    if (!c->heap[p]) { delete c; return fail("null heap pointer"); }
  }
  c->mc_heap = (char*)mc_ptr;
  if (cudaMalloc(&c->ctrl, sizeof(Ctrl) * (size_t)nlocal) != cudaSuccess) { delete c; return fail("cudaMalloc(ctrl) failed"); }
  cudaMemset(c->ctrl, 0, sizeof(Ctrl) * (size_t)nlocal);
  // An emulated world owns all heaps and clears their pads and inboxes here.
  // With one rank per process the heaps arrive zero-filled and peers may
  // already be signalling, so they must not be cleared again.
  if (nlocal > 1 || P == 1)
    for (int l = 0; l < nlocal; ++l) cudaMemset(c->heap[rank + l], 0, c->sig_bytes + c->ll_bytes);
  if (cudaDeviceSynchronize() != cudaSuccess) { cudaFree(c->ctrl); delete c; return fail("CUDA error while clearing the heap"); }
  World& w = c->world;
  std::memset(&w, 0, sizeof(w));
  w.P = P;
  w.rank0 = rank;
  w.nlocal = nlocal;
  w.timeout_ns = c->timeout_ns;
  for (int p = 0; p < P; ++p) {
    w.sig[p] = (unsigned long long*)c->sig_ptr(p);
    w.ll[p] = c->ll_ptr(p);
    w.work[p] = c->scratch_ptr(p);
  }
  for (int l = 0; l < nlocal; ++l) w.ctrl[rank + l] = c->ctrl + l;
  return c;
}

void chb_collective_cache_clear(chb_comm* c);

void chb_comm_destroy(chb_comm* c) {
  if (!c) return;
  chb_collective_cache_clear(c);
  for (auto& kv : c->blobs) cudaFree(kv.second);
  for (auto& kv : c->ll_blobs) cudaFree(kv.second.first);
  if (c->ctrl) cudaFree(c->ctrl);
  if (c->trace) cudaFree(c->trace);
  for (void* q : c->ipc_opened) cudaIpcCloseMemHandle(q);
  if (c->owned_heap) cudaFree(c->owned_heap);
  if (c->vmm) chb_vmm_destroy(c->vmm);      // collective: every rank destroys its communicator
  delete c;
}

int chb_comm_set_timeout_us(chb_comm* c, unsigned long long us) {
  if (!c) return CHB_ERR_ARG;
  c->timeout_ns = us * 1000ull;
  c->world.timeout_ns = c->timeout_ns;
  return CHB_SUCCESS;
}

// info: P, rank, nlocal, sig_bytes, ll_bytes, scratch_bytes, user_bytes, heap_bytes, ll payload capacity, sm_count, has multicast
int chb_comm_info(const chb_comm* c, int64_t* info, int n) {
  if (!c || !info) return CHB_ERR_ARG;
  int64_t v[11] = {c->P, c->rank, c->nlocal, (int64_t)c->sig_bytes, (int64_t)c->ll_bytes, (int64_t)c->scratch_bytes,
                   (int64_t)c->user_bytes, (int64_t)c->heap_bytes, (int64_t)c->ll_lines_per_src * 8, c->sm_count,
                   c->mc_heap ? 1 : 0};
  for (int i = 0; i < n && i < 11; ++i) info[i] = v[i];
  return CHB_SUCCESS;
}

void* chb_comm_user_ptr(const chb_comm* c, int local_index) {
  if (!c || local_index < 0 || local_index >= c->nlocal) return nullptr;
  return c->user_ptr(c->rank + local_index);
}
void* chb_comm_scratch_ptr(const chb_comm* c, int local_index) {
  if (!c || local_index < 0 || local_index >= c->nlocal) return nullptr;
  return c->scratch_ptr(c->rank + local_index);
}

// Bounded barrier over all ranks on `stream`.  timeout_us == 0 uses the
// communicator's default.  Completion status is read with chb_comm_status.
int chb_barrier(chb_comm* c, unsigned long long timeout_us, cudaStream_t stream) {
  if (!c) return CHB_ERR_ARG;
  dim3 grid(1, (unsigned)c->nlocal, 1), block(32, 1, 1);
  World w = c->world;
  unsigned long long tmo = timeout_us * 1000ull;
  void* args[] = {&w, &tmo};
  cudaError_t e;
  if (c->nlocal > 1) e = cudaLaunchCooperativeKernel((const void*)barrier_kernel, grid, block, args, 0, stream);
  else e = cudaLaunchKernel((const void*)barrier_kernel, grid, block, args, 0, stream);
  if (e != cudaSuccess) { c->last_error = std::string("barrier launch failed: ") + cudaGetErrorString(e); return CHB_ERR_CUDA; }
  return CHB_SUCCESS;
}

// Synchronises `stream` and reads the control block of local rank `local_index`:
// status[0] code (0 ok; see StatusCode), [1] rank, [2] round, [3] peer,
// [4] expected, [5] seen, [6] launches completed, [7] epoch.
// Returns CHB_SUCCESS, CHB_ERR_TIMEOUT when a bounded wait expired, or CHB_ERR_CUDA.
int chb_comm_status(chb_comm* c, int local_index, unsigned long long* status8, cudaStream_t stream) {
  if (!c || local_index < 0 || local_index >= c->nlocal) return CHB_ERR_ARG;
  cudaError_t e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) { c->last_error = std::string("stream error: ") + cudaGetErrorString(e); return CHB_ERR_CUDA; }
  Ctrl h;
  e = cudaMemcpy(&h, c->ctrl + local_index, sizeof(Ctrl), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) { c->last_error = std::string("status copy failed: ") + cudaGetErrorString(e); return CHB_ERR_CUDA; }
  if (status8) {
    for (int i = 0; i < 7; ++i) status8[i] = h.status[i];
    status8[7] = h.epoch;
  }
  return (h.abort || h.status[0]) ? CHB_ERR_TIMEOUT : CHB_SUCCESS;
}

// Clears the sticky abort flag and the status word of the local ranks.  After
// an expired wait the ranks' counters may disagree; callers re-create the
// communicator (collectively) before they rely on it again.
int chb_comm_clear_error(chb_comm* c, cudaStream_t stream) {
  if (!c) return CHB_ERR_ARG;
  reset_ctrl_kernel<<<1, 32, 0, stream>>>(c->ctrl, c->nlocal);
  return cudaGetLastError() == cudaSuccess ? CHB_SUCCESS : CHB_ERR_CUDA;
}

// Per-round tracing of program launches: for every local rank the interpreter
// stamps %globaltimer when round t may start (its waits are satisfied) and when
// the round is complete on that rank.  The counterpart of the reference's
// optional per-phase MPI_Wtime prints under DEBUG_MODE
// (testing/custom_implementations/work_dir/all_reduce/all_reduce_radix_batch.cpp:228-232,480-489).
// rounds == 0 switches tracing off.
int chb_comm_trace_enable(chb_comm* c, int rounds) {
  if (!c || rounds < 0) return CHB_ERR_ARG;
  cudaDeviceSynchronize();
  if (c->trace) { cudaFree(c->trace); c->trace = nullptr; }
  c->trace_rounds = rounds;
  for (int p = 0; p < kMaxRanks; ++p) c->world.trace[p] = nullptr;
  c->world.trace_rounds = rounds;
  if (rounds == 0) return CHB_SUCCESS;
  const size_t per = (size_t)rounds * 2;
  if (cudaMalloc(&c->trace, per * 8 * (size_t)c->nlocal) != cudaSuccess) return CHB_ERR_NO_MEM;
  cudaMemset(c->trace, 0, per * 8 * (size_t)c->nlocal);
  for (int l = 0; l < c->nlocal; ++l) c->world.trace[c->rank + l] = c->trace + per * l;
  return cudaDeviceSynchronize() == cudaSuccess ? CHB_SUCCESS : CHB_ERR_CUDA;
}
// Copies 2 * rounds stamps (start, end per round, ns) of a local rank after synchronising the stream.
int chb_comm_trace_read(chb_comm* c, int local_index, unsigned long long* out, int rounds, cudaStream_t stream) {
  if (!c || !out || !c->trace || local_index < 0 || local_index >= c->nlocal || rounds > c->trace_rounds) return CHB_ERR_ARG;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return CHB_ERR_CUDA;
  const size_t per = (size_t)c->trace_rounds * 2;
  return cudaMemcpy(out, c->trace + per * local_index, (size_t)rounds * 16, cudaMemcpyDeviceToHost) == cudaSuccess
             ? CHB_SUCCESS : CHB_ERR_CUDA;
}

// ---- cudaIpc helpers: one allocation per rank, exported as a 64-byte handle
int chb_ipc_alloc(size_t bytes, void** ptr, void* handle64) {
  if (!ptr || !handle64) return CHB_ERR_ARG;
  if (cudaMalloc(ptr, bytes) != cudaSuccess) return CHB_ERR_NO_MEM;
  cudaMemset(*ptr, 0, bytes);
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, *ptr) != cudaSuccess) { cudaFree(*ptr); *ptr = nullptr; return CHB_ERR_CUDA; }
  static_assert(sizeof(h) == 64, "cudaIpcMemHandle_t is 64 bytes");
  std::memcpy(handle64, &h, 64);
  return cudaDeviceSynchronize() == cudaSuccess ? CHB_SUCCESS : CHB_ERR_CUDA;
}
int chb_ipc_open(const void* handle64, void** ptr) {
  if (!ptr || !handle64) return CHB_ERR_ARG;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, 64);
  return cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess ? CHB_SUCCESS : CHB_ERR_CUDA;
}
int chb_ipc_close(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? CHB_SUCCESS : CHB_ERR_CUDA; }
int chb_dev_alloc(size_t bytes, void** ptr) {
  if (!ptr) return CHB_ERR_ARG;
  if (cudaMalloc(ptr, bytes) != cudaSuccess) return CHB_ERR_NO_MEM;
  cudaMemset(*ptr, 0, bytes);
  return cudaDeviceSynchronize() == cudaSuccess ? CHB_SUCCESS : CHB_ERR_CUDA;
}
int chb_dev_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? CHB_SUCCESS : CHB_ERR_CUDA; }

// ---- native constructors: no Python, no torch.distributed ------------------------------------------
// All P ranks on the current GPU (one process): one allocation split P ways.
chb_comm* chb_comm_create_emulated(int P, size_t ll_payload_bytes, size_t scratch_bytes, size_t user_bytes,
                                   char* err, int errlen) {
  auto fail = [&](const char* m) -> chb_comm* {
    if (err && errlen > 0) std::snprintf(err, (size_t)errlen, "%s", m);
    return nullptr;
  };
  if (P < 1 || P > kMaxRanks) return fail("number of ranks must be between 1 and 16");
  const size_t hb = chb_heap_bytes(P, ll_payload_bytes, scratch_bytes, user_bytes);
  void* base = nullptr;
  if (cudaMalloc(&base, hb * (size_t)P) != cudaSuccess) return fail("cudaMalloc(heap) failed");
  cudaMemset(base, 0, hb * (size_t)P);
  void* ptrs[kMaxRanks];
  for (int p = 0; p < P; ++p) ptrs[p] = (char*)base + hb * (size_t)p;
  chb_comm* c = chb_comm_create(0, P, P, ptrs, nullptr, ll_payload_bytes, scratch_bytes, user_bytes, err, errlen);
  if (!c) { cudaFree(base); return nullptr; }
  c->owned_heap = base;
  return c;
}

// One rank per process and per GPU of one box: every rank allocates its heap on the current device,
// the cudaIpc handles travel through the bootstrap's allgather, peers' heaps are mapped.
chb_comm* chb_comm_create_ipc(chb_bootstrap* boot, size_t ll_payload_bytes, size_t scratch_bytes, size_t user_bytes,
                              char* err, int errlen) {
  auto fail = [&](const std::string& m) -> chb_comm* {
    if (err && errlen > 0) std::snprintf(err, (size_t)errlen, "%s", m.c_str());
    if (boot) chb_bootstrap_abort(boot);
    return nullptr;
  };
  if (!boot) return fail("null bootstrap");
  const int P = chb_bootstrap_world(boot), rank = chb_bootstrap_rank(boot);
  if (P < 1 || P > kMaxRanks) return fail("number of ranks must be between 1 and 16");
  const size_t hb = chb_heap_bytes(P, ll_payload_bytes, scratch_bytes, user_bytes);
  void* mine = nullptr;
  char handle[64];
  if (chb_ipc_alloc(hb, &mine, handle) != CHB_SUCCESS) return fail("cudaIpc allocation of the heap failed");
  std::vector<char> all(64 * (size_t)P);
  if (chb_bootstrap_allgather(boot, handle, all.data(), 64) != CHB_SUCCESS) { cudaFree(mine); return fail("handle exchange failed"); }
  void* ptrs[kMaxRanks];
  std::vector<void*> opened;
  for (int p = 0; p < P; ++p) {
    if (p == rank) { ptrs[p] = mine; continue; }
    void* q = nullptr;
    if (chb_ipc_open(all.data() + 64 * (size_t)p, &q) != CHB_SUCCESS) {
      for (void* o : opened) cudaIpcCloseMemHandle(o);
      cudaFree(mine);
      return fail("cannot map the heap of rank " + std::to_string(p) + " (no peer access?)");
    }
    opened.push_back(q);
    ptrs[p] = q;
  }
  chb_comm* c = chb_comm_create(rank, P, 1, ptrs, nullptr, ll_payload_bytes, scratch_bytes, user_bytes, err, errlen);
  if (!c) {
    for (void* o : opened) cudaIpcCloseMemHandle(o);
    cudaFree(mine);
    chb_bootstrap_abort(boot);
    return nullptr;
  }
  c->owned_heap = mine;
  c->ipc_opened = opened;
  // nobody signals into a heap before every rank has set up
  if (chb_bootstrap_barrier(boot) != CHB_SUCCESS) { chb_comm_destroy(c); return fail("ranks did not all finish the set-up"); }
  return c;
}

// One rank per process and per GPU of one box, heaps from the virtual-memory allocator (symm/vmm.cc): peers are
// mapped through shareable allocation handles, and when every device supports it the heaps also get an
// NVLink multicast alias, so that the multimem kernels run without Python.  want_multicast: 0 / 1.
// Returns NULL with CHB_ERR_UNSUPPORTED in *code (if given) when the platform lacks shareable handles: callers
// fall back to chb_comm_create_ipc.
chb_comm* chb_comm_create_vmm(chb_bootstrap* boot, size_t ll_payload_bytes, size_t scratch_bytes, size_t user_bytes,
                              int want_multicast, int* code, char* err, int errlen) {
  auto fail = [&](int rc, const std::string& m) -> chb_comm* {
    if (code) *code = rc;
    if (err && errlen > 0) std::snprintf(err, (size_t)errlen, "%s", m.c_str());
    return nullptr;
  };
  if (code) *code = CHB_SUCCESS;
  if (!boot) return fail(CHB_ERR_ARG, "null bootstrap");
  const int P = chb_bootstrap_world(boot), rank = chb_bootstrap_rank(boot);
  if (P < 1 || P > kMaxRanks) return fail(CHB_ERR_ARG, "number of ranks must be between 1 and 16");
  cudaFree(nullptr);                                   // the primary context exists before the driver API is used
  const size_t hb = chb_heap_bytes(P, ll_payload_bytes, scratch_bytes, user_bytes);
  chb_vmm_heap* heap = nullptr;
  char why[256] = {0};
  int rc = chb_vmm_create(boot, hb, want_multicast, &heap, why, sizeof why);
  if (rc) return fail(rc, why);
  // pads and inboxes start at zero, and nobody signals into a heap before every rank has cleared its own
  if (cudaMemset(chb_vmm_ptr(heap, rank), 0, chb_vmm_bytes(heap)) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) {
    chb_bootstrap_abort(boot);
    return fail(CHB_ERR_CUDA, "clearing the heap failed");
  }
  if (chb_bootstrap_barrier(boot)) return fail(CHB_ERR_OTHER, "ranks did not all finish the set-up");
  void* ptrs[kMaxRanks];
  for (int p = 0; p < P; ++p) ptrs[p] = chb_vmm_ptr(heap, p);
  chb_comm* c = chb_comm_create(rank, P, 1, ptrs, chb_vmm_multicast_ptr(heap), ll_payload_bytes, scratch_bytes, user_bytes, err, errlen);
  if (!c) {
    chb_bootstrap_abort(boot);
    if (code) *code = CHB_ERR_OTHER;
    return nullptr;
  }
  c->vmm = heap;
  if (chb_bootstrap_barrier(boot) != CHB_SUCCESS) { chb_comm_destroy(c); return fail(CHB_ERR_OTHER, "ranks did not all finish the set-up"); }
  return c;
}

}  // extern "C"

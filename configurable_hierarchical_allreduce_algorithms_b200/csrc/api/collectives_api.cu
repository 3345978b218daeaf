// One-call collectives on a communicator (program cache + dispatch to the
// interpreter, flagged-line or multimem kernels) and the reference-compatible
// entry points declared in chb_compat.h.
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "../sched/algos.h"
#include "../symm/comm.h"
#include "chb.h"
#include "chb_compat.h"
#include "program_handle.h"

extern "C" {
void chb_program_release(chb_comm* c, const chb_program* p);
int chb_run_program(chb_comm* c, const chb_program* p, int dtype, int op, const void* const* in,
                    void* const* out, float scale, int nctas, cudaStream_t stream);
int chb_run_program_ll(chb_comm* c, const chb_program* p, int dtype, int op, const void* const* in,
                       void* const* out, float scale, int nctas, cudaStream_t stream);
long long chb_program_ll_lines(const chb_program* p, int esz);
int chb_ll_collective(chb_comm* c, int mode, int dtype, int op, const void* const* in, void* const* out,
                      long long count, float scale, int nctas, cudaStream_t stream);
long long chb_ll_max_bytes(const chb_comm* c);
int chb_ag_bulk(chb_comm* c, const void* const* in, void* const* out, long long nbytes, int nctas, cudaStream_t stream);
int chb_nvls_collective(chb_comm* c, int mode, int dtype, const void* in, void* out, long long count,
                        float scale, int nctas, cudaStream_t stream);
}

namespace chb { Builder gen_a2av_tuna(int P, const std::vector<int64_t>& counts, int r, int b); }

namespace {

using Key = std::tuple<int, std::string, int, int, int, int64_t, int>;
struct Cache {
  std::map<Key, chb_program*> progs;
  std::map<std::vector<int64_t>, chb_program*> a2av;   // key: r, b, then the P x P count matrix
  ~Cache() {
    for (auto& kv : progs) delete kv.second;
    for (auto& kv : a2av) delete kv.second;
  }
};
// one cache per communicator, owned here so that comm.h stays free of it; the map itself is shared by
// all host threads (calls on ONE communicator are not thread safe, calls on different ones are)
std::mutex g_cache_mu;
std::map<chb_comm*, Cache>& caches() {
  static std::map<chb_comm*, Cache> m;
  return m;
}
Cache& cache_of(chb_comm* c) {
  std::lock_guard<std::mutex> g(g_cache_mu);
  return caches()[c];     // references into a std::map stay valid when other keys are added
}
// A caller that sweeps message sizes compiles one program per size; beyond this many the cache starts over.
constexpr size_t kMaxCachedPrograms = 1024;

const char* coll_name(int coll) {
  switch (coll) {
    case CHB_ALLREDUCE: return "allreduce";
    case CHB_REDUCE_SCATTER: return "reduce_scatter";
    case CHB_ALLGATHER: return "allgather";
    case CHB_ALLTOALL: return "alltoall";
    case CHB_GATHER: return "gather";
    case CHB_PHASE: return "phase";
  }
  return "";
}

bool all_symmetric(const chb_comm* c, const void* const* ptrs) {
  for (int l = 0; l < c->nlocal; ++l) {
    const char* p = (const char*)ptrs[l];
    const char* u = c->user_ptr(c->rank + l);
    if (p < u || p >= u + c->user_bytes) return false;
  }
  return true;
}

int get_program(chb_comm* c, int coll, const char* algo, int k, int b, int aux, int64_t count, int flags,
                chb_program** out) {
  Key key(coll, algo, k, b, aux, count, flags);
  Cache& ca = cache_of(c);
  auto it = ca.progs.find(key);
  if (it != ca.progs.end()) { *out = it->second; return CHB_SUCCESS; }
  if (ca.progs.size() >= kMaxCachedPrograms) {
    // launches that still read the device copies must finish first
    if (cudaDeviceSynchronize() != cudaSuccess) { c->last_error = "device synchronisation failed"; return CHB_ERR_CUDA; }
    for (auto& kv : ca.progs) { chb_program_release(c, kv.second); delete kv.second; }
    ca.progs.clear();
  }
  try {
    chb::AlgoSpec s;
    s.coll = coll_name(coll);
    s.algo = algo;
    s.P = c->P;
    s.k = k;
    s.b = b;
    s.count = count;
    s.aux = aux;
    chb::Builder B = chb::build_algorithm(s);
    chb::LowerOpts o;
    o.in_symmetric = (flags & 1) != 0;
    o.out_symmetric = (flags & 2) != 0;
    o.in_place = (flags & 4) != 0;
    auto* p = new chb_program;
    p->prog = B.lower(o);
    ca.progs[key] = p;
    *out = p;
    return CHB_SUCCESS;
  } catch (const std::exception& e) {
    c->last_error = e.what();
    return c->last_error.find("count") != std::string::npos ? CHB_ERR_COUNT : CHB_ERR_ARG;
  }
}

}  // namespace

extern "C" {

void chb_collective_cache_clear(chb_comm* c) {
  std::lock_guard<std::mutex> g(g_cache_mu);
  caches().erase(c);
}

// Generic entry: in / out hold one pointer per local rank.  algo is a step
// program name (chb_list_algorithms), "ll" or "nvls".  count as in chb.h.
int chb_collective(chb_comm* c, int coll, const char* algo, int k, int b, int aux, int dtype, int op,
                   const void* const* in, void* const* out, int64_t count, float scale, int nctas,
                   cudaStream_t stream) {
  if (!c || !algo || !in || !out) return CHB_ERR_ARG;
  if (!std::strcmp(algo, "bulk")) {
    if (coll != CHB_ALLGATHER) return CHB_ERR_UNSUPPORTED;
    return chb_ag_bulk(c, in, out, count * (long long)chb_dtype_size(dtype), nctas, stream);
  }
  if (!std::strcmp(algo, "ll2")) {
    if (coll != CHB_ALLREDUCE) return CHB_ERR_UNSUPPORTED;
    return chb_ll_collective(c, 3, dtype, op, in, out, count, scale, nctas, stream);
  }
  if (!std::strcmp(algo, "ll")) {
    int mode = coll == CHB_ALLREDUCE ? 0 : coll == CHB_REDUCE_SCATTER ? 1 : coll == CHB_ALLGATHER ? 2 : -1;
    if (mode < 0) return CHB_ERR_UNSUPPORTED;
    return chb_ll_collective(c, mode, dtype, op, in, out, count, scale, nctas, stream);
  }
  if (!std::strncmp(algo, "nvls", 4)) {
    if (op != CHB_SUM) return CHB_ERR_OP;
    int mode = coll == CHB_ALLREDUCE ? (!std::strcmp(algo, "nvls1") ? 3 : 0) : coll == CHB_REDUCE_SCATTER ? 1
             : coll == CHB_ALLGATHER ? 2 : -1;
    if (mode < 0) return CHB_ERR_UNSUPPORTED;
    return chb_nvls_collective(c, mode, dtype, in[0], out[0], count, scale, nctas, stream);
  }
  // "<name>:ll" / "<name>:pull" pin the way a step program is executed; without a suffix, collectives in
  // which every rank depends on every rank run with flagged lines up to CHB_LL_PROGRAM_MAX bytes
  // (default 4 MiB of payload, if the messages fit the inbox: measured break-even with the pull interpreter on
  // 8 GPUs) and with the pull interpreter above that.
  std::string name(algo);
  int mode = 0;                                   // 0 auto, 1 flagged lines, 2 pull
  {
    const size_t colon = name.find(':');
    if (colon != std::string::npos) {
      const std::string m = name.substr(colon + 1);
      name.resize(colon);
      if (m == "ll") mode = 1;
      else if (m == "pull") mode = 2;
      else { c->last_error = "unknown execution mode '" + m + "' (ll | pull)"; return CHB_ERR_ARG; }
    }
  }
  algo = name.c_str();
  // (the launch-parity argument of the inbox needs every rank's result to depend on every rank's input: a gather
  // or a stand-alone phase does not qualify)
  const bool ll_kind = coll == CHB_ALLREDUCE || coll == CHB_REDUCE_SCATTER || coll == CHB_ALLGATHER || coll == CHB_ALLTOALL;
  if (mode == 1 && !ll_kind) { c->last_error = "flagged-line execution covers allreduce, reduce-scatter, allgather and all-to-all"; return CHB_ERR_UNSUPPORTED; }
  // In place means in == out, except for the allgather, whose in-place form is
  // "my block already sits at its slot of the output" (in == out + rank * block):
  // that needs no staging, the self copy is a no-op.
  bool in_place = false, ag_alias = false;
  for (int l = 0; l < c->nlocal; ++l) {
    if (coll == CHB_ALLGATHER) {
      const char* slot = (const char*)out[l] + (int64_t)(c->rank + l) * count * chb_dtype_size(dtype);
      if ((const char*)in[l] == slot) { ag_alias = true; continue; }
    }
    in_place |= (in[l] == out[l]);
  }
  int flags = 0;
  if (in_place) flags = 4;
  else flags = (all_symmetric(c, in) ? 1 : 0) | (all_symmetric(c, (const void* const*)out) ? 2 : 0);
  // aliased allgather inputs sit at a different heap offset on every rank, so
  // peers cannot address them as "my input pointer, your heap": stage them
  if (ag_alias) flags &= ~1;
  chb_program* p = nullptr;
  if (mode != 2 && ll_kind && c->P > 1) {
    static const long long ll_max = [] {
      const char* e = std::getenv("CHB_LL_PROGRAM_MAX");
      return e ? std::atoll(e) : (4ll << 20);
    }();
    const int esz = chb_dtype_size(dtype);
    const long long payload = (long long)count * esz * (coll == CHB_ALLREDUCE ? 1 : c->P);
    if (mode == 1 || payload <= ll_max) {
      // owners push, nobody reads a peer's buffers: lowered without staging whatever the buffers are
      const int ll_flags = 3 | (in_place ? 4 : 0);
      int rc = get_program(c, coll, algo, k, b, aux, count, ll_flags, &p);
      if (rc) return rc;
      const long long need = chb_program_ll_lines(p, esz);
      if (need <= (long long)c->P * (long long)c->ll_lines_per_src)
        return chb_run_program_ll(c, p, dtype, op, in, out, scale, nctas, stream);
      if (mode == 1) { c->last_error = "messages of this program exceed the flagged-line inbox"; return CHB_ERR_COUNT; }
    }
  }
  int rc = get_program(c, coll, algo, k, b, aux, count, flags, &p);
  if (rc) return rc;
  return chb_run_program(c, p, dtype, op, in, out, scale, nctas, stream);
}

// ---------------------------------------------------------------- reference-compatible calls
static cudaStream_t g_compat_stream = nullptr;
void chb_set_stream(cudaStream_t s) { g_compat_stream = s; }

static int one(CHB_Comm comm, int coll, const char* algo, const void* sendbuf, void* recvbuf, int64_t count,
               CHB_Datatype dt, CHB_Op op, int k, int b, int aux) {
  if (!comm) return CHB_ERR_ARG;
  if (comm->nlocal != 1) { comm->last_error = "reference-compatible calls need one rank per process"; return CHB_ERR_ARG; }
  const void* in = sendbuf;
  if (sendbuf == CHB_IN_PLACE) {
    // MPI's meaning: reductions take their input from recvbuf; an allgather finds each rank's block already at
    // its slot of recvbuf.  A gather or a stand-alone phase has no in-place form.
    if (coll == CHB_ALLREDUCE || coll == CHB_REDUCE_SCATTER) in = recvbuf;
    else if (coll == CHB_ALLGATHER) in = (const char*)recvbuf + (int64_t)comm->rank * count * chb_dtype_size(dt);
    else { comm->last_error = "CHB_IN_PLACE is defined for allreduce, reduce-scatter and allgather only"; return CHB_ERR_ARG; }
  }
  return chb_collective(comm, coll, algo, k, b, aux, dt, op, &in, &recvbuf, count, 1.0f, 0, g_compat_stream);
}

int allgather_radix_batch(char* sendbuf, int sendcount, CHB_Datatype datatype, char* recvbuf, CHB_Comm comm, int k, int b) {
  return one(comm, CHB_ALLGATHER, "radix_batch", sendbuf, recvbuf, sendcount, datatype, CHB_SUM, k, b, 0);
}
int reduce_scatter_radix_batch(const void* sendbuf, void* recvbuf, int64_t recvcount, CHB_Datatype datatype, CHB_Op op,
                               CHB_Comm comm, int k, int b) {
  if (sendbuf == CHB_IN_PLACE) {
    // in place: recvbuf holds the P*recvcount inputs and receives the result at its start
    return one(comm, CHB_REDUCE_SCATTER, "radix_batch", CHB_IN_PLACE, recvbuf, recvcount, datatype, op, k, b, 0);
  }
  return one(comm, CHB_REDUCE_SCATTER, "radix_batch", sendbuf, recvbuf, recvcount, datatype, op, k, b, 0);
}
int all_reduce_radix_batch(char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm, int k, int b) {
  return one(comm, CHB_ALLREDUCE, "radix_batch", sendbuf, recvbuf, count, datatype, op, k, b, 0);
}
int all_reduce_semi_radix_batch(char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm, int k, int b) {
  return one(comm, CHB_ALLREDUCE, "semi_radix_batch", sendbuf, recvbuf, count, datatype, op, k, b, 0);
}
int reduce_scatter_radix_block(char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm, int r, int b) {
  return one(comm, CHB_REDUCE_SCATTER, "radix_block", sendbuf, recvbuf, count, datatype, op, r, b, 0);
}
int allgather_k_brucks(char* sendbuf, int sendcount, CHB_Datatype datatype, char* recvbuf, CHB_Comm comm, int k) {
  return one(comm, CHB_ALLGATHER, "k_brucks", sendbuf, recvbuf, sendcount, datatype, CHB_SUM, k, 1, 0);
}
int gather_k_nomial(char* sendbuf, int sendcount, CHB_Datatype datatype, char* recvbuf, CHB_Comm comm, int k, int root) {
  return one(comm, CHB_GATHER, "k_nomial", sendbuf, recvbuf, sendcount, datatype, CHB_SUM, k, 1, root);
}

// stand-alone phases (reference: all_gather_0_3_beta.cpp:36,141,377; intra_reduce_scatter_radix.cpp:208;
// inter_linear_reduce.cpp:11; intra_scatter_radix_batch.cpp:11)
int intra_gather_k_nomial(char* sendbuf, int count, CHB_Datatype datatype, char* recvbuf, CHB_Comm comm, int k, int b) {
  return one(comm, CHB_PHASE, "intra_gather_k_nomial", sendbuf, recvbuf, count, datatype, CHB_SUM, k, b, 0);
}
int intra_allgather_k_brucks(char* sendbuf, int count, CHB_Datatype datatype, char* recvbuf, CHB_Comm comm, int k, int b) {
  return one(comm, CHB_PHASE, "intra_allgather_k_brucks", sendbuf, recvbuf, count, datatype, CHB_SUM, k, b, 0);
}
int inter_allgather_linear(char* sendbuf, int sendcount, CHB_Datatype datatype, char* recvbuf, CHB_Comm comm, int b) {
  return one(comm, CHB_PHASE, "inter_allgather_linear", sendbuf, recvbuf, sendcount, datatype, CHB_SUM, 2, b, 0);
}
int intra_reduce_scatter_radix_batch(const void* sendbuf, void* recvbuf, int64_t recvcount, CHB_Datatype datatype, CHB_Op op,
                                     CHB_Comm comm, int k, int b) {
  return one(comm, CHB_PHASE, "intra_reduce_scatter_radix_batch", sendbuf, recvbuf, recvcount, datatype, op, k, b, 0);
}
int inter_reduce_linear(const void* sendbuf, void* recvbuf, int64_t recvcount, CHB_Datatype datatype, CHB_Op op,
                        CHB_Comm comm, int b) {
  return one(comm, CHB_PHASE, "inter_reduce_linear", sendbuf, recvbuf, recvcount, datatype, op, 2, b, 0);
}
int intra_scatter_radix_batch(char* sendbuf, int recvcount, CHB_Datatype datatype, char* recvbuf, CHB_Comm comm, int k, int b) {
  return one(comm, CHB_PHASE, "intra_scatter_radix_batch", sendbuf, recvbuf, recvcount, datatype, CHB_SUM, k, b, 0);
}

#define CHB_AR0(NAME, ALGO)                                                                                   \
  int NAME(const char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm) {  \
    return one(comm, CHB_ALLREDUCE, ALGO, sendbuf, recvbuf, count, datatype, op, 2, 1, 0);                    \
  }
CHB_AR0(MPICH_Allreduce_recursive_doubling, "recursive_doubling")
CHB_AR0(MPICH_Allreduce_ring, "ring")
CHB_AR0(MPICH_Allreduce_reduce_scatter_allgather, "reduce_scatter_allgather")
#undef CHB_AR0
int MPICH_Allreduce_recursive_multiplying(const char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op,
                                          CHB_Comm comm, int k) {
  return one(comm, CHB_ALLREDUCE, "recursive_multiplying", sendbuf, recvbuf, count, datatype, op, k, 1, 0);
}
int MPICH_Allreduce_k_reduce_scatter_allgather(const char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op,
                                               CHB_Comm comm, int k, int single_phase_recv) {
  // single_phase_recv selects how many receive phases are pre-posted in the
  // two-sided original; a pull schedule has no receives to post, so it is accepted and ignored
  (void)single_phase_recv;
  return one(comm, CHB_ALLREDUCE, "k_reduce_scatter_allgather", sendbuf, recvbuf, count, datatype, op, k, 1, 0);
}
int MPICH_Allreduce_recursive_exchange(const char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op,
                                       CHB_Comm comm, int k, int single_phase_recv) {
  (void)single_phase_recv;
  return one(comm, CHB_ALLREDUCE, "recursive_exchange", sendbuf, recvbuf, count, datatype, op, k, 1, 0);
}
int MPICH_Allreduce_inter_reduce_exchange_bcast(const char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op,
                                                CHB_Comm comm, int ranks_per_node) {
  return one(comm, CHB_ALLREDUCE, "inter_reduce_exchange_bcast", sendbuf, recvbuf, count, datatype, op, 2, 1, ranks_per_node);
}
#define CHB_RS0(NAME, ALGO)                                                                                        \
  int NAME(const void* sendbuf, void* recvbuf, int64_t recvcount, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm) { \
    return one(comm, CHB_REDUCE_SCATTER, ALGO, sendbuf, recvbuf, recvcount, datatype, op, 2, 1, 0);                  \
  }
CHB_RS0(MPICH_reduce_scatter_rec_halving, "recursive_halving")
CHB_RS0(MPICH_reduce_scatter_rec_doubling, "recursive_doubling")
CHB_RS0(MPICH_reduce_scatter_pairwise, "pairwise")
#undef CHB_RS0
int MPICH_reduce_scatter_radix(const void* sendbuf, void* recvbuf, int64_t recvcount, CHB_Datatype datatype, CHB_Op op,
                               CHB_Comm comm, int k) {
  return one(comm, CHB_REDUCE_SCATTER, "radix", sendbuf, recvbuf, recvcount, datatype, op, k, 1, 0);
}

int MPICH_reduce_scatter_k_nomial(const char* sendbuf, char* recvbuf, int count, CHB_Datatype datatype, CHB_Op op, CHB_Comm comm, int k) {
  return one(comm, CHB_REDUCE_SCATTER, "k_nomial", sendbuf, recvbuf, count, datatype, op, k, 1, 0);
}

// Reference: testing/custom_implementations/work_dir/reduce_scatter/debug/tuna.cpp:9-270.
int tuna2_algorithm(int r, int b, char* sendbuf, int* sendcounts, int* sdispls, CHB_Datatype sendtype,
                    char* recvbuf, int* recvcounts, int* rdispls, CHB_Datatype recvtype, CHB_Comm comm) {
  if (!comm || !sendbuf || !recvbuf || !sendcounts || !recvcounts || !sdispls || !rdispls) return CHB_ERR_ARG;
  chb_comm* c = comm;
  if (c->nlocal != 1) { c->last_error = "reference-compatible calls need one rank per process"; return CHB_ERR_ARG; }
  if (sendtype != recvtype) { c->last_error = "tuna2_algorithm: send and receive types must match"; return CHB_ERR_UNSUPPORTED; }
  const int P = c->P;
  int64_t s = 0, q = 0;
  for (int i = 0; i < P; ++i) {
    if (sendcounts[i] < 0 || recvcounts[i] < 0) return CHB_ERR_COUNT;
    if (sdispls[i] != s || rdispls[i] != q) { c->last_error = "tuna2_algorithm: blocks must be packed"; return CHB_ERR_UNSUPPORTED; }
    s += sendcounts[i];
    q += recvcounts[i];
  }
  // every rank needs the whole count matrix to know where its blocks sit in the peers' buffers
  std::vector<int> all((size_t)P * P);
  {
    int *d_in = nullptr, *d_out = nullptr;
    if (cudaMalloc(&d_in, sizeof(int) * P) != cudaSuccess || cudaMalloc(&d_out, sizeof(int) * P * P) != cudaSuccess) {
      cudaFree(d_in);
      return CHB_ERR_NO_MEM;
    }
    cudaMemcpyAsync(d_in, sendcounts, sizeof(int) * P, cudaMemcpyHostToDevice, g_compat_stream);
    const void* in1 = d_in;
    void* out1 = d_out;
    int rc = chb_collective(c, CHB_ALLGATHER, "radix_batch", 2, 1, 0, CHB_I32, CHB_SUM, &in1, &out1, P, 1.0f, 0, g_compat_stream);
    if (rc == CHB_SUCCESS) {
      cudaMemcpyAsync(all.data(), d_out, sizeof(int) * P * P, cudaMemcpyDeviceToHost, g_compat_stream);
      if (cudaStreamSynchronize(g_compat_stream) != cudaSuccess) rc = CHB_ERR_CUDA;
    }
    cudaFree(d_in);
    cudaFree(d_out);
    if (rc) return rc;
  }
  for (int i = 0; i < P; ++i)
    if (all[(size_t)i * P + c->rank] != recvcounts[i]) { c->last_error = "tuna2_algorithm: recvcounts disagree with the senders' counts"; return CHB_ERR_COUNT; }
  std::vector<int64_t> key{r, b};
  key.insert(key.end(), all.begin(), all.end());
  Cache& ca = cache_of(c);
  chb_program* p = nullptr;
  auto it = ca.a2av.find(key);
  if (it != ca.a2av.end()) {
    p = it->second;
  } else {
    try {
      std::vector<int64_t> m(all.begin(), all.end());
      chb::Builder B = chb::gen_a2av_tuna(P, m, r < 2 ? 2 : r, (b <= 0 || b > P) ? P : b);
      p = new chb_program;
      p->prog = B.lower(chb::LowerOpts{});
      ca.a2av[key] = p;
    } catch (const std::exception& e) {
      c->last_error = e.what();
      return CHB_ERR_ARG;
    }
  }
  const void* in = sendbuf;
  void* out = recvbuf;
  return chb_run_program(c, p, sendtype, CHB_SUM, &in, &out, 1.0f, 0, g_compat_stream);
}

}  // extern "C"

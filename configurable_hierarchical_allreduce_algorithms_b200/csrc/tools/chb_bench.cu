// Native benchmark driver and launcher: the reference's main.cpp files without MPI and
// without Python.  One process per GPU is forked by the launcher itself (the role of
// mpiexec), the ranks meet through the shared-memory bootstrap, build a communicator over
// cudaIpc heaps and sweep message sizes, algorithms and radices, checking every repetition
// on the device against the definition of the collective.
//
//   chb_bench <n_iter> [--overwrite] [b=<group>] [base=<elements>] [num_nodes=<n>] [radix_increment=<step>]
//             [coll=allreduce|reduce_scatter|allgather] [dtype=int32|fp32|fp64|bf16] [op=sum|max|min]
//             [algos=a,b,...] [reps=50] [out=<file.csv>] [ngpus=<N>] [emulate=<P>] [symmetric=1] [vendor=0]
//
// Same argv grammar, sweep and CSV columns as the reference's drivers
// (testing/custom_implementations/work_dir/all_reduce/main.cpp:111-199, .../all_gather/main.cpp:109-201,
// .../reduce_scatter/main.cpp:169-264): sizes double n_iter times from `base` elements per rank,
// k = 2 .. b-1 for the hierarchical algorithm, `reps` checked repetitions per configuration, one row
// per repetition: algorithm_name,k,b,nprocs,send_count,time,is_correct (+ dtype,op,bytes,algbw_GBs,
// busbw_GBs,ngpus), correctness AND-reduced and time MAX-reduced over ranks (reduce_scatter/main.cpp:79-83).
// The library baseline row (MPICH_allreduce / reduce_scatter_standard / allgather_standard there) is NCCL,
// loaded at run time if present.  emulate=P runs P ranks on one GPU in this process instead.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <dirent.h>
#include <dlfcn.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include <algorithm>

#include "../api/chb.h"
#include "../api/chb_compat.h"
#include "../boot/bootstrap.h"

namespace {

// payload bytes one source may have in flight in a rank's flagged-line inbox (per launch parity): a 4 MiB
// allreduce still fits as a push program on 2 to 8 GPUs; the inbox takes 16 * P * this many bytes of each heap
constexpr size_t kInboxBytes = 4u << 20;

struct Opts {
  int n_iter = 0;
  bool overwrite = false;
  int b = 0, num_nodes = 1, radix_increment = 1, reps = 50, ngpus = 0, emulate = 0, symmetric = 0, vendor = 1;
  long long base = 1;
  std::string coll = "allreduce", dtype = "int32", op = "sum", algos, out;
};

[[noreturn]] void usage(const char* why) {
  std::fprintf(stderr, "%s\nusage: chb_bench <n_iter> [--overwrite] [b=] [base=] [num_nodes=] [radix_increment=] "
                       "[coll=] [dtype=] [op=] [algos=] [reps=] [out=] [ngpus=] [emulate=] [symmetric=] [vendor=]\n", why);
  std::exit(2);
}

Opts parse(int argc, char** argv) {
  Opts o;
  if (argc < 2 || !(argv[1][0] >= '0' && argv[1][0] <= '9')) usage("the first argument is the number of doublings");
  o.n_iter = std::atoi(argv[1]);
  for (int i = 2; i < argc; ++i) {
    std::string a = argv[i];
    if (a == "--overwrite") { o.overwrite = true; continue; }
    size_t eq = a.find('=');
    if (eq == std::string::npos) usage(("Unknown parameter: " + a).c_str());
    std::string k = a.substr(0, eq), v = a.substr(eq + 1);
    if (k == "b") o.b = std::atoi(v.c_str());
    else if (k == "base") o.base = std::atoll(v.c_str());
    else if (k == "num_nodes") o.num_nodes = std::atoi(v.c_str());
    else if (k == "radix_increment") o.radix_increment = std::max(1, std::atoi(v.c_str()));
    else if (k == "reps") o.reps = std::atoi(v.c_str());
    else if (k == "ngpus") o.ngpus = std::atoi(v.c_str());
    else if (k == "emulate") o.emulate = std::atoi(v.c_str());
    else if (k == "symmetric") o.symmetric = std::atoi(v.c_str());
    else if (k == "vendor") o.vendor = std::atoi(v.c_str());
    else if (k == "coll") o.coll = v;
    else if (k == "dtype") o.dtype = v;
    else if (k == "op") o.op = v;
    else if (k == "algos") o.algos = v;
    else if (k == "out") o.out = v;
    else usage(("Unknown parameter: " + a).c_str());
  }
  return o;
}

// ---- device side: deterministic inputs and the check ----------------------------------------------
__host__ __device__ inline int pattern(int rank, long long i, int mod) { return (int)(((long long)rank * 1009 + i * 31 + 7) % mod); }

template <typename T> __device__ inline T from_int(int v) { return (T)v; }
template <> __device__ inline __nv_bfloat16 from_int<__nv_bfloat16>(int v) { return __float2bfloat16((float)v); }
template <typename T> __device__ inline double to_double(T v) { return (double)v; }
template <> __device__ inline double to_double<__nv_bfloat16>(__nv_bfloat16 v) { return (double)__bfloat162float(v); }

template <typename T>
__global__ void fill_kernel(T* x, long long n, int rank, int mod) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    x[i] = from_int<T>(pattern(rank, i, mod));
}

// coll: 0 allreduce, 1 reduce_scatter, 2 allgather; n = elements per block; op: 0 sum, 1 max, 2 min
template <typename T>
__global__ void check_kernel(const T* y, long long n_out, int coll, int rank, int P, long long n, int mod, int op,
                             unsigned long long* bad) {
  unsigned long long mine = 0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n_out; i += (long long)gridDim.x * blockDim.x) {
    long long e;
    if (coll == 2) {
      e = pattern((int)(i / n), i % n, mod);
    } else {
      const long long idx = coll == 1 ? (long long)rank * n + i : i;
      e = pattern(0, idx, mod);
      for (int r = 1; r < P; ++r) {
        const long long v = pattern(r, idx, mod);
        e = op == 0 ? e + v : (op == 1 ? (v > e ? v : e) : (v < e ? v : e));
      }
    }
    if (to_double<T>(y[i]) != (double)e) ++mine;
  }
  if (mine) atomicAdd(bad, mine);
}

struct DT { const char* name; int id; int size; int mod; };
const DT kDtypes[] = {{"int32", CHB_I32, 4, 97}, {"fp32", CHB_F32, 4, 97}, {"fp64", CHB_F64, 8, 97}, {"bf16", CHB_BF16, 2, 13}};

void fill(void* x, long long n, int rank, const DT& d) {
  const int blocks = (int)std::min<long long>(1184, (n + 255) / 256 > 0 ? (n + 255) / 256 : 1);
  switch (d.id) {
    case CHB_I32: fill_kernel<int><<<blocks, 256>>>((int*)x, n, rank, d.mod); break;
    case CHB_F32: fill_kernel<float><<<blocks, 256>>>((float*)x, n, rank, d.mod); break;
    case CHB_F64: fill_kernel<double><<<blocks, 256>>>((double*)x, n, rank, d.mod); break;
    default: fill_kernel<__nv_bfloat16><<<blocks, 256>>>((__nv_bfloat16*)x, n, rank, d.mod); break;
  }
}
void check(const void* y, long long n_out, int coll, int rank, int P, long long n, const DT& d, int op, unsigned long long* bad) {
  const int blocks = (int)std::min<long long>(1184, (n_out + 255) / 256 > 0 ? (n_out + 255) / 256 : 1);
  switch (d.id) {
    case CHB_I32: check_kernel<int><<<blocks, 256>>>((const int*)y, n_out, coll, rank, P, n, d.mod, op, bad); break;
    case CHB_F32: check_kernel<float><<<blocks, 256>>>((const float*)y, n_out, coll, rank, P, n, d.mod, op, bad); break;
    case CHB_F64: check_kernel<double><<<blocks, 256>>>((const double*)y, n_out, coll, rank, P, n, d.mod, op, bad); break;
    default: check_kernel<__nv_bfloat16><<<blocks, 256>>>((const __nv_bfloat16*)y, n_out, coll, rank, P, n, d.mod, op, bad); break;
  }
}

// ---- NCCL, loaded at run time (the library baseline row) -------------------------------------------
struct Nccl {
  typedef struct { char internal[128]; } UniqueId;
  void* lib = nullptr;
  void* comm = nullptr;
  int (*GetUniqueId)(UniqueId*) = nullptr;
  int (*CommInitRank)(void**, int, UniqueId, int) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*ReduceScatter)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
  int (*CommDestroy)(void*) = nullptr;
  bool load() {
    lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!lib) return false;
    GetUniqueId = (decltype(GetUniqueId))dlsym(lib, "ncclGetUniqueId");
    CommInitRank = (decltype(CommInitRank))dlsym(lib, "ncclCommInitRank");
    AllReduce = (decltype(AllReduce))dlsym(lib, "ncclAllReduce");
    ReduceScatter = (decltype(ReduceScatter))dlsym(lib, "ncclReduceScatter");
    AllGather = (decltype(AllGather))dlsym(lib, "ncclAllGather");
    CommDestroy = (decltype(CommDestroy))dlsym(lib, "ncclCommDestroy");
    return GetUniqueId && CommInitRank && AllReduce && ReduceScatter && AllGather && CommDestroy;
  }
  static int dtype(int chb) { return chb == CHB_I32 ? 2 : chb == CHB_F32 ? 7 : chb == CHB_F64 ? 8 : 9; }
  static int redop(int op) { return op == 0 ? 0 : op == 1 ? 2 : 3; }
};

std::vector<std::string> split(const std::string& s) {
  std::vector<std::string> v;
  size_t a = 0;
  while (a <= s.size()) {
    size_t b = s.find(',', a);
    if (b == std::string::npos) b = s.size();
    if (b > a) v.push_back(s.substr(a, b - a));
    a = b + 1;
  }
  return v;
}

bool takes_radix(const std::string& a) {
  static const char* k[] = {"radix_batch", "k_reduce_scatter_allgather", "recursive_multiplying", "recursive_exchange", "radix",
                            "k_brucks", "semi_radix_batch", "custom", "radix_block"};
  for (const char* x : k) if (a == x) return true;
  return false;
}
bool takes_group(const std::string& a) { return a == "radix_batch" || a == "semi_radix_batch" || a == "custom" || a == "radix_block"; }

#define CUDA_OK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::fprintf(stderr, "rank %d: %s: %s\n", rank0, #x, cudaGetErrorString(e_)); return 1; } } while (0)

// One process: `nlocal` ranks starting at rank0 (nlocal == P when emulated, else 1).
int run(const Opts& o, chb_comm* comm, chb_bootstrap* boot, int P, int rank0, int nlocal, int ngpus) {
  const int coll = o.coll == "allreduce" ? CHB_ALLREDUCE : o.coll == "reduce_scatter" ? CHB_REDUCE_SCATTER : CHB_ALLGATHER;
  const int collc = coll == CHB_ALLREDUCE ? 0 : coll == CHB_REDUCE_SCATTER ? 1 : 2;
  const int op = o.op == "sum" ? 0 : o.op == "max" ? 1 : 2;
  const int chb_op = op == 0 ? CHB_SUM : op == 1 ? CHB_MAX : CHB_MIN;
  const DT* d = nullptr;
  for (const DT& x : kDtypes) if (o.dtype == x.name) d = &x;
  if (!d) { std::fprintf(stderr, "unknown dtype %s\n", o.dtype.c_str()); return 2; }
  const int b = o.b ? o.b : P;
  const long long max_n = o.base << std::max(0, o.n_iter - 1);
  const long long max_in = coll == CHB_ALLGATHER ? max_n : max_n * P, max_out = coll == CHB_REDUCE_SCATTER ? max_n : max_n * P;

  std::vector<void*> in(nlocal), out(nlocal);
  unsigned long long* bad = nullptr;
  CUDA_OK(cudaMalloc(&bad, 8));
  for (int l = 0; l < nlocal; ++l) {
    if (o.symmetric) {
      char* u = (char*)chb_comm_user_ptr(comm, l);
      in[l] = u;
      out[l] = u + ((size_t)max_in * d->size + 255) / 256 * 256;
    } else {
      CUDA_OK(cudaMalloc(&in[l], (size_t)max_in * d->size));
      CUDA_OK(cudaMalloc(&out[l], (size_t)max_out * d->size));
    }
  }
  Nccl nccl;
  bool have_nccl = false;
  if (o.vendor && boot && P > 1 && nccl.load()) {
    Nccl::UniqueId id;
    std::memset(&id, 0, sizeof id);
    if (rank0 == 0) nccl.GetUniqueId(&id);
    std::vector<char> all(sizeof id * (size_t)P);
    if (chb_bootstrap_allgather(boot, &id, all.data(), sizeof id)) return 1;
    std::memcpy(&id, all.data(), sizeof id);
    have_nccl = nccl.CommInitRank(&nccl.comm, P, id, rank0) == 0;
  }
  FILE* csv = nullptr;
  if (rank0 == 0) {
    char def[128];
    std::snprintf(def, sizeof def, "results%d_%d_%d.csv", P, o.num_nodes, b);
    const std::string path = o.out.empty() ? def : o.out;
    const bool fresh = o.overwrite || access(path.c_str(), F_OK) != 0;
    csv = std::fopen(path.c_str(), fresh ? "w" : "a");
    if (!csv) { std::fprintf(stderr, "cannot open %s\n", path.c_str()); return 1; }
    if (fresh) std::fprintf(csv, "algorithm_name,k,b,nprocs,send_count,time,is_correct,dtype,op,bytes,algbw_GBs,busbw_GBs,ngpus,p50_us,roofline_frac\n");
  }
  std::vector<std::string> algos = split(o.algos);
  if (algos.empty()) {
    algos = {"radix_batch"};
    const char* base_ar[] = {"recursive_doubling", "ring", "reduce_scatter_allgather", "k_reduce_scatter_allgather", "recursive_multiplying", "recursive_exchange"};
    const char* base_rs[] = {"recursive_halving", "recursive_doubling", "pairwise", "radix"};
    const char* base_ag[] = {"k_brucks", "ring"};
    if (coll == CHB_ALLREDUCE) for (const char* a : base_ar) algos.push_back(a);
    if (coll == CHB_REDUCE_SCATTER) for (const char* a : base_rs) algos.push_back(a);
    if (coll == CHB_ALLGATHER) for (const char* a : base_ag) algos.push_back(a);
  }
  cudaEvent_t e0, e1;
  CUDA_OK(cudaEventCreate(&e0));
  CUDA_OK(cudaEventCreate(&e1));
  int failures = 0;

  // `reps` timed, checked repetitions of one configuration; 0, or 1 when this rank has to give up
  auto run_one = [&](const std::string& name, const char* algo, int k, int bb, long long n) -> int {
    const long long count = coll == CHB_ALLREDUCE ? n * P : n;       // chb_collective's count convention
    const long long n_out = coll == CHB_REDUCE_SCATTER ? n : n * P;
    const int kk = k ? k : 2, gb = bb ? bb : 1;
    std::vector<std::pair<double, std::string>> rows;    // one per repetition, written once their median is known
    auto flush_rows = [&]() {
      if (!csv || rows.empty()) return;
      std::vector<double> ts;
      for (auto& r : rows) ts.push_back(r.first);
      std::sort(ts.begin(), ts.end());
      const double p50 = ts[ts.size() / 2];
      // share of the NVLink roofline: bytes one GPU moves per direction over the measured 770 GB/s peer rate
      const double total = (double)n * P * d->size;
      const double factor = coll == CHB_ALLREDUCE ? 2.0 * (P - 1) / P : (double)(P - 1) / P;
      const double frac = (ngpus > 1 && P > 1) ? (total * factor / 770e9) / p50 : 0.0;
      for (auto& r : rows) std::fprintf(csv, "%s,%.3f,%.4f\n", r.second.c_str(), p50 * 1e6, frac);
      std::fflush(csv);
    };
    for (int rep = 0; rep < o.reps; ++rep) {
      for (int l = 0; l < nlocal; ++l) cudaMemsetAsync(out[l], 0xFF, (size_t)n_out * d->size);
      cudaDeviceSynchronize();
      if (boot && chb_bootstrap_barrier(boot)) return 1;
      cudaEventRecord(e0);
      int rc = 0;
      if (algo) {
        rc = chb_collective(comm, coll, algo, kk, gb, 0, d->id, chb_op, in.data(), out.data(), count, 1.0f, 0, nullptr);
      } else {
        const size_t cnt = coll == CHB_ALLREDUCE ? (size_t)n * P : (size_t)n;
        if (coll == CHB_ALLREDUCE) rc = nccl.AllReduce(in[0], out[0], cnt, Nccl::dtype(d->id), Nccl::redop(op), nccl.comm, nullptr);
        else if (coll == CHB_REDUCE_SCATTER) rc = nccl.ReduceScatter(in[0], out[0], cnt, Nccl::dtype(d->id), Nccl::redop(op), nccl.comm, nullptr);
        else rc = nccl.AllGather(in[0], out[0], cnt, Nccl::dtype(d->id), nccl.comm, nullptr);
      }
      if (rc) {
        // a capability this communicator lacks (no multicast alias, inbox too small ...): the same on every rank
        if (rank0 == 0) std::fprintf(stderr, "skipped %s k=%d b=%d count=%lld: %s\n", name.c_str(), k, bb, n,
                                     algo ? chb_comm_last_error(comm) : "library call failed");
        return 0;
      }
      cudaEventRecord(e1);
      if (cudaEventSynchronize(e1) != cudaSuccess) { std::fprintf(stderr, "rank %d: CUDA error after %s\n", rank0, name.c_str()); return 1; }
      float ms = 0;
      cudaEventElapsedTime(&ms, e0, e1);
      cudaMemset(bad, 0, 8);
      for (int l = 0; l < nlocal; ++l) check(out[l], n_out, collc, rank0 + l, P, n, *d, op, bad);
      unsigned long long hbad = 0;
      cudaMemcpy(&hbad, bad, 8, cudaMemcpyDeviceToHost);
      unsigned long long st[8];
      int ok = hbad == 0 && chb_comm_status(comm, 0, st, nullptr) == CHB_SUCCESS;
      double t = ms * 1e-3;
      if (boot) {
        struct { double t; int ok; } mine = {t, ok}, all[64];
        if (chb_bootstrap_allgather(boot, &mine, all, sizeof mine)) return 1;
        for (int r = 0; r < P; ++r) { t = std::max(t, all[r].t); ok = ok && all[r].ok; }
      }
      if (!ok) ++failures;
      if (csv) {
        const double total = (double)n * P * d->size;
        const double factor = coll == CHB_ALLREDUCE ? 2.0 * (P - 1) / P : (double)(P - 1) / P;
        char line[512];
        std::snprintf(line, sizeof line, "%s,%d,%d,%d,%lld,%.9f,%d,%s,%s,%.0f,%.4f,%.4f,%d", name.c_str(), k, bb, P, n, t, ok,
                      d->name, o.op.c_str(), total, total / t / 1e9, total / t / 1e9 * factor, ngpus);
        rows.emplace_back(t, line);
      }
    }
    flush_rows();
    return 0;
  };

  for (int it = 0; it < o.n_iter; ++it) {
    const long long n = o.base << it;
    const long long n_in = coll == CHB_ALLGATHER ? n : n * P;
    for (int l = 0; l < nlocal; ++l) fill(in[l], n_in, rank0 + l, *d);
    CUDA_OK(cudaDeviceSynchronize());
    for (const std::string& a : algos) {
      std::string name = o.coll + "_" + a;
      if (a == "radix_batch") name = coll == CHB_ALLREDUCE ? "all_reduce_radix_batch" : coll == CHB_REDUCE_SCATTER ? "reduce_scatter_radix_batch" : "allgather_radix_batch";
      if (takes_radix(a)) {
        const int hi = a == "radix_batch" ? std::max(3, b) : std::max(3, P);
        for (int k = 2; k < hi; k += o.radix_increment)
          if (run_one(name, a.c_str(), k, takes_group(a) ? b : 0, n)) return 1;
      } else if (run_one(name, a.c_str(), 0, 0, n)) {
        return 1;
      }
    }
    if (have_nccl) {
      const char* vname = coll == CHB_ALLREDUCE ? "MPICH_allreduce" : coll == CHB_REDUCE_SCATTER ? "reduce_scatter_standard" : "allgather_standard";
      if (run_one(vname, nullptr, 0, 0, n)) return 1;
    }
  }
  if (csv) std::fclose(csv);
  if (have_nccl) nccl.CommDestroy(nccl.comm);
  cudaDeviceSynchronize();
  if (rank0 == 0) std::printf("chb_bench: %s on %d ranks done, %d incorrect repetitions\n", o.coll.c_str(), P, failures);
  return failures ? 3 : 0;
}

int count_gpus() {
  int n = 0;
  if (DIR* d = opendir("/dev")) {
    while (dirent* e = readdir(d)) {
      const char* s = e->d_name;
      if (!std::strncmp(s, "nvidia", 6) && s[6] >= '0' && s[6] <= '9') ++n;
    }
    closedir(d);
  }
  return n > 0 ? n : 1;
}

}  // namespace

int main(int argc, char** argv) {
  Opts o = parse(argc, argv);
  if (o.coll != "allreduce" && o.coll != "reduce_scatter" && o.coll != "allgather") usage("coll must be allreduce, reduce_scatter or allgather");
  if (o.op != "sum" && o.op != "max" && o.op != "min") usage("op must be sum, max or min");
  const int esz = o.dtype == "fp64" ? 8 : o.dtype == "bf16" ? 2 : 4;
  char err[256] = "";
  if (o.emulate > 0) {
    const int P = o.emulate;
    if (o.b && P % o.b) usage("b must divide the number of ranks");
    const size_t total = (size_t)(o.base << std::max(0, o.n_iter - 1)) * P * esz;
    chb_comm* c = chb_comm_create_emulated(P, 1 << 20, 4 * total + (32u << 20), o.symmetric ? 2 * total + 4096 : 4096, err, sizeof err);
    if (!c) { std::fprintf(stderr, "communicator: %s\n", err); return 1; }
    int rc = run(o, c, nullptr, P, 0, P, 1);
    chb_comm_destroy(c);
    return rc;
  }
  // launcher: fork before anything touches CUDA
  const int P = o.ngpus > 0 ? o.ngpus : count_gpus();
  if (o.b && P % o.b) usage("b must divide the number of ranks");
  char name[64];
  std::snprintf(name, sizeof name, "/chb_bench_%d", (int)getpid());
  std::vector<pid_t> kids(P);
  for (int r = 0; r < P; ++r) {
    kids[r] = fork();
    if (kids[r] < 0) { std::perror("fork"); return 1; }
    if (kids[r] == 0) {
      if (cudaSetDevice(r) != cudaSuccess) { std::fprintf(stderr, "rank %d: no such GPU\n", r); _exit(1); }
      chb_bootstrap* boot = nullptr;
      if (chb_bootstrap_create(name, r, P, 60000, &boot)) { std::fprintf(stderr, "rank %d: rendezvous failed\n", r); _exit(1); }
      const size_t total = (size_t)(o.base << std::max(0, o.n_iter - 1)) * P * esz;
      // heaps from the virtual-memory allocator (with the NVLink multicast alias where the devices have one, so that
      // algos=nvls works here too); cudaIpc heaps where shareable allocation handles are missing, or with CHB_VMM=0
      chb_comm* c = nullptr;
      const char* vmm_env = std::getenv("CHB_VMM");
      if (!vmm_env || std::strcmp(vmm_env, "0") != 0) {
        const char* nvls_env = std::getenv("CHB_NVLS");
        int code = 0;
        c = chb_comm_create_vmm(boot, kInboxBytes, 4 * total + (32u << 20), o.symmetric ? 2 * total + 4096 : 4096,
                                (nvls_env && !std::strcmp(nvls_env, "0")) ? 0 : 1, &code, err, sizeof err);
        if (!c && code != CHB_ERR_UNSUPPORTED) { std::fprintf(stderr, "rank %d: communicator: %s\n", r, err); chb_bootstrap_destroy(boot); _exit(1); }
      }
      if (!c) c = chb_comm_create_ipc(boot, kInboxBytes, 4 * total + (32u << 20), o.symmetric ? 2 * total + 4096 : 4096, err, sizeof err);
      if (!c) { std::fprintf(stderr, "rank %d: communicator: %s\n", r, err); chb_bootstrap_destroy(boot); _exit(1); }
      int rc = run(o, c, boot, P, r, 1, P);
      if (rc == 1) chb_bootstrap_abort(boot);      // the others stop waiting for this rank
      chb_comm_destroy(c);
      chb_bootstrap_destroy(boot);
      _exit(rc);
    }
  }
  int worst = 0;
  for (int r = 0; r < P; ++r) {
    int st = 0;
    waitpid(kids[r], &st, 0);
    const int code = WIFEXITED(st) ? WEXITSTATUS(st) : 1;
    if (code > worst) worst = code;
  }
  return worst;
}

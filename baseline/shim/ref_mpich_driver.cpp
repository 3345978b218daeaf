// Runs the reference's MPICH-style baselines (compiled unmodified against the thread-per-rank shim) on an
// int32 pattern and prints every rank's output.
//   ref_mpich_driver <name> P k n seed [inplace]
// name: ar_recursive_doubling | ar_ring | ar_reduce_scatter_allgather | ar_recursive_multiplying |
//       ar_k_reduce_scatter_allgather | ar_recursive_exchange | rs_rec_halving | rs_pairwise | rs_radix
// n: elements per rank block (allreduce vectors hold P*n elements).
#include <cstdio>
#include <cstdlib>
#include <string>
#include <thread>
#include <vector>

#include "mpi.h"

int MPICH_Allreduce_recursive_doubling(const char*, char*, int, MPI_Datatype, MPI_Op, MPI_Comm);
int MPICH_Allreduce_ring(const char*, char*, int, MPI_Datatype, MPI_Op, MPI_Comm);
int MPICH_Allreduce_reduce_scatter_allgather(const char*, char*, int, MPI_Datatype, MPI_Op, MPI_Comm);
int MPICH_Allreduce_recursive_multiplying(const char*, char*, int, MPI_Datatype, MPI_Op, MPI_Comm, int);
int MPICH_Allreduce_k_reduce_scatter_allgather(const char*, char*, int, MPI_Datatype, MPI_Op, MPI_Comm, int, int);
int MPICH_Allreduce_recursive_exchange(const char*, char*, int, MPI_Datatype, MPI_Op, MPI_Comm, int, int);
int MPICH_reduce_scatter_rec_halving(const char*, char*, int, MPI_Datatype, MPI_Op, MPI_Comm);
int MPICH_reduce_scatter_pairwise(const void*, void*, MPI_Aint, MPI_Datatype, MPI_Op, MPI_Comm);
int MPICH_reduce_scatter_radix(const void*, void*, MPI_Aint, MPI_Datatype, MPI_Op, MPI_Comm, int);

static int pattern(int seed, int r, long i) { return (int)((seed * 31L + r * 1009L + i * 7L) % 97); }

int main(int argc, char** argv) {
  if (argc < 6) { std::fprintf(stderr, "usage: ref_mpich_driver <name> P k n seed [inplace]\n"); return 2; }
  const std::string name = argv[1];
  const int P = std::atoi(argv[2]), k = std::atoi(argv[3]);
  const long n = std::atol(argv[4]);
  const int seed = std::atoi(argv[5]);
  const bool inplace = argc > 6 && std::string(argv[6]) == "inplace";
  const bool ar = name.rfind("ar_", 0) == 0;
  const long nin = n * P, nout = ar ? n * P : n;
  shim_init(P);
  std::vector<std::vector<int>> out(P);
  std::vector<int> rcs(P, 0);
  std::vector<std::thread> th;
  for (int r = 0; r < P; ++r) th.emplace_back([&, r] {
    shim_set_rank(r);
    std::vector<int> s(nin);
    for (long i = 0; i < nin; ++i) s[i] = pattern(seed, r, i);
    out[r].assign(inplace ? nin : nout, -17);
    if (inplace) out[r] = s;
    const char* sb = inplace ? (const char*)MPI_IN_PLACE : (const char*)s.data();
    char* rb = (char*)out[r].data();
    const int cnt = (int)(ar ? nin : n);
    if (name == "ar_recursive_doubling") rcs[r] = MPICH_Allreduce_recursive_doubling(sb, rb, cnt, MPI_INT, MPI_SUM, 0);
    else if (name == "ar_ring") rcs[r] = MPICH_Allreduce_ring(sb, rb, cnt, MPI_INT, MPI_SUM, 0);
    else if (name == "ar_reduce_scatter_allgather") rcs[r] = MPICH_Allreduce_reduce_scatter_allgather(sb, rb, cnt, MPI_INT, MPI_SUM, 0);
    else if (name == "ar_recursive_multiplying") rcs[r] = MPICH_Allreduce_recursive_multiplying(sb, rb, cnt, MPI_INT, MPI_SUM, 0, k);
    else if (name == "ar_k_reduce_scatter_allgather") rcs[r] = MPICH_Allreduce_k_reduce_scatter_allgather(sb, rb, cnt, MPI_INT, MPI_SUM, 0, k, 1);
    else if (name == "ar_recursive_exchange") rcs[r] = MPICH_Allreduce_recursive_exchange(sb, rb, cnt, MPI_INT, MPI_SUM, 0, k, 1);
    else if (name == "rs_rec_halving") rcs[r] = MPICH_reduce_scatter_rec_halving(sb, rb, cnt, MPI_INT, MPI_SUM, 0);
    else if (name == "rs_pairwise") rcs[r] = MPICH_reduce_scatter_pairwise(sb, rb, n, MPI_INT, MPI_SUM, 0);
    else if (name == "rs_radix") rcs[r] = MPICH_reduce_scatter_radix(sb, rb, n, MPI_INT, MPI_SUM, 0, k);
    else rcs[r] = -1;
    out[r].resize(nout);      // in place, the reduce-scatter result is at the start of the buffer
  });
  for (auto& t : th) t.join();
  int bad = shim_failed();
  for (int v : rcs) bad |= (v != 0);
  std::printf("%d", bad);
  for (int r = 0; r < P; ++r) for (int v : out[r]) std::printf(" %d", v);
  std::printf("\n");
  return bad;
}

// Runs the reference's MPICH-style baselines (compiled unmodified against the thread-per-rank shim) on an
// int32 pattern and prints every rank's output.
//   ref_mpich_driver <name> P k n seed [inplace]
// name: ar_recursive_doubling | ar_ring | ar_reduce_scatter_allgather | ar_recursive_multiplying |
//       ar_k_reduce_scatter_allgather | ar_recursive_exchange | ar_smp (2 ranks per node) | rs_rec_halving |
//       rs_rec_doubling | rs_pairwise | rs_radix |
//       the earlier variants rs_radix_block (k = radix, extra argument batch) | rs_k_nomial | ag_k_brucks |
//       gather_k_nomial (root 0) | a2av_tuna2 (k = radix, extra argument batch; rank s sends n + (s + 2 d) % 3
//       elements to rank d)
// n: elements per rank block (allreduce vectors hold P*n elements).  The sixth argument is "inplace" or the batch.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
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
int MPICH_reduce_scatter_rec_doubling(const void*, void*, MPI_Aint, MPI_Datatype, MPI_Op, MPI_Comm);
int MPICH_Allreduce_inter_reduce_exchange_bcast(const char*, char*, int, MPI_Datatype, MPI_Op, MPI_Comm);   // built with RANKS_PER_NODE=2
int reduce_scatter_radix_block(char*, char*, int, MPI_Datatype, MPI_Op, MPI_Comm, int, int);
int MPICH_reduce_scatter_k_nomial(const char*, char*, int, MPI_Datatype, MPI_Op, MPI_Comm, int);
int allgather_k_brucks(char*, int, MPI_Datatype, char*, MPI_Comm, int);
int gather_k_nomial(char*, int, MPI_Datatype, char*, MPI_Comm, int, int);
int tuna2_algorithm(int, int, char*, int*, int*, MPI_Datatype, char*, int*, int*, MPI_Datatype, MPI_Comm);

static int pattern(int seed, int r, long i) { return (int)((seed * 31L + r * 1009L + i * 7L) % 97); }

int main(int argc, char** argv) {
  if (argc < 6) { std::fprintf(stderr, "usage: ref_mpich_driver <name> P k n seed [inplace]\n"); return 2; }
  const std::string name = argv[1];
  const int P = std::atoi(argv[2]), k = std::atoi(argv[3]);
  const long n = std::atol(argv[4]);
  const int seed = std::atoi(argv[5]);
  const bool inplace = argc > 6 && std::string(argv[6]) == "inplace";
  const bool as_float = argc > 6 && std::string(argv[6]) == "float";   // float32 values that do not add exactly; bit patterns are printed
  const int batch = (argc > 6 && !inplace && !as_float) ? std::atoi(argv[6]) : 1;
  const bool ar = name.rfind("ar_", 0) == 0;
  long nin = n * P, nout = ar ? n * P : n;
  if (name == "ag_k_brucks" || name == "gather_k_nomial") { nin = n; nout = n * P; }
  auto a2a = [&](int s_, int d_) { return (int)n + (s_ + 2 * d_) % 3; };
  if (name == "a2av_tuna2") {      // sizes differ per rank: take the largest, the print below clips per rank
    nin = nout = 0;
    for (int q = 0; q < P; ++q) { long a = 0, b2 = 0; for (int d = 0; d < P; ++d) { a += a2a(q, d); b2 += a2a(d, q); } nin = std::max(nin, a); nout = std::max(nout, b2); }
  }
  shim_init(P);
  std::vector<std::vector<int>> out(P);
  std::vector<int> rcs(P, 0);
  std::vector<std::thread> th;
  for (int r = 0; r < P; ++r) th.emplace_back([&, r] {
    shim_set_rank(r);
    std::vector<int> s(nin);
    for (long i = 0; i < nin; ++i) s[i] = pattern(seed, r, i);
    if (as_float)
      for (long i = 0; i < nin; ++i) { float f = (float)pattern(seed, r, i) / 7.0f + (float)r * 0.37f; std::memcpy(&s[i], &f, 4); }
    const MPI_Datatype T = as_float ? MPI_FLOAT : MPI_INT;
    out[r].assign(inplace ? nin : nout, -17);
    if (inplace) out[r] = s;
    const char* sb = inplace ? (const char*)MPI_IN_PLACE : (const char*)s.data();
    char* rb = (char*)out[r].data();
    const int cnt = (int)(ar ? nin : n);
    if (name == "ar_recursive_doubling") rcs[r] = MPICH_Allreduce_recursive_doubling(sb, rb, cnt, T, MPI_SUM, 0);
    else if (name == "ar_ring") rcs[r] = MPICH_Allreduce_ring(sb, rb, cnt, T, MPI_SUM, 0);
    else if (name == "ar_reduce_scatter_allgather") rcs[r] = MPICH_Allreduce_reduce_scatter_allgather(sb, rb, cnt, T, MPI_SUM, 0);
    else if (name == "ar_recursive_multiplying") rcs[r] = MPICH_Allreduce_recursive_multiplying(sb, rb, cnt, T, MPI_SUM, 0, k);
    else if (name == "ar_k_reduce_scatter_allgather") rcs[r] = MPICH_Allreduce_k_reduce_scatter_allgather(sb, rb, cnt, T, MPI_SUM, 0, k, 1);
    else if (name == "ar_recursive_exchange") rcs[r] = MPICH_Allreduce_recursive_exchange(sb, rb, cnt, T, MPI_SUM, 0, k, 1);
    else if (name == "rs_rec_halving") rcs[r] = MPICH_reduce_scatter_rec_halving(sb, rb, cnt, T, MPI_SUM, 0);
    else if (name == "rs_pairwise") rcs[r] = MPICH_reduce_scatter_pairwise(sb, rb, n, T, MPI_SUM, 0);
    else if (name == "rs_radix") rcs[r] = MPICH_reduce_scatter_radix(sb, rb, n, T, MPI_SUM, 0, k);
    else if (name == "rs_rec_doubling") rcs[r] = MPICH_reduce_scatter_rec_doubling(sb, rb, n, T, MPI_SUM, 0);
    else if (name == "ar_smp") rcs[r] = MPICH_Allreduce_inter_reduce_exchange_bcast(sb, rb, cnt, T, MPI_SUM, 0);
    else if (name == "rs_radix_block") rcs[r] = reduce_scatter_radix_block((char*)s.data(), rb, (int)n, MPI_INT, MPI_SUM, 0, k, batch);
    else if (name == "rs_k_nomial") rcs[r] = MPICH_reduce_scatter_k_nomial(sb, rb, (int)n, MPI_INT, MPI_SUM, 0, k);
    else if (name == "ag_k_brucks") rcs[r] = allgather_k_brucks((char*)s.data(), (int)n, MPI_INT, rb, 0, k);
    else if (name == "gather_k_nomial") rcs[r] = gather_k_nomial((char*)s.data(), (int)n, MPI_INT, rb, 0, k, 0);
    else if (name == "a2av_tuna2") {
      std::vector<int> sc(P), sd(P), rc(P), rd(P);
      int a = 0, b2 = 0;
      for (int d = 0; d < P; ++d) { sc[d] = a2a(r, d); sd[d] = a; a += sc[d]; rc[d] = a2a(d, r); rd[d] = b2; b2 += rc[d]; }
      rcs[r] = tuna2_algorithm(k, batch, (char*)s.data(), sc.data(), sd.data(), MPI_INT, rb, rc.data(), rd.data(), MPI_INT, 0);
    }
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

// Runs the reference's stand-alone phase functions (compiled unmodified against the thread-per-rank
// shim) on an int32 pattern and prints every rank's output buffer, which starts filled with -17 so
// that entries a phase leaves alone can be told apart.
//   ref_phase_driver <phase> P k b c seed
// phase: intra_gather_k_nomial | inter_allgather_linear | intra_allgather_k_brucks |
//        intra_reduce_scatter_radix_batch | inter_reduce_linear | intra_scatter_radix_batch
// c is the count argument of the call; buffer lengths follow from it (T = ceil((P/b)/b) stages):
//   gather b*c out / c in; lane allgather b*c in, T*b*c out; Bruck T*c in, (P/b)*c out;
//   intra reduce-scatter P*c in, T*b*c out; lane reduce T*b*c in, b*c out; scatter b*c in, c out.
#include <cstdio>
#include <cstdlib>
#include <string>
#include <thread>
#include <vector>

#include "mpi.h"

int intra_gather_k_nomial(char*, int, MPI_Datatype, char*, MPI_Comm, int, int);
int intra_allgather_k_brucks(char*, int, MPI_Datatype, char*, MPI_Comm, int, int);
int inter_allgather_linear(char*, int, MPI_Datatype, char*, MPI_Comm, int);
int intra_reduce_scatter_radix_batch(const void*, void*, MPI_Aint, MPI_Datatype, MPI_Op, MPI_Comm, int, int);
int inter_reduce_linear(const void*, void*, MPI_Aint, MPI_Datatype, MPI_Op, MPI_Comm, int);
int intra_scatter_radix_batch(char*, int, MPI_Datatype, char*, MPI_Comm, int, int);

static int pattern(int seed, int r, long i) { return (int)((seed * 31L + r * 1009L + i * 7L) % 97); }

int main(int argc, char** argv) {
  if (argc < 7) { std::fprintf(stderr, "usage: ref_phase_driver <phase> P k b c seed\n"); return 2; }
  const std::string ph = argv[1];
  const int P = std::atoi(argv[2]), k = std::atoi(argv[3]), b = std::atoi(argv[4]);
  const long c = std::atol(argv[5]);
  const int seed = std::atoi(argv[6]);
  const int G = P / b, T = (G + b - 1) / b;
  long nin = 0, nout = 0;
  if (ph == "intra_gather_k_nomial") { nin = c; nout = b * c; }
  else if (ph == "inter_allgather_linear") { nin = b * c; nout = (long)T * b * c; }
  else if (ph == "intra_allgather_k_brucks") { nin = T * c; nout = (long)G * c; }
  else if (ph == "intra_reduce_scatter_radix_batch") { nin = (long)P * c; nout = (long)T * b * c; }
  else if (ph == "inter_reduce_linear") { nin = (long)T * b * c; nout = b * c; }
  else if (ph == "intra_scatter_radix_batch") { nin = b * c; nout = c; }
  else { std::fprintf(stderr, "unknown phase\n"); return 2; }
  shim_init(P);
  std::vector<std::vector<int>> out(P);
  std::vector<int> rcs(P, 0);
  std::vector<std::thread> th;
  for (int r = 0; r < P; ++r) th.emplace_back([&, r] {
    shim_set_rank(r);
    std::vector<int> s(nin);
    out[r].assign(nout, -17);
    for (long i = 0; i < nin; ++i) s[i] = pattern(seed, r, i);
    char* sb = (char*)s.data();
    char* rb = (char*)out[r].data();
    if (ph == "intra_gather_k_nomial") rcs[r] = intra_gather_k_nomial(sb, (int)c, MPI_INT, rb, 0, k, b);
    else if (ph == "inter_allgather_linear") rcs[r] = inter_allgather_linear(sb, (int)c, MPI_INT, rb, 0, b);
    else if (ph == "intra_allgather_k_brucks") rcs[r] = intra_allgather_k_brucks(sb, (int)c, MPI_INT, rb, 0, k, b);
    else if (ph == "intra_reduce_scatter_radix_batch") rcs[r] = intra_reduce_scatter_radix_batch(sb, rb, c, MPI_INT, MPI_SUM, 0, k, b);
    else if (ph == "inter_reduce_linear") rcs[r] = inter_reduce_linear(sb, rb, c, MPI_INT, MPI_SUM, 0, b);
    else rcs[r] = intra_scatter_radix_batch(sb, (int)c, MPI_INT, rb, 0, k, b);
  });
  for (auto& t : th) t.join();
  int bad = shim_failed();
  for (int v : rcs) bad |= (v != 0);
  std::printf("%d", bad);
  for (int r = 0; r < P; ++r) for (int v : out[r]) std::printf(" %d", v);
  std::printf("\n");
  return bad;
}

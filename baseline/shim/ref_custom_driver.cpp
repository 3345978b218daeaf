// Runs the reference's earlier "custom" allreduce (store-and-forward reduce-scatter + hierarchical allgather in
// one function, all_reduce_custom_0_2.cpp; it is also called all_reduce_radix_batch there, hence a binary of its
// own) on an int32 pattern and prints every rank's result.
//   ref_custom_driver P r b n seed        (vectors of P*n elements)
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>

#include "mpi.h"

int all_reduce_radix_batch(char*, char*, int, MPI_Datatype, MPI_Op, MPI_Comm, int, int);

static int pattern(int seed, int r, long i) { return (int)((seed * 31L + r * 1009L + i) % 97); }

int main(int argc, char** argv) {
  if (argc < 6) { std::fprintf(stderr, "usage: ref_custom_driver P r b n seed\n"); return 2; }
  const int P = std::atoi(argv[1]), r_ = std::atoi(argv[2]), b = std::atoi(argv[3]);
  const long n = std::atol(argv[4]);
  const int seed = std::atoi(argv[5]);
  shim_init(P);
  std::vector<std::vector<int>> out(P);
  std::vector<int> rcs(P, 0);
  std::vector<std::thread> th;
  for (int r = 0; r < P; ++r) th.emplace_back([&, r] {
    shim_set_rank(r);
    std::vector<int> s(n * P);
    out[r].assign(n * P, -17);
    for (long i = 0; i < n * P; ++i) s[i] = pattern(seed, r, i);
    rcs[r] = all_reduce_radix_batch((char*)s.data(), (char*)out[r].data(), (int)(n * P), MPI_INT, MPI_SUM, 0, r_, b);
  });
  for (auto& t : th) t.join();
  int bad = shim_failed();
  for (int v : rcs) bad |= (v != 0);
  std::printf("%d", bad);
  for (int r = 0; r < P; ++r) for (int v : out[r]) std::printf(" %d", v);
  std::printf("\n");
  return bad;
}

// Runs the reference's own collectives (compiled unmodified against the
// thread-per-rank shim) for timing and for golden checks.
//   ref_driver time  <ar|rs|ag> P k b bytes_per_rank steps warmup
//   ref_driver check <ar|rs|ag|semi> P k b elems_per_rank seed (int32 pattern, prints every rank's result;
//                    semi = all_reduce_semi_radix_batch)
//   ref_driver checkf <ar|rs|semi> P k b elems_per_rank seed   (float32 values that do not add exactly; prints bit patterns)
// Timing follows the reference's drivers: Barrier; t0; call; Barrier; t1
// (testing/custom_implementations/work_dir/all_reduce/main.cpp:56-66), here
// taken as the maximum over ranks.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "mpi.h"

int allgather_radix_batch(char*, int, MPI_Datatype, char*, MPI_Comm, int, int);
int reduce_scatter_radix_batch(const void*, void*, MPI_Aint, MPI_Datatype, MPI_Op, MPI_Comm, int, int);
int all_reduce_radix_batch(char*, char*, int, MPI_Datatype, MPI_Op, MPI_Comm, int, int);
int all_reduce_semi_radix_batch(char*, char*, int, MPI_Datatype, MPI_Op, MPI_Comm, int, int);   // "semi" in check mode

static int pattern(int seed, int r, long i) { return (int)((seed * 31L + r * 1009L + i) % 97); }

int main(int argc, char** argv) {
  if (argc < 8) { std::fprintf(stderr, "usage: see source\n"); return 2; }
  const std::string mode = argv[1], coll = argv[2];
  const int P = std::atoi(argv[3]), k = std::atoi(argv[4]), b = std::atoi(argv[5]);
  shim_init(P);
  if (mode == "checkf") {
    // the same on float32 values that do not add exactly: the printed bit patterns depend on the order of the additions
    const long n = std::atol(argv[6]);
    const int seed = std::atoi(argv[7]);
    std::vector<std::vector<float>> out(P);
    std::vector<std::thread> th;
    auto fpat = [&](int r, long i) { return (float)pattern(seed, r, i) / 7.0f + (float)r * 0.37f; };
    for (int r = 0; r < P; ++r) th.emplace_back([&, r] {
      shim_set_rank(r);
      if (coll == "rs") {
        std::vector<float> s(n * P); out[r].assign(n, -1.f);
        for (long i = 0; i < n * P; ++i) s[i] = fpat(r, i);
        reduce_scatter_radix_batch(s.data(), out[r].data(), n, MPI_FLOAT, MPI_SUM, 0, k, b);
      } else {
        std::vector<float> s(n * P); out[r].assign(n * P, -1.f);
        for (long i = 0; i < n * P; ++i) s[i] = fpat(r, i);
        if (coll == "semi") all_reduce_semi_radix_batch((char*)s.data(), (char*)out[r].data(), (int)(n * P), MPI_FLOAT, MPI_SUM, 0, k, b);
        else all_reduce_radix_batch((char*)s.data(), (char*)out[r].data(), (int)(n * P), MPI_FLOAT, MPI_SUM, 0, k, b);
      }
    });
    for (auto& t : th) t.join();
    std::printf("%d", shim_failed());
    for (int r = 0; r < P; ++r) for (float v : out[r]) { unsigned u; std::memcpy(&u, &v, 4); std::printf(" %u", u); }
    std::printf("\n");
    return shim_failed();
  }
  if (mode == "check") {
    const long n = std::atol(argv[6]);
    const int seed = std::atoi(argv[7]);
    std::vector<std::vector<int>> out(P);
    std::vector<std::thread> th;
    for (int r = 0; r < P; ++r) th.emplace_back([&, r] {
      shim_set_rank(r);
      if (coll == "ag") {
        std::vector<int> s(n); out[r].assign(n * P, -1);
        for (long i = 0; i < n; ++i) s[i] = pattern(seed, r, i);
        allgather_radix_batch((char*)s.data(), (int)n, MPI_INT, (char*)out[r].data(), 0, k, b);
      } else if (coll == "rs") {
        std::vector<int> s(n * P); out[r].assign(n, -1);
        for (long i = 0; i < n * P; ++i) s[i] = pattern(seed, r, i);
        reduce_scatter_radix_batch(s.data(), out[r].data(), n, MPI_INT, MPI_SUM, 0, k, b);
      } else {
        std::vector<int> s(n * P); out[r].assign(n * P, -1);
        for (long i = 0; i < n * P; ++i) s[i] = pattern(seed, r, i);
        if (coll == "semi") all_reduce_semi_radix_batch((char*)s.data(), (char*)out[r].data(), (int)(n * P), MPI_INT, MPI_SUM, 0, k, b);
        else all_reduce_radix_batch((char*)s.data(), (char*)out[r].data(), (int)(n * P), MPI_INT, MPI_SUM, 0, k, b);
      }
    });
    for (auto& t : th) t.join();
    std::printf("%d", shim_failed());
    for (int r = 0; r < P; ++r) for (int v : out[r]) std::printf(" %d", v);
    std::printf("\n");
    return shim_failed();
  }
  const long bytes = std::atol(argv[6]);
  const int steps = std::atoi(argv[7]), warmup = argc > 8 ? std::atoi(argv[8]) : 1;
  const long n = bytes / 4;  // floats per rank (ar: whole vector; rs: P*n in; ag: n in)
  std::vector<double> worst(steps, 0.0);
  std::vector<int> ok(P, 1);
  std::vector<std::thread> th;
  for (int r = 0; r < P; ++r) th.emplace_back([&, r] {
    shim_set_rank(r);
    const long per = (coll == "ar") ? n / P * P : n;
    std::vector<float> s((coll == "ag") ? per : (coll == "rs" ? per * P : per));
    std::vector<float> o((coll == "ag") ? per * P : (coll == "rs" ? per : per));
    for (size_t i = 0; i < s.size(); ++i) s[i] = (float)((r * 7 + (long)i) % 13) * 0.25f;
    for (int it = -warmup; it < steps; ++it) {
      MPI_Barrier(0);
      double t0 = MPI_Wtime();
      if (coll == "ag") allgather_radix_batch((char*)s.data(), (int)per, MPI_FLOAT, (char*)o.data(), 0, k, b);
      else if (coll == "rs") reduce_scatter_radix_batch(s.data(), o.data(), per, MPI_FLOAT, MPI_SUM, 0, k, b);
      else all_reduce_radix_batch((char*)s.data(), (char*)o.data(), (int)per, MPI_FLOAT, MPI_SUM, 0, k, b);
      MPI_Barrier(0);
      double t1 = MPI_Wtime();
      if (it >= 0 && r == 0) worst[it] = t1 - t0;  // both barriers are global: every rank sees the same interval
    }
    if (coll == "ar") {  // spot check: element i = sum over ranks
      for (long i = 0; i < per; i += (per / 64 + 1)) {
        float e = 0;
        for (int q = 0; q < P; ++q) e += (float)((q * 7 + i) % 13) * 0.25f;
        if (o[i] != e) ok[r] = 0;
      }
    }
  });
  for (auto& t : th) t.join();
  double tot = 0;
  for (double v : worst) tot += v;
  int all = !shim_failed();
  for (int v : ok) all &= v;
  std::printf("{\"ms_per_step\": %.6f, \"steps\": %d, \"is_correct\": %d}\n", tot / steps * 1e3, steps, all);
  return all ? 0 : 1;
}

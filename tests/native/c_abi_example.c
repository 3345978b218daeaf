/* A plain C consumer of the library: an emulated 4-rank world on one GPU driven
 * through the generic entry point, and the reference-compatible signature on a
 * one-rank communicator.  Built and run by tests/test_c_abi.py. */
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>

#include "chb.h"
#include "chb_compat.h"

#define CHECK(x) do { int rc_ = (x); if (rc_) { printf("FAIL %s -> %d\n", #x, rc_); return 1; } } while (0)

int main(void) {
  enum { P = 4, N = 4096 };
  char err[256] = {0};
  size_t hb = chb_heap_bytes(P, 65536, 1 << 20, 1 << 20);
  char* base = NULL;
  if (cudaMalloc((void**)&base, hb * P) != cudaSuccess) { printf("FAIL cudaMalloc\n"); return 1; }
  cudaMemset(base, 0, hb * P);
  void* heaps[P];
  for (int p = 0; p < P; ++p) heaps[p] = base + hb * p;
  struct chb_comm* comm = chb_comm_create(0, P, P, heaps, NULL, 65536, 1 << 20, 1 << 20, err, sizeof err);
  if (!comm) { printf("FAIL create: %s\n", err); return 1; }
  float *in[P], *out[P], *host = (float*)malloc(sizeof(float) * N);
  for (int p = 0; p < P; ++p) {
    cudaMalloc((void**)&in[p], sizeof(float) * N);
    cudaMalloc((void**)&out[p], sizeof(float) * N);
    for (int i = 0; i < N; ++i) host[i] = (float)(p + 1) + 0.001f * (float)(i % 7);
    cudaMemcpy(in[p], host, sizeof(float) * N, cudaMemcpyHostToDevice);
  }
  const char* algos[3] = {"radix_batch", "ll", "ring"};
  for (int a = 0; a < 3; ++a) {
    CHECK(chb_collective(comm, CHB_ALLREDUCE, algos[a], 2, 2, 0, CHB_F32, CHB_SUM, (const void* const*)in,
                         (void* const*)out, N, 1.0f, 0, 0));
    unsigned long long st[8];
    CHECK(chb_comm_status(comm, 0, st, 0));
    cudaMemcpy(host, out[2], sizeof(float) * N, cudaMemcpyDeviceToHost);
    for (int i = 0; i < N; ++i) {
      float e = 10.0f + 4 * 0.001f * (float)(i % 7);
      if (host[i] < e - 1e-4f || host[i] > e + 1e-4f) { printf("FAIL %s value %d: %f vs %f\n", algos[a], i, host[i], e); return 1; }
    }
  }
  /* wrong group size comes back as an error code, nothing is launched */
  if (chb_collective(comm, CHB_ALLREDUCE, "radix_batch", 2, 3, 0, CHB_F32, CHB_SUM, (const void* const*)in,
                     (void* const*)out, N, 1.0f, 0, 0) != CHB_ERR_ARG) { printf("FAIL expected CHB_ERR_ARG\n"); return 1; }
  chb_comm_destroy(comm);
  /* reference-compatible signature on a one-rank communicator */
  cudaMemset(base, 0, hb);
  void* one[1] = {base};
  struct chb_comm* c1 = chb_comm_create(0, 1, 1, one, NULL, 65536, 1 << 20, 1 << 20, err, sizeof err);
  if (!c1) { printf("FAIL create one: %s\n", err); return 1; }
  CHECK(all_reduce_radix_batch((char*)in[1], (char*)out[1], N, CHB_F32, CHB_SUM, c1, 2, 1));
  CHECK(MPICH_Allreduce_recursive_doubling((const char*)in[1], (char*)out[0], N, CHB_F32, CHB_SUM, c1));
  CHECK(reduce_scatter_radix_batch(CHB_IN_PLACE, out[1], N, CHB_F32, CHB_SUM, c1, 2, 1));
  cudaDeviceSynchronize();
  cudaMemcpy(host, out[0], sizeof(float) * N, cudaMemcpyDeviceToHost);
  if (host[3] < 2.002f || host[3] > 2.004f) { printf("FAIL one-rank value %f\n", host[3]); return 1; }
  chb_comm_destroy(c1);
  printf("C ABI OK %s\n", chb_version());
  return 0;
}

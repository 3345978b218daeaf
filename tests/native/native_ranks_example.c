/* One rank per GPU from plain C, without MPI and without Python: the launcher forks, the ranks meet
 * through the shared-memory bootstrap, build a communicator over cudaIpc heaps and call a collective
 * through the reference's signature.  Usage: native_ranks_example <number of GPUs>
 * (cc native_ranks_example.c -I csrc/api -I csrc/boot -I $CUDA/include -L . -lchb -L $CUDA/lib64 -lcudart) */
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <sys/wait.h>
#include <unistd.h>

#include "bootstrap.h"
#include "chb.h"
#include "chb_compat.h"

static int rank_main(const char* name, int rank, int world) {
  const int n = (1 << 16) / world * world;    /* elements of the allreduce vector: a multiple of the ranks */
  if (cudaSetDevice(rank) != cudaSuccess) return 10;
  struct chb_bootstrap* boot = NULL;
  if (chb_bootstrap_create(name, rank, world, 60000, &boot)) return 11;
  char err[256];
  struct chb_comm* comm = chb_comm_create_ipc(boot, 1 << 20, 16u << 20, 4096, err, sizeof err);
  if (!comm) { fprintf(stderr, "rank %d: %s\n", rank, err); chb_bootstrap_destroy(boot); return 12; }

  int* h = (int*)malloc(sizeof(int) * n);
  for (int i = 0; i < n; ++i) h[i] = rank + i % 7;
  int *x = NULL, *y = NULL;
  cudaMalloc((void**)&x, sizeof(int) * n);
  cudaMalloc((void**)&y, sizeof(int) * n);
  cudaMemcpy(x, h, sizeof(int) * n, cudaMemcpyHostToDevice);

  int rc = all_reduce_radix_batch((char*)x, (char*)y, n, CHB_I32, CHB_SUM, comm, 2, 1);     /* k = 2, b = 1 */
  if (!rc) rc = MPICH_Allreduce_ring((const char*)x, (char*)y, n, CHB_I32, CHB_SUM, comm);
  unsigned long long status[8];
  if (!rc) rc = chb_comm_status(comm, 0, status, NULL);                                      /* synchronises the stream */
  cudaMemcpy(h, y, sizeof(int) * n, cudaMemcpyDeviceToHost);
  int bad = rc != 0;
  for (int i = 0; i < n && !bad; ++i) bad = h[i] != world * (i % 7) + world * (world - 1) / 2;

  chb_bootstrap_barrier(boot);                /* nobody frees a heap that a peer may still read */
  chb_comm_destroy(comm);
  chb_bootstrap_destroy(boot);
  cudaFree(x);
  cudaFree(y);
  free(h);
  return bad ? 13 : 0;
}

int main(int argc, char** argv) {
  const int world = argc > 1 ? atoi(argv[1]) : 2;
  if (world < 1 || world > 16) return 2;
  char name[64];
  snprintf(name, sizeof name, "/chb_example_%d", (int)getpid());
  pid_t kids[16];
  for (int r = 0; r < world; ++r) {           /* fork before anything touches CUDA */
    kids[r] = fork();
    if (kids[r] == 0) _exit(rank_main(name, r, world));
  }
  int worst = 0;
  for (int r = 0; r < world; ++r) {
    int st = 0;
    waitpid(kids[r], &st, 0);
    int code = WIFEXITED(st) ? WEXITSTATUS(st) : 1;
    if (code > worst) worst = code;
  }
  printf(worst ? "NATIVE RANKS FAILED (%d)\n" : "NATIVE RANKS OK\n", worst);
  return worst;
}

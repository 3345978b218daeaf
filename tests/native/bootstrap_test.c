/* The shared-memory rendezvous from plain C: forked ranks exchange blobs, meet at barriers,
 * and - in the second half - notice within the deadline that one rank never shows up. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/wait.h>
#include <unistd.h>

#include "bootstrap.h"

static int run_rank(const char* name, int rank, int world, int timeout_ms, int rounds) {
  struct chb_bootstrap* b = NULL;
  int rc = chb_bootstrap_create(name, rank, world, timeout_ms, &b);
  if (rc) return 100 + rc;
  if (chb_bootstrap_rank(b) != rank || chb_bootstrap_world(b) != world) return 2;
  for (int it = 0; it < rounds; ++it) {
    char mine[64], all[64 * 16];
    memset(mine, 0, sizeof mine);
    snprintf(mine, sizeof mine, "rank %d round %d", rank, it);
    if (chb_bootstrap_allgather(b, mine, all, 64)) return 3;
    for (int r = 0; r < world; ++r) {
      char want[64];
      snprintf(want, sizeof want, "rank %d round %d", r, it);
      if (strcmp(all + 64 * r, want)) return 4;
    }
    if (chb_bootstrap_barrier(b)) return 5;
  }
  chb_bootstrap_destroy(b);
  return 0;
}

int main(void) {
  char name[64];
  const int world = 4;
  /* 1: everybody arrives */
  snprintf(name, sizeof name, "/chb_boot_test_%d_a", (int)getpid());
  pid_t kids[8];
  for (int r = 0; r < world; ++r) {
    kids[r] = fork();
    if (kids[r] == 0) _exit(run_rank(name, r, world, 20000, 50));
  }
  for (int r = 0; r < world; ++r) {
    int st = 0;
    waitpid(kids[r], &st, 0);
    if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) { printf("rank %d failed: status %d\n", r, WIFEXITED(st) ? WEXITSTATUS(st) : -1); return 1; }
  }
  /* 2: rank 3 never starts: the others give up after the deadline with CHB_ERR_TIMEOUT (6) or,
   * once one of them has raised the abort flag, CHB_ERR_OTHER (2) */
  snprintf(name, sizeof name, "/chb_boot_test_%d_b", (int)getpid());
  for (int r = 0; r < world - 1; ++r) {
    kids[r] = fork();
    if (kids[r] == 0) _exit(run_rank(name, r, world, 500, 1));
  }
  for (int r = 0; r < world - 1; ++r) {
    int st = 0;
    waitpid(kids[r], &st, 0);
    int code = WIFEXITED(st) ? WEXITSTATUS(st) : -1;
    if (code != 106 && code != 102) { printf("rank %d: expected a timeout, got %d\n", r, code); return 1; }
  }
  printf("BOOTSTRAP OK\n");
  return 0;
}

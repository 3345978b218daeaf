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

/* every rank hands a pipe's read end to all others; each then reads, through its duplicates, what the owners wrote */
static int run_fd_rank(const char* name, int rank, int world, int offers) {
  struct chb_bootstrap* b = NULL;
  if (chb_bootstrap_create(name, rank, world, 20000, &b)) return 10;
  int pp[2] = {-1, -1};
  if (offers) {
    if (pipe(pp)) return 11;
    char msg[32];
    snprintf(msg, sizeof msg, "from %d", rank);
    for (int r = 0; r < world - 1; ++r)           /* one copy per reader: a pipe's bytes are consumed */
      if (write(pp[1], msg, 16) != 16) return 12;
  }
  int fds[16];
  if (chb_bootstrap_exchange_fds(b, offers ? pp[0] : -1, fds)) return 13;
  for (int r = 0; r < world; ++r) {
    if (r == rank) { if (fds[r] != (offers ? pp[0] : -1)) return 14; continue; }
    const int r_offers = (r % 2 == 0) || offers == 2;
    if (!r_offers) { if (fds[r] != -1) return 15; continue; }
    char got[16], want[32];
    if (fds[r] < 0 || read(fds[r], got, 16) != 16) return 16;
    snprintf(want, sizeof want, "from %d", r);
    if (strcmp(got, want)) return 17;
    close(fds[r]);
  }
  if (chb_bootstrap_barrier(b)) return 18;
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
  /* 3: descriptors travel between the ranks: everybody offers one (mode 2), then only the even ranks do (mode 1 / 0) */
  for (int mode = 0; mode < 2; ++mode) {
    snprintf(name, sizeof name, "/chb_boot_test_%d_c%d", (int)getpid(), mode);
    for (int r = 0; r < world; ++r) {
      kids[r] = fork();
      if (kids[r] == 0) _exit(run_fd_rank(name, r, world, mode == 0 ? 2 : (r % 2 == 0 ? 1 : 0)));
    }
    for (int r = 0; r < world; ++r) {
      int st = 0;
      waitpid(kids[r], &st, 0);
      if (!WIFEXITED(st) || WEXITSTATUS(st) != 0) { printf("descriptor exchange, rank %d failed: status %d\n", r, WIFEXITED(st) ? WEXITSTATUS(st) : -1); return 1; }
    }
  }
  printf("BOOTSTRAP OK\n");
  return 0;
}

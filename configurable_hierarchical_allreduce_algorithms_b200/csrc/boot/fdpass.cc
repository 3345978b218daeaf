// File descriptors between the ranks of one box (see bootstrap.h): the carrier of CUDA virtual-memory
// allocation handles (POSIX file-descriptor handle type) from the rank that owns an allocation to the
// ranks that map it.  Plays the part that the MPI library's shared-memory transport plays for the
// reference, whose ranks never share memory themselves.
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../api/chb.h"
#include "bootstrap.h"

namespace {

// abstract address (leading NUL): lives in no file system, disappears with the socket
socklen_t address_of(const char* job, int rank, sockaddr_un* a) {
  std::memset(a, 0, sizeof *a);
  a->sun_family = AF_UNIX;
  const int n = std::snprintf(a->sun_path + 1, sizeof a->sun_path - 1, "chb%s.%d", job, rank);
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + (size_t)n);
}

int64_t now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (int64_t)ts.tv_sec * 1000 + ts.tv_nsec / 1000000;
}

}  // namespace

extern "C" int chb_bootstrap_exchange_fds(chb_bootstrap* b, int my_fd, int* fds) {
  if (!b || !fds) return CHB_ERR_ARG;
  const int P = chb_bootstrap_world(b), rank = chb_bootstrap_rank(b);
  const char* job = chb_bootstrap_name(b);
  for (int r = 0; r < P; ++r) fds[r] = -1;
  fds[rank] = my_fd;
  // who offers a descriptor at all
  std::vector<int> offers((size_t)P, 0);
  const int mine = my_fd >= 0 ? 1 : 0;
  int rc = chb_bootstrap_allgather(b, &mine, offers.data(), sizeof(int));
  if (rc) return rc;
  int sock = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  if (sock < 0) { chb_bootstrap_abort(b); return CHB_ERR_OTHER; }
  sockaddr_un me;
  const socklen_t melen = address_of(job, rank, &me);
  if (bind(sock, (sockaddr*)&me, melen) != 0) { close(sock); chb_bootstrap_abort(b); return CHB_ERR_OTHER; }
  rc = chb_bootstrap_barrier(b);                       // every socket is bound before anybody sends
  if (rc) { close(sock); return rc; }
  if (my_fd >= 0)
    for (int r = 0; r < P; ++r) {
      if (r == rank) continue;
      sockaddr_un to;
      const socklen_t tolen = address_of(job, r, &to);
      int32_t payload = rank;
      iovec iov{&payload, sizeof payload};
      alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {0};
      msghdr m{};
      m.msg_name = &to;
      m.msg_namelen = tolen;
      m.msg_iov = &iov;
      m.msg_iovlen = 1;
      m.msg_control = ctrl;
      m.msg_controllen = sizeof ctrl;
      cmsghdr* c = CMSG_FIRSTHDR(&m);
      c->cmsg_level = SOL_SOCKET;
      c->cmsg_type = SCM_RIGHTS;
      c->cmsg_len = CMSG_LEN(sizeof(int));
      std::memcpy(CMSG_DATA(c), &my_fd, sizeof(int));
      if (sendmsg(sock, &m, 0) < 0) { close(sock); chb_bootstrap_abort(b); return CHB_ERR_OTHER; }
    }
  int expect = 0;
  for (int r = 0; r < P; ++r) expect += (r != rank && offers[(size_t)r]) ? 1 : 0;
  const int64_t deadline = now_ms() + 30000;
  int got = 0, result = CHB_SUCCESS;
  while (got < expect) {
    pollfd pf{sock, POLLIN, 0};
    const int64_t left = deadline - now_ms();
    if (left <= 0 || poll(&pf, 1, (int)(left < 200 ? left : 200)) < 0) { if (left <= 0) { result = CHB_ERR_TIMEOUT; break; } continue; }
    if (!(pf.revents & POLLIN)) continue;
    int32_t payload = -1;
    iovec iov{&payload, sizeof payload};
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {0};
    msghdr m{};
    m.msg_iov = &iov;
    m.msg_iovlen = 1;
    m.msg_control = ctrl;
    m.msg_controllen = sizeof ctrl;
    if (recvmsg(sock, &m, MSG_CMSG_CLOEXEC) < (ssize_t)sizeof payload) continue;
    cmsghdr* c = CMSG_FIRSTHDR(&m);
    if (!c || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS || payload < 0 || payload >= P) continue;
    int fd = -1;
    std::memcpy(&fd, CMSG_DATA(c), sizeof(int));
    if (fds[payload] >= 0 && payload != rank) close(fds[payload]);
    fds[payload] = fd;
    ++got;
  }
  if (result != CHB_SUCCESS) chb_bootstrap_abort(b);
  const int rc2 = chb_bootstrap_barrier(b);            // nobody closes its socket while a peer may still send to it
  close(sock);
  if (result == CHB_SUCCESS && rc2) result = rc2;
  if (result != CHB_SUCCESS)
    for (int r = 0; r < P; ++r)
      if (r != rank && fds[r] >= 0) { close(fds[r]); fds[r] = -1; }
  return result;
}

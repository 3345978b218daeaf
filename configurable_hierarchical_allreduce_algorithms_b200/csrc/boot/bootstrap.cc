// Shared-memory rendezvous of the ranks of one box (see bootstrap.h).
#include "bootstrap.h"

#include <fcntl.h>
#include <sched.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <cstdint>
#include <cstring>
#include <new>
#include <string>

#include "../api/chb.h"

namespace {

constexpr uint32_t kMagic = 0x43484231u;   // "CHB1"
constexpr int kMaxWorld = 64;

struct Segment {
  std::atomic<uint32_t> magic;
  std::atomic<uint32_t> world;
  std::atomic<uint32_t> attached;
  std::atomic<uint32_t> count;   // barrier arrivals of the current generation
  std::atomic<uint32_t> gen;     // barrier generation
  std::atomic<uint32_t> abort;
  char pad[40];
  char slots[kMaxWorld][CHB_BOOT_SLOT_BYTES];
};
static_assert(std::atomic<uint32_t>::is_always_lock_free, "cross-process atomics must be lock free");

int64_t now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (int64_t)ts.tv_sec * 1000 + ts.tv_nsec / 1000000;
}

void relax(int spins) {
  if (spins < 200) sched_yield();
  else usleep(50);
}

}  // namespace

struct chb_bootstrap {
  std::string name;
  int rank = 0, world = 1, timeout_ms = 30000;
  Segment* seg = nullptr;
};

extern "C" {

int chb_bootstrap_create(const char* name, int rank, int world, int timeout_ms, chb_bootstrap** out) {
  if (!name || name[0] != '/' || !out || world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return CHB_ERR_ARG;
  if (timeout_ms <= 0) timeout_ms = 30000;
  const int64_t deadline = now_ms() + timeout_ms;
  int fd = -1;
  if (rank == 0) {
    shm_unlink(name);   // a stale segment of a crashed job with the same name
    fd = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd < 0) return CHB_ERR_OTHER;
    if (ftruncate(fd, (off_t)sizeof(Segment)) != 0) { close(fd); shm_unlink(name); return CHB_ERR_NO_MEM; }
  } else {
    int spins = 0;
    for (;;) {
      fd = shm_open(name, O_RDWR, 0600);
      if (fd >= 0) {
        struct stat st;
        if (fstat(fd, &st) == 0 && (size_t)st.st_size >= sizeof(Segment)) break;   // rank 0 has sized it
        close(fd);
        fd = -1;
      }
      if (now_ms() > deadline) return CHB_ERR_TIMEOUT;
      relax(++spins);
    }
  }
  void* m = mmap(nullptr, sizeof(Segment), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (m == MAP_FAILED) { if (rank == 0) shm_unlink(name); return CHB_ERR_NO_MEM; }
  Segment* s = (Segment*)m;
  if (rank == 0) {
    // a fresh segment is zero-filled; publish the parameters last
    s->world.store((uint32_t)world);
    s->attached.store(0);
    s->count.store(0);
    s->gen.store(0);
    s->abort.store(0);
    s->magic.store(kMagic, std::memory_order_release);
  } else {
    int spins = 0;
    while (s->magic.load(std::memory_order_acquire) != kMagic) {
      if (now_ms() > deadline) { munmap(m, sizeof(Segment)); return CHB_ERR_TIMEOUT; }
      relax(++spins);
    }
    if ((int)s->world.load() != world) { munmap(m, sizeof(Segment)); return CHB_ERR_ARG; }
  }
  auto* b = new (std::nothrow) chb_bootstrap;
  if (!b) { munmap(m, sizeof(Segment)); return CHB_ERR_NO_MEM; }
  b->name = name;
  b->rank = rank;
  b->world = world;
  b->timeout_ms = timeout_ms;
  b->seg = s;
  s->attached.fetch_add(1);
  int rc = chb_bootstrap_barrier(b);
  if (rc != CHB_SUCCESS) { chb_bootstrap_destroy(b); return rc; }
  *out = b;
  return CHB_SUCCESS;
}

int chb_bootstrap_rank(const chb_bootstrap* b) { return b ? b->rank : -1; }
int chb_bootstrap_world(const chb_bootstrap* b) { return b ? b->world : 0; }
const char* chb_bootstrap_name(const chb_bootstrap* b) { return b ? b->name.c_str() : ""; }

int chb_bootstrap_barrier(chb_bootstrap* b) {
  if (!b) return CHB_ERR_ARG;
  Segment* s = b->seg;
  if (s->abort.load()) return CHB_ERR_OTHER;
  const uint32_t g = s->gen.load(std::memory_order_acquire);
  if (s->count.fetch_add(1, std::memory_order_acq_rel) + 1 == (uint32_t)b->world) {
    s->count.store(0, std::memory_order_relaxed);
    s->gen.store(g + 1, std::memory_order_release);
    return CHB_SUCCESS;
  }
  const int64_t deadline = now_ms() + b->timeout_ms;
  int spins = 0;
  while (s->gen.load(std::memory_order_acquire) == g) {
    if (s->abort.load()) return CHB_ERR_OTHER;
    if (now_ms() > deadline) { s->abort.store(1); return CHB_ERR_TIMEOUT; }
    relax(++spins);
  }
  return CHB_SUCCESS;
}

int chb_bootstrap_allgather(chb_bootstrap* b, const void* mine, void* all, size_t bytes) {
  if (!b || !mine || !all || bytes > CHB_BOOT_SLOT_BYTES) return CHB_ERR_ARG;
  std::memcpy(b->seg->slots[b->rank], mine, bytes);
  int rc = chb_bootstrap_barrier(b);          // every slot is written
  if (rc) return rc;
  for (int r = 0; r < b->world; ++r) std::memcpy((char*)all + (size_t)r * bytes, b->seg->slots[r], bytes);
  return chb_bootstrap_barrier(b);            // every slot is read: it may be overwritten
}

void chb_bootstrap_abort(chb_bootstrap* b) {
  if (b) b->seg->abort.store(1);
}

void chb_bootstrap_destroy(chb_bootstrap* b) {
  if (!b) return;
  if (b->seg) munmap(b->seg, sizeof(Segment));
  if (b->rank == 0) shm_unlink(b->name.c_str());
  delete b;
}

}  // extern "C"

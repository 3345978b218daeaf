// Thread-per-rank implementation of the calls declared in mpi.h (see there).
//
// Ranks are threads of one process.  Small point-to-point sends are eager (the
// payload is packed into the destination's mailbox); a non-blocking send of 64 KiB
// or more of a basic type is a rendezvous: the mailbox entry only points at the
// sender's buffer, the receiver copies from it once (what a shared-memory MPI does
// for large messages) and the send request completes when that copy is done.
// Receives match on (communicator, source, tag) in arrival order.  A rank that
// waits, for a send or a receive, keeps completing all the receives it has posted,
// as an MPI progress engine would.  Communicators are rank lists created by
// MPI_Comm_split; the few collectives the reference's sources call are done by
// publishing buffer pointers and meeting at the communicator's barrier.
// Derived datatypes are lists of (byte displacement, byte length) segments.
#include "mpi.h"

#include <algorithm>
#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <vector>

namespace { struct Rdv { bool done = false; }; }   // guarded by the SENDER's mailbox mutex
struct ShimRequest {
  bool recv; void* buf; int count; MPI_Datatype type; int peer, tag; MPI_Comm comm;
  bool done = false;                 // receive completed (by whichever wait of this rank made progress)
  std::shared_ptr<Rdv> rdv;          // rendezvous send: completes when the receiver has copied
};
namespace {
constexpr size_t kRendezvousBytes = 64 << 10;
struct Message {
  int comm, src, tag; std::unique_ptr<char[]> data; size_t bytes;
  const void* ref = nullptr;         // rendezvous: the sender's buffer (data is empty)
  std::shared_ptr<Rdv> rdv;
  int gsrc = -1;                     // global rank of the sender (whose mailbox guards rdv)
};
struct Mailbox { std::mutex m; std::condition_variable cv; std::deque<Message> q; };
struct Comm {
  std::vector<int> ranks;                 // global ranks, in communicator order
  std::mutex m;
  std::condition_variable cv;
  int count = 0;
  long gen = 0;
  std::vector<const void*> pub;           // one published pointer per member
  std::vector<std::pair<int, int>> split; // (color, key) per member during MPI_Comm_split
  std::map<int, int> split_ids;           // color -> new communicator
};
struct Segments { std::vector<std::pair<long, long>> seg; long bytes = 0; };

int g_n = 0;
std::vector<std::unique_ptr<Mailbox>> g_box;
std::vector<std::unique_ptr<Comm>> g_comms;       // index = MPI_Comm; 0 = world
std::mutex g_reg_m;                               // guards growth of g_comms / g_types
std::vector<Segments> g_types;                    // derived datatypes, id = kTypeBase + index
constexpr int kTypeBase = 1000;
thread_local int t_rank = -1;
thread_local bool g_rendezvous_ok = true;
thread_local std::vector<ShimRequest*> t_posted;  // receives this rank has posted and not yet waited for
bool g_fail = false;

size_t basic_bytes(MPI_Datatype d) { return d == MPI_FLOAT ? 4 : (size_t)d; }
bool derived(MPI_Datatype d) { return d >= kTypeBase; }
Segments type_of(MPI_Datatype d) {
  std::lock_guard<std::mutex> l(g_reg_m);
  return g_types[(size_t)(d - kTypeBase)];
}
size_t type_bytes(MPI_Datatype d) { return derived(d) ? (size_t)type_of(d).bytes : basic_bytes(d); }

// No lock: the table's storage is reserved once (shim_init), entries are only appended, and a rank learns a new
// communicator's index behind the barrier of MPI_Comm_split.  This is on the path of every send and receive.
Comm& comm_of(MPI_Comm c) { return *g_comms[(size_t)c]; }
int comm_rank(Comm& c) {
  for (size_t i = 0; i < c.ranks.size(); ++i)
    if (c.ranks[i] == t_rank) return (int)i;
  return -1;
}
void comm_barrier(Comm& c) {
  std::unique_lock<std::mutex> l(c.m);
  long gen = c.gen;
  if (++c.count == (int)c.ranks.size()) { c.count = 0; ++c.gen; c.cv.notify_all(); }
  else c.cv.wait(l, [&] { return c.gen != gen; });
}

// `count` elements of type d starting at buf as one contiguous byte string, and back
void pack(const void* buf, int count, MPI_Datatype d, char* out) {
  if (!derived(d)) { std::memcpy(out, buf, (size_t)count * basic_bytes(d)); return; }
  Segments s = type_of(d);
  for (int i = 0; i < count; ++i)      // the reference only ever sends one element of a derived type
    for (auto& g : s.seg) { std::memcpy(out, (const char*)buf + g.first, (size_t)g.second); out += g.second; }
}
void unpack(const char* in, size_t bytes, void* buf, int count, MPI_Datatype d) {
  if (!derived(d)) { std::memcpy(buf, in, bytes); return; }
  Segments s = type_of(d);
  for (int i = 0; i < count; ++i)
    for (auto& g : s.seg) {
      size_t n = std::min(bytes, (size_t)g.second);
      std::memcpy((char*)buf + g.first, in, n);
      in += n;
      bytes -= n;
    }
}

template <class T> void reduce(const T* a, T* b, int n, MPI_Op op) {
  if (op == MPI_SUM) for (int i = 0; i < n; ++i) b[i] = a[i] + b[i];
  else if (op == MPI_MAX) for (int i = 0; i < n; ++i) b[i] = a[i] > b[i] ? a[i] : b[i];
  else for (int i = 0; i < n; ++i) b[i] = a[i] < b[i] ? a[i] : b[i];
}
}  // namespace

void shim_init(int n) {
  g_n = n;
  g_box.clear();
  for (int i = 0; i < n; ++i) g_box.emplace_back(new Mailbox);
  g_comms.clear();
  g_comms.reserve(1 << 16);
  g_comms.emplace_back(new Comm);
  for (int i = 0; i < n; ++i) g_comms[0]->ranks.push_back(i);
  g_comms[0]->pub.assign((size_t)n, nullptr);
  g_comms[0]->split.assign((size_t)n, {0, 0});
  g_types.clear();
  g_fail = false;
}
void shim_set_rank(int r) { t_rank = r; }
int shim_failed() { return g_fail ? 1 : 0; }

int MPI_Comm_rank(MPI_Comm c, int* r) { *r = comm_rank(comm_of(c)); return MPI_SUCCESS; }
int MPI_Comm_size(MPI_Comm c, int* s) { *s = (int)comm_of(c).ranks.size(); return MPI_SUCCESS; }
int MPI_Type_size(MPI_Datatype d, int* s) { *s = (int)type_bytes(d); return MPI_SUCCESS; }

int MPI_Comm_split(MPI_Comm parent, int color, int key, MPI_Comm* out) {
  Comm& p = comm_of(parent);
  const int me = comm_rank(p);
  p.split[(size_t)me] = {color, key};
  comm_barrier(p);                                  // every (color, key) is published
  if (me == 0) {
    p.split_ids.clear();
    std::map<int, std::vector<std::pair<std::pair<int, int>, int>>> groups;   // color -> ((key, parent rank), global rank)
    for (size_t i = 0; i < p.ranks.size(); ++i)
      if (p.split[i].first != MPI_UNDEFINED) groups[p.split[i].first].push_back({{p.split[i].second, (int)i}, p.ranks[i]});
    for (auto& kv : groups) {
      std::sort(kv.second.begin(), kv.second.end());
      auto c = std::unique_ptr<Comm>(new Comm);
      for (auto& e : kv.second) c->ranks.push_back(e.second);
      c->pub.assign(c->ranks.size(), nullptr);
      c->split.assign(c->ranks.size(), {0, 0});
      std::lock_guard<std::mutex> l(g_reg_m);
      g_comms.push_back(std::move(c));
      p.split_ids[kv.first] = (int)g_comms.size() - 1;
    }
  }
  comm_barrier(p);                                  // the new communicators exist
  *out = color == MPI_UNDEFINED ? MPI_COMM_NULL : p.split_ids[color];
  comm_barrier(p);                                  // everybody has read its id before the next split reuses the table
  return MPI_SUCCESS;
}
int MPI_Comm_free(MPI_Comm* c) { *c = MPI_COMM_NULL; return MPI_SUCCESS; }

int MPI_Isend(const void* buf, int count, MPI_Datatype d, int dst, int tag, MPI_Comm c, MPI_Request* r) {
  *r = new ShimRequest{false, nullptr, 0, d, dst, tag, c};
  Comm& cm = comm_of(c);
  if (dst < 0 || dst >= (int)cm.ranks.size()) { g_fail = true; return MPI_ERR_ARG; }
  const int gdst = cm.ranks[(size_t)dst];
  size_t n = (size_t)count * type_bytes(d);
  Message m{c, comm_rank(cm), tag, nullptr, n};
  if (g_rendezvous_ok && !derived(d) && n >= kRendezvousBytes) {
    m.ref = buf;
    m.rdv = std::make_shared<Rdv>();
    m.gsrc = t_rank;
    (*r)->rdv = m.rdv;
  } else {
    m.data.reset(new char[n ? n : 1]);
    pack(buf, count, d, m.data.get());
  }
  { std::lock_guard<std::mutex> l(g_box[gdst]->m); g_box[gdst]->q.push_back(std::move(m)); }
  g_box[gdst]->cv.notify_all();
  return MPI_SUCCESS;
}
int MPI_Irecv(void* buf, int count, MPI_Datatype d, int src, int tag, MPI_Comm c, MPI_Request* r) {
  *r = new ShimRequest{true, buf, count, d, src, tag, c};
  t_posted.push_back(*r);
  return MPI_SUCCESS;
}

namespace {
// Complete, in posting order, every posted receive of this rank whose message has arrived.  Called with this
// rank's mailbox locked; the lock is dropped while a payload is copied.
void progress(Mailbox& b, std::unique_lock<std::mutex>& l) {
  for (size_t i = 0; i < t_posted.size(); ++i) {
    ShimRequest* r = t_posted[i];
    if (r->done) continue;
    for (auto it = b.q.begin(); it != b.q.end(); ++it) {
      if (!(it->comm == r->comm && it->src == r->peer && it->tag == r->tag)) continue;
      Message m = std::move(*it);
      b.q.erase(it);
      l.unlock();
      const size_t cap = (size_t)r->count * type_bytes(r->type);
      if (m.bytes > cap) g_fail = true;  // truncation
      unpack(m.ref ? (const char*)m.ref : m.data.get(), std::min(m.bytes, cap), r->buf, r->count, r->type);
      if (m.rdv) {
        Mailbox& sb = *g_box[(size_t)m.gsrc];
        { std::lock_guard<std::mutex> g(sb.m); m.rdv->done = true; }
        sb.cv.notify_all();
      }
      l.lock();
      r->done = true;
      break;
    }
  }
}
}  // namespace

int MPI_Wait(MPI_Request* rp, MPI_Status*) {
  ShimRequest* r = *rp;
  if (!r) return MPI_SUCCESS;
  if (r->recv || r->rdv) {
    Mailbox& b = *g_box[t_rank];
    std::unique_lock<std::mutex> l(b.m);
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
      progress(b, l);
      if (r->recv ? r->done : r->rdv->done) break;
      b.cv.wait_for(l, std::chrono::milliseconds(200));
      if (std::chrono::steady_clock::now() - t0 > std::chrono::seconds(120)) { g_fail = true; break; }
    }
    if (r->recv) t_posted.erase(std::find(t_posted.begin(), t_posted.end(), r));
  }
  delete r;
  *rp = nullptr;
  return MPI_SUCCESS;
}
int MPI_Waitall(int n, MPI_Request* r, MPI_Status*) {
  for (int i = 0; i < n; ++i) MPI_Wait(&r[i], nullptr);
  return MPI_SUCCESS;
}
int MPI_Send(const void* buf, int count, MPI_Datatype d, int dst, int tag, MPI_Comm c) {
  // always eager: a blocking send returns at once, as it does for the sizes the phase sources were tested with
  MPI_Request r;
  g_rendezvous_ok = false;
  int rc = MPI_Isend(buf, count, d, dst, tag, c, &r);
  g_rendezvous_ok = true;
  MPI_Wait(&r, nullptr);
  return rc;
}
int MPI_Recv(void* buf, int count, MPI_Datatype d, int src, int tag, MPI_Comm c, MPI_Status*) {
  MPI_Request r;
  MPI_Irecv(buf, count, d, src, tag, c, &r);
  return MPI_Wait(&r, nullptr);
}
int MPI_Sendrecv(const void* sb, int sc, MPI_Datatype sd, int dst, int stag, void* rb, int rc, MPI_Datatype rd, int src,
                 int rtag, MPI_Comm c, MPI_Status*) {
  MPI_Request rs, rr;
  MPI_Irecv(rb, rc, rd, src, rtag, c, &rr);
  int e = MPI_Isend(sb, sc, sd, dst, stag, c, &rs);
  MPI_Wait(&rr, nullptr);
  MPI_Wait(&rs, nullptr);
  return e;
}

int MPI_Reduce_local(const void* in, void* io, int n, MPI_Datatype d, MPI_Op op) {
  if (d == MPI_INT) reduce((const int*)in, (int*)io, n, op);
  else if (d == MPI_FLOAT) reduce((const float*)in, (float*)io, n, op);
  else if (d == MPI_DOUBLE) reduce((const double*)in, (double*)io, n, op);
  else return MPI_ERR_ARG;
  return MPI_SUCCESS;
}
int MPI_Op_commutative(MPI_Op, int* c) { *c = 1; return MPI_SUCCESS; }
int MPI_Barrier(MPI_Comm c) { comm_barrier(comm_of(c)); return MPI_SUCCESS; }

// ---- the collectives that the reference's sources call inside their algorithms
int MPI_Allreduce(const void* sendbuf, void* recvbuf, int n, MPI_Datatype d, MPI_Op op, MPI_Comm c) {
  if (sendbuf == MPI_IN_PLACE) { g_fail = true; return MPI_ERR_OTHER; }
  Comm& cm = comm_of(c);
  cm.pub[(size_t)comm_rank(cm)] = sendbuf;
  comm_barrier(cm);
  std::vector<char> acc((size_t)n * type_bytes(d));
  std::memcpy(acc.data(), cm.pub[0], acc.size());
  int rc = MPI_SUCCESS;
  for (size_t q = 1; q < cm.ranks.size() && rc == MPI_SUCCESS; ++q) rc = MPI_Reduce_local(cm.pub[q], acc.data(), n, d, op);
  comm_barrier(cm);                                            // every rank has read every send buffer
  std::memcpy(recvbuf, acc.data(), acc.size());
  return rc;
}
int MPI_Reduce(const void* sendbuf, void* recvbuf, int n, MPI_Datatype d, MPI_Op op, int root, MPI_Comm c) {
  if (sendbuf == MPI_IN_PLACE) { g_fail = true; return MPI_ERR_OTHER; }
  Comm& cm = comm_of(c);
  const int me = comm_rank(cm);
  cm.pub[(size_t)me] = sendbuf;
  comm_barrier(cm);
  int rc = MPI_SUCCESS;
  if (me == root) {
    std::memcpy(recvbuf, cm.pub[0], (size_t)n * type_bytes(d));
    for (size_t q = 1; q < cm.ranks.size() && rc == MPI_SUCCESS; ++q) rc = MPI_Reduce_local(cm.pub[q], recvbuf, n, d, op);
  }
  comm_barrier(cm);
  return rc;
}
int MPI_Bcast(void* buf, int n, MPI_Datatype d, int root, MPI_Comm c) {
  Comm& cm = comm_of(c);
  const int me = comm_rank(cm);
  cm.pub[(size_t)me] = buf;
  comm_barrier(cm);
  if (me != root) std::memcpy(buf, cm.pub[(size_t)root], (size_t)n * type_bytes(d));
  comm_barrier(cm);
  return MPI_SUCCESS;
}
int MPI_Allgatherv(const void* sendbuf, int, MPI_Datatype, void* recvbuf, const int* cnts, const int* displs, MPI_Datatype d,
                   MPI_Comm c) {
  if (sendbuf != MPI_IN_PLACE) { g_fail = true; return MPI_ERR_OTHER; }
  Comm& cm = comm_of(c);
  const int me = comm_rank(cm);
  cm.pub[(size_t)me] = recvbuf;
  comm_barrier(cm);                     // every pointer is published and every own block is in place
  const size_t e = type_bytes(d);
  for (int q = 0; q < (int)cm.ranks.size(); ++q)
    if (q != me)
      std::memcpy((char*)recvbuf + (size_t)displs[q] * e, (const char*)cm.pub[(size_t)q] + (size_t)displs[q] * e, (size_t)cnts[q] * e);
  comm_barrier(cm);                     // nobody's buffer changes while a peer still copies from it
  return MPI_SUCCESS;
}

// ---- derived datatypes (what the recursive-doubling reduce-scatter builds: two blocks of a basic type)
int MPI_Type_create_hindexed(int count, const int* blocklens, const MPI_Aint* displs, MPI_Datatype old, MPI_Datatype* out) {
  if (derived(old)) { g_fail = true; return MPI_ERR_ARG; }
  Segments s;
  for (int i = 0; i < count; ++i) {
    const long n = (long)blocklens[i] * (long)basic_bytes(old);
    if (n > 0) s.seg.push_back({(long)displs[i], n});
    s.bytes += n;
  }
  std::lock_guard<std::mutex> l(g_reg_m);
  g_types.push_back(std::move(s));
  *out = kTypeBase + (int)g_types.size() - 1;
  return MPI_SUCCESS;
}
int MPI_Type_commit(MPI_Datatype*) { return MPI_SUCCESS; }
int MPI_Type_free(MPI_Datatype* d) { *d = MPI_DATATYPE_NULL; return MPI_SUCCESS; }
int MPI_Type_get_extent(MPI_Datatype d, MPI_Aint* lb, MPI_Aint* extent) {
  *lb = 0;
  *extent = (MPI_Aint)type_bytes(d);
  return MPI_SUCCESS;
}
int MPI_Type_get_true_extent(MPI_Datatype d, MPI_Aint* lb, MPI_Aint* extent) { return MPI_Type_get_extent(d, lb, extent); }

// ---- only the reference's own test mains call these; the mains are compiled (some are not behind a macro) but never run
int MPI_Init(int*, char***) { g_fail = true; return MPI_ERR_OTHER; }
int MPI_Finalize() { return MPI_SUCCESS; }
int MPI_Abort(MPI_Comm, int) { g_fail = true; return MPI_ERR_OTHER; }
int MPI_Allgather(const void*, int, MPI_Datatype, void*, int, MPI_Datatype, MPI_Comm) { g_fail = true; return MPI_ERR_OTHER; }
int MPI_Gather(const void*, int, MPI_Datatype, void*, int, MPI_Datatype, int, MPI_Comm) { g_fail = true; return MPI_ERR_OTHER; }
int MPI_Scatter(const void*, int, MPI_Datatype, void*, int, MPI_Datatype, int, MPI_Comm) { g_fail = true; return MPI_ERR_OTHER; }
int MPI_Reduce_scatter(const void*, void*, const int*, MPI_Datatype, MPI_Op, MPI_Comm) { g_fail = true; return MPI_ERR_OTHER; }
int MPI_Reduce_scatter_block(const void*, void*, int, MPI_Datatype, MPI_Op, MPI_Comm) { g_fail = true; return MPI_ERR_OTHER; }
int MPI_Alltoallv(const void*, const int*, const int*, MPI_Datatype, void*, const int*, const int*, MPI_Datatype, MPI_Comm) {
  g_fail = true;
  return MPI_ERR_OTHER;
}
double MPI_Wtime() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

// Thread-per-rank implementation of the calls declared in mpi.h (see there).
#include "mpi.h"

#include <chrono>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <memory>
#include <mutex>
#include <vector>

struct ShimRequest { bool recv; void* buf; size_t bytes; int peer, tag; };
namespace {
struct Message { int src, tag; std::unique_ptr<char[]> data; size_t bytes; };
struct Mailbox { std::mutex m; std::condition_variable cv; std::deque<Message> q; };
int g_n = 0;
std::vector<std::unique_ptr<Mailbox>> g_box;
thread_local int t_rank = -1;
bool g_fail = false;
std::mutex g_bar_m;
std::condition_variable g_bar_cv;
int g_bar_count = 0;
long g_bar_gen = 0;
size_t type_bytes(MPI_Datatype d) { return d == MPI_FLOAT ? 4 : (size_t)d; }
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
  g_fail = false;
  g_bar_count = 0;
}
void shim_set_rank(int r) { t_rank = r; }
int shim_failed() { return g_fail ? 1 : 0; }

int MPI_Comm_rank(MPI_Comm, int* r) { *r = t_rank; return MPI_SUCCESS; }
int MPI_Comm_size(MPI_Comm, int* s) { *s = g_n; return MPI_SUCCESS; }
int MPI_Type_size(MPI_Datatype d, int* s) { *s = (int)type_bytes(d); return MPI_SUCCESS; }

int MPI_Isend(const void* buf, int count, MPI_Datatype d, int dst, int tag, MPI_Comm, MPI_Request* r) {
  *r = new ShimRequest{false, nullptr, 0, dst, tag};
  if (dst < 0 || dst >= g_n) { g_fail = true; return MPI_ERR_ARG; }
  size_t n = (size_t)count * type_bytes(d);
  Message m{t_rank, tag, std::unique_ptr<char[]>(new char[n ? n : 1]), n};
  std::memcpy(m.data.get(), buf, n);
  { std::lock_guard<std::mutex> l(g_box[dst]->m); g_box[dst]->q.push_back(std::move(m)); }
  g_box[dst]->cv.notify_all();
  return MPI_SUCCESS;
}
int MPI_Irecv(void* buf, int count, MPI_Datatype d, int src, int tag, MPI_Comm, MPI_Request* r) {
  *r = new ShimRequest{true, buf, (size_t)count * type_bytes(d), src, tag};
  return MPI_SUCCESS;
}
int MPI_Wait(MPI_Request* rp, MPI_Status*) {
  ShimRequest* r = *rp;
  if (!r) return MPI_SUCCESS;
  if (r->recv) {
    Mailbox& b = *g_box[t_rank];
    std::unique_lock<std::mutex> l(b.m);
    for (;;) {
      bool found = false;
      for (auto it = b.q.begin(); it != b.q.end(); ++it)
        if (it->src == r->peer && it->tag == r->tag) {
          if (it->bytes > r->bytes) g_fail = true;  // truncation
          std::memcpy(r->buf, it->data.get(), it->bytes < r->bytes ? it->bytes : r->bytes);
          b.q.erase(it);
          found = true;
          break;
        }
      if (found) break;
      if (b.cv.wait_for(l, std::chrono::seconds(60)) == std::cv_status::timeout) { g_fail = true; break; }
    }
  }
  delete r;
  *rp = nullptr;
  return MPI_SUCCESS;
}
int MPI_Waitall(int n, MPI_Request* r, MPI_Status*) {
  for (int i = 0; i < n; ++i) MPI_Wait(&r[i], nullptr);
  return MPI_SUCCESS;
}
int MPI_Reduce_local(const void* in, void* io, int n, MPI_Datatype d, MPI_Op op) {
  if (d == MPI_INT) reduce((const int*)in, (int*)io, n, op);
  else if (d == MPI_FLOAT) reduce((const float*)in, (float*)io, n, op);
  else if (d == MPI_DOUBLE) reduce((const double*)in, (double*)io, n, op);
  else return MPI_ERR_ARG;
  return MPI_SUCCESS;
}
int MPI_Barrier(MPI_Comm) {
  std::unique_lock<std::mutex> l(g_bar_m);
  long gen = g_bar_gen;
  if (++g_bar_count == g_n) { g_bar_count = 0; ++g_bar_gen; g_bar_cv.notify_all(); }
  else g_bar_cv.wait(l, [&] { return g_bar_gen != gen; });
  return MPI_SUCCESS;
}
int MPI_Send(const void* buf, int count, MPI_Datatype d, int dst, int tag, MPI_Comm c) {
  MPI_Request r;
  int rc = MPI_Isend(buf, count, d, dst, tag, c, &r);
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
  MPI_Wait(&rs, nullptr);
  MPI_Wait(&rr, nullptr);
  return e;
}
int MPI_Op_commutative(MPI_Op, int* c) { *c = 1; return MPI_SUCCESS; }
int MPI_Allgatherv(const void* sendbuf, int, MPI_Datatype, void* recvbuf, const int* cnts, const int* displs, MPI_Datatype d,
                   MPI_Comm c) {
  if (sendbuf != MPI_IN_PLACE) { g_fail = true; return MPI_ERR_OTHER; }
  static std::vector<char*> bufs;
  { std::lock_guard<std::mutex> l(g_bar_m); if ((int)bufs.size() != g_n) bufs.assign(g_n, nullptr); bufs[t_rank] = (char*)recvbuf; }
  MPI_Barrier(c);                       // every pointer is published and every own block is in place
  const size_t e = type_bytes(d);
  for (int q = 0; q < g_n; ++q)
    if (q != t_rank) std::memcpy((char*)recvbuf + (size_t)displs[q] * e, bufs[q] + (size_t)displs[q] * e, (size_t)cnts[q] * e);
  MPI_Barrier(c);                       // nobody's buffer changes while a peer still copies from it
  return MPI_SUCCESS;
}
int MPI_Init(int*, char***) { g_fail = true; return MPI_ERR_OTHER; }
int MPI_Finalize() { return MPI_SUCCESS; }
int MPI_Abort(MPI_Comm, int) { g_fail = true; return MPI_ERR_OTHER; }
int MPI_Allgather(const void*, int, MPI_Datatype, void*, int, MPI_Datatype, MPI_Comm) { g_fail = true; return MPI_ERR_OTHER; }
int MPI_Allreduce(const void* sendbuf, void* recvbuf, int n, MPI_Datatype d, MPI_Op op, MPI_Comm c) {
  // (the store-and-forward all-to-all-v agrees on its largest block this way)
  if (sendbuf == MPI_IN_PLACE) { g_fail = true; return MPI_ERR_OTHER; }
  static std::vector<const void*> bufs;
  { std::lock_guard<std::mutex> l(g_bar_m); if ((int)bufs.size() != g_n) bufs.assign(g_n, nullptr); bufs[t_rank] = sendbuf; }
  MPI_Barrier(c);
  std::memcpy(recvbuf, bufs[0], (size_t)n * type_bytes(d));
  int rc = MPI_SUCCESS;
  for (int q = 1; q < g_n && rc == MPI_SUCCESS; ++q) rc = MPI_Reduce_local(bufs[q], recvbuf, n, d, op);
  MPI_Barrier(c);
  return rc;
}
int MPI_Reduce(const void*, void*, int, MPI_Datatype, MPI_Op, int, MPI_Comm) { g_fail = true; return MPI_ERR_OTHER; }
int MPI_Bcast(void*, int, MPI_Datatype, int, MPI_Comm) { g_fail = true; return MPI_ERR_OTHER; }
int MPI_Gather(const void*, int, MPI_Datatype, void*, int, MPI_Datatype, int, MPI_Comm) { g_fail = true; return MPI_ERR_OTHER; }
int MPI_Scatter(const void*, int, MPI_Datatype, void*, int, MPI_Datatype, int, MPI_Comm) { g_fail = true; return MPI_ERR_OTHER; }
int MPI_Reduce_scatter(const void*, void*, const int*, MPI_Datatype, MPI_Op, MPI_Comm) { g_fail = true; return MPI_ERR_OTHER; }
int MPI_Alltoallv(const void*, const int*, const int*, MPI_Datatype, void*, const int*, const int*, MPI_Datatype, MPI_Comm) {
  g_fail = true;
  return MPI_ERR_OTHER;
}
double MPI_Wtime() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

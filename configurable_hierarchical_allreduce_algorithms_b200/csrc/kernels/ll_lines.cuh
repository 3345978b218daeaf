// Flagged 16-byte lines {data, flag, data, flag}: the unit of every push-style (LL) kernel here.
// A line is written with one 16-byte store, so payload and flag arrive together; the reader polls
// its own memory until both flag words carry the value of the current launch.
#pragma once
#include "common.cuh"

namespace chb {

__device__ __forceinline__ void st_line(char* p, unsigned d0, unsigned d1, unsigned flag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d0), "r"(flag), "r"(d1), "r"(flag) : "memory");
}
__device__ __forceinline__ void ld_line(const char* p, unsigned& d0, unsigned& f0, unsigned& d1, unsigned& f1) {
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(d0), "=r"(f0), "=r"(d1), "=r"(f1) : "l"(p) : "memory");
}

// 8 payload bytes starting at byte offset `off` of a block of `nbytes` bytes
// (shorter at the tail; missing bytes read as zero).
__device__ __forceinline__ uint2 load_payload(const char* base, long long off, long long nbytes) {
  uint2 v = make_uint2(0u, 0u);
  if (off + 8 <= nbytes && ((reinterpret_cast<unsigned long long>(base + off) & 7ull) == 0ull)) {
    v = *reinterpret_cast<const uint2*>(base + off);
  } else {
    unsigned char* b = reinterpret_cast<unsigned char*>(&v);
    for (int i = 0; i < 8 && off + i < nbytes; ++i) b[i] = (unsigned char)base[off + i];
  }
  return v;
}
__device__ __forceinline__ void store_payload(char* base, long long off, long long nbytes, uint2 v) {
  if (off + 8 <= nbytes && ((reinterpret_cast<unsigned long long>(base + off) & 7ull) == 0ull)) {
    *reinterpret_cast<uint2*>(base + off) = v;
  } else {
    const unsigned char* b = reinterpret_cast<const unsigned char*>(&v);
    for (int i = 0; i < 8 && off + i < nbytes; ++i) base[off + i] = (char)b[i];
  }
}

template <typename T>
__device__ __forceinline__ void payload_to_acc(uint2 v, typename Elem<T>::Acc* a) {
  const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
  for (int i = 0; i < (int)(8 / sizeof(T)); ++i) a[i] = Elem<T>::up(e[i]);
}
template <typename T>
__device__ __forceinline__ void payload_combine(int op, uint2 v, typename Elem<T>::Acc* a) {
  const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
  for (int i = 0; i < (int)(8 / sizeof(T)); ++i) a[i] = combine<typename Elem<T>::Acc>(op, a[i], Elem<T>::up(e[i]));
}
template <typename T>
__device__ __forceinline__ uint2 acc_to_payload(typename Elem<T>::Acc* a, float scale, bool do_scale) {
  uint2 v;
  T* e = reinterpret_cast<T*>(&v);
#pragma unroll
  for (int i = 0; i < (int)(8 / sizeof(T)); ++i) {
    typename Elem<T>::Acc x = a[i];
    if (do_scale) x = (typename Elem<T>::Acc)(x * scale);
    e[i] = Elem<T>::down(x);
  }
  return v;
}

// Bounded poll of one inbox line; false on expiry / abort.
__device__ __forceinline__ bool poll_line(const char* line, unsigned flag, uint2& v, Ctrl* c,
                                          unsigned long long timeout_ns, int rank, long long l, int p) {
  unsigned d0, f0, d1, f1;
  ld_line(line, d0, f0, d1, f1);
  if (f0 != flag || f1 != flag) {
    const unsigned long long t0 = globaltimer_ns();
    unsigned spins = 0;
    for (;;) {
      ld_line(line, d0, f0, d1, f1);
      if (f0 == flag && f1 == flag) break;
      if ((++spins & 31u) == 0u) {
        if (ld_volatile_u32(&c->abort)) return false;
        if (globaltimer_ns() - t0 > timeout_ns) {
          record_timeout(c, ST_TIMEOUT_LL, rank, (int)l, p, flag, f0);
          return false;
        }
      }
    }
  }
  v = make_uint2(d0, d1);
  return true;
}

// Several inbox lines at once: every first read is issued before any flag is looked at, so a group of lines
// that have already arrived costs one memory latency instead of one per line; a line that has not arrived is
// then polled on its own (bounded).  line[i] == nullptr skips slot i and leaves v[i] alone.
constexpr int kLineGroup = 4;
__device__ __forceinline__ bool poll_lines(const char* const (&line)[kLineGroup], const int (&peer)[kLineGroup],
                                           unsigned flag, uint2 (&v)[kLineGroup], Ctrl* c,
                                           unsigned long long timeout_ns, int rank, long long l) {
  unsigned d0[kLineGroup], f0[kLineGroup], d1[kLineGroup], f1[kLineGroup];
#pragma unroll
  for (int i = 0; i < kLineGroup; ++i) {
    d0[i] = d1[i] = 0u;
    f0[i] = f1[i] = flag;
    if (line[i] != nullptr) ld_line(line[i], d0[i], f0[i], d1[i], f1[i]);
  }
#pragma unroll
  for (int i = 0; i < kLineGroup; ++i) {
    if (line[i] == nullptr) continue;
    if (f0[i] == flag && f1[i] == flag) v[i] = make_uint2(d0[i], d1[i]);
    else if (!poll_line(line[i], flag, v[i], c, timeout_ns, rank, l, peer[i])) return false;
  }
  return true;
}

}  // namespace chb

// Device-side building blocks shared by all collective kernels: the world
// descriptor (peer pointers), bounded flag waits, the per-rank grid barrier,
// 16-byte vector load / reduce / store for every element type.
//
// Synchronisation model.  Every rank owns a signal pad (u64 per peer) in its
// symmetric heap.  Peers write monotonically increasing epoch values into
// "their" slot of my pad with st.release.sys; I poll my own (local) pad with
// ld.acquire.sys.  Values are never reset, so a stale flag can only be too
// small, never falsely satisfy a wait.  Every wait is bounded by %globaltimer:
// on expiry the kernel records {code, rank, round, peer, expected, seen} in the
// rank's control block, raises the sticky abort flag and returns; nothing
// traps and nothing spins forever.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../sched/types.h"

namespace chb {

constexpr int kMaxRanks = 16;
constexpr int kSigSlots = 2048;         // u64 slots per signal pad (first kMaxRanks used by programs)
constexpr int kSigBarrierBase = 16;     // slots [16,32): stand-alone barrier kernel
constexpr int kSigNvlsBase = 32;        // slots [32, 2048): NVLS kernels, kMaxRanks per CTA index

enum StatusCode : unsigned {
  ST_OK = 0,
  ST_TIMEOUT_ENTRY = 1,   // peer never finished the previous collective
  ST_TIMEOUT_ROUND = 2,   // peer never completed the round this rank depends on
  ST_TIMEOUT_EXIT = 3,    // peer never finished reading this rank's buffers
  ST_TIMEOUT_GRID = 4,    // a CTA of this rank never reached the rank-local barrier
  ST_TIMEOUT_LL = 5,      // a flagged line never arrived
  ST_TIMEOUT_BARRIER = 6, // stand-alone barrier
  ST_OUT_OF_RANGE = 7,    // a step would touch memory outside its buffer (checked builds only); the step is skipped
};

// Per-rank control block in the rank's own device memory.
struct Ctrl {
  unsigned long long epoch;      // rounds completed by all earlier program launches
  unsigned long long ll_seq;     // number of earlier flagged-line (LL) launches
  unsigned long long bar_seq;    // number of earlier stand-alone / NVLS barriers
  unsigned int bar_count;        // rank-local grid barrier arrivals (0 between launches)
  unsigned int exit_count;       // CTAs that left the current launch
  unsigned int abort;            // sticky: a bounded wait expired
  unsigned int pad0;
  unsigned long long status[8];  // code, rank, round, peer, expected, seen, launches, reserved
};

struct World {
  int P;                 // ranks in the communicator
  int rank0;             // first rank executed by this launch (blockIdx.y adds to it)
  int nlocal;            // ranks executed by this launch (1, or P when emulated on one GPU)
  int reserved;
  unsigned long long timeout_ns;
  unsigned long long* sig[kMaxRanks];   // signal pad of every rank (peer-mapped)
  char* work[kMaxRanks];                // symmetric scratch of every rank (peer-mapped)
  char* ll[kMaxRanks];                  // flagged-line inbox of every rank (peer-mapped)
  Ctrl* ctrl[kMaxRanks];                // control blocks (valid for local ranks only)
  unsigned long long* trace[kMaxRanks]; // optional per-round %globaltimer stamps of local ranks (null = off)
  int trace_rounds;                     // capacity of a trace buffer in rounds
  int reserved2;
};

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_volatile_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_volatile_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void record_timeout(Ctrl* c, unsigned code, int rank, int round, int peer,
                                               unsigned long long expected, unsigned long long seen) {
  if (atomicExch(&c->abort, 1u) == 0u) {
    c->status[1] = (unsigned long long)rank;
    c->status[2] = (unsigned long long)(long long)round;
    c->status[3] = (unsigned long long)(long long)peer;
    c->status[4] = expected;
    c->status[5] = seen;
    __threadfence();
    c->status[0] = code;
  }
}

// Wait until *flag >= target.  Returns false if the wait expired or the rank
// was aborted by another thread.
__device__ __forceinline__ bool wait_flag_ge(const unsigned long long* flag, unsigned long long target,
                                             Ctrl* c, unsigned long long timeout_ns, unsigned code,
                                             int rank, int round, int peer) {
  unsigned long long v = ld_acquire_sys(flag);
  if (v >= target) return true;
  const unsigned long long t0 = globaltimer_ns();
  unsigned spins = 0;
  for (;;) {
    v = ld_acquire_sys(flag);
    if (v >= target) return true;
    if ((++spins & 31u) == 0u) {
      if (ld_volatile_u32(&c->abort)) return false;
      if (globaltimer_ns() - t0 > timeout_ns) {
        record_timeout(c, code, rank, round, peer, target, v);
        return false;
      }
    }
  }
}

// Rank-local barrier across the CTAs of one launch (blockIdx.x dimension).
// `gen` counts the barriers this CTA has passed in the current launch.
// Must be called by all threads of the CTA.  Returns false on abort/expiry.
__device__ __forceinline__ bool rank_barrier(Ctrl* c, unsigned nctas, unsigned& gen,
                                             unsigned long long timeout_ns, int rank, int round) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    int ok = 1;
    if (nctas > 1) {
      __threadfence();
      atomicAdd(&c->bar_count, 1u);
      const unsigned target = (gen + 1u) * nctas;
      unsigned seen = ld_volatile_u32(&c->bar_count);
      if (seen < target) {
        const unsigned long long t0 = globaltimer_ns();
        unsigned spins = 0;
        for (;;) {
          seen = ld_volatile_u32(&c->bar_count);
          if (seen >= target) break;
          if ((++spins & 31u) == 0u) {
            if (ld_volatile_u32(&c->abort)) { ok = 0; break; }
            if (globaltimer_ns() - t0 > timeout_ns) {
              record_timeout(c, ST_TIMEOUT_GRID, rank, round, -1, target, seen);
              ok = 0;
              break;
            }
          }
        }
      }
      __threadfence();
    }
    if (ld_volatile_u32(&c->abort)) ok = 0;
    s_ok = ok;
  }
  __syncthreads();
  ++gen;
  return s_ok != 0;
}

// Bookkeeping at the very end of a launch: the last CTA of the rank to leave
// re-arms the rank barrier and publishes the advanced counters.
template <class F>
__device__ __forceinline__ void rank_exit(Ctrl* c, unsigned nctas, F publish) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    unsigned old = atomicAdd(&c->exit_count, 1u);
    if (old == nctas - 1u) {
      c->bar_count = 0u;
      c->exit_count = 0u;
      publish(c);
      c->status[6] += 1ull;
      __threadfence();
    }
  }
}

// Cross-rank barrier at CTA granularity: CTA c of this rank meets CTA c of every
// peer (all ranks launch the same grid).  `seq` is a per-communicator barrier
// sequence number (Ctrl::bar_seq based); slots are never reset.
// Returns false on expiry.
__device__ __forceinline__ bool cta_barrier(const World& w, Ctrl* c, int rank, unsigned long long seq) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  const int q = threadIdx.x;
  if (q < w.P && q != rank) {
    __threadfence_system();
    const int slot = kSigNvlsBase + (int)blockIdx.x * kMaxRanks;
    st_release_sys(&w.sig[q][slot + rank], seq);
    if (!wait_flag_ge(&w.sig[rank][slot + q], seq, c, w.timeout_ns, ST_TIMEOUT_BARRIER, rank, -2, q)) s_ok = 0;
  }
  __syncthreads();
  return s_ok != 0;
}

// ------------------------------------------------------------------ element types

template <typename T> struct Elem;  // acc type, elements per 16 bytes, conversions

template <> struct Elem<float> {
  using Acc = float; static constexpr int kPerVec = 4;
  __device__ static Acc up(float v) { return v; }
  __device__ static float down(Acc v) { return v; }
};
template <> struct Elem<int32_t> {
  using Acc = int32_t; static constexpr int kPerVec = 4;
  __device__ static Acc up(int32_t v) { return v; }
  __device__ static int32_t down(Acc v) { return v; }
};
template <> struct Elem<double> {
  using Acc = double; static constexpr int kPerVec = 2;
  __device__ static Acc up(double v) { return v; }
  __device__ static double down(Acc v) { return v; }
};
template <> struct Elem<int64_t> {
  using Acc = int64_t; static constexpr int kPerVec = 2;
  __device__ static Acc up(int64_t v) { return v; }
  __device__ static int64_t down(Acc v) { return v; }
};
template <> struct Elem<uint8_t> {
  using Acc = uint32_t; static constexpr int kPerVec = 16;
  __device__ static Acc up(uint8_t v) { return v; }
  __device__ static uint8_t down(Acc v) { return (uint8_t)v; }
};
template <> struct Elem<__nv_bfloat16> {
  using Acc = float; static constexpr int kPerVec = 8;
  __device__ static Acc up(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 down(Acc v) { return __float2bfloat16_rn(v); }
};
template <> struct Elem<__half> {
  using Acc = float; static constexpr int kPerVec = 8;
  __device__ static Acc up(__half v) { return __half2float(v); }
  __device__ static __half down(Acc v) { return __float2half_rn(v); }
};

template <typename A>
__device__ __forceinline__ A combine(int op, A a, A b) {
  switch (op) {
    case OP_SUM: return a + b;
    case OP_MAX: return a > b ? a : b;
    case OP_MIN: return a < b ? a : b;
    default: return a * b;
  }
}

union alignas(16) Vec16 {
  uint4 u;
  float f[4];
  int32_t i[4];
  double d[2];
  int64_t l[2];
  uint8_t b[16];
  __nv_bfloat16 h[8];
  __half g[8];
};

// 16-byte load that bypasses L1 (peer data must come from the owner's L2).
__device__ __forceinline__ uint4 ld16_cg(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void st16(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }
// 256-bit global accesses (sm_100): half the requests of the 128-bit form for the same bytes.
// p must be 32-byte aligned.  Loads bypass L1 like ld16_cg (peers write this memory).
__device__ __forceinline__ void ld32_cg(const void* p, uint4& lo, uint4& hi) {
  unsigned long long a, b, c, d;
  asm volatile("ld.global.cg.v4.b64 {%0,%1,%2,%3}, [%4];" : "=l"(a), "=l"(b), "=l"(c), "=l"(d) : "l"(p) : "memory");
  lo = make_uint4((unsigned)a, (unsigned)(a >> 32), (unsigned)b, (unsigned)(b >> 32));
  hi = make_uint4((unsigned)c, (unsigned)(c >> 32), (unsigned)d, (unsigned)(d >> 32));
}
__device__ __forceinline__ void st32(void* p, const uint4& lo, const uint4& hi) {
  const unsigned long long a = (unsigned long long)lo.x | ((unsigned long long)lo.y << 32);
  const unsigned long long b = (unsigned long long)lo.z | ((unsigned long long)lo.w << 32);
  const unsigned long long c = (unsigned long long)hi.x | ((unsigned long long)hi.y << 32);
  const unsigned long long d = (unsigned long long)hi.z | ((unsigned long long)hi.w << 32);
  asm volatile("st.global.v4.b64 [%0], {%1,%2,%3,%4};" ::"l"(p), "l"(a), "l"(b), "l"(c), "l"(d) : "memory");
}

template <typename T>
__device__ __forceinline__ void vec_to_acc(const uint4& v, typename Elem<T>::Acc* a) {
  const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
  for (int i = 0; i < Elem<T>::kPerVec; ++i) a[i] = Elem<T>::up(e[i]);
}
template <typename T>
__device__ __forceinline__ void vec_combine(int op, const uint4& v, typename Elem<T>::Acc* a) {
  const T* e = reinterpret_cast<const T*>(&v);
  if (op == OP_SUM) {
#pragma unroll
    for (int i = 0; i < Elem<T>::kPerVec; ++i) a[i] = a[i] + Elem<T>::up(e[i]);
  } else {
#pragma unroll
    for (int i = 0; i < Elem<T>::kPerVec; ++i) a[i] = combine<typename Elem<T>::Acc>(op, a[i], Elem<T>::up(e[i]));
  }
}
template <typename T>
__device__ __forceinline__ uint4 acc_to_vec(const typename Elem<T>::Acc* a) {
  uint4 v;
  T* e = reinterpret_cast<T*>(&v);
#pragma unroll
  for (int i = 0; i < Elem<T>::kPerVec; ++i) e[i] = Elem<T>::down(a[i]);
  return v;
}
template <typename T>
__device__ __forceinline__ void acc_scale(typename Elem<T>::Acc* a, float s) {
#pragma unroll
  for (int i = 0; i < Elem<T>::kPerVec; ++i) a[i] = (typename Elem<T>::Acc)(a[i] * s);
}

}  // namespace chb

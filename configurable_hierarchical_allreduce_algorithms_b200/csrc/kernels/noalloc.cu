// Allocation-free variant of the flagged-line one-shot allreduce for P ranks
// that share one GPU (see api/chb_noalloc.h for the contract and for who needs
// it).  Same algorithm as ll.cu — every rank pushes {data, flag, data, flag}
// lines into its peers' inboxes and polls its own inbox, sums run in rank
// order — but the inboxes and control words live in a fixed array that is part
// of the library image instead of a communicator's heap.
#include <cstdio>
#include <cstring>

#include "../api/chb.h"
#include "../api/chb_noalloc.h"
#include "common.cuh"

namespace chb {
namespace {

constexpr int kNaThreads = 256;
constexpr int kNaCtrlStride = 128;                                         // bytes per rank
constexpr int kNaCtrlBytes = CHB_NOALLOC_MAX_RANKS * kNaCtrlStride;        // 1 KiB
constexpr long long kNaLines = CHB_NOALLOC_MAX_BYTES / 8;                  // lines per (dst, src) pair
constexpr long long kNaInboxPerRank = (long long)CHB_NOALLOC_MAX_RANKS * kNaLines * 16;
constexpr long long kNaScratchBytes = kNaCtrlBytes + (long long)CHB_NOALLOC_MAX_RANKS * kNaInboxPerRank;
constexpr unsigned kNaFlag = 1u;  // the used lines are cleared before every launch, so one flag value is enough
static_assert(sizeof(Ctrl) <= kNaCtrlStride, "control block must fit its slot");

// The only working memory of this entry point.  In host code this name is a
// host-side stand-in, not a device address: the address the kernel uses comes
// from cudaGetSymbolAddress (scratch_for_current_device below).
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNaScratchBytes];

struct NaIo {
  const char* in[CHB_NOALLOC_MAX_RANKS];
  char* out[CHB_NOALLOC_MAX_RANKS];
};

__device__ __forceinline__ void na_st_line(unsigned char* p, unsigned d0, unsigned d1) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d0), "r"(kNaFlag), "r"(d1), "r"(kNaFlag) : "memory");
}
__device__ __forceinline__ void na_ld_line(const unsigned char* p, unsigned& d0, unsigned& f0, unsigned& d1, unsigned& f1) {
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(d0), "=r"(f0), "=r"(d1), "=r"(f1) : "l"(p) : "memory");
}
__device__ __forceinline__ uint2 na_load(const char* base, long long off, long long nbytes) {
  uint2 v = make_uint2(0u, 0u);
  if (off + 8 <= nbytes) {
    v = *reinterpret_cast<const uint2*>(base + off);
  } else {
    unsigned char* b = reinterpret_cast<unsigned char*>(&v);
    for (int i = 0; i < 8 && off + i < nbytes; ++i) b[i] = (unsigned char)base[off + i];
  }
  return v;
}
__device__ __forceinline__ void na_store(char* base, long long off, long long nbytes, uint2 v) {
  if (off + 8 <= nbytes) {
    *reinterpret_cast<uint2*>(base + off) = v;
  } else {
    const unsigned char* b = reinterpret_cast<const unsigned char*>(&v);
    for (int i = 0; i < 8 && off + i < nbytes; ++i) base[off + i] = (char)b[i];
  }
}

// grid = (ctas per rank, P); one cooperative launch runs all ranks.
template <typename T>
__global__ void __launch_bounds__(kNaThreads)
noalloc_allreduce_kernel(unsigned char* scratch, NaIo io, int P, long long nbytes, int op, float scale,
                         unsigned long long timeout_ns) {
  using Acc = typename Elem<T>::Acc;
  constexpr int PE = (int)(8 / sizeof(T));
  const int rank = (int)blockIdx.y;
  Ctrl* c = reinterpret_cast<Ctrl*>(scratch + rank * kNaCtrlStride);
  unsigned char* inbox = scratch + kNaCtrlBytes;
  const long long nlines = (nbytes + 7) / 8;
  const long long TT = (long long)gridDim.x * blockDim.x;
  const long long l0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const char* in = io.in[rank];
  char* out = io.out[rank];
  // push my lines into every peer's inbox: slot [dst][src = me][line]
  for (long long l = l0; l < nlines; l += TT) {
    const uint2 mine = na_load(in, l * 8, nbytes);
    for (int i = 1; i < P; ++i) {
      const int p = (rank + i) % P;
      na_st_line(inbox + (long long)p * kNaInboxPerRank + ((long long)rank * kNaLines + l) * 16, mine.x, mine.y);
    }
  }
  // collect, combining in rank order so that all ranks get identical bits
  for (long long l = l0; l < nlines; l += TT) {
    const uint2 mine = na_load(in, l * 8, nbytes);
    Acc a[PE];
    bool failed = false;
    for (int p = 0; p < P; ++p) {
      uint2 v = mine;
      if (p != rank) {
        const unsigned char* line = inbox + (long long)rank * kNaInboxPerRank + ((long long)p * kNaLines + l) * 16;
        unsigned d0, f0, d1, f1;
        na_ld_line(line, d0, f0, d1, f1);
        if (f0 != kNaFlag || f1 != kNaFlag) {
          const unsigned long long t0 = globaltimer_ns();
          unsigned spins = 0;
          for (;;) {
            na_ld_line(line, d0, f0, d1, f1);
            if (f0 == kNaFlag && f1 == kNaFlag) break;
            if ((++spins & 31u) == 0u) {
              if (ld_volatile_u32(&c->abort)) { failed = true; break; }
              if (globaltimer_ns() - t0 > timeout_ns) {
                record_timeout(c, ST_TIMEOUT_LL, rank, (int)l, p, kNaFlag, f0);
                failed = true;
                break;
              }
            }
          }
        }
        if (failed) break;
        v = make_uint2(d0, d1);
      }
      const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
      for (int i = 0; i < PE; ++i) a[i] = (p == 0) ? Elem<T>::up(e[i]) : combine<Acc>(op, a[i], Elem<T>::up(e[i]));
    }
    if (failed) break;
    uint2 r;
    T* e = reinterpret_cast<T*>(&r);
#pragma unroll
    for (int i = 0; i < PE; ++i) e[i] = Elem<T>::down(scale != 1.0f ? (Acc)(a[i] * scale) : a[i]);
    na_store(out, l * 8, nbytes, r);
  }
}

typedef void (*NaFn)(unsigned char*, NaIo, int, long long, int, float, unsigned long long);
NaFn pick(int dtype) {
  switch (dtype) {
    case DT_F32: return noalloc_allreduce_kernel<float>;
    case DT_BF16: return noalloc_allreduce_kernel<__nv_bfloat16>;
    case DT_F16: return noalloc_allreduce_kernel<__half>;
    case DT_I32: return noalloc_allreduce_kernel<int32_t>;
    case DT_F64: return noalloc_allreduce_kernel<double>;
    case DT_I64: return noalloc_allreduce_kernel<int64_t>;
    case DT_U8: return noalloc_allreduce_kernel<uint8_t>;
  }
  return nullptr;
}

// Device address of the scratch array on the current device; looked up once
// per device (the lookup is the set-up step that must not happen under stream
// capture).  Returns null and fills msg on failure.
constexpr int kMaxDevices = 64;
unsigned char* g_scratch_addr[kMaxDevices] = {nullptr};

unsigned char* scratch_for_current_device(char* msg, size_t msglen) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    std::snprintf(msg, msglen, "cannot identify the current CUDA device: %s", cudaGetErrorString(e));
    return nullptr;
  }
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) {
      std::snprintf(msg, msglen, "cudaGetSymbolAddress(scratch) failed on device %d: %s", dev, cudaGetErrorString(e));
      return nullptr;
    }
    g_scratch_addr[dev] = static_cast<unsigned char*>(p);
  }
  return g_scratch_addr[dev];
}

}  // namespace
}  // namespace chb

using namespace chb;

extern "C" {

int chb_allreduce_oneshot_noalloc(int P, int dtype, int op, const void* const* in, void* const* out,
                                  int64_t count, float scale, cudaStream_t stream, char* err, int errlen) {
  char msg[256] = {0};
  auto fail = [&](int code) {
    if (err && errlen > 0) std::snprintf(err, (size_t)errlen, "%s", msg);
    return code;
  };
  if (!in || !out) { std::snprintf(msg, sizeof msg, "in / out pointer tables are null"); return fail(CHB_ERR_ARG); }
  if (P < 1 || P > CHB_NOALLOC_MAX_RANKS) {
    std::snprintf(msg, sizeof msg, "P = %d is outside 1..%d, the capacity of the fixed scratch array", P, CHB_NOALLOC_MAX_RANKS);
    return fail(CHB_ERR_COUNT);
  }
  NaFn fn = pick(dtype);
  if (!fn) { std::snprintf(msg, sizeof msg, "unknown dtype %d", dtype); return fail(CHB_ERR_ARG); }
  if (op < OP_SUM || op > OP_PROD) { std::snprintf(msg, sizeof msg, "unknown reduction %d", op); return fail(CHB_ERR_OP); }
  // the range test comes before the multiplication: a huge count must not wrap around to a small size
  const long long max_count = CHB_NOALLOC_MAX_BYTES / dtype_size(dtype);
  const long long nbytes = (count < 0 || count > max_count) ? -1 : (long long)count * dtype_size(dtype);
  if (nbytes < 0) {
    std::snprintf(msg, sizeof msg, "%lld elements per rank exceed the fixed scratch capacity of %d bytes "
                  "(%lld elements of this type); use a communicator for larger messages",
                  (long long)count, CHB_NOALLOC_MAX_BYTES, max_count);
    return fail(CHB_ERR_COUNT);
  }
  NaIo io{};
  for (int r = 0; r < P; ++r) {
    if (!in[r] || !out[r] || ((((uintptr_t)in[r]) | ((uintptr_t)out[r])) & 7u)) {
      std::snprintf(msg, sizeof msg, "buffer of rank %d is null or not 8-byte aligned", r);
      return fail(CHB_ERR_ARG);
    }
    io.in[r] = (const char*)in[r];
    io.out[r] = (char*)out[r];
  }
  if (nbytes == 0) return CHB_SUCCESS;
  unsigned char* scratch = scratch_for_current_device(msg, sizeof msg);
  if (!scratch) return fail(CHB_ERR_CUDA);
  // The array still holds the previous call's flags and status: clear, in stream order, the control
  // words and exactly the lines this call uses.  The inbox is a table of (destination, source) rows of
  // kNaLines lines each; the first nlines lines of the rows of the P destinations are one 2-D fill.
  const long long nlines = (nbytes + 7) / 8;
  cudaError_t e = cudaMemsetAsync(scratch, 0, (size_t)kNaCtrlBytes, stream);
  if (e == cudaSuccess)
    e = cudaMemset2DAsync(scratch + kNaCtrlBytes, (size_t)(kNaLines * 16), 0, (size_t)(nlines * 16),
                          (size_t)P * CHB_NOALLOC_MAX_RANKS, stream);
  if (e != cudaSuccess) { std::snprintf(msg, sizeof msg, "clearing the scratch array failed: %s", cudaGetErrorString(e)); return fail(CHB_ERR_CUDA); }
  int nctas = (int)((nlines + kNaThreads - 1) / kNaThreads);
  if (nctas > 4) nctas = 4;
  dim3 grid((unsigned)nctas, (unsigned)P, 1), block(kNaThreads, 1, 1);
  long long nb = nbytes;
  unsigned long long timeout_ns = 2000000000ull;
  void* args[] = {&scratch, &io, &P, &nb, &op, &scale, &timeout_ns};
  // all ranks wait for each other's lines, so they must be co-resident
  e = cudaLaunchCooperativeKernel((const void*)fn, grid, block, args, 0, stream);
  if (e != cudaSuccess) { std::snprintf(msg, sizeof msg, "launch failed: %s", cudaGetErrorString(e)); return fail(CHB_ERR_CUDA); }
  return CHB_SUCCESS;
}

int chb_noalloc_status(cudaStream_t stream) {
  char msg[128];
  unsigned char* scratch = scratch_for_current_device(msg, sizeof msg);
  if (!scratch) return CHB_ERR_CUDA;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return CHB_ERR_CUDA;
  unsigned char host[kNaCtrlBytes];
  if (cudaMemcpy(host, scratch, sizeof host, cudaMemcpyDeviceToHost) != cudaSuccess) return CHB_ERR_CUDA;
  for (int r = 0; r < CHB_NOALLOC_MAX_RANKS; ++r) {
    Ctrl c;
    std::memcpy(&c, host + r * kNaCtrlStride, sizeof c);
    if (c.abort || c.status[0]) return CHB_ERR_TIMEOUT;
  }
  return CHB_SUCCESS;
}

}  // extern "C"

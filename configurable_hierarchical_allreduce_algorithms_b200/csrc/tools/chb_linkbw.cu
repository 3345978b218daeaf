// chb_linkbw: what one GPU can move over NVLink with its own SMs, the denominator of every roofline
// that the program kernels are held against.  Two GPUs in one process with peer access: a plain copy
// kernel reads the peer's memory (pull), writes it (push) or copies locally, with one GPU active or
// both at once (every collective keeps both directions of a link busy, so "both" is the figure that
// applies to them).  Usage:  chb_linkbw [MiB per copy = 512] [iterations = 4]
// Prints one line per (access width, mode, directions, CTAs): GB/s per direction.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>

#define CK(x)                                                                      \
  do {                                                                             \
    cudaError_t e_ = (x);                                                          \
    if (e_ != cudaSuccess) {                                                       \
      std::fprintf(stderr, "%s: %s (line %d)\n", #x, cudaGetErrorString(e_), __LINE__); \
      std::exit(1);                                                                \
    }                                                                              \
  } while (0)

namespace {

template <int W>   // bytes per access: 16 or 32
__global__ void __launch_bounds__(512) copy_kernel(const char* __restrict__ src, char* __restrict__ dst, long long nbytes) {
  const long long nvec = nbytes / W;
  const long long T = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  constexpr int U = 4;   // loads in flight per thread
  for (; i + (U - 1) * T < nvec; i += U * T) {
    if (W == 16) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v[u].x), "=r"(v[u].y), "=r"(v[u].z), "=r"(v[u].w) : "l"(src + (i + u * T) * 16));
#pragma unroll
      for (int u = 0; u < U; ++u)
        asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst + (i + u * T) * 16), "r"(v[u].x), "r"(v[u].y), "r"(v[u].z), "r"(v[u].w) : "memory");
    } else {
      unsigned long long v[U][4];
#pragma unroll
      for (int u = 0; u < U; ++u)
        asm volatile("ld.global.cg.v4.b64 {%0,%1,%2,%3}, [%4];" : "=l"(v[u][0]), "=l"(v[u][1]), "=l"(v[u][2]), "=l"(v[u][3]) : "l"(src + (i + u * T) * 32));
#pragma unroll
      for (int u = 0; u < U; ++u)
        asm volatile("st.global.v4.b64 [%0], {%1,%2,%3,%4};" ::"l"(dst + (i + u * T) * 32), "l"(v[u][0]), "l"(v[u][1]), "l"(v[u][2]), "l"(v[u][3]) : "memory");
    }
  }
  for (; i < nvec; i += T)
    for (int q = 0; q < W / 16; ++q)
      reinterpret_cast<uint4*>(dst + i * W)[q] = reinterpret_cast<const uint4*>(src + i * W)[q];
}

}  // namespace

int main(int argc, char** argv) {
  const long long mib = argc > 1 ? std::atoll(argv[1]) : 512;
  const int iters = argc > 2 ? std::atoi(argv[2]) : 4;
  if (mib < 1 || mib > 4096 || iters < 2 || iters > 100) {
    std::fprintf(stderr, "usage: chb_linkbw [MiB per copy, 1..4096] [iterations, 2..100]\n");
    return 2;
  }
  int n = 0;
  CK(cudaGetDeviceCount(&n));
  if (n < 2) {
    std::printf("chb_linkbw: needs two GPUs, found %d\n", n);
    return 0;
  }
  const long long B = mib << 20;
  char *a[2], *b[2];
  cudaStream_t s[2];
  cudaEvent_t e0[2], e1[2];
  for (int d = 0; d < 2; ++d) {
    CK(cudaSetDevice(d));
    int can = 0;
    CK(cudaDeviceCanAccessPeer(&can, d, 1 - d));
    if (!can) {
      std::printf("chb_linkbw: GPU %d cannot access GPU %d\n", d, 1 - d);
      return 0;
    }
    CK(cudaDeviceEnablePeerAccess(1 - d, 0));
    CK(cudaMalloc(&a[d], B));
    CK(cudaMalloc(&b[d], B));
    CK(cudaMemset(a[d], 1, B));
    CK(cudaMemset(b[d], 2, B));
    CK(cudaStreamCreate(&s[d]));
    CK(cudaEventCreate(&e0[d]));
    CK(cudaEventCreate(&e1[d]));
  }
  for (int d = 0; d < 2; ++d) {
    CK(cudaSetDevice(d));
    CK(cudaDeviceSynchronize());
  }
  const int ctas[] = {32, 64, 148, 296};
  const char* names[] = {"pull (read peer)", "push (write peer)", "local copy"};
  std::printf("width_bytes,mode,directions,ctas,GBps_gpu0,GBps_gpu1\n");
  for (int W : {16, 32})
    for (int mode = 0; mode < 3; ++mode)
      for (int both = 0; both < 2; ++both)
        for (int nc : ctas) {
          float best[2] = {1e30f, 1e30f};
          for (int it = 0; it < iters; ++it) {
            for (int d = 0; d < (both ? 2 : 1); ++d) {
              CK(cudaSetDevice(d));
              const char* src = mode == 0 ? a[1 - d] : a[d];
              char* dst = mode == 1 ? b[1 - d] : b[d];
              CK(cudaEventRecord(e0[d], s[d]));
              if (W == 16) copy_kernel<16><<<nc, 512, 0, s[d]>>>(src, dst, B);
              else copy_kernel<32><<<nc, 512, 0, s[d]>>>(src, dst, B);
              CK(cudaEventRecord(e1[d], s[d]));
            }
            for (int d = 0; d < (both ? 2 : 1); ++d) {
              CK(cudaSetDevice(d));
              CK(cudaStreamSynchronize(s[d]));
              float ms = 0.f;
              CK(cudaEventElapsedTime(&ms, e0[d], e1[d]));
              if (it > 0 && ms < best[d]) best[d] = ms;   // the first pass is the warm-up
            }
          }
          std::printf("%d,%s,%s,%d,%.1f,", W, names[mode], both ? "both" : "one", nc, B / (best[0] * 1e-3) / 1e9);
          if (both) std::printf("%.1f\n", B / (best[1] * 1e-3) / 1e9);
          else std::printf("\n");
        }
  for (int d = 0; d < 2; ++d) {
    CK(cudaSetDevice(d));
    CK(cudaFree(a[d]));
    CK(cudaFree(b[d]));
  }
  return 0;
}

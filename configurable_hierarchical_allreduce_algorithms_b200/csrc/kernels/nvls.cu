// In-switch (NVLS) collectives: multimem.ld_reduce pulls the sum of one
// address over all GPUs of the multicast object out of the NVSwitch,
// multimem.st writes one value to all of them.
//
//   allreduce (two-shot) : rank r reduces slice r and broadcasts it
//   allreduce (one-shot) : every rank reduces the whole vector for itself
//   reduce-scatter       : rank r reduces block r into a local buffer
//   allgather            : rank r broadcasts its block into everybody's output
//
// These are switch-side multicast operations on plain global addresses, not
// TMA cluster multicast.  The buffers must live in the symmetric heap (the
// multicast alias covers the heap only).  Each CTA pairs up with the CTA of
// the same index on every peer for the entry / exit barriers, so all ranks
// launch the same grid.  No reference counterpart: the reference reduces on
// the host after MPI receives
// (testing/custom_implementations/work_dir/all_reduce/all_reduce_radix_batch.cpp:353-364).
#include <cstdio>

#include "../api/chb.h"
#include "../symm/comm.h"
#include "common.cuh"

namespace chb {

constexpr int kNvlsThreads = 512;
constexpr int kNvlsMaxCtas = (kSigSlots - kSigNvlsBase) / kMaxRanks;
enum { NV_AR2 = 0, NV_RS = 1, NV_AG = 2, NV_AR1 = 3 };

template <typename T> struct MM;
template <> struct MM<float> {
  __device__ static uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  __device__ static void st(void* p, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};
template <> struct MM<__nv_bfloat16> {
  __device__ static uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  __device__ static void st(void* p, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};
template <> struct MM<__half> {
  __device__ static uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  __device__ static void st(void* p, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
};

template <typename T>
__device__ __forceinline__ uint4 scale_vec(uint4 v, float s) {
  typename Elem<T>::Acc a[Elem<T>::kPerVec];
  vec_to_acc<T>(v, a);
  acc_scale<T>(a, s);
  return acc_to_vec<T>(a);
}

// mc_in / mc_out: multicast addresses; loc_in / loc_out: this rank's own addresses.
// nvec: 16-byte vectors in the whole vector (AR) or in one block (RS, AG).
template <typename T, int MODE>
__global__ void __launch_bounds__(kNvlsThreads, 1)
nvls_kernel(World w, const char* mc_in, char* mc_out, const char* loc_in, char* loc_out, long long nvec, float scale) {
  const int rank = w.rank0;
  const int P = w.P;
  Ctrl* c = w.ctrl[rank];
  __shared__ unsigned long long s_seq;
  if (threadIdx.x == 0) s_seq = ld_volatile_u64(&c->bar_seq);
  __syncthreads();
  const unsigned long long seq = s_seq;
  const bool do_scale = scale != 1.0f;
  const long long TT = (long long)gridDim.x * blockDim.x;
  const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  bool ok = !ld_volatile_u32(&c->abort);
  // every peer has entered: its inputs are final, its outputs may be overwritten
  ok = ok && cta_barrier(w, c, rank, seq + 1ull);
  if (ok) {
    // U independent 16-byte operations per thread keep enough bytes in flight
    // to cover the switch round trip
    constexpr int U = 8;
    long long lo = 0, hi = nvec;        // range of vectors this rank works on
    long long src_base = 0;             // added to the index on the source side
    if (MODE == NV_AR2) { lo = nvec * rank / P; hi = nvec * (rank + 1) / P; }
    if (MODE == NV_RS || MODE == NV_AG) src_base = nvec * rank;
    for (long long i0 = lo + g; i0 < hi; i0 += TT * U) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + (long long)u * TT;
        if (i < hi) {
          if (MODE == NV_AG) v[u] = ld16_cg(loc_in + i * 16);
          else if (MODE == NV_RS) v[u] = MM<T>::ld_reduce(mc_in + (src_base + i) * 16);
          else v[u] = MM<T>::ld_reduce(mc_in + i * 16);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + (long long)u * TT;
        if (i < hi) {
          if (MODE != NV_AG && do_scale) v[u] = scale_vec<T>(v[u], scale);
          if (MODE == NV_AR2) MM<T>::st(mc_out + i * 16, v[u]);
          else if (MODE == NV_AG) MM<T>::st(mc_out + (src_base + i) * 16, v[u]);
          else st16(loc_out + i * 16, v[u]);
        }
      }
    }
  }
  // all my reads of the peers' inputs and my multicast stores are done
  if (ok) cta_barrier(w, c, rank, seq + 2ull);
  rank_exit(c, gridDim.x, [&](Ctrl* cc) { cc->bar_seq = seq + 2ull; });
}

typedef void (*NvlsFn)(World, const char*, char*, const char*, char*, long long, float);

template <int MODE>
static NvlsFn pick_nvls(int dtype) {
  switch (dtype) {
    case DT_F32: return nvls_kernel<float, MODE>;
    case DT_BF16: return nvls_kernel<__nv_bfloat16, MODE>;
    case DT_F16: return nvls_kernel<__half, MODE>;
  }
  return nullptr;
}

}  // namespace chb

using namespace chb;

extern "C" {

// mode: 0 two-shot allreduce, 1 reduce-scatter, 2 allgather, 3 one-shot allreduce.
// count: vector length (allreduce) or elements per rank (reduce-scatter, allgather).
// in / out are this rank's buffers inside the symmetric heap (out of a
// reduce-scatter or one-shot allreduce may be any local buffer).  Sum only.
int chb_nvls_collective(chb_comm* c, int mode, int dtype, const void* in, void* out, long long count,
                        float scale, int nctas, cudaStream_t stream) {
  if (!c || !in || !out || count < 0) return CHB_ERR_ARG;
  if (!c->mc_heap || c->nlocal != 1) { c->last_error = "communicator has no multicast alias"; return CHB_ERR_UNSUPPORTED; }
  NvlsFn fn = mode == NV_AR2 ? pick_nvls<NV_AR2>(dtype) : mode == NV_RS ? pick_nvls<NV_RS>(dtype)
            : mode == NV_AG ? pick_nvls<NV_AG>(dtype) : mode == NV_AR1 ? pick_nvls<NV_AR1>(dtype) : nullptr;
  if (!fn) { c->last_error = "multimem kernels cover f32 / bf16 / f16 sums"; return CHB_ERR_OP; }
  const long long bytes = count * (long long)dtype_size(dtype);
  if (bytes % 16) { c->last_error = "multimem kernels need a multiple of 16 bytes per block"; return CHB_ERR_COUNT; }
  const bool need_in_sym = mode != NV_AG, need_out_sym = (mode == NV_AR2 || mode == NV_AG);
  const char* mc_in = nullptr;
  char* mc_out = nullptr;
  if (need_in_sym) {
    char* t = c->translate(in, c->rank, c->rank);
    if (!t || ((uintptr_t)in & 15)) { c->last_error = "input must be a 16-byte aligned symmetric buffer"; return CHB_ERR_ARG; }
    mc_in = c->mc_heap + ((const char*)in - c->heap[c->rank]);
  }
  if (need_out_sym) {
    char* t = c->translate(out, c->rank, c->rank);
    if (!t || ((uintptr_t)out & 15)) { c->last_error = "output must be a 16-byte aligned symmetric buffer"; return CHB_ERR_ARG; }
    mc_out = c->mc_heap + ((char*)out - c->heap[c->rank]);
  }
  if ((((uintptr_t)in) | ((uintptr_t)out)) & 15) { c->last_error = "buffers must be 16-byte aligned"; return CHB_ERR_ARG; }
  const long long nvec = bytes / 16;
  if (nctas <= 0) {
    long long work = (mode == NV_AR2) ? nvec / c->P : nvec;
    nctas = (int)((work + kNvlsThreads * 4 - 1) / (kNvlsThreads * 4));
    if (nctas > 64) nctas = 64;
  }
  if (nctas > kNvlsMaxCtas) nctas = kNvlsMaxCtas;
  if (nctas > c->max_ctas) nctas = c->max_ctas;
  if (nctas < 1) nctas = 1;
  World w = c->world;
  const char* loc_in = (const char*)in;
  char* loc_out = (char*)out;
  long long nv = nvec;
  void* args[] = {&w, &mc_in, &mc_out, &loc_in, &loc_out, &nv, &scale};
  dim3 grid((unsigned)nctas, 1, 1), block(kNvlsThreads, 1, 1);
  cudaError_t e = cudaLaunchKernel((const void*)fn, grid, block, args, 0, stream);
  if (e != cudaSuccess) { c->last_error = std::string("nvls launch failed: ") + cudaGetErrorString(e); return CHB_ERR_CUDA; }
  return CHB_SUCCESS;
}

}  // extern "C"

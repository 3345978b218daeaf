// Reduce-scatter with a block-scaled fp8 (e4m3) wire format: every rank
// quantises the blocks it owes its peers into 128-element groups with one fp32
// scale each (1 byte per element + 4 bytes per 128 on the wire instead of 2 or
// 4 bytes per element), peers pull their block, dequantise and accumulate in
// fp32.  Quantisation, exchange, accumulation, output scale and cast are one
// kernel; a rank's own block never goes through fp8.
// No reference counterpart (the reference moves MPI_INT / MPI_DOUBLE as is).
#include <cuda_fp8.h>

#include <cstdio>

#include "../api/chb.h"
#include "../symm/comm.h"
#include "common.cuh"

namespace chb {

constexpr int kFp8Threads = 512;
constexpr int kGroup = 128;  // elements per scale

struct Fp8Io {
  const char* in[kMaxRanks];
  char* out[kMaxRanks];
};

template <typename T> __device__ __forceinline__ void load4(const T* p, float* x);
template <> __device__ __forceinline__ void load4<float>(const float* p, float* x) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float* x) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) x[i] = __bfloat162float(e[i]);
}
template <typename T> __device__ __forceinline__ void store4(T* p, const float* x);
template <> __device__ __forceinline__ void store4<float>(float* p, const float* x) {
  *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float* x) {
  __nv_bfloat16 e[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) e[i] = __float2bfloat16_rn(x[i]);
  *reinterpret_cast<uint2*>(p) = *reinterpret_cast<uint2*>(e);
}

__device__ __forceinline__ float2 fp8x2_to_float2(unsigned short b) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)b, __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

// n: elements per block, a multiple of 128.  Wire layout in each rank's
// scratch: P*n fp8 bytes, then P*n/128 fp32 scales.
template <typename T>
__global__ void __launch_bounds__(kFp8Threads, 1)
fp8_rs_kernel(World w, Fp8Io io, long long n, float out_scale) {
  const int rank = w.rank0 + (int)blockIdx.y;
  const int P = w.P;
  const unsigned nct = gridDim.x;
  Ctrl* c = w.ctrl[rank];
  __shared__ unsigned long long s_seq;
  if (threadIdx.x == 0) s_seq = ld_volatile_u64(&c->bar_seq);
  __syncthreads();
  const unsigned long long seq = s_seq;
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)nct * blockDim.x) >> 5;
  const long long gpb = n / kGroup;                 // groups per block
  const T* in = reinterpret_cast<const T*>(io.in[rank]);
  unsigned char* wire = reinterpret_cast<unsigned char*>(w.work[rank]);
  float* scales = reinterpret_cast<float*>(wire + (long long)P * n);
  bool ok = !ld_volatile_u32(&c->abort);
  // The wire buffer shares the scratch with step programs, whose peers may
  // still be reading it: wait until every peer has left its last program launch.
  {
    __shared__ int s_entry_ok;
    if (threadIdx.x == 0) s_entry_ok = 1;
    __syncthreads();
    if ((int)threadIdx.x < P && (int)threadIdx.x != rank)
      if (!wait_flag_ge(&w.sig[rank][threadIdx.x], ld_volatile_u64(&c->epoch), c, w.timeout_ns, ST_TIMEOUT_ENTRY,
                        rank, -1, (int)threadIdx.x))
        s_entry_ok = 0;
    __syncthreads();
    ok = ok && s_entry_ok != 0;
  }
  // ---- quantise the blocks owed to the peers: one warp per 128-element group,
  // U groups per iteration so that several loads are in flight per lane
  constexpr int U = 4;
  if (ok)
    for (long long g0 = warp * U; g0 < gpb * P; g0 += nwarps * U) {
      float x[U][4];
      bool live[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long g = g0 + u;
        live[u] = g < gpb * P && g / gpb != rank;
        if (live[u]) load4<T>(in + g * kGroup + lane * 4, x[u]);
        else x[u][0] = x[u][1] = x[u][2] = x[u][3] = 0.f;
      }
      float amax[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        amax[u] = fmaxf(fmaxf(fabsf(x[u][0]), fabsf(x[u][1])), fmaxf(fabsf(x[u][2]), fabsf(x[u][3])));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int u = 0; u < U; ++u) amax[u] = fmaxf(amax[u], __shfl_xor_sync(0xffffffffu, amax[u], o));
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (!live[u]) continue;
        const long long g = g0 + u;
        const float sc = amax[u] > 0.f ? amax[u] * (1.0f / 448.0f) : 1.0f;
        const float inv = 1.0f / sc;
        // two hardware conversions (cvt ... e4m3x2) per lane
        const unsigned lo = __nv_cvt_float2_to_fp8x2(make_float2(x[u][0] * inv, x[u][1] * inv), __NV_SATFINITE, __NV_E4M3);
        const unsigned hi = __nv_cvt_float2_to_fp8x2(make_float2(x[u][2] * inv, x[u][3] * inv), __NV_SATFINITE, __NV_E4M3);
        const unsigned packed = lo | (hi << 16);
        *reinterpret_cast<unsigned*>(wire + g * kGroup + lane * 4) = packed;
        if (lane == 0) scales[g] = sc;
      }
    }
  unsigned gen = 0;
  ok = rank_barrier(c, nct, gen, w.timeout_ns, rank, 0) && ok;
  ok = ok && (P == 1 || cta_barrier(w, c, rank, seq + 1ull));
  // ---- pull my block from every peer, dequantise, accumulate in rank order
  if (ok) {
    T* out = reinterpret_cast<T*>(io.out[rank]);
    for (long long g0 = warp * U; g0 < gpb; g0 += nwarps * U) {
      float acc[U][4];
#pragma unroll
      for (int u = 0; u < U; ++u) acc[u][0] = acc[u][1] = acc[u][2] = acc[u][3] = 0.f;
      for (int q = 0; q < P; ++q) {
        if (q == rank) {
#pragma unroll
          for (int u = 0; u < U; ++u) {
            if (g0 + u >= gpb) continue;
            float x[4];
            load4<T>(in + ((long long)rank * gpb + g0 + u) * kGroup + lane * 4, x);
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[u][i] += x[i];
          }
        } else {
          const unsigned char* pw = reinterpret_cast<const unsigned char*>(w.work[q]);
          const float* ps = reinterpret_cast<const float*>(pw + (long long)P * n);
          unsigned packed[U];
          float sc[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const long long gg = (long long)rank * gpb + g0 + u;
            const bool lv = g0 + u < gpb;
            packed[u] = lv ? __ldcg(reinterpret_cast<const unsigned*>(pw + gg * kGroup + lane * 4)) : 0u;
            sc[u] = lv ? __ldcg(ps + gg) : 0.f;
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const float2 a = fp8x2_to_float2((unsigned short)(packed[u] & 0xffffu));
            const float2 b = fp8x2_to_float2((unsigned short)(packed[u] >> 16));
            acc[u][0] += a.x * sc[u]; acc[u][1] += a.y * sc[u];
            acc[u][2] += b.x * sc[u]; acc[u][3] += b.y * sc[u];
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (g0 + u >= gpb) continue;
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[u][i] *= out_scale;
        store4<T>(out + (g0 + u) * kGroup + lane * 4, acc[u]);
      }
    }
  }
  // peers are done with my wire buffer
  if (ok && P > 1) cta_barrier(w, c, rank, seq + 2ull);
  rank_exit(c, nct, [&](Ctrl* cc) { cc->bar_seq = seq + 2ull; });
}

}  // namespace chb

using namespace chb;

extern "C" {

// Reduce-scatter (sum) of P blocks of n elements with the fp8 wire format.
// dtype: CHB_F32 or CHB_BF16.  n must be a multiple of 128.  in / out: one
// pointer per local rank (any device memory, 16-byte aligned).
int chb_rs_fp8_wire(chb_comm* c, int dtype, const void* const* in, void* const* out, long long n,
                    float out_scale, int nctas, cudaStream_t stream) {
  if (!c || !in || !out || n < 0) return CHB_ERR_ARG;
  if (n % kGroup) { c->last_error = "block length must be a multiple of 128 elements"; return CHB_ERR_COUNT; }
  if (dtype != DT_F32 && dtype != DT_BF16) { c->last_error = "fp8 wire format takes f32 or bf16 data"; return CHB_ERR_OP; }
  const size_t need = (size_t)c->P * (size_t)n + (size_t)c->P * (size_t)(n / kGroup) * 4;
  if (need > c->scratch_bytes) { c->last_error = "wire buffer does not fit the symmetric scratch"; return CHB_ERR_NO_MEM; }
  Fp8Io io{};
  for (int l = 0; l < c->nlocal; ++l) {
    if ((((uintptr_t)in[l]) | ((uintptr_t)out[l])) & 15u) { c->last_error = "buffers must be 16-byte aligned"; return CHB_ERR_ARG; }
    io.in[c->rank + l] = (const char*)in[l];
    io.out[c->rank + l] = (char*)out[l];
  }
  if (n == 0) return CHB_SUCCESS;
  const int max_pair_ctas = (kSigSlots - kSigNvlsBase) / kMaxRanks;
  int budget = c->max_ctas / c->nlocal;
  if (nctas <= 0) nctas = (int)(((long long)c->P * n / kGroup + 15) / 16 / 4);
  if (nctas > 120) nctas = 120;
  if (nctas > max_pair_ctas) nctas = max_pair_ctas;
  if (nctas > budget) nctas = budget;
  if (nctas < 1) nctas = 1;
  World w = c->world;
  dim3 grid((unsigned)nctas, (unsigned)c->nlocal, 1), block(kFp8Threads, 1, 1);
  void* args[] = {&w, &io, &n, &out_scale};
  const void* fn = dtype == DT_F32 ? (const void*)fp8_rs_kernel<float> : (const void*)fp8_rs_kernel<__nv_bfloat16>;
  cudaError_t e = (c->nlocal > 1 || nctas > 1) ? cudaLaunchCooperativeKernel(fn, grid, block, args, 0, stream)
                                               : cudaLaunchKernel(fn, grid, block, args, 0, stream);
  if (e != cudaSuccess) { c->last_error = std::string("fp8 reduce-scatter launch failed: ") + cudaGetErrorString(e); return CHB_ERR_CUDA; }
  return CHB_SUCCESS;
}

}  // extern "C"

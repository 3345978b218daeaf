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

constexpr int kFp8Threads = 1024;   // 32 warps per SM at <= 64 registers: the kernel is bound by instruction issue, not by bytes
constexpr int kGroup = 128;  // elements per scale
constexpr int kPeerBatch = 4; // peers whose wire data is loaded together in the pull phase

struct Fp8Io {
  const char* in[kMaxRanks];
  char* out[kMaxRanks];
};

// 8 consecutive elements per lane: a 128-element group is 16 lanes, a warp covers two groups.
template <typename T> __device__ __forceinline__ void load8(const T* p, float* x);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* x) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* x) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(e[i]); x[2 * i] = f.x; x[2 * i + 1] = f.y; }
}
// Eight elements as loaded, before conversion: lets the next iteration's loads be issued early at
// a quarter (bf16) or the same (fp32) register cost of the converted values.
template <typename T> struct Raw8;
template <> struct Raw8<float> { float4 a, b; };
template <> struct Raw8<__nv_bfloat16> { uint4 v; };
__device__ __forceinline__ void load_raw(const float* p, Raw8<float>& r) {
  r.a = reinterpret_cast<const float4*>(p)[0];
  r.b = reinterpret_cast<const float4*>(p)[1];
}
__device__ __forceinline__ void load_raw(const __nv_bfloat16* p, Raw8<__nv_bfloat16>& r) { r.v = *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void unpack(const Raw8<float>& r, float* x) {
  x[0] = r.a.x; x[1] = r.a.y; x[2] = r.a.z; x[3] = r.a.w; x[4] = r.b.x; x[5] = r.b.y; x[6] = r.b.z; x[7] = r.b.w;
}
__device__ __forceinline__ void unpack(const Raw8<__nv_bfloat16>& r, float* x) {
  const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&r.v);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(e[i]); x[2 * i] = f.x; x[2 * i + 1] = f.y; }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float* x);
template <> __device__ __forceinline__ void store8<float>(float* p, const float* x) {
  reinterpret_cast<float4*>(p)[0] = make_float4(x[0], x[1], x[2], x[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(x[4], x[5], x[6], x[7]);
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float* x) {
  uint4 v;
  __nv_bfloat162* e = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) e[i] = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = v;
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
  const int sub = threadIdx.x & 15;                         // lane inside its 16-lane group
  const int hw = (threadIdx.x >> 4) & 1;                    // which half of the warp
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)nct * blockDim.x) >> 5;
  const long long gpb = n / kGroup;                         // groups per block
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
  constexpr int U = 2;   // groups in flight per half-warp (two 16-lane halves per warp, 32 warps per SM)
  // ---- quantise the blocks owed to the peers (the loads of the next iteration are issued before the
  // arithmetic of this one: the phase is bound by bytes in flight, not by instructions)
  if (ok) {
    const long long total = gpb * P, stride = nwarps * 2 * U;
    Raw8<T> cur[U], nxt[U];
    auto fetch = [&](long long gw, Raw8<T>* r) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long g = gw + hw * U + u;
        if (g < total && g / gpb != rank) load_raw(in + g * kGroup + sub * 8, r[u]);
      }
    };
    long long gw = warp * 2 * U;
    if (gw < total) fetch(gw, cur);
    for (; gw < total; gw += stride) {   // trip count uniform per warp (shuffles below)
      if (gw + stride < total) fetch(gw + stride, nxt);
      const long long g0 = gw + hw * U;
      float x[U][8];
      bool live[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long g = g0 + u;
        live[u] = g < total && g / gpb != rank;
        if (live[u]) unpack(cur[u], x[u]);
        else {
#pragma unroll
          for (int i = 0; i < 8; ++i) x[u][i] = 0.f;
        }
      }
      float amax[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        amax[u] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax[u] = fmaxf(amax[u], fabsf(x[u][i]));
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1)
#pragma unroll
        for (int u = 0; u < U; ++u) amax[u] = fmaxf(amax[u], __shfl_xor_sync(0xffffffffu, amax[u], o));
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (!live[u]) continue;
        const long long g = g0 + u;
        const float sc = amax[u] > 0.f ? amax[u] * (1.0f / 448.0f) : 1.0f;
        const float inv = 1.0f / sc;
        unsigned q[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)   // hardware pair conversions (cvt ... e4m3x2)
          q[i] = __nv_cvt_float2_to_fp8x2(make_float2(x[u][2 * i] * inv, x[u][2 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
        *reinterpret_cast<uint2*>(wire + g * kGroup + sub * 8) = make_uint2(q[0] | (q[1] << 16), q[2] | (q[3] << 16));
        if (sub == 0) scales[g] = sc;
      }
#pragma unroll
      for (int u = 0; u < U; ++u) cur[u] = nxt[u];
    }
  }
  unsigned gen = 0;
  ok = rank_barrier(c, nct, gen, w.timeout_ns, rank, 0) && ok;
  ok = ok && (P == 1 || cta_barrier(w, c, rank, seq + 1ull));
  // ---- pull my block from every peer, dequantise, accumulate in a fixed order
  if (ok) {
    T* out = reinterpret_cast<T*>(io.out[rank]);
    for (long long gw = warp * 2 * U; gw < gpb; gw += nwarps * 2 * U) {
      const long long g0 = gw + hw * U;
      float acc[U][8];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[u][i] = 0.f;
      // my own block never goes through fp8
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (g0 + u >= gpb) continue;
        float x[8];
        load8<T>(in + ((long long)rank * gpb + g0 + u) * kGroup + sub * 8, x);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[u][i] += x[i];
      }
      // the peers' contributions, kPeerBatch peers at a time so that their loads are in flight together
      // (order: rank+1, rank+2, ... - fixed, so results repeat bit for bit; it also spreads the peers'
      // egress instead of every rank starting at rank 0)
      for (int j0 = 0; j0 < P - 1; j0 += kPeerBatch) {
        uint2 packed[kPeerBatch][U];
        float sc_lane[kPeerBatch];     // lane u of a half-warp holds the scale of its group u: one request per peer, not U
#pragma unroll
        for (int jj = 0; jj < kPeerBatch; ++jj) {
          const int j = j0 + jj;
          const bool pv = j < P - 1;
          int q = rank + 1 + j;
          if (q >= P) q -= P;
          const unsigned char* pw = reinterpret_cast<const unsigned char*>(w.work[pv ? q : rank]);
          const float* ps = reinterpret_cast<const float*>(pw + (long long)P * n);
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const long long gg = (long long)rank * gpb + g0 + u;
            const bool lv = pv && g0 + u < gpb;
            packed[jj][u] = lv ? __ldcg(reinterpret_cast<const uint2*>(pw + gg * kGroup + sub * 8)) : make_uint2(0u, 0u);
          }
          sc_lane[jj] = (pv && sub < U && g0 + sub < gpb) ? __ldcg(ps + (long long)rank * gpb + g0 + sub) : 0.f;
        }
        float sc[kPeerBatch][U];
#pragma unroll
        for (int jj = 0; jj < kPeerBatch; ++jj)
#pragma unroll
          for (int u = 0; u < U; ++u) sc[jj][u] = __shfl_sync(0xffffffffu, sc_lane[jj], hw * 16 + u);
#pragma unroll
        for (int jj = 0; jj < kPeerBatch; ++jj)
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const float2 a0 = fp8x2_to_float2((unsigned short)(packed[jj][u].x & 0xffffu));
            const float2 a1 = fp8x2_to_float2((unsigned short)(packed[jj][u].x >> 16));
            const float2 a2 = fp8x2_to_float2((unsigned short)(packed[jj][u].y & 0xffffu));
            const float2 a3 = fp8x2_to_float2((unsigned short)(packed[jj][u].y >> 16));
            const float f = sc[jj][u];
            acc[u][0] += a0.x * f; acc[u][1] += a0.y * f; acc[u][2] += a1.x * f; acc[u][3] += a1.y * f;
            acc[u][4] += a2.x * f; acc[u][5] += a2.y * f; acc[u][6] += a3.x * f; acc[u][7] += a3.y * f;
          }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (g0 + u >= gpb) continue;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[u][i] *= out_scale;
        store8<T>(out + (g0 + u) * kGroup + sub * 8, acc[u]);
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
  if (nctas <= 0) nctas = (int)(((long long)c->P * n / kGroup + 127) / 128);   // about four half-warp iterations per CTA
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

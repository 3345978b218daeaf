// ZeRO-style sharded optimizer step in one kernel: the gradient reduce-scatter
// (rank r sums shard r of every rank's flat fp32 gradient buffer, straight from
// the peers' symmetric heaps or in the NVSwitch with multimem.ld_reduce) is
// fused with the AdamW update of the fp32 master shard and the cast of the
// updated shard to the bf16 parameter buffer that the following allgather
// distributes.  The reduced gradient never touches memory.
// No reference counterpart (the reference has no optimizer); its reduce-scatter
// is testing/custom_implementations/work_dir/reduce_scatter/reduce_scatter_radix_batch.cpp:200-653.
#include <cstdio>

#include "../api/chb.h"
#include "../symm/comm.h"
#include "common.cuh"

namespace chb {

constexpr int kAdamThreads = 512;

struct AdamIo {
  const float* grad[kMaxRanks];       // flat gradient buffer of every rank (peer-mapped), P*n elements
  float* master[kMaxRanks];           // local ranks only: fp32 master shard, n elements
  float* m[kMaxRanks];                // first moment shard
  float* v[kMaxRanks];                // second moment shard
  __nv_bfloat16* param[kMaxRanks];    // where the updated bf16 shard goes (n elements)
};

struct AdamHyper {
  float lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, grad_scale;
};

__device__ __forceinline__ float4 mm_ld_reduce_f32(const void* p) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ float adam_one(float g, float& w, float& m, float& v, const AdamHyper& h) {
  m = h.beta1 * m + (1.0f - h.beta1) * g;
  v = h.beta2 * v + (1.0f - h.beta2) * g * g;
  const float mhat = m / h.bias_corr1, vhat = v / h.bias_corr2;
  w -= h.lr * (mhat / (sqrtf(vhat) + h.eps) + h.weight_decay * w);
  return w;
}

// n must be a multiple of 4 (shards are padded by the caller).
__global__ void __launch_bounds__(kAdamThreads, 1)
rs_adam_kernel(World w, AdamIo io, long long n, AdamHyper h, const char* mc_grad) {
  const int rank = w.rank0 + (int)blockIdx.y;
  const int P = w.P;
  Ctrl* c = w.ctrl[rank];
  __shared__ unsigned long long s_seq;
  if (threadIdx.x == 0) s_seq = ld_volatile_u64(&c->bar_seq);
  __syncthreads();
  const unsigned long long seq = s_seq;
  bool ok = !ld_volatile_u32(&c->abort);
  // every peer's gradients are final
  ok = ok && (P == 1 || cta_barrier(w, c, rank, seq + 1ull));
  if (ok) {
    const long long nvec = n / 4;
    const long long TT = (long long)gridDim.x * blockDim.x;
    const long long base = (long long)rank * nvec;
    float4* mw = reinterpret_cast<float4*>(io.master[rank]);
    float4* mm = reinterpret_cast<float4*>(io.m[rank]);
    float4* mv = reinterpret_cast<float4*>(io.v[rank]);
    uint2* po = reinterpret_cast<uint2*>(io.param[rank]);
    constexpr int U = 4;
    for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < nvec; i0 += TT * U) {
      float4 g[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + (long long)u * TT;
        g[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < nvec) {
          if (mc_grad) {
            g[u] = mm_ld_reduce_f32(mc_grad + (base + i) * 16);
          } else {
            for (int q = 0; q < P; ++q) {   // rank order: identical bits on every run
              const uint4 t = ld16_cg(reinterpret_cast<const char*>(io.grad[q]) + (base + i) * 16);
              const float4 x = *reinterpret_cast<const float4*>(&t);
              g[u].x += x.x; g[u].y += x.y; g[u].z += x.z; g[u].w += x.w;
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = i0 + (long long)u * TT;
        if (i < nvec) {
          float4 ww = mw[i], m1 = mm[i], v1 = mv[i];
          const float s = h.grad_scale;
          __nv_bfloat16 o[4];
          o[0] = __float2bfloat16_rn(adam_one(g[u].x * s, ww.x, m1.x, v1.x, h));
          o[1] = __float2bfloat16_rn(adam_one(g[u].y * s, ww.y, m1.y, v1.y, h));
          o[2] = __float2bfloat16_rn(adam_one(g[u].z * s, ww.z, m1.z, v1.z, h));
          o[3] = __float2bfloat16_rn(adam_one(g[u].w * s, ww.w, m1.w, v1.w, h));
          mw[i] = ww; mm[i] = m1; mv[i] = v1;
          po[i] = *reinterpret_cast<uint2*>(o);
        }
      }
    }
  }
  // peers are done reading my gradients: the caller may zero them afterwards
  if (ok && P > 1) cta_barrier(w, c, rank, seq + 2ull);
  rank_exit(c, gridDim.x, [&](Ctrl* cc) { cc->bar_seq = seq + 2ull; });
}

// Plain (unsharded) variant for the data-parallel path: the gradient has
// already been allreduced; AdamW on the fp32 master, bf16 copy of the result.
__global__ void __launch_bounds__(kAdamThreads)
adam_flat_kernel(const float* __restrict__ grad, float* master, float* m, float* v, __nv_bfloat16* param,
                 long long n, AdamHyper h) {
  const long long nvec = n / 4;
  const long long TT = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += TT) {
    const float4 g = reinterpret_cast<const float4*>(grad)[i];
    float4 ww = reinterpret_cast<float4*>(master)[i], m1 = reinterpret_cast<float4*>(m)[i],
           v1 = reinterpret_cast<float4*>(v)[i];
    const float s = h.grad_scale;
    __nv_bfloat16 o[4];
    o[0] = __float2bfloat16_rn(adam_one(g.x * s, ww.x, m1.x, v1.x, h));
    o[1] = __float2bfloat16_rn(adam_one(g.y * s, ww.y, m1.y, v1.y, h));
    o[2] = __float2bfloat16_rn(adam_one(g.z * s, ww.z, m1.z, v1.z, h));
    o[3] = __float2bfloat16_rn(adam_one(g.w * s, ww.w, m1.w, v1.w, h));
    reinterpret_cast<float4*>(master)[i] = ww;
    reinterpret_cast<float4*>(m)[i] = m1;
    reinterpret_cast<float4*>(v)[i] = v1;
    reinterpret_cast<uint2*>(param)[i] = *reinterpret_cast<uint2*>(o);
  }
}

}  // namespace chb

using namespace chb;

extern "C" {

// grad: one flat fp32 gradient buffer per local rank inside the symmetric heap
// (P*n elements); master / m / v: fp32 shards of n elements; param_shard: bf16
// destination of the updated shard (n elements).  hyper: lr, beta1, beta2, eps,
// weight_decay, bias_corr1, bias_corr2, grad_scale.  use_multimem != 0 reduces
// in the switch (needs a multicast alias).  n must be a multiple of 4.
int chb_rs_adam(chb_comm* c, const void* const* grad, void* const* master, void* const* m, void* const* v,
                void* const* param_shard, long long n, const float* hyper, int use_multimem, int nctas,
                cudaStream_t stream) {
  if (!c || !grad || !master || !m || !v || !param_shard || !hyper || n < 0) return CHB_ERR_ARG;
  if (n % 4) { c->last_error = "shard length must be a multiple of 4"; return CHB_ERR_COUNT; }
  AdamIo io{};
  for (int l = 0; l < c->nlocal; ++l) {
    const int r = c->rank + l;
    io.master[r] = (float*)master[l];
    io.m[r] = (float*)m[l];
    io.v[r] = (float*)v[l];
    io.param[r] = (__nv_bfloat16*)param_shard[l];
    io.grad[r] = (const float*)grad[l];
    if (((uintptr_t)grad[l] | (uintptr_t)master[l] | (uintptr_t)m[l] | (uintptr_t)v[l]) & 15u || ((uintptr_t)param_shard[l] & 7u)) {
      c->last_error = "buffers must be 16-byte aligned (bf16 shard: 8-byte)";
      return CHB_ERR_ARG;
    }
  }
  const char* mc = nullptr;
  if (c->nlocal == 1) {
    for (int q = 0; q < c->P; ++q) {
      char* t = c->translate(grad[0], c->rank, q);
      if (!t) { c->last_error = "gradient buffer is not inside the symmetric heap"; return CHB_ERR_ARG; }
      io.grad[q] = (const float*)t;
    }
    if (use_multimem) {
      if (!c->mc_heap) { c->last_error = "communicator has no multicast alias"; return CHB_ERR_UNSUPPORTED; }
      mc = c->mc_heap + ((const char*)grad[0] - c->heap[c->rank]);
    }
  } else if (use_multimem) {
    return CHB_ERR_UNSUPPORTED;
  }
  if (n == 0) return CHB_SUCCESS;
  AdamHyper h{hyper[0], hyper[1], hyper[2], hyper[3], hyper[4], hyper[5], hyper[6], hyper[7]};
  const int max_pair_ctas = (kSigSlots - kSigNvlsBase) / kMaxRanks;
  int budget = c->max_ctas / c->nlocal;
  if (nctas <= 0) nctas = (int)((n / 4 + kAdamThreads * 4 - 1) / (kAdamThreads * 4));
  if (nctas > 96) nctas = 96;
  if (nctas > max_pair_ctas) nctas = max_pair_ctas;
  if (nctas > budget) nctas = budget;
  if (nctas < 1) nctas = 1;
  World w = c->world;
  dim3 grid((unsigned)nctas, (unsigned)c->nlocal, 1), block(kAdamThreads, 1, 1);
  void* args[] = {&w, &io, &n, &h, &mc};
  cudaError_t e = c->nlocal > 1 ? cudaLaunchCooperativeKernel((const void*)rs_adam_kernel, grid, block, args, 0, stream)
                                : cudaLaunchKernel((const void*)rs_adam_kernel, grid, block, args, 0, stream);
  if (e != cudaSuccess) { c->last_error = std::string("rs_adam launch failed: ") + cudaGetErrorString(e); return CHB_ERR_CUDA; }
  return CHB_SUCCESS;
}

// AdamW on a flat fp32 master with a bf16 copy of the result; n % 4 == 0, 16-byte aligned buffers.
int chb_adam_flat(const void* grad, void* master, void* m, void* v, void* param_bf16, long long n,
                  const float* hyper, cudaStream_t stream) {
  if (!grad || !master || !m || !v || !param_bf16 || !hyper || n < 0 || (n % 4)) return CHB_ERR_ARG;
  if (((uintptr_t)grad | (uintptr_t)master | (uintptr_t)m | (uintptr_t)v) & 15u || ((uintptr_t)param_bf16 & 7u)) return CHB_ERR_ARG;
  if (n == 0) return CHB_SUCCESS;
  AdamHyper h{hyper[0], hyper[1], hyper[2], hyper[3], hyper[4], hyper[5], hyper[6], hyper[7]};
  long long blocks = (n / 4 + kAdamThreads - 1) / kAdamThreads;
  if (blocks > 148 * 4) blocks = 148 * 4;
  adam_flat_kernel<<<(unsigned)blocks, kAdamThreads, 0, stream>>>((const float*)grad, (float*)master, (float*)m, (float*)v,
                                                                   (__nv_bfloat16*)param_bf16, n, h);
  return cudaGetLastError() == cudaSuccess ? CHB_SUCCESS : CHB_ERR_CUDA;
}

}  // extern "C"

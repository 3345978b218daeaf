// Gradient bucket fill for the data-parallel path: one launch per bucket moves
// the gradients of all its parameters (bf16, fp16 or fp32, wherever autograd left
// them) into the bucket's flat fp32 buffer in symmetric memory, either
// overwriting a slot (first micro-batch after zero_grad) or adding to it
// (gradient accumulation).  The bucket is the input of the allreduce kernel
// that follows on the side stream, whose 1/P scale is fused into its last step.
// This replaces one eager cast-and-add per parameter.
// No reference counterpart: the reference stops at the allreduce primitive
// (testing/custom_implementations/work_dir/all_reduce/all_reduce_radix_batch.cpp:202).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../api/chb.h"

namespace chb {

constexpr int kBucketSlots = 48;      // tensors per launch (the table travels as a kernel argument)
constexpr int kBucketThreads = 256;

struct BucketTable {
  const void* src[kBucketSlots];
  long long dst_off[kBucketSlots];    // element offset in the bucket
  long long n[kBucketSlots];
  unsigned char mode[kBucketSlots];   // bit 0: overwrite instead of add; bits 1-2: source type (0 f32, 1 bf16, 2 f16)
  int count;
};

template <typename S>
__device__ __forceinline__ float to_f32(S v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

// One tensor: 4 elements per thread and iteration when both sides allow vector accesses.
template <typename S>
__device__ __forceinline__ void fill_one(const S* __restrict__ src, float* __restrict__ dst, long long n, bool overwrite,
                                         long long g, long long stride) {
  const bool vec = ((reinterpret_cast<uintptr_t>(src) % (4 * sizeof(S))) == 0) && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0);
  const long long nv = vec ? n / 4 : 0;
  for (long long i = g; i < nv; i += stride) {
    float x[4];
    if (sizeof(S) == 4) {
      const float4 t = reinterpret_cast<const float4*>(src)[i];
      x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w;
    } else {
      const uint2 t = reinterpret_cast<const uint2*>(src)[i];
      const S* e = reinterpret_cast<const S*>(&t);
#pragma unroll
      for (int j = 0; j < 4; ++j) x[j] = to_f32<S>(e[j]);
    }
    float4 o = make_float4(x[0], x[1], x[2], x[3]);
    if (!overwrite) {
      const float4 a = reinterpret_cast<const float4*>(dst)[i];
      o.x += a.x; o.y += a.y; o.z += a.z; o.w += a.w;
    }
    reinterpret_cast<float4*>(dst)[i] = o;
  }
  for (long long e = nv * 4 + g; e < n; e += stride) dst[e] = overwrite ? to_f32<S>(src[e]) : dst[e] + to_f32<S>(src[e]);
}

// grid: (blocks per tensor, tensors)
__global__ void __launch_bounds__(kBucketThreads)
bucket_fill_kernel(BucketTable t, float* __restrict__ bucket) {
  const int k = (int)blockIdx.y;
  if (k >= t.count) return;
  const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long stride = (long long)gridDim.x * blockDim.x;
  float* dst = bucket + t.dst_off[k];
  const bool overwrite = (t.mode[k] & 1u) != 0;
  switch ((t.mode[k] >> 1) & 3u) {
    case 0: fill_one<float>(reinterpret_cast<const float*>(t.src[k]), dst, t.n[k], overwrite, g, stride); break;
    case 1: fill_one<__nv_bfloat16>(reinterpret_cast<const __nv_bfloat16*>(t.src[k]), dst, t.n[k], overwrite, g, stride); break;
    default: fill_one<__half>(reinterpret_cast<const __half*>(t.src[k]), dst, t.n[k], overwrite, g, stride); break;
  }
}

}  // namespace chb

using namespace chb;

extern "C" {

// bucket[dst_off[i] .. +n[i]) (+)= src[i] for i < count, any count (launched in groups of 48 tensors).
// src_dtype[i]: CHB_F32 / CHB_BF16 / CHB_F16; overwrite[i] != 0 replaces the slot instead of adding to it.
int chb_bucket_fill(float* bucket, int count, const void* const* src, const long long* dst_off, const long long* n,
                    const int* src_dtype, const unsigned char* overwrite, cudaStream_t stream) {
  if (!bucket || count < 0 || (count && (!src || !dst_off || !n || !src_dtype || !overwrite))) return CHB_ERR_ARG;
  for (int base = 0; base < count; base += kBucketSlots) {
    BucketTable t{};
    t.count = count - base < kBucketSlots ? count - base : kBucketSlots;
    long long big = 0;
    for (int i = 0; i < t.count; ++i) {
      const int d = src_dtype[base + i];
      const int code = d == CHB_F32 ? 0 : d == CHB_BF16 ? 1 : d == CHB_F16 ? 2 : -1;
      if (code < 0 || n[base + i] < 0 || dst_off[base + i] < 0) return CHB_ERR_ARG;
      t.src[i] = src[base + i];
      t.dst_off[i] = dst_off[base + i];
      t.n[i] = n[base + i];
      t.mode[i] = (unsigned char)((overwrite[base + i] ? 1 : 0) | (code << 1));
      big = n[base + i] > big ? n[base + i] : big;
    }
    long long bx = (big / 4 + kBucketThreads * 4 - 1) / (kBucketThreads * 4);   // about four vectors per thread
    if (bx < 1) bx = 1;
    if (bx > 512) bx = 512;
    bucket_fill_kernel<<<dim3((unsigned)bx, (unsigned)t.count, 1), kBucketThreads, 0, stream>>>(t, bucket);
    if (cudaGetLastError() != cudaSuccess) return CHB_ERR_CUDA;
  }
  return CHB_SUCCESS;
}

}  // extern "C"

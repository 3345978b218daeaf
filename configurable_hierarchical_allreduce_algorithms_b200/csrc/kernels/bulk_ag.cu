// Allgather by bulk asynchronous copies (the TMA engine): one elected thread per
// CTA streams 16 KiB chunks peer-global -> shared -> local-global through a ring
// of shared-memory stages, completion tracked by mbarriers (loads) and bulk
// groups (stores).  No register staging and almost no issue slots: the SMs
// stay free for whatever runs next to the collective.  Every load is a plain
// one-destination bulk copy into this CTA's own shared memory; a peer's memory
// is read directly.
// Every wait is bounded.
//
// Replaces the inter-group linear allgather / broadcast of the reference
// (testing/custom_implementations/work_dir/all_gather/all_gather_radix_batch_1_0.cpp:148-163)
// in its flat (b = 1) form: every rank fetches every block from its owner.
#include <cstdio>
#include <mutex>

#include "../api/chb.h"
#include "../symm/comm.h"
#include "common.cuh"

namespace chb {

constexpr int kBulkThreads = 128;
constexpr int kBulkStages = 8;
constexpr int kBulkChunk = 16384;  // bytes; multiple of 16
constexpr int kBulkLag = 3;        // stores allowed in flight before a stage is refilled (< kBulkStages)
constexpr int kBulkSmem = kBulkStages * kBulkChunk;

struct BulkIo {
  const char* in[kMaxRanks];   // every rank's block (peer-mapped)
  char* out[kMaxRanks];        // local ranks' outputs
};

__device__ __forceinline__ unsigned smem_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulk_load(unsigned dst_smem, const void* src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, unsigned src_smem, unsigned bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_wait_read_lag() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kBulkLag) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// nbytes: bytes per block (multiple of 16); all pointers 16-byte aligned.
__global__ void __launch_bounds__(kBulkThreads)
ag_bulk_kernel(World w, BulkIo io, long long nbytes) {
  extern __shared__ __align__(128) unsigned char stage_mem[];
  unsigned char (*stage)[kBulkChunk] = reinterpret_cast<unsigned char (*)[kBulkChunk]>(stage_mem);
  __shared__ __align__(8) unsigned long long bars[kBulkStages];
  const int rank = w.rank0 + (int)blockIdx.y;
  const int P = w.P;
  Ctrl* c = w.ctrl[rank];
  __shared__ unsigned long long s_seq;
  if (threadIdx.x == 0) {
    s_seq = ld_volatile_u64(&c->bar_seq);
    for (int s = 0; s < kBulkStages; ++s) mbar_init(smem_addr(&bars[s]), 1);
    asm volatile("fence.proxy.async;" ::: "memory");
  }
  __syncthreads();
  const unsigned long long seq = s_seq;
  bool ok = !ld_volatile_u32(&c->abort);
  // peers' blocks are final, and nobody still reads the output I am about to overwrite
  ok = ok && (P == 1 || cta_barrier(w, c, rank, seq + 1ull));
  if (ok && threadIdx.x == 0) {
    // the flags were read through the generic proxy, the copies below go through the async proxy
    asm volatile("fence.proxy.async;" ::: "memory");
    const long long nch = (nbytes + kBulkChunk - 1) / kBulkChunk;
    const long long nct = gridDim.x;
    // this CTA takes chunks blockIdx.x, blockIdx.x + nct, ... of every block and alternates between the
    // owners, so that local copies and NVLink reads are in flight together
    const long long mych = (nch > (long long)blockIdx.x) ? (nch - blockIdx.x + nct - 1) / nct : 0;
    const long long mine = mych * P;
    auto item = [&](long long k, const char*& src, char*& dst, unsigned& bytes) {
      const int owner = (int)((rank + k % P) % P);            // my own block first, then the next ranks
      const long long off = ((long long)blockIdx.x + (k / P) * nct) * kBulkChunk;
      const long long left = nbytes - off;
      bytes = (unsigned)(left < kBulkChunk ? left : kBulkChunk);
      src = io.in[owner] + off;
      dst = io.out[rank] + (long long)owner * nbytes + off;
    };
    const long long pre = mine < kBulkStages ? mine : kBulkStages;
    for (long long k = 0; k < pre; ++k) {
      const char* src; char* dst; unsigned bytes;
      item(k, src, dst, bytes);
      const unsigned bar = smem_addr(&bars[k % kBulkStages]);
      mbar_expect_tx(bar, bytes);
      bulk_load(smem_addr(stage[k % kBulkStages]), src, bytes, bar);
    }
    bool failed = false;
    long long issued = pre;                          // loads started so far (items 0 .. issued-1)
    long long k_failed = -1;
    for (long long k = 0; k < mine && !failed; ++k) {
      const int s = (int)(k % kBulkStages);
      const unsigned bar = smem_addr(&bars[s]);
      const unsigned parity = (unsigned)((k / kBulkStages) & 1);
      if (!mbar_try_wait(bar, parity)) {
        const unsigned long long t0 = globaltimer_ns();
        unsigned spins = 0;
        while (!mbar_try_wait(bar, parity)) {
          if ((++spins & 63u) == 0u && globaltimer_ns() - t0 > w.timeout_ns) {
            record_timeout(c, ST_TIMEOUT_ROUND, rank, (int)k, -3, (unsigned long long)k, 0ull);
            failed = true;
            k_failed = k;
            break;
          }
        }
        if (failed) break;
      }
      const char* src; char* dst; unsigned bytes;
      item(k, src, dst, bytes);
      bulk_store(dst, smem_addr(stage[s]), bytes);
      const long long j = k - kBulkLag;              // its store is kBulkLag groups back
      if (j >= 0 && j + kBulkStages < mine) {
        bulk_wait_read_lag();                        // store j has read its stage: it may be refilled
        const int sj = (int)(j % kBulkStages);
        const unsigned barj = smem_addr(&bars[sj]);
        item(j + kBulkStages, src, dst, bytes);
        mbar_expect_tx(barj, bytes);
        bulk_load(smem_addr(stage[sj]), src, bytes, barj);
        issued = j + kBulkStages + 1;
      }
    }
    if (failed) {
      // Loads k_failed .. issued-1 may still be writing this CTA's shared memory: give each one more bounded
      // wait before the CTA (and with it the shared memory) goes away; what is still pending after that is
      // noted in the status word (seen = number of loads that never completed).
      unsigned long long pending = 0;
      for (long long i = k_failed; i < issued; ++i) {
        const unsigned bar = smem_addr(&bars[i % kBulkStages]);
        const unsigned parity = (unsigned)((i / kBulkStages) & 1);
        const unsigned long long t0 = globaltimer_ns();
        bool done = mbar_try_wait(bar, parity);
        unsigned spins = 0;
        while (!done && !((++spins & 63u) == 0u && globaltimer_ns() - t0 > w.timeout_ns)) done = mbar_try_wait(bar, parity);
        if (!done) ++pending;
      }
      c->status[5] = pending;
    }
    bulk_wait_all();                                 // all my stores have landed
    if (failed) ok = false;
  }
  __syncthreads();
  if (ld_volatile_u32(&c->abort)) ok = false;
  // peers are done reading my block
  if (ok && P > 1) cta_barrier(w, c, rank, seq + 2ull);
  rank_exit(c, gridDim.x, [&](Ctrl* cc) { cc->bar_seq = seq + 2ull; });
}

}  // namespace chb

using namespace chb;

extern "C" {

// Allgather of `nbytes` per rank.  in: this rank's block inside the symmetric
// heap (one pointer per local rank); out: P * nbytes.  16-byte alignment and
// nbytes % 16 == 0 are required (bulk copies start on 16-byte boundaries).
int chb_ag_bulk(chb_comm* c, const void* const* in, void* const* out, long long nbytes, int nctas, cudaStream_t stream) {
  if (!c || !in || !out || nbytes < 0) return CHB_ERR_ARG;
  if (nbytes % 16) { c->last_error = "bulk allgather needs a multiple of 16 bytes per block"; return CHB_ERR_COUNT; }
  BulkIo io{};
  for (int l = 0; l < c->nlocal; ++l) {
    if ((((uintptr_t)in[l]) | ((uintptr_t)out[l])) & 15u) { c->last_error = "bulk allgather needs 16-byte aligned buffers"; return CHB_ERR_ARG; }
    io.in[c->rank + l] = (const char*)in[l];
    io.out[c->rank + l] = (char*)out[l];
  }
  if (c->nlocal == 1) {
    // every rank's block sits at its own offset of the symmetric output when the call is in place
    // (in == out + rank * nbytes); otherwise all inputs share one heap offset
    const char* slot = (const char*)out[0] + (long long)c->rank * nbytes;
    const bool alias = (const char*)in[0] == slot;
    for (int q = 0; q < c->P; ++q) {
      const void* mine_as_q = alias ? (const void*)((const char*)out[0] + (long long)q * nbytes) : in[0];
      char* t = c->translate(mine_as_q, c->rank, q);
      if (!t) { c->last_error = "bulk allgather input must be inside the symmetric heap"; return CHB_ERR_ARG; }
      io.in[q] = t;
    }
  }
  if (nbytes == 0) return CHB_SUCCESS;
  const int max_pair_ctas = (kSigSlots - kSigNvlsBase) / kMaxRanks;
  int budget = c->max_ctas / c->nlocal;           // 128 KiB of shared memory: one CTA per SM
  static bool attr_set[64] = {};
  static std::mutex attr_mu;                      // several host threads may make their first call at once
  std::lock_guard<std::mutex> attr_lock(attr_mu);
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    if (cudaFuncSetAttribute((const void*)ag_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkSmem) != cudaSuccess) {
      c->last_error = "bulk allgather: cannot reserve shared memory";
      return CHB_ERR_CUDA;
    }
    attr_set[dev] = true;
  }
  const long long chunks = (nbytes + kBulkChunk - 1) / kBulkChunk;
  if (nctas <= 0 || nctas > chunks) nctas = (int)(chunks < 128 ? chunks : 128);
  if (nctas > 128) nctas = 128;
  if (nctas > max_pair_ctas) nctas = max_pair_ctas;
  if (nctas > budget) nctas = budget;
  if (nctas < 1) nctas = 1;
  World w = c->world;
  dim3 grid((unsigned)nctas, (unsigned)c->nlocal, 1), block(kBulkThreads, 1, 1);
  void* args[] = {&w, &io, &nbytes};
  cudaError_t e = c->nlocal > 1 ? cudaLaunchCooperativeKernel((const void*)ag_bulk_kernel, grid, block, args, kBulkSmem, stream)
                                : cudaLaunchKernel((const void*)ag_bulk_kernel, grid, block, args, kBulkSmem, stream);
  if (e != cudaSuccess) { c->last_error = std::string("bulk allgather launch failed: ") + cudaGetErrorString(e); return CHB_ERR_CUDA; }
  return CHB_SUCCESS;
}

}  // extern "C"

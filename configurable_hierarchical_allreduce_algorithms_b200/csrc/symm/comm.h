// Host-side communicator: the symmetric heap of every rank, carved into a
// signal pad, the flagged-line (LL) inbox, scratch for step programs and a
// region from which callers can allocate peer-visible tensors.
//
//   heap of rank p:  [ signal pad | LL inbox | scratch | user region ]
//
// The heap pointers come from outside (csrc/symm/ipc.cc for cudaIpc handles,
// a VMM/multicast allocator on the Python side, or one allocation split P ways
// when all ranks are emulated on one GPU), so that the same kernels run in all
// three settings.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <map>
#include <string>
#include <vector>

#include "../kernels/common.cuh"

struct chb_program;

struct chb_comm {
  int P = 1;
  int rank = 0;        // first local rank
  int nlocal = 1;      // P when emulated on one GPU
  int device = 0;
  size_t sig_bytes = 0, ll_bytes = 0, scratch_bytes = 0, user_bytes = 0, heap_bytes = 0;
  size_t ll_lines_per_src = 0;
  std::vector<char*> heap;      // [P] peer-mapped base pointers
  char* mc_heap = nullptr;      // multicast alias of the heap (NVLS), or null
  chb::Ctrl* ctrl = nullptr;    // [nlocal] control blocks, device memory owned by the comm
  unsigned long long* trace = nullptr;  // [nlocal][2 * trace_rounds] round stamps, or null
  int trace_rounds = 0;
  chb::World world{};           // device view handed to kernels
  unsigned long long timeout_ns = 10ull * 1000 * 1000 * 1000;
  int max_ctas = 0;             // co-resident CTA budget per rank
  int sm_count = 0;
  // device copies of compiled programs, keyed by the program's unique id
  std::map<uint64_t, void*> blobs;
  std::map<uint64_t, long long> blob_table_bytes;   // per program: bytes of the largest rank's own table entries
  // flagged-line form of compiled programs: key = program id * 16 + element size; value = device tables
  // and the line count of the busiest level (sizes the grid)
  std::map<uint64_t, std::pair<void*, std::pair<long long, long long>>> ll_blobs;   // blob, (busiest level lines, largest rank table bytes)
  std::string last_error;
  // set only by the native constructors (chb_comm_create_ipc / chb_comm_create_emulated), which own the heap
  void* owned_heap = nullptr;
  std::vector<void*> ipc_opened;
  struct chb_vmm_heap* vmm = nullptr;   // heaps (and multicast alias) from the virtual-memory allocator

  char* sig_ptr(int p) const { return heap[p]; }
  char* ll_ptr(int p) const { return heap[p] + sig_bytes; }
  char* scratch_ptr(int p) const { return heap[p] + sig_bytes + ll_bytes; }
  char* user_ptr(int p) const { return heap[p] + sig_bytes + ll_bytes + scratch_bytes; }
  bool is_local(int p) const { return p >= rank && p < rank + nlocal; }
  // peer-visible address of a pointer inside a local rank's heap, else null
  char* translate(const void* ptr, int owner_local_rank, int peer) const {
    const char* c = (const char*)ptr;
    const char* b = heap[owner_local_rank];
    if (c < b || c >= b + heap_bytes) return nullptr;
    return heap[peer] + (c - b);
  }
};

// CHB_TABLES_IN_SMEM=0 keeps the program kernels' schedule tables in global memory (for A/B timing and debugging)
inline bool tables_in_smem_wanted() {
  static const bool on = [] {
    const char* e = std::getenv("CHB_TABLES_IN_SMEM");
    return !(e && e[0] == '0');
  }();
  return on;
}


// Native symmetric heap: CUDA virtual-memory allocations shared between the
// ranks of one box, with an optional NVLink multicast alias.
//
//   every rank    cuMemCreate (POSIX file-descriptor handle type), export the
//                 descriptor, hand it to every peer (bootstrap's descriptor
//                 exchange), import the peers' descriptors, reserve address
//                 ranges, map, enable access: heap[p] is peer-mapped for all p
//   multicast     rank 0 creates the multicast object, its descriptor travels
//                 the same way; every rank adds its device, then binds its heap
//                 allocation at offset 0 and maps the object: stores to the
//                 alias reach every GPU, multimem.ld_reduce on it sums in the switch
//
// With this the communicators of the native launcher and of plain C callers
// get the multimem kernels without Python (torch's symmetric memory was the
// only source of the alias before).  The driver API is reached through
// dlopen("libcuda.so.1"), so the library still loads on a machine without a
// GPU driver.  Everything is capability-gated: no multicast support means a
// heap without alias, no descriptor handle type means CHB_ERR_UNSUPPORTED and
// the caller falls back to cudaIpc.
//
// Teardown order matters on a shared NVSwitch domain: all ranks meet first (no
// kernel of a peer may still use the alias), then unmap and unbind, meet
// again, and only then release.  A rank that dies while its memory is bound is
// not something this code can repair.
//
// No reference counterpart: the reference's buffers are malloc'ed host arrays
// handed to MPI (testing/custom_implementations/work_dir/all_gather/all_gather_radix_batch_1_0.cpp:60-64).
#include <cuda.h>
#include <dlfcn.h>
#include <unistd.h>

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../api/chb.h"
#include "../boot/bootstrap.h"
#include "vmm.h"

namespace {

#define CHB_STR2(x) #x
#define CHB_STR(x) CHB_STR2(x)
// cuda.h maps some names to versioned symbols (cuMemMap stays, cuCtxGetDevice stays, ...): stringify after expansion
#define CHB_DRV(name) reinterpret_cast<decltype(&name)>(sym(CHB_STR(name)))

struct Driver {
  void* h = nullptr;
  bool ok = false;
  void* sym(const char* n) { return h ? dlsym(h, n) : nullptr; }
  decltype(&cuInit) Init = nullptr;
  decltype(&cuCtxGetDevice) CtxGetDevice = nullptr;
  decltype(&cuDeviceGetAttribute) DeviceGetAttribute = nullptr;
  decltype(&cuMemGetAllocationGranularity) MemGetAllocationGranularity = nullptr;
  decltype(&cuMemCreate) MemCreate = nullptr;
  decltype(&cuMemRelease) MemRelease = nullptr;
  decltype(&cuMemExportToShareableHandle) MemExportToShareableHandle = nullptr;
  decltype(&cuMemImportFromShareableHandle) MemImportFromShareableHandle = nullptr;
  decltype(&cuMemAddressReserve) MemAddressReserve = nullptr;
  decltype(&cuMemAddressFree) MemAddressFree = nullptr;
  decltype(&cuMemMap) MemMap = nullptr;
  decltype(&cuMemUnmap) MemUnmap = nullptr;
  decltype(&cuMemSetAccess) MemSetAccess = nullptr;
  decltype(&cuMulticastCreate) MulticastCreate = nullptr;
  decltype(&cuMulticastAddDevice) MulticastAddDevice = nullptr;
  decltype(&cuMulticastBindMem) MulticastBindMem = nullptr;
  decltype(&cuMulticastUnbind) MulticastUnbind = nullptr;
  decltype(&cuMulticastGetGranularity) MulticastGetGranularity = nullptr;
  decltype(&cuGetErrorString) GetErrorString = nullptr;

  bool load() {
    if (ok) return true;
    h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return false;
    Init = CHB_DRV(cuInit);
    CtxGetDevice = CHB_DRV(cuCtxGetDevice);
    DeviceGetAttribute = CHB_DRV(cuDeviceGetAttribute);
    MemGetAllocationGranularity = CHB_DRV(cuMemGetAllocationGranularity);
    MemCreate = CHB_DRV(cuMemCreate);
    MemRelease = CHB_DRV(cuMemRelease);
    MemExportToShareableHandle = CHB_DRV(cuMemExportToShareableHandle);
    MemImportFromShareableHandle = CHB_DRV(cuMemImportFromShareableHandle);
    MemAddressReserve = CHB_DRV(cuMemAddressReserve);
    MemAddressFree = CHB_DRV(cuMemAddressFree);
    MemMap = CHB_DRV(cuMemMap);
    MemUnmap = CHB_DRV(cuMemUnmap);
    MemSetAccess = CHB_DRV(cuMemSetAccess);
    MulticastCreate = CHB_DRV(cuMulticastCreate);
    MulticastAddDevice = CHB_DRV(cuMulticastAddDevice);
    MulticastBindMem = CHB_DRV(cuMulticastBindMem);
    MulticastUnbind = CHB_DRV(cuMulticastUnbind);
    MulticastGetGranularity = CHB_DRV(cuMulticastGetGranularity);
    GetErrorString = CHB_DRV(cuGetErrorString);
    ok = Init && CtxGetDevice && DeviceGetAttribute && MemGetAllocationGranularity && MemCreate && MemRelease &&
         MemExportToShareableHandle && MemImportFromShareableHandle && MemAddressReserve && MemAddressFree && MemMap &&
         MemUnmap && MemSetAccess;
    return ok;
  }
  bool has_multicast() const {
    return MulticastCreate && MulticastAddDevice && MulticastBindMem && MulticastUnbind && MulticastGetGranularity;
  }
  std::string why(CUresult r) {
    const char* s = nullptr;
    if (GetErrorString) GetErrorString(r, &s);
    return s ? s : ("CUresult " + std::to_string((int)r));
  }
};

Driver& drv() {
  static Driver d;
  return d;
}

size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace

struct chb_vmm_heap {
  int P = 0, rank = 0, device = 0;
  size_t bytes = 0;                                   // mapped size of every heap (granularity-rounded)
  CUmemGenericAllocationHandle mine = 0;
  std::vector<CUmemGenericAllocationHandle> imported; // [P], 0 for self
  std::vector<CUdeviceptr> va;                        // [P] mapped bases
  CUmemGenericAllocationHandle mc = 0;
  CUdeviceptr mc_va = 0;
  bool mc_bound = false;
  chb_bootstrap* boot = nullptr;
};

extern "C" {

// Pure layout arithmetic, also used by the tests: the size every rank maps for a request of `bytes`, given
// the allocation granularity and (0 = none) the multicast granularity.
size_t chb_vmm_mapped_size(size_t bytes, size_t mem_granularity, size_t mc_granularity) {
  size_t g = mem_granularity ? mem_granularity : 1;
  if (mc_granularity > g) g = round_up(mc_granularity, g);      // both are powers of two in practice
  return round_up(bytes ? bytes : 1, g);
}

void chb_vmm_destroy(chb_vmm_heap* hp) {
  if (!hp) return;
  Driver& d = drv();
  // nobody's kernels use the heaps or the alias any more
  if (hp->boot) chb_bootstrap_barrier(hp->boot);
  if (hp->mc_va) { d.MemUnmap(hp->mc_va, hp->bytes); d.MemAddressFree(hp->mc_va, hp->bytes); }
  if (hp->mc_bound) d.MulticastUnbind(hp->mc, (CUdevice)hp->device, 0, hp->bytes);
  for (int p = 0; p < hp->P; ++p)
    if (p < (int)hp->va.size() && hp->va[p]) { d.MemUnmap(hp->va[p], hp->bytes); d.MemAddressFree(hp->va[p], hp->bytes); }
  // every rank has unmapped before any allocation goes away
  if (hp->boot) chb_bootstrap_barrier(hp->boot);
  if (hp->mc) d.MemRelease(hp->mc);
  for (auto h : hp->imported) if (h) d.MemRelease(h);
  if (hp->mine) d.MemRelease(hp->mine);
  delete hp;
}

// One heap of `bytes` (rounded up) per rank on the current device of each rank, all peer-mapped.
// want_multicast: 0 never, 1 if every rank's device supports it.  Collective over the bootstrap's ranks.
int chb_vmm_create(chb_bootstrap* boot, size_t bytes, int want_multicast, chb_vmm_heap** out, char* err, int errlen) {
  auto fail = [&](int code, const std::string& m) {
    if (err && errlen > 0) std::snprintf(err, (size_t)errlen, "%s", m.c_str());
    return code;
  };
  if (!boot || !out) return fail(CHB_ERR_ARG, "null argument");
  *out = nullptr;
  Driver& d = drv();
  const int P = chb_bootstrap_world(boot), rank = chb_bootstrap_rank(boot);
  // ---- capabilities, agreed by all ranks before anything is allocated
  struct Caps { int driver, fd_handles, multicast; unsigned long long mem_gran, mc_gran; } mine{0, 0, 0, 0, 0};
  CUdevice dev = 0;
  CUmemAllocationProp prop{};
  if (d.load() && d.Init(0) == CUDA_SUCCESS && d.CtxGetDevice(&dev) == CUDA_SUCCESS) {
    mine.driver = 1;
    int v = 0;
    if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev) == CUDA_SUCCESS) mine.fd_handles = v;
    v = 0;
    if (want_multicast && d.has_multicast() &&
        d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) == CUDA_SUCCESS) mine.multicast = v;
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = (int)dev;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t g = 0;
    if (d.MemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS) mine.mem_gran = g;
  }
  std::vector<Caps> all((size_t)P);
  if (chb_bootstrap_allgather(boot, &mine, all.data(), sizeof mine)) return fail(CHB_ERR_OTHER, "capability exchange failed");
  bool usable = true, mcast = want_multicast != 0 && P > 1;
  size_t mem_gran = 0;
  for (const Caps& c : all) {
    usable = usable && c.driver && c.fd_handles && c.mem_gran;
    mcast = mcast && c.multicast;
    mem_gran = c.mem_gran > mem_gran ? (size_t)c.mem_gran : mem_gran;
  }
  if (!usable) return fail(CHB_ERR_UNSUPPORTED, "the CUDA driver, or shareable (file-descriptor) allocation handles, are not available on every rank");
  size_t mc_gran = 0;
  CUmulticastObjectProp mprop{};
  if (mcast) {
    mprop.numDevices = (unsigned)P;
    mprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mprop.size = round_up(bytes ? bytes : 1, mem_gran);
    size_t g = 0;
    if (d.MulticastGetGranularity(&g, &mprop, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS) mc_gran = g;
    // granularities agree by construction (same devices, same size) but are exchanged anyway: all ranks must map the same size
    unsigned long long gq = mc_gran;
    std::vector<unsigned long long> gs((size_t)P);
    if (chb_bootstrap_allgather(boot, &gq, gs.data(), sizeof gq)) return fail(CHB_ERR_OTHER, "granularity exchange failed");
    for (auto x : gs) { if (!x) mcast = false; mc_gran = x > mc_gran ? (size_t)x : mc_gran; }
  }
  auto* hp = new chb_vmm_heap;
  hp->P = P;
  hp->rank = rank;
  hp->device = (int)dev;
  hp->boot = boot;
  hp->bytes = chb_vmm_mapped_size(bytes, mem_gran, mcast ? mc_gran : 0);
  hp->imported.assign((size_t)P, 0);
  hp->va.assign((size_t)P, 0);
  auto bail = [&](int code, const std::string& m) {
    chb_bootstrap_abort(boot);          // peers' waits return at once instead of running into their deadline
    hp->boot = nullptr;                 // and the teardown below must not wait for them either
    chb_vmm_destroy(hp);
    return fail(code, m);
  };
  CUresult r = d.MemCreate(&hp->mine, hp->bytes, &prop, 0);
  if (r != CUDA_SUCCESS) return bail(CHB_ERR_NO_MEM, "cuMemCreate(heap): " + d.why(r));
  int my_fd = -1;
  r = d.MemExportToShareableHandle(&my_fd, hp->mine, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
  if (r != CUDA_SUCCESS) return bail(CHB_ERR_CUDA, "cuMemExportToShareableHandle: " + d.why(r));
  std::vector<int> fds((size_t)P, -1);
  int rc = chb_bootstrap_exchange_fds(boot, my_fd, fds.data());
  if (rc) { close(my_fd); hp->boot = nullptr; chb_vmm_destroy(hp); return fail(rc, "descriptor exchange between the ranks failed"); }
  CUmemAccessDesc access{};
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = (int)dev;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  std::string problem;
  for (int p = 0; p < P && problem.empty(); ++p) {
    CUmemGenericAllocationHandle h = hp->mine;
    if (p != rank) {
      r = d.MemImportFromShareableHandle(&h, (void*)(uintptr_t)fds[(size_t)p], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      if (r != CUDA_SUCCESS) { problem = "import of rank " + std::to_string(p) + "'s heap: " + d.why(r); break; }
      hp->imported[(size_t)p] = h;
    }
    CUdeviceptr va = 0;
    r = d.MemAddressReserve(&va, hp->bytes, mc_gran > mem_gran ? mc_gran : mem_gran, 0, 0);
    if (r != CUDA_SUCCESS) { problem = "cuMemAddressReserve: " + d.why(r); break; }
    r = d.MemMap(va, hp->bytes, 0, h, 0);
    if (r != CUDA_SUCCESS) { d.MemAddressFree(va, hp->bytes); problem = "cuMemMap(rank " + std::to_string(p) + "): " + d.why(r); break; }
    hp->va[(size_t)p] = va;
    r = d.MemSetAccess(va, hp->bytes, &access, 1);
    if (r != CUDA_SUCCESS) problem = "cuMemSetAccess(rank " + std::to_string(p) + "): " + d.why(r);
  }
  for (int p = 0; p < P; ++p) if (fds[(size_t)p] >= 0) close(fds[(size_t)p]);   // imported handles keep the memory alive
  if (!problem.empty()) return bail(CHB_ERR_CUDA, problem);
  // ---- multicast alias
  if (mcast) {
    int mc_fd = -1;
    int created = 1;
    if (rank == 0) {
      mprop.size = hp->bytes;
      r = d.MulticastCreate(&hp->mc, &mprop);
      if (r == CUDA_SUCCESS) r = d.MemExportToShareableHandle(&mc_fd, hp->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
      if (r != CUDA_SUCCESS) { created = 0; mc_fd = -1; if (hp->mc) { d.MemRelease(hp->mc); hp->mc = 0; } }
    }
    std::vector<int> oks((size_t)P);
    if (chb_bootstrap_allgather(boot, &created, oks.data(), sizeof created)) return bail(CHB_ERR_OTHER, "multicast agreement failed");
    if (oks[0]) {
      std::vector<int> mfds((size_t)P, -1);
      rc = chb_bootstrap_exchange_fds(boot, rank == 0 ? mc_fd : -1, mfds.data());
      if (rc) { hp->boot = nullptr; chb_vmm_destroy(hp); return fail(rc, "multicast descriptor exchange failed"); }
      int step_ok = 1;
      if (rank != 0) {
        r = d.MemImportFromShareableHandle(&hp->mc, (void*)(uintptr_t)mfds[0], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
        if (r != CUDA_SUCCESS) { step_ok = 0; hp->mc = 0; }
      }
      if (mfds[0] >= 0) close(mfds[0]);
      if (step_ok && d.MulticastAddDevice(hp->mc, dev) != CUDA_SUCCESS) step_ok = 0;
      // every device is part of the object before anybody binds memory to it
      if (chb_bootstrap_allgather(boot, &step_ok, oks.data(), sizeof step_ok)) return bail(CHB_ERR_OTHER, "multicast agreement failed");
      bool all_ok = true;
      for (int v : oks) all_ok = all_ok && v;
      if (all_ok) {
        r = d.MulticastBindMem(hp->mc, 0, hp->mine, 0, hp->bytes, 0);
        step_ok = r == CUDA_SUCCESS ? 1 : 0;
        hp->mc_bound = step_ok != 0;
        if (step_ok) {
          CUdeviceptr va = 0;
          if (d.MemAddressReserve(&va, hp->bytes, mc_gran, 0, 0) == CUDA_SUCCESS) {
            if (d.MemMap(va, hp->bytes, 0, hp->mc, 0) == CUDA_SUCCESS && d.MemSetAccess(va, hp->bytes, &access, 1) == CUDA_SUCCESS) hp->mc_va = va;
            else { d.MemUnmap(va, hp->bytes); d.MemAddressFree(va, hp->bytes); step_ok = 0; }
          } else step_ok = 0;
        }
        if (chb_bootstrap_allgather(boot, &step_ok, oks.data(), sizeof step_ok)) return bail(CHB_ERR_OTHER, "multicast agreement failed");
        for (int v : oks) all_ok = all_ok && v;
      }
      if (!all_ok) {
        // the alias must work on all ranks or be absent on all: take it down again everywhere
        if (hp->mc_va) { d.MemUnmap(hp->mc_va, hp->bytes); d.MemAddressFree(hp->mc_va, hp->bytes); hp->mc_va = 0; }
        if (hp->mc_bound) { d.MulticastUnbind(hp->mc, dev, 0, hp->bytes); hp->mc_bound = false; }
        chb_bootstrap_barrier(boot);
        if (hp->mc) { d.MemRelease(hp->mc); hp->mc = 0; }
      }
    }
  }
  *out = hp;
  return CHB_SUCCESS;
}

void* chb_vmm_ptr(const chb_vmm_heap* hp, int rank) { return (hp && rank >= 0 && rank < hp->P) ? (void*)hp->va[(size_t)rank] : nullptr; }
void* chb_vmm_multicast_ptr(const chb_vmm_heap* hp) { return hp ? (void*)hp->mc_va : nullptr; }
size_t chb_vmm_bytes(const chb_vmm_heap* hp) { return hp ? hp->bytes : 0; }

}  // extern "C"

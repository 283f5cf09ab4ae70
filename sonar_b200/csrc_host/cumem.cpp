// GPU virtual-memory allocator for sleep / wake-up.
//
// Every allocation is a reserved virtual address range backed by a physical handle of the CUDA
// virtual-memory-management API.  "Sleep" copies the bytes of a tagged set of allocations to host
// memory (or drops them), unmaps and releases the physical memory, and keeps the address range;
// "wake" creates new physical memory, maps it at the SAME address and copies the bytes back.
// Tensors, CUDA graphs and kernel arguments that hold those addresses therefore stay valid across a
// sleep, while the GPU memory is free for another process in between.
//
// sonar_cumem_malloc / sonar_cumem_free have the signature of a PyTorch pluggable allocator
// (torch.cuda.memory.CUDAPluggableAllocator), so a torch MemPool can route the model weights and
// the KV cache through this file.  The allocations made while a tag is current carry that tag.
//
// The driver library is opened at run time (dlopen), so this file builds and loads on machines
// without a GPU; every entry point then returns an error code.
//
// Role parity: the reference's csrc/cumem_allocator.cpp (tagged pools "weights"/"kv_cache",
// offload / discard / restore).
#include <dlfcn.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <map>
#include <mutex>
#include <string>

#include <cuda.h>

#define SONAR_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

struct Driver {
  void* lib = nullptr;
  bool ok = false;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
  CUresult (*MemAddressFree)(CUdeviceptr, size_t);
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
  CUresult (*MemRelease)(CUmemGenericAllocationHandle);
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
  CUresult (*MemUnmap)(CUdeviceptr, size_t);
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
  CUresult (*MemcpyDtoH)(void*, CUdeviceptr, size_t);
  CUresult (*MemcpyHtoD)(CUdeviceptr, const void*, size_t);
  CUresult (*MemHostAlloc)(void**, size_t, unsigned int);
  CUresult (*MemFreeHost)(void*);
  CUresult (*CtxSynchronize)();
  CUresult (*DevicePrimaryCtxRetain)(CUcontext*, CUdevice);
  CUresult (*CtxSetCurrent)(CUcontext);
  CUresult (*CtxGetCurrent)(CUcontext*);
};

Driver g_drv;
std::once_flag g_drv_once;

template <typename F>
bool load_sym(void* lib, F& fn, const char* name) {
  fn = reinterpret_cast<F>(dlsym(lib, name));
  return fn != nullptr;
}

void load_driver() {
  void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) return;
  Driver& d = g_drv;
  d.lib = lib;
  bool ok = true;
  ok &= load_sym(lib, d.MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
  ok &= load_sym(lib, d.MemAddressReserve, "cuMemAddressReserve");
  ok &= load_sym(lib, d.MemAddressFree, "cuMemAddressFree");
  ok &= load_sym(lib, d.MemCreate, "cuMemCreate");
  ok &= load_sym(lib, d.MemRelease, "cuMemRelease");
  ok &= load_sym(lib, d.MemMap, "cuMemMap");
  ok &= load_sym(lib, d.MemUnmap, "cuMemUnmap");
  ok &= load_sym(lib, d.MemSetAccess, "cuMemSetAccess");
  ok &= load_sym(lib, d.MemcpyDtoH, "cuMemcpyDtoH_v2");
  ok &= load_sym(lib, d.MemcpyHtoD, "cuMemcpyHtoD_v2");
  ok &= load_sym(lib, d.MemHostAlloc, "cuMemHostAlloc");
  ok &= load_sym(lib, d.MemFreeHost, "cuMemFreeHost");
  ok &= load_sym(lib, d.CtxSynchronize, "cuCtxSynchronize");
  ok &= load_sym(lib, d.DevicePrimaryCtxRetain, "cuDevicePrimaryCtxRetain");
  ok &= load_sym(lib, d.CtxSetCurrent, "cuCtxSetCurrent");
  ok &= load_sym(lib, d.CtxGetCurrent, "cuCtxGetCurrent");
  d.ok = ok;
}

bool driver() {
  std::call_once(g_drv_once, load_driver);
  return g_drv.ok;
}

struct Block {
  size_t size = 0;            // mapped size (multiple of the granularity)
  int device = 0;
  std::string tag;
  CUmemGenericAllocationHandle handle = 0;
  bool mapped = false;
  void* host_copy = nullptr;  // pinned backup while asleep (offload), else null
};

std::mutex g_mu;
std::map<CUdeviceptr, Block> g_blocks;
std::string g_tag = "default";
int g_last_error = 0;

CUmemAllocationProp prop_for(int device) {
  CUmemAllocationProp p;
  memset(&p, 0, sizeof(p));
  p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  p.location.id = device;
  return p;
}

bool ensure_ctx(int device) {
  CUcontext cur = nullptr;
  if (g_drv.CtxGetCurrent(&cur) == CUDA_SUCCESS && cur != nullptr) return true;
  CUcontext ctx;
  if (g_drv.DevicePrimaryCtxRetain(&ctx, device) != CUDA_SUCCESS) return false;
  return g_drv.CtxSetCurrent(ctx) == CUDA_SUCCESS;
}

// create physical memory and map it at `ptr`
CUresult back(CUdeviceptr ptr, Block& b) {
  CUmemAllocationProp p = prop_for(b.device);
  CUresult rc = g_drv.MemCreate(&b.handle, b.size, &p, 0);
  if (rc != CUDA_SUCCESS) return rc;
  rc = g_drv.MemMap(ptr, b.size, 0, b.handle, 0);
  if (rc != CUDA_SUCCESS) { g_drv.MemRelease(b.handle); b.handle = 0; return rc; }
  CUmemAccessDesc acc;
  memset(&acc, 0, sizeof(acc));
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = b.device;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  rc = g_drv.MemSetAccess(ptr, b.size, &acc, 1);
  if (rc != CUDA_SUCCESS) { g_drv.MemUnmap(ptr, b.size); g_drv.MemRelease(b.handle); b.handle = 0; return rc; }
  b.mapped = true;
  return CUDA_SUCCESS;
}

void unback(CUdeviceptr ptr, Block& b) {
  if (!b.mapped) return;
  g_drv.MemUnmap(ptr, b.size);
  g_drv.MemRelease(b.handle);
  b.handle = 0;
  b.mapped = false;
}

}  // namespace

SONAR_EXPORT int sonar_cumem_available() { return driver() ? 1 : 0; }
SONAR_EXPORT int sonar_cumem_last_error() { return g_last_error; }

SONAR_EXPORT void sonar_cumem_set_tag(const char* tag) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_tag = tag ? tag : "default";
}

// PyTorch pluggable-allocator entry points -------------------------------------------------------
SONAR_EXPORT void* sonar_cumem_malloc(ssize_t size, int device, void* /*stream*/) {
  if (!driver() || size <= 0 || !ensure_ctx(device)) return nullptr;
  CUmemAllocationProp p = prop_for(device);
  size_t gran = 0;
  CUresult rc = g_drv.MemGetAllocationGranularity(&gran, &p, CU_MEM_ALLOC_GRANULARITY_MINIMUM);
  if (rc != CUDA_SUCCESS || gran == 0) { g_last_error = (int)rc; return nullptr; }
  Block b;
  b.size = ((size_t)size + gran - 1) / gran * gran;
  b.device = device;
  CUdeviceptr ptr = 0;
  rc = g_drv.MemAddressReserve(&ptr, b.size, 0, 0, 0);
  if (rc != CUDA_SUCCESS) { g_last_error = (int)rc; return nullptr; }
  rc = back(ptr, b);
  if (rc != CUDA_SUCCESS) { g_last_error = (int)rc; g_drv.MemAddressFree(ptr, b.size); return nullptr; }
  std::lock_guard<std::mutex> lk(g_mu);
  b.tag = g_tag;
  g_blocks[ptr] = b;
  return reinterpret_cast<void*>(ptr);
}

SONAR_EXPORT void sonar_cumem_free(void* p, ssize_t /*size*/, int /*device*/, void* /*stream*/) {
  if (!driver() || p == nullptr) return;
  CUdeviceptr ptr = reinterpret_cast<CUdeviceptr>(p);
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_blocks.find(ptr);
  if (it == g_blocks.end()) return;
  Block& b = it->second;
  unback(ptr, b);
  if (b.host_copy) g_drv.MemFreeHost(b.host_copy);
  g_drv.MemAddressFree(ptr, b.size);
  g_blocks.erase(it);
}

// Sleep: release the physical memory of every live allocation whose tag equals `tag` (all tags if
// null).  offload != 0 keeps a pinned host copy for wake-up.  Returns bytes released, or -1.
SONAR_EXPORT long long sonar_cumem_sleep(const char* tag, int offload) {
  if (!driver()) return -1;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_drv.CtxSynchronize() != CUDA_SUCCESS) return -1;
  long long freed = 0;
  for (auto& kv : g_blocks) {
    Block& b = kv.second;
    if (!b.mapped || (tag && b.tag != tag)) continue;
    if (offload) {
      void* h = nullptr;
      CUresult rc = g_drv.MemHostAlloc(&h, b.size, 0);
      if (rc != CUDA_SUCCESS) { g_last_error = (int)rc; return -1; }
      rc = g_drv.MemcpyDtoH(h, kv.first, b.size);
      if (rc != CUDA_SUCCESS) { g_last_error = (int)rc; g_drv.MemFreeHost(h); return -1; }
      b.host_copy = h;
    }
    unback(kv.first, b);
    freed += (long long)b.size;
  }
  return freed;
}

// Wake: back every sleeping allocation of `tag` (all if null) with new physical memory at its old
// address and restore the offloaded bytes.  Returns bytes mapped, or -1.
SONAR_EXPORT long long sonar_cumem_wake(const char* tag) {
  if (!driver()) return -1;
  std::lock_guard<std::mutex> lk(g_mu);
  long long mapped = 0;
  for (auto& kv : g_blocks) {
    Block& b = kv.second;
    if (b.mapped || (tag && b.tag != tag)) continue;
    if (!ensure_ctx(b.device)) return -1;
    CUresult rc = back(kv.first, b);
    if (rc != CUDA_SUCCESS) { g_last_error = (int)rc; return -1; }
    if (b.host_copy) {
      rc = g_drv.MemcpyHtoD(kv.first, b.host_copy, b.size);
      g_drv.MemFreeHost(b.host_copy);
      b.host_copy = nullptr;
      if (rc != CUDA_SUCCESS) { g_last_error = (int)rc; return -1; }
    }
    mapped += (long long)b.size;
  }
  return mapped;
}

// out[0] = live allocations, out[1] = mapped bytes, out[2] = sleeping bytes, out[3] = host-copy bytes
SONAR_EXPORT void sonar_cumem_stats(const char* tag, long long* out) {
  std::lock_guard<std::mutex> lk(g_mu);
  out[0] = out[1] = out[2] = out[3] = 0;
  for (auto& kv : g_blocks) {
    const Block& b = kv.second;
    if (tag && b.tag != tag) continue;
    out[0] += 1;
    if (b.mapped) out[1] += (long long)b.size; else out[2] += (long long)b.size;
    if (b.host_copy) out[3] += (long long)b.size;
  }
}

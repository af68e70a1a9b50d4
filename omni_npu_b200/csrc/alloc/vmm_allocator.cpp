// Sleep-mode device allocator on CUDA virtual memory management.
//
// Every allocation reserves a virtual address range, creates a physical handle and
// maps it.  `sleep` copies the allocations whose tag is in the offload list to pinned
// host memory and unmaps + releases the physical memory of ALL allocations while
// keeping their virtual addresses reserved; `wake` creates and maps new physical
// memory at the same addresses and copies the saved bytes back.  Tensors that live
// in the pool therefore stay valid objects across a sleep/wake cycle.
//
// The table of allocations lives here, not in Python: malloc/free are called from
// inside the PyTorch caching allocator and must not take the GIL.  The entry points
// `omni_vmm_malloc` / `omni_vmm_free` have the signature torch's
// CUDAPluggableAllocator expects.
//
// The CUDA driver is reached through a table of function pointers, filled from
// libcuda.so.1 at first use.  `omni_vmm_set_driver` installs another table (tests
// install a host-memory fake, so the bookkeeping is testable without a GPU).
//
// Role of the C extension `npu_mem_allocator` used by omni_npu/worker/npu_mem_pool.py:57-96
// (create-and-map / unmap-and-release / memcpy / my_malloc / my_free), with the
// Python-side bookkeeping of NpuMemAllocator (:109-284) folded in.

#include <dlfcn.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

extern "C" {

// Minimal driver-API surface (values follow cuda.h; only what is used is declared so
// the file builds without CUDA headers on a CPU-only host).
typedef int VmmResult;                 // CUresult, 0 = success
typedef unsigned long long VmmDevPtr;  // CUdeviceptr
typedef unsigned long long VmmHandle;  // CUmemGenericAllocationHandle

struct VmmDriver {
  // reserve `size` bytes of virtual address space (alignment = granularity)
  VmmResult (*address_reserve)(VmmDevPtr* ptr, size_t size, size_t alignment);
  VmmResult (*address_free)(VmmDevPtr ptr, size_t size);
  // physical memory on `device`
  VmmResult (*create)(VmmHandle* handle, size_t size, int device);
  VmmResult (*release)(VmmHandle handle);
  VmmResult (*map)(VmmDevPtr ptr, size_t size, VmmHandle handle);
  VmmResult (*set_access_rw)(VmmDevPtr ptr, size_t size, int device);
  VmmResult (*unmap)(VmmDevPtr ptr, size_t size);
  VmmResult (*granularity)(size_t* out, int device);
  VmmResult (*host_alloc)(void** out, size_t size);
  VmmResult (*host_free)(void* p);
  VmmResult (*copy_d2h)(void* dst, VmmDevPtr src, size_t size);
  VmmResult (*copy_h2d)(VmmDevPtr dst, const void* src, size_t size);
  VmmResult (*sync)();
};

}  // extern "C"

namespace {

struct Allocation {
  size_t size = 0;          // mapped size (multiple of the granularity)
  size_t requested = 0;
  int device = 0;
  VmmHandle handle = 0;
  bool mapped = false;
  std::string tag;
  void* host_copy = nullptr;
};

struct State {
  std::mutex mu;
  VmmDriver drv{};
  bool have_driver = false;
  std::map<VmmDevPtr, Allocation> table;
  std::string current_tag = "default";
  bool enabled_tagging = true;
  int last_error = 0;
  char last_error_where[96] = {0};
  unsigned long long n_malloc = 0, n_free = 0, n_sleep = 0, n_wake = 0;
};

State& S() {
  static State s;
  return s;
}

void set_error(State& s, int code, const char* where) {
  s.last_error = code;
  std::snprintf(s.last_error_where, sizeof(s.last_error_where), "%s", where);
}

// ---- real driver, resolved at run time ---------------------------------------------
namespace real {
void* lib = nullptr;
// cuda.h structures, restated with the fields this file sets
struct MemLocation {
  int type;  // CU_MEM_LOCATION_TYPE_DEVICE = 1
  int id;
};
struct AllocationProp {
  int type;                  // CU_MEM_ALLOCATION_TYPE_PINNED = 1
  int requestedHandleTypes;  // 0
  MemLocation location;
  void* win32HandleMetaData;
  struct {
    unsigned char compressionType;
    unsigned char gpuDirectRDMACapable;
    unsigned short usage;
    unsigned char reserved[4];
  } allocFlags;
};
struct AccessDesc {
  MemLocation location;
  int flags;  // CU_MEM_ACCESS_FLAGS_PROT_READWRITE = 3
};
typedef int (*fn_reserve)(VmmDevPtr*, size_t, size_t, VmmDevPtr, unsigned long long);
typedef int (*fn_addr_free)(VmmDevPtr, size_t);
typedef int (*fn_create)(VmmHandle*, size_t, const AllocationProp*, unsigned long long);
typedef int (*fn_release)(VmmHandle);
typedef int (*fn_map)(VmmDevPtr, size_t, size_t, VmmHandle, unsigned long long);
typedef int (*fn_set_access)(VmmDevPtr, size_t, const AccessDesc*, size_t);
typedef int (*fn_unmap)(VmmDevPtr, size_t);
typedef int (*fn_gran)(size_t*, const AllocationProp*, int);
typedef int (*fn_host_alloc)(void**, size_t);
typedef int (*fn_host_free)(void*);
typedef int (*fn_d2h)(void*, VmmDevPtr, size_t);
typedef int (*fn_h2d)(VmmDevPtr, const void*, size_t);
typedef int (*fn_sync)();
fn_reserve p_reserve;
fn_addr_free p_addr_free;
fn_create p_create;
fn_release p_release;
fn_map p_map;
fn_set_access p_set_access;
fn_unmap p_unmap;
fn_gran p_gran;
fn_host_alloc p_host_alloc;
fn_host_free p_host_free;
fn_d2h p_d2h;
fn_h2d p_h2d;
fn_sync p_sync;

AllocationProp prop_for(int device) {
  AllocationProp p;
  std::memset(&p, 0, sizeof(p));
  p.type = 1;
  p.location.type = 1;
  p.location.id = device;
  return p;
}
VmmResult address_reserve(VmmDevPtr* ptr, size_t size, size_t alignment) {
  return p_reserve(ptr, size, alignment, 0, 0);
}
VmmResult address_free(VmmDevPtr ptr, size_t size) { return p_addr_free(ptr, size); }
VmmResult create(VmmHandle* h, size_t size, int device) {
  AllocationProp p = prop_for(device);
  return p_create(h, size, &p, 0);
}
VmmResult release(VmmHandle h) { return p_release(h); }
VmmResult map(VmmDevPtr ptr, size_t size, VmmHandle h) { return p_map(ptr, size, 0, h, 0); }
VmmResult set_access_rw(VmmDevPtr ptr, size_t size, int device) {
  AccessDesc d;
  d.location.type = 1;
  d.location.id = device;
  d.flags = 3;
  return p_set_access(ptr, size, &d, 1);
}
VmmResult unmap(VmmDevPtr ptr, size_t size) { return p_unmap(ptr, size); }
VmmResult granularity(size_t* out, int device) {
  AllocationProp p = prop_for(device);
  return p_gran(out, &p, 0 /* CU_MEM_ALLOC_GRANULARITY_MINIMUM */);
}
VmmResult host_alloc(void** out, size_t size) { return p_host_alloc(out, size); }
VmmResult host_free(void* p) { return p_host_free(p); }
VmmResult copy_d2h(void* dst, VmmDevPtr src, size_t size) { return p_d2h(dst, src, size); }
VmmResult copy_h2d(VmmDevPtr dst, const void* src, size_t size) { return p_h2d(dst, src, size); }
VmmResult sync() { return p_sync(); }

bool load(VmmDriver* out) {
  lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
  if (!lib) return false;
#define OMNI_SYM(var, type, name)                \
  var = reinterpret_cast<type>(dlsym(lib, name)); \
  if (!var) return false;
  OMNI_SYM(p_reserve, fn_reserve, "cuMemAddressReserve")
  OMNI_SYM(p_addr_free, fn_addr_free, "cuMemAddressFree")
  OMNI_SYM(p_create, fn_create, "cuMemCreate")
  OMNI_SYM(p_release, fn_release, "cuMemRelease")
  OMNI_SYM(p_map, fn_map, "cuMemMap")
  OMNI_SYM(p_set_access, fn_set_access, "cuMemSetAccess")
  OMNI_SYM(p_unmap, fn_unmap, "cuMemUnmap")
  OMNI_SYM(p_gran, fn_gran, "cuMemGetAllocationGranularity")
  OMNI_SYM(p_host_alloc, fn_host_alloc, "cuMemAllocHost_v2")
  OMNI_SYM(p_host_free, fn_host_free, "cuMemFreeHost")
  OMNI_SYM(p_d2h, fn_d2h, "cuMemcpyDtoH_v2")
  OMNI_SYM(p_h2d, fn_h2d, "cuMemcpyHtoD_v2")
  OMNI_SYM(p_sync, fn_sync, "cuCtxSynchronize")
#undef OMNI_SYM
  out->address_reserve = address_reserve;
  out->address_free = address_free;
  out->create = create;
  out->release = release;
  out->map = map;
  out->set_access_rw = set_access_rw;
  out->unmap = unmap;
  out->granularity = granularity;
  out->host_alloc = host_alloc;
  out->host_free = host_free;
  out->copy_d2h = copy_d2h;
  out->copy_h2d = copy_h2d;
  out->sync = sync;
  return true;
}
}  // namespace real

bool ensure_driver(State& s) {
  if (s.have_driver) return true;
  if (!real::load(&s.drv)) {
    set_error(s, -1, "libcuda.so.1 not available");
    return false;
  }
  s.have_driver = true;
  return true;
}

bool tag_listed(const std::string& tag, const char* const* tags, int n) {
  for (int i = 0; i < n; ++i)
    if (tags[i] && tag == tags[i]) return true;
  return false;
}

}  // namespace

extern "C" {

// Install a driver table (tests).  Passing nullptr goes back to libcuda.
void omni_vmm_set_driver(const VmmDriver* drv) {
  State& s = S();
  std::lock_guard<std::mutex> g(s.mu);
  if (drv) {
    s.drv = *drv;
    s.have_driver = true;
  } else {
    s.have_driver = false;
  }
}

void omni_vmm_set_tag(const char* tag) {
  State& s = S();
  std::lock_guard<std::mutex> g(s.mu);
  s.current_tag = tag ? tag : "default";
}

// torch CUDAPluggableAllocator malloc: (size, device, stream) -> device pointer
void* omni_vmm_malloc(long long size, int device, void* /*stream*/) {
  State& s = S();
  std::lock_guard<std::mutex> g(s.mu);
  if (!ensure_driver(s) || size <= 0) return nullptr;
  size_t gran = 0;
  int rc = s.drv.granularity(&gran, device);
  if (rc != 0 || gran == 0) {
    set_error(s, rc, "granularity");
    return nullptr;
  }
  Allocation a;
  a.requested = static_cast<size_t>(size);
  a.size = (a.requested + gran - 1) / gran * gran;
  a.device = device;
  a.tag = s.current_tag;
  VmmDevPtr ptr = 0;
  if ((rc = s.drv.address_reserve(&ptr, a.size, gran)) != 0) {
    set_error(s, rc, "address_reserve");
    return nullptr;
  }
  if ((rc = s.drv.create(&a.handle, a.size, device)) != 0) {
    set_error(s, rc, "create");
    s.drv.address_free(ptr, a.size);
    return nullptr;
  }
  if ((rc = s.drv.map(ptr, a.size, a.handle)) != 0 || (rc = s.drv.set_access_rw(ptr, a.size, device)) != 0) {
    set_error(s, rc, "map");
    s.drv.release(a.handle);
    s.drv.address_free(ptr, a.size);
    return nullptr;
  }
  a.mapped = true;
  s.table[ptr] = a;
  ++s.n_malloc;
  return reinterpret_cast<void*>(ptr);
}

// torch CUDAPluggableAllocator free: (ptr, size, device, stream)
void omni_vmm_free(void* p, long long /*size*/, int /*device*/, void* /*stream*/) {
  State& s = S();
  std::lock_guard<std::mutex> g(s.mu);
  const VmmDevPtr ptr = reinterpret_cast<VmmDevPtr>(p);
  auto it = s.table.find(ptr);
  if (it == s.table.end()) return;
  Allocation& a = it->second;
  if (a.mapped) {
    s.drv.unmap(ptr, a.size);
    s.drv.release(a.handle);
  }
  if (a.host_copy) s.drv.host_free(a.host_copy);
  s.drv.address_free(ptr, a.size);
  s.table.erase(it);
  ++s.n_free;
}

// Offload the allocations tagged with one of `offload_tags` to pinned host memory,
// then give the physical memory of every allocation back.  Returns the number of
// bytes released, or a negative driver error.
long long omni_vmm_sleep(const char* const* offload_tags, int n_tags) {
  State& s = S();
  std::lock_guard<std::mutex> g(s.mu);
  if (!s.have_driver) return 0;
  int rc = s.drv.sync();
  if (rc != 0) {
    set_error(s, rc, "sync");
    return -1;
  }
  long long released = 0;
  for (auto& kv : s.table) {
    Allocation& a = kv.second;
    if (!a.mapped) continue;
    if (tag_listed(a.tag, offload_tags, n_tags)) {
      if (!a.host_copy && (rc = s.drv.host_alloc(&a.host_copy, a.size)) != 0) {
        a.host_copy = nullptr;
        set_error(s, rc, "host_alloc");
        return -1;
      }
      if ((rc = s.drv.copy_d2h(a.host_copy, kv.first, a.size)) != 0) {
        set_error(s, rc, "copy_d2h");
        return -1;
      }
    }
    if ((rc = s.drv.unmap(kv.first, a.size)) != 0 || (rc = s.drv.release(a.handle)) != 0) {
      set_error(s, rc, "unmap");
      return -1;
    }
    a.mapped = false;
    a.handle = 0;
    released += static_cast<long long>(a.size);
  }
  ++s.n_sleep;
  return released;
}

// Map new physical memory for the allocations whose tag is listed (all when n_tags == 0)
// and restore what was offloaded.  Returns the bytes mapped, or a negative error.
long long omni_vmm_wake(const char* const* tags, int n_tags) {
  State& s = S();
  std::lock_guard<std::mutex> g(s.mu);
  if (!s.have_driver) return 0;
  long long mapped = 0;
  int rc;
  for (auto& kv : s.table) {
    Allocation& a = kv.second;
    if (a.mapped) continue;
    if (n_tags > 0 && !tag_listed(a.tag, tags, n_tags)) continue;
    if ((rc = s.drv.create(&a.handle, a.size, a.device)) != 0) {
      set_error(s, rc, "create (wake)");
      return -1;
    }
    if ((rc = s.drv.map(kv.first, a.size, a.handle)) != 0 ||
        (rc = s.drv.set_access_rw(kv.first, a.size, a.device)) != 0) {
      set_error(s, rc, "map (wake)");
      s.drv.release(a.handle);
      return -1;
    }
    a.mapped = true;
    if (a.host_copy) {
      if ((rc = s.drv.copy_h2d(kv.first, a.host_copy, a.size)) != 0) {
        set_error(s, rc, "copy_h2d");
        return -1;
      }
      s.drv.host_free(a.host_copy);
      a.host_copy = nullptr;
    }
    mapped += static_cast<long long>(a.size);
  }
  ++s.n_wake;
  return mapped;
}

// out[0] live allocations, [1] mapped bytes, [2] unmapped (sleeping) bytes, [3] host backup
// bytes, [4] mallocs, [5] frees, [6] sleeps, [7] wakes
void omni_vmm_stats(long long* out) {
  State& s = S();
  std::lock_guard<std::mutex> g(s.mu);
  long long mapped = 0, unmapped = 0, host = 0;
  for (auto& kv : s.table) {
    (kv.second.mapped ? mapped : unmapped) += static_cast<long long>(kv.second.size);
    if (kv.second.host_copy) host += static_cast<long long>(kv.second.size);
  }
  out[0] = static_cast<long long>(s.table.size());
  out[1] = mapped;
  out[2] = unmapped;
  out[3] = host;
  out[4] = static_cast<long long>(s.n_malloc);
  out[5] = static_cast<long long>(s.n_free);
  out[6] = static_cast<long long>(s.n_sleep);
  out[7] = static_cast<long long>(s.n_wake);
}

// Bytes in use by allocations with this tag (nullptr = all tags).
long long omni_vmm_usage(const char* tag) {
  State& s = S();
  std::lock_guard<std::mutex> g(s.mu);
  long long n = 0;
  for (auto& kv : s.table)
    if (!tag || kv.second.tag == tag) n += static_cast<long long>(kv.second.size);
  return n;
}

int omni_vmm_last_error(char* where, int cap) {
  State& s = S();
  std::lock_guard<std::mutex> g(s.mu);
  if (where && cap > 0) std::snprintf(where, static_cast<size_t>(cap), "%s", s.last_error_where);
  return s.last_error;
}

}  // extern "C"

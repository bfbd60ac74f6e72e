// Implementation of the cuMem region layer (see vmm.h).
#include "vmm.h"

#include <cuda.h>
#include <dlfcn.h>
#include <fcntl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <unistd.h>

#include <chrono>
#include <map>
#include <mutex>
#include <vector>

#ifndef MFD_CLOEXEC
#define MFD_CLOEXEC 0x0001U
#endif

namespace {

thread_local char g_err[512] = "";
void set_err(const char* fmt, const char* what, long code) { snprintf(g_err, sizeof g_err, fmt, what, code); }

// ------------------------------------------------------------------------------------------------
// driver abstraction
// ------------------------------------------------------------------------------------------------
struct Driver {
  virtual ~Driver() {}
  virtual int granularity(int dev, size_t* out) = 0;
  virtual int create(int dev, size_t bytes, uint64_t* h) = 0;
  virtual int release(uint64_t h) = 0;
  virtual int reserve(size_t bytes, size_t align, uintptr_t* va) = 0;
  virtual int free_va(uintptr_t va, size_t bytes) = 0;
  virtual int map(uintptr_t va, size_t bytes, uint64_t h) = 0;
  virtual int unmap(uintptr_t va, size_t bytes) = 0;
  virtual int set_access(uintptr_t va, size_t bytes, int dev) = 0;
  virtual int export_fd(uint64_t h, int* fd) = 0;
  virtual int import_fd(int fd, uint64_t* h) = 0;
  virtual int retain(void* ptr, uint64_t* h) = 0;
  virtual int copy(uintptr_t dst, uintptr_t src, size_t n) = 0;
  virtual int any_copy(void* dst, const void* src, size_t n) = 0;
  virtual int device_count() = 0;
  virtual int pointer_device(const void* ptr) = 0;   // -1 when unknown
  virtual int address_range(const void* ptr, uintptr_t* base, size_t* size) { (void)ptr; (void)base; (void)size; return 1; }
  // A dma-buf descriptor for [ptr, ptr + size): *offset is where ptr lies inside the exported range.
  virtual int dmabuf_fd(const void* ptr, size_t size, int* fd, uint64_t* offset) { (void)ptr; (void)size; (void)fd; (void)offset; return 1; }
};

// ---- real CUDA driver, resolved at run time -----------------------------------------------------
struct CudaDriver : Driver {
  void* lib = nullptr;
  CUresult (*GetProcAddress)(const char*, void**, int, cuuint64_t, CUdriverProcAddressQueryResult*) = nullptr;
  CUresult (*Init)(unsigned) = nullptr;
  CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MemRetainAllocationHandle)(CUmemGenericAllocationHandle*, void*) = nullptr;
  CUresult (*MemcpyDtoD)(CUdeviceptr, CUdeviceptr, size_t) = nullptr;
  CUresult (*CtxSynchronize)() = nullptr;
  CUresult (*Memcpy)(CUdeviceptr, CUdeviceptr, size_t) = nullptr;
  CUresult (*DeviceGetCount)(int*) = nullptr;
  CUresult (*PointerGetAttribute)(void*, CUpointer_attribute, CUdeviceptr) = nullptr;
  CUresult (*MemGetAddressRange)(CUdeviceptr*, size_t*, CUdeviceptr) = nullptr;
  CUresult (*MemGetHandleForAddressRange)(void*, CUdeviceptr, size_t, CUmemRangeHandleType, unsigned long long) = nullptr;
  CUresult (*StreamCreate)(CUstream*, unsigned int) = nullptr;
  CUresult (*StreamSynchronize)(CUstream) = nullptr;
  CUresult (*MemcpyAsync)(CUdeviceptr, CUdeviceptr, size_t, CUstream) = nullptr;
  CUresult (*CtxGetCurrent)(CUcontext*) = nullptr;

  template <class F>
  bool sym(const char* name, F& fn) {
    void* p = nullptr;
    CUdriverProcAddressQueryResult q;
    if (GetProcAddress(name, &p, 12000, CU_GET_PROC_ADDRESS_DEFAULT, &q) != CUDA_SUCCESS || !p) {
      set_err("driver symbol %s not found (%ld)", name, 0);
      return false;
    }
    fn = reinterpret_cast<F>(p);
    return true;
  }
  bool load() {
    lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) {
      set_err("%s: cannot dlopen libcuda.so.1 (%ld)", "vmm", 0);
      return false;
    }
    GetProcAddress = reinterpret_cast<decltype(GetProcAddress)>(dlsym(lib, "cuGetProcAddress_v2"));
    if (!GetProcAddress) {
      set_err("%s: cuGetProcAddress_v2 missing (%ld)", "vmm", 0);
      return false;
    }
    bool ok = sym("cuInit", Init) && sym("cuGetErrorString", GetErrorString) &&
              sym("cuDeviceGetAttribute", DeviceGetAttribute) &&
              sym("cuMemGetAllocationGranularity", MemGetAllocationGranularity) && sym("cuMemCreate", MemCreate) &&
              sym("cuMemRelease", MemRelease) && sym("cuMemAddressReserve", MemAddressReserve) &&
              sym("cuMemAddressFree", MemAddressFree) && sym("cuMemMap", MemMap) && sym("cuMemUnmap", MemUnmap) &&
              sym("cuMemSetAccess", MemSetAccess) && sym("cuMemExportToShareableHandle", MemExportToShareableHandle) &&
              sym("cuMemImportFromShareableHandle", MemImportFromShareableHandle) &&
              sym("cuMemRetainAllocationHandle", MemRetainAllocationHandle) && sym("cuMemcpyDtoD", MemcpyDtoD) &&
              sym("cuCtxSynchronize", CtxSynchronize);
    if (!ok) return false;
    // used only by the plugin's device-buffer registration: their absence must not disable the region layer
    (void)sym("cuMemcpy", Memcpy);
    (void)sym("cuDeviceGetCount", DeviceGetCount);
    (void)sym("cuPointerGetAttribute", PointerGetAttribute);
    (void)sym("cuMemGetAddressRange", MemGetAddressRange);
    (void)sym("cuMemGetHandleForAddressRange", MemGetHandleForAddressRange);
    (void)sym("cuStreamCreate", StreamCreate);
    (void)sym("cuStreamSynchronize", StreamSynchronize);
    (void)sym("cuMemcpyAsync", MemcpyAsync);
    (void)sym("cuCtxGetCurrent", CtxGetCurrent);
    g_err[0] = 0;
    return chk(Init(0), "cuInit") == 0;
  }
  int chk(CUresult r, const char* what) {
    if (r == CUDA_SUCCESS) return 0;
    const char* s = nullptr;
    if (GetErrorString) GetErrorString(r, &s);
    snprintf(g_err, sizeof g_err, "%s failed: %s (CUresult %d)", what, s ? s : "?", (int)r);
    return (int)r;
  }
  CUmemAllocationProp prop(int dev) {
    CUmemAllocationProp p;
    memset(&p, 0, sizeof p);
    p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    p.location.id = dev;
    p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    int gdr = 0;
    if (DeviceGetAttribute(&gdr, CU_DEVICE_ATTRIBUTE_GPU_DIRECT_RDMA_WITH_CUDA_VMM_SUPPORTED, dev) == CUDA_SUCCESS && gdr)
      p.allocFlags.gpuDirectRDMACapable = 1;  // a NIC may read these pages (src/fuselink.cc:26)
    return p;
  }
  int granularity(int dev, size_t* out) override {
    CUmemAllocationProp p = prop(dev);
    // the granularity is queried BEFORE any size arithmetic (the reference divides by it first, src/fuselink.cc:15-17)
    return chk(MemGetAllocationGranularity(out, &p, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
  }
  int create(int dev, size_t bytes, uint64_t* h) override {
    CUmemAllocationProp p = prop(dev);
    CUmemGenericAllocationHandle hh;
    int rc = chk(MemCreate(&hh, bytes, &p, 0), "cuMemCreate");
    *h = (uint64_t)hh;
    return rc;
  }
  int release(uint64_t h) override { return chk(MemRelease((CUmemGenericAllocationHandle)h), "cuMemRelease"); }
  int reserve(size_t bytes, size_t align, uintptr_t* va) override {
    CUdeviceptr p = 0;
    int rc = chk(MemAddressReserve(&p, bytes, align, 0, 0), "cuMemAddressReserve");
    *va = (uintptr_t)p;
    return rc;
  }
  int free_va(uintptr_t va, size_t bytes) override { return chk(MemAddressFree((CUdeviceptr)va, bytes), "cuMemAddressFree"); }
  int map(uintptr_t va, size_t bytes, uint64_t h) override {
    return chk(MemMap((CUdeviceptr)va, bytes, 0, (CUmemGenericAllocationHandle)h, 0), "cuMemMap");
  }
  int unmap(uintptr_t va, size_t bytes) override { return chk(MemUnmap((CUdeviceptr)va, bytes), "cuMemUnmap"); }
  int set_access(uintptr_t va, size_t bytes, int dev) override {
    CUmemAccessDesc d;
    memset(&d, 0, sizeof d);
    d.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    d.location.id = dev;
    d.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    return chk(MemSetAccess((CUdeviceptr)va, bytes, &d, 1), "cuMemSetAccess");
  }
  int export_fd(uint64_t h, int* fd) override {
    return chk(MemExportToShareableHandle(fd, (CUmemGenericAllocationHandle)h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
               "cuMemExportToShareableHandle");
  }
  int import_fd(int fd, uint64_t* h) override {
    CUmemGenericAllocationHandle hh;
    int rc = chk(MemImportFromShareableHandle(&hh, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR),
                 "cuMemImportFromShareableHandle");
    *h = (uint64_t)hh;
    return rc;
  }
  int retain(void* ptr, uint64_t* h) override {
    CUmemGenericAllocationHandle hh;
    int rc = chk(MemRetainAllocationHandle(&hh, ptr), "cuMemRetainAllocationHandle");
    *h = (uint64_t)hh;
    return rc;
  }
  // Copies run on a stream of their own (non-blocking, one per thread and context) and only that stream is waited for.
  // A synchronous cuMemcpy or a context-wide synchronise would also wait for every kernel on the default stream -- and a
  // communication library's progress thread that calls into this layer must never wait for the kernels it is feeding.
  CUstream private_stream() {
    if (!StreamCreate || !StreamSynchronize || !MemcpyAsync || !CtxGetCurrent) return nullptr;
    static thread_local std::map<CUcontext, CUstream> streams;
    CUcontext ctx = nullptr;
    if (CtxGetCurrent(&ctx) != CUDA_SUCCESS || !ctx) return nullptr;
    auto it = streams.find(ctx);
    if (it != streams.end()) return it->second;
    CUstream st = nullptr;
    if (StreamCreate(&st, CU_STREAM_NON_BLOCKING) != CUDA_SUCCESS) return nullptr;
    streams[ctx] = st;
    return st;
  }
  int copy(uintptr_t dst, uintptr_t src, size_t n) override {
    if (CUstream st = private_stream()) {
      int rc = chk(MemcpyAsync((CUdeviceptr)dst, (CUdeviceptr)src, n, st), "cuMemcpyAsync");
      if (rc) return rc;
      return chk(StreamSynchronize(st), "cuStreamSynchronize");
    }
    int rc = chk(MemcpyDtoD((CUdeviceptr)dst, (CUdeviceptr)src, n), "cuMemcpyDtoD");
    if (rc) return rc;
    return chk(CtxSynchronize(), "cuCtxSynchronize");
  }
  int any_copy(void* dst, const void* src, size_t n) override {
    if (CUstream st = private_stream()) {
      int rc = chk(MemcpyAsync((CUdeviceptr)(uintptr_t)dst, (CUdeviceptr)(uintptr_t)src, n, st), "cuMemcpyAsync");
      if (rc) return rc;
      return chk(StreamSynchronize(st), "cuStreamSynchronize");
    }
    if (!Memcpy) { set_err("%s: cuMemcpy not available (%ld)", "vmm", 0); return 1; }
    return chk(Memcpy((CUdeviceptr)(uintptr_t)dst, (CUdeviceptr)(uintptr_t)src, n), "cuMemcpy");
  }
  int device_count() override {
    int n = 0;
    return DeviceGetCount && DeviceGetCount(&n) == CUDA_SUCCESS ? n : 0;
  }
  int address_range(const void* ptr, uintptr_t* base, size_t* size) override {
    if (!MemGetAddressRange) return 1;
    CUdeviceptr b = 0;
    size_t n = 0;
    if (MemGetAddressRange(&b, &n, (CUdeviceptr)(uintptr_t)ptr) != CUDA_SUCCESS || !n) return 1;
    *base = (uintptr_t)b;
    *size = n;
    return 0;
  }
  int dmabuf_fd(const void* ptr, size_t size, int* fd, uint64_t* offset) override {
    if (!MemGetHandleForAddressRange) { set_err("%s: cuMemGetHandleForAddressRange not available (%ld)", "vmm", 0); return 1; }
    // address and size have to be multiples of the host page size: export the pages around the range
    const uintptr_t page = (uintptr_t)sysconf(_SC_PAGESIZE);
    const uintptr_t lo = (uintptr_t)ptr / page * page;
    const uintptr_t hi = ((uintptr_t)ptr + size + page - 1) / page * page;
    int out = -1;
    int rc = chk(MemGetHandleForAddressRange(&out, (CUdeviceptr)lo, hi - lo, CU_MEM_RANGE_HANDLE_TYPE_DMA_BUF_FD, 0),
                 "cuMemGetHandleForAddressRange");
    if (rc) return rc;
    *fd = out;
    *offset = (uintptr_t)ptr - lo;
    return 0;
  }
  int pointer_device(const void* ptr) override {
    int ord = -1;
    if (!PointerGetAttribute) return -1;
    if (PointerGetAttribute(&ord, CU_POINTER_ATTRIBUTE_DEVICE_ORDINAL, (CUdeviceptr)(uintptr_t)ptr) != CUDA_SUCCESS) return -1;
    return ord;
  }
};

// ---- fake driver: physical memory = memfd, mapping = mmap(MAP_SHARED|MAP_FIXED) ------------------
struct FakeDriver : Driver {
  std::mutex mu;
  std::map<uint64_t, size_t> handles;       // handle (an fd) -> bytes
  std::map<uintptr_t, uint64_t> mapped;     // va -> handle
  int granularity(int, size_t* out) override { *out = 2u << 20; return 0; }
  int create(int, size_t bytes, uint64_t* h) override {
    int fd = (int)syscall(319 /*memfd_create*/, "fl_vmm_fake", MFD_CLOEXEC);
    if (fd < 0 || ftruncate(fd, (off_t)bytes) != 0) { set_err("%s: memfd_create/ftruncate failed (%ld)", "fake", fd); return 1; }
    std::lock_guard<std::mutex> l(mu);
    handles[(uint64_t)fd] = bytes;
    *h = (uint64_t)fd;
    return 0;
  }
  int release(uint64_t h) override {
    std::lock_guard<std::mutex> l(mu);
    handles.erase(h);
    close((int)h);
    return 0;
  }
  int reserve(size_t bytes, size_t, uintptr_t* va) override {
    void* p = mmap(nullptr, bytes, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
    if (p == MAP_FAILED) { set_err("%s: mmap reserve failed (%ld)", "fake", 0); return 1; }
    *va = (uintptr_t)p;
    return 0;
  }
  int free_va(uintptr_t va, size_t bytes) override { return munmap((void*)va, bytes) == 0 ? 0 : 1; }
  int map(uintptr_t va, size_t bytes, uint64_t h) override {
    void* p = mmap((void*)va, bytes, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_FIXED, (int)h, 0);
    if (p == MAP_FAILED) { set_err("%s: mmap map failed (%ld)", "fake", 0); return 1; }
    std::lock_guard<std::mutex> l(mu);
    mapped[va] = h;
    return 0;
  }
  int unmap(uintptr_t va, size_t bytes) override {
    void* p = mmap((void*)va, bytes, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE | MAP_FIXED, -1, 0);
    std::lock_guard<std::mutex> l(mu);
    mapped.erase(va);
    return p == MAP_FAILED ? 1 : 0;
  }
  int set_access(uintptr_t, size_t, int) override { return 0; }
  int export_fd(uint64_t h, int* fd) override { *fd = dup((int)h); return *fd < 0 ? 1 : 0; }
  int import_fd(int fd, uint64_t* h) override {
    int d = dup(fd);
    if (d < 0) return 1;
    off_t sz = lseek(d, 0, SEEK_END);
    std::lock_guard<std::mutex> l(mu);
    handles[(uint64_t)d] = (size_t)sz;
    *h = (uint64_t)d;
    return 0;
  }
  int retain(void* ptr, uint64_t* h) override {
    std::lock_guard<std::mutex> l(mu);
    auto it = mapped.find((uintptr_t)ptr);
    if (it == mapped.end()) { set_err("%s: pointer is not the base of a mapping (%ld)", "fake", 0); return 1; }
    int d = dup((int)it->second);
    handles[(uint64_t)d] = handles[it->second];
    *h = (uint64_t)d;
    return 0;
  }
  int copy(uintptr_t dst, uintptr_t src, size_t n) override { memcpy((void*)dst, (void*)src, n); return 0; }
  int any_copy(void* dst, const void* src, size_t n) override { memcpy(dst, src, n); return 0; }
  int device_count() override {
    const char* e = getenv("FUSELINK_VMM_FAKE_NGPUS");
    return e ? atoi(e) : 8;
  }
  int pointer_device(const void*) override { return -1; }
  // the memfd behind the mapping that contains ptr stands in for the dma-buf
  int dmabuf_fd(const void* ptr, size_t size, int* fd, uint64_t* offset) override {
    std::lock_guard<std::mutex> l(mu);
    auto it = mapped.upper_bound((uintptr_t)ptr);
    if (it == mapped.begin()) { set_err("%s: pointer is not inside a mapping (%ld)", "fake", 0); return 1; }
    --it;
    const size_t bytes = handles[it->second];
    if ((uintptr_t)ptr + size > it->first + bytes) { set_err("%s: range crosses the end of its mapping (%ld)", "fake", 0); return 1; }
    const int d = dup((int)it->second);
    if (d < 0) return 1;
    *fd = d;
    *offset = (uintptr_t)ptr - it->first;
    return 0;
  }
};

Driver* g_drv = nullptr;
int g_backend = -1;
std::mutex g_mu;

struct Slab {
  uint64_t handle = 0;
  int device = -1;
  bool mapped = false;
};

}  // namespace

struct FlVmmRegion {
  uintptr_t va = 0;
  size_t size = 0;
  size_t slab_bytes = 0;
  std::vector<Slab> slabs;
  std::vector<int> access;  // devices granted RW
  bool owns_va = true;      // adopted regions keep the foreign VA reservation
  bool owns_phys = true;    // aliases / imports hold their own references but did not allocate
  bool pooled = false;      // slabs come from (and return to) the slab pool
};

namespace {
std::map<uintptr_t, FlVmmRegion*> g_regions;  // by base VA
std::map<int, size_t> g_usage;

size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int map_all(FlVmmRegion* r) {
  for (size_t i = 0; i < r->slabs.size(); ++i) {
    int rc = g_drv->map(r->va + i * r->slab_bytes, r->slab_bytes, r->slabs[i].handle);
    if (rc) return rc;
    r->slabs[i].mapped = true;
  }
  for (int dev : r->access) {
    int rc = g_drv->set_access(r->va, r->size, dev);
    if (rc) return rc;
  }
  return 0;
}
void register_region(FlVmmRegion* r) {
  std::lock_guard<std::mutex> l(g_mu);
  g_regions[r->va] = r;
}
}  // namespace

extern "C" {

const char* fl_vmm_last_error(void) { return g_err; }
int fl_vmm_backend(void) { return g_backend; }

int fl_vmm_init(int backend) {
  std::lock_guard<std::mutex> l(g_mu);
  if (g_drv && g_backend == backend) return 0;
  if (g_drv && !g_regions.empty()) {
    set_err("%s: cannot switch backend while regions exist (%ld)", "vmm", (long)g_regions.size());
    return 1;
  }
  delete g_drv;
  g_drv = nullptr;
  g_backend = -1;
  if (backend == 1) {
    g_drv = new FakeDriver();
  } else {
    CudaDriver* d = new CudaDriver();
    if (!d->load()) {
      delete d;
      return 1;
    }
    g_drv = d;
  }
  g_backend = backend;
  return 0;
}

int fl_vmm_granularity(int device, size_t* out) {
  if (!g_drv) { set_err("%s: fl_vmm_init not called (%ld)", "vmm", 0); return 1; }
  return g_drv->granularity(device, out);
}

FlVmmRegion* fl_vmm_create(int device, size_t size, size_t slab_bytes) {
  if (!g_drv) { set_err("%s: fl_vmm_init not called (%ld)", "vmm", 0); return nullptr; }
  size_t gran = 0;
  if (g_drv->granularity(device, &gran) || gran == 0) return nullptr;
  if (size == 0) { set_err("%s: zero-sized region (%ld)", "vmm", 0); return nullptr; }
  if (slab_bytes == 0) slab_bytes = round_up(size, gran);
  slab_bytes = round_up(slab_bytes, gran);
  FlVmmRegion* r = new FlVmmRegion();
  r->slab_bytes = slab_bytes;
  r->size = round_up(size, slab_bytes);
  const size_t n = r->size / slab_bytes;
  if (g_drv->reserve(r->size, slab_bytes > gran ? gran : slab_bytes, &r->va)) { delete r; return nullptr; }
  r->access.push_back(device);
  for (size_t i = 0; i < n; ++i) {
    Slab s;
    if (g_drv->create(device, slab_bytes, &s.handle)) { fl_vmm_destroy(r); return nullptr; }
    s.device = device;
    r->slabs.push_back(s);
    std::lock_guard<std::mutex> l(g_mu);
    g_usage[device] += slab_bytes;
  }
  if (map_all(r)) { fl_vmm_destroy(r); return nullptr; }
  register_region(r);
  return r;
}

FlVmmRegion* fl_vmm_adopt(void* ptr, size_t size, int owner_device) {
  if (!g_drv) { set_err("%s: fl_vmm_init not called (%ld)", "vmm", 0); return nullptr; }
  size_t gran = 0;
  if (g_drv->granularity(owner_device, &gran) || gran == 0) return nullptr;
  if (((uintptr_t)ptr % gran) || size == 0) { set_err("%s: adopted pointer must be granularity aligned (%ld)", "vmm", (long)gran); return nullptr; }
  FlVmmRegion* r = new FlVmmRegion();
  r->va = (uintptr_t)ptr;
  r->size = round_up(size, gran);
  r->slab_bytes = r->size;
  r->owns_va = false;
  r->owns_phys = false;     // the memory behind the address was allocated elsewhere: it is not in this layer's usage count
  r->access.push_back(owner_device);
  Slab s;
  if (g_drv->retain(ptr, &s.handle)) { delete r; return nullptr; }
  s.device = owner_device;
  s.mapped = true;
  r->slabs.push_back(s);
  register_region(r);
  return r;
}

FlVmmRegion* fl_vmm_import(int device, const int* fds, int nslabs, size_t slab_bytes) {
  if (!g_drv) { set_err("%s: fl_vmm_init not called (%ld)", "vmm", 0); return nullptr; }
  if (nslabs < 1 || slab_bytes == 0) { set_err("%s: bad import arguments (%ld)", "vmm", nslabs); return nullptr; }
  FlVmmRegion* r = new FlVmmRegion();
  r->slab_bytes = slab_bytes;
  r->size = slab_bytes * (size_t)nslabs;
  r->owns_phys = false;
  size_t gran = 0;
  if (g_drv->granularity(device, &gran) || g_drv->reserve(r->size, gran, &r->va)) { delete r; return nullptr; }
  r->access.push_back(device);
  for (int i = 0; i < nslabs; ++i) {
    Slab s;
    if (g_drv->import_fd(fds[i], &s.handle)) { fl_vmm_destroy(r); return nullptr; }
    s.device = -1;  // physical location is the exporter's business
    r->slabs.push_back(s);
  }
  if (map_all(r)) { fl_vmm_destroy(r); return nullptr; }
  register_region(r);
  return r;
}

FlVmmRegion* fl_vmm_alias(FlVmmRegion* src, int device) {
  if (!g_drv || !src) return nullptr;
  std::vector<int> fds;
  for (auto& s : src->slabs) {
    int fd = -1;
    if (g_drv->export_fd(s.handle, &fd)) { for (int f : fds) close(f); return nullptr; }
    fds.push_back(fd);
  }
  FlVmmRegion* r = fl_vmm_import(device, fds.data(), (int)fds.size(), src->slab_bytes);
  for (int f : fds) close(f);
  if (r) for (size_t i = 0; i < r->slabs.size(); ++i) r->slabs[i].device = src->slabs[i].device;
  return r;
}

void fl_vmm_destroy(FlVmmRegion* r) {
  if (!r || !g_drv) return;
  {
    std::lock_guard<std::mutex> l(g_mu);
    g_regions.erase(r->va);
  }
  for (size_t i = 0; i < r->slabs.size(); ++i) {
    Slab& s = r->slabs[i];
    if (s.mapped && r->owns_va) g_drv->unmap(r->va + i * r->slab_bytes, r->slab_bytes);
    if (s.handle) {
      g_drv->release(s.handle);
      if (r->owns_phys && s.device >= 0) {
        std::lock_guard<std::mutex> l(g_mu);
        if (g_usage[s.device] >= r->slab_bytes) g_usage[s.device] -= r->slab_bytes;
      }
    }
  }
  if (r->owns_va && r->va) g_drv->free_va(r->va, r->size);
  delete r;
}

void* fl_vmm_ptr(const FlVmmRegion* r) { return r ? (void*)r->va : nullptr; }
size_t fl_vmm_size(const FlVmmRegion* r) { return r ? r->size : 0; }
size_t fl_vmm_slab_bytes(const FlVmmRegion* r) { return r ? r->slab_bytes : 0; }
int fl_vmm_num_slabs(const FlVmmRegion* r) { return r ? (int)r->slabs.size() : 0; }
int fl_vmm_slab_device(const FlVmmRegion* r, int slab) {
  if (!r || slab < 0 || slab >= (int)r->slabs.size()) return -1;
  return r->slabs[slab].device;
}

int fl_vmm_export_fd(FlVmmRegion* r, int slab, int* fd_out) {
  if (!r || !g_drv || slab < 0 || slab >= (int)r->slabs.size()) { set_err("%s: bad slab (%ld)", "export", slab); return 1; }
  return g_drv->export_fd(r->slabs[slab].handle, fd_out);
}

int fl_vmm_grant(FlVmmRegion* r, int device) {
  if (!r || !g_drv) return 1;
  for (int d : r->access) if (d == device) return 0;
  int rc = g_drv->set_access(r->va, r->size, device);
  if (!rc) r->access.push_back(device);
  return rc;
}

int fl_vmm_remap_slab(FlVmmRegion* r, int slab, int target_device, int keep_contents, const int* access_devices,
                      int n_access, long* usec_out) {
  if (!r || !g_drv || slab < 0 || slab >= (int)r->slabs.size()) { set_err("%s: bad slab (%ld)", "remap", slab); return 1; }
  auto t0 = std::chrono::steady_clock::now();
  Slab& s = r->slabs[slab];
  const uintptr_t va = r->va + (size_t)slab * r->slab_bytes;
  uint64_t nh = 0;
  int rc = g_drv->create(target_device, r->slab_bytes, &nh);
  if (rc) return rc;
  if (keep_contents) {
    // stage through a temporary mapping of the new memory while the old one is still mapped
    uintptr_t tmp = 0;
    size_t gran = 0;
    g_drv->granularity(target_device, &gran);
    rc = g_drv->reserve(r->slab_bytes, gran, &tmp);
    if (!rc) rc = g_drv->map(tmp, r->slab_bytes, nh);
    if (!rc) rc = g_drv->set_access(tmp, r->slab_bytes, target_device);
    if (!rc && !r->access.empty() && r->access[0] != target_device) rc = g_drv->set_access(tmp, r->slab_bytes, r->access[0]);
    if (!rc) rc = g_drv->copy(tmp, va, r->slab_bytes);
    if (tmp) {
      g_drv->unmap(tmp, r->slab_bytes);
      g_drv->free_va(tmp, r->slab_bytes);
    }
    if (rc) { g_drv->release(nh); return rc; }
  }
  rc = g_drv->unmap(va, r->slab_bytes);
  if (rc) { g_drv->release(nh); return rc; }
  s.mapped = false;
  g_drv->release(s.handle);
  {
    std::lock_guard<std::mutex> l(g_mu);
    if (r->owns_phys && s.device >= 0 && g_usage[s.device] >= r->slab_bytes) g_usage[s.device] -= r->slab_bytes;
    g_usage[target_device] += r->slab_bytes;
  }
  s.handle = nh;
  s.device = target_device;
  r->owns_phys = true;
  rc = g_drv->map(va, r->slab_bytes, nh);
  if (rc) return rc;
  s.mapped = true;
  if (n_access > 0 && access_devices) {
    for (int i = 0; i < n_access; ++i) {
      rc = g_drv->set_access(va, r->slab_bytes, access_devices[i]);
      if (rc) return rc;
    }
  } else {
    for (int d : r->access) {
      rc = g_drv->set_access(va, r->slab_bytes, d);
      if (rc) return rc;
    }
  }
  if (usec_out)
    *usec_out = (long)std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
  return 0;
}

int fl_vmm_ptr2dev(const void* ptr) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_regions.upper_bound((uintptr_t)ptr);
  if (it == g_regions.begin()) return -1;
  --it;
  FlVmmRegion* r = it->second;
  const uintptr_t p = (uintptr_t)ptr;
  if (p < r->va || p >= r->va + r->size) return -1;
  return r->slabs[(p - r->va) / r->slab_bytes].device;
}

int fl_vmm_address_range(const void* ptr, void** base, size_t* size) {
  {
    std::lock_guard<std::mutex> l(g_mu);
    auto it = g_regions.upper_bound((uintptr_t)ptr);
    if (it != g_regions.begin()) {
      --it;
      FlVmmRegion* r = it->second;
      const uintptr_t p = (uintptr_t)ptr;
      if (p >= r->va && p < r->va + r->size) {
        const size_t slab = (p - r->va) / r->slab_bytes;
        *base = reinterpret_cast<void*>(r->va + slab * r->slab_bytes);
        *size = r->slab_bytes;
        return 0;
      }
    }
  }
  if (!g_drv) return 1;
  uintptr_t b = 0;
  size_t n = 0;
  if (g_drv->address_range(ptr, &b, &n)) return 1;
  *base = reinterpret_cast<void*>(b);
  *size = n;
  return 0;
}

int fl_vmm_dmabuf_fd(const void* ptr, size_t size, int* fd_out, uint64_t* offset_out) {
  if (!g_drv || !ptr || !size || !fd_out || !offset_out) return 1;
  return g_drv->dmabuf_fd(ptr, size, fd_out, offset_out);
}

int fl_vmm_memcpy(void* dst, const void* src, size_t bytes) {
  if (!g_drv) { set_err("%s: fl_vmm_init not called (%ld)", "vmm", 0); return 1; }
  return g_drv->any_copy(dst, src, bytes);
}

int fl_vmm_device_count(void) { return g_drv ? g_drv->device_count() : 0; }

int fl_vmm_pointer_device(const void* ptr) {
  const int known = fl_vmm_ptr2dev(ptr);
  if (known >= 0 || !g_drv) return known;
  return g_drv->pointer_device(ptr);
}

size_t fl_vmm_usage(int device) {
  std::lock_guard<std::mutex> l(g_mu);
  auto it = g_usage.find(device);
  return it == g_usage.end() ? 0 : it->second;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// slab pool
// ------------------------------------------------------------------------------------------------
namespace {
struct Pool {
  size_t slab_bytes = 0;
  std::vector<std::vector<uint64_t>> free_handles;   // per device
  bool ready = false;
};
Pool g_pool;

bool pool_take(int dev, uint64_t* h) {
  std::lock_guard<std::mutex> l(g_mu);
  if (!g_pool.ready || dev < 0 || dev >= (int)g_pool.free_handles.size() || g_pool.free_handles[dev].empty()) return false;
  *h = g_pool.free_handles[dev].back();
  g_pool.free_handles[dev].pop_back();
  return true;
}
void pool_give(int dev, uint64_t h) {
  std::lock_guard<std::mutex> l(g_mu);
  if (g_pool.ready && dev >= 0 && dev < (int)g_pool.free_handles.size()) g_pool.free_handles[dev].push_back(h);
}
}  // namespace

extern "C" {

int fl_pool_init(int ndev, int slabs_per_dev, size_t slab_bytes) {
  if (!g_drv) { set_err("%s: fl_vmm_init not called (%ld)", "pool", 0); return 1; }
  if (g_pool.ready) { set_err("%s: already initialised (%ld)", "pool", 0); return 1; }
  if (ndev < 1 || ndev > 64) { set_err("%s: bad device count (%ld)", "pool", ndev); return 1; }
  if (slabs_per_dev <= 0) slabs_per_dev = 256;
  if (slab_bytes == 0) slab_bytes = 2u << 20;
  size_t gran = 0;
  if (g_drv->granularity(0, &gran) || gran == 0) return 1;
  slab_bytes = round_up(slab_bytes, gran);
  g_pool.slab_bytes = slab_bytes;
  g_pool.free_handles.assign(ndev, {});
  for (int d = 0; d < ndev; ++d) {
    for (int i = 0; i < slabs_per_dev; ++i) {
      uint64_t h = 0;
      if (g_drv->create(d, slab_bytes, &h)) {
        g_pool.ready = true;
        fl_pool_shutdown();
        return 1;
      }
      g_pool.free_handles[d].push_back(h);
      std::lock_guard<std::mutex> l(g_mu);
      g_usage[d] += slab_bytes;
    }
  }
  g_pool.ready = true;
  return 0;
}

void fl_pool_shutdown(void) {
  if (!g_pool.ready || !g_drv) return;
  for (size_t d = 0; d < g_pool.free_handles.size(); ++d) {
    for (uint64_t h : g_pool.free_handles[d]) {
      g_drv->release(h);
      std::lock_guard<std::mutex> l(g_mu);
      if (g_usage[(int)d] >= g_pool.slab_bytes) g_usage[(int)d] -= g_pool.slab_bytes;
    }
  }
  g_pool.free_handles.clear();
  g_pool.ready = false;
}

int fl_pool_free_slabs(int dev) {
  std::lock_guard<std::mutex> l(g_mu);
  if (!g_pool.ready || dev < 0 || dev >= (int)g_pool.free_handles.size()) return 0;
  return (int)g_pool.free_handles[dev].size();
}

size_t fl_pool_slab_bytes(void) { return g_pool.slab_bytes; }

FlVmmRegion* fl_pool_alloc(int dev, size_t size) {
  if (!g_pool.ready || size == 0) { set_err("%s: pool not initialised or zero size (%ld)", "pool", 0); return nullptr; }
  const size_t sb = g_pool.slab_bytes;
  const size_t n = (size + sb - 1) / sb;
  if ((size_t)fl_pool_free_slabs(dev) < n) { set_err("%s: not enough free slabs on the device (%ld needed)", "pool", (long)n); return nullptr; }
  FlVmmRegion* r = new FlVmmRegion();
  r->slab_bytes = sb;
  r->size = n * sb;
  r->pooled = true;
  r->access.push_back(dev);
  if (g_drv->reserve(r->size, sb, &r->va)) { delete r; return nullptr; }
  for (size_t i = 0; i < n; ++i) {
    Slab s;
    pool_take(dev, &s.handle);
    s.device = dev;
    r->slabs.push_back(s);
  }
  if (map_all(r)) { fl_pool_release(r); return nullptr; }
  register_region(r);
  return r;
}

FlVmmRegion* fl_pool_register(void* ptr, size_t size, int owner_dev) {
  if (!g_pool.ready) { set_err("%s: pool not initialised (%ld)", "pool", 0); return nullptr; }
  const size_t sb = g_pool.slab_bytes;
  if (size == 0 || size % sb || ((uintptr_t)ptr % sb)) { set_err("%s: pointer and size must be multiples of the slab size (%ld)", "pool", (long)sb); return nullptr; }
  const size_t n = size / sb;
  if ((size_t)fl_pool_free_slabs(owner_dev) < n) { set_err("%s: not enough free slabs on the owner (%ld needed)", "pool", (long)n); return nullptr; }
  // stage the contents in pool slabs through a temporary mapping, then swap the mappings under the user's address
  FlVmmRegion* r = new FlVmmRegion();
  r->va = (uintptr_t)ptr;
  r->size = size;
  r->slab_bytes = sb;
  r->owns_va = false;
  r->pooled = true;
  r->access.push_back(owner_dev);
  uintptr_t tmp = 0;
  if (g_drv->reserve(sb, sb, &tmp)) { delete r; return nullptr; }
  int rc = 0;
  for (size_t i = 0; i < n && !rc; ++i) {
    Slab s;
    pool_take(owner_dev, &s.handle);
    s.device = owner_dev;
    rc = g_drv->map(tmp, sb, s.handle);
    if (!rc) rc = g_drv->set_access(tmp, sb, owner_dev);
    if (!rc) rc = g_drv->copy(tmp, r->va + i * sb, sb);
    g_drv->unmap(tmp, sb);
    r->slabs.push_back(s);
  }
  g_drv->free_va(tmp, sb);
  if (!rc) rc = g_drv->unmap(r->va, size);          // the caller's original backing is dropped here
  if (!rc) rc = map_all(r);
  if (rc) {
    for (auto& s : r->slabs) pool_give(s.device, s.handle);
    delete r;
    return nullptr;
  }
  register_region(r);
  return r;
}

int fl_pool_remap(FlVmmRegion* r, int slab, int target_dev, int keep_contents, const int* access_devices, int n_access,
                  long* usec_out) {
  if (!r || !r->pooled || slab < 0 || slab >= (int)r->slabs.size()) { set_err("%s: not a pool region / bad slab (%ld)", "pool", slab); return 1; }
  auto t0 = std::chrono::steady_clock::now();
  uint64_t nh = 0;
  if (!pool_take(target_dev, &nh)) { set_err("%s: no free slab on the target device (%ld)", "pool", target_dev); return 1; }
  Slab& s = r->slabs[slab];
  const size_t sb = r->slab_bytes;
  const uintptr_t va = r->va + (size_t)slab * sb;
  int rc = 0;
  if (keep_contents) {
    uintptr_t tmp = 0;
    rc = g_drv->reserve(sb, sb, &tmp);
    if (!rc) rc = g_drv->map(tmp, sb, nh);
    if (!rc) rc = g_drv->set_access(tmp, sb, target_dev);
    if (!rc && !r->access.empty() && r->access[0] != target_dev) rc = g_drv->set_access(tmp, sb, r->access[0]);
    if (!rc) rc = g_drv->copy(tmp, va, sb);
    if (tmp) { g_drv->unmap(tmp, sb); g_drv->free_va(tmp, sb); }
  }
  if (!rc) rc = g_drv->unmap(va, sb);
  if (rc) { pool_give(target_dev, nh); return rc; }
  pool_give(s.device, s.handle);                    // the slab of the OLD device goes back to the OLD device's pool
  s.handle = nh;
  s.device = target_dev;
  rc = g_drv->map(va, sb, nh);
  if (rc) return rc;
  if (n_access > 0 && access_devices) {
    for (int i = 0; i < n_access && !rc; ++i) rc = g_drv->set_access(va, sb, access_devices[i]);
  } else {
    for (int d : r->access) if (!rc) rc = g_drv->set_access(va, sb, d);
  }
  if (usec_out)
    *usec_out = (long)std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
  return rc;
}

void fl_pool_release(FlVmmRegion* r) {
  if (!r || !g_drv) return;
  {
    std::lock_guard<std::mutex> l(g_mu);
    g_regions.erase(r->va);
  }
  for (size_t i = 0; i < r->slabs.size(); ++i) {
    if (r->slabs[i].mapped) g_drv->unmap(r->va + i * r->slab_bytes, r->slab_bytes);
    if (r->slabs[i].handle) pool_give(r->slabs[i].device, r->slabs[i].handle);
  }
  if (r->owns_va && r->va) g_drv->free_va(r->va, r->size);
  delete r;
}

}  // extern "C"

// cuMem (CUDA virtual memory management) layer: regions made of physical slabs that can be exported to
// other processes, mapped by every peer GPU, aliased, and re-homed onto another GPU without changing
// their virtual address.
//
// What it answers in the reference:
//   * FuseLinkMemRegionInit (src/fuselink.cc:4-59): per-GPU physical allocations + alias VAs, then the
//     ORIGINAL VA of a buffer is re-mapped onto memory of a relay GPU        -> fl_vmm_adopt + fl_vmm_remap_slab
//   * MemRemap / CreateMem with its "Remap time" log (src/plugin.cc:1106-1165) -> fl_vmm_remap_slab(usec)
//   * the 2 MiB slab pool of src/cumem.cu (register/remap/free/ptr2dev/usage)  -> slabs of a region, fl_vmm_ptr2dev,
//     fl_vmm_usage
// and what it adds: export/import of the slabs as POSIX fds so that every rank's buffers are addressable
// from every GPU of the box (the symmetric heap the device kernels store into).
//
// The driver is reached through a function table loaded with dlopen, so this file builds and loads on a
// machine without a GPU.  A second table backed by memfd + mmap ("fake driver") gives the same aliasing
// semantics on the CPU and is what the CPU tests run against.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct FlVmmRegion FlVmmRegion;

// backend: 0 = CUDA driver, 1 = fake (memfd/mmap).  Returns 0 on success.
int fl_vmm_init(int backend);
int fl_vmm_backend(void);
const char* fl_vmm_last_error(void);

int fl_vmm_granularity(int device, size_t* out);
// `size` is rounded up to a whole number of slabs; slab_bytes == 0 means one slab; slab_bytes is rounded up
// to the allocation granularity.  The region is mapped read/write for `device`.
FlVmmRegion* fl_vmm_create(int device, size_t size, size_t slab_bytes);
// Take over an existing VMM allocation (for instance a staging buffer another library allocated with
// cuMemCreate): the handle behind `ptr` is retained and the region can then be re-homed.
FlVmmRegion* fl_vmm_adopt(void* ptr, size_t size, int owner_device);
// Map slabs exported by another process (or another region) into a fresh VA range, RW for `device`.
FlVmmRegion* fl_vmm_import(int device, const int* fds, int nslabs, size_t slab_bytes);
// A second VA range over the same physical slabs (the reference's per-GPU alias addresses).
FlVmmRegion* fl_vmm_alias(FlVmmRegion* r, int device);
void fl_vmm_destroy(FlVmmRegion* r);

void* fl_vmm_ptr(const FlVmmRegion* r);
size_t fl_vmm_size(const FlVmmRegion* r);
size_t fl_vmm_slab_bytes(const FlVmmRegion* r);
int fl_vmm_num_slabs(const FlVmmRegion* r);
int fl_vmm_slab_device(const FlVmmRegion* r, int slab);
int fl_vmm_export_fd(FlVmmRegion* r, int slab, int* fd_out);
int fl_vmm_grant(FlVmmRegion* r, int device);
// Back slab `slab` with new physical memory on `target_device`, keeping the virtual address.  With
// `keep_contents` the bytes are carried over.  `access_devices`/`n_access` list the GPUs that get RW access
// to the new mapping (the reference opens it to the source GPU only, src/fuselink.cc:52-56).
int fl_vmm_remap_slab(FlVmmRegion* r, int slab, int target_device, int keep_contents, const int* access_devices,
                      int n_access, long* usec_out);
// Which device backs the slab that contains ptr (-1 if ptr is not inside a known region).
int fl_vmm_ptr2dev(const void* ptr);
// The mapping that contains `ptr`: base address and size of the physical allocation mapped there (for a region of this
// layer, the slab).  What the reference asks cuMemGetAddressRange for before it takes a buffer over
// (src/plugin.cc:1186-1194): NCCL registers sub-ranges of larger allocations.  Returns 0 on success.
int fl_vmm_address_range(const void* ptr, void** base, size_t* size);
// A dma-buf file descriptor for the memory mapped at [ptr, ptr + size) right now (cuMemGetHandleForAddressRange), for a
// NIC registration of device memory without a peer-memory kernel module.  The exported range is widened to whole host
// pages; *offset_out is where `ptr` lies inside it.  A buffer that was re-homed needs a descriptor taken AFTER the move:
// one taken before names the old physical memory.  The caller closes the descriptor.  Returns 0 on success.
int fl_vmm_dmabuf_fd(const void* ptr, size_t size, int* fd_out, uint64_t* offset_out);
// Synchronous copy between any two addresses the backend knows (device or host, unified addressing).
int fl_vmm_memcpy(void* dst, const void* src, size_t bytes);
// Device that owns `ptr`: a region of this layer, else what the driver reports, else -1.
int fl_vmm_pointer_device(const void* ptr);
// Number of devices the backend sees (fake backend: FUSELINK_VMM_FAKE_NGPUS or 8).
int fl_vmm_device_count(void);
// Bytes of physical memory this layer currently holds on `device`.
size_t fl_vmm_usage(int device);

// ---- slab pool -------------------------------------------------------------------------------------------
// Physical slabs created up-front per device, so that re-homing a live buffer costs an unmap + map + set-access and
// no allocation.  This is the fine-grained design of the reference's src/cumem.cu (256 slabs of 2 MiB per GPU,
// register_cumem / remap_cumem / free_cumem / show_cumem_usage): a registered buffer is re-backed slab by slab from its
// owner's pool, and any single slab can then be re-backed from another GPU's pool.  Sizes are size_t throughout (the
// reference's int arithmetic overflows at 2 GiB, src/cumem.cu:146-147) and a remap always takes the slab of the device
// it was asked for (src/cumem.cu:76-83 reuses the old device's handle).
int fl_pool_init(int ndev, int slabs_per_dev, size_t slab_bytes);   // 0 slabs_per_dev => 256, 0 slab_bytes => 2 MiB
void fl_pool_shutdown(void);
int fl_pool_free_slabs(int dev);                                     // slabs still available on `dev`
size_t fl_pool_slab_bytes(void);
// A fresh region of `size` bytes backed by pool slabs of `dev`.
FlVmmRegion* fl_pool_alloc(int dev, size_t size);
// Take over an existing cuMem allocation at `ptr` (size a multiple of the slab size): its contents are carried into
// slabs of the owner's pool and the address stays valid.
FlVmmRegion* fl_pool_register(void* ptr, size_t size, int owner_dev);
// Re-back slab `slab` of a pool region from `target_dev`'s pool; the old slab goes back to its pool.
int fl_pool_remap(FlVmmRegion* r, int slab, int target_dev, int keep_contents, const int* access_devices, int n_access,
                  long* usec_out);
// Return every slab of the region to the pools and drop the region (the address range is freed if this layer reserved it).
void fl_pool_release(FlVmmRegion* r);

#ifdef __cplusplus
}
#endif

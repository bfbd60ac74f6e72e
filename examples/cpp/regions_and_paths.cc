// The host-side C API without Python: a region is created, exported as a file descriptor, mapped a second time, re-homed
// onto another device with its contents kept, and a transfer is planned over the idleness monitor.
//
//   g++ -std=c++17 -I fuselink_b200/include -I $CUDA_HOME/include examples/cpp/regions_and_paths.cc \
//       -L fuselink_b200/lib -lfuselink -Wl,-rpath,$PWD/fuselink_b200/lib -o regions_and_paths
//   ./regions_and_paths            # CUDA driver          ./regions_and_paths --fake     # memfd stand-in, no GPU needed
#include <stdio.h>
#include <string.h>
#include <unistd.h>

#include <vector>

#include "fuselink.h"

int main(int argc, char** argv) {
  const bool fake = argc > 1 && !strcmp(argv[1], "--fake");
  if (fl_vmm_init(fake ? 1 : 0)) { fprintf(stderr, "vmm: %s\n", fl_vmm_last_error()); return 1; }
  size_t gran = 0;
  fl_vmm_granularity(0, &gran);
  FlVmmRegion* r = fl_vmm_create(0, 4 * gran, gran);             // four slabs on device 0
  if (!r) { fprintf(stderr, "create: %s\n", fl_vmm_last_error()); return 1; }
  std::vector<unsigned char> pattern(fl_vmm_size(r));
  for (size_t i = 0; i < pattern.size(); ++i) pattern[i] = (unsigned char)(i * 31 + 7);
  fl_vmm_memcpy(fl_vmm_ptr(r), pattern.data(), pattern.size());

  // a second mapping of the same memory, through exported descriptors (what a peer process would do)
  std::vector<int> fds(fl_vmm_num_slabs(r));
  for (int s = 0; s < (int)fds.size(); ++s)
    if (fl_vmm_export_fd(r, s, &fds[s])) { fprintf(stderr, "export: %s\n", fl_vmm_last_error()); return 1; }
  FlVmmRegion* peer = fl_vmm_import(0, fds.data(), (int)fds.size(), fl_vmm_slab_bytes(r));
  for (int fd : fds) close(fd);
  if (!peer) { fprintf(stderr, "import: %s\n", fl_vmm_last_error()); return 1; }
  std::vector<unsigned char> back(pattern.size());
  fl_vmm_memcpy(back.data(), fl_vmm_ptr(peer), back.size());
  if (back != pattern) { fprintf(stderr, "the second mapping shows other bytes\n"); return 2; }

  // slab 2 moves to device 1 (if there is one), the address and the bytes stay
  const int ndev = fl_vmm_device_count();
  long usec = 0;
  if (ndev > 1) {
    const int access[2] = {0, 1};
    if (fl_vmm_remap_slab(r, 2, 1, 1, access, 2, &usec)) { fprintf(stderr, "remap: %s\n", fl_vmm_last_error()); return 1; }
    fl_vmm_memcpy(back.data(), fl_vmm_ptr(r), back.size());
    if (back != pattern) { fprintf(stderr, "contents changed by the remap\n"); return 2; }
  }
  printf("region of %zu bytes in %d slabs; slab 2 now on device %d (remap %ld us); usage dev0 %zu dev1 %zu\n", fl_vmm_size(r),
         fl_vmm_num_slabs(r), fl_vmm_slab_device(r, 2), usec, fl_vmm_usage(0), fl_vmm_usage(1));

  // path selection: device 0 sends 64 MiB to device 1 while 2 and 3 are idle and 4 is busy
  FlMonitor* m = fl_monitor_open("", 1, 8, 1, 160);
  const uint64_t now = fl_monitor_now_ns();
  fl_monitor_post_bytes(m, FL_DIR_TX, 4, 1 << 20, now);
  FlSelectorCfg cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.degree = 3; cfg.step = 1; cfg.min_stripe_bytes = 1 << 20; cfg.align = 256; cfg.allow_relay = 1;
  FlStripe stripes[8];
  const int n = fl_select_paths(m, &cfg, 0, 1, 64ull << 20, 0, stripes, 8, now);
  unsigned long long total = 0;
  for (int i = 0; i < n; ++i) {
    printf("  stripe %d: via path %d, offset %llu, %llu bytes\n", i, stripes[i].path, (unsigned long long)stripes[i].offset,
           (unsigned long long)stripes[i].bytes);
    total += stripes[i].bytes;
    if (stripes[i].path == 4) { fprintf(stderr, "a busy path was chosen\n"); return 2; }
  }
  if (total != (64ull << 20)) { fprintf(stderr, "stripes do not add up\n"); return 2; }
  fl_monitor_close(m, 0);
  fl_vmm_destroy(peer);
  fl_vmm_destroy(r);
  printf("OK\n");
  return 0;
}

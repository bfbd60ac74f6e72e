// fl_net_harness: drives a ncclNet plugin the way NCCL's proxy thread does, without NCCL and without GPUs.
//
//   fl_net_harness <plugin.so> recv <handle-file> [options] <size> [<size> ...]
//   fl_net_harness <plugin.so> send <handle-file> [options] <size> [<size> ...]
//
// The receiver listens, writes the 128-byte handle to <handle-file>, accepts, and receives every message
// in chunks (--chunk, default 512 KiB) with at most --inflight (default 8) requests outstanding; the
// sender mirrors it.  Payloads are fp32 uniform[-1,1] generated from --seed on both sides, so the receiver
// can compare bit for bit without a side channel.  Exit code 0 = all messages identical.
//
// Options: --chunk N  --inflight N  --seed N  --dev N  --abi 6|7|8  --channels N (connections side by side)  --threads
// (one thread per channel, each moving every message on its own connection, the way NCCL runs one proxy thread per
// device)  --die-after-chunks N (sender exits
// abruptly after N chunks: peer-failure test)  --expect-error (receiver: a transfer error is the
// expected outcome; exit 0 if it is reported within the timeout, 3 if the transfer hangs or succeeds).
#include <dlfcn.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <deque>
#include <string>
#include <thread>
#include <vector>

#include "nccl_net_abi.h"

static inline uint64_t next_u64(uint64_t& rng_state) {  // xorshift64*
  rng_state ^= rng_state >> 12;
  rng_state ^= rng_state << 25;
  rng_state ^= rng_state >> 27;
  return rng_state * 2685821657736338717ull;
}
static void fill(std::vector<float>& v, uint64_t seed, size_t msg_index) {
  uint64_t rng_state = seed * 0x9E3779B97F4A7C15ull + msg_index * 0xD1B54A32D192ED03ull + 1;
  for (auto& x : v) x = (float)((double)(next_u64(rng_state) >> 11) / (double)(1ull << 53) * 2.0 - 1.0);
}
static double now_s() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec + ts.tv_nsec * 1e-9;
}
static void logger(ncclDebugLogLevel lvl, unsigned long, const char*, int, const char* fmt, ...) {
  if (lvl != NCCL_LOG_WARN && !getenv("FL_HARNESS_VERBOSE")) return;
  va_list ap;
  va_start(ap, fmt);
  vfprintf(stderr, fmt, ap);
  va_end(ap);
  fputc('\n', stderr);
}

// one calling convention over the three ABI versions
struct Api {
  int abi = 7;
  ncclNet_v6_t* v6 = nullptr;
  ncclNet_v7_t* v7 = nullptr;
  ncclNet_v8_t* v8 = nullptr;
#define PICK(f) (abi == 6 ? v6->f : abi == 7 ? v7->f : v8->f)
  ncclResult_t init() { return PICK(init)(logger); }
  ncclResult_t devices(int* n) { return PICK(devices)(n); }
  ncclResult_t listen(int dev, void* h, void** lc) { return PICK(listen)(dev, h, lc); }
  ncclResult_t connect(int dev, void* h, void** sc) {
    if (abi == 6) return v6->connect(dev, h, sc);
    ncclNetDeviceHandle_v7_t* dh = nullptr;
    return abi == 7 ? v7->connect(dev, h, sc, &dh) : v8->connect(dev, h, sc, &dh);
  }
  ncclResult_t accept(void* lc, void** rc) {
    if (abi == 6) return v6->accept(lc, rc);
    ncclNetDeviceHandle_v7_t* dh = nullptr;
    return abi == 7 ? v7->accept(lc, rc, &dh) : v8->accept(lc, rc, &dh);
  }
  int ptr_type = NCCL_PTR_HOST;
  ncclResult_t regMr(void* c, void* d, size_t s, void** mh) {
    if (abi == 8) return v8->regMr(c, d, s, ptr_type, mh);
    return abi == 6 ? v6->regMr(c, d, (int)s, ptr_type, mh) : v7->regMr(c, d, (int)s, ptr_type, mh);
  }
  ncclResult_t regMrDmaBuf(void* c, void* d, size_t s, uint64_t off, int fd, void** mh) { return PICK(regMrDmaBuf)(c, d, s, ptr_type, off, fd, mh); }
  ncclResult_t deregMr(void* c, void* mh) { return PICK(deregMr)(c, mh); }
  ncclResult_t isend(void* c, void* d, int s, int tag, void* mh, void** r) { return PICK(isend)(c, d, s, tag, mh, r); }
  ncclResult_t irecv(void* c, void* d, int s, int tag, void* mh, void** r) { return PICK(irecv)(c, 1, &d, &s, &tag, &mh, r); }
  ncclResult_t test(void* r, int* done, int* sz) { return PICK(test)(r, done, sz); }
  ncclResult_t iflush(void* c, void* d, int s, void* mh, void** r) { return PICK(iflush)(c, 1, &d, &s, &mh, r); }
  ncclResult_t closeSend(void* c) { return PICK(closeSend)(c); }
  ncclResult_t closeRecv(void* c) { return PICK(closeRecv)(c); }
  ncclResult_t closeListen(void* c) { return PICK(closeListen)(c); }
#undef PICK
};

int main(int argc, char** argv) {
  if (argc < 5) {
    fprintf(stderr, "usage: %s <plugin.so> send|recv <handle-file> [options] <size>...\n", argv[0]);
    return 2;
  }
  const char* so = argv[1];
  const bool is_send = !strcmp(argv[2], "send");
  const std::string hfile = argv[3];
  size_t chunk = 512 * 1024;
  int inflight = 8, dev = 0, die_after = -1, channel = 0, nch = 1;
  uint64_t seed = 0;
  bool expect_error = false, device_bufs = false, threaded = false, do_flush = false, nccl_dmabuf = false;
  const char* inject_event = nullptr;
  size_t reg_offset = 0;
  Api api;
  std::vector<size_t> sizes;
  for (int i = 4; i < argc; ++i) {
    std::string a = argv[i];
    auto val = [&]() { return strtoull(argv[++i], nullptr, 0); };
    if (a == "--chunk") chunk = val();
    else if (a == "--inflight") inflight = (int)val();
    else if (a == "--seed") seed = val();
    else if (a == "--dev") dev = (int)val();
    else if (a == "--abi") api.abi = (int)val();
    else if (a == "--channels") nch = (int)val();          // connections used side by side; chunk c travels on channel c % N
    else if (a == "--channel") channel = (int)val();      // receiver: burn this many channel ids first
    else if (a == "--die-after-chunks") die_after = (int)val();
    else if (a == "--expect-error") expect_error = true;
    else if (a == "--threads") threaded = true;
    else if (a == "--reg-offset") reg_offset = (size_t)val();  // device buffers: the registered buffer starts this far into its allocation
    else if (a == "--flush") do_flush = true;               // receiver: iflush the whole buffer after every message
    else if (a == "--inject-event") inject_event = argv[++i];   // raise an asynchronous device event after init (software NIC)
    else if (a == "--nccl-dmabuf") { device_bufs = true; nccl_dmabuf = true; }   // register through regMrDmaBuf with a descriptor taken beforehand, as NCCL does
    else if (a == "--device-buffers") device_bufs = true;   // buffers come from the plugin's cuMem layer and are registered as CUDA
    else sizes.push_back(strtoull(a.c_str(), nullptr, 0));
  }
  void* lib = dlopen(so, RTLD_NOW);
  if (!lib) { fprintf(stderr, "dlopen: %s\n", dlerror()); return 2; }
  api.v6 = (ncclNet_v6_t*)dlsym(lib, "ncclNetPlugin_v6");
  api.v7 = (ncclNet_v7_t*)dlsym(lib, "ncclNetPlugin_v7");
  api.v8 = (ncclNet_v8_t*)dlsym(lib, "ncclNetPlugin_v8");
  if (!api.v6 || !api.v7 || !api.v8) { fprintf(stderr, "plugin symbols missing\n"); return 2; }
  if (strcmp(api.v7->name, "FuseLink")) { fprintf(stderr, "unexpected plugin name %s\n", api.v7->name); return 2; }
  if (api.init() != ncclSuccess) { fprintf(stderr, "init failed\n"); return 2; }
  if (inject_event) {
    auto inject = (void (*)(int, const char*))dlsym(lib, "fuselink_soft_inject_event");
    if (inject) inject(0, inject_event);
    usleep(200 * 1000);                                       // the device's watcher thread logs it
  }
  int ndev = 0;
  api.devices(&ndev);
  if (dev >= ndev) { fprintf(stderr, "device %d of %d\n", dev, ndev); return 2; }

  if (nch < 1 || nch > 16) { fprintf(stderr, "--channels must be in [1, 16]\n"); return 2; }
  char handle[NCCL_NET_HANDLE_MAXSIZE];
  std::vector<void*> lcomms(nch, nullptr), comms(nch, nullptr);
  const double t_limit = now_s() + 120.0;
  if (!is_send) {
    for (int i = 0; i < channel; ++i) {   // every listen takes the next global channel id
      void* tmp = nullptr;
      if (api.listen(dev, handle, &tmp) == ncclSuccess) api.closeListen(tmp);
    }
    std::string tmp = hfile + ".tmp";
    FILE* f = fopen(tmp.c_str(), "wb");
    for (int c = 0; c < nch; ++c) {
      if (api.listen((dev + c) % ndev, handle, &lcomms[c]) != ncclSuccess) { fprintf(stderr, "listen failed\n"); return 2; }
      fwrite(handle, 1, sizeof handle, f);
    }
    fclose(f);
    rename(tmp.c_str(), hfile.c_str());
    for (int c = 0; c < nch; ++c) {
      while (!comms[c]) {
        if (api.accept(lcomms[c], &comms[c]) != ncclSuccess) { fprintf(stderr, "accept failed\n"); return 2; }
        if (now_s() > t_limit) { fprintf(stderr, "accept timed out\n"); return 3; }
        if (!comms[c]) usleep(200);
      }
    }
  } else {
    FILE* f = nullptr;
    while (!(f = fopen(hfile.c_str(), "rb"))) {
      if (now_s() > t_limit) { fprintf(stderr, "no handle file\n"); return 3; }
      usleep(1000);
    }
    std::vector<char> handles((size_t)nch * sizeof handle);
    if (fread(handles.data(), 1, handles.size(), f) != handles.size()) { fprintf(stderr, "short handle file\n"); return 2; }
    fclose(f);
    for (int c = 0; c < nch; ++c) {
      memcpy(handle, handles.data() + (size_t)c * sizeof handle, sizeof handle);
      while (!comms[c]) {
        if (api.connect((dev + c) % ndev, handle, &comms[c]) != ncclSuccess) { fprintf(stderr, "connect failed\n"); return 2; }
        if (now_s() > t_limit) { fprintf(stderr, "connect timed out\n"); return 3; }
        if (!comms[c]) usleep(200);
      }
    }
  }
  void* comm = comms[0];

  if (device_bufs) api.ptr_type = NCCL_PTR_CUDA;
  std::atomic<size_t> total_bytes{0};
  std::atomic<int> chunks_done_total{0}, flushes{0};
  const double t0 = now_s();
  std::atomic<long long> xfer_ns{0};           // time inside the post/test loops only (no payload generation, no compare), max over threads
  // moves every message over the connections [ch0, ch0 + nch): chunk c of a message travels on connection ch0 + c % nch
  auto transfer = [&](const int ch0, const int nch, uint64_t seed) -> int {
  int rc = 0;
  double my_xfer = 0;
  for (size_t mi = 0; mi < sizes.size() && rc == 0; ++mi) {
    const size_t bytes = sizes[mi];
    std::vector<float> host((bytes + 3) / 4), expect;
    float* bufp = host.data();
    void* region = nullptr;
    if (device_bufs) {
      // a "GPU" buffer from the plugin's cuMem layer (memfd-backed when FUSELINK_VMM_FAKE=1), owned by device `dev`
      auto create = (void* (*)(int, size_t, size_t))dlsym(lib, "fl_vmm_create");
      auto vptr = (void* (*)(const void*))dlsym(lib, "fl_vmm_ptr");
      region = create ? create(dev, host.size() * 4 + 16 + reg_offset, 0) : nullptr;
      if (!region) { fprintf(stderr, "fl_vmm_create failed\n"); return 2; }
      bufp = (float*)((char*)vptr(region) + reg_offset);
    }
    struct BufView { float* p; size_t n; float* data() { return p; } size_t size() { return n; } } buf{bufp, host.size()};
    if (is_send) { fill(host, seed, mi); if (!host.empty()) memcpy(bufp, host.data(), host.size() * 4); }
    else { expect.resize(host.size()); fill(expect, seed, mi); if (!host.empty()) memset(bufp, 0xA5, host.size() * 4); }
    std::vector<void*> mhs(nch, nullptr);
    for (int c = 0; c < nch; ++c) {
      if (nccl_dmabuf) {
        auto get_fd = (int (*)(const void*, size_t, int*, uint64_t*))dlsym(lib, "fl_vmm_dmabuf_fd");
        int fd = -1;
        uint64_t off = 0;
        if (!get_fd || get_fd(buf.data(), buf.size() > 0 ? buf.size() * 4 : 1, &fd, &off)) { fprintf(stderr, "no dma-buf for the buffer\n"); return 2; }
        const ncclResult_t e = api.regMrDmaBuf(comms[ch0 + c], buf.data(), buf.size() * 4, off, fd, &mhs[c]);
        close(fd);
        if (e != ncclSuccess) { fprintf(stderr, "regMrDmaBuf failed\n"); return 2; }
      } else if (api.regMr(comms[ch0 + c], buf.data(), buf.size() * 4, &mhs[c]) != ncclSuccess) {
        fprintf(stderr, "regMr failed\n");
        return 2;
      }
    }
    if (device_bufs && mi == 0) {
      auto p2d = (int (*)(const void*))dlsym(lib, "fl_vmm_ptr2dev");
      printf("REGISTERED device-buffer owner %d now-backed-by %d\n", dev, p2d ? p2d(bufp) : -1);
    }
    const size_t nchunks = bytes == 0 ? 1 : (bytes + chunk - 1) / chunk;
    size_t next = 0, done_chunks = 0;
    std::vector<std::deque<void*>> reqs(nch);
    const double msg_limit = now_s() + 90.0;
    const double x0 = now_s();
    while (done_chunks < nchunks && rc == 0) {
      // post: chunk `next` belongs to channel next % nch; stop at the first channel that is full or would block
      while (next < nchunks) {
        const int c = (int)(next % nch);
        if ((int)reqs[c].size() >= inflight) break;
        const size_t off = next * chunk;
        const int len = (int)(bytes - off < chunk ? bytes - off : chunk);
        void* r = nullptr;
        ncclResult_t e = is_send ? api.isend(comms[ch0 + c], (char*)buf.data() + off, len, (int)(mi * 1000003 + next), mhs[c], &r)
                                 : api.irecv(comms[ch0 + c], (char*)buf.data() + off, len, (int)(mi * 1000003 + next), mhs[c], &r);
        if (e != ncclSuccess) { fprintf(stderr, "%s failed with %d\n", is_send ? "isend" : "irecv", (int)e); rc = 4; break; }
        if (!r) break;   // would block
        reqs[c].push_back(r);
        ++next;
      }
      if (rc) break;
      for (int c = 0; c < nch && rc == 0; ++c) {
        if (reqs[c].empty()) continue;
        int done = 0, sz = 0;
        ncclResult_t e = api.test(reqs[c].front(), &done, &sz);
        if (e != ncclSuccess) { fprintf(stderr, "test failed with %d\n", (int)e); rc = 4; break; }
        if (done) {
          reqs[c].pop_front();
          ++done_chunks;
          ++chunks_done_total;
          if (is_send && die_after >= 0 && chunks_done_total >= die_after) _exit(9);   // abrupt death: no close, no flush
        }
      }
      if (now_s() > msg_limit) { fprintf(stderr, "message %zu timed out\n", mi); rc = 3; }
    }
    my_xfer += now_s() - x0;
    if (rc == 0 && !is_send && do_flush && bytes > 0) {
      void* fr = nullptr;
      const int flen = (int)(bytes < chunk ? bytes : chunk);
      if (api.iflush(comms[ch0], buf.data(), flen, mhs[0], &fr) != ncclSuccess) { fprintf(stderr, "iflush failed\n"); rc = 4; }
      int fdone = fr ? 0 : 1, fsz = 0;
      const double flimit = now_s() + 30.0;
      while (rc == 0 && !fdone) {
        if (api.test(fr, &fdone, &fsz) != ncclSuccess) { fprintf(stderr, "flush test failed\n"); rc = 4; }
        if (now_s() > flimit) { fprintf(stderr, "flush timed out\n"); rc = 3; }
      }
      if (rc == 0) flushes += fr ? 1 : 0;
    }
    if (rc == 0 && !is_send && bytes > 0 && memcmp(buf.data(), expect.data(), bytes) != 0) {
      size_t bad = 0;
      while (bad < bytes && ((char*)buf.data())[bad] == ((char*)expect.data())[bad]) ++bad;
      fprintf(stderr, "message %zu (%zu bytes) differs at byte %zu\n", mi, bytes, bad);
      rc = 5;
    }
    for (int c = 0; c < nch; ++c) api.deregMr(comms[ch0 + c], mhs[c]);
    if (region) {
      auto destroy = (void (*)(void*))dlsym(lib, "fl_vmm_destroy");
      if (destroy) destroy(region);
    }
    total_bytes += bytes;
  }
  long long mine = (long long)(my_xfer * 1e9), cur = xfer_ns.load();
  while (mine > cur && !xfer_ns.compare_exchange_weak(cur, mine)) {}
  return rc;
  };
  int rc = 0;
  if (!threaded) {
    rc = transfer(0, nch, seed);
  } else {
    std::vector<int> rcs(nch, 0);
    std::vector<std::thread> th;
    for (int c = 0; c < nch; ++c) th.emplace_back([&, c] { rcs[c] = transfer(c, 1, seed + 1000003ull * c); });
    for (auto& t : th) t.join();
    for (int c = 0; c < nch; ++c)
      if (rcs[c] && !rc) rc = rcs[c];
  }
  const double dt = now_s() - t0;
  if (expect_error) {
    if (rc == 4) { printf("EXPECTED-ERROR after %.3f s\n", dt); rc = 0; }
    else if (rc == 0) { fprintf(stderr, "transfer succeeded but an error was expected\n"); rc = 3; }
  } else if (rc == 0) {
    const double xs = xfer_ns.load() / 1e9;
    printf("OK %s %zu bytes in %.4f s (%.3f GB/s) abi v%d; transfer loops alone %.4f s (%.3f GB/s)\n", is_send ? "sent" : "received", total_bytes.load(),
           dt, total_bytes.load() / dt / 1e9, api.abi, xs, xs > 0 ? total_bytes.load() / xs / 1e9 : 0.0);
  }
  auto decisions = (unsigned long long (*)(void))dlsym(lib, "fuselink_plugin_decisions");
  auto fallbacks = (unsigned long long (*)(void))dlsym(lib, "fuselink_plugin_fallbacks");
  auto direct_b = (unsigned long long (*)(void))dlsym(lib, "fuselink_plugin_direct_bytes");
  auto direct_m = (unsigned long long (*)(void))dlsym(lib, "fuselink_plugin_direct_msgs");
  auto rdma_ctr = (void (*)(unsigned long long*, unsigned long long*, unsigned long long*))dlsym(lib, "fuselink_rdma_counters");
  if (rdma_ctr && is_send) {
    unsigned long long m = 0, pc = 0, w = 0;
    rdma_ctr(&m, &pc, &w);
    if (m) printf("RDMA messages %llu pieces %llu work-requests %llu\n", m, pc, w);
  }
  auto mr_ctr = (void (*)(unsigned long long*, unsigned long long*, unsigned long long*))dlsym(lib, "fuselink_rdma_mr_counters");
  if (mr_ctr) {
    unsigned long long regs = 0, hits = 0, dmabuf = 0;
    mr_ctr(&regs, &hits, &dmabuf);
    if (regs) printf("MR registrations %llu cache-hits %llu dma-buf %llu\n", regs, hits, dmabuf);
  }
  auto failovers = (unsigned long long (*)(void))dlsym(lib, "fuselink_plugin_failovers");
  if (failovers && is_send && failovers()) printf("FAILOVERS %llu\n", failovers());
  auto rfail = (unsigned long long (*)(void))dlsym(lib, "fuselink_rdma_failovers");
  if (rfail && rfail()) printf("RDMA-FAILOVERS %llu\n", rfail());
  auto peer_regions = (int (*)(void*))dlsym(lib, "fuselink_comm_peer_regions");
  if (peer_regions && is_send && device_bufs) printf("PEER-REGIONS-MAPPED %d\n", peer_regions(comms[0]));
  if (direct_b && is_send) printf("DIRECT bytes %llu msgs %llu of %zu bytes\n", direct_b(), direct_m ? direct_m() : 0ull, total_bytes.load());
  if (do_flush && !is_send) printf("FLUSHES %d\n", flushes.load());
  if (decisions && !is_send) printf("SELECTOR decisions %llu fallbacks %llu channels %d\n", decisions(), fallbacks ? fallbacks() : 0ull, nch);
  for (int c = 0; c < nch; ++c) {
    if (is_send) api.closeSend(comms[c]);
    else { api.closeRecv(comms[c]); api.closeListen(lcomms[c]); }
  }
  (void)comm;
  return rc;
}

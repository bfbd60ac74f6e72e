#include "nvl_channel.h"

#include <errno.h>
#include <stddef.h>
#include <stdio.h>
#include <string.h>
#include <unistd.h>

#include "logging.h"
#include "../mem/vmm.h"

namespace flnet {

void nvl_sockaddr(uint64_t token, sockaddr_un* sa, socklen_t* len) {
  memset(sa, 0, sizeof *sa);
  sa->sun_family = AF_UNIX;
  const int n = snprintf(sa->sun_path + 1, sizeof sa->sun_path - 1, "fuselink-nvl-%016llx", (unsigned long long)token);
  *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

int nvl_send_fds(int sock, const NvlExportMsg& msg, const int* fds, int nfds) {
  char cbuf[CMSG_SPACE(sizeof(int) * 16)];
  if (nfds > 16) return -1;
  memset(cbuf, 0, sizeof cbuf);
  iovec iov{const_cast<NvlExportMsg*>(&msg), sizeof msg};
  msghdr mh;
  memset(&mh, 0, sizeof mh);
  mh.msg_iov = &iov;
  mh.msg_iovlen = 1;
  if (nfds > 0) {
    mh.msg_control = cbuf;
    mh.msg_controllen = CMSG_SPACE(sizeof(int) * nfds);
    cmsghdr* cm = CMSG_FIRSTHDR(&mh);
    cm->cmsg_level = SOL_SOCKET;
    cm->cmsg_type = SCM_RIGHTS;
    cm->cmsg_len = CMSG_LEN(sizeof(int) * nfds);
    memcpy(CMSG_DATA(cm), fds, sizeof(int) * nfds);
  }
  ssize_t r;
  do { r = sendmsg(sock, &mh, MSG_NOSIGNAL); } while (r < 0 && errno == EINTR);
  return r == (ssize_t)sizeof msg ? 0 : -1;
}

// returns 1 when a message was read, 0 when nothing is waiting, -1 on error / closed
int nvl_recv_fds(int sock, NvlExportMsg* msg, int* fds, int* nfds) {
  char cbuf[CMSG_SPACE(sizeof(int) * 16)];
  iovec iov{msg, sizeof *msg};
  msghdr mh;
  memset(&mh, 0, sizeof mh);
  mh.msg_iov = &iov;
  mh.msg_iovlen = 1;
  mh.msg_control = cbuf;
  mh.msg_controllen = sizeof cbuf;
  ssize_t r = recvmsg(sock, &mh, MSG_DONTWAIT | MSG_CMSG_CLOEXEC);
  if (r < 0) return (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) ? 0 : -1;
  if (r == 0) return -1;
  *nfds = 0;
  for (cmsghdr* cm = CMSG_FIRSTHDR(&mh); cm; cm = CMSG_NXTHDR(&mh, cm)) {
    if (cm->cmsg_level == SOL_SOCKET && cm->cmsg_type == SCM_RIGHTS) {
      const int n = (int)((cm->cmsg_len - CMSG_LEN(0)) / sizeof(int));
      memcpy(fds, CMSG_DATA(cm), sizeof(int) * n);
      *nfds = n;
    }
  }
  if (r != (ssize_t)sizeof *msg || msg->magic != kNvlMagic || *nfds != msg->nslabs) {
    for (int i = 0; i < *nfds; ++i) close(fds[i]);
    return -1;
  }
  return 1;
}

// sender: map every region the peer has announced so far
void nvl_ingest(Comm* c, int device) {
  while (c->nvl_fd >= 0) {
    NvlExportMsg msg;
    int fds[16], nfds = 0;
    const int rc = nvl_recv_fds(c->nvl_fd, &msg, fds, &nfds);
    if (rc == 0) return;
    if (rc < 0) {
      close(c->nvl_fd);
      c->nvl_fd = -1;                              // direct path off for this connection; TCP carries on
      return;
    }
    if (msg.nslabs == 0) {                         // the peer deregistered the region: unmap it
      for (auto it = c->peer_mrs.begin(); it != c->peer_mrs.end(); ++it) {
        if (it->id == msg.mr_id) {
          if (it->region) fl_vmm_destroy(reinterpret_cast<FlVmmRegion*>(it->region));
          c->peer_mrs.erase(it);
          break;
        }
      }
      continue;
    }
    FlVmmRegion* r = fl_vmm_import(device < 0 ? 0 : device, fds, nfds, (size_t)msg.slab_bytes);
    for (int i = 0; i < nfds; ++i) close(fds[i]);
    if (!r) {
      FL_WARN("direct path: cannot map the peer's region %u (%s); that region stays on the staged path", msg.mr_id, fl_vmm_last_error());
      c->peer_mrs.push_back({msg.mr_id, nullptr, 0, nullptr});
      continue;
    }
    c->peer_mrs.push_back({msg.mr_id, fl_vmm_ptr(r), msg.size, r});
    FL_INFO("direct path: peer region %u (%llu bytes) mapped at %p", msg.mr_id, (unsigned long long)msg.size, fl_vmm_ptr(r));
  }
}

}  // namespace flnet

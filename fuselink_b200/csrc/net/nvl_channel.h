// Same-host side channel of the TCP transport (the "direct path").
//
// A receive buffer that lives in a cuMem allocation can be written by a sender on the same machine without
// touching host memory: the receiver hands the allocation's file descriptors over a Unix socket
// (SCM_RIGHTS), the sender maps them, stores the payload through that mapping and sends a frame header with
// no payload.  The reference gets the same effect inside one process by copying from the relay GPU's alias
// address (src/fuselink.cc:25-41); across processes the descriptor has to travel, which is what this does.
// The socket lives in the abstract namespace under a random token published in the listen handle, so a
// sender on another host (or in another network namespace) simply fails to connect and stays on TCP.
#pragma once
#include <stdint.h>
#include <sys/socket.h>
#include <sys/un.h>

#include "tcp_transport.h"

namespace flnet {

// abstract-namespace address of a listener's side channel
void nvl_sockaddr(uint64_t token, sockaddr_un* sa, socklen_t* len);
// One message with up to 16 descriptors attached (nfds == 0: a plain notice).  Returns 0 on success.
int nvl_send_fds(int sock, const NvlExportMsg& msg, const int* fds, int nfds);
// Returns 1 when a message was read (its descriptors in fds[0..*nfds)), 0 when nothing is waiting, -1 on error / closed.
int nvl_recv_fds(int sock, NvlExportMsg* msg, int* fds, int* nfds);
// Sender: take in everything the peer has announced so far -- map newly exported regions for `device`, unmap the ones it
// has deregistered (nslabs == 0).  On a broken channel the direct path is switched off for the connection.
void nvl_ingest(Comm* c, int device);

}  // namespace flnet

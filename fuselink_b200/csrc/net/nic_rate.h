// Line rate of emulated NICs (FUSELINK_TCP_NIC_MBPS, per NIC index): one token bucket per NIC, shared by every connection of the
// process -- or, with FUSELINK_TCP_NIC_SHM=/name, by every process that names the segment -- so that experiments on one machine see
// what several NICs of limited speed give: a single path is held to the rate of its NIC, stripes over idle NICs add up.  Used by
// the TCP transport's virtual NICs and by the software RDMA NIC.
#pragma once
#include <stddef.h>

namespace flnet {
// How many of `want` bytes device `dev` may put on the wire now (0: at line rate, come back later; `want` when no rate is set).
size_t nic_allowance(int dev, size_t want);
}  // namespace flnet

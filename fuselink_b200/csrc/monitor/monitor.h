// Link/NIC idleness monitor and path selector.
//
// Reference behaviour (src/monitor.h:18-55, src/monitor.cpp:159-193, src/fuselink.h:190-267): a daemon owns
// a POSIX shared segment with, per NIC group, a tx and an rx status in {IDLE, BUSY, BORROWED} plus a
// last-active timestamp; every 160 us it takes a named semaphore and flips entries whose timestamp is
// older than 160 us back to IDLE.  Clients take the same semaphore to borrow an idle NIC of another group
// or to stamp activity.  The connection manager asks the client which NIC a channel should use.
//
// This rebuild keeps the states, the lease-by-timestamp rule and the borrow/stamp API, and changes the
// mechanics: the table is a fixed array of cache-line-sized slots updated only with atomics (no
// semaphore, no lock held across processes), the sweeper is a thread that can live in any process, the
// activity signal can be a byte counter that GPU kernels bump (posted vs completed bytes), and a selector
// turns the table into a striping decision (direct path + idle relay paths).
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FL_MON_MAX_PATHS 64          // >= MAX_NIC_NUM (16) of the reference; one path per GPU link / NIC
#define FL_MON_DEFAULT_TIMEOUT_US 160

enum FlPathStatus { FL_PATH_IDLE = 0, FL_PATH_BUSY = 1, FL_PATH_BORROWED = 2, FL_PATH_DEAD = 3 };
enum FlPathDir { FL_DIR_TX = 0, FL_DIR_RX = 1 };

typedef struct FlMonitor FlMonitor;

// Create (owner=1: create + zero the segment) or open (owner=0) the table.  shm_name == NULL or "" keeps the
// table in private memory (single process).  n_groups x paths_per_group <= FL_MON_MAX_PATHS.
FlMonitor* fl_monitor_open(const char* shm_name, int owner, int n_groups, int paths_per_group, int timeout_us);
void fl_monitor_close(FlMonitor* m, int unlink_shm);
const char* fl_monitor_last_error(void);

int fl_monitor_num_paths(const FlMonitor* m);
int fl_monitor_timeout_us(const FlMonitor* m);

// sweeper thread: IDLE-ifies stale entries, expires leases, refreshes bandwidth estimates
int fl_monitor_start(FlMonitor* m, int period_us);
void fl_monitor_stop(FlMonitor* m);
// one sweep at an explicit time (ns); what the thread calls, exposed so tests can drive time themselves
void fl_monitor_sweep(FlMonitor* m, uint64_t now_ns);
uint64_t fl_monitor_now_ns(void);

// activity
void fl_monitor_mark_active(FlMonitor* m, int dir, int path, uint64_t now_ns);         // -> BUSY, stamp
void fl_monitor_post_bytes(FlMonitor* m, int dir, int path, uint64_t bytes, uint64_t now_ns);
void fl_monitor_complete_bytes(FlMonitor* m, int dir, int path, uint64_t bytes, uint64_t now_ns);
// Counters that somebody else increments (for instance a GPU kernel writing mapped pinned memory): the
// sweeper folds counters[path] into the completed-bytes view of direction `dir`.
void fl_monitor_attach_counters(FlMonitor* m, int dir, const volatile uint64_t* counters);
// borrow an IDLE path that belongs to another group than `group`; `mask` bit p set = path p allowed.
// Returns the path index or -1.  The first idle candidate after `primary` (round-robin) wins.
int fl_monitor_borrow_idle(FlMonitor* m, int dir, int group, int primary, uint64_t mask, uint64_t now_ns);
void fl_monitor_release(FlMonitor* m, int dir, int path);
// Take a path for oneself without competing for it: succeeds (1) when the path is idle (it becomes BORROWED by `owner`) or
// already held by `owner`, fails (0) when somebody else is active on it.  The claim lapses like any lease.  `owner` is any
// id that is unique among the users of the table (a process id).
int fl_monitor_claim(FlMonitor* m, int dir, int path, int owner, uint64_t now_ns);
void fl_monitor_mark_dead(FlMonitor* m, int dir, int path, int dead);

// observation
int fl_monitor_status(const FlMonitor* m, int dir, int path);
uint64_t fl_monitor_outstanding(const FlMonitor* m, int dir, int path);
double fl_monitor_bandwidth_gbs(const FlMonitor* m, int dir, int path);
// bit p set = path p is IDLE in direction dir (the 32-bit availability mask the reference piggy-backs in
// the immediate data, src/plugin.cc:1441-1451, widened to 64 paths)
uint64_t fl_monitor_idle_mask(const FlMonitor* m, int dir);
uint64_t fl_monitor_decisions(const FlMonitor* m);

// ---- selector -----------------------------------------------------------------------------------------
typedef struct {
  int path;                 // relay path (GPU / NIC index); == dst for the direct stripe
  unsigned long long offset;
  unsigned long long bytes;
} FlStripe;

typedef struct {
  int degree;               // max number of paths used for one transfer (NCCL_FUSELINK_DEGREE)
  int step;                 // rotation step between consecutive transfers (NCCL_FUSELINK_STEP)
  unsigned long long min_stripe_bytes;   // a relay stripe is never smaller than this
  unsigned long long align;              // stripe boundaries are multiples of this (chunk size)
  int allow_relay;          // 0: always answer "direct"
} FlSelectorCfg;

// Split [0, bytes) of a src->dst transfer into stripes.  Stripe 0 is always the direct path.  Relay paths are
// borrowed from the monitor (tx direction) among paths other than src and dst; the caller releases them
// (or lets the lease expire) when the transfer is done.  Returns the number of stripes (>= 1).
int fl_select_paths(FlMonitor* m, const FlSelectorCfg* cfg, int src, int dst, unsigned long long bytes,
                    unsigned long long transfer_index, FlStripe* out, int max_out, uint64_t now_ns);

#ifdef __cplusplus
}
#endif

// Common types, enums and constants shared by the host runtime and the device API.
//
// Mirrors the public contract of the reference's include/rocshmem/rocshmem_common.hpp:36-126
// (status codes, reduction ops, signal ops, compare ops, thread levels, context option bits,
// ctx/team handle types), re-designed for a CUDA VMM symmetric heap:
//   * a team handle is the device address of the team's descriptor inside the reserved
//     ("internal") region of the symmetric heap, so device code can dereference it directly;
//   * every bounded wait reports a time-out through ROCSHMEM_ERROR / the error record instead of
//     spinning for ever.
#pragma once

#include <stddef.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define ROCSHMEM_HD __host__ __device__
#define ROCSHMEM_D __device__
#define ROCSHMEM_H __host__
#else
#define ROCSHMEM_HD
#define ROCSHMEM_D
#define ROCSHMEM_H
#endif

namespace rocshmem {

enum ROCSHMEM_STATUS {
  ROCSHMEM_SUCCESS = 0,
  ROCSHMEM_ERROR = 1,
};

enum ROCSHMEM_OP {
  ROCSHMEM_SUM,
  ROCSHMEM_MAX,
  ROCSHMEM_MIN,
  ROCSHMEM_PROD,
  ROCSHMEM_AND,
  ROCSHMEM_OR,
  ROCSHMEM_XOR,
  ROCSHMEM_REPLACE
};

enum ROCSHMEM_SIGNAL_OPS {
  ROCSHMEM_SIGNAL_SET,
  ROCSHMEM_SIGNAL_ADD,
};

enum rocshmem_cmps {
  ROCSHMEM_CMP_EQ,
  ROCSHMEM_CMP_NE,
  ROCSHMEM_CMP_GT,
  ROCSHMEM_CMP_GE,
  ROCSHMEM_CMP_LT,
  ROCSHMEM_CMP_LE,
};

enum rocshmem_thread_ops {
  ROCSHMEM_THREAD_SINGLE,
  ROCSHMEM_THREAD_FUNNELED,
  ROCSHMEM_THREAD_WG_FUNNELED,
  ROCSHMEM_THREAD_SERIALIZED,
  ROCSHMEM_THREAD_MULTIPLE
};

enum rocshmem_team_configs {
  ROCSHMEM_TEAM_DEFAULT_CONFIGS,
  ROCSHMEM_TEAM_NUM_CONTEXTS
};

typedef struct {
  int num_contexts;
} rocshmem_team_config_t;

// Sync-array sizes kept for source compatibility with active-set style host calls. The runtime
// owns all synchronisation state, so user pSync arrays are accepted and ignored.
constexpr size_t ROCSHMEM_REDUCE_MIN_WRKDATA_SIZE = 1024;
constexpr size_t ROCSHMEM_BARRIER_SYNC_SIZE = 256;
constexpr size_t ROCSHMEM_REDUCE_SYNC_SIZE = 256;
constexpr size_t ROCSHMEM_BCAST_SYNC_SIZE = ROCSHMEM_BARRIER_SYNC_SIZE;
constexpr size_t ROCSHMEM_ALLTOALL_SYNC_SIZE = ROCSHMEM_BARRIER_SYNC_SIZE + 1;
constexpr size_t ROCSHMEM_FCOLLECT_SYNC_SIZE = ROCSHMEM_ALLTOALL_SYNC_SIZE;
constexpr size_t ROCSHMEM_SYNC_VALUE = 0;

const int ROCSHMEM_CTX_ZERO = 0;
const int ROCSHMEM_CTX_NOSTORE = 1;
const int ROCSHMEM_CTX_SERIALIZED = 2;
const int ROCSHMEM_CTX_WG_PRIVATE = 4;
const int ROCSHMEM_CTX_SHARED = 8;

// Limits (defaults; the env vars of the same names lower or raise the first three).
constexpr int ROCSHMEM_MAX_PES = 64;            // PEs addressable in one window
constexpr int ROCSHMEM_DEFAULT_MAX_TEAMS = 40;  // slot 0 is TEAM_WORLD
constexpr int ROCSHMEM_DEFAULT_MAX_CTXS = 1024;
constexpr int ROCSHMEM_DEFAULT_MAX_HOST_CTXS = 40;
constexpr int ROCSHMEM_TEAM_SLOTS = 64;         // hard upper bound on ROCSHMEM_MAX_NUM_TEAMS
constexpr int ROCSHMEM_CTX_SLOTS = 4096;        // hard upper bound on ROCSHMEM_MAX_NUM_CONTEXTS
constexpr size_t ROCSHMEM_ALIGNMENT = 128;      // allocation granularity of rocshmem_malloc

// ---------------------------------------------------------------------------------------------
// Device-visible descriptors. They live in the internal region of every PE's heap at identical
// offsets, so "the same object on PE p" is reached by the usual symmetric translation.
// ---------------------------------------------------------------------------------------------

// Which wait / check recorded an error (see rocshmem_error_record).
enum rocshmem_error_kind : uint32_t {
  ROCSHMEM_ERR_NONE = 0,
  ROCSHMEM_ERR_WAIT_TIMEOUT = 1,     // wait_until family ran out of budget
  ROCSHMEM_ERR_BARRIER_TIMEOUT = 2,  // barrier / sync / collective flag wait ran out of budget
  ROCSHMEM_ERR_BAD_PE = 3,           // debug build: pe outside [0, n_pes)
  ROCSHMEM_ERR_BAD_ADDRESS = 4,      // debug build: symmetric address outside the heap
  ROCSHMEM_ERR_CTX_EXHAUSTED = 5,
  ROCSHMEM_ERR_PROXY_TIMEOUT = 6,    // reverse-offload ring: no slot / no completion in time
  ROCSHMEM_ERR_GRID_TIMEOUT = 7,     // intra-kernel grid barrier ran out of budget
  ROCSHMEM_ERR_KERNEL = 8,           // a library kernel gave up (mbarrier, TMEM, ...)
};

// First error wins (count keeps increasing); the host reads it with rocshmemx_get_error().
struct rocshmem_error_record {
  unsigned int count;
  uint32_t kind;
  int pe;         // PE involved (peer waited for, bad pe, ...) or -1
  int where;      // call-site tag
  uint64_t addr;
  uint64_t expected;
  uint64_t observed;
};

// Team descriptor. One per (PE, team slot).
struct rocshmem_team_dev {
  int pe_start;   // first member, world numbering
  int stride;     // world stride between members
  int size;       // number of members
  int my_pe;      // my index in the team, -1 if this PE is not a member
  int slot;       // index into the per-team sync pools
  int valid;
  int world_size;
  int my_pe_world;
  // Monotonic epochs of the team's collectives. Every member performs the same sequence of
  // collectives, so the counters agree without communication. Flags are never reset: a waiter
  // compares against the epoch it expects (>=), which removes the reset phase and its races.
  unsigned long long barrier_epoch;
  // Calls of the flag-in-word small allreduce on this team so far (its words carry the call's number).
  unsigned long long ll_epoch;
  // NVLink multicast mapping of the heap that spans exactly this team's members (nullptr: none).
  char *mc_base;
};

// Context descriptor (device pool entry).
struct rocshmem_ctx_dev {
  long long options;
  rocshmem_team_dev *team;
  int id;
  int in_use;
  unsigned long long ops;  // operations issued through this context (stats)
};

typedef struct {
  void *ctx_opaque;   // rocshmem_ctx_dev* (device) or host context object
  void *team_opaque;  // rocshmem_team_dev* of the context's team
} rocshmem_ctx_t;

typedef rocshmem_team_dev *rocshmem_team_t;
#define ROCSHMEM_TEAM_INVALID ((::rocshmem::rocshmem_team_t) nullptr)

// Counters of device-side API use; compiled in with -DROCSHMEM_PROFILE (reference: src/stats.hpp).
enum rocshmem_stat_id {
  ROCSHMEM_STAT_PUT = 0, ROCSHMEM_STAT_PUT_NBI, ROCSHMEM_STAT_P, ROCSHMEM_STAT_GET,
  ROCSHMEM_STAT_GET_NBI, ROCSHMEM_STAT_G, ROCSHMEM_STAT_PUT_WARP, ROCSHMEM_STAT_PUT_BLOCK,
  ROCSHMEM_STAT_GET_WARP, ROCSHMEM_STAT_GET_BLOCK, ROCSHMEM_STAT_PUT_SIGNAL,
  ROCSHMEM_STAT_SIGNAL_FETCH, ROCSHMEM_STAT_AMO_FETCH, ROCSHMEM_STAT_AMO_NOFETCH,
  ROCSHMEM_STAT_FENCE, ROCSHMEM_STAT_QUIET, ROCSHMEM_STAT_WAIT, ROCSHMEM_STAT_TEST,
  ROCSHMEM_STAT_BARRIER, ROCSHMEM_STAT_SYNC, ROCSHMEM_STAT_BROADCAST, ROCSHMEM_STAT_REDUCE,
  ROCSHMEM_STAT_FCOLLECT, ROCSHMEM_STAT_ALLTOALL, ROCSHMEM_STAT_CTX_CREATE,
  ROCSHMEM_STAT_CTX_DESTROY, ROCSHMEM_STAT_BYTES_PUT, ROCSHMEM_STAT_BYTES_GET,
  ROCSHMEM_STAT_PROXY_CMD, ROCSHMEM_STAT_TIMEOUTS,
  // Nanoseconds spent by device threads, summed over threads (reference: the reverse-offload profiler's
  // WAITING_ON_SLOT / PACK_QUEUE + THREAD_FENCE / WAITING_ON_HOST / SHMEM_WAIT buckets,
  // src/reverse_offload/profiler.hpp:36-50).
  ROCSHMEM_STAT_PROXY_SLOT_NS, ROCSHMEM_STAT_PROXY_PACK_NS, ROCSHMEM_STAT_PROXY_HOST_NS,
  ROCSHMEM_STAT_WAIT_NS,
  ROCSHMEM_NUM_STATS
};

// The reverse-offload command ring (host-thread proxy fallback). Lives in pinned, device-mapped
// host memory; the device produces, one host thread consumes.
struct rocshmem_proxy_cmd {
  volatile unsigned int valid;   // 0 free, 1 published by the device, 2 being executed
  unsigned int type;             // rocshmem_proxy_op
  int pe;
  int status_slot;               // index into the completion array, -1 for fire-and-forget
  unsigned long long dst;        // symmetric address (initiator's view)
  unsigned long long src;
  unsigned long long size;       // bytes, or atomic operand
  unsigned long long cond;       // compare value for CAS
  unsigned int op;               // amo sub-operation / signal op
  unsigned int dtype_size;
  unsigned long long team_slot;  // collectives: sync-pool slot of the team (0: world)
};
static_assert(sizeof(rocshmem_proxy_cmd) == 64, "one command per 64-byte line");

enum rocshmem_proxy_op : unsigned int {
  ROCSHMEM_PROXY_NOP = 0,
  ROCSHMEM_PROXY_PUT = 1,
  ROCSHMEM_PROXY_GET = 2,
  ROCSHMEM_PROXY_AMO_FADD = 3,
  ROCSHMEM_PROXY_AMO_CAS = 4,
  ROCSHMEM_PROXY_QUIET = 5,
  ROCSHMEM_PROXY_BARRIER = 6,
  ROCSHMEM_PROXY_SIGNAL = 7,
  // Host-executed forms of the remaining operations (world team): `pe` is the root, `size` the payload in
  // bytes (elements for REDUCE), `cond` the element type (rocshmem_dtype) and `op` the reduction operator.
  ROCSHMEM_PROXY_FENCE = 8,
  ROCSHMEM_PROXY_BROADCAST = 9,
  ROCSHMEM_PROXY_REDUCE = 10,
  ROCSHMEM_PROXY_FCOLLECT = 11,
  ROCSHMEM_PROXY_ALLTOALL = 12,
  ROCSHMEM_PROXY_P = 13,          // single element put by value: `size` holds the bits, dtype_size its width
  ROCSHMEM_PROXY_AMO = 14,        // any other atomic: `op` is the host's operation code (fetch 0, swap 1, cas 2,
                                  // add 3, and 4, or 5, xor 6), `size` the operand, `cond` the compare value
};

struct rocshmem_proxy_ring {
  rocshmem_proxy_cmd *cmds;               // [capacity], pinned host memory (device-mapped)
  unsigned int capacity;                  // power of two
  unsigned int n_status;
  unsigned long long *write_index;        // device memory: next slot to reserve
  volatile unsigned long long *read_index;  // pinned host: slots retired by the host thread
  volatile unsigned long long *status;    // pinned host [n_status]: 0 pending, 1 done, 2 failed
  volatile unsigned long long *fetched;   // pinned host [n_status]: value returned by fetching ops
};

// One per local PE; copied into __constant__ memory of every CUDA module that uses the device API.
struct rocshmem_device_state {
  int my_pe;
  int n_pes;
  int n_local;            // PEs hosted by this process on this GPU (1 unless emulation mode)
  int local_index;        // index of this PE among the process's local PEs
  char *heap_base;        // this PE's heap inside the window
  char *window_base;      // PE 0's heap; PE p's heap is window_base + p * heap_stride
  size_t heap_stride;     // bytes between consecutive PEs' heaps (user heap + internal region)
  size_t heap_size;       // user-visible heap bytes (ROCSHMEM_HEAP_SIZE)
  char *mc_base;          // NVLS multicast mapping of the heap (nullptr when unavailable)
  char *internal_base;    // this PE's internal region (= heap_base + heap_size)

  // Internal region, local addresses. Remote instances are reached by translation.
  rocshmem_team_dev *teams;            // [max_teams]
  rocshmem_ctx_dev *ctxs;              // [max_ctxs]
  unsigned long long *ctx_free_mask;   // bitmask over ctxs, 1 = free
  unsigned long long *barrier_flags;   // [max_teams][ROCSHMEM_MAX_PES] arrival epochs
  unsigned long long *lib_flags;       // [ROCSHMEM_LIB_FLAG_WORDS] flags of library kernels
  unsigned long long *lib_state;       // [ROCSHMEM_LIB_STATE_WORDS] local epochs of library kernels
  unsigned long long *ll_buf;          // [ROCSHMEM_TEAM_SLOTS][2][n_pes][ROCSHMEM_LL_WORDS] small-allreduce mailboxes
  char *scratch;                       // staging for library collectives
  size_t scratch_size;
  rocshmem_error_record *error;        // first-error record
  unsigned long long *stats;           // [ROCSHMEM_NUM_STATS]
  rocshmem_proxy_ring *proxy;          // nullptr unless the proxy is enabled

  int max_teams;
  int max_ctxs;
  unsigned long long wait_timeout_ns;  // budget of every device-side wait
  int debug_checks;                    // 1: validate pe / symmetric addresses on the device
  int use_proxy;                       // bit 0: route thread-level RMA/AMO through the host proxy;
                                       // bit 1: coalesce contiguous messages of neighbouring lanes first;
                                       // bit 2: block-level collectives are executed by the proxy
  int device_ordinal;                  // CUDA device that hosts this PE
};

// Library (multi-block) collectives: block b of a PE synchronises with block b of every peer, so
// flags are indexed [team slot][block][peer] and local epochs [team slot][block].
constexpr int ROCSHMEM_LIB_MAX_BLOCKS = 256;
constexpr int ROCSHMEM_LIB_FLAG_WORDS = ROCSHMEM_TEAM_SLOTS * ROCSHMEM_LIB_MAX_BLOCKS * ROCSHMEM_MAX_PES;
constexpr int ROCSHMEM_LIB_STATE_WORDS = ROCSHMEM_TEAM_SLOTS * ROCSHMEM_LIB_MAX_BLOCKS;
constexpr int ROCSHMEM_MAX_LOCAL_PES = 8;
// Small allreduce: every member owns a mailbox of this many 8-byte words (4 bytes of data + the call's number) in
// every other member's heap, two per team slot (calls alternate between them).
constexpr int ROCSHMEM_LL_WORDS = 512;

}  // namespace rocshmem

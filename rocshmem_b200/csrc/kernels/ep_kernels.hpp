// Expert-parallel MoE dispatch / combine on the symmetric heap, and the block-scaled fp8 helpers.
// Host-callable launchers; pointers to symmetric memory are addresses on the process's first local PE.
//
// No counterpart exists in the reference (its nearest primitive is the fixed-size alltoall,
// src/ipc/context_ipc_tmpl_device.hpp:474-501); the operations are built from the same ingredients
// the reference exposes - peer stores, signals, bounded waits, teams - fused into two kernels.
#pragma once

#include <cstddef>
#include <cstdint>

#include "rocshmem/rocshmem_common.h"

namespace rocshmem {
namespace kernels {

constexpr int EP_META_WORDS = 32;      // 128-byte metadata record per received row
constexpr int EP_META_IDX = 0;         // [0, top_k): expert index local to the receiver, -1 if elsewhere
constexpr int EP_META_WEIGHT = 8;      // [8, 8 + top_k): gate weights (float bits)
constexpr int EP_META_SRC_TOKEN = 16;  // token index on the source rank
constexpr int EP_META_SRC_RANK = 17;   // source rank (team numbering)
constexpr int EP_META_RANK = 24;       // [24, 24 + top_k): position of this (token, k) pair among the source's
                                       // pairs for the same expert (staged hand-out and low-latency kernels)
constexpr int EP_MAX_TOPK = 8;
constexpr int EP_MAX_HIDDEN = 8192;
constexpr int EP_MAX_RANKS = 32;       // destinations live in the lanes of a warp

enum EpLayout : int {
  EP_LAYOUT_COMPACT = 0,  // rows of source s start at the sum of the counts of sources < s
  EP_LAYOUT_SLOTTED = 1,  // rows of source s start at s * max_tokens: no count round-trip before
                          // sending (low-latency mode), at the price of gaps in the receive buffer
};

struct EpConfig {
  int num_experts;     // global, divisible by the team size
  int top_k;           // <= 8
  int hidden;          // multiple of 512, <= 8192
  int max_tokens;      // per rank and call
  int quantize;        // 1: dispatch carries e4m3 rows + one fp32 scale per 128 elements; 0: bf16 rows
  int layout;          // EpLayout
  int blocks;          // blocks per PE (the same on every member)
  int dynamic;         // 1: dispatch hands (token, destination) pairs to warps through per-destination counters;
                       //    combine hands tokens out through a counter. 0: fixed per-block shares of whole tokens.
  int expert_layout;   // 1: the dispatch kernel also writes the expert-grouped pair lists (EpBuffers::lay_*)
  int low_latency;     // 1: one non-cooperative launch, a block per token, slotted layout, per-source signals
};

// What dispatch and combine accept (0) or refuse (1 = cudaErrorInvalidValue). Pure host logic, shared by the
// launchers and the CPU unit tests.
inline int ep_config_error(const EpConfig &cfg, int team_size, int num_tokens) {
  // Destinations live in the lanes of a warp (slot shuffles, per-lane weights), hence at most 32 ranks.
  if (team_size < 1 || team_size > EP_MAX_RANKS) return 1;
  if (cfg.num_experts < team_size || cfg.num_experts % team_size || cfg.num_experts > 1024) return 1;
  if (cfg.top_k < 1 || cfg.top_k > EP_MAX_TOPK) return 1;
  if (cfg.hidden < 512 || cfg.hidden % 512 || cfg.hidden > EP_MAX_HIDDEN) return 1;
  if (num_tokens < 0 || num_tokens > cfg.max_tokens) return 1;
  // block_pair_barrier keeps one flag row per block.
  if (cfg.blocks < 1 || cfg.blocks > ROCSHMEM_LIB_MAX_BLOCKS) return 1;
  if (cfg.low_latency && cfg.layout != EP_LAYOUT_SLOTTED) return 1;
  return 0;
}

// Blocks of a low-latency combine: a function of the configuration only, because every member must launch the
// same number (block b pairs with block b of the peers) while their token counts may differ.
inline int ep_ll_combine_blocks(const EpConfig &cfg) {
  const int warps = cfg.max_tokens * 4;
  const int blocks = (warps + 3) / 4;
  return blocks < 1 ? 1 : (blocks > ROCSHMEM_LIB_MAX_BLOCKS ? ROCSHMEM_LIB_MAX_BLOCKS : blocks);
}

// Words of EpBuffers::work_counter.
constexpr int EP_WORK_DISPATCH = 0;    // [2][EP_MAX_RANKS]: next item per destination, by call parity
constexpr int EP_WORK_COMBINE = 64;    // tokens handed out by all combine calls so far (never reset)
constexpr int EP_WORK_LL_DONE = 65;    // low-latency dispatch: blocks that have finished sending
constexpr int EP_WORK_LL_ROWS = 66;    // [EP_MAX_RANKS]: rows sent to each destination by the running call
constexpr int EP_WORK_WORDS = 128;

// Symmetric buffers of one dispatcher (all allocated by the caller on the symmetric heap).
struct EpBuffers {
  void *recv_x;             // [P * max_tokens, hidden] uint8 (quantize) or bf16
  float *recv_scales;       // [P * max_tokens, hidden / 128]
  int *recv_meta;           // [P * max_tokens, EP_META_WORDS]
  // Both double-buffered by call parity: a peer that is one call ahead does not overwrite words that
  // this PE still reads.
  unsigned long long *cnt_in;   // [2][P][P] packed (epoch << 32 | tokens source s sends to rank d), full matrix
  unsigned long long *exp_in;   // [2][P][experts_per_rank] packed (epoch << 32 | rows for local expert e from s)
  // local scratch (symmetric allocation for simplicity, only ever accessed by its owner)
  int *sent_slot;           // [max_tokens][P] row index at destination d, -1 if not sent
  unsigned long long *tok_mask;  // [max_tokens] bit d set: token goes to rank d
  int *blk_cnt;             // [blocks][P]
  int *exp_cnt;             // [2][num_experts] double-buffered by call parity
  unsigned long long *grid_counter;  // [1]
  // [16] device timestamps (ns) written by block 0: dispatch phases in [0, 8), combine in [8, 16).
  // Always on: eight 8-byte stores per kernel.
  unsigned long long *phase_ns;
  // outputs, local
  int *recv_info;           // [0] total rows, [1 + s] first row of source s, [1 + P + s] rows of source s,
                            // [1 + 2 P + e] (row, k) pairs of local expert e
  unsigned long long *work_counter;  // [EP_WORK_WORDS], see EP_WORK_*
  // Pair hand-out (dynamic == 1), local.
  int *stage_meta;          // [max_tokens, EP_META_WORDS] record of every token with global expert ids
  int *item_tok;            // [P][max_tokens] token of this rank's i-th row for destination d
  // Expert-grouped pair lists (expert_layout == 1), local outputs: positions lay_offsets[e] .. lay_offsets[e + 1]
  // belong to local expert e; lay_row / lay_k / lay_w give the received row, the top-k position and the gate
  // weight of the pair at a position.
  int *lay_offsets;         // [experts_per_rank + 1]
  int *lay_row;             // [P * max_tokens * top_k]
  int *lay_k;
  float *lay_w;
};

// x [T, hidden] bf16, topk_idx [T, top_k] int32 (global expert ids, -1 = unused), topk_w [T, top_k] fp32.
// `epoch` must increase by one per dispatch call on these buffers (the same value on every member).
int ep_dispatch(rocshmem_team_t team, const EpConfig &cfg, const EpBuffers &buf, const void *x,
                const int *topk_idx, const float *topk_w, int num_tokens, unsigned epoch, void *stream);

// y: symmetric [P * max_tokens, hidden] bf16 in the row layout produced by dispatch. out [T, hidden]
// bf16 (local). Every token receives the sum over the ranks it was sent to of that rank's row,
// scaled (weighted != 0) by the sum of the token's gate weights of the experts living on that rank.
// `combine_calls_base` (dynamic mode only): value of work_counter[EP_WORK_COMBINE] when this call starts, i.e. the
// sum over the earlier combine calls on these buffers of ep_combine_fetches(cfg, their num_tokens).
// In low-latency mode a token is shared by four warps and the closing "done reading" barrier is left out: `y` may
// be rewritten only after the next dispatch on these buffers has completed on this rank (every peer finishes its
// combine before it starts that dispatch, and the dispatch waits for every peer's signal).
int ep_combine(rocshmem_team_t team, const EpConfig &cfg, const EpBuffers &buf, const void *y, void *out,
               const int *topk_idx, const float *topk_w, int num_tokens, int weighted, void *stream,
               unsigned long long combine_calls_base = 0);
// Counter increments of one dynamic combine call: one per token plus one failing fetch per warp.
unsigned long long ep_combine_fetches(const EpConfig &cfg, int num_tokens);

// Stand-alone 1x128 block-scaled e4m3 quantisation of [rows, hidden] bf16 and its inverse.
int fp8_quantize_1x128(const void *x_bf16, void *q_u8, float *scales, size_t rows, int hidden, void *stream);
int fp8_dequantize_1x128(const void *q_u8, const float *scales, void *x_bf16, size_t rows, int hidden, void *stream);

// Groups received rows by local expert for a grouped GEMM: for every local expert e, the indices of
// the rows whose top-k contains e, written contiguously; offsets[e] .. offsets[e + 1]. `pair_k`
// receives the top-k position inside the row's metadata. Returns through `offsets` (E_local + 1).
int ep_expert_layout(const int *recv_meta, const int *recv_info, int n_ranks, int max_tokens, int layout,
                     int experts_per_rank, int top_k, int *offsets, int *row_index, int *pair_k,
                     int *cursor_scratch, void *stream);

int ep_default_blocks();

}  // namespace kernels
}  // namespace rocshmem

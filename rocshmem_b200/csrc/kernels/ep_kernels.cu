// Expert-parallel MoE dispatch and combine as fused kernels over NVLink peer memory.
//
// Dispatch, normal mode (one cooperative kernel per rank):
//   A. every block scans its share of the tokens: destination-rank bitmask per token (a token that
//      selects several experts of one rank is sent to that rank once), per-block per-rank counts,
//      per-expert counts and the position of every (token, k) pair among this rank's pairs for its expert;
//   B. after one grid barrier each block derives its write offsets; block 0 publishes this rank's row
//      of the rank-to-rank count matrix, and the per-expert counts, to every peer as single 64-bit
//      words that carry the call's epoch in their upper half (data and "ready" flag in one store, so
//      no fence and no separate flag);
//   C. rows are quantised to e4m3 with one fp32 scale per 128 elements in registers (amax by shuffles
//      inside 8-lane groups) and stored with 16-byte peer stores straight into their final rows of the
//      destinations' receive buffers, together with the scales and a 128-byte metadata record. There is
//      no receiver-side copy. Two ways of sharing the work:
//        fixed shares   a warp owns whole tokens of its block and sends each to all its destinations;
//        pairs          warps take (token, destination) pairs from per-destination counters, so that no warp is
//                       left with eight destinations while another has one; a row is quantised again for every
//                       destination (re-reading it from L2 costs less than a staging pass that idles the links);
//   D. blocks pair up with the same block of every peer (release/acquire flags), so when the kernel
//      has finished on a rank, everything sent to that rank is visible to its next kernel;
//   E. on request, after one more grid barrier, all blocks turn the received metadata into the expert-grouped
//      pair lists a grouped GEMM consumes (no atomics: a pair's position is its expert's offset + the pairs of
//      earlier sources + the position its source gave it).
//
// Dispatch, low-latency mode (one ordinary launch, a block of four warps per token, slotted layout): rows go out as
// soon as they are quantised, the last block to finish sends one signal word per destination that carries the row
// count (release), then waits for the signals of all sources. No grid barrier, no count round-trip.
//
// Combine (one kernel per rank) is a pull: for each of its tokens a warp reads the result rows from
// the (up to top_k) ranks the token went to, 16 bytes per lane with the loads of all sources in
// flight together, accumulates in fp32 with the per-rank gate weight, and writes the bf16 row once.
// Pulling needs no staging memory and no receive-side reduction pass. In low-latency mode four warps share a
// token.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "ep_kernels.hpp"
#include "launch.cuh"
#include "lib_common.cuh"

namespace rocshmem {
namespace kernels {

namespace {

constexpr unsigned kEpThreads = 512;
constexpr unsigned kCombineThreads = 384;  // 170 registers per thread: room for 16 loads in flight
constexpr int kMaxIters = EP_MAX_HIDDEN / 512;  // 16 iterations of 512 elements per warp

using detail::remote_ptr;
using detail::team_pe_to_world;

__device__ __forceinline__ unsigned long long pack(unsigned epoch, unsigned value) {
  return (static_cast<unsigned long long>(epoch) << 32) | value;
}

// Spin (bounded) until the word carries `epoch`; returns its payload, or 0 with *ok = false. A tag that is newer
// than `epoch` can never turn into `epoch` again (the sender is a call ahead of what the buffers allow), so it is
// reported at once instead of after the whole budget.
__device__ __forceinline__ unsigned wait_packed(const unsigned long long *p, unsigned epoch, int peer, bool *ok) {
  unsigned long long v = detail::ld_relaxed_sys(p);
  if (static_cast<unsigned>(v >> 32) != epoch) {
    detail::SpinBudget budget(st().wait_timeout_ns);
    while (static_cast<unsigned>((v = detail::ld_relaxed_sys(p)) >> 32) != epoch) {
      const bool newer = static_cast<int>(static_cast<unsigned>(v >> 32) - epoch) > 0;
      if (newer || !budget.keep_going()) {
        detail::record_error(ROCSHMEM_ERR_BARRIER_TIMEOUT, peer, newer ? 71 : 70, p, epoch, v);
        *ok = false;
        return 0;
      }
    }
  }
  return static_cast<unsigned>(v & 0xffffffffu);
}

struct DispatchArgs {
  EpConfig cfg;
  EpBuffers buf;
  const __nv_bfloat16 *x;
  const int *topk_idx;
  const float *topk_w;
  int num_tokens;
  unsigned epoch;
  rocshmem_team_t team;
};

__device__ __forceinline__ float group8_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
  return v;
}

__device__ __forceinline__ unsigned pack_fp8x4(float a, float b, float c, float d) {
  unsigned lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  unsigned hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// Quantises the 16 bf16 values held by a lane (two int4) with the scale of its 8-lane group.
__device__ __forceinline__ int4 quantize16(const int4 &a, const int4 &b, float *scale_out) {
  const __nv_bfloat162 *pa = reinterpret_cast<const __nv_bfloat162 *>(&a);
  const __nv_bfloat162 *pb = reinterpret_cast<const __nv_bfloat162 *>(&b);
  float v[16];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
    v[2 * i] = fa.x; v[2 * i + 1] = fa.y;
    v[8 + 2 * i] = fb.x; v[8 + 2 * i + 1] = fb.y;
  }
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  amax = group8_max(amax);
  // e4m3 represents magnitudes up to 448. An all-zero block keeps scale 1 so that 0 * scale == 0.
  const float scale = amax > 0.f ? amax * (1.0f / 448.0f) : 1.0f;
  const float inv = amax > 0.f ? 448.0f / amax : 1.0f;
  *scale_out = scale;
  int4 q;
  q.x = pack_fp8x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
  q.y = pack_fp8x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
  q.z = pack_fp8x4(v[8] * inv, v[9] * inv, v[10] * inv, v[11] * inv);
  q.w = pack_fp8x4(v[12] * inv, v[13] * inv, v[14] * inv, v[15] * inv);
  return q;
}

// Copies `nvec` 16-byte vectors with all loads of a batch (N per lane) in flight before the first store.
template <int N>
__device__ __forceinline__ void copy_row_vec(int4 *dst, const int4 *src, int nvec, unsigned lane) {
  for (int v0 = 0; v0 < nvec; v0 += 32 * N) {
    int4 r[N];
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const int v = v0 + i * 32 + int(lane);
      if (v < nvec) r[i] = __ldcg(src + v);
    }
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const int v = v0 + i * 32 + int(lane);
      if (v < nvec) dst[v] = r[i];
    }
  }
}

// Exclusive prefix sum of data[0 .. n) in place (n <= 1024), done by the first warp of the block; returns the
// total through *total. Callers synchronise the block before and after.
__device__ __forceinline__ void warp0_exclusive_scan(int *data, int n, int *total) {
  if (threadIdx.x >= 32) return;
  const int lane = threadIdx.x;
  const int chunk = (n + 31) / 32;
  const int lo = min(n, lane * chunk), hi = min(n, lo + chunk);
  int sum = 0;
  for (int i = lo; i < hi; ++i) sum += data[i];
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  int run = incl - sum;
  for (int i = lo; i < hi; ++i) {
    const int c = data[i];
    data[i] = run;
    run += c;
  }
  if (lane == 31) *total = incl;
}

// Receive-side bookkeeping shared by the dispatch kernels: rows per source, first row per source, rows per local
// expert. Called by one whole block once every source's counts are known to have been sent.
__device__ __forceinline__ void write_recv_info(const DispatchArgs &a, const rocshmem_team_dev *t, int *recv_info,
                                                const unsigned long long *cnt_in, const unsigned long long *exp_in) {
  const int P = t->size, me = t->my_pe, epr = a.cfg.num_experts / P;
  const unsigned tid = threadIdx.x, nthr = blockDim.x;
  for (unsigned s = tid; s < unsigned(P); s += nthr) {
    bool good = true;
    int start = 0, mine = 0;
    for (int s2 = 0; s2 <= int(s); ++s2) {
      const int c = static_cast<int>(wait_packed(cnt_in + s2 * P + me, a.epoch, s2, &good));
      if (s2 < int(s)) start += c; else mine = c;
    }
    recv_info[1 + s] = a.cfg.layout == EP_LAYOUT_SLOTTED ? int(s) * a.cfg.max_tokens : start;
    recv_info[1 + P + s] = mine;
    if (s == unsigned(P - 1)) recv_info[0] = start + mine;
  }
  for (unsigned e = tid; e < unsigned(epr); e += nthr) {
    bool good = true;
    int sum = 0;
    for (int s = 0; s < P; ++s) sum += static_cast<int>(wait_packed(exp_in + s * epr + e, a.epoch, s, &good));
    recv_info[1 + 2 * P + e] = sum;
  }
}

// Expert-grouped pair lists from the metadata of the received rows. s_off / s_src are shared-memory tables of
// experts_per_rank + 1 and P * experts_per_rank ints. Every thread of every calling block takes part; `part` of
// `parts` selects the share of the rows this block scans. All rows must be visible to the caller.
__device__ __forceinline__ bool build_expert_layout(const DispatchArgs &a, const rocshmem_team_dev *t,
                                                    const unsigned long long *cnt_in,
                                                    const unsigned long long *exp_in, const int *recv_meta,
                                                    int *s_off, int *s_src, int *s_total, unsigned part,
                                                    unsigned parts) {
  const int P = t->size, me = t->my_pe, epr = a.cfg.num_experts / P, K = a.cfg.top_k;
  const unsigned tid = threadIdx.x, nthr = blockDim.x;
  int *lay_offsets = rebase(a.buf.lay_offsets), *lay_row = rebase(a.buf.lay_row), *lay_k = rebase(a.buf.lay_k);
  float *lay_w = rebase(a.buf.lay_w);
  const int cap = P * a.cfg.max_tokens * K;
  bool ok = true;
  for (unsigned e = tid; e < unsigned(epr); e += nthr) {
    int run = 0;
    for (int s = 0; s < P; ++s) {
      s_src[s * epr + e] = run;  // pairs of expert e that come from sources before s
      run += static_cast<int>(wait_packed(exp_in + s * epr + e, a.epoch, s, &ok));
    }
    s_off[e] = run;
  }
  __syncthreads();
  warp0_exclusive_scan(s_off, epr, s_total);
  __syncthreads();
  if (part == 0) {
    for (unsigned e = tid; e < unsigned(epr); e += nthr) lay_offsets[e] = s_off[e];
    if (tid == 0) lay_offsets[epr] = *s_total;
  }
  int start = 0;
  for (int s = 0; s < P; ++s) {
    const int count = static_cast<int>(wait_packed(cnt_in + s * P + me, a.epoch, s, &ok));
    const int first = a.cfg.layout == EP_LAYOUT_SLOTTED ? s * a.cfg.max_tokens : start;
    start += count;
    for (int i = part * nthr + tid; i < count * K; i += parts * nthr) {
      const int row = first + i / K, k = i % K;
      const int *meta = recv_meta + size_t(row) * EP_META_WORDS;
      const int e = meta[EP_META_IDX + k];
      if (e >= 0 && e < epr) {
        const int pos = s_off[e] + s_src[s * epr + e] + meta[EP_META_RANK + k];
        if (pos < 0 || pos >= cap) continue;  // inconsistent record: never write outside the lists
        lay_row[pos] = row;
        lay_k[pos] = k;
        lay_w[pos] = __int_as_float(meta[EP_META_WEIGHT + k]);
      }
    }
  }
  return ok;
}

// STAGED: (token, destination) pairs handed out through counters (see the top of the file); otherwise fixed shares
// of whole tokens.
template <bool STAGED>
__global__ void __launch_bounds__(kEpThreads, 1) ep_dispatch_kernel(DispatchArgs a) {
  // masks [tpb] u64, ranks among the block's tokens per destination [tpb][P] int, pair ranks [tpb][K] int
  extern __shared__ __align__(16) unsigned char s_dyn[];
  __shared__ int s_rank_cnt[EP_MAX_RANKS];
  __shared__ int s_blk_base[EP_MAX_RANKS];
  __shared__ int s_total[EP_MAX_RANKS];
  __shared__ int s_base[EP_MAX_RANKS];
  __shared__ int s_exp_cnt[1024];   // phase A: pairs per expert in this block; phase E: offsets per local expert
  __shared__ int s_exp_base[1024];  // phase A: first position of the block's pairs; phase E: pairs of earlier sources
  // Read back as float4 vectors, so the array needs 16-byte alignment (float alone guarantees 4).
  __shared__ __align__(16) float s_scales[kEpThreads / 32][EP_MAX_HIDDEN / 128];
  __shared__ int s_ok;
  __shared__ int s_lay_total;

  const rocshmem_team_dev *t = detail::team_of(a.team);
  if (t->my_pe < 0) return;
  const int P = t->size, me = t->my_pe;
  const int E = a.cfg.num_experts, epr = E / P, K = a.cfg.top_k, H = a.cfg.hidden;
  const int T = a.num_tokens;
  const unsigned tid = threadIdx.x, nthr = blockDim.x, b = blockIdx.x, B = gridDim.x;
  const unsigned epoch = a.epoch;
  const int parity = epoch & 1;

  const __nv_bfloat16 *x = rebase(a.x);
  const int *topk_idx = rebase(a.topk_idx);
  const float *topk_w = rebase(a.topk_w);
  char *recv_x = static_cast<char *>(rebase(a.buf.recv_x));
  float *recv_scales = rebase(a.buf.recv_scales);
  int *recv_meta = rebase(a.buf.recv_meta);
  unsigned long long *cnt_in = rebase(a.buf.cnt_in) + size_t(parity) * P * P;
  unsigned long long *exp_in = rebase(a.buf.exp_in) + size_t(parity) * P * epr;
  int *sent_slot = rebase(a.buf.sent_slot);
  unsigned long long *tok_mask = rebase(a.buf.tok_mask);
  int *blk_cnt = rebase(a.buf.blk_cnt);
  int *exp_cnt = rebase(a.buf.exp_cnt);
  unsigned long long *grid_counter = rebase(a.buf.grid_counter);
  int *recv_info = rebase(a.buf.recv_info);
  int *stage_meta = STAGED ? rebase(a.buf.stage_meta) : nullptr;
  int *item_tok = STAGED ? rebase(a.buf.item_tok) : nullptr;

  const int tpb = (a.cfg.max_tokens + B - 1) / B;  // tokens per block, fixed for the buffer's life
  const int t0 = min(T, int(b) * tpb), t1 = min(T, t0 + tpb);
  unsigned long long *s_mask = reinterpret_cast<unsigned long long *>(s_dyn);
  int *s_rank_in_block = reinterpret_cast<int *>(s_dyn + size_t(tpb) * sizeof(unsigned long long));
  int *s_pair_rank = s_rank_in_block + size_t(tpb) * P;
  unsigned long long *phase_ns = rebase(a.buf.phase_ns);
  const bool stamp = (b == 0 && tid == 0);
  if (stamp) phase_ns[0] = detail::now_ns();
  // Grid barriers of one call: 1 (fixed shares), 2 (staged pairs), + 1 with the expert layout.
  const unsigned long long rounds = (STAGED ? 2ull : 1ull) + (a.cfg.expert_layout ? 1ull : 0ull);
  unsigned long long round = rounds * (epoch - 1);
  unsigned long long *work = STAGED ? rebase(a.buf.work_counter) + EP_WORK_DISPATCH : nullptr;
  if (STAGED && b == 0 && tid < EP_MAX_RANKS) work[(parity ^ 1) * EP_MAX_RANKS + tid] = 0;  // for the next call

  // ---- A: routing scan ------------------------------------------------------------------------------
  for (unsigned i = tid; i < EP_MAX_RANKS; i += nthr) s_rank_cnt[i] = 0;
  for (unsigned i = tid; i < unsigned(E); i += nthr) s_exp_cnt[i] = 0;
  if (tid == 0) s_ok = 1;
  __syncthreads();
  for (int tok = t0 + tid; tok < t1; tok += nthr) {
    unsigned long long mask = 0;
    for (int k = 0; k < K; ++k) {
      const int e = topk_idx[size_t(tok) * K + k];
      int rank = 0;
      if (e >= 0 && e < E) {
        mask |= 1ull << (e / epr);
        rank = atomicAdd(&s_exp_cnt[e], 1);
      }
      s_pair_rank[(tok - t0) * K + k] = rank;
    }
    tok_mask[tok] = mask;
    s_mask[tok - t0] = mask;
    for (unsigned long long m = mask; m; m &= m - 1) atomicAdd(&s_rank_cnt[__ffsll(static_cast<long long>(m)) - 1], 1);
  }
  __syncthreads();
  for (unsigned d = tid; d < unsigned(P); d += nthr) blk_cnt[b * P + d] = s_rank_cnt[d];
  for (unsigned e = tid; e < unsigned(E); e += nthr) {
    s_exp_base[e] = s_exp_cnt[e] ? atomicAdd(&exp_cnt[parity * E + e], s_exp_cnt[e]) : 0;
  }
  // Position of every token of the block among the block's tokens that go to the same rank (does not
  // depend on other blocks, so it is done before the grid barrier).
  for (unsigned d = tid; d < unsigned(P); d += nthr) {
    int running = 0;
    for (int i = 0; i < t1 - t0; ++i) {
      s_rank_in_block[i * P + d] = running;
      running += static_cast<int>((s_mask[i] >> d) & 1ull);
    }
    s_blk_base[d] = 0;
    s_total[d] = 0;
  }
  if (stamp) phase_ns[1] = detail::now_ns();
  if (!grid_barrier(grid_counter, ++round, B)) return;
  if (stamp) phase_ns[2] = detail::now_ns();

  // ---- B: offsets and count exchange -------------------------------------------------------------------
  // All (block, rank) counts are read in one round of independent loads.
  for (unsigned i = tid; i < B * unsigned(P); i += nthr) {
    const int c = blk_cnt[i];
    if (c) {
      const unsigned bb = i / P, d = i % P;
      atomicAdd(&s_total[d], c);
      if (bb < b) atomicAdd(&s_blk_base[d], c);
    }
  }
  __syncthreads();
  if (b == 0) {
    // Row `me` of the count matrix goes to everybody; expert counts go to the expert's owner.
    for (unsigned i = tid; i < unsigned(P * P); i += nthr) {
      const int j = i / P, d = i % P;
      detail::st_relaxed_sys(remote_ptr(cnt_in + me * P + d, team_pe_to_world(t, j)), pack(epoch, s_total[d]));
    }
    for (unsigned e = tid; e < unsigned(E); e += nthr) {
      const int owner = e / epr;
      detail::st_relaxed_sys(remote_ptr(exp_in + me * epr + (e % epr), team_pe_to_world(t, owner)),
                             pack(epoch, static_cast<unsigned>(exp_cnt[parity * E + e])));
      exp_cnt[(parity ^ 1) * E + e] = 0;  // cleared for the next call
    }
  }
  const unsigned warp = tid / 32, lane = tid % 32, nwarps = nthr / 32;
  const int iters = H / 512;
  const int nscale = H / 128;
  constexpr int kBatch = 8;  // iterations (of 512 elements) whose loads are issued together
  if (STAGED) {
    // ---- one record per token (global expert ids, weights, pair positions) for whichever warp sends its rows ------
    for (int tok = t0 + warp; tok < t1; tok += nwarps) {
      if (s_mask[tok - t0] == 0) continue;
      int word = 0;
      if (lane < unsigned(K)) {
        word = topk_idx[size_t(tok) * K + lane];
      } else if (lane >= unsigned(EP_META_WEIGHT) && lane < unsigned(EP_META_WEIGHT + K)) {
        word = __float_as_int(topk_w[size_t(tok) * K + lane - EP_META_WEIGHT]);
      } else if (lane == unsigned(EP_META_SRC_TOKEN)) {
        word = tok;
      } else if (lane == unsigned(EP_META_SRC_RANK)) {
        word = me;
      } else if (lane >= unsigned(EP_META_RANK) && lane < unsigned(EP_META_RANK + K)) {
        const int k = lane - EP_META_RANK;
        const int e = topk_idx[size_t(tok) * K + k];
        word = (e >= 0 && e < E) ? s_exp_base[e] + s_pair_rank[(tok - t0) * K + k] : 0;
      }
      stage_meta[size_t(tok) * EP_META_WORDS + lane] = word;
    }
  }
  if (a.cfg.layout == EP_LAYOUT_SLOTTED) {
    for (unsigned d = tid; d < unsigned(P); d += nthr) s_base[d] = me * a.cfg.max_tokens;
  } else {
    // base[d] = rows that ranks before me send to d. Needs rows 0 .. me-1 of the matrix.
    bool ok = true;
    for (unsigned d = tid; d < unsigned(P); d += nthr) {
      int base = 0;
      for (int s = 0; s < me; ++s) base += static_cast<int>(wait_packed(cnt_in + s * P + d, epoch, s, &ok));
      s_base[d] = base;
    }
    if (!ok) atomicExch(&s_ok, 0);
  }
  __syncthreads();
  if (STAGED) {
    // A failed count wait must not leave the other blocks waiting at the second barrier for ever: every block
    // reaches it (its waits are bounded), and gives up afterwards.
    if (s_ok) {
      for (int i = tid; i < (t1 - t0) * P; i += nthr) {
        const int tk = i / P, d = i % P;
        const bool goes = (s_mask[tk] >> d) & 1ull;
        const int item = s_blk_base[d] + s_rank_in_block[tk * P + d];  // index among my rows for d
        sent_slot[size_t(t0 + tk) * P + d] = goes ? s_base[d] + item : -1;
        if (goes) item_tok[size_t(d) * a.cfg.max_tokens + item] = t0 + tk;
      }
    }
    if (!grid_barrier(grid_counter, ++round, B)) return;
  }
  if (!s_ok) return;
  if (stamp) phase_ns[3] = detail::now_ns();

  if (STAGED) {
    // ---- C (pairs): warps take (token, destination) pairs from per-destination counters ------------------------
    // Warps start on different destinations and move on when a destination's rows are all taken. A row is
    // quantised again for every destination it goes to (it comes from L2 after the first time): cheaper than a
    // staging pass during which the links would idle.
    const unsigned gwarp = b * nwarps + warp;
    for (int dd = 0; dd < P; ++dd) {
      const int d = (me + 1 + gwarp + dd) % P;
      const int w = team_pe_to_world(t, d);
      const unsigned long long total = static_cast<unsigned long long>(s_total[d]);
      if (total == 0) continue;
      unsigned long long *queue = work + parity * EP_MAX_RANKS + d;
      unsigned long long next = 0;
      if (lane == 0) next = atomicAdd(queue, 1ull);
      next = __shfl_sync(0xffffffffu, next, 0);
      while (next < total) {
        const int item = static_cast<int>(next);
        // The next item is claimed now, so that the counter's round trip overlaps this item's copies.
        unsigned long long after = 0;
        if (lane == 0) after = atomicAdd(queue, 1ull);
        const int tok = __ldcg(item_tok + size_t(d) * a.cfg.max_tokens + item);
        const int slot = s_base[d] + item;
        const int rec = __ldcg(stage_meta + size_t(tok) * EP_META_WORDS + lane);
        const int4 *row = reinterpret_cast<const int4 *>(x + size_t(tok) * H);
        if (a.cfg.quantize) {
          int4 *dst = reinterpret_cast<int4 *>(remote_ptr(recv_x + size_t(slot) * H, w));
          for (int i0 = 0; i0 < iters; i0 += kBatch) {
            int4 raw[2 * kBatch];
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
              if (i0 + i < iters) {
                raw[2 * i] = row[((i0 + i) * 512 + lane * 16) / 8];
                raw[2 * i + 1] = row[((i0 + i) * 512 + lane * 16) / 8 + 1];
              }
            }
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
              if (i0 + i < iters) {
                float scale;
                dst[(i0 + i) * 32 + lane] = quantize16(raw[2 * i], raw[2 * i + 1], &scale);
                if ((lane & 7) == 0) s_scales[warp][(i0 + i) * 4 + lane / 8] = scale;
              }
            }
          }
          __syncwarp();
          if (lane < unsigned(nscale / 4)) {
            reinterpret_cast<float4 *>(remote_ptr(recv_scales + size_t(slot) * nscale, w))[lane] =
                reinterpret_cast<const float4 *>(s_scales[warp])[lane];
          }
          __syncwarp();
        } else {
          copy_row_vec<8>(reinterpret_cast<int4 *>(remote_ptr(recv_x + size_t(slot) * H * 2, w)), row, H / 8, lane);
        }
        int word = rec;
        if (lane < unsigned(EP_MAX_TOPK)) word = (lane < unsigned(K) && rec >= 0 && rec / epr == d) ? rec % epr : -1;
        remote_ptr(recv_meta + size_t(slot) * EP_META_WORDS, w)[lane] = word;
        next = __shfl_sync(0xffffffffu, after, 0);
      }
    }
  } else {
  // ---- C (fixed shares): quantise and send, one warp per token ---------------------------------------------
  for (int tok = t0 + warp; tok < t1; tok += nwarps) {
    const unsigned long long mask = s_mask[tok - t0];
    // Lane d keeps the row index on destination d; everybody reads it with a shuffle.
    int my_slot = -1;
    if (lane < unsigned(P) && ((mask >> lane) & 1ull)) {
      my_slot = s_base[lane] + s_blk_base[lane] + s_rank_in_block[(tok - t0) * P + lane];
    }
    if (lane < unsigned(P)) sent_slot[size_t(tok) * P + lane] = my_slot;
    if (mask == 0) continue;
    const int4 *row = reinterpret_cast<const int4 *>(x + size_t(tok) * H);
    int k_idx = -1, k_rank = 0;
    float k_w = 0.f;
    if (lane < unsigned(K)) {
      k_idx = topk_idx[size_t(tok) * K + lane];
      k_w = topk_w[size_t(tok) * K + lane];
      if (k_idx >= 0 && k_idx < E) k_rank = s_exp_base[k_idx] + s_pair_rank[(tok - t0) * K + lane];
    }
    if (a.cfg.quantize) {
      for (int i0 = 0; i0 < iters; i0 += kBatch) {
        // All loads of the batch are in flight before the first value is used: one memory round
        // trip per 4096 elements instead of one per 512.
        int4 raw[2 * kBatch];
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
          if (i0 + i < iters) {
            // lane l holds elements [(i0+i)*512 + l*16, +16) = two int4
            raw[2 * i] = row[((i0 + i) * 512 + lane * 16) / 8];
            raw[2 * i + 1] = row[((i0 + i) * 512 + lane * 16) / 8 + 1];
          }
        }
        int4 q[kBatch];
#pragma unroll
        for (int i = 0; i < kBatch; ++i) {
          if (i0 + i < iters) {
            float scale;
            q[i] = quantize16(raw[2 * i], raw[2 * i + 1], &scale);
            if ((lane & 7) == 0) s_scales[warp][(i0 + i) * 4 + lane / 8] = scale;
          }
        }
        for (int dd = 0; dd < P; ++dd) {
          const int d = (me + dd) % P;  // rotate so the ranks do not all start on the same destination
          const int slot = __shfl_sync(0xffffffffu, my_slot, d);
          if (slot < 0) continue;
          int4 *dst = reinterpret_cast<int4 *>(remote_ptr(recv_x + size_t(slot) * H, team_pe_to_world(t, d)));
#pragma unroll
          for (int i = 0; i < kBatch; ++i) {
            if (i0 + i < iters) dst[(i0 + i) * 32 + lane] = q[i];
          }
        }
      }
      __syncwarp();
    }
    for (int dd = 0; dd < P; ++dd) {
      const int d = (me + dd) % P;
      const int slot = __shfl_sync(0xffffffffu, my_slot, d);
      if (slot < 0) continue;
      const int w = team_pe_to_world(t, d);
      if (a.cfg.quantize) {
        if (lane < unsigned(nscale / 4)) {
          float4 sc = reinterpret_cast<const float4 *>(s_scales[warp])[lane];
          reinterpret_cast<float4 *>(remote_ptr(recv_scales + size_t(slot) * nscale, w))[lane] = sc;
        }
      } else {
        copy_row_vec<4>(reinterpret_cast<int4 *>(remote_ptr(recv_x + size_t(slot) * H * 2, w)), row, H / 8, lane);
      }
      int *meta = remote_ptr(recv_meta + size_t(slot) * EP_META_WORDS, w);
      if (lane < unsigned(K)) {
        meta[EP_META_IDX + lane] = (k_idx >= 0 && k_idx / epr == d) ? k_idx % epr : -1;
        meta[EP_META_WEIGHT + lane] = __float_as_int(k_w);
        meta[EP_META_RANK + lane] = k_rank;
      } else if (lane == 16) {
        meta[EP_META_SRC_TOKEN] = tok;
      } else if (lane == 17) {
        meta[EP_META_SRC_RANK] = me;
      }
    }
    __syncwarp();
  }
  }

  // ---- D: completion ------------------------------------------------------------------------------------------
  if (stamp) phase_ns[4] = detail::now_ns();
  bool ok = block_pair_barrier(t, b);
  if (stamp) phase_ns[5] = detail::now_ns();
  if (b == 0 && ok) write_recv_info(a, t, recv_info, cnt_in, exp_in);
  if (a.cfg.expert_layout) {
    // ---- E: expert-grouped pair lists. Rows written by any block of a peer must be visible: every block of this
    // PE has passed its pair barrier once the grid barrier completes.
    if (!grid_barrier(grid_counter, ++round, B)) return;
    if (ok) build_expert_layout(a, t, cnt_in, exp_in, recv_meta, s_exp_cnt, s_exp_base, &s_lay_total, b, B);
  }
  __syncthreads();
  if (stamp) phase_ns[6] = detail::now_ns();
}

// ---- low-latency dispatch ------------------------------------------------------------------------------------------

constexpr unsigned kLlThreads = 128;

__global__ void __launch_bounds__(kLlThreads) ep_ll_dispatch_kernel(DispatchArgs a) {
  __shared__ int s_e[EP_MAX_TOPK];
  __shared__ int s_rank[EP_MAX_TOPK];
  __shared__ float s_w[EP_MAX_TOPK];
  __shared__ int s_slot[EP_MAX_RANKS];
  __shared__ __align__(16) float s_scales[EP_MAX_HIDDEN / 128];
  __shared__ int s_last;
  __shared__ int s_off[1024];
  __shared__ int s_src[1024];
  __shared__ int s_lay_total;

  const rocshmem_team_dev *t = detail::team_of(a.team);
  if (t->my_pe < 0) return;
  const int P = t->size, me = t->my_pe;
  const int E = a.cfg.num_experts, epr = E / P, K = a.cfg.top_k, H = a.cfg.hidden;
  const int T = a.num_tokens;
  const unsigned tid = threadIdx.x, nthr = blockDim.x;
  const unsigned warp = tid / 32, lane = tid % 32, nwarps = nthr / 32;
  const unsigned epoch = a.epoch;
  const int parity = epoch & 1;

  const __nv_bfloat16 *x = rebase(a.x);
  const int *topk_idx = rebase(a.topk_idx);
  const float *topk_w = rebase(a.topk_w);
  char *recv_x = static_cast<char *>(rebase(a.buf.recv_x));
  float *recv_scales = rebase(a.buf.recv_scales);
  int *recv_meta = rebase(a.buf.recv_meta);
  unsigned long long *cnt_in = rebase(a.buf.cnt_in) + size_t(parity) * P * P;
  unsigned long long *exp_in = rebase(a.buf.exp_in) + size_t(parity) * P * epr;
  int *sent_slot = rebase(a.buf.sent_slot);
  int *exp_cnt = rebase(a.buf.exp_cnt);  // [E] pairs per expert so far (first half of the array)
  int *recv_info = rebase(a.buf.recv_info);
  unsigned long long *work = rebase(a.buf.work_counter);
  unsigned long long *phase_ns = rebase(a.buf.phase_ns);
  if (blockIdx.x == 0 && tid == 0) phase_ns[0] = detail::now_ns();

  // Normally one token per block; the loop serves launches whose grid had to be capped.
  const int iters = H / 512, nscale = H / 128;
  constexpr int kWarps = kLlThreads / 32, kMine = (EP_MAX_HIDDEN / 512 + kWarps - 1) / kWarps;
  for (int tok = blockIdx.x; tok < T; tok += gridDim.x) {
    // The row does not depend on the routing: its loads are issued first and travel while the slots are taken.
    // The warps share the row: warp w takes the 512-element pieces w, w + 4, ...
    const int4 *row = reinterpret_cast<const int4 *>(x + size_t(tok) * H);
    int4 raw[2 * kMine];
    if (a.cfg.quantize) {
#pragma unroll
      for (int m = 0; m < kMine; ++m) {
        const int i = warp + m * kWarps;
        if (i < iters) {
          raw[2 * m] = row[(i * 512 + lane * 16) / 8];
          raw[2 * m + 1] = row[(i * 512 + lane * 16) / 8 + 1];
        }
      }
    }
    if (tid < unsigned(K)) {
      const int e = topk_idx[size_t(tok) * K + tid];
      const bool valid = e >= 0 && e < E;
      s_e[tid] = valid ? e : -1;
      s_w[tid] = topk_w[size_t(tok) * K + tid];
      s_rank[tid] = valid ? atomicAdd(&exp_cnt[e], 1) : 0;
    }
    __syncthreads();
    if (tid < unsigned(P)) {
      bool goes = false;
      for (int k = 0; k < K; ++k) goes = goes || (s_e[k] >= 0 && s_e[k] / epr == int(tid));
      int slot = -1;
      if (goes) {
        slot = me * a.cfg.max_tokens + static_cast<int>(atomicAdd(work + EP_WORK_LL_ROWS + tid, 1ull));
      }
      s_slot[tid] = slot;
      sent_slot[size_t(tok) * P + tid] = slot;
    }
    __syncthreads();
    if (a.cfg.quantize) {
#pragma unroll
      for (int m = 0; m < kMine; ++m) {
        const int i = warp + m * kWarps;
        if (i < iters) {
          float scale;
          const int4 q = quantize16(raw[2 * m], raw[2 * m + 1], &scale);
          if ((lane & 7) == 0) s_scales[i * 4 + lane / 8] = scale;
          for (int dd = 0; dd < P; ++dd) {
            const int d = (me + dd) % P;
            const int slot = s_slot[d];
            if (slot < 0) continue;
            reinterpret_cast<int4 *>(remote_ptr(recv_x + size_t(slot) * H, team_pe_to_world(t, d)))[i * 32 + lane] = q;
          }
        }
      }
      __syncthreads();
    }
    // Scales, record (and the bf16 row without quantisation): one destination per warp and step.
    for (int dd = warp; dd < P; dd += nwarps) {
      const int d = (me + dd) % P;
      const int slot = s_slot[d];
      if (slot < 0) continue;
      const int w = team_pe_to_world(t, d);
      if (a.cfg.quantize) {
        if (lane < unsigned(nscale / 4)) {
          reinterpret_cast<float4 *>(remote_ptr(recv_scales + size_t(slot) * nscale, w))[lane] =
              reinterpret_cast<const float4 *>(s_scales)[lane];
        }
      } else {
        copy_row_vec<8>(reinterpret_cast<int4 *>(remote_ptr(recv_x + size_t(slot) * H * 2, w)), row, H / 8, lane);
      }
      int word = 0;
      if (lane < unsigned(EP_MAX_TOPK)) {
        word = (lane < unsigned(K) && s_e[lane] >= 0 && s_e[lane] / epr == d) ? s_e[lane] % epr : -1;
      } else if (lane >= unsigned(EP_META_WEIGHT) && lane < unsigned(EP_META_WEIGHT + K)) {
        word = __float_as_int(s_w[lane - EP_META_WEIGHT]);
      } else if (lane == unsigned(EP_META_SRC_TOKEN)) {
        word = tok;
      } else if (lane == unsigned(EP_META_SRC_RANK)) {
        word = me;
      } else if (lane >= unsigned(EP_META_RANK) && lane < unsigned(EP_META_RANK + K)) {
        word = s_rank[lane - EP_META_RANK];
      }
      remote_ptr(recv_meta + size_t(slot) * EP_META_WORDS, w)[lane] = word;
    }
    __syncthreads();  // the shared tables are reused by the next token
  }

  // ---- completion: the last block to finish signals every destination, then collects the sources' signals ------
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();  // this block's rows, before the count
    const unsigned long long prev = atomicAdd(work + EP_WORK_LL_DONE, 1ull);
    s_last = (prev == gridDim.x - 1) ? 1 : 0;
    if (s_last) __threadfence_system();
  }
  __syncthreads();
  if (!s_last) return;
  if (tid == 0) phase_ns[4] = detail::now_ns();
  for (unsigned e = tid; e < unsigned(E); e += nthr) {
    const int owner = e / epr;
    const int c = __ldcg(exp_cnt + e);
    detail::st_relaxed_sys(remote_ptr(exp_in + me * epr + (e % epr), team_pe_to_world(t, owner)),
                           pack(epoch, static_cast<unsigned>(c)));
    exp_cnt[e] = 0;  // this block is the only one left: cleared for the next call
  }
  __syncthreads();
  if (tid < unsigned(P)) {
    const unsigned long long c = __ldcg(work + EP_WORK_LL_ROWS + tid);
    // Release: the rows of all blocks (ordered before this store through the done counter and the fences around
    // it) and the expert counts above are visible to whoever acquires the word.
    detail::st_release_sys(remote_ptr(cnt_in + me * P + tid, team_pe_to_world(t, tid)),
                           pack(epoch, static_cast<unsigned>(c)));
    work[EP_WORK_LL_ROWS + tid] = 0;
  }
  if (tid == 0) work[EP_WORK_LL_DONE] = 0;
  // Receive side: the signal of source s says how many rows it sent and that they have landed.
  bool ok = true;
  if (tid < unsigned(P)) {
    wait_packed(cnt_in + tid * P + me, epoch, tid, &ok);
    detail::fence_sys();  // acquire side of the sources' release stores
  }
  ok = __syncthreads_and(ok ? 1 : 0) != 0;
  if (tid == 0) phase_ns[5] = detail::now_ns();
  if (!ok) return;
  write_recv_info(a, t, recv_info, cnt_in, exp_in);
  if (a.cfg.expert_layout) build_expert_layout(a, t, cnt_in, exp_in, recv_meta, s_off, s_src, &s_lay_total, 0, 1);
  __syncthreads();
  if (tid == 0) phase_ns[6] = detail::now_ns();
}

struct CombineArgs {
  EpConfig cfg;
  EpBuffers buf;
  const __nv_bfloat16 *y;
  __nv_bfloat16 *out;
  const int *topk_idx;
  const float *topk_w;
  int num_tokens;
  int weighted;
  rocshmem_team_t team;
  unsigned long long work_base;  // dynamic mode: counter value at which this call's tokens start
  int split;                     // warps that share one token (1, 2 or 4), each taking a slice of the row
  int closing;                   // 0: no "done reading" barrier at the end (low-latency mode)
};

// Sums `n_src` rows (scaled by wgt) into dst. U vectors per source are loaded before any is used, so
// up to S * U 16-byte loads are in flight per lane.
template <int S, int U>
__device__ __forceinline__ void combine_row(int4 *dst, const int4 **src, const float *wgt, int n_src,
                                            int vbegin, int nvec, unsigned lane) {
  for (int v0 = vbegin + lane; v0 < nvec; v0 += 32 * U) {
    int4 raw[S][U];
#pragma unroll
    for (int s = 0; s < S; ++s) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (s < n_src && v0 + 32 * u < nvec) raw[s][u] = src[s][v0 + 32 * u];
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (v0 + 32 * u < nvec) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll
        for (int s = 0; s < S; ++s) {
          if (s < n_src) {
            const __nv_bfloat162 *p2 = reinterpret_cast<const __nv_bfloat162 *>(&raw[s][u]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = __bfloat1622float2(p2[i]);
              acc[2 * i] = fmaf(f.x, wgt[s], acc[2 * i]);
              acc[2 * i + 1] = fmaf(f.y, wgt[s], acc[2 * i + 1]);
            }
          }
        }
        int4 o;
        __nv_bfloat162 *o2 = reinterpret_cast<__nv_bfloat162 *>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        dst[v0 + 32 * u] = o;
      }
    }
  }
}

// DYNAMIC: warps take tokens from a device-wide counter (a token costs as many remote rows as it has sources, one
// to eight, so fixed shares differ a lot); the counter only grows, the host tells every call where it starts.
template <bool DYNAMIC>
__global__ void __launch_bounds__(kCombineThreads, 1) ep_combine_kernel(CombineArgs a) {
  __shared__ const int4 *s_src[kCombineThreads / 32][EP_MAX_TOPK];
  __shared__ float s_wgt[kCombineThreads / 32][EP_MAX_TOPK];
  const rocshmem_team_dev *t = detail::team_of(a.team);
  if (t->my_pe < 0) return;
  const int P = t->size;
  const int E = a.cfg.num_experts, epr = E / P, K = a.cfg.top_k, H = a.cfg.hidden;
  const __nv_bfloat16 *y = rebase(a.y);
  __nv_bfloat16 *out = rebase(a.out);
  const int *sent_slot = rebase(a.buf.sent_slot);
  const int *topk_idx = rebase(a.topk_idx);
  const float *topk_w = rebase(a.topk_w);

  unsigned long long *phase_ns = rebase(a.buf.phase_ns);
  const bool stamp = (blockIdx.x == 0 && threadIdx.x == 0);
  if (stamp) phase_ns[8] = detail::now_ns();
  // Every member's result rows are complete (its producers ran before this kernel on its stream).
  if (!block_pair_barrier(t, blockIdx.x)) return;
  if (stamp) phase_ns[9] = detail::now_ns();

  const unsigned lane = threadIdx.x % 32;
  const unsigned gwarp = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  const unsigned nwarps = gridDim.x * (blockDim.x / 32);
  const int nvec = H / 8;  // int4 vectors of 8 bf16 per row
  unsigned long long *work = DYNAMIC ? rebase(a.buf.work_counter) + EP_WORK_COMBINE : nullptr;
  const int split = DYNAMIC ? 1 : a.split;
  const int part = gwarp % split;
  const int vbegin = nvec / split * part, vend = nvec / split * (part + 1);
  // Dynamic: the counter is fetched one token ahead, so that its round trip overlaps the current token's loads.
  unsigned long long pending = 0;
  if (DYNAMIC && lane == 0) pending = atomicAdd(work, 1ull) - a.work_base;
  for (int tok_static = gwarp / split;; tok_static += nwarps / split) {
    int tok;
    if (DYNAMIC) {
      const unsigned long long next = __shfl_sync(0xffffffffu, pending, 0);
      if (next >= static_cast<unsigned long long>(a.num_tokens)) break;
      tok = static_cast<int>(next);
      if (lane == 0) pending = atomicAdd(work, 1ull) - a.work_base;
    } else {
      if (tok_static >= a.num_tokens) break;
      tok = tok_static;
    }
    // Lane d owns destination rank d: its row index there and the gate weight of that rank.
    // Lanes < K fetch one (expert, weight) pair each, so all small loads are issued at once.
    int my_slot = -1;
    if (lane < unsigned(P)) my_slot = sent_slot[size_t(tok) * P + lane];
    int k_e = -1;
    float k_w = 0.f;
    if (a.weighted && lane < unsigned(K)) {
      k_e = topk_idx[size_t(tok) * K + lane];
      k_w = topk_w[size_t(tok) * K + lane];
    }
    float my_w = 1.f;
    if (a.weighted) {
      my_w = 0.f;
      for (int k = 0; k < K; ++k) {
        const int e = __shfl_sync(0xffffffffu, k_e, k);
        const float w = __shfl_sync(0xffffffffu, k_w, k);
        if (e >= 0 && e / epr == int(lane)) my_w += w;
      }
    }
    const unsigned active = __ballot_sync(0xffffffffu, my_slot >= 0);
    // Source row pointers and weights live in shared memory (one set per warp): the registers are
    // needed for the loads in flight.
    const int4 **src = s_src[threadIdx.x / 32];
    float *wgt = s_wgt[threadIdx.x / 32];
    const int n_src = min(__popc(active), EP_MAX_TOPK);
    if (my_slot >= 0) {
      const int pos = __popc(active & ((1u << lane) - 1u));
      if (pos < EP_MAX_TOPK) {
        src[pos] = reinterpret_cast<const int4 *>(remote_ptr(y + size_t(my_slot) * H, team_pe_to_world(t, lane)));
        wgt[pos] = my_w;
      }
    }
    __syncwarp();
    int4 *dst = reinterpret_cast<int4 *>(out + size_t(tok) * H);
    if (n_src <= 4) {
      combine_row<4, 4>(dst, src, wgt, n_src, vbegin, vend, lane);
    } else {
      combine_row<8, 2>(dst, src, wgt, n_src, vbegin, vend, lane);
    }
    __syncwarp();
  }
  if (stamp) phase_ns[10] = detail::now_ns();
  // Nobody reuses its result rows while a peer may still be reading them. Nothing is handed over
  // here (the output rows are local), so the relaxed form suffices.
  if (a.closing) block_pair_barrier(t, blockIdx.x, false);
  if (stamp) phase_ns[11] = detail::now_ns();
}

// ---- stand-alone block-scaled fp8 helpers ----------------------------------------------------------------------

__global__ void __launch_bounds__(256) fp8_quantize_kernel(const __nv_bfloat16 *x, unsigned char *q, float *scales,
                                                           size_t rows, int hidden) {
  const unsigned lane = threadIdx.x % 32;
  const size_t gwarp = size_t(blockIdx.x) * (blockDim.x / 32) + threadIdx.x / 32;
  const size_t nwarps = size_t(gridDim.x) * (blockDim.x / 32);
  const int iters = hidden / 512, nscale = hidden / 128;
  for (size_t r = gwarp; r < rows; r += nwarps) {
    const int4 *row = reinterpret_cast<const int4 *>(x + r * hidden);
    int4 *dst = reinterpret_cast<int4 *>(q + r * hidden);
    for (int i = 0; i < iters; ++i) {
      const int4 lo = row[(i * 512 + lane * 16) / 8], hi = row[(i * 512 + lane * 16) / 8 + 1];
      float scale;
      dst[i * 32 + lane] = quantize16(lo, hi, &scale);
      if ((lane & 7) == 0) scales[r * nscale + i * 4 + lane / 8] = scale;
    }
  }
}

__global__ void __launch_bounds__(256) fp8_dequantize_kernel(const unsigned char *q, const float *scales,
                                                             __nv_bfloat16 *x, size_t rows, int hidden) {
  const size_t total = rows * size_t(hidden) / 16;  // 16 fp8 values per thread step
  const int nscale = hidden / 128;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const size_t elem = i * 16, r = elem / hidden, c = elem % hidden;
    const float scale = scales[r * nscale + c / 128];
    const int4 raw = reinterpret_cast<const int4 *>(q)[i];
    const unsigned short *p = reinterpret_cast<const unsigned short *>(&raw);
    int4 o[2];
    __nv_bfloat162 *o2 = reinterpret_cast<__nv_bfloat162 *>(o);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(p[k], __NV_E4M3);
      const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&h));
      o2[k] = __floats2bfloat162_rn(f.x * scale, f.y * scale);
    }
    reinterpret_cast<int4 *>(x)[2 * i] = o[0];
    reinterpret_cast<int4 *>(x)[2 * i + 1] = o[1];
  }
}

// ---- rows grouped by local expert ---------------------------------------------------------------------------------

__global__ void ep_expert_offsets_kernel(const int *recv_info_a, int n_ranks, int experts_per_rank, int *offsets_a,
                                         int *cursor_a) {
  const int *recv_info = rebase(recv_info_a);
  int *offsets = rebase(offsets_a), *cursor = rebase(cursor_a);
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < experts_per_rank; ++e) {
      offsets[e] = run;
      cursor[e] = 0;
      run += recv_info[1 + 2 * n_ranks + e];
    }
    offsets[experts_per_rank] = run;
  }
}

__global__ void ep_expert_layout_kernel(const int *recv_meta_a, const int *recv_info_a, int n_ranks, int top_k,
                                        const int *offsets_a, int *row_index_a, int *pair_k_a, int *cursor_a) {
  const int *recv_meta = rebase(recv_meta_a), *recv_info = rebase(recv_info_a), *offsets = rebase(offsets_a);
  int *row_index = rebase(row_index_a), *pair_k = rebase(pair_k_a), *cursor = rebase(cursor_a);
  for (int s = 0; s < n_ranks; ++s) {
    const int start = recv_info[1 + s], count = recv_info[1 + n_ranks + s];
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < count * top_k; i += gridDim.x * blockDim.x) {
      const int row = start + i / top_k, k = i % top_k;
      const int e = recv_meta[size_t(row) * EP_META_WORDS + EP_META_IDX + k];
      if (e >= 0) {
        const int pos = offsets[e] + atomicAdd(&cursor[e], 1);
        row_index[pos] = row;
        pair_k[pos] = k;
      }
    }
  }
}

int validate(const EpConfig &cfg, int team_size, int num_tokens) {
  return ep_config_error(cfg, team_size, num_tokens) ? cudaErrorInvalidValue : 0;
}

int ll_combine_blocks(const EpConfig &cfg) { return ep_ll_combine_blocks(cfg); }

}  // namespace

int ep_default_blocks() {
  Runtime &rt = Runtime::instance();
  // One block per SM (the kernels are written for one resident block of 512 threads per SM), shared
  // between the PEs of the process when it hosts several.
  int per_pe = device_sm_count() / std::max(1, rt.n_local());
  return std::max(1, std::min<int>(per_pe, ROCSHMEM_LIB_MAX_BLOCKS));
}

unsigned long long ep_combine_fetches(const EpConfig &cfg, int num_tokens) {
  return static_cast<unsigned long long>(num_tokens) + static_cast<unsigned long long>(cfg.blocks) * (kCombineThreads / 32);
}

int ep_dispatch(rocshmem_team_t team, const EpConfig &cfg, const EpBuffers &buf, const void *x,
                const int *topk_idx, const float *topk_w, int num_tokens, unsigned epoch, void *stream) {
  Runtime &rt = Runtime::instance();
  HostTeam *ht = rt.team_from_handle(team);
  if (!ht) return cudaErrorInvalidValue;
  if (int rc = validate(cfg, ht->world.size, num_tokens)) return rc;
  if (cfg.expert_layout && (!buf.lay_offsets || !buf.lay_row || !buf.lay_k || !buf.lay_w)) return cudaErrorInvalidValue;
  DispatchArgs a{cfg, buf, static_cast<const __nv_bfloat16 *>(x), topk_idx, topk_w, num_tokens, epoch, team};
  if (cfg.low_latency) {
    if (buf.work_counter == nullptr) return cudaErrorInvalidValue;
    // A block per token; with several PEs per process the launch is cooperative and must fit the GPU at once.
    unsigned blocks = static_cast<unsigned>(std::max(1, std::min(num_tokens, 4096)));
    if (rt.n_local() > 1) {
      blocks = std::min(blocks, coresident_blocks_per_pe(ep_ll_dispatch_kernel, kLlThreads, 0, rt.n_local()));
    }
    return launch_pes(ep_ll_dispatch_kernel, blocks, kLlThreads, 0, static_cast<cudaStream_t>(stream), false, a);
  }
  const int tpb = (cfg.max_tokens + cfg.blocks - 1) / cfg.blocks;
  const size_t smem = size_t(tpb) * ((ht->world.size + cfg.top_k) * sizeof(int) + sizeof(unsigned long long));
  if (smem > 40 * 1024) return cudaErrorInvalidValue;  // use more blocks for this many tokens
  if (cfg.dynamic) {
    if (!buf.work_counter || !buf.stage_meta || !buf.item_tok) return cudaErrorInvalidValue;
    return launch_pes(ep_dispatch_kernel<true>, cfg.blocks, kEpThreads, smem, static_cast<cudaStream_t>(stream), true,
                      a);
  }
  return launch_pes(ep_dispatch_kernel<false>, cfg.blocks, kEpThreads, smem, static_cast<cudaStream_t>(stream), true,
                    a);
}

int ep_combine(rocshmem_team_t team, const EpConfig &cfg, const EpBuffers &buf, const void *y, void *out,
               const int *topk_idx, const float *topk_w, int num_tokens, int weighted, void *stream,
               unsigned long long combine_calls_base) {
  Runtime &rt = Runtime::instance();
  HostTeam *ht = rt.team_from_handle(team);
  if (!ht) return cudaErrorInvalidValue;
  if (int rc = validate(cfg, ht->world.size, num_tokens)) return rc;
  CombineArgs a{cfg, buf, static_cast<const __nv_bfloat16 *>(y), static_cast<__nv_bfloat16 *>(out), topk_idx,
                topk_w, num_tokens, weighted, team, combine_calls_base, 1, 1};
  if (cfg.low_latency) {
    // Four warps per token, one token per block of 128 threads, no closing barrier.
    a.split = (cfg.hidden / 8) % 4 == 0 ? 4 : 1;
    a.closing = 0;
    unsigned blocks = static_cast<unsigned>(ll_combine_blocks(cfg));
    if (rt.n_local() > 1) {
      blocks = std::min(blocks, coresident_blocks_per_pe(ep_combine_kernel<false>, kLlThreads, 0, rt.n_local()));
    }
    return launch_pes(ep_combine_kernel<false>, blocks, kLlThreads, 0, static_cast<cudaStream_t>(stream), false, a);
  }
  if (cfg.dynamic) {
    if (buf.work_counter == nullptr) return cudaErrorInvalidValue;
    return launch_pes(ep_combine_kernel<true>, cfg.blocks, kCombineThreads, 0, static_cast<cudaStream_t>(stream), false,
                      a);
  }
  return launch_pes(ep_combine_kernel<false>, cfg.blocks, kCombineThreads, 0, static_cast<cudaStream_t>(stream), false,
                    a);
}

int fp8_quantize_1x128(const void *x, void *q, float *scales, size_t rows, int hidden, void *stream) {
  if (hidden % 512 || hidden <= 0) return cudaErrorInvalidValue;
  if (rows == 0) return 0;
  unsigned blocks = static_cast<unsigned>(std::min<size_t>((rows + 7) / 8, size_t(device_sm_count()) * 8));
  fp8_quantize_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16 *>(x), static_cast<unsigned char *>(q), scales, rows, hidden);
  return cudaGetLastError();
}

int fp8_dequantize_1x128(const void *q, const float *scales, void *x, size_t rows, int hidden, void *stream) {
  if (hidden % 128 || hidden <= 0) return cudaErrorInvalidValue;
  if (rows == 0) return 0;
  size_t steps = rows * size_t(hidden) / 16;
  unsigned blocks = static_cast<unsigned>(std::min<size_t>((steps + 255) / 256, size_t(device_sm_count()) * 8));
  fp8_dequantize_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned char *>(q), scales, static_cast<__nv_bfloat16 *>(x), rows, hidden);
  return cudaGetLastError();
}

int ep_expert_layout(const int *recv_meta, const int *recv_info, int n_ranks, int max_tokens, int layout,
                     int experts_per_rank, int top_k, int *offsets, int *row_index, int *pair_k,
                     int *cursor_scratch, void *stream_v) {
  (void)max_tokens;
  (void)layout;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (int rc = launch_pes(ep_expert_offsets_kernel, 1, 32, 0, stream, false, recv_info, n_ranks, experts_per_rank,
                          offsets, cursor_scratch)) {
    return rc;
  }
  Runtime &rt = Runtime::instance();
  unsigned blocks = static_cast<unsigned>(std::max(1, device_sm_count() / std::max(1, rt.n_local())));
  return launch_pes(ep_expert_layout_kernel, blocks, 256, 0, stream, false, recv_meta, recv_info, n_ranks, top_k,
                    static_cast<const int *>(offsets), row_index, pair_k, cursor_scratch);
}

}  // namespace kernels
}  // namespace rocshmem

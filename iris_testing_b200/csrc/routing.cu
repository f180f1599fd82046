// Routing kernels: softmax -> top-k router, and the dispatch plan (per-expert
// histogram, stable rank of every routed copy inside its expert bucket, packed
// send order, and the push of this rank's counts to every peer).
//
// Counterparts in the reference project: the router math of utils.py:201-202,
// the Python bucket/pack loop of utils.py:204-246, the offset builders of
// utils.py:20-31 and benchmark.py:44-49, and the counts exchange kernel of
// kernels.py:21-66 (folded into plan_finalize_kernel).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <atomic>

#include "moe_args.h"
#include "sm100_ptx.cuh"
#include "topk.cuh"

namespace b200 {

// Generic CUDA-core router: one warp per token.  logits = x[t,:] . Wr[:, e] (+ bias[e]);
// probabilities = softmax over experts; outputs the top-k (index, probability).
// Wr is [D, E] row-major as in the reference.  Used for shapes the tensor-core
// router cannot take; O(T*D*E) loads from L2.
__global__ void router_topk_simple_kernel(const __nv_bfloat16* __restrict__ x,
                                          const __nv_bfloat16* __restrict__ wr,
                                          const float* __restrict__ bias, int T, int D, int E, int k,
                                          int renorm, int* __restrict__ topk_idx,
                                          float* __restrict__ topk_w, float* __restrict__ logits_out) {
  extern __shared__ float sm_logits[];   // [warps][E]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  float* lg = sm_logits + warp * E;
  for (int t = blockIdx.x * warps + warp; t < T; t += gridDim.x * warps) {
    const __nv_bfloat16* xr = x + static_cast<size_t>(t) * D;
    for (int e0 = 0; e0 < E; e0 += 8) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int d = lane; d < D; d += 32) {
        const float xv = __bfloat162float(xr[d]);
        const __nv_bfloat16* wrow = wr + static_cast<size_t>(d) * E + e0;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (e0 + j < E) acc[j] += xv * __bfloat162float(wrow[j]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float a = acc[j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (lane == 0 && e0 + j < E) lg[e0 + j] = a + (bias ? bias[e0 + j] : 0.f);
      }
    }
    __syncwarp();
    // softmax statistics
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, lg[e]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += __expf(lg[e] - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (logits_out) for (int e = lane; e < E; e += 32) logits_out[static_cast<size_t>(t) * E + e] = lg[e];
    // top-k: lane-local candidates, then a k-round warp argmax merge
    TopK tk; tk.init();
    for (int e = lane; e < E; e += 32) tk.push(lg[e], e);
    float wsum = 0.f;
    float my_w = 0.f; int my_i = 0;
    for (int r = 0; r < k; ++r) {
      float bv = tk.v[0]; int bi = tk.i[0] < 0 ? 0x7fffffff : tk.i[0];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (tk.i[0] == bi) {   // the winning lane pops its head
#pragma unroll
        for (int j = 0; j < ROUTER_MAX_K - 1; ++j) { tk.v[j] = tk.v[j + 1]; tk.i[j] = tk.i[j + 1]; }
        tk.v[ROUTER_MAX_K - 1] = -INFINITY; tk.i[ROUTER_MAX_K - 1] = -1;
      }
      const float p = __expf(bv - mx) / sum;
      wsum += p;
      if (lane == r) { my_w = p; my_i = bi; }
    }
    if (lane < k) {
      topk_idx[static_cast<size_t>(t) * k + lane] = my_i;
      topk_w[static_cast<size_t>(t) * k + lane] = renorm ? my_w / wsum : my_w;
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------
// Plan, step 1: one CTA per expert walks the flat (token, slot) list in order
// and gives every copy routed to that expert its stable rank in the bucket.
// ---------------------------------------------------------------------------
__global__ void plan_rank_kernel(const int* __restrict__ topk_idx, int n_flat, int num_experts,
                                 int* __restrict__ rank_in_bucket, int* __restrict__ counts) {
  // Each warp owns one contiguous segment of the list: pass 1 counts its hits, a scan over
  // the warp totals gives every segment its base rank, pass 2 hands out the ranks.  Only
  // two block-wide barriers, whatever the list length.
  __shared__ int warp_base[33];
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int seg = ((n_flat + nwarps - 1) / nwarps + 31) & ~31;
  const int lo = min(warp * seg, n_flat), hi = min(lo + seg, n_flat);
  int cnt = 0;
  for (int i = lo + lane; i < hi; i += 32) cnt += (topk_idx[i] == e) ? 1 : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if (lane == 0) warp_base[warp + 1] = cnt;
  __syncthreads();
  if (warp == 0) {
    int v = (lane < nwarps) ? warp_base[lane + 1] : 0;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane < nwarps) warp_base[lane + 1] = incl;   // inclusive: base of warp w is warp_base[w]
    if (lane == 0) warp_base[0] = 0;
  }
  __syncthreads();
  int running = warp_base[warp];
  for (int base = lo; base < hi; base += 32) {
    const int i = base + lane;
    const bool hit = (i < hi) && (topk_idx[i] == e);
    const unsigned b = __ballot_sync(0xffffffffu, hit);
    if (hit) rank_in_bucket[i] = running + __popc(b & ((1u << lane) - 1u));
    running += __popc(b);
  }
  if (threadIdx.x == 0) counts[e] = warp_base[nwarps];
  (void)num_experts;
}

// ---------------------------------------------------------------------------
// Plan, step 2: bucket offsets (exclusive scan over experts), the packed send
// order, and -- when `peer_counts` is given -- the push of this rank's counts
// row to every rank followed by an epoch-stamped flag.  Before touching a
// peer's tables the kernel checks that the peer has retired the iteration that
// last used the same parity slot.
// ---------------------------------------------------------------------------
struct PlanPushArgs {
  int world, rank;
  uint32_t epoch;                 // stamp to publish (iteration + 1)
  uint32_t need_iter_done;        // every peer's iter_done must be >= this
  const uint32_t* iter_done;      // [world] local: iterations retired by each peer
  unsigned long long peer_counts[B200_MAX_WORLD];  // int [world][E_total] table on each rank
  unsigned long long peer_flags[B200_MAX_WORLD];   // uint32 [world] flags on each rank
  int* status;
  unsigned long long wait_budget_ns;
  // Device-side iteration state: when iter_ptr is set, it = *iter_ptr replaces the two
  // stamps above (epoch = it + 1, need = max(it - 1, 0)) and the peer tables above name
  // parity 0; (it & 1) * stride selects the copy in use.
  const uint32_t* iter_ptr;
  unsigned long long stride_counts;
  unsigned long long stride_flags;
};

__global__ void plan_finalize_kernel(const int* __restrict__ topk_idx,
                                     const int* __restrict__ rank_in_bucket,
                                     const int* __restrict__ counts, int n_flat, int num_experts,
                                     int* __restrict__ bucket_start, int* __restrict__ send_order,
                                     int* __restrict__ dst_slot, PlanPushArgs push, int do_push) {
  __shared__ int s_start[B200_MAX_EXPERTS + 1];
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < num_experts; ++e) { s_start[e] = acc; acc += counts[e]; }
    s_start[num_experts] = acc;
    s_abort = 0;
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    for (int e = threadIdx.x; e <= num_experts; e += blockDim.x) bucket_start[e] = s_start[e];
    if (do_push) {
      uint32_t epoch = push.epoch, need = push.need_iter_done;
      unsigned long long off_counts = 0, off_flags = 0;
      if (push.iter_ptr != nullptr) {
        const uint32_t it = __ldcg(push.iter_ptr);
        epoch = it + 1u;
        need = it > 0u ? it - 1u : 0u;
        if (it & 1u) { off_counts = push.stride_counts; off_flags = push.stride_flags; }
      }
      WaitCtx w; w.abort_flag = &s_abort; w.status = push.status; w.budget_ns = push.wait_budget_ns;
      if (threadIdx.x < push.world)
        wait_flag_geq(push.iter_done + threadIdx.x, need, w, ST_TIMEOUT_ITER);
      __syncthreads();
      for (int p = 0; p < push.world; ++p) {
        int* dst = reinterpret_cast<int*>(push.peer_counts[p] + off_counts) + push.rank * num_experts;
        for (int e = threadIdx.x; e < num_experts; e += blockDim.x) dst[e] = counts[e];
      }
      __syncthreads();
      if (threadIdx.x < push.world) {
        fence_acq_rel_sys();
        st_release_sys(reinterpret_cast<uint32_t*>(push.peer_flags[threadIdx.x] + off_flags) + push.rank,
                       epoch);
      }
    }
  }
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_flat; i += gridDim.x * blockDim.x) {
    const int e = topk_idx[i];
    if (e < 0 || e >= num_experts) continue;
    const int pos = s_start[e] + rank_in_bucket[i];
    send_order[pos] = i;
    if (dst_slot) dst_slot[i] = pos;
  }
}

// ---------------------------------------------------------------------------
// Small-token path: router AND plan in ONE launch (instead of three launches).
// For a few thousand routed copies the layer is launch- and latency-bound, and the router GEMM on
// tensor cores (TMEM allocation, barriers, 148 CTAs) costs more than the arithmetic.  Here one to
// eight warps per token form the logits with 16-byte loads from the K-major router weights (the
// tokens spread over up to 148 CTAs, so that the cold loads of a wide hidden dimension run in
// parallel), the same softmax / top-k code picks the experts, and the CTA that
// finishes LAST (a ticket in global memory; nobody waits) builds the plan in shared memory
// (stable ranks per expert by ballot, scan, send order) and pushes the counts to the peers.
// Limits (checked by the launcher): n_flat <= SMALL_MAX_FLAT, experts <= B200_MAX_EXPERTS.
// ---------------------------------------------------------------------------
constexpr int SMALL_MAX_FLAT = 4096;
constexpr int SMALL_THREADS = 256;
constexpr int SMALL_EG = 8;            // experts per pass over a token's row

__global__ void __launch_bounds__(SMALL_THREADS)
route_plan_small_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wr_kmajor,
                        const float* __restrict__ bias, int T, int D, int E, int k, int renorm,
                        int* __restrict__ topk_idx, float* __restrict__ topk_w, int* __restrict__ counts,
                        int* __restrict__ bucket_start, int* __restrict__ send_order,
                        int* __restrict__ dst_slot, PlanPushArgs push, int do_push, unsigned int* ticket,
                        int wpt) {
  __shared__ float s_lg[SMALL_THREADS / 32][B200_MAX_EXPERTS];
  __shared__ short s_idx[SMALL_MAX_FLAT];
  __shared__ short s_rank[SMALL_MAX_FLAT];
  __shared__ int s_cnt[B200_MAX_EXPERTS];
  __shared__ int s_start[B200_MAX_EXPERTS + 1];
  __shared__ int s_abort;
  __shared__ int s_last;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
  const int n_flat = T * k;
  if (tid == 0) s_abort = 0;
  // ---- router: `wpt` warps per token (a power of two up to the warps of the CTA; the host picks
  // it so that a small batch still fills the SMs).  Each warp of a token takes every wpt-th group
  // of 32 sixteen-byte pieces of the row, the partial logits meet in shared memory and the
  // token's first warp does softmax and top-k.
  const int d16 = D / 8;
  const int tpc = nwarps / wpt;                       // tokens per CTA and pass
  const int sub = warp % wpt, slot = warp / wpt;
  for (int base = blockIdx.x * tpc; base < T; base += gridDim.x * tpc) {   // uniform per CTA
    const int t = base + slot;
    const bool tv = t < T;
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(tv ? t : 0) * D);
    // Experts in groups of eight with independent accumulators, two 16-byte pieces of the row per
    // trip: 18 (cold) loads are in flight together instead of one dependent pair at a time.
    for (int e0 = 0; e0 < E; e0 += SMALL_EG) {
      float acc[SMALL_EG];
#pragma unroll
      for (int j = 0; j < SMALL_EG; ++j) acc[j] = 0.f;
      if (tv) {
#pragma unroll 2
        for (int i = lane + 32 * sub; i < d16; i += 32 * wpt) {
          const uint4 xv = __ldg(xr + i);
          uint4 wv[SMALL_EG];
#pragma unroll
          for (int j = 0; j < SMALL_EG; ++j)
            wv[j] = __ldg(reinterpret_cast<const uint4*>(wr_kmajor + static_cast<size_t>(min(e0 + j, E - 1)) * D) + i);
          const __nv_bfloat162* xa = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
          for (int j = 0; j < SMALL_EG; ++j) {
            const __nv_bfloat162* wa = reinterpret_cast<const __nv_bfloat162*>(&wv[j]);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 a = __bfloat1622float2(xa[q]), b = __bfloat1622float2(wa[q]);
              acc[j] = fmaf(a.x, b.x, acc[j]);
              acc[j] = fmaf(a.y, b.y, acc[j]);
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < SMALL_EG; ++j) {
        float a = acc[j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        if (lane == 0 && e0 + j < E) s_lg[warp][e0 + j] = a;
      }
    }
    __syncthreads();                                  // every warp's partial logits are in place
    if (tv && sub == 0) {
      float* lg = s_lg[warp];
      for (int e = lane; e < E; e += 32) {
        float v = bias ? bias[e] : 0.f;
        for (int s2 = 0; s2 < wpt; ++s2) v += s_lg[warp + s2][e];
        lg[e] = v;
      }
      __syncwarp();
      float mx = -INFINITY;
      for (int e = lane; e < E; e += 32) mx = fmaxf(mx, lg[e]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      float sum = 0.f;
      for (int e = lane; e < E; e += 32) sum += __expf(lg[e] - mx);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      TopK tk; tk.init();
      for (int e = lane; e < E; e += 32) tk.push(lg[e], e);
      float wsum = 0.f, my_w = 0.f;
      int my_i = 0;
      for (int r = 0; r < k; ++r) {
        float bv = tk.v[0]; int bi = tk.i[0] < 0 ? 0x7fffffff : tk.i[0];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
          const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
          if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (tk.i[0] == bi) {   // the winning lane pops its head
#pragma unroll
          for (int j = 0; j < ROUTER_MAX_K - 1; ++j) { tk.v[j] = tk.v[j + 1]; tk.i[j] = tk.i[j + 1]; }
          tk.v[ROUTER_MAX_K - 1] = -INFINITY; tk.i[ROUTER_MAX_K - 1] = -1;
        }
        const float p = __expf(bv - mx) / sum;
        wsum += p;
        if (lane == r) { my_w = p; my_i = bi; }
      }
      if (lane < k) {
        topk_idx[static_cast<size_t>(t) * k + lane] = my_i;
        topk_w[static_cast<size_t>(t) * k + lane] = renorm ? my_w / wsum : my_w;
      }
    }
    __syncthreads();                                  // the partial-logit rows are reused by the next pass
  }
  // ---- hand-over: every CTA publishes its choices and takes a ticket; the last one plans
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const unsigned int prev = atomicAdd(ticket, 1u);
    s_last = prev == gridDim.x - 1u;
    if (s_last) *ticket = 0u;          // re-armed for the next launch on this stream
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int i = tid; i < n_flat; i += blockDim.x) {
    const int e = __ldcg(topk_idx + i);
    s_idx[i] = static_cast<short>(min(max(e, 0), E - 1));
  }
  __syncthreads();
  // ---- plan: stable rank of every routed copy inside its expert bucket
  for (int e = warp; e < E; e += nwarps) {
    int running = 0;
    for (int base = 0; base < n_flat; base += 32) {
      const int i = base + lane;
      const bool hit = i < n_flat && s_idx[i] == e;
      const unsigned b = __ballot_sync(0xffffffffu, hit);
      if (hit) s_rank[i] = static_cast<short>(running + __popc(b & ((1u << lane) - 1u)));
      running += __popc(b);
    }
    if (lane == 0) s_cnt[e] = running;
  }
  __syncthreads();
  if (tid == 0) {
    int acc = 0;
    for (int e = 0; e < E; ++e) { s_start[e] = acc; acc += s_cnt[e]; }
    s_start[E] = acc;
  }
  __syncthreads();
  for (int e = tid; e <= E; e += blockDim.x) {
    bucket_start[e] = s_start[e];
    if (e < E) counts[e] = s_cnt[e];
  }
  for (int i = tid; i < n_flat; i += blockDim.x) {
    const int pos = s_start[s_idx[i]] + s_rank[i];
    send_order[pos] = i;
    if (dst_slot) dst_slot[i] = pos;
  }
  if (do_push) {     // same protocol as plan_finalize_kernel
    uint32_t epoch = push.epoch, need = push.need_iter_done;
    unsigned long long off_counts = 0, off_flags = 0;
    if (push.iter_ptr != nullptr) {
      const uint32_t it = __ldcg(push.iter_ptr);
      epoch = it + 1u;
      need = it > 0u ? it - 1u : 0u;
      if (it & 1u) { off_counts = push.stride_counts; off_flags = push.stride_flags; }
    }
    WaitCtx w; w.abort_flag = &s_abort; w.status = push.status; w.budget_ns = push.wait_budget_ns;
    if (tid < push.world) wait_flag_geq(push.iter_done + tid, need, w, ST_TIMEOUT_ITER);
    __syncthreads();
    for (int p = 0; p < push.world; ++p) {
      int* dst = reinterpret_cast<int*>(push.peer_counts[p] + off_counts) + push.rank * E;
      for (int e = tid; e < E; e += blockDim.x) dst[e] = s_cnt[e];
    }
    __syncthreads();
    if (tid < push.world) {
      fence_acq_rel_sys();
      st_release_sys(reinterpret_cast<uint32_t*>(push.peer_flags[tid] + off_flags) + push.rank, epoch);
    }
  }
}

// ---------------------------------------------------------------------------
// Capacity of a padded exchange, computed on the device across all ranks (no host round
// trip).  Every rank pushes its send_counts row ([dst][e]) into slot [rank] of a table on
// every peer and stamps a flag with the epoch; once all flags show the epoch, each rank
// reduces the full [src][dst][e] table to
//   out[0] = CAP: the largest (src, dst, expert) cell -- the rule of utils.py:118-121,
//   out[1] = M:   the most rows any rank sends to any one rank -- the fixed message size of
//                 README.md:5-7 (every pair sends M rows, zero padded),
//   out[2] = the most rows any rank receives (what a receive buffer must hold),
//   out[3] = the rows this rank receives.
// Tables and flags are double-buffered by epoch parity: a rank can be at most one epoch
// ahead of the slowest reader (it cannot finish an epoch before everyone has pushed it).
// ---------------------------------------------------------------------------
struct CapacityArgs {
  int world, rank, e_local;
  uint32_t epoch;
  unsigned long long peer_table[B200_MAX_WORLD];   // int [2][world][world * e_local] on each rank
  unsigned long long peer_flags[B200_MAX_WORLD];   // uint32 [2][world] on each rank
  int* status;
  unsigned long long budget_ns;
};

__global__ void capacity_kernel(const int* __restrict__ send_counts, CapacityArgs a, int* __restrict__ out) {
  __shared__ int s_abort;
  __shared__ int s_red[4];
  const int W = a.world, EL = a.e_local, ET = W * EL, tid = threadIdx.x;
  const unsigned par = a.epoch & 1u;
  if (tid == 0) { s_abort = 0; s_red[0] = s_red[1] = s_red[2] = s_red[3] = 0; }
  __syncthreads();
  for (int p = 0; p < W; ++p) {
    int* row = reinterpret_cast<int*>(a.peer_table[p]) + (static_cast<size_t>(par) * W + a.rank) * ET;
    for (int i = tid; i < ET; i += blockDim.x) row[i] = send_counts[i];
  }
  __syncthreads();
  WaitCtx w; w.abort_flag = &s_abort; w.status = a.status; w.budget_ns = a.budget_ns;
  if (tid < W) {
    fence_acq_rel_sys();
    st_release_sys(reinterpret_cast<uint32_t*>(a.peer_flags[tid]) + par * W + a.rank, a.epoch);
    wait_flag_geq(reinterpret_cast<const uint32_t*>(a.peer_flags[a.rank]) + par * W + tid, a.epoch, w,
                  ST_TIMEOUT_COUNTS);
  }
  __syncthreads();
  if (s_abort) return;
  const int* tab = reinterpret_cast<const int*>(a.peer_table[a.rank]) + static_cast<size_t>(par) * W * ET;
  // one thread per (src, dst) pair
  for (int pr = tid; pr < W * W; pr += blockDim.x) {
    const int src = pr / W, dst = pr - src * W;
    int cell = 0, pair = 0;
    for (int e = 0; e < EL; ++e) {
      const int c = __ldcg(tab + (src * W + dst) * EL + e);
      cell = max(cell, c);
      pair += c;
    }
    atomicMax(&s_red[0], cell);
    atomicMax(&s_red[1], pair);
  }
  __syncthreads();
  for (int dst = tid; dst < W; dst += blockDim.x) {
    int recv = 0;
    for (int src = 0; src < W; ++src)
      for (int e = 0; e < EL; ++e) recv += __ldcg(tab + (src * W + dst) * EL + e);
    atomicMax(&s_red[2], recv);
    if (dst == a.rank) s_red[3] = recv;
  }
  __syncthreads();
  if (tid < 4) out[tid] = s_red[tid];
}

// Gathers the packed send payload: payload[j, :] = x[send_order[j] / topk, :].
__global__ void pack_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ send_order,
                                 int n_flat, int topk, int row16, uint4* __restrict__ payload) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int j = warp; j < n_flat; j += nwarps) {
    const int t = send_order[j] / topk;
    const uint4* src = x + static_cast<size_t>(t) * row16;
    uint4* dst = payload + static_cast<size_t>(j) * row16;
    for (int i = lane; i < row16; i += 32) dst[i] = ld_nc_16(src + i);
  }
}

}  // namespace b200

extern "C" {

int b200_router_topk_simple(const void* x, const void* wr, const float* bias, int T, int D, int E,
                            int k, int renorm, int* topk_idx, float* topk_w, float* logits_out,
                            void* stream) {
  if (k < 1 || k > b200::ROUTER_MAX_K || k > E || E > 1024) return -1;
  if (T == 0) return 0;
  const int warps = 4;
  const int blocks = (T + warps - 1) / warps;
  b200::router_topk_simple_kernel<<<blocks < 65535 * 8 ? blocks : 65535 * 8, warps * 32,
                                    warps * E * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(wr), bias, T, D, E, k,
      renorm, topk_idx, topk_w, logits_out);
  b200_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

// topk_idx [n_flat] -> rank_in_bucket [n_flat], counts [E], bucket_start [E+1],
// send_order [n_flat], dst_slot [n_flat] (optional).  `push` may be null.
int b200_plan(const int* topk_idx, int n_flat, int num_experts, int* rank_in_bucket, int* counts,
              int* bucket_start, int* send_order, int* dst_slot, const b200::PlanPushArgs* push,
              void* stream) {
  if (num_experts < 1 || num_experts > B200_MAX_EXPERTS) return -1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  b200::plan_rank_kernel<<<num_experts, 1024, 0, st>>>(topk_idx, n_flat, num_experts, rank_in_bucket,
                                                       counts);
  b200_count_launches(1);
  b200::PlanPushArgs pz;
  memset(&pz, 0, sizeof(pz));
  int blocks = (n_flat + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 1184) blocks = 1184;
  b200::plan_finalize_kernel<<<blocks, 256, 0, st>>>(topk_idx, rank_in_bucket, counts, n_flat,
                                                     num_experts, bucket_start, send_order, dst_slot,
                                                     push ? *push : pz, push ? 1 : 0);
  b200_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

int b200_pack_rows(const void* x, const int* send_order, int n_flat, int topk, int hidden_dim,
                   void* payload, void* stream) {
  if (hidden_dim % 8 != 0) return -1;
  if (n_flat == 0) return 0;
  int blocks = (n_flat + 7) / 8;
  if (blocks > 148 * 8) blocks = 148 * 8;
  b200::pack_rows_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), send_order, n_flat, topk, hidden_dim / 8,
      static_cast<uint4*>(payload));
  b200_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"

// Router + plan of a small batch in one launch (see route_plan_small_kernel).  wr_kmajor is the
// router matrix as [E, D]; outputs as b200_router_topk_simple + b200_plan.  `ticket` is one zeroed
// word of device memory owned by the caller (launches that may overlap need separate words); the
// kernel leaves it zero.  Returns -2 when the batch is too large for this path.
extern "C" int b200_route_plan_small(const void* x, const void* wr_kmajor, const float* bias, int T, int D,
                                     int E, int k, int renorm, int* topk_idx, float* topk_w, int* counts,
                                     int* bucket_start, int* send_order, int* dst_slot,
                                     const b200::PlanPushArgs* push, unsigned int* ticket, void* stream) {
  if (k < 1 || k > b200::ROUTER_MAX_K || k > E || E < 1 || E > B200_MAX_EXPERTS || D % 8 != 0 || T < 0 ||
      ticket == nullptr)
    return -1;
  if (static_cast<long long>(T) * k > b200::SMALL_MAX_FLAT) return -2;
  b200::PlanPushArgs pz;
  memset(&pz, 0, sizeof(pz));
  const int warps = b200::SMALL_THREADS / 32;
  // warps per token: as many as still leave every token of the batch a place on the 148 SMs
  int wpt = warps;
  while (wpt > 1 && static_cast<long long>(T) * wpt > 148LL * warps) wpt >>= 1;
  const int tpc = warps / wpt;
  const int grid = std::max(1, std::min((T + tpc - 1) / tpc, 148));
  b200::route_plan_small_kernel<<<grid, b200::SMALL_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(wr_kmajor), bias, T, D, E, k,
      renorm, topk_idx, topk_w, counts, bucket_start, send_order, dst_slot, push ? *push : pz, push ? 1 : 0,
      ticket, wpt);
  b200_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int b200_route_plan_small_max_flat() { return b200::SMALL_MAX_FLAT; }

extern "C" int b200_capacity(const int* send_counts, const b200::CapacityArgs* a, int* out, void* stream) {
  if (a == nullptr || a->world < 1 || a->world > B200_MAX_WORLD || a->e_local < 1 ||
      a->world * a->e_local > B200_MAX_EXPERTS || a->rank < 0 || a->rank >= a->world || a->epoch == 0)
    return -1;
  b200::capacity_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(send_counts, *a, out);
  b200_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int b200_abi_size_capacity_args() { return static_cast<int>(sizeof(b200::CapacityArgs)); }

extern "C" int b200_abi_size_plan_push_args() { return static_cast<int>(sizeof(b200::PlanPushArgs)); }

// ---------------------------------------------------------------------------
// Allocation-free plan (declared and documented in plan_noalloc.h).
// ---------------------------------------------------------------------------
#include "plan_noalloc.h"

namespace b200 {
// The temporary of the plan kernels (one int per routed copy).  In host code
// this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) int g_plan_scratch[B200_PLAN_NOALLOC_MAX];

constexpr int kMaxDevices = 64;
// Device address of the array per device.  Atomic so that two host threads making the first
// call together is harmless (both resolve the same address; nothing is allocated either way).
static std::atomic<int*> g_plan_scratch_addr[kMaxDevices];
}  // namespace b200

extern "C" {

int b200_plan_noalloc_max(void) { return B200_PLAN_NOALLOC_MAX; }

int b200_plan_noalloc(const int* topk_idx, int n_flat, int num_experts, int* counts,
                      int* bucket_start, int* send_order, int* dst_slot, void* stream) {
  if (n_flat < 0 || num_experts < 1 || num_experts > B200_MAX_EXPERTS || topk_idx == nullptr ||
      counts == nullptr || bucket_start == nullptr || send_order == nullptr)
    return B200_PLAN_NOALLOC_BAD_ARG;
  if (n_flat > B200_PLAN_NOALLOC_MAX) return B200_PLAN_NOALLOC_TOO_LARGE;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= b200::kMaxDevices) return B200_PLAN_NOALLOC_NO_DEVICE;
  // once per device, with that device current: resolve the array's device address
  int* scratch = b200::g_plan_scratch_addr[dev].load(std::memory_order_relaxed);
  if (scratch == nullptr) {
    int* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), b200::g_plan_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (p == nullptr) return B200_PLAN_NOALLOC_NO_DEVICE;
    b200::g_plan_scratch_addr[dev].store(p, std::memory_order_relaxed);
    scratch = p;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  b200::plan_rank_kernel<<<num_experts, 1024, 0, st>>>(topk_idx, n_flat, num_experts, scratch, counts);
  b200_count_launches(1);
  b200::PlanPushArgs pz;
  memset(&pz, 0, sizeof(pz));
  int blocks = (n_flat + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 1184) blocks = 1184;
  b200::plan_finalize_kernel<<<blocks, 256, 0, st>>>(topk_idx, scratch, counts, n_flat, num_experts,
                                                     bucket_start, send_order, dst_slot, pz, 0);
  b200_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"

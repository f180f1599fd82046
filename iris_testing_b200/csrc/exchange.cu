// Stand-alone (unfused) expert-parallel exchange kernels over symmetric peer
// memory: the padded dispatch with the reference's buffer contract, its mirror
// (padded return), token shuffle / unshuffle, the slot reduction that ends the
// fused combine, the SiLU gate and the cross-rank barrier.
//
// Counterparts in the reference project: kernels.py:21-66 (counts exchange) and
// kernels.py:69-146 (token exchange) become padded_dispatch_kernel; the shuffle
// design of kernels.py:150-205 / layers/token_shuffle.py:31-56 becomes
// shuffle_kernel; the host barrier of benchmark.py:194 becomes barrier_kernel.
// The return path, unshuffle, slot reduction and activation have no reference
// counterpart.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <string.h>

#include "moe_args.h"
#include "sm100_ptx.cuh"

namespace b200 {

struct PeerTable {
  unsigned long long p[B200_MAX_WORLD];
};

// One warp copies a row of `row16` 16-byte chunks with up to eight loads in flight per lane
// (a remote store costs microseconds of latency; the copy is throughput- not latency-bound
// only with enough independent accesses outstanding).
__device__ __forceinline__ void copy_row_16(uint4* dst, const uint4* src, int row16, int lane) {
  for (int i = lane; i < row16; i += 256) {
    uint4 v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (i + 32 * j < row16) v[j] = ld_16(src + i + 32 * j);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (i + 32 * j < row16) st_16(dst + i + 32 * j, v[j]);
  }
}

// ---------------------------------------------------------------------------
// Padded dispatch.  Layouts (identical to the reference's data contract):
//   send_payload [sum_send, H]  rows ordered by destination, then local expert
//   send_counts  [world, e_local]
//   dst_offsets  [world]        first payload row of each destination
//   pca          [e_local, world]  on the destination: pca[e, src] = rows sent
//   token_buf    [e_local, world, CAP, H] on the destination
//   counts_ready [1], token_sync [e_local]: arrival counters on the destination
// Grid: (m_tiles, e_local, world).  A block copies up to `block_m` rows of one
// (dst, expert) cell and then adds 1 to token_sync[expert] on dst -- the
// per-tile completion rule (receiver expects sum_src ceil(pca[e,src]/block_m)).
// Blocks with blockIdx.x == 0 and blockIdx.y == 0 also deliver the counts.
// ---------------------------------------------------------------------------
__global__ void padded_dispatch_kernel(const uint4* __restrict__ payload,
                                       const int* __restrict__ send_counts,
                                       const int* __restrict__ dst_offsets, PeerTable peer_pca,
                                       PeerTable peer_token_buf, PeerTable peer_counts_ready,
                                       PeerTable peer_token_sync, int rank, int world, int e_local,
                                       int cap, int row16, int block_m, int* status) {
  // Destinations are visited in rank-rotated order (this rank first, then rank+1, ...):
  // at any moment the ranks target different peers instead of all flooding rank 0's links.
  const int dst = (rank + static_cast<int>(blockIdx.z)) % world, e = blockIdx.y, mt = blockIdx.x;
  if (mt == 0 && e == 0) {
    int* pca = reinterpret_cast<int*>(peer_pca.p[dst]);
    for (int e2 = threadIdx.x; e2 < e_local; e2 += blockDim.x)
      pca[e2 * world + rank] = send_counts[dst * e_local + e2];
    __syncthreads();
    if (threadIdx.x == 0) {
      fence_acq_rel_sys();
      red_add_release_sys(reinterpret_cast<uint32_t*>(peer_counts_ready.p[dst]), 1u);
    }
  }
  const int n_true = send_counts[dst * e_local + e];
  if (n_true > cap && mt == 0 && threadIdx.x == 0) report_status(status, ST_OVERFLOW);
  const int n = min(n_true, cap);            // rows beyond the cell's capacity are dropped
  const int m0 = mt * block_m;
  if (m0 >= n) return;                       // empty tile: nothing to send, nothing to signal
  int eoff = 0;
  for (int e2 = 0; e2 < e; ++e2) eoff += send_counts[dst * e_local + e2];
  const size_t src_row0 = static_cast<size_t>(dst_offsets[dst]) + eoff + m0;
  uint4* tb = reinterpret_cast<uint4*>(peer_token_buf.p[dst]);
  const size_t dst_row0 = (static_cast<size_t>(e) * world + rank) * cap + m0;
  const int rows = min(block_m, n - m0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int r = warp; r < rows; r += nwarps) {
    const uint4* s = payload + (src_row0 + r) * row16;
    uint4* d = tb + (dst_row0 + r) * row16;
    copy_row_16(d, s, row16, lane);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_acq_rel_sys();
    red_add_release_sys(reinterpret_cast<uint32_t*>(peer_token_sync.p[dst]) + e, 1u);
  }
}

// ---------------------------------------------------------------------------
// Padded return (the mirror): the expert rank sends the processed rows of
// cell (e, src) back to rank src, where they land in
//   ret_buf [world(expert rank), e_local, CAP, H]
// so that row (dst, e, m) of ret_buf answers payload row
// dst_offsets[dst] + expert_offs[dst, e] + m.  ret_sync[world] on the source
// counts tiles per expert rank.
// ---------------------------------------------------------------------------
__global__ void padded_return_kernel(const uint4* __restrict__ out_buf, const int* __restrict__ pca,
                                     PeerTable peer_ret_buf, PeerTable peer_ret_sync, int rank,
                                     int world, int e_local, int cap, int row16, int block_m) {
  const int src = (rank + static_cast<int>(blockIdx.z)) % world, e = blockIdx.y, mt = blockIdx.x;   // rank-rotated
  const int n = min(pca[e * world + src], cap);
  const int m0 = mt * block_m;
  if (m0 >= n) return;
  const int rows = min(block_m, n - m0);
  const size_t in_row0 = (static_cast<size_t>(e) * world + src) * cap + m0;
  uint4* rb = reinterpret_cast<uint4*>(peer_ret_buf.p[src]);
  const size_t out_row0 = (static_cast<size_t>(rank) * e_local + e) * cap + m0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int r = warp; r < rows; r += nwarps) {
    const uint4* s = out_buf + (in_row0 + r) * row16;
    uint4* d = rb + (out_row0 + r) * row16;
    copy_row_16(d, s, row16, lane);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_acq_rel_sys();
    red_add_release_sys(reinterpret_cast<uint32_t*>(peer_ret_sync.p[src]) + rank, 1u);
  }
}

// ---------------------------------------------------------------------------
// Re-usable padded exchange (no memset, no separate barrier between calls).
//
// Same buffer contract as above, driven by an epoch number that the host increments per call:
//  * a rank announces "I have entered epoch i" to every peer only after it has zeroed its own
//    pca / counts_ready / token_sync (whose previous values its consumer, earlier in the same
//    stream, is done with); a sender writes into a destination only after it has seen that
//    announcement, so a fast rank can never write into buffers a slow rank still reads --
//    the race the reference closes with a memset and a host barrier per call
//    (benchmark.py:247-272);
//  * rows move as bulk copies (global -> shared -> the peer's global memory): a tile of a cell is
//    one contiguous block in the packed payload and in token_buf, so each worker warp streams it
//    through two 16 KiB buffers and then adds 1 to token_sync[expert] on the destination (per-tile
//    completion rule, kernels.py:136-146).
// `mirror` selects the return direction: tiles of out_buf[e, src] go to ret_buf[rank, e] on src
// and are counted in ret_sync[rank] there (no announcement is needed: a return follows the
// dispatch it answers).
// ---------------------------------------------------------------------------
constexpr int A2A_WARPS = 4;
constexpr int A2A_CHUNK = 16384;

struct PaddedArgs {
  PeerTable pca, token_buf, counts_ready, token_sync, entered;   // dispatch; mirror: token_buf = ret_buf,
                                                                 // token_sync = ret_sync
  const uint32_t* entered_local;   // [world] on this rank: epochs the peers have entered
  uint32_t epoch;
  int rank, world, e_local, cap, block_m;
  long long row_bytes;
  int mirror;
  int plain;       // 1: rows move as 16-byte loads/stores of all threads of a block instead of bulk copies
  int* status;
  unsigned long long budget_ns;
};

__global__ void __launch_bounds__(256)
padded_bulk_kernel(const uint8_t* __restrict__ src_rows, const int* __restrict__ counts,
                   const int* __restrict__ dst_offsets, PaddedArgs a) {
  extern __shared__ __align__(128) uint8_t a2a_smem[];
  __shared__ uint64_t bars[A2A_WARPS][2];
  __shared__ int s_abort;
  __shared__ int s_eoff[B200_MAX_EXPERTS];     // dispatch: first payload row of cell (dst, e)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int W = a.world, EL = a.e_local;
  if (tid == 0) s_abort = 0;
  if (lane == 0 && warp < A2A_WARPS) {
    mbar_init(&bars[warp][0], 1);
    mbar_init(&bars[warp][1], 1);
    fence_mbar_init();
  }
  if (!a.mirror) {
    for (int c = tid; c < W * EL; c += blockDim.x) {
      const int d = c / EL, e = c - d * EL;
      int off = dst_offsets[d];
      for (int e2 = 0; e2 < e; ++e2) off += counts[d * EL + e2];
      s_eoff[c] = off;
    }
  }
  __syncthreads();
  WaitCtx w; w.abort_flag = &s_abort; w.status = a.status; w.budget_ns = a.budget_ns;

  if (!a.mirror) {
    // ---- announce this epoch (after re-arming the local flags), then deliver the counts
    if (blockIdx.x == 0) {
      int* pca = reinterpret_cast<int*>(a.pca.p[a.rank]);
      for (int i = tid; i < EL * W; i += blockDim.x) pca[i] = 0;
      for (int e = tid; e < EL; e += blockDim.x) reinterpret_cast<uint32_t*>(a.token_sync.p[a.rank])[e] = 0u;
      if (tid == 0) *reinterpret_cast<uint32_t*>(a.counts_ready.p[a.rank]) = 0u;
      __syncthreads();
      if (tid < W) {
        fence_acq_rel_sys();
        st_release_sys(reinterpret_cast<uint32_t*>(a.entered.p[tid]) + a.rank, a.epoch);
      }
    }
    for (int d = blockIdx.x; d < W; d += gridDim.x) {
      const int dst = (a.rank + d) % W;
      if (tid == 0) wait_flag_geq(a.entered_local + dst, a.epoch, w, ST_TIMEOUT_BARRIER);
      __syncthreads();
      if (!s_abort) {
        int* pca = reinterpret_cast<int*>(a.pca.p[dst]);
        for (int e = tid; e < EL; e += blockDim.x) pca[e * W + a.rank] = counts[dst * EL + e];
      }
      __syncthreads();
      if (tid == 0 && !s_abort) {
        fence_acq_rel_sys();
        red_add_release_sys(reinterpret_cast<uint32_t*>(a.counts_ready.p[dst]), 1u);
      }
    }
  }

  const int tpc = (a.cap + a.block_m - 1) / a.block_m;
  const long long total = static_cast<long long>(W) * EL * tpc;
  if (a.plain) {
    // ---- tiles: one block per unit, every warp copies rows with eight 16-byte accesses in
    // flight per lane; several blocks per SM hide each other's end-of-tile fence
    __shared__ unsigned s_entered;
    if (tid == 0) s_entered = a.mirror ? 0xffffffffu : 0u;
    __syncthreads();
    const int nwarps = blockDim.x >> 5;
    const int row16 = static_cast<int>(a.row_bytes / 16);
    for (long long u = blockIdx.x; u < total; u += gridDim.x) {
      const int d = static_cast<int>(u % W);
      const long long rest = u / W;
      const int e = static_cast<int>(rest % EL), mt = static_cast<int>(rest / EL);
      const int peer = (a.rank + d) % W;
      const int n_true = a.mirror ? __ldcg(counts + e * W + peer) : counts[peer * EL + e];
      if (n_true > a.cap && mt == 0 && tid == 0) report_status(a.status, ST_OVERFLOW);
      const int n = min(n_true, a.cap);
      const int m0 = mt * a.block_m;
      if (m0 >= n) continue;
      const int rows = min(a.block_m, n - m0);
      if (!(s_entered >> peer & 1u)) {          // uniform: s_entered only changes between barriers
        if (tid == 0 && wait_flag_geq(a.entered_local + peer, a.epoch, w, ST_TIMEOUT_BARRIER))
          s_entered |= 1u << peer;
        __syncthreads();
        if (s_abort) break;
      }
      const uint8_t* src;
      uint8_t* dst;
      if (!a.mirror) {
        src = src_rows + (static_cast<long long>(s_eoff[peer * EL + e]) + m0) * a.row_bytes;
        dst = reinterpret_cast<uint8_t*>(a.token_buf.p[peer]) +
              ((static_cast<long long>(e) * W + a.rank) * a.cap + m0) * a.row_bytes;
      } else {
        src = src_rows + ((static_cast<long long>(e) * W + peer) * a.cap + m0) * a.row_bytes;
        dst = reinterpret_cast<uint8_t*>(a.token_buf.p[peer]) +
              ((static_cast<long long>(a.rank) * EL + e) * a.cap + m0) * a.row_bytes;
      }
      for (int r = warp; r < rows; r += nwarps)
        copy_row_16(reinterpret_cast<uint4*>(dst + r * a.row_bytes),
                    reinterpret_cast<const uint4*>(src + r * a.row_bytes), row16, lane);
      __syncthreads();
      if (tid == 0) {
        fence_acq_rel_sys();
        red_add_release_sys(reinterpret_cast<uint32_t*>(a.token_sync.p[peer]) + (a.mirror ? a.rank : e), 1u);
      }
    }
    return;
  }

  // ---- tiles: one worker warp per unit, lane 0 drives the bulk copies
  if (lane != 0 || warp >= A2A_WARPS) return;
  uint8_t* buf[2] = {a2a_smem + (warp * 2) * A2A_CHUNK, a2a_smem + (warp * 2 + 1) * A2A_CHUNK};
  uint32_t phase[2] = {0u, 0u};
  unsigned entered_ok = a.mirror ? 0xffffffffu : 0u;
  const long long worker = static_cast<long long>(blockIdx.x) * A2A_WARPS + warp;
  const long long nworkers = static_cast<long long>(gridDim.x) * A2A_WARPS;
  for (long long u = worker; u < total; u += nworkers) {
    // the peer index runs fastest, rotated by rank: at any moment all links are in use and
    // the ranks target different peers
    const int d = static_cast<int>(u % W);
    const long long rest = u / W;
    const int e = static_cast<int>(rest % EL), mt = static_cast<int>(rest / EL);
    const int peer = (a.rank + d) % W;
    const int n_true = a.mirror ? __ldcg(counts + e * W + peer) : counts[peer * EL + e];
    if (n_true > a.cap && mt == 0) report_status(a.status, ST_OVERFLOW);
    const int n = min(n_true, a.cap);             // rows beyond the cell's capacity are dropped
    const int m0 = mt * a.block_m;
    if (m0 >= n) continue;                        // empty tile: nothing to send, nothing to signal
    const int rows = min(a.block_m, n - m0);
    if (!(entered_ok >> peer & 1u)) {
      if (!wait_flag_geq(a.entered_local + peer, a.epoch, w, ST_TIMEOUT_BARRIER)) break;
      entered_ok |= 1u << peer;
    }
    const uint8_t* src;
    uint8_t* dst;
    if (!a.mirror) {
      src = src_rows + (static_cast<long long>(s_eoff[peer * EL + e]) + m0) * a.row_bytes;
      dst = reinterpret_cast<uint8_t*>(a.token_buf.p[peer]) +
            ((static_cast<long long>(e) * W + a.rank) * a.cap + m0) * a.row_bytes;
    } else {
      src = src_rows + ((static_cast<long long>(e) * W + peer) * a.cap + m0) * a.row_bytes;
      dst = reinterpret_cast<uint8_t*>(a.token_buf.p[peer]) +
            ((static_cast<long long>(a.rank) * EL + e) * a.cap + m0) * a.row_bytes;
    }
    const long long bytes = rows * a.row_bytes;
    const int nchunks = static_cast<int>((bytes + A2A_CHUNK - 1) / A2A_CHUNK);
    bool ok = true;
    {
      const uint32_t sz = static_cast<uint32_t>(min(static_cast<long long>(A2A_CHUNK), bytes));
      mbar_expect_tx(&bars[warp][0], sz);
      bulk_load_1d(buf[0], src, sz, &bars[warp][0]);
    }
    for (int c = 0; c < nchunks && ok; ++c) {
      const int b = c & 1;
      const long long off = static_cast<long long>(c) * A2A_CHUNK;
      const uint32_t sz = static_cast<uint32_t>(min(static_cast<long long>(A2A_CHUNK), bytes - off));
      if (c + 1 < nchunks) {
        // the other buffer's previous store (chunk c-1) must have been read before it is refilled
        bulk_wait_group_read<0>();
        const long long off2 = off + A2A_CHUNK;
        const uint32_t sz2 = static_cast<uint32_t>(min(static_cast<long long>(A2A_CHUNK), bytes - off2));
        mbar_expect_tx(&bars[warp][b ^ 1], sz2);
        bulk_load_1d(buf[b ^ 1], src + off2, sz2, &bars[warp][b ^ 1]);
      }
      ok = mbar_wait(&bars[warp][b], phase[b], w, ST_TIMEOUT_PIPE_FULL);
      phase[b] ^= 1u;
      if (!ok) break;
      bulk_store_1d(dst + off, buf[b], sz);
      bulk_commit_group();
    }
    // the tile's rows are in the peer's memory before its arrival is counted there
    bulk_wait_group<0>();
    if (!ok) break;
    fence_proxy_async();
    fence_acq_rel_sys();
    uint32_t* flag = reinterpret_cast<uint32_t*>(a.token_sync.p[peer]) + (a.mirror ? a.rank : e);
    red_add_release_sys(flag, 1u);
  }
  bulk_wait_group<0>();
}

// Waits (bounded) until a dispatch has fully landed on this rank: counts_ready == world and
// token_sync[e] == sum_src ceil(min(pca[e, src], cap) / block_m).  The device-side counterpart
// of the host spin-waits of unit_tests.py:17-43; replaces a cross-rank barrier after the call.
__global__ void padded_wait_kernel(const int* pca, const uint32_t* counts_ready, const uint32_t* token_sync,
                                   int world, int e_local, int cap, int block_m, int* status,
                                   unsigned long long budget_ns) {
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  WaitCtx w; w.abort_flag = &s_abort; w.status = status; w.budget_ns = budget_ns;
  if (threadIdx.x == 0) wait_flag_geq(counts_ready, static_cast<uint32_t>(world), w, ST_TIMEOUT_COUNTS);
  __syncthreads();
  for (int e = threadIdx.x; e < e_local && !s_abort; e += blockDim.x) {
    uint32_t expect = 0;
    for (int s = 0; s < world; ++s) expect += (min(__ldcg(pca + e * world + s), cap) + block_m - 1) / block_m;
    wait_flag_geq(token_sync + e, expect, w, ST_TIMEOUT_TILE_READY);
  }
}

// y[t, :] = sum_slot w[t, slot] * ret_buf[cell(t, slot), :] -- the top-k
// weighted sum on the source rank.  dst_slot[t*k+slot] is the payload row of
// that copy; bucket_start / send_counts locate its (dst, e, m) cell.
// Waits (bounded) until every expert rank has returned its tiles.
__global__ void weighted_gather_kernel(const __nv_bfloat16* __restrict__ ret_buf,
                                       const int* __restrict__ dst_slot,
                                       const int* __restrict__ topk_idx,
                                       const int* __restrict__ bucket_start,
                                       const float* __restrict__ topk_w, uint32_t* ret_sync,
                                       const int* __restrict__ send_counts, int T, int topk, int world,
                                       int e_local, int cap, int H, int block_m,
                                       __nv_bfloat16* __restrict__ y, int* status,
                                       unsigned long long budget_ns, unsigned int* ticket) {
  __shared__ int s_abort;
  __shared__ int s_last;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  if (threadIdx.x < world) {
    uint32_t expect = 0;
    for (int e = 0; e < e_local; ++e)
      expect += (min(send_counts[threadIdx.x * e_local + e], cap) + block_m - 1) / block_m;
    WaitCtx w; w.abort_flag = &s_abort; w.status = status; w.budget_ns = budget_ns;
    wait_flag_geq(ret_sync + threadIdx.x, expect, w, ST_TIMEOUT_COMBINE);
  }
  __syncthreads();
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  for (int t = warp; t < T && !s_abort; t += nwarps) {
    for (int c0 = lane * 8; c0 < H; c0 += 256) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int s = 0; s < topk; ++s) {
        const int flat = t * topk + s;
        const int ge = topk_idx[flat];
        const int m = dst_slot[flat] - bucket_start[ge];
        if (m >= cap) continue;   // dropped by capacity
        const size_t row = static_cast<size_t>(ge) * cap + m;   // [dst, e] flattens to ge
        const uint4 v = ld_16(reinterpret_cast<const uint4*>(ret_buf + row * H + c0));
        const float wv = topk_w[flat];
        const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(h2[j]);
          acc[2 * j] += wv * f.x;
          acc[2 * j + 1] += wv * f.y;
        }
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * H + c0) = o;
    }
  }
  // With a ticket counter the last block re-arms ret_sync for the next exchange: every block
  // has seen all of this exchange's arrivals, and the next return cannot start before this
  // rank's next dispatch, which follows this kernel in its stream.
  if (ticket != nullptr) {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      s_last = (atomicAdd(ticket, 1u) == gridDim.x - 1) ? 1 : 0;
    }
    __syncthreads();
    if (s_last) {
      if (threadIdx.x < world) ret_sync[threadIdx.x] = 0u;
      if (threadIdx.x == 0) *ticket = 0u;
    }
  }
}

// ---------------------------------------------------------------------------
// Token shuffle: drop the padding.  packed[off(e,src) + m, :] = token_buf[e, src, m, :]
// for m < pca[e, src], off = exclusive cumsum of pca in (e, src) order.  With
// `wait` set, first waits (bounded) for counts_ready >= world and for
// token_sync[e] >= sum_src ceil(pca[e,src]/block_m).  `inverse` scatters back.
// ---------------------------------------------------------------------------
__global__ void shuffle_kernel(uint4* token_buf, uint4* packed, const int* pca,
                               const uint32_t* counts_ready, const uint32_t* token_sync, int world,
                               int e_local, int cap, int row16, int block_m, int wait, int inverse,
                               int* group_rows, int max_rows, int* status,
                               unsigned long long budget_ns) {
  __shared__ int s_off[B200_MAX_EXPERTS + 1];   // e_local * world cells
  __shared__ int s_abort;
  const int cells = e_local * world;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  WaitCtx w; w.abort_flag = &s_abort; w.status = status; w.budget_ns = budget_ns;
  if (wait) {
    if (threadIdx.x == 0) wait_flag_geq(counts_ready, static_cast<uint32_t>(world), w, ST_TIMEOUT_COUNTS);
    __syncthreads();
    if (threadIdx.x < e_local && !s_abort) {
      uint32_t expect = 0;
      for (int s = 0; s < world; ++s)
        expect += (min(__ldcg(pca + threadIdx.x * world + s), cap) + block_m - 1) / block_m;
      wait_flag_geq(token_sync + threadIdx.x, expect, w, ST_TIMEOUT_TILE_READY);
    }
    __syncthreads();
    if (s_abort) return;
  }
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int c = 0; c < cells; ++c) { s_off[c] = acc; acc += min(__ldcg(pca + c), cap); }
    s_off[cells] = acc;
  }
  __syncthreads();
  if (blockIdx.x == 0 && group_rows != nullptr)
    for (int e = threadIdx.x; e < e_local; e += blockDim.x)
      group_rows[e] = s_off[(e + 1) * world] - s_off[e * world];
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  // the packed buffer holds max_rows rows: more valid rows than that are reported, not copied
  if (s_off[cells] > max_rows && blockIdx.x == 0 && threadIdx.x == 0) {
    report_status(status, ST_OVERFLOW);
    if (status != nullptr) atomicMax(status + 1, s_off[cells]);
  }
  const int total = min(s_off[cells], max_rows);
  int cell = 0;
  for (int r = warp; r < total; r += nwarps) {
    while (r >= s_off[cell + 1]) ++cell;
    const int m = r - s_off[cell];
    uint4* pad = token_buf + (static_cast<size_t>(cell) * cap + m) * row16;
    uint4* pk = packed + static_cast<size_t>(r) * row16;
    if (!inverse) for (int i = lane; i < row16; i += 32) pk[i] = ld_16(pad + i);
    else          for (int i = lane; i < row16; i += 32) pad[i] = ld_16(pk + i);
  }
}

// ---------------------------------------------------------------------------
// Slot reduction ending the fused combine: wait (bounded) until `expected`
// (row, n-tile) units have landed in out_slots, then y[t] = sum_slot
// out_slots[dst_slot[t*k+slot]] in slot order (deterministic).  The last block to finish
// re-arms the per-iteration state (arrival counter, this parity's tile-ready
// counters) and tells every peer that this rank has retired the iteration.
// ---------------------------------------------------------------------------
struct RetireArgs {
  int world, rank;
  uint32_t iter_done_value;          // iterations retired after this one
  unsigned long long peer_iter_done[B200_MAX_WORLD];   // uint32 [world] on each rank
  uint32_t* ready_counters;          // this parity's tile-ready counters (local)
  int num_ready;
  unsigned int* ticket;              // local scratch counter (zero between launches)
  // Device-side iteration state: when iter_ptr is set, it = *iter_ptr; the counters of
  // parity (it & 1) are re-armed, iter_done is published as it + 1 and *iter_ptr becomes it + 1.
  uint32_t* iter_ptr;
  unsigned long long stride_ready;   // bytes between the two parity copies of ready_counters
};

template <int KMAX>   // topk <= KMAX; about eight 16-byte loads per lane are kept in flight
__global__ void slot_reduce_kernel(const __nv_bfloat16* out_slots, const int* __restrict__ dst_slot,
                                   uint32_t* arrived, uint32_t expected, int T, int topk, int H,
                                   __nv_bfloat16* __restrict__ y, RetireArgs ra, int* status,
                                   unsigned long long budget_ns) {
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    s_abort = 0;
    // A kernel of this step has already reported an error on this rank: its rows will never
    // arrive, so do not wait for them (the iteration is still retired below).
    if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) {
      s_abort = 1;
    } else {
      WaitCtx w; w.abort_flag = &s_abort; w.status = status; w.budget_ns = budget_ns;
      wait_flag_geq(arrived, expected, w, ST_TIMEOUT_COMBINE);
    }
  }
  __syncthreads();
  if (!s_abort) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int nwarps = (gridDim.x * blockDim.x) >> 5;
    constexpr int U = 8 / KMAX;    // 16-byte column chunks per lane in flight at once (times topk loads)
    for (int t = warp; t < T; t += nwarps) {
      // results sit at the row's position in the packed send order (dst_slot), or at
      // t*topk+s when no map is given
      size_t row[KMAX];
#pragma unroll
      for (int s = 0; s < KMAX; ++s)
        if (s < topk)
          row[s] = dst_slot != nullptr ? static_cast<size_t>(__ldg(dst_slot + t * topk + s))
                                       : static_cast<size_t>(t) * topk + s;
      for (int cb = lane * 8; cb < H; cb += 256 * U) {
        uint4 v[U][KMAX];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c0 = cb + u * 256;
#pragma unroll
          for (int s = 0; s < KMAX; ++s)
            if (s < topk && c0 < H)
              v[u][s] = ld_16(reinterpret_cast<const uint4*>(out_slots + row[s] * H + c0));
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int c0 = cb + u * 256;
          if (c0 >= H) continue;
          float acc[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
          for (int s = 0; s < KMAX; ++s) {
            if (s < topk) {
              const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&v[u][s]);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h2[j]);
                acc[2 * j] += f.x;
                acc[2 * j + 1] += f.y;
              }
            }
          }
          uint4 o;
          o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
          o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
          *reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * H + c0) = o;
        }
      }
    }
  }
  // retire the iteration (last block only)
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    s_last = (atomicAdd(ra.ticket, 1u) == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_last) {
    uint32_t done_value = ra.iter_done_value;
    uint32_t* ready = ra.ready_counters;
    if (ra.iter_ptr != nullptr) {
      const uint32_t it = __ldcg(ra.iter_ptr);
      done_value = it + 1u;
      if (it & 1u) ready = reinterpret_cast<uint32_t*>(reinterpret_cast<char*>(ready) + ra.stride_ready);
    }
    for (int i = threadIdx.x; i < ra.num_ready; i += blockDim.x) ready[i] = 0u;
    __syncthreads();
    if (threadIdx.x == 0) {
      *arrived = 0u;
      *ra.ticket = 0u;
      if (ra.iter_ptr != nullptr) *ra.iter_ptr = done_value;   // the next iteration's kernels read this
    }
    __syncthreads();
    if (threadIdx.x < ra.world) {
      fence_acq_rel_sys();
      st_release_sys(reinterpret_cast<uint32_t*>(ra.peer_iter_done[threadIdx.x]) + ra.rank, done_value);
    }
  }
}

// h[r, j] = silu(gate[r, j]) * up[r, j]
__global__ void silu_gate_kernel(const __nv_bfloat162* __restrict__ gate,
                                 const __nv_bfloat162* __restrict__ up,
                                 __nv_bfloat162* __restrict__ out, size_t n2) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n2;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const float2 g = __bfloat1622float2(gate[i]);
    const float2 u = __bfloat1622float2(up[i]);
    out[i] = __floats2bfloat162_rn(g.x / (1.f + __expf(-g.x)) * u.x, g.y / (1.f + __expf(-g.y)) * u.y);
  }
}

// Cross-rank barrier: publish `epoch` into slot [rank] of every peer's flag
// array, then wait (bounded) until all local slots have reached it.
__global__ void barrier_kernel(PeerTable peer_flags, uint32_t* local_flags, int rank, int world,
                               uint32_t epoch, int* status, unsigned long long budget_ns) {
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  if (threadIdx.x < world) {
    fence_acq_rel_sys();
    st_release_sys(reinterpret_cast<uint32_t*>(peer_flags.p[threadIdx.x]) + rank, epoch);
    WaitCtx w; w.abort_flag = &s_abort; w.status = status; w.budget_ns = budget_ns;
    wait_flag_geq(local_flags + threadIdx.x, epoch, w, ST_TIMEOUT_BARRIER);
  }
}

}  // namespace b200


extern "C" {

using b200::PeerTable;

static PeerTable make_table(const unsigned long long* p, int world) {
  PeerTable t;
  memset(&t, 0, sizeof(t));
  for (int i = 0; i < world && i < B200_MAX_WORLD; ++i) t.p[i] = p[i];
  return t;
}

int b200_padded_dispatch(const void* payload, const int* send_counts, const int* dst_offsets,
                         const unsigned long long* peer_pca, const unsigned long long* peer_token_buf,
                         const unsigned long long* peer_counts_ready,
                         const unsigned long long* peer_token_sync, int rank, int world, int e_local,
                         int cap, int hidden_dim, int block_m, int* status, void* stream) {
  if (hidden_dim % 8 != 0 || world > B200_MAX_WORLD || world * e_local > B200_MAX_EXPERTS ||
      block_m < 1 || cap < 1)
    return -1;
  dim3 grid((cap + block_m - 1) / block_m, e_local, world);
  b200::padded_dispatch_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(payload), send_counts, dst_offsets, make_table(peer_pca, world),
      make_table(peer_token_buf, world), make_table(peer_counts_ready, world),
      make_table(peer_token_sync, world), rank, world, e_local, cap, hidden_dim / 8, block_m, status);
  b200_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

int b200_padded_return(const void* out_buf, const int* pca, const unsigned long long* peer_ret_buf,
                       const unsigned long long* peer_ret_sync, int rank, int world, int e_local,
                       int cap, int hidden_dim, int block_m, void* stream) {
  if (hidden_dim % 8 != 0 || world > B200_MAX_WORLD || block_m < 1 || cap < 1) return -1;
  dim3 grid((cap + block_m - 1) / block_m, e_local, world);
  b200::padded_return_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(out_buf), pca, make_table(peer_ret_buf, world),
      make_table(peer_ret_sync, world), rank, world, e_local, cap, hidden_dim / 8, block_m);
  b200_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

// Epoch-driven padded dispatch (mirror = 0) or return (mirror = 1); see padded_bulk_kernel.
// dispatch: rows = packed payload, counts = send_counts [world, e_local], dst_offsets [world];
// return:   rows = out_buf [e_local, world, cap, H], counts = pca [e_local, world], dst_offsets unused,
//           peer_token_buf = ret_buf, peer_token_sync = ret_sync.
int b200_padded_exchange(const void* rows, const int* counts, const int* dst_offsets,
                         const unsigned long long* peer_pca, const unsigned long long* peer_token_buf,
                         const unsigned long long* peer_counts_ready,
                         const unsigned long long* peer_token_sync,
                         const unsigned long long* peer_entered, const void* entered_local,
                         unsigned int epoch, int rank, int world, int e_local, int cap, int hidden_dim,
                         int elem_bytes, int block_m, int mirror, int num_blocks, int plain, int* status,
                         unsigned long long budget_ns, void* stream) {
  if (world < 1 || world > B200_MAX_WORLD || world * e_local > B200_MAX_EXPERTS || block_m < 1 || cap < 1 ||
      (static_cast<long long>(hidden_dim) * elem_bytes) % 16 != 0 || num_blocks < 1 ||
      (reinterpret_cast<uintptr_t>(rows) & 15u) != 0)
    return -1;
  static bool configured = false;
  const int smem = b200::A2A_WARPS * 2 * b200::A2A_CHUNK;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(b200::padded_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  b200::PaddedArgs a;
  memset(&a, 0, sizeof(a));
  if (!mirror) {
    a.pca = make_table(peer_pca, world);
    a.counts_ready = make_table(peer_counts_ready, world);
    a.entered = make_table(peer_entered, world);
    a.entered_local = static_cast<const uint32_t*>(entered_local);
  }
  a.token_buf = make_table(peer_token_buf, world);
  a.token_sync = make_table(peer_token_sync, world);
  a.epoch = epoch;
  a.rank = rank; a.world = world; a.e_local = e_local; a.cap = cap; a.block_m = block_m;
  a.row_bytes = static_cast<long long>(hidden_dim) * elem_bytes;
  a.mirror = mirror;
  a.plain = plain ? 1 : 0;
  a.status = status;
  a.budget_ns = budget_ns;
  if (plain)
    b200::padded_bulk_kernel<<<num_blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(rows), counts, dst_offsets, a);
  else
    b200::padded_bulk_kernel<<<num_blocks, b200::A2A_WARPS * 32, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(rows), counts, dst_offsets, a);
  b200_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

int b200_padded_wait(const int* pca, const void* counts_ready, const void* token_sync, int world,
                     int e_local, int cap, int block_m, int* status, unsigned long long budget_ns,
                     void* stream) {
  if (world < 1 || e_local < 1 || block_m < 1) return -1;
  b200::padded_wait_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      pca, static_cast<const uint32_t*>(counts_ready), static_cast<const uint32_t*>(token_sync), world,
      e_local, cap, block_m, status, budget_ns);
  b200_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

int b200_weighted_gather(const void* ret_buf, const int* dst_slot, const int* topk_idx,
                         const int* bucket_start, const float* topk_w, void* ret_sync,
                         const int* send_counts, int T, int topk, int world, int e_local, int cap,
                         int hidden_dim, int block_m, void* y, int* status,
                         unsigned long long budget_ns, unsigned int* ticket, void* stream) {
  if (hidden_dim % 8 != 0 || world > 32) return -1;
  int blocks = (T + 7) / 8;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 8) blocks = 148 * 8;
  b200::weighted_gather_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(ret_buf), dst_slot, topk_idx, bucket_start, topk_w,
      static_cast<uint32_t*>(ret_sync), send_counts, T, topk, world, e_local, cap, hidden_dim,
      block_m, static_cast<__nv_bfloat16*>(y), status, budget_ns, ticket);
  b200_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

int b200_shuffle(void* token_buf, void* packed, const int* pca, const void* counts_ready,
                 const void* token_sync, int world, int e_local, int cap, int hidden_dim, int block_m,
                 int wait, int inverse, int* group_rows, int max_rows, int* status,
                 unsigned long long budget_ns, void* stream) {
  if (hidden_dim % 8 != 0 || world * e_local > B200_MAX_EXPERTS || max_rows < 0) return -1;
  b200::shuffle_kernel<<<148 * 4, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint4*>(token_buf), static_cast<uint4*>(packed), pca,
      static_cast<const uint32_t*>(counts_ready), static_cast<const uint32_t*>(token_sync), world,
      e_local, cap, hidden_dim / 8, block_m, wait, inverse, group_rows, max_rows, status, budget_ns);
  b200_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

int b200_slot_reduce(const void* out_slots, const int* dst_slot, void* arrived, unsigned int expected,
                     int T, int topk,
                     int hidden_dim, void* y, const b200::RetireArgs* ra, int* status,
                     unsigned long long budget_ns, void* stream) {
  if (hidden_dim % 8 != 0 || ra == nullptr || topk < 1 || topk > 8) return -1;
  int blocks = (T + 7) / 8;
  if (blocks < 1) blocks = 1;
  if (blocks > 148 * 4) blocks = 148 * 4;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto* os = static_cast<const __nv_bfloat16*>(out_slots);
  auto* ar = static_cast<uint32_t*>(arrived);
  auto* yo = static_cast<__nv_bfloat16*>(y);
  if (topk <= 2)
    b200::slot_reduce_kernel<2><<<blocks, 256, 0, st>>>(os, dst_slot, ar, expected, T, topk, hidden_dim, yo,
                                                        *ra, status, budget_ns);
  else if (topk <= 4)
    b200::slot_reduce_kernel<4><<<blocks, 256, 0, st>>>(os, dst_slot, ar, expected, T, topk, hidden_dim, yo,
                                                        *ra, status, budget_ns);
  else
    b200::slot_reduce_kernel<8><<<blocks, 256, 0, st>>>(os, dst_slot, ar, expected, T, topk, hidden_dim, yo,
                                                        *ra, status, budget_ns);
  b200_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

int b200_silu_gate(const void* gate, const void* up, void* out, long long n, void* stream) {
  if (n % 2 != 0) return -1;
  if (n == 0) return 0;
  long long n2 = n / 2;
  long long blocks = (n2 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  b200::silu_gate_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat162*>(gate), static_cast<const __nv_bfloat162*>(up),
      static_cast<__nv_bfloat162*>(out), static_cast<size_t>(n2));
  b200_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

int b200_barrier(const unsigned long long* peer_flags, void* local_flags, int rank, int world,
                 unsigned int epoch, int* status, unsigned long long budget_ns, void* stream) {
  if (world > B200_MAX_WORLD) return -1;
  b200::barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      make_table(peer_flags, world), static_cast<uint32_t*>(local_flags), rank, world, epoch, status,
      budget_ns);
  b200_count_launches(1);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"

extern "C" int b200_abi_size_retire_args() { return static_cast<int>(sizeof(b200::RetireArgs)); }

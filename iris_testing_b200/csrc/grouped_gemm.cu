// Persistent grouped GEMM for sm_100a: bf16 x bf16 -> fp32 on tcgen05 tensor
// cores with TMEM accumulators, operands staged by (non-multicast) TMA.
//
//   C_g[m_g, N] = A_g[m_g, K] * W_g[N, K]^T      for g in [0, G)
//
// A is one packed row-major buffer (groups back to back, ragged m_g read from a
// device array), W is [G*N, K] row-major ("K-major" for both operands).
//
// One CTA per SM, warp-specialised:
//   warp 0      TMA producer (one lane)
//   warp 1      TMEM owner + MMA issuer (one lane)
//   warps 2-5   epilogue: TMEM -> registers -> shared staging -> coalesced stores
//   warps 6-9   (fused-dispatch build only) token senders: gather this rank's
//               routed rows and store them into the owning rank's receive
//               buffer over NVLink, then signal the M-tile they landed in.
//
// Epilogues: plain store, SiLU-gated (gate/up column blocks interleaved per
// 256-wide weight tile), "combine" (scale by the row's top-k weight and store
// straight into the source rank's return buffer at the row's send-order
// position, then count arrivals there) and "router" (one thread per token:
// softmax over the accumulator row, top-k in registers).
//
// Two geometries (template parameter CG): one CTA per 128 x 256 tile, or a
// pair of CTAs (cluster of 2, tcgen05 cta_group::2) per 256 x 256 tile in which
// each CTA stages its own half of both operands with plain TMA loads.
//
// Role of this file relative to the reference project: the persistent grouped
// GEMM sketched in kernels.py:207-289 / layers/expert.py:6-65, the token
// exchange of kernels.py:69-146 (fused in as the sender role) and the
// combine step the reference does not have.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "moe_args.h"
#include "sm100_ptx.cuh"
#include "topk.cuh"

namespace b200 {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int MAX_STAGES = 6;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;            // 16 KiB per CTA
constexpr int STG_COLS = 64;                          // columns per epilogue pass
constexpr int STG_ROW_BYTES = STG_COLS * 2;           // 128 B rows, 16-byte chunks XOR-swizzled by row
constexpr int STG_WARP_BYTES = 32 * STG_ROW_BYTES;    // one epilogue warp's 32 x 64 box (a TMA store box)
constexpr int STG_BYTES = 4 * STG_WARP_BYTES;         // 16 KiB
constexpr int TMEM_COLS = 512;                        // two 256-column accumulators
constexpr int NUM_THREADS_PLAIN = 192;
constexpr int SENDER_WARPS = 4;    // token-sender warps per CTA in the fused-dispatch build
constexpr int NUM_THREADS_FUSED = NUM_THREADS_PLAIN + SENDER_WARPS * 32;
constexpr int SEND_ROWS = 32;   // rows per sender work unit (aligned in the destination expert's row space)

struct __align__(16) ControlSmem {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t drain;
  uint32_t tmem_base;
  int abort_flag;
  int overflow;       // set during set-up only: this rank neither sends nor computes
  int total_mtiles;
  int total_units;
  int g_rows[B200_MAX_GROUPS];
  int g_row_start[B200_MAX_GROUPS + 1];
  int g_mtile_start[B200_MAX_GROUPS + 1];   // in 128-row tiles (arrival counters)
  int g_sched_start[B200_MAX_GROUPS + 1];   // in scheduling tiles (128 rows x CTAs per pair)
  int total_sched;
  // sender tables (fused dispatch), indexed by rotated bucket number
  int b_count[B200_MAX_EXPERTS];       // rows this rank sends to the bucket
  int b_send_start[B200_MAX_EXPERTS];  // first row of the bucket in send_order
  int b_dst_row[B200_MAX_EXPERTS];     // first destination row in the peer buffer
  int b_dst_rel0[B200_MAX_EXPERTS];    // that row relative to the expert's first row
  int b_dst_mtile0[B200_MAX_EXPERTS];  // index of the expert's first M-tile at the peer
  int b_dst_rank[B200_MAX_EXPERTS];
  int b_unit_start[B200_MAX_EXPERTS + 1];
  int ready_seen[64];                  // producer's direct-mapped cache of complete M-tiles
};

// Per-variant geometry.  CG = CTAs cooperating on one MMA (tcgen05 cta_group): with CG == 2
// the pair computes a 256-row tile, each CTA staging its own 128 rows of A and its own
// 128 of every 256 weight rows.  NT = 256-column accumulators that make up one tile:
//  * NT == 1: a 256-column tile; the two TMEM accumulators double-buffer (the epilogue of
//    tile i overlaps the MMAs of tile i+1); a stage is 32 KiB per CTA of a pair, six fit.
//  * NT == 2 (pairs only): a 512-column tile that uses BOTH accumulators at once, so one
//    stage of activations feeds twice the math: 25 % fewer operand bytes come out of L2
//    per FLOP, which under the power cap is worth more clock than the lost double
//    buffering costs (measured on B200: with three quarters of the operand loads skipped
//    the same kernel holds 1350 MHz instead of 1035 MHz).  The epilogue is hidden
//    by letting the second half's MMAs of the next tile trail the first half's by up to
//    STAGES-1 k-blocks.  A stage is 48 KiB per CTA, four fit.
template <int CG, int NT = 1>
struct Geo {
  static_assert(NT == 1 || CG == 2, "wide tiles are built from CTA pairs");
  static constexpr int STAGES = NT == 2 ? 4 : (CG == 2 ? 6 : 4);
  static constexpr int B_ROWS = BN / CG;                       // weight rows per CTA per accumulator
  static constexpr int B_HALF_BYTES = B_ROWS * BK * 2;
  static constexpr int B_STAGE_BYTES = NT * B_HALF_BYTES;
  static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  static constexpr int TM = BM * CG;                   // rows of a scheduling tile
  static constexpr int TILE_N = BN * NT;               // weight rows (accumulator columns) of a tile
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + STG_BYTES + (int)sizeof(ControlSmem) + 1024;
  static_assert(SMEM_BYTES <= 232448, "exceeds 227 KiB of shared memory per CTA");
};

// Maps a linear tile index to (group, m-tile, n-tile).  Tiles are ordered per
// group in chunks of `gm` M-tiles; inside a chunk the M index runs fastest so
// that concurrently running CTAs share a few weight tiles and a chunk of A
// that stays resident in L2 while the N index sweeps.
__host__ __device__ __forceinline__ bool decode_tile(const ControlSmem& c, int G, int TN, int gm, int idx,
                                            int& cursor, int& g, int& m, int& n) {
  while (cursor < G && idx >= TN * c.g_sched_start[cursor + 1]) ++cursor;
  if (cursor >= G) return false;
  g = cursor;
  const int tm = c.g_sched_start[g + 1] - c.g_sched_start[g];
  const int j = idx - TN * c.g_sched_start[g];
  // even out the chunks of this group: 16 M-tiles with a target of 12 become 8 + 8, not 12 + 4
  const int nchunks = (tm + gm - 1) / gm;
  gm = (tm + nchunks - 1) / nchunks;
  const int chunk_tiles = gm * TN;
  const int ch = j / chunk_tiles;
  const int r = j - ch * chunk_tiles;
  const int cm = (gm < tm - ch * gm) ? gm : (tm - ch * gm);
  n = r / cm;
  m = ch * gm + (r - n * cm);
  return true;
}

// Which tiles a scheduler (a CTA, or a CTA pair) takes: first, first + stride, ...
// Even rounds: with R = ceil(tiles / schedulers) rounds needed anyway, only ceil(tiles / R)
// schedulers take tiles, R each (the last ones maybe one fewer), instead of all of them taking
// R - 1 and a few taking one more.  The makespan in tiles is the same; when the kernel streams
// weights (few rows per expert) the last round no longer runs on a handful of SMs that cannot
// draw the full memory bandwidth.  Schedulers past the stride sit out (first = total).
__host__ __device__ __forceinline__ void tile_walk(int total, int schedulers, int sched_id, int& first,
                                                   int& stride) {
  const int rounds = (total + schedulers - 1) / schedulers;
  stride = rounds > 0 ? (total + rounds - 1) / rounds : schedulers;
  first = sched_id < stride ? sched_id : total;
}

// Exclusive scan of g_rows into g_row_start / g_mtile_start by one warp.
__device__ __forceinline__ void scan_groups(ControlSmem& c, int G, int lane, int sched_rows) {
  int row_carry = 0, tile_carry = 0, sched_carry = 0;
  for (int base = 0; base < G; base += 32) {
    const int g = base + lane;
    const int rows = (g < G) ? c.g_rows[g] : 0;
    const int tiles = (rows + BM - 1) / BM;
    const int sched = (rows + sched_rows - 1) / sched_rows;
    int rs = rows, ts = tiles, ss = sched;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int r2 = __shfl_up_sync(0xffffffffu, rs, o);
      const int t2 = __shfl_up_sync(0xffffffffu, ts, o);
      const int s2 = __shfl_up_sync(0xffffffffu, ss, o);
      if (lane >= o) { rs += r2; ts += t2; ss += s2; }
    }
    if (g < G) {
      c.g_row_start[g] = row_carry + rs - rows;
      c.g_mtile_start[g] = tile_carry + ts - tiles;
      c.g_sched_start[g] = sched_carry + ss - sched;
    }
    row_carry += __shfl_sync(0xffffffffu, rs, 31);
    tile_carry += __shfl_sync(0xffffffffu, ts, 31);
    sched_carry += __shfl_sync(0xffffffffu, ss, 31);
  }
  if (lane == 0) {
    c.g_row_start[G] = row_carry;
    c.g_mtile_start[G] = tile_carry;
    c.total_mtiles = tile_carry;
    c.g_sched_start[G] = sched_carry;
    c.total_sched = sched_carry;
  }
}

// silu(g) = g * sigmoid(g) = 0.5 g * tanh(0.5 g) + 0.5 g: one special-function op (tanh.approx,
// relative error about 2^-11, below the bf16 rounding of the result) and two FMAs per element.
// (The IEEE-rounded reciprocal of the exp form made the gated epilogue six times slower than
// the plain one: 12 us per 128 x 256 accumulator.)
__device__ __forceinline__ float silu_f(float g) {
  const float h = 0.5f * g;
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
  return fmaf(h, t, h);
}

// Reads a routing count.  On the device the table has been staged in shared memory (one
// coalesced read of the peer-written table per CTA); the host build of these helpers
// (index-arithmetic tests) reads plain memory.
__host__ __device__ __forceinline__ int load_count(const int* p) { return *p; }

// Rows this rank receives for local expert e: sum over sources of counts_all[src][me][e].
__host__ __device__ __forceinline__ int received_rows(const int* cnt, int W, int EL, int me, int e) {
  int rows = 0;
  for (int s = 0; s < W; ++s) rows += load_count(cnt + ((s * W + me) * EL + e));
  return rows;
}

// Fills sender-table entry `bi` of rank `me` from counts_all[src][dst][e]; returns false when
// the bucket would overrun the destination's receive capacity.
// Buckets are visited expert-major, and inside an expert destination-rotated starting with this
// rank: every rank's expert 0 fills first, each from its nearest "upstream" ranks first.  The
// receive layout orders the source segments of an expert the same way (self, self-1, self-2,
// ... modulo the world), so rows land in the order the consumer's M-tiles need them.
__host__ __device__ __forceinline__ bool fill_bucket(ControlSmem& c, const int* cnt, int W, int EL,
                                                     int me, int bi, int cap_rows) {
  const int ET = W * EL;
  const int e = bi / W, r = bi - e * W;
  const int dst = (me + r) % W;
  const int ge = dst * EL + e;
  const int n = load_count(cnt + ((me * W + dst) * EL + e));
  int send_start = 0;
  for (int q = 0; q < ge; ++q) send_start += load_count(cnt + (me * ET + q));
  int group_start = 0, mtile0 = 0;
  for (int e2 = 0; e2 < e; ++e2) {
    const int rows = received_rows(cnt, W, EL, dst, e2);
    group_start += rows;
    mtile0 += (rows + BM - 1) / BM;
  }
  int within = 0;   // rows of the sources that precede this rank in dst's segment order
  for (int q = 0; q < r; ++q) within += load_count(cnt + ((((dst - q + W) % W) * W + dst) * EL + e));
  c.b_count[bi] = n;
  c.b_send_start[bi] = send_start;
  c.b_dst_row[bi] = group_start + within;
  c.b_dst_rel0[bi] = within;
  c.b_dst_mtile0[bi] = mtile0;
  c.b_dst_rank[bi] = dst;
  // units are (bucket, aligned block of SEND_ROWS destination rows); stored un-scanned for now
  c.b_unit_start[bi + 1] = (n > 0) ? ((within + n - 1) / SEND_ROWS - within / SEND_ROWS + 1) : 0;
  return !(n > 0 && group_start + within + n > cap_rows) && n >= 0;
}

// Builds the sender tables and this rank's group sizes from the all-ranks
// routing counts (`cnt` = counts_all[src][dst][e], staged in shared memory).  Runs on every
// thread of the CTA.
__device__ __forceinline__ void build_dispatch_tables(ControlSmem& c, const b200_dispatch_args& d,
                                                      const int* cnt, int tid, int nthreads, WaitCtx& w) {
  const int W = d.world, EL = d.e_local, ET = W * EL, me = d.rank;
  for (int e = tid; e < EL; e += nthreads) c.g_rows[e] = received_rows(cnt, W, EL, me, e);
  for (int bi = tid; bi < ET; bi += nthreads) {
    if (!fill_bucket(c, cnt, W, EL, me, bi, d.cap_rows)) {
      report_status(w.status, ST_OVERFLOW);
      c.overflow = 1;
      *w.abort_flag = 1;
    }
  }
}

template <int EPI, bool FUSED, int CG, int NT>
__global__ void __launch_bounds__(FUSED ? NUM_THREADS_FUSED : NUM_THREADS_PLAIN, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a0,
                    const __grid_constant__ CUtensorMap tmap_a1,
                    const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_o, const b200_gemm_args ga,
                    const b200_dispatch_args da_in, const b200_combine_args ca_in,
                    const b200_router_args ra) {
  // Per-parity state: the iteration number lives in device memory (when iter_ptr is set), so
  // the same launch arguments serve every iteration and a captured graph can be replayed.
  b200_dispatch_args da = da_in;
  b200_combine_args ca = ca_in;
  uint32_t parity = 0;
  if constexpr (FUSED) {
    if (da.iter_ptr != nullptr) {
      const uint32_t it = __ldcg(da.iter_ptr);
      parity = it & 1u;
      da.epoch = it + 1u;
      if (parity) {
        da.counts_all = reinterpret_cast<const int*>(reinterpret_cast<const char*>(da.counts_all) + da.stride_counts);
        da.counts_flag = reinterpret_cast<const uint32_t*>(reinterpret_cast<const char*>(da.counts_flag) + da.stride_flag);
#pragma unroll
        for (int r = 0; r < B200_MAX_WORLD; ++r) {
          da.peer_recv[r] += da.stride_recv;
          da.peer_meta[r] += da.stride_meta;
          da.peer_ready[r] += da.stride_ready;
        }
      }
    }
  }
  if constexpr (EPI == B200_EPI_COMBINE) {
    if (ca.iter_ptr != nullptr && (__ldcg(ca.iter_ptr) & 1u))
      ca.row_meta = reinterpret_cast<const char*>(ca.row_meta) + ca.stride_meta;
  }
  const CUtensorMap& tmap_a = (FUSED && parity) ? tmap_a1 : tmap_a0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  using S = Geo<CG, NT>;
  constexpr int STAGES = S::STAGES;
  constexpr int STAGE_BYTES = S::STAGE_BYTES;
  uint8_t* stage_base = smem;
  uint8_t* staging = smem + STAGES * STAGE_BYTES;
  ControlSmem& c = *reinterpret_cast<ControlSmem*>(staging + STG_BYTES);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int nthreads = blockDim.x;
  const int G = FUSED ? da.e_local : ga.num_groups;
  const int TN = (ga.N + S::TILE_N - 1) / S::TILE_N;
  const int KB = (ga.K + BK - 1) / BK;
  const int gm = ga.group_m > 0 ? ga.group_m : 16;
  // CTA pair bookkeeping: both CTAs of a pair walk the same tile list; CTA `cta_rank`
  // owns rows [cta_rank*128, +128) of each 256-row tile and half of the weight rows.
  const uint32_t cta_rank = (CG == 2) ? cluster_ctarank() : 0u;
  const int sched_id = blockIdx.x / CG;
  const int sched_stride = gridDim.x / CG;

  WaitCtx w;
  w.abort_flag = &c.abort_flag;
  w.status = ga.status;
  w.budget_ns = ga.wait_budget_ns;

  // ---------------------------------------------------------------- set-up
  if (tid == 0) {
    c.abort_flag = 0;
    c.overflow = 0;
    c.total_units = 0;
    for (int i = 0; i < 64; ++i) c.ready_seen[i] = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&c.full[s], 1);
      mbar_init(&c.empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&c.tmem_full[a], 1);
      mbar_init(&c.tmem_empty[a], 128 * CG);   // every epilogue thread of the pair arrives
    }
    mbar_init(&c.drain, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (ga.tma_store) tma_prefetch_desc(&tmap_o);
  }
  if (warp == 1) {
    if constexpr (CG == 2) {
      tmem_alloc_pair(&c.tmem_base, TMEM_COLS);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(&c.tmem_base, TMEM_COLS);
      tmem_relinquish();
    }
  }
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();   // the peer's barriers exist before anyone signals them

  if constexpr (FUSED) {
    if (da.trace != nullptr && blockIdx.x == 0 && tid == 0) da.trace[0] = globaltimer_ns();
    // every rank's routing counts must have landed before offsets can be built
    if (tid < da.world) wait_flag_geq(da.counts_flag + tid, da.epoch, w, ST_TIMEOUT_COUNTS);
    __syncthreads();
    // One coalesced read of the peer-written table (world * experts ints, at most 4 KiB) into the
    // still idle epilogue staging buffer; the tables are then built from shared memory.
    int* cnt_s = reinterpret_cast<int*>(staging);
    if (!c.abort_flag) {
      const int ncnt = da.world * da.world * da.e_local;
      for (int i = tid; i < ncnt; i += nthreads) cnt_s[i] = __ldcg(da.counts_all + i);
    }
    __syncthreads();
    if (!c.abort_flag) build_dispatch_tables(c, da, cnt_s, tid, nthreads, w);
    __syncthreads();
    if (tid == 0) {
      const int ET = da.world * da.e_local;
      int acc = 0;
      c.b_unit_start[0] = 0;
      for (int b = 0; b < ET; ++b) {
        acc += c.b_unit_start[b + 1];
        c.b_unit_start[b + 1] = acc;
      }
      c.total_units = acc;
    }
    if (blockIdx.x == 0 && tid < da.e_local && da.group_rows_out != nullptr)
      da.group_rows_out[tid] = c.g_rows[tid];
  } else {
    for (int g = tid; g < G; g += nthreads) {
      int r = ga.group_rows != nullptr ? ga.group_rows[g] : ga.single_group_rows;
      c.g_rows[g] = r < 0 ? 0 : r;
    }
  }
  __syncthreads();
  if (warp == 0) scan_groups(c, G, lane, S::TM);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();

  // The group sizes come from device memory: when they add up to more rows than the activation
  // (and output) buffer holds, nothing is sent, computed or stored; the host reads the status.
  if (tid == 0 && c.g_row_start[G] > (FUSED ? static_cast<long long>(da.cap_rows) : ga.a_rows)) {
    report_status(w.status, ST_OVERFLOW);
    if (w.status != nullptr) atomicMax(w.status + 1, c.g_row_start[G]);   // rows that were needed
    c.overflow = 1;
    c.abort_flag = 1;
  }
  __syncthreads();

  const uint32_t tmem_base = c.tmem_base;
  const int total_tiles = c.total_sched * TN;
  int tile_first, tile_stride;
  tile_walk(total_tiles, sched_stride, sched_id, tile_first, tile_stride);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int cursor = 0, stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      bool ok = !c.abort_flag;
      // L2 eviction priorities (ga.l2_hints): bit 0 keeps the activation chunk that every N-tile
      // of the sweep re-reads, bit 1 lets the once-streamed weights leave first.
      const bool hinted = EPI != B200_EPI_ROUTER && (ga.l2_hints & 3) != 0;
      const uint64_t pol_a = (ga.l2_hints & 1) ? l2_policy_evict_last() : l2_policy_evict_normal();
      const uint64_t pol_b = (ga.l2_hints & 2) ? l2_policy_evict_first() : l2_policy_evict_normal();
      for (int idx = tile_first; ok && idx < total_tiles; idx += tile_stride) {
        int g, m, n;
        if (!decode_tile(c, G, TN, gm, idx, cursor, g, m, n)) break;
        const int half0 = m * S::TM + static_cast<int>(cta_rank) * BM;   // first row of my half
        const int row0 = c.g_row_start[g] + half0;
        if constexpr (FUSED) {
          const int expect = min(BM, c.g_rows[g] - half0);
          const int mt = c.g_mtile_start[g] + m * CG + static_cast<int>(cta_rank);
          // the same M-tile comes back once per N-tile: poll its counter only the first time
          if (expect > 0 && c.ready_seen[mt & 63] != mt + 1) {
            const uint32_t* ready = reinterpret_cast<const uint32_t*>(da.peer_ready[da.rank]) + mt;
            const uint64_t t_wait = da.trace != nullptr ? globaltimer_ns() : 0ull;
            if (!wait_flag_geq(ready, static_cast<uint32_t>(expect), w, ST_TIMEOUT_TILE_READY)) {
              ok = false;
              break;
            }
            fence_proxy_async();   // peer-written rows are read by the async proxy next
            c.ready_seen[mt & 63] = mt + 1;
            if (da.trace != nullptr) {   // overlap analysis: when did this tile become usable
              const uint64_t t_now = globaltimer_ns();
              if (mt < da.trace_tiles) atomicCAS(da.trace + 2 + mt, 0ull, t_now);   // first observer wins
              atomicAdd(da.trace + 1, t_now - t_wait);
            }
          }
        }
        if constexpr (EPI == B200_EPI_ROUTER) {
          // The router streams its activations once, in 128-byte pieces 2*K bytes apart (one
          // piece per row and k-block): poor DRAM page locality.  The rows of a tile are one
          // contiguous region, so ask L2 for it up front in large sequential requests; the
          // tiled loads below then hit L2.
          if (ga.a_base != nullptr) {
            const int rows_here = min(BM, c.g_rows[g] - half0);
            const size_t row_bytes = static_cast<size_t>(ga.K) * 2;
            const char* base = static_cast<const char*>(ga.a_base) + static_cast<size_t>(row0) * row_bytes;
            const size_t total = static_cast<size_t>(max(rows_here, 0)) * row_bytes;
            for (size_t off = 0; off < total; off += 32768)
              l2_prefetch_bulk(base + off, static_cast<uint32_t>(min(static_cast<size_t>(32768), total - off)));
          }
        }
        // first weight row of accumulator 0 for this CTA; accumulator 1 (wide tiles) is BN rows on
        const int brow = g * ga.N + n * S::TILE_N + static_cast<int>(cta_rank) * S::B_ROWS;
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait(&c.empty[stage], phase ^ 1u, w, ST_TIMEOUT_PIPE_EMPTY)) { ok = false; break; }
          uint8_t* sa = stage_base + stage * STAGE_BYTES;
          if (ga.l2_hints & 8) {
            // measurement aid (results are wrong): only every fourth k-block is fetched, the others
            // reuse whatever the stage holds -- shows what the operand traffic costs
            if ((kb & 3) != 0) {
              if (cta_rank == 0) mbar_arrive(&c.full[stage]);
              ++issued;
              if (++stage == STAGES) { stage = 0; phase ^= 1u; }
              continue;
            }
          }
          if constexpr (CG == 2) {
            // the pair leader's barrier collects the bytes of both CTAs' loads
            if (cta_rank == 0) mbar_expect_tx(&c.full[stage], STAGE_BYTES * 2);
            const uint32_t lead_bar = map_to_cta(&c.full[stage], 0);
            if (hinted) {
              tma_load_2d_pair_hint(sa, &tmap_a, lead_bar, kb * BK, row0, pol_a);
#pragma unroll
              for (int h = 0; h < NT; ++h)
                tma_load_2d_pair_hint(sa + A_STAGE_BYTES + h * S::B_HALF_BYTES, &tmap_b, lead_bar, kb * BK,
                                      brow + h * BN, pol_b);
            } else {
              tma_load_2d_pair(sa, &tmap_a, lead_bar, kb * BK, row0);
#pragma unroll
              for (int h = 0; h < NT; ++h)
                tma_load_2d_pair(sa + A_STAGE_BYTES + h * S::B_HALF_BYTES, &tmap_b, lead_bar, kb * BK,
                                 brow + h * BN);
            }
          } else if (hinted) {
            mbar_expect_tx(&c.full[stage], static_cast<uint32_t>(STAGE_BYTES));
            tma_load_2d_hint(sa, &tmap_a, &c.full[stage], kb * BK, row0, pol_a);
            tma_load_2d_hint(sa + A_STAGE_BYTES, &tmap_b, &c.full[stage], kb * BK, brow, pol_b);
          } else {
            // the router's weight box holds only mma_n rows (the host encodes its map that way)
            const uint32_t tx = (EPI == B200_EPI_ROUTER && ga.mma_n > 0)
                                    ? static_cast<uint32_t>(A_STAGE_BYTES + ga.mma_n * BK * 2)
                                    : static_cast<uint32_t>(STAGE_BYTES);
            mbar_expect_tx(&c.full[stage], tx);
            tma_load_2d(sa, &tmap_a, &c.full[stage], kb * BK, row0);
            tma_load_2d(sa + A_STAGE_BYTES, &tmap_b, &c.full[stage], kb * BK, brow);
          }
          ++issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      // Retire every load still in flight before shared memory is released.  In a CTA
      // pair the leader's barriers account for both CTAs' loads, and the pair leaves
      // together (cluster barrier at teardown), so only the leader drains.
      const int pending = (CG == 2 && cta_rank != 0) ? 0 : min(issued, STAGES);
      for (int i = 0; i < pending; ++i) {
        // walk back from the most recent issue
        int s = stage - 1 - i;
        uint32_t ph = phase;
        if (s < 0) { s += STAGES; ph ^= 1u; }
        WaitCtx wd = w;
        int no_abort = 0;
        wd.abort_flag = &no_abort;   // drain even when the CTA has given up
        mbar_wait(&c.full[s], ph, wd, ST_TIMEOUT_DRAIN);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0) {
      const uint32_t idesc = make_idesc_bf16_f32(S::TM, ga.mma_n > 0 ? ga.mma_n : BN);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = !c.abort_flag;
      for (int idx = tile_first; ok && idx < total_tiles; idx += tile_stride, ++it) {
        if constexpr (NT == 2) {
          // Wide tile: accumulator h takes weight rows [h*256, +256) of the tile.  Accumulator 0 must
          // be free before the first MMA; accumulator 1's MMAs may trail by up to LAG k-blocks
          // (their stages stay occupied meanwhile), which covers the time the epilogue of the
          // previous tile still needs for its second half.
          constexpr int LAG = STAGES - 1;
          const uint32_t par = static_cast<uint32_t>(it & 1);
          if (!mbar_wait(&c.tmem_empty[0], par ^ 1u, w, ST_TIMEOUT_TMEM_EMPTY)) break;
          tc_fence_after_sync();
          bool h1_free = false;
          int deferred = 0, dstage = stage, dkb = 0;      // k-blocks whose accumulator-1 MMAs are pending
          for (int kb = 0; kb < KB; ++kb) {
            if (!mbar_wait(&c.full[stage], phase, w, ST_TIMEOUT_PIPE_FULL)) { ok = false; break; }
            tc_fence_after_sync();
            {
              const uint32_t sa = smem_u32(stage_base + stage * STAGE_BYTES);
              const uint64_t adesc = make_smem_desc_sw128(sa);
              const uint64_t bdesc = make_smem_desc_sw128(sa + A_STAGE_BYTES);
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k)
                umma_bf16_ss_pair(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            ++deferred;
            if (!h1_free) {
              if (deferred >= LAG || kb == KB - 1) {
                if (!mbar_wait(&c.tmem_empty[1], par ^ 1u, w, ST_TIMEOUT_TMEM_EMPTY)) { ok = false; break; }
                h1_free = true;
              } else if (mbar_try_wait(&c.tmem_empty[1], par ^ 1u)) {
                h1_free = true;
              }
              if (h1_free) tc_fence_after_sync();
            }
            if (h1_free) {
              for (; deferred > 0; --deferred, ++dkb) {
                const uint32_t sa = smem_u32(stage_base + dstage * STAGE_BYTES);
                const uint64_t adesc = make_smem_desc_sw128(sa);
                const uint64_t bdesc = make_smem_desc_sw128(sa + A_STAGE_BYTES + S::B_HALF_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                  umma_bf16_ss_pair(tmem_base + BN, adesc + 2 * k, bdesc + 2 * k, idesc, (dkb | k) != 0 ? 1u : 0u);
                umma_commit_pair(&c.empty[dstage], 3);     // both accumulators have consumed the stage
                if (++dstage == STAGES) dstage = 0;
              }
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
          umma_commit_pair(&c.tmem_full[0], 3);
          continue;
        }
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&c.tmem_empty[acc], acc_phase ^ 1u, w, ST_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < KB; ++kb) {
          if (!mbar_wait(&c.full[stage], phase, w, ST_TIMEOUT_PIPE_FULL)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(stage_base + stage * STAGE_BYTES);
          const uint64_t adesc = make_smem_desc_sw128(sa);
          const uint64_t bdesc = make_smem_desc_sw128(sa + A_STAGE_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advancing 16 elements along K = 32 bytes = 2 descriptor units
            if constexpr (CG == 2)
              umma_bf16_ss_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
            else
              umma_bf16_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // frees the stage in both CTAs of a pair
          if constexpr (CG == 2) umma_commit_pair(&c.empty[stage], 3);
          else umma_commit(&c.empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if constexpr (CG == 2) umma_commit_pair(&c.tmem_full[acc], 3);
        else umma_commit(&c.tmem_full[acc]);
      }
      // all MMAs issued by this thread must retire before TMEM is freed
      if constexpr (CG == 2) umma_commit_pair(&c.drain, 1);
      else umma_commit(&c.drain);
      WaitCtx wd = w;
      int no_abort = 0;
      wd.abort_flag = &no_abort;
      mbar_wait(&c.drain, 0, wd, ST_TIMEOUT_DRAIN);
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue
    constexpr int OUT_TILE = (EPI == B200_EPI_SILU_GATE) ? BN / 2 : BN;   // output cols per tile
    constexpr int PASSES = OUT_TILE / STG_COLS;
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    const int row_in_tile = q * 32 + lane;
    // this warp's 32 x 64 staging box; the 16-byte chunk j of row r sits at chunk j ^ (r & 7)
    // (the 128-byte swizzle of a TMA store box, and conflict-free for the accesses below)
    uint8_t* warp_stg = staging + q * STG_WARP_BYTES;
    uint8_t* my_stg = warp_stg + lane * STG_ROW_BYTES;
    const uint64_t pol_o = l2_policy_evict_first();
    bool store_pending = false;   // lane 0: a bulk store may still be reading the staging box
    int cursor = 0, it = 0;
    int pending_arrivals = 0;   // combine epilogue: rows stored for rank `lane`, not yet published
    // accumulators are handed back on the pair leader's barrier
    const uint32_t tmem_empty_addr[2] = {map_to_cta(&c.tmem_empty[0], 0), map_to_cta(&c.tmem_empty[1], 0)};
    for (int idx = tile_first; idx < total_tiles; idx += tile_stride, ++it) {
      int g, m, n;
      if (!decode_tile(c, G, TN, gm, idx, cursor, g, m, n)) break;
      // NT == 1: the two accumulators alternate from tile to tile; NT == 2: both belong to this tile
      const int acc_first = NT == 2 ? 0 : (it & 1);
      const uint32_t acc_phase = NT == 2 ? static_cast<uint32_t>(it & 1) : static_cast<uint32_t>((it >> 1) & 1);
      const int half0 = m * S::TM + static_cast<int>(cta_rank) * BM;
      const int rows_in_tile = min(BM, c.g_rows[g] - half0);      // may be <= 0 for the upper half
      const int row0 = c.g_row_start[g] + half0;
      bool valid = row_in_tile < rows_in_tile;

      // warp-uniform decision: the TMEM loads below need the whole warp
      const bool prof = ga.dbg != nullptr && blockIdx.x == 0 && warp == 2 && lane == 0;
      const uint64_t t_w0 = prof ? globaltimer_ns() : 0ull;
      const bool got = mbar_wait(&c.tmem_full[acc_first], acc_phase, w, ST_TIMEOUT_TMEM_FULL);
      if (!__all_sync(0xffffffffu, got)) break;
      if (prof) atomicAdd(ga.dbg + 0, globaltimer_ns() - t_w0);
      tc_fence_after_sync();
      // Row metadata is read only now: in the fused-dispatch build it is written by the
      // sending rank together with the row, and the accumulator being complete implies
      // that the producer has seen the tile's arrival count.
      unsigned long long my_dst = 0;     // byte address of this thread's output row
      float wgt = 1.0f;
      int dst_rank = -1;
      if constexpr (EPI == B200_EPI_COMBINE) {
        if (valid) {
          const uint2 meta = __ldcg(reinterpret_cast<const uint2*>(ca.row_meta) + row0 + row_in_tile);
          dst_rank = static_cast<int>(meta.x >> 24);
          const int slot = static_cast<int>(meta.x & 0xFFFFFFu);
          wgt = __uint_as_float(meta.y);
          if (dst_rank >= ca.world || slot >= ca.max_slots) {
            report_status(w.status, ST_BAD_INDEX);
            valid = false;
            dst_rank = -1;
          } else {
            my_dst = ca.peer_out[dst_rank] +
                     static_cast<unsigned long long>(slot) * ca.out_row_stride * 2ull;
          }
        }
      } else {
        my_dst = reinterpret_cast<unsigned long long>(ga.out) +
                 static_cast<unsigned long long>(row0 + row_in_tile) * ga.ldo * 2ull;
      }

#pragma unroll 1
      for (int hh = 0; hh < NT; ++hh) {
      const int acc = acc_first + hh;
      const int n_sub = n * NT + hh;        // 256-column accumulator index along N
      uint64_t t_p = prof ? globaltimer_ns() : 0ull;
      uint64_t t_math = 0, t_store = 0;
      const uint32_t t_acc = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;

      if constexpr (EPI == B200_EPI_ROUTER) {
        // One thread owns one token: its logits are the first E columns of the accumulator.
        const int E = ra.num_experts;
        float mx = -CUDART_INF_F;
        for (int c0 = 0; c0 < E; c0 += 32) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_acc + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (c0 + j < E)
              mx = fmaxf(mx, __uint_as_float(v[j]) + (ra.bias != nullptr ? __ldg(ra.bias + c0 + j) : 0.f));
        }
        TopK tk;
        tk.init();
        float sum = 0.f;
        for (int c0 = 0; c0 < E; c0 += 32) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_acc + c0, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            if (c0 + j < E) {
              const float lg = __uint_as_float(v[j]) + (ra.bias != nullptr ? __ldg(ra.bias + c0 + j) : 0.f);
              sum += __expf(lg - mx);
              tk.push(lg, c0 + j);
            }
          }
        }
        tc_fence_before_sync();
        if constexpr (CG == 2) mbar_arrive_cluster(tmem_empty_addr[acc]);
          else mbar_arrive(&c.tmem_empty[acc]);
        if (valid) {
          const float inv = 1.0f / sum;
          float p[ROUTER_MAX_K];
          float psum = 0.f;
#pragma unroll
          for (int j = 0; j < ROUTER_MAX_K; ++j) {
            p[j] = (j < ra.topk) ? __expf(tk.v[j] - mx) * inv : 0.f;
            psum += p[j];
          }
          const float scale = ra.renorm ? 1.0f / psum : 1.0f;
          const size_t o = static_cast<size_t>(row0 + row_in_tile) * ra.topk;
#pragma unroll
          for (int j = 0; j < ROUTER_MAX_K; ++j) {
            if (j < ra.topk) {
              ra.topk_idx[o + j] = tk.i[j];
              ra.topk_w[o + j] = p[j] * scale;
            }
          }
        }
        continue;
      }

#pragma unroll 1
      for (int p = 0; p < PASSES; ++p) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int cc = p * STG_COLS + h * 32;
          uint32_t v[32];
          uint32_t packed[16];
          if constexpr (EPI == B200_EPI_SILU_GATE) {
            uint32_t u[32];
            tmem_ld_32x32b_x32(t_acc + cc, v);             // gate block
            tmem_ld_32x32b_x32(t_acc + BN / 2 + cc, u);    // up block
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float a0 = silu_f(__uint_as_float(v[2 * i])) * __uint_as_float(u[2 * i]);
              const float a1 = silu_f(__uint_as_float(v[2 * i + 1])) * __uint_as_float(u[2 * i + 1]);
              packed[i] = pack_bf16x2(a0, a1);
            }
          } else {
            tmem_ld_32x32b_x32(t_acc + cc, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              packed[i] = pack_bf16x2(__uint_as_float(v[2 * i]) * wgt,
                                      __uint_as_float(v[2 * i + 1]) * wgt);
            }
          }
          if (h == 0 && store_pending) {   // the previous pass's bulk store must have read the box
            bulk_wait_group_read<0>();
            store_pending = false;
          }
          if (h == 0) __syncwarp();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            *reinterpret_cast<uint4*>(my_stg + (((h * 4 + i) ^ (lane & 7)) << 4)) =
                make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
          }
        }
        if (prof) { const uint64_t t2 = globaltimer_ns(); t_math += t2 - t_p; t_p = t2; }
        if (p == PASSES - 1) {
          // every TMEM read of this accumulator is done: hand it back to the MMA warp
          tc_fence_before_sync();
          if constexpr (CG == 2) mbar_arrive_cluster(tmem_empty_addr[acc]);
          else mbar_arrive(&c.tmem_empty[acc]);
        }
        const int box_col0 = n_sub * OUT_TILE + p * STG_COLS;
        if (EPI != B200_EPI_COMBINE && ga.tma_store && rows_in_tile >= (q + 1) * 32) {
          // all 32 rows of this warp are rows of the group: one bulk tensor store writes the box
          // (columns past the output width are clipped by the tensor map)
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && box_col0 < ga.n_out) {
            if (ga.l2_hints & 4) tma_store_2d_hint(&tmap_o, warp_stg, box_col0, row0 + q * 32, pol_o);
            else tma_store_2d(&tmap_o, warp_stg, box_col0, row0 + q * 32);
            bulk_commit_group();
            store_pending = true;
          }
          if (prof) { const uint64_t t2 = globaltimer_ns(); t_store += t2 - t_p; t_p = t2; }
          continue;
        }
        __syncwarp();
        // ragged tile or scattered rows: coalesced write-out, 8 lanes cover one 128-byte row
        // segment, 4 rows per step
        const int col0 = box_col0 + (lane & 7) * 8;
#pragma unroll
        for (int rr = 0; rr < 8; ++rr) {
          const int r = rr * 4 + (lane >> 3);
          const unsigned long long dst = __shfl_sync(0xffffffffu, my_dst, r);
          const int rvalid = __shfl_sync(0xffffffffu, valid ? 1 : 0, r);
          if (rvalid && col0 < ga.n_out) {
            const uint4 val = *reinterpret_cast<const uint4*>(
                warp_stg + r * STG_ROW_BYTES + (((lane & 7) ^ (r & 7)) << 4));
            st_16(reinterpret_cast<void*>(dst + static_cast<unsigned long long>(col0) * 2ull), val);
          }
        }
        __syncwarp();
        if (prof) { const uint64_t t2 = globaltimer_ns(); t_store += t2 - t_p; t_p = t2; }
      }
      if (prof) {
        atomicAdd(ga.dbg + 1, t_math);
        atomicAdd(ga.dbg + 2, t_store);
        atomicAdd(ga.dbg + 3, 1ull);
      }

      if constexpr (EPI == B200_EPI_COMBINE) {
        // One arrival count per (row, n-tile).  The receiver only acts on the grand total,
        // so the counts are kept per destination rank (lane r of the warp keeps rank r's)
        // and published once, after this warp's last tile: a system-scope fence per tile
        // would stall the epilogue longer than a short-K tile takes to compute.
        const int cnt_rank = (n_sub * OUT_TILE < ga.n_out) ? dst_rank : -1;   // a half past the output width
        const unsigned grp = __match_any_sync(0xffffffffu, cnt_rank);
        const int leader_cnt = (cnt_rank >= 0 && lane == (__ffs(grp) - 1)) ? __popc(grp) : 0;
#pragma unroll
        for (int r = 0; r < B200_MAX_WORLD; ++r) {
          // sum over the (at most one per group) leaders whose destination is rank r
          const unsigned m = __ballot_sync(0xffffffffu, leader_cnt > 0 && cnt_rank == r);
          if (m != 0u) {
            const int c2 = __shfl_sync(0xffffffffu, leader_cnt, __ffs(m) - 1);
            if (lane == r) pending_arrivals += c2;
          }
        }
      }
      }   // accumulators of the tile
    }
    if (store_pending) bulk_wait_group<0>();   // shared memory stays allocated until the stores are done
    if constexpr (EPI == B200_EPI_COMBINE) {
      __syncwarp();
      if (lane < ca.world && pending_arrivals > 0) {
        fence_acq_rel_sys();
        red_add_release_sys(reinterpret_cast<uint32_t*>(ca.peer_arrived[lane]),
                            static_cast<uint32_t>(pending_arrivals));
      }
    }
  } else {
    // ------------------------------------------------------------ token senders
    if constexpr (FUSED) {
      const int stid = tid - NUM_THREADS_PLAIN;   // index inside the sender group
      const int swarp = stid >> 5;
      const int ET = da.world * da.e_local;
      const int total_units = c.overflow ? 0 : c.total_units;   // uniform: written during set-up only
      const int k16 = ga.K / 8;                 // 16-byte chunks per token row
      int bcur = 0;
      // The loop bound is uniform over the sender warps (they meet at a
      // named barrier per unit), so it must not depend on the abort flag.
      for (int u = blockIdx.x; u < total_units; u += gridDim.x) {
        while (bcur < ET && u >= c.b_unit_start[bcur + 1]) ++bcur;
        if (bcur >= ET) break;
        const int j = u - c.b_unit_start[bcur];
        const int rel0 = c.b_dst_rel0[bcur];
        const int nrows = c.b_count[bcur];
        const int blk = rel0 / SEND_ROWS + j;    // aligned row block inside the destination expert
        const int tile = blk / (BM / SEND_ROWS); // the 128-row M-tile whose counter it feeds
        const int p_lo = max(0, blk * SEND_ROWS - rel0);
        const int p_hi = min(nrows, (blk + 1) * SEND_ROWS - rel0);
        const int dst = c.b_dst_rank[bcur];
        const int send0 = c.b_send_start[bcur];
        const int drow0 = c.b_dst_row[bcur];
        uint8_t* recv = reinterpret_cast<uint8_t*>(da.peer_recv[dst]);
        uint2* meta = reinterpret_cast<uint2*>(da.peer_meta[dst]);
        for (int p = p_lo + swarp; p < p_hi; p += SENDER_WARPS) {
          const int flat = __ldg(da.send_order + send0 + p);
          const int t = flat / da.topk;
          const int drow = drow0 + p;
          if (t < 0 || t >= da.num_tokens || drow >= da.cap_rows) {
            if (lane == 0) report_status(w.status, ST_BAD_INDEX);
            continue;
          }
          const uint4* src = reinterpret_cast<const uint4*>(da.x) + static_cast<size_t>(t) * k16;
          uint4* out = reinterpret_cast<uint4*>(recv + static_cast<size_t>(drow) * ga.K * 2);
          for (int i = lane; i < k16; i += 256) {
            uint4 v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (i + 32 * j < k16) v[j] = ld_nc_16(src + i + 32 * j);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (i + 32 * j < k16) st_16(out + i + 32 * j, v[j]);
          }
          if (lane == 0) {
            uint2 mv;
            // the row's position in this rank's packed send order: results come back to that
            // position, so the rows of one (destination, expert) bucket return to consecutive
            // addresses (sequential remote writes) instead of to scattered token slots
            mv.x = (static_cast<uint32_t>(da.rank) << 24) | static_cast<uint32_t>(send0 + p);
            mv.y = __float_as_uint(__ldg(da.topk_weight + flat));
            meta[drow] = mv;
          }
        }
        // all sender warps have stored their rows of this unit
        asm volatile("bar.sync 1, %0;" ::"n"(SENDER_WARPS * 32) : "memory");
        if (stid == 0 && !da.drop_signal) {
          // Only rows that were stored are announced, and only into the counter array's bounds
          // (rows past the receive capacity were skipped above and reported).
          const int mt = c.b_dst_mtile0[bcur] + tile;
          const int stored = min(p_hi, da.cap_rows - drow0) - p_lo;
          if (mt >= da.cap_mtiles) {
            report_status(w.status, ST_BAD_INDEX);
          } else if (stored > 0) {
            uint32_t* ctr = reinterpret_cast<uint32_t*>(da.peer_ready[dst]) + mt;
            if (dst == da.rank) {       // rows and counter are in this GPU's memory
              fence_acq_rel_gpu();
              red_add_release_gpu(ctr, static_cast<uint32_t>(stored));
            } else {
              fence_acq_rel_sys();
              red_add_release_sys(ctr, static_cast<uint32_t>(stored));
            }
            if (da.trace != nullptr && dst == da.rank && mt < da.trace_tiles)
              da.trace[2 + da.trace_tiles + mt] = globaltimer_ns();
          }
        }
      }
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before_sync();
  __syncthreads();
  if constexpr (CG == 2) cluster_sync_all();   // the leader's MMAs read both CTAs' shared memory
  if (warp == 1) {
    tc_fence_after_sync();
    if constexpr (CG == 2) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

// Row-major bf16 matrix [rows, cols]; box = [box_rows, 64 columns]; 128-byte swizzle.
static int make_tmap_bf16(CUtensorMap* tm, const void* base, long long rows, long long cols,
                          int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (cols * 2) % 16 != 0 || rows <= 0) return -2;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

// Error code of launch_variant when not even one CTA (pair) of the variant can be resident.
constexpr int ERR_NOT_RESIDENT = -18;

template <int EPI, bool FUSED, int CG, int NT>
static int launch_variant(const CUtensorMap& ta, const CUtensorMap& ta1, const CUtensorMap& tb,
                          const CUtensorMap& to, const b200_gemm_args& ga,
                          const b200_dispatch_args& da, const b200_combine_args& ca,
                          const b200_router_args& ra, int ctas, cudaStream_t stream) {
  static bool configured = false;
  static int resident_clusters = -1;
  auto kern = grouped_gemm_kernel<EPI, FUSED, CG, NT>;
  constexpr int smem = Geo<CG, NT>::SMEM_BYTES;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(CG == 2 ? (ctas / 2) * 2 : ctas, 1, 1);
  cfg.blockDim = dim3(FUSED ? NUM_THREADS_FUSED : NUM_THREADS_PLAIN, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  // The kernel is persistent and its CTAs wait on one another (sender work is strided over the
  // whole grid; consumers here and on other ranks poll for it), so every CTA must be resident
  // at once: the grid is clamped to what this context can hold (asked once per variant).
  if (resident_clusters < 0) {
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
      (void)cudaGetLastError();
      n = 0;
    }
    resident_clusters = n;
  }
  if (resident_clusters < 1) return ERR_NOT_RESIDENT;
  if (static_cast<int>(cfg.gridDim.x) > resident_clusters * CG) cfg.gridDim.x = resident_clusters * CG;
  b200_count_launches(1);
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kern, ta, ta1, tb, to, ga, da, ca, ra));
}

template <int CG, int NT>
static int launch_geometry(int epi, int fused, const CUtensorMap& ta, const CUtensorMap& ta1,
                           const CUtensorMap& tb, const CUtensorMap& to, const b200_gemm_args& ga,
                           const b200_dispatch_args& d, const b200_combine_args& c,
                           const b200_router_args& r, int ctas, cudaStream_t st) {
  if (!fused) {
    switch (epi) {
      case B200_EPI_STORE: return launch_variant<B200_EPI_STORE, false, CG, NT>(ta, ta1, tb, to, ga, d, c, r, ctas, st);
      case B200_EPI_SILU_GATE: return launch_variant<B200_EPI_SILU_GATE, false, CG, NT>(ta, ta1, tb, to, ga, d, c, r, ctas, st);
      case B200_EPI_COMBINE: return launch_variant<B200_EPI_COMBINE, false, CG, NT>(ta, ta1, tb, to, ga, d, c, r, ctas, st);
      case B200_EPI_ROUTER:
        if constexpr (CG == 1) return launch_variant<B200_EPI_ROUTER, false, 1, 1>(ta, ta1, tb, to, ga, d, c, r, ctas, st);
        break;
    }
  } else {
    switch (epi) {
      case B200_EPI_STORE: return launch_variant<B200_EPI_STORE, true, CG, NT>(ta, ta1, tb, to, ga, d, c, r, ctas, st);
      case B200_EPI_SILU_GATE: return launch_variant<B200_EPI_SILU_GATE, true, CG, NT>(ta, ta1, tb, to, ga, d, c, r, ctas, st);
      case B200_EPI_COMBINE: return launch_variant<B200_EPI_COMBINE, true, CG, NT>(ta, ta1, tb, to, ga, d, c, r, ctas, st);
    }
  }
  return -15;
}

}  // namespace b200

extern "C" {

// Launches the grouped GEMM.  `a`/`a_rows` describe the packed activation
// buffer (for the fused-dispatch build: this rank's receive buffer and its
// capacity), `w` is [G*N, K].  Returns 0 or a negative (descriptor) / positive
// (cudaError_t) error code.  Nothing is allocated.
//
// The kernel is persistent and (in the fused builds) its CTAs and the other ranks wait for
// one another: it needs its CTAs resident together, so it wants the SMs to itself.  The grid
// is `num_ctas` clamped to what the context can hold at once; CTA pairs fall back to single
// CTAs where no pair fits.
int b200_grouped_gemm(const void* a, long long a_rows, const void* w, int epi, int fused,
                      const b200_gemm_args* ga, const b200_dispatch_args* da,
                      const b200_combine_args* ca, const b200_router_args* ra, int num_ctas,
                      void* stream) {
  using namespace b200;
  if (ga == nullptr || ga->K % 8 != 0) return -10;
  if (epi != B200_EPI_ROUTER && (ga->N % 8 != 0 || ga->n_out % 8 != 0)) return -10;
  const int G = fused ? (da ? da->e_local : 0) : ga->num_groups;
  if (G <= 0 || G > B200_MAX_GROUPS) return -11;
  if (fused && (da == nullptr || da->world * da->e_local > B200_MAX_EXPERTS ||
                da->world > B200_MAX_WORLD || da->cap_rows > a_rows || da->cap_mtiles < 1))
    return -12;
  if (epi == B200_EPI_COMBINE && ca == nullptr) return -13;
  if (epi == B200_EPI_ROUTER && (ra == nullptr || ra->num_experts > BN || ra->num_experts < 1 ||
                                 ra->topk < 1 || ra->topk > ROUTER_MAX_K || ra->topk > ra->num_experts))
    return -16;
  if (ga->mma_n != 0 && (ga->mma_n % 16 != 0 || ga->mma_n < 16 || ga->mma_n > BN)) return -17;
  if (num_ctas <= 0) return -14;
  CUtensorMap ta, ta1, tb, to;
  int r = make_tmap_bf16(&ta, a, a_rows, ga->K, BM);
  if (r != 0) return r;
  // second parity copy of the receive buffer (fused build with device-side iteration state)
  const void* a1 = (fused && da != nullptr && da->iter_ptr != nullptr)
                       ? static_cast<const void*>(static_cast<const char*>(a) + da->stride_recv)
                       : a;
  r = make_tmap_bf16(&ta1, a1, a_rows, ga->K, BM);
  if (r != 0) return r;
  b200_dispatch_args dz;
  b200_combine_args cz;
  b200_router_args rz;
  memset(&dz, 0, sizeof(dz));
  memset(&cz, 0, sizeof(cz));
  memset(&rz, 0, sizeof(rz));
  const b200_router_args& r2 = ra ? *ra : rz;
  const b200_dispatch_args& d = da ? *da : dz;
  const b200_combine_args& c = ca ? *ca : cz;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  b200_gemm_args ga_auto = *ga;
  ga_auto.a_rows = a_rows;
  // EPI 0/1: boxes of 32 full rows x 64 columns leave through bulk tensor stores when the
  // output rows are 16-byte aligned; ragged boxes take the per-lane path.
  to = ta;
  const bool plain_out = epi == B200_EPI_STORE || epi == B200_EPI_SILU_GATE;
  if (plain_out && ga->tma_store >= 0 && ga->out != nullptr && ga->ldo >= ga->n_out &&
      (ga->ldo * 2) % 16 == 0 && (reinterpret_cast<uintptr_t>(ga->out) & 15u) == 0) {
    EncodeTiledFn enc = get_encode_fn();
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(ga->n_out), static_cast<cuuint64_t>(a_rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ga->ldo) * 2};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(STG_COLS), 32u};
    cuuint32_t estr[2] = {1, 1};
    ga_auto.tma_store =
        (enc != nullptr &&
         enc(&to, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ga->out, dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
            ? 1
            : 0;
    if (!ga_auto.tma_store) to = ta;
  } else {
    ga_auto.tma_store = 0;
  }
  bool pair = ga->cta_pair != 0 && num_ctas >= 2 && epi != B200_EPI_ROUTER;
  for (int attempt = 0; attempt < 2; ++attempt) {
    int b_box = pair ? BN / 2 : BN;
    if (epi == B200_EPI_ROUTER && ga->mma_n > 0) b_box = ga->mma_n;   // few experts: a short weight box
    r = make_tmap_bf16(&tb, w, static_cast<long long>(G) * ga->N, ga->K, b_box);
    if (r != 0) return r - 10;
    // L2 blocking: a chunk of `group_m` M-tiles of A is swept across all N-tiles and should stay
    // resident in L2 meanwhile (126 MB L2 shared with the streamed weights and the output); larger
    // chunks re-read A from HBM once per N-tile, smaller ones re-read the weights more often.
    // Measured on B200 with K = 14336: chunks of 22-44 MB run 8-10 % faster than 117 MB chunks under
    // sustained (power-capped) load, while short cool runs prefer the largest chunk by 4-5 %;
    // about 48 MB per chunk, at most 16 M-tiles, is the compromise.
    if (ga->group_m <= 0) {
      const long long tile_bytes = static_cast<long long>(pair ? 2 * BM : BM) * ga->K * 2;
      long long gm = (48ll << 20) / (tile_bytes > 0 ? tile_bytes : 1);
      ga_auto.group_m = static_cast<int>(gm < 1 ? 1 : (gm > 16 ? 16 : gm));
    }
    ga_auto.cta_pair = pair ? 1 : 0;
    // Wide (512-column) tiles: fewer operand bytes per FLOP, no accumulator double buffering.
    // Only on request (wide_tiles > 0): measured on B200, the epilogue time they expose costs
    // more than the saved operand traffic gains on the layer shapes of this library.
    const bool wide = pair && ga->wide_tiles > 0 && ga->N >= 2 * BN;
    r = !pair ? launch_geometry<1, 1>(epi, fused, ta, ta1, tb, to, ga_auto, d, c, r2, num_ctas, st)
        : wide ? launch_geometry<2, 2>(epi, fused, ta, ta1, tb, to, ga_auto, d, c, r2, num_ctas, st)
               : launch_geometry<2, 1>(epi, fused, ta, ta1, tb, to, ga_auto, d, c, r2, num_ctas, st);
    if (r == ERR_NOT_RESIDENT && pair) {   // no pair fits in this context: single-CTA tiles
      pair = false;
      continue;
    }
    return r;
  }
  return r;
}

int b200_gemm_smem_bytes() { return b200::Geo<1>::SMEM_BYTES; }
int b200_gemm_smem_bytes_wide() { return b200::Geo<2, 2>::SMEM_BYTES; }

}  // extern "C"

// Sizes of the argument blocks, so that a binding in another language can check its mirrors.
extern "C" void b200_abi_sizes_gemm(int* out) {
  out[0] = static_cast<int>(sizeof(b200_gemm_args));
  out[1] = static_cast<int>(sizeof(b200_dispatch_args));
  out[2] = static_cast<int>(sizeof(b200_combine_args));
  out[3] = static_cast<int>(sizeof(b200_router_args));
}

// ---------------------------------------------------------------------------
// Host builds of the index arithmetic above, for tests that check tile coverage and the
// cross-rank row layout without a GPU.  They run the same decode_tile / fill_bucket code.
// ---------------------------------------------------------------------------
extern "C" int b200_debug_tile_order(const int* group_rows, int G, int TN, int group_m, int tile_rows,
                                     int* out_gmn, int max_tiles) {
  using namespace b200;
  if (G < 1 || G > B200_MAX_GROUPS || TN < 1 || group_m < 1 || (tile_rows != BM && tile_rows != 2 * BM))
    return -1;
  ControlSmem* c = new ControlSmem();
  int rows_acc = 0, sched_acc = 0, mt_acc = 0;
  for (int g = 0; g < G; ++g) {
    const int r = group_rows[g] < 0 ? 0 : group_rows[g];
    c->g_rows[g] = r;
    c->g_row_start[g] = rows_acc;
    c->g_mtile_start[g] = mt_acc;
    c->g_sched_start[g] = sched_acc;
    rows_acc += r;
    mt_acc += (r + BM - 1) / BM;
    sched_acc += (r + tile_rows - 1) / tile_rows;
  }
  c->g_row_start[G] = rows_acc;
  c->g_mtile_start[G] = mt_acc;
  c->g_sched_start[G] = sched_acc;
  c->total_sched = sched_acc;
  const int total = sched_acc * TN;
  int cursor = 0, written = 0;
  for (int idx = 0; idx < total && written < max_tiles; ++idx, ++written) {
    int g, m, n;
    if (!decode_tile(*c, G, TN, group_m, idx, cursor, g, m, n)) break;
    out_gmn[3 * written + 0] = g;
    out_gmn[3 * written + 1] = m;
    out_gmn[3 * written + 2] = n;
  }
  delete c;
  return written == total ? total : -2;
}

// owner[t] = the scheduler that takes tile t under tile_walk (every tile exactly once).
extern "C" int b200_debug_tile_walk(int total, int schedulers, int* owner) {
  if (total < 0 || schedulers < 1) return -1;
  for (int t = 0; t < total; ++t) owner[t] = -1;
  for (int sid = 0; sid < schedulers; ++sid) {
    int first, stride;
    b200::tile_walk(total, schedulers, sid, first, stride);
    if (stride < 1) return -2;
    for (int t = first; t < total; t += stride) {
      if (owner[t] != -1) return -3;
      owner[t] = sid;
    }
  }
  return 0;
}

// tables: [7][world * e_local] = count, send_start, dst_row, dst_rel0, dst_mtile0, dst_rank, units
extern "C" int b200_debug_dispatch_tables(const int* counts_all, int world, int e_local, int rank,
                                          int cap_rows, int* g_rows, int* tables) {
  using namespace b200;
  const int ET = world * e_local;
  if (world < 1 || world > B200_MAX_WORLD || ET > B200_MAX_EXPERTS || rank < 0 || rank >= world) return -1;
  ControlSmem* c = new ControlSmem();
  int ok = 1;
  for (int e = 0; e < e_local; ++e) g_rows[e] = received_rows(counts_all, world, e_local, rank, e);
  for (int bi = 0; bi < ET; ++bi) {
    if (!fill_bucket(*c, counts_all, world, e_local, rank, bi, cap_rows)) ok = 0;
    tables[0 * ET + bi] = c->b_count[bi];
    tables[1 * ET + bi] = c->b_send_start[bi];
    tables[2 * ET + bi] = c->b_dst_row[bi];
    tables[3 * ET + bi] = c->b_dst_rel0[bi];
    tables[4 * ET + bi] = c->b_dst_mtile0[bi];
    tables[5 * ET + bi] = c->b_dst_rank[bi];
    tables[6 * ET + bi] = c->b_unit_start[bi + 1];
  }
  delete c;
  return ok;
}

// Plain-C argument blocks shared by the host launchers and the device kernels
// of the MoE expert-parallel pipeline.  All pointers are device pointers in the
// calling rank's address space; "peer_*" arrays hold, per rank, the address at
// which that rank's copy of a symmetric buffer is mapped locally.
#pragma once
#include <stdint.h>

#define B200_MAX_WORLD 8
#define B200_MAX_GROUPS 128    // local experts per rank
#define B200_MAX_EXPERTS 128   // experts in the whole EP group

// Epilogue selectors of the grouped GEMM.
#define B200_EPI_STORE 0       // out[row, n]            = acc
#define B200_EPI_SILU_GATE 1   // out[row, n]            = silu(acc_gate) * acc_up
#define B200_EPI_COMBINE 2     // peer_out[src][slot, n] = weight(row) * acc
#define B200_EPI_ROUTER 3      // per row: softmax over the N logits, then top-k (idx, weight)

#ifdef __cplusplus
extern "C" {
#endif

// Routing / dispatch side of the fused "dispatch -> grouped GEMM" kernel.
typedef struct {
  int world;
  int rank;
  int e_local;
  int topk;
  int num_tokens;                 // T: tokens held by this rank
  const void* x;                  // [T, K] bf16, this rank's tokens
  const int* send_order;          // [T*topk] flat (t*topk+slot), sorted by (expert, t, slot)
  const float* topk_weight;       // [T*topk]
  const int* counts_all;          // [world(src)][world(dst)][e_local], written by peers
  const uint32_t* counts_flag;    // [world], epoch stamped by each source rank
  uint32_t epoch;                 // 1-based iteration stamp expected in counts_flag
  int cap_rows;                   // receive capacity (rows) of every rank
  int cap_mtiles;                 // entries of every rank's tile-ready counter array
  int drop_signal;                // testing aid: do not signal tile arrival
  unsigned long long peer_recv[B200_MAX_WORLD];   // bf16 [cap_rows, K]
  unsigned long long peer_meta[B200_MAX_WORLD];   // uint2 [cap_rows]: {src<<24|send position, weight}
  unsigned long long peer_ready[B200_MAX_WORLD];  // uint32 [cap_mtiles] rows landed per M-tile
  int* group_rows_out;            // [e_local] rows per local expert (for the second GEMM)
  // Iteration state kept on the device (so that a captured CUDA graph can be replayed):
  // when iter_ptr is set, the kernel reads it = *iter_ptr, uses epoch = it + 1 and adds
  // (it & 1) * stride to every per-parity pointer above (which then name parity 0).
  const uint32_t* iter_ptr;
  unsigned long long stride_counts;   // bytes between the two parity copies of counts_all
  unsigned long long stride_flag;     // ... of counts_flag
  unsigned long long stride_recv;     // ... of the receive buffer
  unsigned long long stride_meta;     // ... of the row metadata
  unsigned long long stride_ready;    // ... of the tile-ready counters
  unsigned long long* trace;      // optional [2 + 2*trace_tiles]: [0] kernel start (ns), [1] summed producer
                                  // stall (ns), [2 + t] time M-tile t was first seen complete,
                                  // [2 + trace_tiles + t] time this rank last published rows of its own tile t
  int trace_tiles;
} b200_dispatch_args;

// Combine side (epilogue of the second grouped GEMM).
typedef struct {
  int world;
  const void* row_meta;           // uint2 [rows]: {src<<24|row in the source's return buffer, weight}
  long long out_row_stride;       // elements between slot rows (= model dim)
  int max_slots;                  // T*topk of the largest rank (bounds check)
  unsigned long long peer_out[B200_MAX_WORLD];      // bf16 [T*topk, D] return buffer per rank (send order)
  unsigned long long peer_arrived[B200_MAX_WORLD];  // uint32 arrival counter per rank
  const uint32_t* iter_ptr;       // when set: row_meta names parity 0 and (it & 1) * stride_meta is added
  unsigned long long stride_meta;
} b200_combine_args;

typedef struct {
  int num_groups;                 // G
  int N;                          // weight rows per group
  int K;                          // reduction dim
  int n_out;                      // output columns (N, or N/2 when gated)
  int group_m;                    // M-tiles per scheduling chunk (L2 blocking)
  const int* group_rows;          // [G] rows per group (compact layout); null when fused-in
  void* out;                      // EPI 0/1 output base
  long long ldo;                  // EPI 0/1 output row stride (elements)
  int* status;                    // this rank's status word
  unsigned long long wait_budget_ns;
  int single_group_rows;          // used when group_rows is null: one group of this many rows
  int mma_n;                      // N of the MMA instruction (multiple of 16, <= 256); 0 = 256
  int cta_pair;                   // 1: two CTAs per MMA (cta_group::2, 256-row tiles)
  const void* a_base;             // activation buffer (same memory the A tensor map covers); used by
                                  // the router build to prefetch whole rows into L2
  long long a_rows;               // rows of the activation (and EPI 0/1 output) buffer: the group sizes
                                  // read on the device may not add up to more (filled by the launcher)
  int l2_hints;                   // L2 eviction priorities: 1 = keep activations (evict last), 2 = stream
                                  // weights (evict first), 4 = stream the EPI 0/1 output; 0 = none
  int tma_store;                  // EPI 0/1: full 32-row boxes leave through bulk tensor stores (set by
                                  // the launcher when the output is 16-byte aligned; -1 on entry forbids it)
  int wide_tiles;                 // CTA pairs: 1 = 512-column tiles (both accumulators per tile); 0 / -1 = off
  unsigned long long* dbg;        // optional [8] profiling words of CTA 0's first epilogue warp: summed ns of
                                  // [0] waiting for an accumulator, [1] reading TMEM + math + staging of
                                  // one accumulator, [2] its stores, [3] accumulators processed
} b200_gemm_args;

// Router epilogue: the accumulator row holds the logits of one token.
typedef struct {
  int num_experts;                // E (<= 256): columns of the accumulator that are logits
  int topk;                       // k (<= 8)
  int renorm;                     // renormalise the k weights to sum to 1
  const float* bias;              // [E] added to the logits, or null
  int* topk_idx;                  // [rows, k]
  float* topk_w;                  // [rows, k]
} b200_router_args;

// Launch accounting: every host launcher adds the kernels it launched; a benchmark reads the
// counter before and after its timed region.
void b200_count_launches(int n);
long long b200_launch_count(void);

#ifdef __cplusplus
}
#endif

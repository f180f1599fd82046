"""Host helpers: data generators, routing/packing front-end, buffer sets, comparisons, waits."""
from .buffers import (CountsBuffers, LocalHeap, ReturnBuffers, ShmemBuffers, TokenBuffers,
                      alloc_counts_buffers, alloc_return_buffers, alloc_shmem_buffers,
                      alloc_token_buffers, reset_counts_sync, reset_dispatch_flags,
                      reset_token_buf_debug, reset_token_sync)
from .compare import (all_ranks_ok, allreduce_max, allreduce_min, allreduce_sum, masked_stats,
                      sync_and_check)
from .gen import (gen_gated_expert_weights, gen_local_tokens, gen_local_weights, gen_router,
                  set_seed, zipf_expert_bias)
from .pack import (build_dst_offsets, build_expert_offsets, compute_capacity_device,
                   compute_capacity_from_pca,
                   route_and_pack, route_and_pack_padding_free)
from .waits import (WaitTimeout, expected_tiles, mark, spin_wait_counts_ready,
                    spin_wait_token_sync)

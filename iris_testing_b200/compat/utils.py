"""Names of the reference's ``utils.py`` (utils.py:20-261), backed by ``iris_testing_b200.utils``."""
from ..utils import (CountsBuffers, ShmemBuffers, TokenBuffers, alloc_counts_buffers,  # noqa: F401
                     alloc_shmem_buffers, alloc_token_buffers, build_expert_offsets,
                     compute_capacity_from_pca, gen_local_tokens, gen_local_weights, gen_router,
                     reset_counts_sync, reset_token_buf_debug, reset_token_sync,
                     route_and_pack_padding_free, set_seed)

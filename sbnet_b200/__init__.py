"""B200-native SBNet block ops: reduce_mask, sparse_gather, sparse_scatter[_var] (sm_100a CUDA behind a C ABI)."""

"""Out-of-place rotated modules (weights prefetched into work buffers while the current shard computes)."""

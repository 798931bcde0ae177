"""(batch x head) sharding across the GPUs of one box.

Every (batch, head) slice of attention is independent (the reference indexes them by
(b*H+h)*S*D, src/shaders/flash_attention.metal:70,181, and views [B*H,S,D] in
src/train/helpers.rs:137-140), so ranks take contiguous ranges of the flattened index and never
exchange data: no collective, no peer access."""


def shard_range(n_slices, world_size, rank):
    """[begin, end) of the slices rank `rank` owns: ceil-sized contiguous blocks, the tail ranks may get fewer or none."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError("rank must be in [0, world_size)")
    per = -(-n_slices // world_size)
    begin = min(n_slices, rank * per)
    return begin, min(n_slices, begin + per)

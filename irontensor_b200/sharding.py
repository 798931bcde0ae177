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


# ---------------------------------------------------------------- head-parallel projections
# With the heads of a layer split over the GPUs (each rank owns heads [h0, h1) and the K/V heads they read),
# the Q/K/V projections need only the rank's rows of Wq, Wk, Wv (src/train/forward.rs:101-103: out = heads *
# head_dim rows per weight), attention runs on the rank's heads with no exchange, and the output projection
# (forward.rs:146: attn [n, heads*head_dim] @ Wo.T) becomes a sum over ranks of partial products over each
# rank's COLUMNS of Wo: the one real exchange step on the path, an all-reduce of [n, hidden].

def head_shard(num_heads, num_kv_heads, world_size, rank):
    """(q_head_begin, q_head_end, kv_head_begin, kv_head_end) for `rank`: whole K/V groups, contiguous, so that every
    query head finds its K/V head on the same rank."""
    if num_heads % num_kv_heads:
        raise ValueError("num_heads must be divisible by num_kv_heads")
    group = num_heads // num_kv_heads
    kb, ke = shard_range(num_kv_heads, world_size, rank)
    return kb * group, ke * group, kb, ke


def qkv_weight_rows(num_heads, num_kv_heads, head_dim, world_size, rank):
    """Row ranges [begin, end) of Wq, Wk and Wv ([heads*head_dim, hidden] each) that `rank` multiplies by."""
    qb, qe, kb, ke = head_shard(num_heads, num_kv_heads, world_size, rank)
    return (qb * head_dim, qe * head_dim), (kb * head_dim, ke * head_dim), (kb * head_dim, ke * head_dim)


def out_projection_all_reduce(partial, group=None):
    """Sums the ranks' partial output projections in place (NCCL on GPUs, gloo in the CPU tests) and returns it.
    `partial` is this rank's attn[:, its heads] @ Wo[:, its columns].T, a torch tensor [n, hidden]."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    return partial


class SummedProjection:
    """A projection whose result is a sum over the ranks, with the reduce-scatter fused into the GEMM.

    Owns one [n, width] bf16 result buffer in symmetric memory (every rank allocates the same, and each can store
    into the others' over NVLink).  run() zeroes this rank's row block, meets the other ranks, runs the GEMM whose
    epilogue adds every row block of the partial product straight into its owner's buffer (it_linear_scatter_add: the
    exchange proceeds tile by tile under the GEMM's own math), meets the ranks again, and all-gathers the finished
    row blocks (NCCL), so that every rank ends with the full sum like out_projection_all_reduce -- at the price of
    one all-gather instead of an all-reduce after the GEMM.  n must be a multiple of the world size."""

    def __init__(self, n, width, group=None):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if n % self.world:
            raise ValueError("the number of rows must be a multiple of the world size")
        self.n, self.width, self.rows = n, width, n // self.world
        self.buf = symm.empty((n, width), dtype=torch.bfloat16, device=torch.device("cuda", torch.cuda.current_device()))
        self.handle = symm.rendezvous(self.buf, self.group)
        self.peers = [int(p) for p in self.handle.buffer_ptrs]
        self.own = self.buf[self.rank * self.rows:(self.rank + 1) * self.rows]

    def run(self, kind, a_ptr, w_ptr, in_dim, out_dim, gather=True):
        """kind 0: a [n, in] W[out, in]^T (width = out); kind 1: a [n, out] W [out, in] (width = in).  Returns the buffer
        (full sum on every rank), or with gather=False this rank's finished row block only."""
        import torch.distributed as dist
        from . import raw
        self.own.zero_()
        self.handle.barrier()          # nobody adds into a block that is not zeroed yet
        raw.linear_scatter_add(kind, self.n, in_dim, out_dim, a_ptr, w_ptr, self.peers, self.rows)
        self.handle.barrier()          # every rank's adds have landed
        if not gather:
            return self.own
        dist.all_gather_into_tensor(self.buf, self.own, group=self.group)
        return self.buf

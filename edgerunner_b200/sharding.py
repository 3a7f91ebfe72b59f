"""Multi-GPU partitioning of the decode path (one process per GPU, torch.distributed for the plumbing).

Attention is independent per (sequence, kv-head group, layer), so the path shards without any reduction:

* by sequence   -- rank r owns sequences [r*B/G, (r+1)*B/G): no communication at all;
* by kv head    -- rank r owns kv heads [r*Hkv/G, (r+1)*Hkv/G) and the q heads that attend to them; its cache
                   holds only those heads.  Per layer batch the ranks exchange their [B, Hq/G, 128] output
                   slices with one all-gather (NCCL over NVLink on GPUs, gloo in the CPU tests).

The reference is single-device (no collective call sites anywhere), so this module has no counterpart there.
"""
import torch
import torch.distributed as dist


def split_range(total, world, rank):
    """Contiguous, balanced [begin, end) of `total` items for `rank` of `world`."""
    base, rem = divmod(int(total), int(world))
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


class HeadShard:
    """kv-head sharding: which kv heads / q heads a rank owns."""

    def __init__(self, num_heads, num_kv_heads, world, rank):
        if num_kv_heads % world:
            raise ValueError("num_kv_heads %d is not divisible by world size %d" % (num_kv_heads, world))
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.group = num_heads // num_kv_heads
        self.world, self.rank = world, rank
        self.kv_begin, self.kv_end = split_range(num_kv_heads, world, rank)
        self.q_begin, self.q_end = self.kv_begin * self.group, self.kv_end * self.group
        self.local_kv_heads = self.kv_end - self.kv_begin
        self.local_heads = self.q_end - self.q_begin

    def slice_q(self, q):
        """q: [..., num_heads, head_dim] -> this rank's heads."""
        return q[..., self.q_begin:self.q_end, :]

    def slice_kv(self, kv):
        return kv[..., self.kv_begin:self.kv_end, :]


def all_gather_heads(local_out, group=None):
    """local_out: [..., local_heads, head_dim] (same shape on every rank) -> [..., world*local_heads, head_dim],
    rank slices concatenated along the head axis in rank order."""
    world = dist.get_world_size(group)
    if world == 1:
        return local_out
    local_out = local_out.contiguous()
    parts = [torch.empty_like(local_out) for _ in range(world)]
    dist.all_gather(parts, local_out, group=group)
    return torch.cat(parts, dim=-2)


def max_over_ranks(value, device=None, group=None):
    """Max of a python float over ranks (used for device-timed benchmark durations)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())

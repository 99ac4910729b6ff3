"""Row sharding of the path across the GPUs of one node.

Every operator on this path is row-wise over tokens (or token x expert rows): no row reads another.  So the
multi-GPU form is a partition of the token range with the small shared state (embedding table, norm weights)
replicated, no collective inside the chain, and one optional gather of outputs at the end
(torch.distributed all_gather: NCCL over NVLink on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations


def row_range(total_rows: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous, balanced partition: rank r owns [total * r // world, total * (r + 1) // world)."""
    if world < 1 or not 0 <= rank < world or total_rows < 0:
        raise ValueError("row_range: bad rank/world/total")
    return total_rows * rank // world, total_rows * (rank + 1) // world


def shard_sizes(total_rows: int, world: int) -> list[int]:
    return [row_range(total_rows, r, world)[1] - row_range(total_rows, r, world)[0] for r in range(world)]


def gather_rows(local, total_rows: int, group=None):
    """All-gather row shards (dim 0) produced under row_range into the full tensor on every rank.

    Shards may differ by one row; they are padded to the largest shard for the collective and trimmed after.
    Returns `local` unchanged when torch.distributed is not initialised (single GPU).
    """
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return local
    world = dist.get_world_size(group)
    sizes = shard_sizes(total_rows, world)
    if local.shape[0] != sizes[dist.get_rank(group)]:
        raise ValueError("gather_rows: local shard does not match row_range")
    if min(sizes) == max(sizes):  # equal shards: one collective straight into the result
        out = torch.empty((total_rows,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    biggest = max(sizes)
    padded = local
    if local.shape[0] != biggest:
        padded = torch.zeros((biggest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        padded[: local.shape[0]] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded.contiguous(), group=group)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)], dim=0)


def any_rank_failed(local_failed: bool, device, group=None) -> bool:
    """Host-side failure agreement: true on every rank if any rank reports a failed step (the gather is then
    skipped and the caller returns a status, as a failed chunk publishes nothing in the reference)."""
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return local_failed
    flag = torch.tensor([1 if local_failed else 0], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
    return bool(flag.item())

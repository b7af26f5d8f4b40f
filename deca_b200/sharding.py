"""Multi-GPU partitioning of the three operator families (one process per GPU).

The reference is single-GPU (its scripts always use device 0).  The operators shard without
any exchange inside the computation: GEMM along M (B replicated), attention along B*H,
row-wise operators along rows.  Each rank runs the unchanged single-GPU kernel on its shard;
the only collective is an optional all-gather of the outputs afterwards
(``torch.distributed``: NCCL on GPUs, gloo in the CPU tests).
"""

from __future__ import annotations


def shard_range(total: int, rank: int, world: int, multiple: int = 1) -> tuple[int, int]:
    """[begin, end) of rank's contiguous share of ``total`` units, in steps of ``multiple``.

    Shares differ by at most one step; trailing ranks may be empty when there are fewer steps
    than ranks.  ``total`` must be a multiple of ``multiple``."""
    if total % multiple != 0:
        raise ValueError(f"{total} is not a multiple of {multiple}")
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    steps = total // multiple
    base, extra = divmod(steps, world)
    begin = rank * base + min(rank, extra)
    end = begin + base + (1 if rank < extra else 0)
    return begin * multiple, end * multiple


def shard_gemm(a, b, rank: int, world: int, tile_m: int = 1):
    """Rank's (A rows, B) of C = A @ B split along M; returns (a_shard, b, (m0, m1))."""
    m0, m1 = shard_range(a.shape[0], rank, world, tile_m if a.shape[0] % tile_m == 0 else 1)
    return a[m0:m1], b, (m0, m1)


def shard_attention(q, k, v, rank: int, world: int):
    """Rank's heads of [B, H, S, D] tensors split along the flattened B*H axis.

    Returns the shards reshaped to [1, heads, S, D] and the (h0, h1) range."""
    B, H = q.shape[:2]
    h0, h1 = shard_range(B * H, rank, world)

    def take(t):
        return t.reshape(B * H, *t.shape[2:])[h0:h1].reshape(1, h1 - h0, *t.shape[2:])

    return take(q), take(k), take(v), (h0, h1)


def shard_rows(x, rank: int, world: int):
    r0, r1 = shard_range(x.shape[0], rank, world)
    return x[r0:r1], (r0, r1)


def all_gather_rows(local, total_rows: int, group=None):
    """Concatenates the ranks' row shards (possibly of unequal height) along dim 0.

    The shard heights are exchanged first, so any contiguous partition whose heights sum to
    ``total_rows`` works (equal heights take the single-buffer all-gather)."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    mine = torch.tensor([local.shape[0]], dtype=torch.int64, device=local.device)
    all_sizes = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(all_sizes, mine, group=group)
    sizes = [int(t.item()) for t in all_sizes]
    if sum(sizes) != total_rows:
        raise ValueError(f"shards hold {sum(sizes)} rows, expected {total_rows}")
    if len(set(sizes)) == 1:
        out = torch.empty((total_rows, *local.shape[1:]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    pad = max(sizes)
    buf = torch.zeros((pad, *local.shape[1:]), dtype=local.dtype, device=local.device)
    buf[: local.shape[0]] = local
    parts = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(parts, buf, group=group)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)], dim=0)

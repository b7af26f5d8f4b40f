"""Multi-GPU partitioning of the three operator families (one process per GPU).

The reference is single-GPU (its scripts always use device 0).  The operators shard without
any exchange inside the computation: GEMM along M (B replicated), attention along B*H,
row-wise operators along rows.  Each rank runs the unchanged single-GPU kernel on its shard;
the only collective is an optional all-gather of the outputs afterwards
(``torch.distributed``: NCCL on GPUs, gloo in the CPU tests).  For the M-sharded GEMM that
all-gather can instead be fused into the kernel: ``GatheredOutput`` holds every rank's copy of
the gathered C in peer-addressable memory and ``gemm_gather`` has the epilogue store each
output panel into all of them over NVLink (``deca_gemm16_gather``); ``attention_gather`` does
the same for the head-sharded attention output (``deca_fa_fwd_f16_gather``).
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


class GatheredOutput:
    """Every rank's copy of a gathered [world * rows_per_rank, cols] output, addressable from
    this process: ``local`` is this rank's copy (a tensor), ``ptrs[r]`` the device address of
    rank r's copy.

    ``GatheredOutput.symmetric`` allocates the copies in torch symmetric memory (one rendezvous
    over the process group; multicast binding is switched off, the kernel uses plain peer
    stores).  ``GatheredOutput.from_tensors`` wraps tensors that already live in one process,
    which is how several ranks are emulated on a single GPU."""

    def __init__(self, local, ptrs, rank: int, rows_per_rank: int, handle=None):
        self.local = local
        self.ptrs = [int(p) for p in ptrs]
        self.rank = rank
        self.world = len(self.ptrs)
        self.rows_per_rank = rows_per_rank
        self._handle = handle  # keeps the symmetric-memory mapping alive
        if local.data_ptr() != self.ptrs[rank]:
            raise ValueError("ptrs[rank] is not the local buffer")
        if local.shape[0] != self.world * rows_per_rank:
            raise ValueError(f"buffer holds {local.shape[0]} rows, expected {self.world} x {rows_per_rank}")

    @classmethod
    def symmetric(cls, rows_per_rank: int, cols: int, dtype, device, group=None):
        import os

        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        group = group if group is not None else dist.group.WORLD
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        local = symm_mem.empty((world * rows_per_rank, cols), dtype=dtype, device=device)
        handle = symm_mem.rendezvous(local, group)
        return cls(local, list(handle.buffer_ptrs), rank, rows_per_rank, handle)

    @classmethod
    def from_tensors(cls, copies, rank: int):
        rows = copies[rank].shape[0]
        if rows % len(copies) != 0:
            raise ValueError(f"{rows} rows do not split over {len(copies)} ranks")
        for t in copies:
            if t.shape != copies[rank].shape or t.dtype != copies[rank].dtype or not t.is_contiguous():
                raise ValueError("the copies must be contiguous tensors of one shape and dtype")
        return cls(copies[rank], [t.data_ptr() for t in copies], rank, rows // len(copies))

    def barrier(self, group=None):
        """All ranks' kernels launched so far have completed (device-wide on each rank), so
        every copy holds every shard.  Host-synchronising; outside timed regions."""
        import torch
        import torch.distributed as dist

        torch.cuda.synchronize(self.local.device)
        if dist.is_available() and dist.is_initialized():
            dist.barrier(group=group)


def gemm_gather(a_shard, b, out: GatheredOutput, cfg=None):
    """C_shard = a_shard @ b, stored by the kernel's epilogue into this rank's rows of every
    copy in ``out`` (see ``deca_gemm16_gather``).  Launches on the current stream and returns
    without synchronising; call ``out.barrier()`` before reading a gathered copy."""
    import ctypes

    import torch

    from . import native
    from .kernels.gemm_b200 import native_cfg

    m, k = a_shard.shape
    n = b.shape[1]
    if m != out.rows_per_rank or out.local.shape[1] != n or b.shape[0] != k:
        raise ValueError(f"shapes do not match: A {tuple(a_shard.shape)}, B {tuple(b.shape)}, "
                         f"gathered {tuple(out.local.shape)} over {out.world} ranks")
    if not (a_shard.is_contiguous() and b.is_contiguous()):
        raise ValueError("A shard and B must be contiguous")
    ptrs = (ctypes.c_void_p * out.world)(*out.ptrs)
    ncfg = native_cfg(cfg) if cfg is not None else None
    rc = native.lib().deca_gemm16_gather(
        native.DTYPE_CODE[str(a_shard.dtype).replace("torch.", "")], a_shard.data_ptr(), b.data_ptr(), ptrs, out.world, out.rank, m, n, k,
        ctypes.byref(ncfg) if ncfg is not None else None, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    native.check(rc, "deca_gemm16_gather")


def attention_gather(q, k, v, out: GatheredOutput, causal: bool = False, softmax_scale=None, cfg=None):
    """O = attention(q, k, v) for this rank's heads ([B, H, S, D] shards of the flattened B * H
    axis), stored by the kernel's epilogue into this rank's heads of every copy in ``out``, whose
    buffers are [world * B * H * S_q, D] (see ``deca_fa_fwd_f16_gather``).  Launches on the
    current stream without synchronising; call ``out.barrier()`` before reading a gathered copy."""
    import ctypes

    import torch

    from . import native
    from .kernels.flash_attn_b200 import native_cfg

    B, H, S_q, D = q.shape
    S_kv = k.shape[2]
    if out.rows_per_rank != B * H * S_q or out.local.shape[1] != D:
        raise ValueError(f"gathered buffer {tuple(out.local.shape)} over {out.world} ranks does not hold "
                         f"{B * H} heads of {S_q} x {D} per rank")
    if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()) or q.dtype != torch.float16:
        raise ValueError("q, k, v must be contiguous float16 tensors")
    scale = float(softmax_scale) if softmax_scale is not None else D ** -0.5
    ptrs = (ctypes.c_void_p * out.world)(*out.ptrs)
    if cfg is None:
        from .operators import FlashAttention

        cfg = FlashAttention(B, H, S_q, S_kv, D, causal=causal).default_config()
    ncfg = native_cfg(cfg)
    rc = native.lib().deca_fa_fwd_f16_gather(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), ptrs, out.world, out.rank, B, H, S_q, S_kv, D, ctypes.c_float(scale),
        int(causal), ctypes.byref(ncfg), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    native.check(rc, "deca_fa_fwd_f16_gather")

"""The fused GEMM + all-gather (and attention + all-gather) across real GPUs: one process per GPU, the gathered output in
torch symmetric memory, peer stores over NVLink.  Needs at least two GPUs (skipped otherwise;
the single-GPU emulation of the same path is in test_gemm_gather_gpu.py).  No rank leaves
early and no kernel waits on a peer: the only cross-rank synchronisation is the host barrier
after the launches."""

import os
import socket

import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, m_shard: int, n: int, k: int):
    import torch.distributed as dist

    from deca_b200 import native
    from deca_b200.sharding import GatheredOutput, gemm_gather

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        g = torch.Generator(device="cpu").manual_seed(4)
        a = (torch.rand(world * m_shard, k, generator=g) * 2 - 1).half().cuda()
        b = (torch.rand(k, n, generator=g) * 2 - 1).half().cuda()
        out = GatheredOutput.symmetric(m_shard, n, torch.float16, a.device)
        out.local.fill_(7.0)
        out.barrier()
        for _ in range(2):  # twice: the second launch overwrites identical values
            gemm_gather(a[rank * m_shard : (rank + 1) * m_shard].contiguous(), b, out)
        out.barrier()
        assert native.last_device_status() == (0, 0, 0)
        # the unsharded kernel on this rank gives the same bits for every row
        from deca_b200.operators import GEMMTC

        want = GEMMTC(world * m_shard, n, k)(a, b)
        torch.cuda.synchronize()
        assert torch.equal(out.local, want), f"rank {rank}: gathered copy differs from the unsharded result"
        out.barrier()

        # attention: two heads per rank, O gathered by the epilogue
        from deca_b200.operators import FlashAttention
        from deca_b200.sharding import attention_gather, shard_attention

        heads, S, D = 2 * world, 512, 128
        q, k, v = (torch.randn(1, heads, S, D, generator=g).half().cuda() for _ in range(3))
        o_all = GatheredOutput.symmetric(2 * S, D, torch.float16, q.device)
        o_all.local.fill_(7.0)
        o_all.barrier()
        qs, ks, vs, _ = shard_attention(q, k, v, rank, world)
        attention_gather(qs.contiguous(), ks.contiguous(), vs.contiguous(), o_all, causal=True)
        o_all.barrier()
        assert native.last_device_status() == (0, 0, 0)
        want_o = FlashAttention(1, heads, S, S, D, causal=True)(q, k, v)
        torch.cuda.synchronize()
        assert torch.equal(o_all.local.view(1, heads, S, D), want_o), f"rank {rank}: gathered O differs"
        o_all.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_gather_across_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(world, _free_port(), 384, 512, 320), nprocs=world, join=True)

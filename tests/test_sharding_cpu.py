"""The N > 1 host path on CPU: two gloo ranks shard each operator family, compute their shard
(with the CPU oracle standing in for the kernel), all-gather the outputs, and compare with the
unsharded result."""

import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_range_covers_everything():
    from deca_b200.sharding import shard_range

    for total, world, mult in ((65536, 8, 256), (1024, 8, 1), (10, 4, 1), (3, 8, 1), (16384, 3, 1), (1280, 4, 128)):
        spans = [shard_range(total, r, world, mult) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
            assert a1 == b0 and a0 <= a1
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= mult and all(sz % mult == 0 for sz in sizes)
    with pytest.raises(ValueError):
        shard_range(100, 0, 4, 64)
    with pytest.raises(ValueError):
        shard_range(100, 4, 4)


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    import oracle
    from deca_b200 import sharding

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        def bits(t):
            return t.contiguous().view(torch.int16).numpy().view(np.uint16)

        def tens(b):
            return torch.from_numpy(b.view(np.int16).copy()).view(torch.float16)

        g = torch.Generator().manual_seed(4)
        # GEMM along M (uneven shares: 5 row blocks over 2 ranks)
        a = (torch.rand(320, 96, generator=g) * 2 - 1).half()
        b = (torch.rand(96, 72, generator=g) * 2 - 1).half()
        a_s, b_s, _ = sharding.shard_gemm(a, b, rank, world, tile_m=64)
        c_s = tens(oracle.gemm16(bits(a_s), bits(b_s)))
        c = sharding.all_gather_rows(c_s, a.shape[0])
        ok_gemm = np.array_equal(bits(c), oracle.gemm16(bits(a), bits(b)))
        # attention along B*H
        qkv = [torch.randn(3, 2, 128, 64, generator=g).half() for _ in range(3)]
        qs, ks, vs, (h0, h1) = sharding.shard_attention(*qkv, rank, world)
        o_s = tens(oracle.attention(bits(qs), bits(ks), bits(vs), causal=True))
        o = sharding.all_gather_rows(o_s.reshape(h1 - h0, 128, 64), 6).reshape(3, 2, 128, 64)
        ok_attn = np.array_equal(bits(o), oracle.attention(*[bits(t) for t in qkv], causal=True))
        # rows
        x = (3 * torch.randn(37, 256, generator=g)).half()
        x_s, _ = sharding.shard_rows(x, rank, world)
        y = sharding.all_gather_rows(tens(oracle.softmax(bits(x_s))), 37)
        ok_rows = np.array_equal(bits(y), oracle.softmax(bits(x)))
        q.put((rank, ok_gemm, ok_attn, ok_rows))
    except Exception as e:  # noqa: BLE001
        q.put((rank, False, False, repr(e)))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_sharding_matches_unsharded():
    import torch.multiprocessing as mp

    import oracle

    oracle.build()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    assert all(r[1] and r[2] and r[3] for r in results), results


def test_gathered_output_host_checks():
    """GatheredOutput and the gather wrappers validate their arguments on the host before any
    launch (CPU tensors suffice: nothing is launched)."""
    import pytest
    import torch

    from deca_b200.sharding import GatheredOutput, attention_gather, gemm_gather

    copies = [torch.zeros(8, 16, dtype=torch.float16) for _ in range(2)]
    out = GatheredOutput.from_tensors(copies, 1)
    assert (out.world, out.rank, out.rows_per_rank) == (2, 1, 4)
    assert out.ptrs == [t.data_ptr() for t in copies] and out.local is copies[1]
    with pytest.raises(ValueError):
        GatheredOutput.from_tensors([torch.zeros(9, 16), torch.zeros(9, 16)], 0)  # 9 rows over 2 ranks
    with pytest.raises(ValueError):
        GatheredOutput.from_tensors([torch.zeros(8, 16), torch.zeros(8, 8)], 0)  # shapes differ
    with pytest.raises(ValueError):
        GatheredOutput(copies[0], [copies[1].data_ptr(), copies[0].data_ptr()], 0, 4)  # ptrs[rank] is not local
    a = torch.zeros(5, 32, dtype=torch.float16)  # 5 rows, but a rank's share is 4
    b = torch.zeros(32, 16, dtype=torch.float16)
    with pytest.raises(ValueError):
        gemm_gather(a, b, out)
    with pytest.raises(ValueError):
        gemm_gather(a[:4], torch.zeros(32, 8, dtype=torch.float16), out)  # N does not match the gathered buffer
    q = torch.zeros(1, 1, 4, 8, dtype=torch.float16)  # 4 rows of 8: the buffer holds 16 columns
    with pytest.raises(ValueError):
        attention_gather(q, q, q, out)

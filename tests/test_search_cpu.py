"""CPU tests of the config search (Solver + cost model), the kernel-spec build flow in worker
processes, and the log-record format of the CLIs."""

import os
import re

import pytest


@pytest.fixture(scope="module")
def arch():
    from deca_b200.arch.B200 import B200

    return B200()


def test_every_gemm_solution_is_valid_and_ranked(arch):
    from deca_b200.cost_model.CostModel import gemm_tc_score, rank_gemm_configs
    from deca_b200.kernels.gemm_b200 import check_config, default_config
    from deca_b200.Solver import solve_gemm_tc

    for shape in ((4096, 4096, 4096), (2048, 2048, 2048), (65536, 8192, 8192), (64, 80, 96), (300, 264, 328)):
        cfgs = solve_gemm_tc(arch, *shape)
        assert cfgs and len(set(cfgs)) == len(cfgs)
        for c in cfgs:
            check_config(c, *shape)
            assert gemm_tc_score(c, arch, *shape) > 0
        ranked = rank_gemm_configs(cfgs, arch, *shape, top_n=24)
        assert len(ranked) == min(24, len(cfgs))
        d = default_config(*shape)
        assert d in cfgs
    # large squares: the model's favourite is the tile shape measured best on B200
    top3 = rank_gemm_configs(solve_gemm_tc(arch, 8192, 8192, 8192), arch, 8192, 8192, 8192)[:3]
    assert all((c.BM, c.BN) == (256, 256) for c in top3)
    # ... in groups of 8 tile rows, the one-CTA tile first and the CTA-pair tile among the first three
    # (either leads by 1 - 3 % depending on the GPU once the kernel runs at the power limit)
    assert (top3[0].cta_group, top3[0].raster) == (1, 8) and any(c.cta_group == 2 and c.raster == 8 for c in top3)
    # at 4096^3, where wave tails leave power to spare, the pair tile leads
    assert rank_gemm_configs(solve_gemm_tc(arch, 4096, 4096, 4096), arch, 4096, 4096, 4096)[0].cta_group == 2
    # fp16-accumulate call sites get the one-CTA, whole-tile part of the same tile space with fp16 accumulators
    from dataclasses import replace

    from deca_b200.operators import GEMMTC

    f16 = solve_gemm_tc(arch, 4096, 4096, 4096, acc_f16=True, acc_splits=2)
    f32 = [c for c in solve_gemm_tc(arch, 4096, 4096, 4096) if c.cta_group == 1 and not c.stream_k]
    assert f16 and all(c.acc_f16 for c in f16)
    assert {replace(c, acc_f16=False) for c in f16} == set(f32)
    op16, op32 = GEMMTC(4096, 4096, 4096, acc="fp16", acc_splits=2), GEMMTC(4096, 4096, 4096)
    assert op16.is_valid(f16[0]) and not op16.is_valid(f32[0]) and not op32.is_valid(f16[0])
    assert op16.default_config().acc_f16 and not op32.default_config().acc_f16
    assert str(f16[0]).endswith(",acc_f16=1") and "acc_f16" not in str(f32[0])


def test_every_attention_solution_is_valid(arch):
    from deca_b200.cost_model.CostModel import rank_fa_configs
    from deca_b200.kernels.flash_attn_b200 import check_config
    from deca_b200.Solver import solve_flash_attn

    for shape in ((4, 16, 4096, 4096, 128), (4, 16, 4096, 4096, 64), (1, 2, 128, 640, 128), (32, 32, 8192, 8192, 128)):
        cfgs = solve_flash_attn(arch, *shape)
        assert cfgs
        for c in cfgs:
            check_config(c, shape[2], shape[3], shape[4])
        for causal in (False, True):
            if causal and shape[2] != shape[3]:
                continue
            assert rank_fa_configs(cfgs, arch, shape, causal)[0] in cfgs
    # measured on B200: two Q tiles per CTA, 128-key tiles, P in tensor memory win at both head dims
    for d in (128, 64):
        best = rank_fa_configs(solve_flash_attn(arch, 4, 16, 4096, 4096, d), arch, (4, 16, 4096, 4096, d))[0]
        assert (best.Bc, best.q_tiles, best.p_tmem, best.stages) == (128, 2, True, 4), best
    # a 128-row problem cannot use the two-tile schedule
    assert rank_fa_configs(solve_flash_attn(arch, 1, 1, 128, 128, 64), arch, (1, 1, 128, 128, 64))[0].q_tiles == 1


def test_every_rowwise_solution_is_valid(arch):
    from deca_b200.cost_model.CostModel import rank_rowwise_configs
    from deca_b200.kernels.rowwise_b200 import check_config
    from deca_b200.Solver import solve_rowwise

    for op in ("softmax", "rmsnorm"):
        for shape in ((16384, 4096), (4096, 1024), (1024, 128256), (3, 1000)):
            cfgs = solve_rowwise(arch, op, *shape)
            assert cfgs, (op, shape)
            for c in cfgs:
                check_config(c, op, *shape, "float16")
            top = rank_rowwise_configs(cfgs, arch, op, *shape, top_n=3)
            assert all(t in cfgs for t in top)
    # measured on B200 over the hidden-size grid: register mode, 64 elements per thread, one row per CTA
    top = rank_rowwise_configs(solve_rowwise(arch, "softmax", 16384, 4096), arch, "softmax", 16384, 4096)[0]
    assert (top.mode, top.threads_per_row, top.rows_per_block, top.vec) == ("reg", 64, 1, 8)
    top = rank_rowwise_configs(solve_rowwise(arch, "rmsnorm", 65536, 8192), arch, "rmsnorm", 65536, 8192)[0]
    assert (top.mode, top.threads_per_row, top.vec) == ("reg", 128, 8)
    # vocabulary rows: the two-pass mode ahead of the one-pass cluster mode (measured 4.2 - 5.1 against 3.0 - 3.8 TB/s)
    ranked = rank_rowwise_configs(solve_rowwise(arch, "softmax", 4096, 128256), arch, "softmax", 4096, 128256)
    assert ranked[0].mode == "twopass" and any(c.mode == "cluster" for c in ranked)
    assert (ranked[0].threads_per_row, ranked[0].hint) == (512, True)  # measured 4.7 TB/s; 256 threads 4.3
    # 32000 columns: 256 threads with two chunks per iteration (measured best) among the first three
    top3 = rank_rowwise_configs(solve_rowwise(arch, "softmax", 8192, 32000), arch, "softmax", 8192, 32000)[:3]
    assert any((c.mode, c.threads_per_row, c.unroll, c.hint) == ("twopass", 256, 2, True) for c in top3)
    # problems that fit in L2: no cache hints, and not one tiny CTA per 2 KB row
    top = rank_rowwise_configs(solve_rowwise(arch, "softmax", 16384, 1024), arch, "softmax", 16384, 1024)[:3]
    assert not top[0].hint and any(c.rows_per_block > 1 for c in top)
    # the persistent bulk-copy mode does not lead on problems that stream for a few microseconds
    assert rank_rowwise_configs(solve_rowwise(arch, "softmax", 4096, 2048), arch, "softmax", 4096, 2048)[0].mode == "reg"
    # rows that cannot live in registers fall back to the two-pass mode
    assert all(c.mode == "twopass" for c in solve_rowwise(arch, "softmax", 1024, 1 << 20))


def _crash(*args):
    os._exit(3)


def test_build_all_in_workers_and_serial_rebuild(tmp_path):
    """Specs are written by spawned workers; a worker that dies breaks the pool and the affected
    configs are rebuilt serially (the reference's behaviour, test_gemm_tc.py:88-97)."""
    from deca_b200.cli import _tune
    from deca_b200.kernels.gemm_b200 import GemmConfig, build_gemm_tc_to_file
    from deca_b200.kernels.module import KernelSpec

    cfgs = [GemmConfig(BN=bn, stages=st) for bn in (128, 256) for st in (3, 4)]
    paths = _tune.build_all(build_gemm_tc_to_file, lambda c, p: ((1024, 1024, 1024), c, "sm_100a", p), cfgs, 2, "t_")
    assert set(paths) == set(cfgs)
    for c, p in paths.items():
        spec = KernelSpec.from_json(open(p).read())
        assert spec.family == "gemm" and GemmConfig(**spec.config) == c
    # invalid configs are reported and skipped, valid ones still come back
    bad = GemmConfig(BN=96)
    out = _tune.build_all(build_gemm_tc_to_file, lambda c, p: ((1024, 1024, 1024), c, "sm_100a", p), [bad, cfgs[0]], 2, "t_")
    assert set(out) == {cfgs[0]}


def test_log_record_format(tmp_path, monkeypatch):
    from deca_b200.cli import _tune

    monkeypatch.setenv("DECA_LOG_DIR", str(tmp_path))
    assert _tune.log_path() == str(tmp_path / "deca_performance.log")
    msg = (f"{_tune.stamp()} [NVIDIA B200]\n DeCA GEMMTC(M=4096, N=4096, K=4096, float16), config: X (cost-model rank 1/24)\n"
           f" throughput: 1386.5 TFLOPS (62% of fp32-acc TC peak), runtime: 0.0989 ms, max err: 3.12e-02\n"
           f" torch: 1427.1 TFLOPS, runtime: 0.0963 ms, ratio: 0.974\n compile time: 0.3 s, total tuning time: 9.1 s\n")
    with open(_tune.log_path(), "a") as log:
        _tune.emit(msg, log)
    text = open(_tune.log_path()).read()
    assert re.match(r"\d{4}-\d\d-\d\d \d\d:\d\d:\d\d \[NVIDIA B200\]\n DeCA GEMMTC\(", text)
    assert text.endswith("\n\n")
    # flags of the three CLIs
    from deca_b200.cli import test_flash_attn, test_gemm_tc, test_rowwise

    a = test_gemm_tc.parse_args([])
    assert (a.shape, a.top_n, a.finalists, a.rounds, a.sweep) == ([4096, 4096, 4096], 24, 3, 5, False)
    a = test_flash_attn.parse_args(["--causal"])
    assert (a.shape, a.top_n, a.causal) == ([4, 16, 4096, 128], 16, True)
    assert test_flash_attn.parse_shape([4, 16, 4096, 128]) == (4, 16, 4096, 4096, 128)
    a = test_rowwise.parse_args(["--op", "rmsnorm", "--dtype", "bf16"])
    assert (a.shape, a.op, a.dtype, a.eps, a.top_n) == ([16384, 4096], "rmsnorm", "bf16", 1e-6, 24)

"""The tune harness on a GPU, as the CLIs drive it: ``build_*_to_file`` writes a kernel file,
``RuntimeMod.load_kernel`` / ``load_flash_attn`` binds it, ``time_evaluator`` verifies the kernel
against the operator's torch reference and times it, ``record`` is the line the CLIs print
(reference: src/RuntimeMod.py:104-109, :156-238; record strings :185-190, :235-238).  A kernel
whose output is out of tolerance must raise the RuntimeError that the CLIs catch and report as
"is not a valid config" (test_gemm_tc.py:126-132)."""

import re

import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

FLOAT = r"[0-9]+\.[0-9]+"
SCI = r"[0-9]\.[0-9]{2}e[-+][0-9]{2}"


@pytest.fixture(scope="module")
def arch():
    from deca_b200.arch.B200 import B200

    return B200()


def test_gemm_record_and_rejection(arch, tmp_path):
    from deca_b200.kernels.gemm_b200 import GemmConfig, build_gemm_tc_to_file
    from deca_b200.operators import GEMMTC
    from deca_b200.RuntimeMod import RuntimeMod

    shape = (512, 768, 256)
    op = GEMMTC(*shape)
    cfg = GemmConfig(BM=128, BN=128, stages=4, raster=2, acc_bufs=2, epi_smem=True)
    path = build_gemm_tc_to_file(shape, cfg, "sm_100a", str(tmp_path / "cfg0.so"))
    rt = RuntimeMod(op, arch, True, cfg)
    rt.load_kernel(path)
    rt.time_evaluator()
    assert rt.execution_time > 0 and rt.throughput == pytest.approx(op.num_flops / rt.execution_time / 1e12)
    atol, rtol = op.tolerance
    assert 0 < rt.max_error <= atol + rtol * 100
    assert re.fullmatch(
        rf"GEMMTC\(M=512, N=768, K=256, float16\) \n\t{re.escape(str(cfg))} \n\tcost time: {FLOAT} ms, "
        rf"throughput: {FLOAT} TFLOPS, max err: {SCI}", rt.record), rt.record

    # a reference the kernel cannot match: the harness must reject the config
    wrong = GEMMTC(*shape)
    wrong.reference = lambda inputs: GEMMTC.reference(wrong, inputs) + 1.0
    rt = RuntimeMod(wrong, arch, True, cfg)
    rt.load_kernel(path)
    with pytest.raises(RuntimeError, match=r"max error .* exceeds atol="):
        rt.time_evaluator()
    assert rt.record == ""

    # in-process build gives the same kernel
    rt = RuntimeMod(op, arch, True, cfg)
    rt.build()
    rt.time_evaluator()
    assert rt.record.startswith("GEMMTC(M=512")


@pytest.mark.parametrize("causal", [False, True])
def test_flash_attention_record_and_rejection(arch, tmp_path, causal):
    from deca_b200.kernels.flash_attn_b200 import FAConfig, build_flash_attn_to_file
    from deca_b200.operators import FlashAttention
    from deca_b200.RuntimeMod import RuntimeMod

    shape = (2, 3, 512, 512, 128)
    op = FlashAttention(*shape, causal=causal)
    cfg = FAConfig(Bc=128, stages=4, q_tiles=2, p_tmem=True, persistent=True)
    path = build_flash_attn_to_file(shape, cfg, op.softmax_scale, "sm_100a", str(tmp_path / "cfg0.so"), causal=causal)
    rt = RuntimeMod(op, arch, True, cfg)
    rt.load_flash_attn(path)
    rt.time_evaluator()
    assert 0 < rt.max_error <= 2e-2
    tail = ", causal" if causal else ""
    assert re.fullmatch(
        rf"FlashAttention\(B=2, H=3, S_q=512, S_kv=512, D=128, float16{tail}\) \n\t{re.escape(str(cfg))} "
        rf"\n\tcost time: {FLOAT} ms, throughput: {FLOAT} TFLOPS, max err: {SCI}", rt.record), rt.record

    wrong = FlashAttention(*shape, causal=causal)
    wrong.reference = lambda inputs: FlashAttention.reference(wrong, inputs) * 1.5
    rt = RuntimeMod(wrong, arch, True, cfg)
    rt.load_flash_attn(path)
    with pytest.raises(RuntimeError, match=r"max error .* exceeds 0.02"):
        rt.time_evaluator()


@pytest.mark.parametrize("kind,dtype", [("softmax", "fp16"), ("rmsnorm", "bf16")])
def test_rowwise_record_and_rejection(arch, tmp_path, kind, dtype):
    from deca_b200.kernels.rowwise_b200 import RowConfig, build_rowwise_to_file
    from deca_b200.operators import RMSNorm, Softmax
    from deca_b200.RuntimeMod import RuntimeMod

    cls = Softmax if kind == "softmax" else RMSNorm
    shape = (1024, 4096)
    op = cls(*shape, dtype)
    cfg = RowConfig(threads_per_row=128, rows_per_block=1, vec=8, mode="reg")
    path = build_rowwise_to_file(kind, shape, op.dtype, cfg, op.eps, "sm_100a", str(tmp_path / "cfg0.so"))
    rt = RuntimeMod(op, arch, False, cfg)
    rt.load_kernel(path)
    rt.time_evaluator()
    assert rt.throughput == pytest.approx(op.num_bytes / rt.execution_time / 1e9)
    assert re.fullmatch(
        rf"{cls.__name__}\(M=1024, N=4096, {op.dtype}\) \n\t{re.escape(str(cfg))} \n\tcost time: {FLOAT} ms, "
        rf"throughput: {FLOAT} GB/s, max err: {SCI}", rt.record), rt.record

    wrong = cls(*shape, dtype)
    wrong.reference = lambda inputs: cls.reference(wrong, inputs) + 0.25
    rt = RuntimeMod(wrong, arch, False, cfg)
    rt.load_kernel(path)
    with pytest.raises(RuntimeError, match=r"exceeds atol="):
        rt.time_evaluator()


def test_measure_configs_reports_invalid_config_and_continues(arch, tmp_path, capsys):
    """The CLI loop: a config that fails verification is printed as invalid and skipped."""
    from deca_b200.cli import _tune
    from deca_b200.kernels.rowwise_b200 import RowConfig, build_rowwise_to_file
    from deca_b200.operators import Softmax

    shape = (512, 2048)
    op = Softmax(*shape, "fp16")
    good = RowConfig(threads_per_row=64, rows_per_block=1, vec=8, mode="reg")
    other = RowConfig(threads_per_row=128, rows_per_block=2, vec=8, mode="reg")
    paths = {c: build_rowwise_to_file("softmax", shape, op.dtype, c, op.eps, "sm_100a", str(tmp_path / f"cfg{i}.so"))
             for i, c in enumerate((good, other))}
    # the second file is replaced by a kernel for another operator: it verifies wrongly
    paths[other] = build_rowwise_to_file("rmsnorm", shape, op.dtype, other, op.eps, "sm_100a", str(tmp_path / "bad.so"))
    res = _tune.measure_configs(op, arch, False, [good, other], paths)
    text = capsys.readouterr().out
    assert [cfg for _, cfg, _, _ in res] == [good]
    assert f"{other} is not a valid config:" in text
    assert "Softmax(M=512, N=2048, float16)" in text

"""The reference's three command lines, end to end on a GPU: enumerate, rank, build in worker
processes, verify, time, compare with the torch baseline, print the record and append it to
``deca_performance.log`` (formats: test_gemm_tc.py:159-167, test_flash_attn.py:143-151,
test_rowwise.py:133-141 of the reference).  Run as the user would, from the repository root."""

import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STAMP = r"\d{4}-\d{2}-\d{2} \d{2}:\d{2}:\d{2} \[NVIDIA B200\]\n"
TAIL = r" compile time: \d+\.\d s, total tuning time: \d+\.\d s\n"
NUM = r"\d+\.\d+"


def run_cli(script, args, tmp_path):
    env = dict(os.environ, DECA_LOG_DIR=str(tmp_path))
    res = subprocess.run([sys.executable, os.path.join(ROOT, script), *args], capture_output=True, text=True, env=env,
                         cwd=str(tmp_path), timeout=600)
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-1500:]
    with open(tmp_path / "deca_performance.log") as f:
        return res.stdout, f.read()


def test_gemm_cli(tmp_path):
    out, log = run_cli("test_gemm_tc.py", ["--shape", "1024", "1024", "512", "--top_n", "3", "--finalists", "2", "--rounds", "1",
                                           "--jobs", "2"], tmp_path)
    assert re.search(r"Find \d+ GEMMTC configs, measuring 3", out)
    assert out.count("cost time:") == 3 and "✅✅✅ " in out
    assert re.fullmatch(
        STAMP + r" DeCA GEMMTC\(M=1024, N=1024, K=512, float16\), config: \S+ \(cost-model rank [1-3]/3\)\n"
        rf" throughput: {NUM} TFLOPS \(\d+% of fp32-acc TC peak\), runtime: {NUM} ms, max err: \d\.\d\de[-+]\d\d\n"
        rf" torch: {NUM} TFLOPS, runtime: {NUM} ms, ratio: {NUM}\n" + TAIL + r"\n", log), log


def test_flash_attention_cli(tmp_path):
    out, log = run_cli("test_flash_attn.py", ["--shape", "1", "4", "1024", "128", "--causal", "--top_n", "3", "--finalists", "2",
                                              "--rounds", "1", "--jobs", "2"], tmp_path)
    assert re.search(r"Find \d+ FlashAttention configs, measuring 3", out)
    assert re.fullmatch(
        STAMP + r" DeCA FlashAttention: B = 1, H = 4, S_q = 1024, S_kv = 1024, D = 128, causal = True, config: \S+ "
        r"\(cost-model rank [1-3]/3\)\n"
        rf" throughput: {NUM} TFLOPS, runtime: {NUM} ms, max err: \d\.\d\de[-+]\d\d\n"
        rf" SDPA-flash: {NUM} TFLOPS, runtime: {NUM} ms, ratio: {NUM}\n" + TAIL + r"\n", log), log


def test_rowwise_cli_and_sweep_files(tmp_path):
    out, log = run_cli("test_rowwise.py", ["--op", "rmsnorm", "--dtype", "bf16", "--shape", "2048", "4096", "--top_n", "3",
                                           "--finalists", "2", "--rounds", "1", "--jobs", "2"], tmp_path)
    assert re.search(r"Find \d+ RMSNorm configs, measuring 3", out)
    assert re.fullmatch(
        STAMP + r" DeCA RMSNorm\(M=2048, N=4096, bfloat16\), config: \S+ \(cost-model rank [1-3]/3\)\n"
        rf" throughput: {NUM} GB/s \(\d+% of DRAM peak\), runtime: {NUM} ms, max err: \d\.\d\de[-+]\d\d\n"
        rf" torch: {NUM} GB/s, runtime: {NUM} ms, ratio: {NUM}\n" + TAIL + r"\n", log), log
    # a second run appends
    _, log2 = run_cli("test_rowwise.py", ["--op", "softmax", "--shape", "512", "1024", "--top_n", "2", "--finalists", "1",
                                          "--rounds", "1", "--jobs", "1"], tmp_path)
    assert log2.startswith(log) and log2.count(" DeCA ") == 2

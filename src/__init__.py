"""The reference's ``src`` import root over the ``deca_b200`` package: with ``<root>/src`` and ``<root>`` on
``sys.path`` (test_gemm_tc.py:23-24 of the reference) ``from operators import GEMMTC``,
``from kernels.gemm_tir import build_gemm_tc_to_file``, ``from Solver import solve_gemm_tc``,
``from RuntimeMod import RuntimeMod`` and ``from src.utils.helper import GPUDetector`` resolve to the
same objects as the ``deca_b200.*`` modules (the classes are re-exported, not redefined)."""

"""``python test_gemm_tc.py [--shape ...] [--sweep] ...``: the reference's command line of the same name,
served by ``deca_b200.cli.test_gemm_tc`` (same flags, progress lines, record and log format)."""

import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [os.path.join(ROOT, "src"), ROOT]

if __name__ == "__main__":
    from deca_b200.cli.test_gemm_tc import main

    main()

"""deca_b200 -- B200 (sm_100a) kernels behind DeCA's operator hot path.

Layout (mirrors the reference's ``src/`` tree so call sites read the same):

* ``operators``  Operator records (GEMMTC, FlashAttention, Softmax, RMSNorm)
* ``kernels``    config dataclasses + validity rules, benchmark helpers, kernel modules
* ``RuntimeMod`` build-or-load one config, verify against the torch reference, time it
* ``Solver`` / ``cost_model``  config enumeration and ranking for B200
* ``arch``       hardware model (``B200``)
* ``native``     ctypes binding of ``libdeca_b200.so`` (C ABI in ``include/deca_b200.h``)
* ``csrc``       the CUDA sources

Importing the package touches neither CUDA nor the native library.
"""

__version__ = "0.1"

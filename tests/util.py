"""Helpers shared by the tests: 16-bit ulp, tolerance checks, torch <-> bit-pattern bridges."""

import numpy as np


def ulp(ref32, dtype):
    """Spacing of the 16-bit type at |ref32| (subnormal range included)."""
    mant = 10 if dtype == "float16" else 7
    emin = -14 if dtype == "float16" else -126
    e = np.floor(np.log2(np.maximum(np.abs(ref32), 2.0**emin)))
    return 2.0 ** (e - mant)


def rowwise_allowed(ref32, dtype, op="softmax"):
    """Tolerance of the row-wise kernels against the fp32 oracle value (before rounding).

    RMSNorm rounds x * rsqrt(..) to the 16-bit type BEFORE the weight multiply, as the reference
    kernel does.  That makes the result a step function of the rsqrt: where x * r sits on a
    rounding boundary, a last-bit difference in r (rsqrt.approx against 1/sqrtf) moves the
    intermediate by one 16-bit ulp, and the result by |w| ulps.  Such elements are rare (a few
    per 100 000); for them the bound is two ulps of the output type on top of the 1e-3.

    fp16: 1e-3 relative; the absolute floor of 3e-8 is half the fp16 subnormal spacing, i.e.
    the rounding any fp16 result carries near zero.
    bf16: a bf16 ulp (2^-8 relative) is coarser than 1e-3, so the bound is 1e-3 relative on the
    fp32 math plus the half-ulp rounding of the 16-bit store.
    """
    if op == "rmsnorm":
        return 1e-3 * np.abs(ref32) + 2.0 * ulp(ref32, dtype)
    if dtype == "float16":
        return 1e-3 * np.abs(ref32) + 3e-8
    return 1e-3 * np.abs(ref32) + 0.5 * ulp(ref32, dtype)


def torch_to_bits(t):
    import torch

    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def bits_to_torch(bits, dtype, device="cuda"):
    import torch

    tdt = {"float16": torch.float16, "bfloat16": torch.bfloat16}[dtype]
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(tdt).to(device)

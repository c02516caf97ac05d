"""Tolerances shared by the parity tests.

Integers, indices and row copies are compared bit for bit.  Floating point:

* fp32 results against the fp32 oracle: rtol 1e-5, with an absolute floor where long sums cancel.
* bf16 / fp16 results against an fp32 oracle that was given the same 16-bit inputs: rtol 2e-2.
  Accumulation is fp32 on both sides, so the two differ by the roundings of 16-bit tensors stored
  on the way (2^-9 relative each for bf16).  The absolute floor, which only matters for entries
  that cancel to almost nothing, is therefore a small multiple of one such rounding of a typical
  element: ``4 * roundings * 2^-9 * rms(want)``.
"""
import torch

BF16_ROUNDING = 2.0 ** -9


def rms(t):
    t = t.float()
    return float(t.pow(2).mean().sqrt()) if t.numel() else 0.0


def half_tol(want, roundings=1):
    """assert_close keywords for a 16-bit result against its fp32 counterpart ``want``."""
    return dict(rtol=2e-2, atol=4 * roundings * BF16_ROUNDING * rms(want))


def assert_half_close(got, want, roundings=1, name=""):
    torch.testing.assert_close(got.float().cpu(), want.float().cpu(), **half_tol(want, roundings),
                               msg=lambda m: f"{name}: {m}")

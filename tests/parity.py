"""Tolerances shared by the parity tests.

Integers, indices and row copies are compared bit for bit.  Floating point:

* fp32 results against the fp32 oracle: rtol 1e-5, with an absolute floor where long sums cancel.
* bf16 / fp16 results against an fp32 oracle that was given the same 16-bit inputs: rtol 2e-2.
  Accumulation is fp32 on both sides, so the two differ by the roundings of 16-bit tensors stored
  on the way (2^-9 relative each for bf16).  The absolute floor only matters for entries that
  cancel to almost nothing: there the error is that of the (large) terms that cancelled, i.e. of
  a typical element.  Floor = ``roundings * 2^-9 * rms(want) * sqrt(2 ln N)``: one rounding of a
  typical element per 16-bit tensor on the way, times the expected extreme of N such errors
  (3.7 for a thousand elements, 5.8 for the 16.8 M outputs of the full-size layer).
"""
import math

import torch

BF16_ROUNDING = 2.0 ** -9


def rms(t):
    t = t.float()
    return float(t.pow(2).mean().sqrt()) if t.numel() else 0.0


def half_tol(want, roundings=1):
    """assert_close keywords for a 16-bit result against its fp32 counterpart ``want``."""
    spread = math.sqrt(2.0 * math.log(max(want.numel(), 16)))
    return dict(rtol=2e-2, atol=roundings * BF16_ROUNDING * rms(want) * spread)


def assert_half_close(got, want, roundings=1, name=""):
    torch.testing.assert_close(got.float().cpu(), want.float().cpu(), **half_tol(want, roundings),
                               msg=lambda m: f"{name}: {m}")

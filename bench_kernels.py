#!/usr/bin/env python
r"""Per-kernel timings of the MoE hot path on one B200, against each kernel's roofline.

    python bench_kernels.py [--only routing|permute|gemm] [--reps N] [--json]

bench.py reports the layer; this script times each CUDA kernel family alone
(CUDA events on the launching stream, L2 flushed between repetitions by writing a
256 MiB buffer) and divides its algorithmic bytes / flops by the time:

* routing kernels at the benchmark layer's size (32768 gate entries, launch-latency
  bound) and at a scaled synthetic size (2^24 entries, 16 experts) where HBM
  throughput is meaningful;
* token permutation kernels at config-2 sizes (16384 tokens, top-2, d_model 1024, bf16);
* the six grouped GEMM products of one layer step at config-2 sizes.

Peaks come from MEASURED_PEAKS.json when present (else the pool's fallback figures).
It is also the small, committed workload that the ncu captures under profiles/ run.
"""
import argparse
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
from fastermoe_b200 import fmoe_cuda as fc, _lib  # noqa: E402


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


class Timer:
    def __init__(self, reps):
        self.reps = reps
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def __call__(self, fn):
        for _ in range(2):
            fn()
        ts = []
        for _ in range(self.reps):
            self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return float(np.median(ts)) * 1e3  # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default=None, choices=["routing", "permute", "gemm"])
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args()
    hbm, tflops, src = peaks()
    t = Timer(args.reps)
    rows = []

    def mem(name, fn, nbytes):
        us = t(fn)
        gbs = nbytes / us / 1e3
        rows.append(dict(kernel=name, us=us, bound="hbm", achieved=gbs, unit="GB/s", peak=hbm, frac=gbs / hbm,
                         algorithmic_bytes=nbytes))

    def tens(name, fn, flops):
        us = t(fn)
        tf = flops / us / 1e6
        rows.append(dict(kernel=name, us=us, bound="tensor", achieved=tf, unit="TFLOP/s", peak=tflops, frac=tf / tflops,
                         algorithmic_flops=flops))

    rng = np.random.default_rng(1)
    if args.only in (None, "routing"):
        for n, tag in ((32768, "config 2"), (1 << 24, "2^24 entries")):
            E = 16
            gate = torch.from_numpy(rng.integers(0, E, size=n)).cuda()
            cnt = torch.zeros(E, dtype=torch.int32, device="cuda")
            mem(f"expert_count ({tag})", lambda: fc.expert_count(gate, cnt), 8 * n + 4 * E)
            # count + positions: gate read twice, pos and inv written
            mem(f"count_and_pos ({tag})", lambda: fc.count_and_pos(gate, E), 2 * 8 * n + 2 * 8 * n)
            ec = torch.full((E,), n // E // 2, dtype=torch.int32, device="cuda")
            mem(f"prune_gate_by_capacity ({tag})", lambda: fc.prune_gate_by_capacity(gate, ec.clone(), E, 1),
                2 * 8 * n + 8 * n)
        W, E = 8, 4
        ecw = torch.from_numpy(rng.integers(0, 5000, size=W * E)).cuda()
        cap = torch.full((E,), 9831, dtype=torch.int32, device="cuda")
        mem("limit_by_capacity (8 workers x 4 experts)", lambda: fc.limit_by_capacity(ecw, cap.clone(), E, W), 16 * W * E)

    T, k, d, h, E = 16384, 2, 1024, 4096, 16
    if args.only in (None, "permute"):
        gate = torch.from_numpy(rng.integers(0, E, size=(T, k))).cuda()
        lec, off, pos, inv = fc.count_and_pos(gate.reshape(-1), E)
        x = torch.randn(T, d, device="cuda").bfloat16()
        buf = torch.randn(T * k, d, device="cuda").bfloat16()
        score = torch.rand(T, k, device="cuda").bfloat16()
        go = torch.randn(T, d, device="cuda").bfloat16()
        b = 2
        mem("local_scatter", lambda: fc.local_scatter(x, pos, pos_div=k), T * k * d * b + 8 * T * k + T * k * d * b)
        mem("local_gather (inverse map)", lambda: fc.local_gather_inv(buf, inv), 2 * T * k * d * b + 8 * T * k)
        mem("local_gather_sum (scatter backward)", lambda: fc.local_gather_sum(buf, inv, T, k), T * k * d * b + T * d * b + 8 * T * k)
        mem("combine_forward (gather + score)", lambda: fc.combine_forward(buf, inv, score), T * k * d * b + T * d * b + 8 * T * k)
        mem("combine_backward", lambda: fc.combine_backward(go, buf, inv, score), (1 + k) * T * d * b + k * T * d * b + 8 * T * k)

    if args.only in (None, "gemm"):
        B = T * k
        counts = np.random.default_rng(0).multinomial(B, np.ones(E) / E)
        offs = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int64, device="cuda")
        x = torch.randn(B, d, device="cuda").bfloat16()
        w1 = (torch.randn(E, h, d, device="cuda") / 32).bfloat16()
        b1 = torch.randn(E, h, device="cuda").bfloat16()
        w2 = (torch.randn(E, d, h, device="cuda") / 64).bfloat16()
        b2 = torch.randn(E, d, device="cuda").bfloat16()
        hm = torch.randn(B, h, device="cuda").bfloat16()
        dv = torch.rand(B, h, device="cuda").bfloat16()
        gy = torch.randn(B, d, device="cuda").bfloat16()
        gh = torch.randn(B, h, device="cuda").bfloat16()
        fl = 2.0 * B * d * h
        N, G = _lib.ACT_NONE, _lib.ACT_GELU
        tens("GEMM fwd1 x.W1^T + b1, GELU, derivative saved", lambda: fc.linear_forward_act(x, offs, w1, b1, G, want_pre=True), fl)
        tens("GEMM fwd2 h.W2^T + b2", lambda: fc.linear_forward_act(hm, offs, w2, b2, N), fl)
        tens("GEMM dgrad2 dY.W2 * gelu'", lambda: _bwd(gy, hm, w2, offs, dv, G, True, False), fl)
        tens("GEMM wgrad2 dY^T.h (+ bias gradient)", lambda: _bwd(gy, hm, w2, offs, None, N, False, True), fl)
        tens("GEMM dgrad1 dH.W1", lambda: _bwd(gh, x, w1, offs, None, N, True, False), fl)
        tens("GEMM wgrad1 dH^T.x (+ bias gradient)", lambda: _bwd(gh, x, w1, offs, None, N, False, True), fl)

    if args.json:
        print(json.dumps({"peaks": {"hbm_gbs": hbm, "bf16_tflops": tflops, "source": src}, "kernels": rows}))
    else:
        print(f"peaks ({src}): HBM {hbm:.0f} GB/s, bf16 {tflops:.0f} TFLOP/s")
        for r in rows:
            print(f"{r['kernel']:52s} {r['us']:9.1f} us  {r['achieved']:9.1f} {r['unit']:8s} {100 * r['frac']:5.1f}% of {r['bound']} peak")


_bufs = {}


def _bwd(gy, x, w, offs, act_pre, act, want_gx, want_gw):
    """One product of fmoe_linear_backward through the C ABI with preallocated outputs."""
    import ctypes
    n_expert, out_feat, in_feat = w.shape
    key = (in_feat, out_feat)
    if key not in _bufs:
        _bufs[key] = (torch.empty(gy.shape[0], in_feat, device="cuda", dtype=w.dtype), torch.empty_like(w),
                      torch.empty(n_expert, out_feat, device="cuda", dtype=w.dtype))
    gx, gw, gb = _bufs[key]
    p = lambda z: ctypes.c_void_p(z.data_ptr()) if z is not None else None
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = _lib.lib.fmoe_linear_backward(p(gy), p(x), p(w), p(offs), p(act_pre), p(gx) if want_gx else None,
                                       p(gw) if want_gw else None, p(gb) if want_gw else None, gy.shape[0], in_feat,
                                       out_feat, n_expert, _lib.BF16, act, 0, None, st)
    assert rc == 0, _lib.last_error()


if __name__ == "__main__":
    main()

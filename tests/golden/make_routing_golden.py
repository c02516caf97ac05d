r"""Records outputs of the reference's own CUDA routing kernels (needs a GPU).

Run on the GPU box after oracle/build_ref.py has built oracle/_ref/fmoe_cuda_ref*.so:

    python tests/golden/make_routing_golden.py [output directory]

writes routing_ref_gpu.npz into the given directory (default: tests/golden/).

Recorded per case: the inputs and what the reference's kernels returned --
``expert_count`` (cuda/local_exchange.cuh:32-61), ``assign_pos`` (:5-16),
``limit_by_capacity`` and ``prune_gate_by_capacity`` (cuda/balancing.cuh:5-46), and
``linear_forward`` / ``linear_backward`` in fp32 (cuda/parallel_linear.cuh:55-161).
The reference's prune kernel indexes its counter array with the raw gate value, so it is
only given gates without -1 entries.
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import build_ref  # noqa: E402

ref = build_ref.load()
assert ref is not None, "build oracle/_ref first (python oracle/build_ref.py)"
out = {}
rng = np.random.default_rng(2024)
for case, (n, E, skip) in enumerate([(64, 4, 0.2), (1000, 7, 0.1), (4096, 16, 0.0), (32768, 16, 0.05), (5000, 200, 0.1)]):
    g = rng.integers(0, E, size=n)
    g[rng.random(n) < skip] = -1
    gate = torch.from_numpy(g).cuda()
    cnt = torch.zeros(E, dtype=torch.int32, device="cuda")
    ref.expert_count(gate, cnt)
    cum = torch.cumsum(cnt, 0).int()
    pos = torch.full((int(cum[-1].item()),), -1, dtype=torch.int64, device="cuda")
    cum_after = cum.clone()
    ref.assign_pos(cum_after, gate, pos)
    out[f"route{case}/gate"], out[f"route{case}/count"] = g, cnt.cpu().numpy()
    out[f"route{case}/pos"], out[f"route{case}/cum_after"] = pos.cpu().numpy(), cum_after.cpu().numpy()
    out[f"route{case}/meta"] = np.array([n, E])
for case, (W, E) in enumerate([(1, 4), (8, 2), (4, 16)]):
    ec = rng.integers(0, 40, size=W * E)
    cap = rng.integers(0, 100, size=E).astype(np.int32)
    cap_t = torch.from_numpy(cap.copy()).cuda()
    eca = ref.limit_by_capacity(torch.from_numpy(ec).cuda(), cap_t, E, W)
    out[f"limit{case}/ec"], out[f"limit{case}/cap"] = ec, cap
    out[f"limit{case}/eca"], out[f"limit{case}/cap_after"] = eca.cpu().numpy(), cap_t.cpu().numpy()
    out[f"limit{case}/meta"] = np.array([W, E])
for case, (n, E) in enumerate([(256, 4), (4096, 16), (20000, 64)]):
    g = rng.integers(0, E, size=n)
    ec = rng.integers(0, 2 * n // E, size=E).astype(np.int32)
    ec_t = torch.from_numpy(ec.copy()).cuda()
    pruned = ref.prune_gate_by_capacity(torch.from_numpy(g).cuda(), ec_t, E, 1)
    out[f"prune{case}/gate"], out[f"prune{case}/ec"] = g, ec
    out[f"prune{case}/pruned"], out[f"prune{case}/ec_after"] = pruned.cpu().numpy(), ec_t.cpu().numpy()
    out[f"prune{case}/meta"] = np.array([n, E])
torch.manual_seed(7)
counts, fin, fout = [5, 0, 9, 3], 24, 40
B = sum(counts)
x = torch.randn(B, fin, device="cuda"); w = torch.randn(len(counts), fout, fin, device="cuda") / 5
b = torch.randn(len(counts), fout, device="cuda"); gy = torch.randn(B, fout, device="cuda")
cnt = torch.tensor(counts, dtype=torch.int64)
y = ref.linear_forward(x, cnt, w, b)
gx, gw, gb = ref.linear_backward(gy, x, cnt, w, b)
for name, t in dict(x=x, w=w, b=b, gy=gy, y=y, gx=gx, gw=gw, gb=gb).items():
    out["linear/" + name] = t.cpu().numpy()
out["linear/counts"] = np.array(counts)
torch.cuda.synchronize()
dst = os.path.join(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "tests", "golden"), "routing_ref_gpu.npz")
os.makedirs(os.path.dirname(dst), exist_ok=True)
np.savez_compressed(dst, **out)
print("wrote", dst, len(out), "arrays")

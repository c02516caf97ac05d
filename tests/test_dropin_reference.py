"""Drop-in proof: the REFERENCE's own Python glue (its fmoe/functions.py, imported unmodified from the
staged copy that oracle/stage_reference.py makes) runs on top of this library's ``fmoe_cuda`` module
and reproduces the outputs recorded from the reference's CPU path (tests/golden/make_golden.py).
The operator sequence is the one the reference's layer and its tests/test_numerical.py:41-46 compose:
prepare_forward -> MOEScatter -> MOELinear -> activation -> MOELinear -> MOEGather -> bmm."""
import os

import numpy as np
import pytest
import torch

from oracle import stage_reference

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_functions():
    if stage_reference.staged() is None and stage_reference.stage() is None:
        pytest.skip("no staged copy of the reference's Python package (baseline/_ref) and no checkout to stage from")
    from fastermoe_b200 import fmoe_cuda as shim
    import sys
    saved = {n: m for n, m in sys.modules.items() if n == "fmoe_cuda" or n == "fmoe" or n.startswith("fmoe.")}
    fmoe, _ = stage_reference.import_reference(shim)
    import fmoe.functions as F
    assert F.fmoe_cuda is shim and os.path.realpath(F.__file__).startswith(os.path.realpath(stage_reference.DEST))
    yield F
    for n in [n for n in sys.modules if n == "fmoe_cuda" or n == "fmoe" or n.startswith("fmoe.")]:
        del sys.modules[n]
    sys.modules.update(saved)


@pytest.mark.parametrize("tag", ["layer_e4_k2_relu", "layer_e16_k2_gelu", "layer_e8_k3_gelu"])
def test_reference_glue_on_this_library(ref_functions, golden, tag):
    F = ref_functions
    z = {k.split("/", 1)[1]: torch.from_numpy(golden[k]) for k in golden.files if k.startswith(tag + "/")}
    T, d, h, E, k, act, _ = z["meta"].tolist()
    act = {2: torch.nn.functional.gelu, 1: torch.relu}[act]
    leaves = {n: z[n].cuda().requires_grad_(True) for n in ("x", "gate_w", "gate_b", "w1", "b1", "w2", "b2")}
    x = leaves["x"]
    idx = z["idx"].cuda()
    logits = torch.nn.functional.linear(x, leaves["gate_w"], leaves["gate_b"])
    score = torch.gather(logits, 1, idx)                    # NaiveGate returns the raw top-k logits
    pos, lec, gec, aec, agec, fwd = F.prepare_forward(idx, E, 1)
    assert not lec.is_cuda and int(fwd.sum()) == T * k and np.array_equal(lec.numpy(), gec.numpy())
    stored = torch.zeros(E, dtype=torch.bool)
    buf = F.MOEScatter.apply(x, torch.div(pos, k, rounding_mode="floor"), lec, gec, stored, T * k, 1)
    hid = act(F.MOELinear.apply(buf, fwd, leaves["w1"], leaves["b1"]))
    y = F.MOELinear.apply(hid, fwd, leaves["w2"], leaves["b2"])
    full = F.MOEGather.apply(y, pos, lec, gec, stored, T * k, 1)
    out = torch.bmm(score.view(T, 1, k), full.view(T, k, d)).reshape(T, d)
    out.sum().backward()
    tol = dict(rtol=1e-5, atol=2e-5)
    torch.testing.assert_close(out.detach().cpu(), z["out"], **tol)
    for n, t in leaves.items():
        torch.testing.assert_close(t.grad.cpu(), z["grad_" + n], **tol, msg=lambda s, n=n: f"grad_{n}: {s}")


def test_reference_gate_utils_on_this_library(ref_functions):
    """The reference's count_by_gate with and without positions (fmoe/functions.py:19-42)."""
    F = ref_functions
    from oracle import moe_oracle as O
    gate = torch.from_numpy(np.random.default_rng(0).integers(0, 6, size=(200, 2))).cuda()
    pos, lec, aec, gec, agec = F.count_by_gate(gate, 6, 1)
    assert np.array_equal(lec.cpu().numpy(), O.expert_count(gate.cpu().numpy(), 6))
    assert np.array_equal(pos.cpu().numpy(), O.assign_pos(gate.cpu().numpy(), 6))
    pos2, lec2, _, _, _ = F.count_by_gate(gate, 6, 1, require_pos=False)
    assert pos2 is None and torch.equal(lec2, lec)

r"""Autograd wrapper of the smart schedule (mirrors fmoe/fused_functions.py)."""
import torch
from torch.autograd import Function

from . import fmoe_cuda
from . import _lib
from .functions import activation_code


class MOEForward(Function):
    r"""local scatter -> pipelined exchange + expert MLP -> rows back in token order
    (fmoe/fused_functions.py:12-61).

    Differences from the reference: the expert parameters are inputs of the
    autograd function, so their gradients are returned to autograd (and
    accumulate normally) instead of being written over ``param.grad``; the
    activation follows the module (ReLU and exact GELU run in the GEMM epilogues).
    The output is the token-side buffer [A, d]; the layer's gather/combine follows.
    """

    @staticmethod
    def forward(ctx, inp, models, routing, top_k, exch, n_rows, act, *flat_params):
        inp = inp.contiguous()
        local_in = fmoe_cuda.local_scatter(inp, routing.pos, pos_div=top_k, n_rows=n_rows)
        params = [[tuple(p for p in node[0].parameters())] if node else [] for node in models]
        res = fmoe_cuda.fused_forward(local_in, params, exch.lec, exch.gec, exch.stored, None,
                                      exch.world_size, False, activation=act)
        out, gib, gmb = res[0], res[1], res[2]
        pre = res[4] if len(res) > 4 else None
        ctx.save_for_backward(routing.inv, gib, gmb, pre if pre is not None else gib.new_empty(0))
        ctx.has_pre = pre is not None
        ctx.params, ctx.exch, ctx.act = params, exch, act
        ctx.top_k, ctx.n_tokens, ctx.n_rows = top_k, inp.shape[0], n_rows
        return out

    @staticmethod
    def backward(ctx, grad_out):
        inv, gib, gmb, pre = ctx.saved_tensors
        exch, params = ctx.exch, ctx.params
        grads = []
        flat = []
        for j, node in enumerate(params):
            if not node:
                grads.append([])
                continue
            gs = tuple(torch.zeros_like(p) for p in node[0])
            grads.append([gs])
            flat.extend(gs)
        (grad_in_buf,) = fmoe_cuda.fused_backward(
            gib, params, gmb, None, grad_out.contiguous(), exch.lec, exch.gec, None, exch.stored, None,
            ctx.n_rows, exch.world_size, False, activation=ctx.act, middle_pre=pre if ctx.has_pre else None,
            grads=grads)
        grad_inp = fmoe_cuda.local_gather_sum(grad_in_buf, inv, ctx.n_tokens, ctx.top_k)
        return (grad_inp, None, None, None, None, None, None, *flat)


def fused_activation(experts):
    """Activation code of a fused expert module, or raises when the smart schedule
    cannot run it (it needs an activation the GEMM epilogue implements)."""
    code = activation_code(getattr(experts, "activation", None))
    if code is None:
        raise RuntimeError("the smart schedule supports ReLU and exact GELU activations only")
    return code

r"""CUDA-graph capture of a training step of an MoE layer.

The layer's forward and backward never read anything back to the host when the bucket sizes can
stay on the device: always at ``world_size == 1`` (the grouped GEMMs take their tile list from the
device-resident offsets), and at ``world_size > 1`` when the counts are swapped through peer memory
and the exchange plan is built on the device (no shadowing policy, fused experts; see
layers._fmoe_general_global_forward).  A whole step is then a fixed sequence of kernel launches and
can be replayed as one CUDA graph.  What remains on the host per step is one graph launch, which
removes the launch gaps at the start of a step that follows a synchronising read of the loss.

With ``world_size > 1`` the captured kernels wait for the peers' rows: every rank must replay its
graph once per step, in step with the others.  Exchange outputs come from a ReceiveArena (the same
buffers at every replay).  A forward that has to read the counts (shadowing policy, NCCL exchange)
cannot be captured: the capture then fails with the error of the host read.
"""
import torch


class GraphedStep:
    """``loss = loss_fn(module(x)); loss.backward()`` captured once, replayed per call.

    ``module``: a ``FMoE`` / ``FMoETransformerMLP`` with ``world_size == 1`` (any
    module whose forward+backward is free of host synchronisation works).
    ``example_input``: a CUDA tensor with the shape and dtype of every later input.
    ``loss_fn``: maps the module output to a scalar (default: sum accumulated in fp32).
    ``input_grad``: also keep the gradient with respect to the input (``.input_grad``).

    Calling the object copies ``x`` (CUDA or pinned host tensor) into the captured
    input buffer on the current stream, replays the graph and returns the loss
    tensor (device-resident, valid until the next call).  Parameter gradients are
    written to ``param.grad`` (the same tensors at every replay: they are
    overwritten, not accumulated); ``output`` holds the module output.
    """

    def __init__(self, module, example_input, loss_fn=None, warmup=3, input_grad=False):
        if not example_input.is_cuda:
            raise ValueError("GraphedStep: example_input must be a CUDA tensor")
        self.module = module
        from . import fmoe_cuda
        self._fc = fmoe_cuda
        self.arena = fmoe_cuda.ReceiveArena() if getattr(module, "world_size", 1) > 1 else None
        self.loss_fn = loss_fn if loss_fn is not None else (lambda out: out.sum(dtype=torch.float32))
        self.static_input = example_input.detach().clone().requires_grad_(input_grad)
        # Parameters that already took part in a backward pass on another stream make autograd
        # warn about the stream of their accumulation nodes; the warm-up below is meant to run
        # on a side stream, so the warning is switched off around it.
        quiet = getattr(torch.autograd.graph, "set_warn_on_accumulate_grad_stream_mismatch", None)
        if quiet is not None:
            quiet(False)
        try:
            side = torch.cuda.Stream(device=example_input.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):       # warm-up off the default stream, as graph capture requires
                for _ in range(max(int(warmup), 1)):
                    self._step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize(example_input.device)
            # gradients must be allocated inside the capture, from the graph's own memory pool
            module.zero_grad(set_to_none=True)
            self.static_input.grad = None
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.output, self.loss = self._step()
        finally:
            if quiet is not None:
                quiet(True)
        self.input_grad = self.static_input.grad

    def _step(self):
        if self.arena is not None:
            self.arena.begin_step()
            self._fc.set_receive_arena(self.arena)
        try:
            out = self.module(self.static_input)
            loss = self.loss_fn(out)
            loss.backward()
        finally:
            if self.arena is not None:
                self._fc.set_receive_arena(None)
        return out, loss

    def __call__(self, x):
        self.static_input.detach().copy_(x, non_blocking=True)
        self.graph.replay()
        return self.loss

    def replay(self):
        """The step once more on the batch the captured input buffer already holds."""
        self.graph.replay()
        return self.loss

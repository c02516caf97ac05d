r"""Where the adapter finds the host framework's state.

The reference's adapter calls ``megatron.get_args()`` and ``megatron.mpu`` wherever it needs the training
arguments or the parallel groups (fmoe/megatron/layers.py:200-204, balance.py:16-20, distributed.py:27-34).
Here those two objects are looked up through this module: ``bind(args=..., mpu=...)`` installs them
explicitly (a trainer that is not Megatron-LM, or a test, passes objects with the attributes that are
used); without a binding they are imported from Megatron-LM, and a clear error says so when it is absent.

Attributes read from ``args``: hidden_size, num_layers, init_method_std, seq_length, micro_batch_size,
tensor_model_parallel_size, data_parallel_size, pipeline_model_parallel_size, world_size, rank,
balance_strategy, and the ones add_fmoe_args defines.  Methods called on ``mpu``:
get_tensor_model_parallel_group (or get_model_parallel_group), get_data_parallel_group.
"""
_bound = {"args": None, "mpu": None}


def bind(args=None, mpu=None):
    """Installs the arguments object and / or the parallel-state object; ``None`` leaves a slot as it is.
    ``unbind()`` clears both."""
    if args is not None:
        _bound["args"] = args
    if mpu is not None:
        _bound["mpu"] = mpu


def unbind():
    _bound["args"] = _bound["mpu"] = None


def _missing(what, err):
    raise ImportError(f"fastermoe_b200.megatron needs {what}: bind it with fastermoe_b200.megatron.bind(...), "
                      "or make Megatron-LM importable") from err


def get_args():
    if _bound["args"] is not None:
        return _bound["args"]
    try:
        from megatron import get_args as native
    except ImportError as e:
        _missing("the training arguments", e)
    return native()


def get_mpu():
    if _bound["mpu"] is not None:
        return _bound["mpu"]
    try:
        from megatron import mpu
    except ImportError as e:
        _missing("the parallel state (mpu)", e)
    return mpu


# The command-line switches of the plug-in (the names a Megatron launch script passes; fmoe/megatron/utils.py).
_SWITCHES = (
    ("--fmoefy", dict(action="store_true", help="replace the MLP blocks by mixture-of-experts blocks")),
    ("--num-experts", dict(type=int, default=None, help="experts per worker")),
    ("--top-k", dict(type=int, default=2, help="experts per token")),
    ("--balance-loss-weight", dict(type=float, default=1, help="factor of the gates' balance loss in the training loss")),
    ("--balance-strategy", dict(type=str, default=None, help="naive | noisy | gshard | switch | hir")),
    ("--hidden-hidden-size", dict(type=int, default=None, help="width of an expert's hidden layer (default 4 x hidden)")),
)


def add_fmoe_args(parser):
    """Adds the plug-in's switches to an argparse parser (Megatron's ``extra_args_provider``)."""
    group = parser.add_argument_group(title="fastmoe")
    for flag, spec in _SWITCHES:
        group.add_argument(flag, **spec)
    return parser

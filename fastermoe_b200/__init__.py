r"""fastermoe_b200: the FasterMoE MoE-layer hot path on NVIDIA B200 (sm_100a).

Public classes keep the names of the reference package ``fmoe``
(fmoe/__init__.py:5-7): :class:`FMoE`, :class:`FMoELinear`,
:class:`FMoETransformerMLP`; the operator module :mod:`fastermoe_b200.fmoe_cuda`
keeps the names of the reference's ``fmoe_cuda`` extension.

Attributes are resolved on first use so that ``fastermoe_b200.build`` can be
imported (to compile the CUDA library) before the library exists.
"""
__all__ = ["FMoE", "FMoELinear", "FMoETransformerMLP", "DistributedGroupedDataParallel", "GraphedStep", "set_phase_hook"]

_HOME = {"FMoE": "layers", "FMoELinear": "layers", "FMoETransformerMLP": "transformer",
         "DistributedGroupedDataParallel": "distributed", "GraphedStep": "graphs", "set_phase_hook": "functions"}


def __getattr__(name):
    if name in _HOME:
        import importlib
        return getattr(importlib.import_module("." + _HOME[name], __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")

r"""fastermoe_b200: the FasterMoE MoE-layer hot path on NVIDIA B200 (sm_100a).

Public classes keep the names of the reference package ``fmoe``
(fmoe/__init__.py:5-7): :class:`FMoE`, :class:`FMoELinear`,
:class:`FMoETransformerMLP`; the operator module :mod:`fastermoe_b200.fmoe_cuda`
keeps the names of the reference's ``fmoe_cuda`` extension.
"""
from .layers import FMoE, FMoELinear
from .transformer import FMoETransformerMLP
from .distributed import DistributedGroupedDataParallel

__all__ = ["FMoE", "FMoELinear", "FMoETransformerMLP", "DistributedGroupedDataParallel"]

r"""Gates: map tokens to experts (same names as the reference's ``fmoe.gates``)."""
from .base_gate import BaseGate
from .naive_gate import NaiveGate
from .noisy_gate import NoisyGate
from .gshard_gate import GShardGate
from .switch_gate import SwitchGate
from .hir_gate import HirGate, HirCapacityGate, gen_hir_gate, gen_hir_capacity_gate
from .utils import limit_by_capacity

"""Model families used by the benchmarks and harnesses."""
from .tp_mlp import TPMLPConfig, TPMLPStack  # noqa: F401
from .moe import MoEConfig, MoELayer  # noqa: F401

"""Small helpers shared by the harnesses and benchmarks."""
from .launch import init_from_env, max_over_ranks  # noqa: F401
from .clocks import ClockSampler  # noqa: F401

"""Small utilities: clock sampling for benchmarks, timers."""
from .clocks import ClockSampler  # noqa: F401

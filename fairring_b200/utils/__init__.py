"""Measurement helpers: device timing, clock sampling."""

from .clocks import ClockSampler  # noqa: F401
from .timing import device_time_ms, max_over_ranks  # noqa: F401

"""Utilities: device timing, clock sampling, bus-bandwidth arithmetic."""
from .timing import ClockSampler, bus_bandwidth_factor, device_time_ms  # noqa: F401

"""Small utilities that are not part of the training path: phase tracing and timing."""

from .trace import enable_nvtx, enable_timing, phase, phase_times

__all__ = ["enable_nvtx", "enable_timing", "phase", "phase_times"]

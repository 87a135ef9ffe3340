"""Configuration, logging, timing and clock-sampling helpers."""
from .config import Config, config  # noqa: F401
from .timing import cuda_time_ms, L2Flusher, ClockSampler  # noqa: F401

"""Helpers: device timing, clock sampling during a timed region, CPU ring simulator binding."""
from .clocks import ClockSampler  # noqa: F401
from .sim import ll_sim, ring_sim  # noqa: F401
from .timing import time_cuda  # noqa: F401

"""ctypes mirror of include/sampler_b200.h."""
from __future__ import annotations

SAMPLER_SYMBOLS: dict = {}

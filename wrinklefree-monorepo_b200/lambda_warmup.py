"""Quantization-strength schedule shared by every BitLinear layer.

Same interface as the reference's wrinklefree/quantization/lambda_warmup.py:21-135:
lambda runs from `min_lambda` (no quantization) to `max_lambda` (full
quantization) over `warmup_steps`; `get_current_lambda()` is 1.0 when no
schedule is installed, which is the only state in which BitLinear takes the
packed-weight CUDA path.
"""
from __future__ import annotations

import math
import sys
from typing import Optional


class LambdaWarmup:
    def __init__(self, warmup_steps: int = 1000, schedule: str = "linear", min_lambda: float = 0.0, max_lambda: float = 1.0):
        if schedule not in ("linear", "cosine"):
            raise ValueError(f"Unknown schedule: {schedule}")
        self.warmup_steps, self.schedule = warmup_steps, schedule
        self.min_lambda, self.max_lambda = min_lambda, max_lambda
        self._current_step = 0
        self._lambda = min_lambda

    def step(self) -> None:
        self._current_step += 1
        if self._current_step >= self.warmup_steps:
            self._lambda = self.max_lambda
            return
        t = self._current_step / self.warmup_steps
        if self.schedule == "cosine":
            t = (1.0 - math.cos(math.pi * t)) / 2.0
        self._lambda = self.min_lambda + t * (self.max_lambda - self.min_lambda)

    @property
    def lambda_val(self) -> float:
        return self._lambda

    @property
    def current_step(self) -> int:
        return self._current_step

    def is_warmup_complete(self) -> bool:
        return self._current_step >= self.warmup_steps

    def state_dict(self) -> dict:
        return {"current_step": self._current_step, "lambda": self._lambda, "warmup_steps": self.warmup_steps,
                "schedule": self.schedule, "min_lambda": self.min_lambda, "max_lambda": self.max_lambda}

    def load_state_dict(self, state: dict) -> None:
        self._current_step = state["current_step"]
        self._lambda = state["lambda"]
        self.warmup_steps = state.get("warmup_steps", self.warmup_steps)
        self.schedule = state.get("schedule", self.schedule)


_global: Optional[LambdaWarmup] = None
_REFERENCE_MODULE = "wrinklefree.quantization.lambda_warmup"


def _reference_module():
    """The reference's own lambda_warmup module when the host process has imported it.  Its trainer installs the
    schedule there (training/stage2.py sets that module's global), so a drop-in layer must read the same global or
    it would run fully quantized while the trainer believes lambda < 1."""
    mod = sys.modules.get(_REFERENCE_MODULE)
    return mod if (mod is not None and mod is not sys.modules.get(__name__)) else None


def get_global_lambda_warmup() -> Optional[LambdaWarmup]:
    ref = _reference_module()
    if ref is not None and ref.get_global_lambda_warmup() is not None:
        return ref.get_global_lambda_warmup()
    return _global


def set_global_lambda_warmup(warmup: Optional[LambdaWarmup]) -> None:
    """Installs the schedule here and, when the reference's module is loaded, there too: one shared state."""
    global _global
    _global = warmup
    ref = _reference_module()
    if ref is not None:
        ref.set_global_lambda_warmup(warmup)


def get_current_lambda() -> float:
    w = get_global_lambda_warmup()
    return 1.0 if w is None else w.lambda_val

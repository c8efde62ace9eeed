"""Learning-rate schedules as pure functions of the optimizer step.

"linear": linear warm-up then constant; "cosine": warm-up then cosine to peak*end_factor;
"wsd": warm-up, stable for ``stable_fraction`` of the post-warm-up steps, then linear decay
to peak*end_factor (reference: omegalax/trainers/lr_schedule.py:8-73).
"""
from __future__ import annotations

import math
from typing import Callable


def build_lr_schedule(kind: str, peak: float, num_steps: int, warmup_steps: int = 0,
                      end_factor: float = 0.1, stable_fraction: float = 0.8) -> Callable[[int], float]:
    kind = kind.lower()
    if kind not in ("linear", "cosine", "wsd"):
        raise ValueError(f"unknown lr_schedule '{kind}' (expected linear, cosine or wsd)")
    warmup_steps = max(int(warmup_steps), 0)
    rest = max(num_steps - warmup_steps, 1)

    def warm(step: int) -> float | None:
        if warmup_steps > 0 and step < warmup_steps:
            return peak * step / warmup_steps
        return None

    def linear(step: int) -> float:
        w = warm(step)
        return peak if w is None else w

    def cosine(step: int) -> float:
        w = warm(step)
        if w is not None:
            return w
        t = min(max(step - warmup_steps, 0) / rest, 1.0)
        end = peak * end_factor
        return end + 0.5 * (peak - end) * (1.0 + math.cos(math.pi * t))

    def wsd(step: int) -> float:
        w = warm(step)
        if w is not None:
            return w
        stable = int(rest * stable_fraction)
        s = step - warmup_steps
        if s < stable:
            return peak
        decay = max(rest - stable, 1)
        t = min((s - stable) / decay, 1.0)
        return peak + (peak * end_factor - peak) * t

    return {"linear": linear, "cosine": cosine, "wsd": wsd}[kind]

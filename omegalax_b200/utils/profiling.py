"""Profiling helpers: named NVTX scopes and a per-kernel device-time table.

``scope(name)`` is the counterpart of the reference's ``jax.named_scope`` sites
(omegalax/models/qwen3/attention.py:67 and the other 16 places): a context manager that pushes
an NVTX range, so that an external profiler and the Kineto trace written by the trainers'
``--profile_dir`` window show the module structure (``attention``, ``mlp``, ``moe``,
``rms_norm``, ``gated_delta_net``, ``vision`` ...).  Scopes cost one host call each and are
off unless ``OMEGALAX_B200_NVTX=1`` or ``enable_scopes(True)``; the trainers switch them on
for the profile window only.

``kernel_time_table(fn)`` runs ``fn`` once under the Kineto CUDA activity tracer and returns
the device time of every kernel, aggregated by name: where a training step spends its time
under real conditions (concurrent streams, warm caches, power-capped clocks), which a
serialised profiler replay does not show.
"""
from __future__ import annotations

import contextlib
import os
import re
from collections import defaultdict

import torch

_enabled = os.environ.get("OMEGALAX_B200_NVTX", "0") == "1"
_depth_names: list[str] = []


def enable_scopes(on: bool = True) -> None:
    global _enabled
    _enabled = bool(on)


def scopes_enabled() -> bool:
    return _enabled


def current_scope() -> str:
    """Slash-joined names of the open scopes (empty when none or when scopes are off)."""
    return "/".join(_depth_names)


@contextlib.contextmanager
def scope(name: str):
    if not _enabled:
        yield
        return
    _depth_names.append(name)
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if cuda:
            torch.cuda.nvtx.range_pop()
        _depth_names.pop()


def scoped(name: str):
    """Decorator form of ``scope`` for module ``forward`` methods."""
    def deco(fn):
        def wrapped(*a, **k):
            if not _enabled:
                return fn(*a, **k)
            with scope(name):
                return fn(*a, **k)
        wrapped.__name__ = getattr(fn, "__name__", "wrapped")
        wrapped.__doc__ = fn.__doc__
        wrapped.__wrapped__ = fn
        return wrapped
    return deco


_TEMPLATE = re.compile(r"\(.*$")


def _short(name: str) -> str:
    name = _TEMPLATE.sub("", name)
    name = name.replace("void ", "").replace("ob::", "")
    return name[:110]


def kernel_time_table(fn, top: int = 40) -> list[dict]:
    """Run ``fn()`` once under the CUDA activity tracer; return rows
    ``{"kernel", "launches", "ms", "share"}`` sorted by device time (largest first)."""
    from torch.profiler import ProfilerActivity, profile

    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        fn()
        torch.cuda.synchronize()
    agg = defaultdict(lambda: [0, 0.0])
    for ev in prof.events():
        if getattr(ev, "device_type", None) is None or "cuda" not in str(ev.device_type).lower():
            continue
        dur = float(getattr(ev, "device_time", 0.0) or getattr(ev, "cuda_time", 0.0) or 0.0)
        if dur <= 0.0:
            dur = float(ev.time_range.elapsed_us()) if getattr(ev, "time_range", None) else 0.0
        a = agg[_short(ev.name)]
        a[0] += 1
        a[1] += dur / 1000.0
    total = sum(v[1] for v in agg.values()) or 1.0
    rows = [{"kernel": k, "launches": v[0], "ms": round(v[1], 3), "share": round(v[1] / total, 4)}
            for k, v in agg.items()]
    rows.sort(key=lambda r: -r["ms"])
    return rows[:top]


def format_table(rows: list[dict]) -> str:
    lines = ["| share | ms | launches | kernel |", "|---|---|---|---|"]
    for r in rows:
        lines.append(f"| {100 * r['share']:.1f} % | {r['ms']:.2f} | {r['launches']} | {r['kernel']} |")
    return "\n".join(lines)

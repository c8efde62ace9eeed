"""Throughput accounting: algorithmic FLOPs per token, step timing, tokens/s and MFU.

Convention (same as omegalax/trainers/perf.py:1-14): matmul FLOPs only (2*m*n*k), training
= 3 x forward, causal text attention counted over visited positions only (2*T*H*K per
token and layer), vision attention block-diagonal over images (sum of N_i^2).
"""
from __future__ import annotations

import datetime
import time
from typing import Any

import numpy as np
import torch

TRAINING_FLOP_MULTIPLIER = 3

# Peak dense bf16 TFLOP/s used as the MFU denominator.  The two "measured" entries are cuBLAS figures
# of one particular B200 under its 1000 W cap (best of ten 8192^3 products; four seconds back to
# back); a ``MEASURED_PEAKS.json`` of the machine at hand replaces them (``measured_peaks()``).
PEAK_TFLOPS: dict[str, float] = {
    "b200": 2250.0,
    "b200_measured_burst": 1613.6,
    "b200_measured_sustained": 1353.4,
    "h100_sxm": 989.0,
    "h100_pcie": 756.0,
    "a100_sxm_80": 312.0,
    "a100_sxm_40": 312.0,
    "a100_pcie_80": 312.0,
    "a100_pcie_40": 312.0,
}


def measured_peaks(path: str | None = None) -> dict | None:
    """Peaks measured on this machine, when a ``MEASURED_PEAKS.json`` (keys ``bf16_tflops``,
    ``bf16_tflops_sustained``, ``hbm_gbs``) is named by ``path`` / ``OMEGALAX_B200_MEASURED_PEAKS`` or
    sits in the working directory or next to the package; its GEMM figures replace the
    ``b200_measured_*`` presets."""
    import json
    import os

    here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    for cand in (path, os.environ.get("OMEGALAX_B200_MEASURED_PEAKS"), "MEASURED_PEAKS.json",
                 os.path.join(here, "MEASURED_PEAKS.json")):
        if cand and os.path.isfile(cand):
            try:
                d = json.load(open(cand))
            except (OSError, ValueError):
                continue
            if "bf16_tflops" in d:
                PEAK_TFLOPS["b200_measured_burst"] = float(d["bf16_tflops"])
            if "bf16_tflops_sustained" in d:
                PEAK_TFLOPS["b200_measured_sustained"] = float(d["bf16_tflops_sustained"])
            return d
    return None


measured_peaks()


def resolve_peak_tflops(spec: str | float | None) -> float | None:
    """None, a number, or a preset key of ``PEAK_TFLOPS``."""
    if spec is None:
        return None
    s = str(spec)
    if s in PEAK_TFLOPS:
        return PEAK_TFLOPS[s]
    try:
        return float(s)
    except ValueError as e:
        raise ValueError(f"Unknown peak_tflops {spec!r}. Use a key from {list(PEAK_TFLOPS)} or a number.") from e


def _attn_block(D: int, H: int, G: int, K: int, T: int, q_mult: int = 1) -> int:
    proj = 2 * D * (H * q_mult + 2 * G) * K
    return proj + 2 * T * H * K + 2 * H * K * D


def _ffn(cfg, layer_idx: int, D: int, *, shared: int = 0) -> int:
    is_moe = cfg.is_moe_layer(layer_idx) if hasattr(cfg, "is_moe_layer") else getattr(cfg, "is_moe", False)
    if is_moe:
        E, k, F = cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size
        f = 2 * D * E + k * (2 * 3 * D * F)
        if shared:
            f += 2 * 3 * D * shared + 2 * D
        return f
    F = getattr(cfg, "mlp_dim", None) or getattr(cfg, "intermediate_size")
    return 2 * 3 * D * F


def _flops_qwen3_like(cfg, T: int) -> int:
    D, H, G, K = cfg.emb_dim, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    per_attn = _attn_block(D, H, G, K, T)
    total = 0
    for i in range(cfg.num_layers):
        total += per_attn + _ffn(cfg, i, D)
    return total + 2 * D * cfg.vocab_size


def _flops_qwen3_5(cfg, T: int) -> int:
    D, H, G, K = cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    nk, nv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
    ak, av = cfg.linear_key_head_dim, cfg.linear_value_head_dim
    key_dim, value_dim = nk * ak, nv * av
    total = 0
    for i, kind in enumerate(cfg.layer_types):
        if kind == "full_attention":
            total += _attn_block(D, H, G, K, T, q_mult=2)  # q projection carries the gate
        else:
            total += (2 * D * (2 * key_dim + value_dim) + 2 * D * value_dim + 2 * 2 * D * nv
                      + 2 * value_dim * D + 2 * nv * ak * av)
        if cfg.is_moe:
            E, k, F = cfg.num_experts, cfg.num_experts_per_tok, cfg.moe_intermediate_size
            total += 2 * D * E + k * (2 * 3 * D * F) + 2 * 3 * D * cfg.shared_expert_intermediate_size + 2 * D
        else:
            total += 2 * 3 * D * cfg.intermediate_size
    return total + 2 * D * cfg.vocab_size


def training_flops_per_token(cfg, seq_len: int) -> int:
    """Training FLOPs per token (already x3).  Accepts Qwen3, Qwen3.5 (text or full) and
    Qwen3-VL configs; for VLM configs only the decoder stack is counted here."""
    if hasattr(cfg, "text_config"):
        cfg = cfg.text_config
    if hasattr(cfg, "layer_types") and hasattr(cfg, "linear_num_value_heads"):
        fwd = _flops_qwen3_5(cfg, seq_len)
    elif hasattr(cfg, "emb_dim"):
        fwd = _flops_qwen3_like(cfg, seq_len)
    else:
        raise TypeError(f"Unsupported config for FLOP counting: {type(cfg)}")
    return fwd * TRAINING_FLOP_MULTIPLIER


def qwen3_vl_vision_training_flops(cfg, image_grid_thw: Any | None) -> int:
    """Vision-tower training FLOPs (x3) of one batch described by ``image_grid_thw`` [(t,h,w)]."""
    if image_grid_thw is None:
        return 0
    grid = np.asarray(image_grid_thw, dtype=np.int64)
    if grid.size == 0:
        return 0
    if grid.ndim != 2 or grid.shape[1] != 3:
        raise ValueError(f"Expected image_grid_thw with shape (num_images, 3), got {grid.shape}.")
    vis = cfg.vision
    m = vis.spatial_merge_size
    n_i = grid[:, 0] * grid[:, 1] * grid[:, 2]
    N = int(n_i.sum())
    N2 = int((n_i * n_i).sum())
    Nm = int((grid[:, 0] * (grid[:, 1] // m) * (grid[:, 2] // m)).sum())
    if N <= 0 or Nm <= 0:
        return 0
    D, F, H = vis.hidden_size, vis.intermediate_size, vis.num_heads
    K = D // H
    in_feat = vis.in_channels * vis.temporal_patch_size * vis.patch_size ** 2
    block = 2 * N * D * 3 * D + 4 * N2 * H * K + 2 * N * D * D + 4 * N * D * F
    md = D * m * m
    mergers = (1 + len(vis.deepstack_visual_indexes)) * (2 * Nm * md * md + 2 * Nm * md * vis.out_hidden_size)
    return (2 * N * in_feat * D + vis.depth * block + mergers) * TRAINING_FLOP_MULTIPLIER


def device_count() -> int:
    import torch.distributed as dist

    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def per_device_flops_per_step(cfg, seq_len: int, batch_size: int, image_grid_thw: Any | None = None) -> float:
    """Training FLOPs of one step over the global batch, divided by the device count."""
    total = training_flops_per_token(cfg, seq_len) * seq_len * batch_size
    if hasattr(cfg, "vision") and hasattr(cfg, "emb_dim"):
        total += qwen3_vl_vision_training_flops(cfg, image_grid_thw)
    return total / max(1, device_count())


class StepTimer:
    """Host wall-clock between step dispatches; the first ``warmup`` deltas are zero."""

    def __init__(self, warmup: int = 2):
        self._warmup = warmup
        self._n = 0
        self._last = datetime.datetime.now()

    def step(self) -> datetime.timedelta:
        now = datetime.datetime.now()
        d = now - self._last
        self._last = now
        self._n += 1
        return datetime.timedelta(0) if self._n <= self._warmup else d


class DeviceStepTimer:
    """Step time from CUDA events on the compute stream, reduced with max over ranks.

    ``step()`` records an event; the time of step i is available once step i+1 has been
    recorded, and is read without stalling the newest step (the read synchronises only on
    an event that is already one step old)."""

    def __init__(self, warmup: int = 2, group=None):
        self._warmup = warmup
        self._events = []
        self._group = group
        self._n = 0

    def step(self) -> datetime.timedelta:
        if not torch.cuda.is_available():
            return datetime.timedelta(0)
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self._events.append(ev)
        self._n += 1
        if len(self._events) < 3 or self._n <= self._warmup + 2:
            if len(self._events) > 3:
                self._events.pop(0)
            return datetime.timedelta(0)
        a, b = self._events[0], self._events[1]
        b.synchronize()
        ms = a.elapsed_time(b)
        self._events.pop(0)
        if self._group is not None or device_count() > 1:
            import torch.distributed as dist

            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self._group)
            ms = float(t.item())
        return datetime.timedelta(milliseconds=ms)


def step_metrics(per_device_flops: float, step_delta: datetime.timedelta, global_tokens_per_step: int,
                 peak_tflops: float | None) -> dict[str, float]:
    sec = step_delta.total_seconds()
    if sec <= 0:
        return dict(step_time_s=0.0, global_tokens_per_sec=0.0, tokens_per_sec_per_device=0.0,
                    tflops_per_device=0.0, mfu=0.0)
    n = device_count()
    gtps = global_tokens_per_step / sec
    fps = per_device_flops / sec
    return dict(step_time_s=sec, global_tokens_per_sec=gtps, tokens_per_sec_per_device=gtps / n,
                tflops_per_device=fps / 1e12, mfu=(fps / (peak_tflops * 1e12)) if peak_tflops else 0.0)


def maybe_log_step_metrics(step_to_log: int, metrics_to_log: dict[str, Any], step_delta: datetime.timedelta, *,
                           is_primary_process: bool, log_every: int, force: bool = False,
                           per_device_flops: float, global_tokens_per_step: int,
                           peak_tflops: float | None, wandb_run: Any = None, batch_size: int = 0,
                           jsonl_file=None) -> dict[str, float] | None:
    """Compute and emit the metrics of one step when it is due; returns them or None."""
    due = is_primary_process and log_every and step_to_log % log_every == 0
    if not (due or force):
        return None
    host = {k: float(v) for k, v in metrics_to_log.items()}
    missing = [k for k in ("loss", "grad_norm") if k not in host]
    if missing:
        raise KeyError(f"Missing required metrics for logging: {missing}")
    host["step"] = step_to_log
    if batch_size > 0:
        host["total_samples"] = step_to_log * batch_size
    host.update(step_metrics(per_device_flops, step_delta, global_tokens_per_step, peak_tflops))
    if wandb_run is not None and is_primary_process:
        wandb_run.log({f"train/{k}": v for k, v in host.items() if k != "step"}, step=step_to_log)
    if jsonl_file is not None and is_primary_process:
        import json

        jsonl_file.write(json.dumps(host) + "\n")
        jsonl_file.flush()
    return host

"""Logical-axis sharding rules and activation layouts.

The mesh has three named axes ``("tp", "fsdp", "dp")`` plus an optional expert axis
``"ep"`` that reuses the fsdp x dp ranks.  A rule maps a logical tensor axis to the mesh
axis (or axes) it is split over; axes of size one are dropped.  The runtime in
``omegalax_b200.parallel`` reads these rules to decide which dimension of which parameter
is split over which process group (reference: omegalax/models/shard_config.py:12-87).
"""
from __future__ import annotations

import dataclasses
from typing import Mapping

Axis = str | tuple[str, ...] | None

DEFAULT_AXIS_RULES: tuple[tuple[str, Axis], ...] = (
    ("batch", ("dp", "fsdp")),
    ("vocab", "tp"),
    ("embed", "fsdp"),
    ("hidden", None),
    ("heads", "tp"),
    ("kv_heads", "tp"),
    ("mlp", "tp"),
    ("experts", "ep"),
)


def _filter_axis(axis: Axis, mesh_shape: Mapping[str, int]) -> Axis:
    if axis is None:
        return None
    axes = (axis,) if isinstance(axis, str) else tuple(axis)
    kept = tuple(a for a in axes if mesh_shape.get(a, 1) > 1)
    if not kept:
        return None
    return kept[0] if len(kept) == 1 else kept


def axis_rules_for_mesh(mesh_shape: Mapping[str, int]) -> tuple[tuple[str, Axis], ...]:
    """Rules with every size-one mesh axis removed (that dimension is replicated)."""
    return tuple((name, _filter_axis(ax, mesh_shape)) for name, ax in DEFAULT_AXIS_RULES)


@dataclasses.dataclass(frozen=True)
class ShardConfig:
    """Activation layouts as tuples of mesh axes per tensor dimension."""

    act_btd: tuple[Axis, ...]
    act_btf: tuple[Axis, ...]
    act_btnh: tuple[Axis, ...]

    @property
    def logits_btv(self) -> tuple[Axis, ...]:
        return (self.act_btd[0], None, self.act_btf[2])

    @staticmethod
    def no_sharding() -> "ShardConfig":
        return ShardConfig((None, None, None), (None, None, None), (None, None, None, None))

    @staticmethod
    def default() -> "ShardConfig":
        b = ("dp", "fsdp")
        return ShardConfig((b, None, None), (b, None, "tp"), (b, None, "tp", None))


def shard_config_for_mesh(cfg: ShardConfig, mesh_shape: Mapping[str, int]) -> ShardConfig:
    return ShardConfig(**{
        f.name: tuple(_filter_axis(a, mesh_shape) for a in getattr(cfg, f.name))
        for f in dataclasses.fields(cfg)
    })

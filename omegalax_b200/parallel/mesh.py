"""Device mesh over ``torch.distributed`` ranks: axes ("tp", "fsdp", "dp"), one process per GPU.

Rank layout is tp-fastest: rank = (dp_i * fsdp + fsdp_i) * tp + tp_i.  Process groups are
created lazily per axis; an expert-parallel group spans the fsdp x dp ranks of one tp
slice.  The helper functions mirror omegalax/distributed/mesh.py:17-126 (mesh creation
with conflict checks, data-parallel size/index, per-process batch size).
"""
from __future__ import annotations

import contextlib
import dataclasses
import os

import torch
import torch.distributed as dist

AXES = ("tp", "fsdp", "dp")
_ACTIVE: "Mesh | None" = None


def world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


@dataclasses.dataclass
class Mesh:
    tp: int
    fsdp: int
    dp: int
    _groups: dict = dataclasses.field(default_factory=dict, repr=False)

    @property
    def shape(self) -> dict[str, int]:
        return {"tp": self.tp, "fsdp": self.fsdp, "dp": self.dp, "ep": self.fsdp * self.dp}

    @property
    def size(self) -> int:
        return self.tp * self.fsdp * self.dp

    def coords(self, r: int | None = None) -> dict[str, int]:
        r = rank() if r is None else r
        return {"tp": r % self.tp, "fsdp": (r // self.tp) % self.fsdp, "dp": r // (self.tp * self.fsdp)}

    def ranks_along(self, axis: str, r: int | None = None) -> list[int]:
        """Global ranks that differ from ``r`` only along ``axis`` ("shard" = fsdp x dp)."""
        c = self.coords(r)
        out = []
        if axis == "shard" or axis == "ep":
            for d in range(self.dp):
                for f in range(self.fsdp):
                    out.append((d * self.fsdp + f) * self.tp + c["tp"])
            return out
        for i in range(getattr(self, axis)):
            cc = dict(c)
            cc[axis] = i
            out.append((cc["dp"] * self.fsdp + cc["fsdp"]) * self.tp + cc["tp"])
        return out

    def group(self, axis: str):
        """Process group along an axis; None when the axis has a single member."""
        n = self.fsdp * self.dp if axis in ("shard", "ep") else getattr(self, axis)
        if n == 1 or world_size() == 1:
            return None
        if axis not in self._groups:
            mine = None
            seen = set()
            for r in range(self.size):
                members = tuple(self.ranks_along(axis, r))
                if members in seen:
                    continue
                seen.add(members)
                g = dist.new_group(list(members))
                if rank() in members:
                    mine = g
            self._groups[axis] = mine
        return self._groups[axis]


def make_mesh(tp_size: int, fsdp_size: int, dp_size: int) -> Mesh:
    n = tp_size * fsdp_size * dp_size
    if n != world_size():
        raise ValueError(f"mesh {tp_size}x{fsdp_size}x{dp_size} = {n} does not match the "
                         f"number of processes ({world_size()})")
    return Mesh(tp_size, fsdp_size, dp_size)


def set_default_mesh(mesh: Mesh | None) -> None:
    global _ACTIVE
    _ACTIVE = mesh


def current_mesh() -> Mesh | None:
    return _ACTIVE


def ensure_mesh(*, tp_size: int | None = None, fsdp_size: int | None = None,
                dp_size: int | None = None) -> Mesh:
    """Return the active mesh, creating it when none exists.  All three sizes are required
    to create one; sizes that are given must agree with an existing mesh."""
    global _ACTIVE
    if _ACTIVE is not None:
        for name, val in (("tp", tp_size), ("fsdp", fsdp_size), ("dp", dp_size)):
            if val is not None and getattr(_ACTIVE, name) != val:
                raise ValueError(f"active mesh has {name}={getattr(_ACTIVE, name)}, requested {val}")
        return _ACTIVE
    if tp_size is None or fsdp_size is None or dp_size is None:
        raise ValueError("tp_size, fsdp_size and dp_size are all required when no mesh is active")
    _ACTIVE = make_mesh(tp_size, fsdp_size, dp_size)
    return _ACTIVE


@contextlib.contextmanager
def mesh_rules(mesh: Mesh):
    """Make ``mesh`` the active mesh inside the block."""
    global _ACTIVE
    prev = _ACTIVE
    _ACTIVE = mesh
    try:
        yield mesh
    finally:
        _ACTIVE = prev


@contextlib.contextmanager
def mesh_rules_for(*, tp_size: int, fsdp_size: int, dp_size: int):
    prev = _ACTIVE
    set_default_mesh(None)
    try:
        with mesh_rules(make_mesh(tp_size, fsdp_size, dp_size)) as m:
            yield m
    finally:
        set_default_mesh(prev)


def required_batch_multiple(mesh: Mesh | None = None) -> int:
    """The global batch is split over the dp and fsdp axes."""
    mesh = mesh or _ACTIVE
    return 1 if mesh is None else mesh.dp * mesh.fsdp


def data_parallel_size(dp_size: int | None = None) -> int:
    """Number of distinct input shards (defaults to the number of batch-sharding ranks)."""
    if dp_size is not None:
        return dp_size
    return required_batch_multiple() if _ACTIVE is not None else world_size()


def data_parallel_index(dp_size: int | None = None) -> int:
    n = data_parallel_size(dp_size)
    if _ACTIVE is not None and dp_size is None:
        c = _ACTIVE.coords()
        return c["dp"] * _ACTIVE.fsdp + c["fsdp"]
    return rank() % n


def process_local_batch_size(global_batch: int, dp_size: int | None = None) -> int:
    n = data_parallel_size(dp_size)
    if global_batch % n:
        raise ValueError(f"global batch {global_batch} is not divisible by data-parallel size {n}")
    return global_batch // n


def init_distributed(backend: str | None = None) -> None:
    """Initialise torch.distributed from the torchrun environment (no-op single process)."""
    if dist.is_initialized() or "RANK" not in os.environ or int(os.environ.get("WORLD_SIZE", "1")) == 1:
        return
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group(backend, device_id=torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))))
    else:
        dist.init_process_group(backend)

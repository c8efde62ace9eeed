"""Sharded, resumable training checkpoints.

Layout under ``save_dir``::

    config.json                      HF-format model config (written once at start)
    000050/                          one directory per saved step (6 digits)
        manifest.json                step, world size, per-parameter global shape / sharding
        rank00000.safetensors        this rank's fp32 shards: <name>.master / .exp_avg / .exp_avg_sq
        input_iter_00000.json        data-iterator state of this rank
        rng_00000.pt                 torch RNG state of this rank

A step directory is written under a temporary name and renamed when every rank is done, so a
crash never leaves a half-written checkpoint; only the newest ``max_to_keep`` are kept.  The
device->host copy happens on the caller's stream; file writing runs on a background thread at
any world size: every rank's thread writes its own files and then a ``rankNNNNN.ok`` marker (or
``.err``), rank 0's thread waits for all markers and only then renames, and the next
``wait_until_finished`` agrees on the outcome over the process group, so a failed write on any
rank neither produces a "valid" checkpoint nor prunes an older good one.
Restore reshards: a checkpoint written with W ranks can be read with any other shard count.
(The reference keeps the same items -- train state incl. optimizer moments and step counters,
rng, input iterator -- through orbax: omegalax/trainers/text.py:94-155,
omegalax/trainers/checkpoint_utils.py:13-43.)
"""
from __future__ import annotations

import json
import os
import shutil
import threading
import time
import warnings
from pathlib import Path
from typing import Any, Protocol

import torch
import torch.distributed as dist


class CheckpointableIterator(Protocol):
    def get_state(self) -> dict: ...
    def set_state(self, state: dict) -> None: ...


def _barrier():
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def _rank():
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _world():
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def _all_ranks_ok(ok: bool) -> bool:
    """Minimum of a success flag over the default process group."""
    if _world() == 1:
        return ok
    dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
    t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(int(t.item()))


class CheckpointUnreadable(RuntimeError):
    """A step directory whose manifest or shard files cannot be opened."""


class CheckpointManager:
    def __init__(self, save_dir: str | os.PathLike, *, save_interval_steps: int | None = None,
                 max_to_keep: int = 2, async_write: bool = True):
        self.dir = Path(save_dir).expanduser().resolve()
        self.dir.mkdir(parents=True, exist_ok=True)
        self.interval = save_interval_steps
        self.max_to_keep = max_to_keep
        self.async_write = async_write
        self._thread: threading.Thread | None = None
        self._error: BaseException | None = None
        self._pending = False          # a save whose outcome the ranks have not agreed on yet
        self.peer_write_timeout_s = 1800.0
        if _rank() == 0:
            self.cleanup_tmp_directories()
        _barrier()

    # ---------------------------------------------------------------- discovery
    def all_steps(self) -> list[int]:
        out = []
        for p in self.dir.iterdir():
            if p.is_dir() and p.name.isdigit() and (p / "manifest.json").exists():
                out.append(int(p.name))
        return sorted(out)

    def latest_step(self) -> int | None:
        steps = self.all_steps()
        return steps[-1] if steps else None

    def cleanup_tmp_directories(self) -> None:
        for p in self.dir.glob("*.tmp"):
            shutil.rmtree(p, ignore_errors=True)

    def step_dir(self, step: int) -> Path:
        return self.dir / f"{step:06d}"

    # ---------------------------------------------------------------- save
    def save(self, step: int, engine, input_iter: CheckpointableIterator | None = None,
             extra: dict[str, Any] | None = None) -> None:
        """Snapshot the engine's shards on the host, then write them in the background."""
        self.wait_until_finished()
        r, w = _rank(), _world()
        tensors: dict[str, torch.Tensor] = {}
        params = []
        for slot, master, m1, m2 in engine.named_master_shards():
            for suffix, t in ((".master", master), (".exp_avg", m1), (".exp_avg_sq", m2)):
                tensors[slot.name + suffix] = t.detach().to("cpu", copy=True)
            params.append({"name": slot.name, "shape": list(slot.shape), "sharded": bool(slot.sharded),
                           "shard_numel": int(slot.shard_numel),
                           "tp_sharded": bool(getattr(slot, "tp_sharded", False)),
                           "ep_product": bool(getattr(slot, "ep_product", False))})
        manifest = {"step": int(step), "world_size": w, "shard_world": int(engine.W),
                    "tp_world": int(getattr(engine, "TP", 1)),
                    "optimizer_step": int(engine.step_count), "params": params, "extra": extra or {}}
        iter_state = input_iter.get_state() if input_iter is not None else None
        manifest["has_iter_state"] = iter_state is not None
        rng_state = {"cpu": torch.get_rng_state()}
        tmp = self.dir / f"{step:06d}.tmp"
        final = self.step_dir(step)
        if r == 0:
            tmp.mkdir(parents=True, exist_ok=True)
        _barrier()

        def write():
            try:
                from safetensors.torch import save_file

                save_file(tensors, str(tmp / f"rank{r:05d}.safetensors"))
                if iter_state is not None:
                    (tmp / f"input_iter_{r:05d}.json").write_text(json.dumps(iter_state))
                torch.save(rng_state, tmp / f"rng_{r:05d}.pt")
                if r == 0:
                    (tmp / "manifest.json").write_text(json.dumps(manifest))
                (tmp / f"rank{r:05d}.ok").write_text("ok")
            except BaseException as e:  # surfaced by wait_until_finished
                self._error = e
                try:
                    (tmp / f"rank{r:05d}.err").write_text(repr(e))
                except Exception:
                    pass

        def write_and_finish():
            write()
            if r != 0:
                return
            # rank 0 renames once every rank's marker is there; no collective runs on this thread
            t0 = time.monotonic()
            while self._error is None:
                if any(tmp.glob("rank*.err")):
                    self._error = RuntimeError("a peer rank failed to write its checkpoint shard")
                    break
                if len(list(tmp.glob("rank*.ok"))) >= w:
                    break
                if time.monotonic() - t0 > self.peer_write_timeout_s:
                    self._error = TimeoutError("peer ranks did not finish writing their checkpoint shards")
                    break
                time.sleep(0.01)
            self._finalize(tmp, final)

        self._pending = True
        if self.async_write:
            self._thread = threading.Thread(target=write_and_finish, daemon=True)
            self._thread.start()
        else:
            write_and_finish()
            self.wait_until_finished()

    def _finalize(self, tmp: Path, final: Path) -> None:
        if self._error is not None:
            return
        for marker in list(tmp.glob("rank*.ok")):
            marker.unlink(missing_ok=True)
        if final.exists():
            shutil.rmtree(final)
        os.replace(tmp, final)
        steps = self.all_steps()
        for s in steps[:-self.max_to_keep] if self.max_to_keep else []:
            shutil.rmtree(self.step_dir(s), ignore_errors=True)

    def wait_until_finished(self) -> None:
        """Join the writer thread; with several ranks, agree on the outcome (a collective: every
        rank calls this at the same point of the loop, as ``save`` / ``restore`` / ``close`` do)."""
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._pending:
            self._pending = False
            everyone_ok = _all_ranks_ok(self._error is None)
            if self._error is None and not everyone_ok:
                self._error = RuntimeError("another rank failed to write its checkpoint shard")
        if self._error is not None:
            e, self._error = self._error, None
            raise RuntimeError("checkpoint write failed") from e

    def close(self) -> None:
        self.wait_until_finished()

    # ---------------------------------------------------------------- restore
    def _open_step(self, step: int):
        """Manifest and open shard files of one step; ``CheckpointUnreadable`` names the file that
        is missing, truncated or not a safetensors file (nothing has been loaded at that point)."""
        from safetensors import safe_open

        d = self.step_dir(step)
        try:
            manifest = json.loads((d / "manifest.json").read_text())
        except (OSError, ValueError) as e:
            raise CheckpointUnreadable(f"checkpoint step {step}: manifest.json is unreadable ({e})") from e
        files = []
        for i in range(manifest["world_size"]):
            path = d / f"rank{i:05d}.safetensors"
            try:
                files.append(safe_open(str(path), framework="pt"))
            except Exception as e:
                raise CheckpointUnreadable(f"checkpoint step {step}: shard {path.name} is unreadable "
                                           f"({type(e).__name__}: {e})") from e
        return manifest, files

    def restore(self, step: int | None, engine, input_iter: CheckpointableIterator | None = None) -> dict:
        """Load master weights and moments into ``engine`` (resharding if needed), the data
        iterator state and the RNG state.  Returns the manifest."""
        from safetensors import safe_open

        self.wait_until_finished()
        if step is None:
            # the newest step whose manifest and shard files all open; a damaged newest step (a
            # truncated or corrupted shard file) is skipped with a warning in favour of the one before
            candidates = sorted(self.all_steps(), reverse=True)
            if not candidates:
                raise ValueError("No checkpoint found to restore.")
            err = None
            for cand in candidates:
                try:
                    manifest, files = self._open_step(cand)
                    step = cand
                    break
                except CheckpointUnreadable as e:
                    warnings.warn(f"{e}; trying the step before it")
                    err = e
            else:
                raise err
        else:
            manifest, files = self._open_step(step)
        d = self.step_dir(step)
        saved_w = manifest["shard_world"]
        saved_tp = int(manifest.get("tp_world", manifest["world_size"] // saved_w))
        tp, tp_rank = int(getattr(engine, "TP", 1)), int(getattr(engine, "tp_rank", 0))
        meta = {p["name"]: p for p in manifest["params"]}
        # ranks are laid out (shard, tp) with tp fastest: shard rank i, tensor-parallel rank t wrote
        # the file of global rank i * saved_tp + t
        per = saved_tp

        def saved_full(key, pm, t):
            """Tensor-parallel rank t's whole (un-sharded over fsdp) value, flat."""
            if pm["sharded"]:
                return torch.cat([files[i * per + t].get_tensor(key).reshape(-1) for i in range(saved_w)])
            return files[t].get_tensor(key).reshape(-1)

        r = _rank()
        model_names = {id(p): n for n, p in engine.model.named_parameters()} if saved_tp != tp else {}
        for slot, master, m1, m2 in engine.named_master_shards():
            if slot.name not in meta:
                raise RuntimeError(f"checkpoint has no entry for parameter '{slot.name}'")
            pm = meta[slot.name]
            retile = saved_tp != tp and (pm.get("tp_sharded", False) or getattr(slot, "tp_sharded", False))
            if list(slot.shape) != pm["shape"] and not retile:
                raise RuntimeError(f"shape mismatch for '{slot.name}': {pm['shape']} vs {list(slot.shape)}")
            t = tp_rank if (saved_tp == tp and pm.get("tp_sharded", False)) else 0
            # experts cut over every rank of the job (shard group x tensor-parallel group), on either
            # side: assemble the whole tensor and take this rank's piece under the current layout
            product = bool(pm.get("ep_product", False) or getattr(slot, "ep_product", False))
            srank = int(getattr(slot, "shard_rank", engine.rank))
            for suffix, dst in ((".master", master), (".exp_avg", m1), (".exp_avg_sq", m2)):
                key = slot.name + suffix
                if product:
                    if pm.get("ep_product", False):   # piece j is in the file of global rank j
                        full = torch.cat([f.get_tensor(key).reshape(-1) for f in files])
                    else:                             # the other layout keeps experts identical over tp
                        full = saved_full(key, pm, 0)
                    src = full[srank * slot.shard_numel:(srank + 1) * slot.shard_numel] if slot.sharded else full
                elif retile:
                    full = _retile_tp(model_names[id(slot.param)], [saved_full(key, pm, i).view(pm["shape"]) for i in range(saved_tp)],
                                      engine, tp, tp_rank)
                    if list(full.shape) != list(slot.shape):
                        raise RuntimeError(f"shape mismatch for '{slot.name}' after changing the tensor-parallel "
                                           f"degree {saved_tp} -> {tp}: {list(full.shape)} vs {list(slot.shape)}")
                    full = full.reshape(-1)
                    src = full[engine.rank * slot.shard_numel:(engine.rank + 1) * slot.shard_numel] if slot.sharded else full
                elif pm["sharded"] == slot.sharded and (not slot.sharded or saved_w == engine.W):
                    src = files[(engine.rank * per if slot.sharded and len(files) > 1 else 0) + t].get_tensor(key)
                    if slot.sharded and len(files) == 1 and saved_w == 1:
                        src = src.reshape(-1)
                else:
                    full = saved_full(key, pm, t)
                    if slot.sharded:
                        src = full[engine.rank * slot.shard_numel:(engine.rank + 1) * slot.shard_numel]
                    else:
                        src = full
                dst.copy_(src.reshape(-1).to(dst.device))
        engine.step_count = int(manifest["optimizer_step"])
        engine.sync_compute_from_master()
        if input_iter is not None:
            p = d / f"input_iter_{r:05d}.json"
            if int(manifest["world_size"]) != _world():
                warnings.warn(f"checkpoint step {step} was written by {manifest['world_size']} ranks and is read by "
                              f"{_world()}: per-rank data-iterator states do not carry over, rank {r} "
                              + ("reuses the state of the same rank index" if p.exists() else "restarts its data iterator"),
                              RuntimeWarning, stacklevel=2)
            elif not p.exists() and manifest.get("has_iter_state", False):
                raise RuntimeError(f"checkpoint step {step} has no data-iterator state for rank {r} ({p.name})")
            if p.exists():
                input_iter.set_state(json.loads(p.read_text()))
        p = d / f"rng_{r:05d}.pt"
        if p.exists():
            torch.set_rng_state(torch.load(p, weights_only=False)["cpu"])
        return manifest


def _retile_tp(name: str, parts: list, engine, tp: int, tp_rank: int):
    """Per-rank slices written with one tensor-parallel degree -> the slice of rank ``tp_rank`` under
    degree ``tp`` (moments are laid out like the weights, so the same rule serves all three)."""
    import importlib

    tp_layout = importlib.import_module(getattr(engine.model, "TP_LAYOUT", "omegalax_b200.models.qwen3.tp_layout"))
    cfg = getattr(engine.model, "cfg", None)
    if cfg is None or not hasattr(engine.model, "tp_size"):
        raise RuntimeError("changing the tensor-parallel degree on restore needs a model with a tensor-parallel layout")
    full = tp_layout.tp_unslice(name, parts, cfg) if len(parts) > 1 else parts[0]
    return tp_layout.tp_slice(name, full, cfg, tp, tp_rank)

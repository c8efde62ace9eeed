"""SFT training for text-only causal language models (Qwen3, Qwen3.5 text).

    run_sft(model_id, TrainConfig(...), data_iter, save_dir=..., tp_size=1, fsdp_size=8, dp_size=1)

One process drives one GPU (launch with torchrun).  The step is: pinned-host -> device copy
of the batch, forward through the sharded engine (full remat), fused linear-cross-entropy,
backward with per-layer gradient reduce-scatter, clip + AdamW on the fp32 shard.  Metrics
are logged one step late so the host never waits on the newest step.
API parity: omegalax/trainers/text.py:43-429.
"""
from __future__ import annotations

import dataclasses
import datetime
import json
import os
from pathlib import Path

import torch
import torch.distributed as dist

from .. import export as export_lib
from ..models.hf_io import save_hf_config
from ..parallel import mesh as mesh_lib
from ..text import api as text_api
from . import checkpoint_utils
from .loss import chunked_cross_entropy_loss, supervised_count
from .lr_schedule import build_lr_schedule
from .optim import MixedPrecisionOptimizer
from .perf import DeviceStepTimer, StepTimer, maybe_log_step_metrics, per_device_flops_per_step

_NUM_LOSS_TILES = 4


def is_primary() -> bool:
    return mesh_lib.rank() == 0


def startup_log(msg: str) -> None:
    if os.environ.get("OMEGALAX_STARTUP_LOG", "1") == "0" or not is_primary():
        return
    print(f"[startup] {msg}", flush=True)


@dataclasses.dataclass(frozen=True)
class TrainConfig:
    seed: int = 0
    batch_size: int = 8          # global batch per micro-step
    seq_len: int = 64
    num_steps: int = 20
    learning_rate: float = 3e-4
    weight_decay: float = 0.01
    warmup_steps: int = 0
    lr_schedule: str = "linear"
    lr_end_factor: float = 0.0
    lr_stable_fraction: float = 0.8
    max_grad_norm: float = 0.0
    grad_accum_steps: int = 1
    print_every: int = 1
    remat_policy: str = "full"
    ep_size: int = 0             # expert parallelism: 0 automatic (over the shard group when experts and peer
                                 # memory exist), 1 off (experts travel like any sharded parameter), the
                                 # shard-group size, or shard-group size x tp size (experts over every rank of
                                 # the job while attention is tensor-parallel; library all-to-all transport)
    ep_transport: str = "auto"   # "auto": the peer-memory exchange kernels where GPUs can map each other's
                                 # memory, else experts travel like any sharded parameter; "a2a": library
                                 # all-to-all on any transport (NCCL baseline, CPU ranks)


def init_model(cfg_or_model_id, rng: int = 0, *, tp_size=None, fsdp_size=None, dp_size=None, **kw):
    return text_api.init_model(cfg_or_model_id, rng, tp_size=tp_size, fsdp_size=fsdp_size, dp_size=dp_size, **kw)


def build_optimizer(model, train_cfg: TrainConfig, *, device=None, init_from_model: bool | None = None):
    """Wrap ``model`` in the sharded mixed-precision AdamW engine.  Parameters on the meta
    device are initialised shard-by-shard; real parameters are adopted as the fp32 master."""
    mesh = mesh_lib.current_mesh()
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    sched = build_lr_schedule(train_cfg.lr_schedule, train_cfg.learning_rate, train_cfg.num_steps,
                              train_cfg.warmup_steps, train_cfg.lr_end_factor, train_cfg.lr_stable_fraction)
    group = mesh.group("shard") if mesh is not None else None
    tp_group = mesh.group("tp") if mesh is not None and mesh.tp > 1 else None
    if tp_group is not None:
        from ..parallel import tp as tp_lib

        tp_lib.set_current(tp_lib.TPContext(tp_group))
    if init_from_model is None:
        init_from_model = not any(p.device.type == "meta" for p in model.parameters())
    shard_world = dist.get_world_size(group) if group is not None else 1
    tp_world = dist.get_world_size(tp_group) if tp_group is not None else 1
    if train_cfg.ep_size not in (0, 1, shard_world, shard_world * tp_world):
        raise ValueError(f"ep_size={train_cfg.ep_size}: experts are sharded over the shard group ({shard_world} ranks "
                         f"here) or over shard group x tensor-parallel group ({shard_world * tp_world}); use 0 "
                         f"(automatic: the shard group), 1 (off), {shard_world} or {shard_world * tp_world}")
    ep_over_tp = tp_world > 1 and train_cfg.ep_size == shard_world * tp_world
    return MixedPrecisionOptimizer(
        model, device=device, shard_group=group, lr=train_cfg.learning_rate, weight_decay=train_cfg.weight_decay,
        max_grad_norm=train_cfg.max_grad_norm, remat=train_cfg.remat_policy, seed=train_cfg.seed,
        init_from_model=init_from_model, lr_schedule=sched, grad_accum_steps=train_cfg.grad_accum_steps,
        tp_group=tp_group,
        expert_parallel=False if train_cfg.ep_size == 1 else ("a2a" if (train_cfg.ep_transport == "a2a" or ep_over_tp) else True),
        ep_over_tp=ep_over_tp)


def tp_rows_loss(model, rows, tok, mask, count):
    """Cross-entropy of this tensor-parallel rank's sequence-parallel rows [B*T/tp, D] against the
    shifted tokens: its share of the global masked mean (the shares add up over the tp group).
    A head split over the vocabulary scores all rows against its slice instead."""
    from ..ops import functional as Fn
    from ..parallel import tp as tp_lib

    tp = tp_lib.current()
    B, T = tok.shape
    m = B * T // tp.size
    tgt = torch.roll(tok, -1, dims=1).reshape(-1)
    msk = torch.roll(mask, -1, dims=1).to(torch.float32)
    msk[:, -1] = 0
    sl = slice(tp.rank * m, (tp.rank + 1) * m)
    if getattr(model, "vocab_parallel", False):   # head split over the vocabulary: all rows, this rank's slice
        return Fn.linear_cross_entropy_vocab_parallel(rows, model.lm_head.weight, tgt, msk.reshape(-1),
                                                      1.0 / count.clamp_min(1.0), tp)
    return Fn.linear_cross_entropy(rows, model.lm_head.weight, tgt[sl], msk.reshape(-1)[sl],
                                   1.0 / count.clamp_min(1.0))


def _loss_and_count(model, cfg, batch, pad_id: int, group):
    tok = batch["token_ids_BT"]
    mask = batch["loss_mask_BT"]
    count = supervised_count(mask, group)
    if getattr(model, "tp_size", 1) > 1:
        # sequence-parallel rows: this tp rank scores its own slice of the (shifted) token rows
        seg = (tok != pad_id).to(torch.int32)
        rows, aux = model(tok, seg, None, 0, return_local_rows=True)
        return tp_rows_loss(model, rows, tok, mask, count), aux / model.tp_size, count
    hidden, aux = text_api.forward(model, tok, pad_id, cfg)
    ce = chunked_cross_entropy_loss(hidden, model.lm_head.weight, tok, mask, num_tiles=_NUM_LOSS_TILES, count=count)
    return ce, aux, count


def make_sft_train_step(cfg, pad_id: int = 0):
    """Returns ``step(optimizer, batch) -> (loss, metrics)``.  ``batch`` holds device tensors
    ``token_ids_BT``, ``attention_mask_BT``, ``loss_mask_BT`` (this rank's rows).  The loss is
    the global masked mean (normalised by the supervised-token count over all data ranks)
    plus the auxiliary router loss (computed from the router statistics of all data ranks; each
    rank adds its 1/W share)."""

    def sft_train_step(optimizer: MixedPrecisionOptimizer, batch: dict):
        group = optimizer.group
        ce, aux, count = _loss_and_count(optimizer.model, cfg, batch, pad_id, group)
        loss = ce + aux / optimizer.W
        loss.backward()
        gnorm = optimizer.update()
        loss_d = loss.detach()
        if optimizer.W > 1:
            loss_d = loss_d.clone()
            dist.all_reduce(loss_d, group=group)
        if optimizer.TP > 1:
            loss_d = loss_d.clone()
            dist.all_reduce(loss_d, group=optimizer.tp_group)
        metrics = {"loss": loss_d, "supervised_tokens": count.squeeze(0),
                   "grad_norm": gnorm if gnorm is not None else torch.zeros((), device=loss_d.device)}
        return loss_d, metrics

    return sft_train_step


def make_sft_eval_step(cfg, pad_id: int = 0):
    def sft_eval_step(model, batch: dict, group=None):
        with torch.no_grad():
            ce, aux, count = _loss_and_count(model, cfg, batch, pad_id, group)
            W = dist.get_world_size(group) if group is not None else 1
            loss = ce + aux / W          # ce is this rank's share of the global mean; aux is averaged
            if W > 1:
                dist.all_reduce(loss, group=group)
        return loss, count.squeeze(0)

    return sft_eval_step


def _device_health_check(optimizer, use_cuda: bool) -> None:
    """Raise if any kernel gave up on a bounded wait, or if an expert-parallel receive buffer
    overflowed, since the last check.  Called wherever the loop already synchronises (metric
    read-out, checkpoint write) and always *before* a checkpoint is written, so that a step
    computed from partial kernel output can never replace a good checkpoint."""
    if not use_cuda:
        return
    from ..ops import lib

    lib.check_status()
    ep = getattr(optimizer, "_ep", None)
    if ep is not None:
        ep.check()


def _write_checkpoint_config(save_dir: Path, cfg) -> None:
    if is_primary():
        save_hf_config(export_lib.model_config_to_hf_dict(cfg), save_dir)


def run_sft(model_id_or_cfg, train_cfg: TrainConfig, data_iter, *, save_dir=None, save_every: int = 0,
            log_every: int = 1, resume: bool = False, pad_id: int = 0, peak_tflops: float | None = None,
            tp_size: int | None = None, fsdp_size: int | None = None, dp_size: int | None = None,
            profile_dir=None, profile_steps: tuple[int, int] = (3, 8), wandb_run=None, val_data_iter=None,
            val_every: int | None = None, val_steps: int = 10, device=None, log_file=None, _family=None,
            pretrained_loader=None, stop_after_step: int | None = None, step_deadline_s: float | None = None,
            heartbeat_s: float | None = None):
    """SFT from a checkpointable iterator of batch dicts (numpy / CPU tensors, this rank's
    rows).  Returns (optimizer, last logged metrics).  ``stop_after_step`` ends this invocation
    early (after the usual final checkpoint) while keeping the schedule of ``num_steps``.
    ``step_deadline_s`` arms a watchdog that dumps all stacks and exits with code 124 when a step
    takes longer; ``heartbeat_s`` makes every rank publish a heartbeat in the rendezvous store and
    check its peers between steps (``PeerFailure`` instead of a collective that never returns)."""
    fam = _family or _TEXT_FAMILY
    save_path = Path(save_dir).expanduser().resolve() if save_dir is not None else None
    if resume:
        if save_path is None:
            raise ValueError("resume=True requires save_dir to be provided.")
        if not save_path.exists():
            raise ValueError(f"resume=True requires an existing checkpoint directory: {save_path}")
        probe = checkpoint_utils.CheckpointManager(save_path)
        if probe.latest_step() is None:
            raise ValueError(f"resume=True but no checkpoints found under: {save_path}")
        model_cfg = fam.api.resolve_config(str(save_path))
        startup_log(f"resolved model config from checkpoint {str(save_path)!r}")
    else:
        model_cfg = fam.api.resolve_config(model_id_or_cfg)
        startup_log("resolved model config")
    mesh = mesh_lib.ensure_mesh(tp_size=tp_size, fsdp_size=fsdp_size, dp_size=dp_size)
    model_cfg = fam.api.align_config_to_mesh(model_cfg, mesh)
    mult = mesh_lib.required_batch_multiple(mesh)
    if train_cfg.batch_size % mult != 0:
        raise ValueError(f"Global batch size {train_cfg.batch_size} must be divisible by the mesh batch multiple {mult}.")
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    torch.manual_seed(train_cfg.seed)

    with mesh_lib.mesh_rules(mesh):
        model, model_cfg = fam.api.init_model(model_cfg, train_cfg.seed, tp_size=tp_size, fsdp_size=fsdp_size,
                                              dp_size=dp_size, meta=True)
        startup_log("initialized model (meta)")
        optimizer = build_optimizer(model, train_cfg, device=device)
        if pretrained_loader is not None and not resume:
            pretrained_loader(optimizer, model_cfg)
            startup_log("loaded pretrained weights")
    startup_log("built optimizer / materialised shards")
    sft_step = fam.make_train_step(model_cfg, pad_id=pad_id)
    eval_step = fam.make_eval_step(model_cfg, pad_id=pad_id) if val_data_iter is not None else None

    accum = train_cfg.grad_accum_steps
    use_cuda = torch.device(device).type == "cuda"
    timer = DeviceStepTimer(warmup=2 * accum) if use_cuda else StepTimer(warmup=2 * accum)
    global_tokens_per_step = train_cfg.seq_len * train_cfg.batch_size * accum

    manager = None
    if save_path is not None:
        save_path.mkdir(parents=True, exist_ok=True)
        _write_checkpoint_config(save_path, model_cfg)
        manager = checkpoint_utils.CheckpointManager(save_path, save_interval_steps=save_every or None)
        startup_log(f"checkpoint manager ready at {str(save_path)!r}")
    start_step = 0
    if resume:
        manifest = manager.restore(None, optimizer, data_iter)
        start_step = int(manifest["step"])
        startup_log(f"restored checkpoint at step {start_step}")

    jsonl = open(log_file, "a") if (log_file and is_primary()) else None
    last_metrics: dict = {}
    prev = None

    def log_prev(force: bool = False):
        nonlocal last_metrics
        if prev is None:
            return
        s, m, delta, flops = prev
        res = maybe_log_step_metrics(s, m, delta, is_primary_process=is_primary(), log_every=log_every, force=force,
                                     per_device_flops=flops, global_tokens_per_step=global_tokens_per_step,
                                     peak_tflops=peak_tflops, wandb_run=wandb_run, jsonl_file=jsonl)
        if res is not None:
            last_metrics = res
            _device_health_check(optimizer, use_cuda)   # the metric read-out above synchronised already
            if is_primary():
                print(" ".join(f"{k}={v:.6g}" if isinstance(v, float) else f"{k}={v}" for k, v in res.items()), flush=True)

    from ..utils.failure import PeerHeartbeat, StepWatchdog

    watchdog = StepWatchdog(step_deadline_s).start() if step_deadline_s else None
    hb = None
    if heartbeat_s and dist.is_initialized() and dist.get_world_size() > 1:
        hb = PeerHeartbeat(dist.get_rank(), dist.get_world_size(), interval_s=heartbeat_s / 4,
                           max_age_s=heartbeat_s).start()
        hb.wait_all_alive(max(30.0, 4 * heartbeat_s))
    prof = None
    p0, p1 = profile_steps
    startup_log("entering training loop")
    end_step = train_cfg.num_steps if stop_after_step is None else min(train_cfg.num_steps, stop_after_step)
    for step_idx in range(start_step, end_step):
        step = step_idx + 1
        if hb is not None:
            hb.check()   # learn of a lost peer on the host, before launching anything that waits for it
        if profile_dir is not None and step_idx == p0 and prof is None:
            prof = _start_profiler(profile_dir)
        acc_loss = acc_sup = acc_gn = 0.0
        acc_flops = 0.0
        acc_time = datetime.timedelta(0)
        for _ in range(accum):
            batch = next(data_iter)
            acc_flops += per_device_flops_per_step(model_cfg, train_cfg.seq_len, train_cfg.batch_size,
                                                   batch.get("image_grid_thw"))
            batch = fam.api.shard_batch_dict(batch, model_cfg, mesh, device)
            _, metrics = sft_step(optimizer, batch)
            acc_time += timer.step()
            acc_loss = acc_loss + metrics["loss"]
            acc_sup = acc_sup + metrics["supervised_tokens"]
            acc_gn = acc_gn + metrics["grad_norm"]
        if prof is not None and step >= p1:
            _stop_profiler(prof, profile_dir)
            prof = None
        lr = float(optimizer.lr_schedule(step_idx))
        window = {"loss": acc_loss / accum, "grad_norm": acc_gn, "supervised_tokens": acc_sup, "lr": lr}
        log_prev()
        prev = (step, window, acc_time, acc_flops)
        if watchdog is not None:
            watchdog.beat(step)
            watchdog.pause()      # checkpoint writes and evaluation are not steps
        if manager is not None and save_every and step % save_every == 0:
            _device_health_check(optimizer, use_cuda)
            manager.save(step, optimizer, data_iter)
        if eval_step is not None and val_every and step % val_every == 0:
            tot = sup = 0.0
            for _ in range(val_steps):
                vb = fam.api.shard_batch_dict(next(val_data_iter), model_cfg, mesh, device)
                vl, vs = eval_step(optimizer.model, vb, optimizer.group)
                tot += float(vl)
                sup += float(vs)
            if is_primary():
                print(f"val step={step} loss={tot / val_steps:.6g} sup_tokens={sup:.0f}", flush=True)
            if wandb_run is not None and is_primary():
                wandb_run.log({"val/loss": tot / val_steps, "val/sup_tokens": sup}, step=step)
        if watchdog is not None:
            watchdog.resume()
    if watchdog is not None:
        watchdog.stop()
    if prof is not None:
        _stop_profiler(prof, profile_dir)
    log_prev(force=True)
    _device_health_check(optimizer, use_cuda)
    if manager is not None:
        if last_metrics and (not save_every or last_metrics["step"] % save_every != 0):
            manager.save(int(last_metrics["step"]), optimizer, data_iter)
        manager.wait_until_finished()
        manager.close()
    if hb is not None:
        # "left" is published only once this rank is past its last step and its last checkpoint
        # barrier: the step loop has no host synchronisation, so a peer may still be one step behind
        # and must not read "left" before its own last hb.check().
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()
        hb.leave()
        hb.stop()
    if jsonl is not None:
        jsonl.close()
    return optimizer, last_metrics


@dataclasses.dataclass
class _Family:
    api: object
    make_train_step: object
    make_eval_step: object


_TEXT_FAMILY = _Family(text_api, make_sft_train_step, make_sft_eval_step)


def _start_profiler(profile_dir):
    """Kineto trace + allocator history for the profile window; also opens the CUDA
    profiler range so an external profiler attached with capture-range can follow it."""
    from ..utils import profiling

    profiling.enable_scopes(True)     # NVTX ranges named after the modules, for this window only
    Path(profile_dir).mkdir(parents=True, exist_ok=True)
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
        torch.cuda.memory._record_memory_history(max_entries=100000)
        torch.cuda.cudart().cudaProfilerStart()
    prof = torch.profiler.profile(activities=acts)
    prof.__enter__()
    if is_primary():
        print(f"[profiler] starting trace -> {profile_dir}", flush=True)
    return prof


def _stop_profiler(prof, profile_dir):
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaProfilerStop()
        try:
            torch.cuda.memory._dump_snapshot(str(Path(profile_dir) / f"memory_rank{mesh_lib.rank()}.pickle"))
            torch.cuda.memory._record_memory_history(enabled=None)
        except Exception:
            pass
    from ..utils import profiling

    profiling.enable_scopes(False)
    prof.__exit__(None, None, None)
    prof.export_chrome_trace(str(Path(profile_dir) / f"trace_rank{mesh_lib.rank()}.json"))
    if is_primary():
        print("[profiler] stopped trace", flush=True)

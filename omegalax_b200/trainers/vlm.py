"""SFT training for vision-language models (Qwen3.5, Qwen3-VL); API parity with
omegalax/trainers/vlm.py.  The batch dict adds ``pixel_values`` [sum N, C*tp*p*p],
``image_grid_thw`` [M,3], ``vision_cu_seqlens`` and ``position_ids_ZBT`` [3,B,T] to the text
keys; a string model id that names a checkpoint directory loads its pretrained weights
unless the run resumes."""
from __future__ import annotations

import dataclasses
import gc
import os

import torch
import torch.distributed as dist

from ..vlm import api as vlm_api
from . import text as _text
from .loss import chunked_cross_entropy_loss, supervised_count
from .text import build_optimizer  # noqa: F401  (same engine for both families)

_NUM_LOSS_TILES = 4


@dataclasses.dataclass(frozen=True)
class TrainConfig(_text.TrainConfig):
    gc_period: int = 0
    text_attn_backend: str = "sm100"


def init_model(cfg_or_model_id, rng: int = 0, *, tp_size=None, fsdp_size=None, dp_size=None, **kw):
    return vlm_api.init_model(cfg_or_model_id, rng, tp_size=tp_size, fsdp_size=fsdp_size, dp_size=dp_size, **kw)


def _forward_loss(model, cfg, batch, pad_id, group):
    tok, mask = batch["token_ids_BT"], batch["loss_mask_BT"]
    grid = batch.get("image_grid_thw")
    if torch.is_tensor(grid):
        grid = [tuple(int(v) for v in row) for row in grid.tolist()]
    count = supervised_count(mask, group)
    tp = getattr(model, "tp_size", 1)
    hidden, aux = vlm_api.forward(model, tok, pad_id, cfg, attention_mask_BT=batch.get("attention_mask_BT"),
                                  pixel_values=batch.get("pixel_values"), image_grid_thw=grid,
                                  vision_cu_seqlens=batch.get("vision_cu_seqlens"),
                                  position_ids_ZBT=batch.get("position_ids_ZBT"), return_local_rows=tp > 1)
    if tp > 1:   # sequence-parallel rows of this tensor-parallel rank
        return _text.tp_rows_loss(model, hidden, tok, mask, count), aux / tp, count
    ce = chunked_cross_entropy_loss(hidden, model.lm_head.weight, tok, mask, num_tiles=_NUM_LOSS_TILES, count=count)
    return ce, aux, count


def make_sft_train_step(cfg, pad_id: int = 0):
    def sft_train_step(optimizer, batch: dict):
        group = optimizer.group
        ce, aux, count = _forward_loss(optimizer.model, cfg, batch, pad_id, group)
        loss = ce + aux / optimizer.W
        loss.backward()
        gnorm = optimizer.update()
        loss_d = loss.detach()
        if optimizer.W > 1:
            loss_d = loss_d.clone()
            dist.all_reduce(loss_d, group=group)
        if getattr(optimizer, "tp_group", None) is not None:   # per-rank row shares add up over tp
            loss_d = loss_d.clone()
            dist.all_reduce(loss_d, group=optimizer.tp_group)
        return loss_d, {"loss": loss_d, "supervised_tokens": count.squeeze(0),
                        "grad_norm": gnorm if gnorm is not None else torch.zeros((), device=loss_d.device)}

    return sft_train_step


def make_sft_eval_step(cfg, pad_id: int = 0):
    def sft_eval_step(model, batch: dict, group=None):
        with torch.no_grad():
            ce, aux, count = _forward_loss(model, cfg, batch, pad_id, group)
            W = dist.get_world_size(group) if group is not None else 1
            loss = ce + aux / W
            if W > 1:
                dist.all_reduce(loss, group=group)
        return loss, count.squeeze(0)

    return sft_eval_step


_VLM_FAMILY = _text._Family(vlm_api, make_sft_train_step, make_sft_eval_step)


def _pretrained_loader(model_dir: str):
    """Stream a HF checkpoint directory into the engine's master shards."""
    def load(optimizer, cfg):
        model, _ = vlm_api.load_pretrained(model_dir, tp_size=None, fsdp_size=None, dp_size=None)
        values = dict(model.named_parameters())
        names = {id(p): n for n, p in optimizer.model.named_parameters()}
        tp = int(getattr(optimizer, "TP", 1))
        layout = None
        if tp > 1:   # the checkpoint holds whole tensors: cut this tensor-parallel rank's slices
            import importlib

            layout = importlib.import_module(getattr(optimizer.model, "TP_LAYOUT", "omegalax_b200.models.qwen3.tp_layout"))
        for u in optimizer.units:
            for s in u.slots:
                n = names[id(s.param)]
                v = values[n].detach()
                if layout is not None:
                    v = layout.tp_slice(n, v, optimizer.model.cfg, tp, optimizer.tp_rank)
                optimizer.load_full_param(s, v)
        optimizer.sync_compute_from_master()
        del model
        gc.collect()
    return load


def run_sft(model_id_or_cfg, train_cfg: TrainConfig, data_iter, **kw):
    """Same loop as the text trainer with the multimodal batch keys; when ``model_id_or_cfg`` is
    a checkpoint directory its weights are loaded before training (not when resuming)."""
    loader = None
    if isinstance(model_id_or_cfg, str) and os.path.isdir(model_id_or_cfg) and not kw.get("resume"):
        import glob

        if glob.glob(os.path.join(model_id_or_cfg, "*.safetensors")):
            loader = _pretrained_loader(model_id_or_cfg)
    return _text.run_sft(model_id_or_cfg, train_cfg, data_iter, _family=_VLM_FAMILY, pretrained_loader=loader, **kw)

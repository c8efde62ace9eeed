"""Qwen3.5: hybrid GatedDeltaNet / gated-attention decoder with dense or MoE (+ shared
expert) feed-forward, and the conditional-generation wrapper that splices vision features
into the token stream (reference: omegalax/models/qwen3_5/model.py)."""
from __future__ import annotations

import math

import torch
from torch import nn

from ...ops import functional as Fn
from ...parallel import tp as tp_lib
from ...ops import moe as moe_ops
from ..qwen3.model import Embedding, ForwardCtx, Linear
from ..qwen3.model import MLP as _SwiGLU
from ..qwen3.utils import count_left_pads
from .attention import Attention
from .config import Qwen3_5Config, Qwen3_5TextConfig
from .deltanet import GatedDeltaNet
from .norms import RMSNorm
from .rope import mrope_half_tables


from ...utils.profiling import scoped


class MLP(_SwiGLU):
    pass


class MoEFeedForward(nn.Module):
    """Top-k routed experts (always renormalised) + a shared expert scaled by
    sigmoid(shared_expert_gate(x)); aux = coef * sum_e (mean prob_e - 1/E)^2."""

    def __init__(self, cfg: Qwen3_5TextConfig, device=None, dtype=None, tp_size: int = 1):
        """Under tensor parallelism the routed experts are replicated (every rank routes its own
        sequence-parallel rows); the shared expert's width is split over tp."""
        super().__init__()
        E, D, F_ = cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size
        self.E, self.k, self.coef = E, cfg.num_experts_per_tok, cfg.router_aux_loss_coef
        kw = dict(device=device, dtype=dtype)
        self.router = Linear(D, E, **kw)
        self.experts_gate_up = nn.Parameter(torch.empty(E, 2 * F_, D, **kw))
        self.experts_down = nn.Parameter(torch.empty(E, D, F_, **kw))
        self.shared_expert = _SwiGLU(D, cfg.shared_expert_intermediate_size, tp_size=tp_size, **kw)
        self.shared_expert_gate = Linear(D, 1, **kw)
        self.ep = None
        self.aux_group = None  # data ranks over which the load-balance statistics are taken
        self.reset_parameters()

    def reset_parameters(self):
        if self.experts_gate_up.device.type != "meta":
            nn.init.normal_(self.experts_gate_up, std=1.0 / math.sqrt(self.experts_gate_up.shape[2]))
            nn.init.normal_(self.experts_down, std=1.0 / math.sqrt(self.experts_down.shape[2]))

    @scoped("moe_ffn")
    def forward(self, x, residual=None):
        probs, w, idx = moe_ops.route(self.router(x), self.k, True)
        if self.ep is not None:
            y = self.ep.moe_mlp(x, w, idx, self.experts_gate_up, self.experts_down)
        else:
            y = moe_ops.moe_mlp(x, w, idx, self.experts_gate_up, self.experts_down)
        gate = torch.sigmoid(torch.nn.functional.linear(x, self.shared_expert_gate.weight.to(x.dtype)))
        y = y + gate * self.shared_expert(x)
        if residual is not None:
            y = y + residual
        return y, moe_ops.load_balance_loss_sq(probs, self.E, self.coef, self.aux_group)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: Qwen3_5TextConfig, layer_idx: int, device=None, dtype=None, tp_size: int = 1):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.tp_size = tp_size
        self.layer_type = cfg.layer_types[layer_idx]
        self.input_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, **kw)
        self.post_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, **kw)
        if self.layer_type == "full_attention":
            self.attn = Attention(cfg, tp_size=tp_size, **kw)
        else:
            self.linear_attn = GatedDeltaNet(cfg, tp_size=tp_size, **kw)
        self.is_moe = cfg.is_moe
        self.mlp = MoEFeedForward(cfg, tp_size=tp_size, **kw) if cfg.is_moe else \
            MLP(cfg.hidden_size, cfg.intermediate_size, tp_size=tp_size, **kw)

    def forward(self, x, ctx: ForwardCtx, cache=None):
        h = self.input_norm(x)
        if self.layer_type == "full_attention":
            x = self.attn(h, ctx, residual=x)
        else:
            x = self.linear_attn(h, ctx, residual=x)
        h = self.post_norm(x)
        if self.is_moe:
            return self.mlp(h, residual=x)
        return self.mlp(h, residual=x), x.new_zeros((), dtype=torch.float32)


class TextModel(nn.Module):
    def __init__(self, cfg: Qwen3_5TextConfig, device=None, dtype=None, tp_size: int = 1):
        super().__init__()
        self.cfg = cfg
        self.tp_size = tp_size
        kw = dict(device=device, dtype=dtype or torch.float32)
        self.embedder = Embedding(cfg.vocab_size, cfg.hidden_size, **kw)
        self.layers = nn.ModuleList(DecoderLayer(cfg, i, tp_size=tp_size, **kw) for i in range(cfg.num_hidden_layers))
        self.final_norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, **kw)
        self.layer_runner = None

    def make_ctx(self, segment_ids, position_ids_ZBT=None) -> ForwardCtx:
        B, T = segment_ids.shape
        dev = segment_ids.device
        if position_ids_ZBT is None:
            pos = torch.arange(T, device=dev)[None, :].expand(B, T)
            position_ids_ZBT = pos[None].expand(3, B, T)
        rot = int(self.cfg.head_dim * self.cfg.partial_rotary_factor)
        sin, cos = mrope_half_tables(position_ids_ZBT, rot, self.cfg.rope_theta, self.cfg.mrope_section)
        cu = torch.arange(B + 1, device=dev, dtype=torch.int32) * T
        return ForwardCtx(B=B, T=T, sin=sin.reshape(B * T, -1), cos=cos.reshape(B * T, -1), cu_seqlens=cu,
                          segment_ids=segment_ids, k_start=None, positions=position_ids_ZBT)

    @scoped("text_model")
    def forward(self, token_ids, segment_ids, position_ids_ZBT=None, inputs_embeds=None, return_local_rows: bool = False):
        """Under tensor parallelism the rows between the blocks are sequence-parallel (this rank
        carries rows [r*M/tp, (r+1)*M/tp) of the flattened token rows); ``return_local_rows``
        returns them [M/tp, D] instead of the gathered [B,T,D]."""
        B, T = segment_ids.shape
        ctx = self.make_ctx(segment_ids, position_ids_ZBT)
        x = self.embedder(token_ids.reshape(-1)) if inputs_embeds is None else inputs_embeds.reshape(B * T, -1)
        tp = tp_lib.current() if self.tp_size > 1 else None
        if tp is not None:
            if (B * T) % tp.size:
                raise ValueError("tensor parallelism needs B*T divisible by tp_size")
            m = B * T // tp.size
            x = x[tp.rank * m:(tp.rank + 1) * m]
        aux_total = torch.zeros((), dtype=torch.float32, device=x.device)
        for layer in self.layers:
            if self.layer_runner is not None:
                x, aux = self.layer_runner(layer, x, ctx)
            else:
                x, aux = layer(x, ctx)
            aux_total = aux_total + aux
        x = self.final_norm(x)
        if tp is not None:
            if return_local_rows:
                return x, aux_total
            x = tp_lib.all_gather_rows(x, tp)
        return x.view(B, T, -1), aux_total


class Qwen3_5ForCausalLM(nn.Module):
    """Text-only model; forward returns hidden states before lm_head and the aux loss."""

    TP_LAYOUT = "omegalax_b200.models.qwen3_5.tp_layout"

    def __init__(self, cfg: Qwen3_5TextConfig, device=None, dtype=None, tp_size: int = 1):
        super().__init__()
        self.cfg = cfg
        self.tp_size = tp_size
        self.model = TextModel(cfg, device=device, dtype=dtype, tp_size=tp_size)
        self.lm_head = Linear(cfg.hidden_size, cfg.vocab_size, device=device, dtype=dtype or torch.float32)

    @property
    def layer_runner(self):
        return self.model.layer_runner

    @layer_runner.setter
    def layer_runner(self, fn):
        self.model.layer_runner = fn

    def train_units(self):
        m = self.model
        return [("embedder", [m.embedder])] + [(f"layers.{i}", [l]) for i, l in enumerate(m.layers)] + \
               [("head", [m.final_norm, self.lm_head])]

    def forward(self, token_ids, segment_ids, cache=None, num_right_pads: int = 0, position_ids_ZBT=None,
                return_local_rows: bool = False):
        return self.model(token_ids, segment_ids, position_ids_ZBT, return_local_rows=return_local_rows)


class Qwen3_5ForConditionalGeneration(nn.Module):
    """Vision tower + text model: image-token embeddings are replaced by vision features."""

    TP_LAYOUT = "omegalax_b200.models.qwen3_5.tp_layout"

    def __init__(self, cfg: Qwen3_5Config, device=None, dtype=None, tp_size: int = 1):
        super().__init__()
        from .vision import VisionModel

        self.cfg = cfg
        self.tp_size = tp_size
        dtype = dtype or torch.float32
        self.visual = VisionModel(cfg.vision_config, device=device, dtype=dtype)
        self.model = TextModel(cfg.text_config, device=device, dtype=dtype, tp_size=tp_size)
        self.lm_head = Linear(cfg.text_config.hidden_size, cfg.text_config.vocab_size, device=device, dtype=dtype)

    @property
    def layer_runner(self):
        return self.model.layer_runner

    @layer_runner.setter
    def layer_runner(self, fn):
        self.model.layer_runner = fn

    def train_units(self):
        m = self.model
        return [("visual", [self.visual]), ("embedder", [m.embedder])] + \
               [(f"layers.{i}", [l]) for i, l in enumerate(m.layers)] + [("head", [m.final_norm, self.lm_head])]

    def forward(self, token_ids, segment_ids, pixel_values=None, image_grid_thw=None, position_ids_ZBT=None,
                return_local_rows: bool = False):
        B, T = token_ids.shape
        embeds = self.model.embedder(token_ids.reshape(-1))
        if pixel_values is not None and pixel_values.numel() > 0:
            feats = self.visual(pixel_values.to(embeds.dtype), image_grid_thw).to(embeds.dtype)
            is_img = (token_ids.reshape(-1) == self.cfg.image_token_id)
            embeds = embeds * (~is_img).unsqueeze(-1).to(embeds.dtype)
            if is_img.is_cuda:   # no host synchronisation; surplus (padded) feature rows add zeros
                pos, ok = Fn.first_true_rows(is_img, feats.shape[0])
                embeds = embeds.index_add(0, pos, feats[: pos.numel()] * ok.to(embeds.dtype))
            else:
                pos = torch.nonzero(is_img, as_tuple=False).squeeze(-1)[: feats.shape[0]]
                embeds = embeds.index_add(0, pos, feats[: pos.numel()])
        return self.model(token_ids, segment_ids, position_ids_ZBT, inputs_embeds=embeds.view(B, T, -1),
                          return_local_rows=return_local_rows)

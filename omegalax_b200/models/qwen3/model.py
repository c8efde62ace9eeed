"""Qwen3 decoder (dense and MoE) as PyTorch modules over the op layer.

Activations travel as packed rows [M = B*T, D].  The hot ops (projections, norms, QK-norm +
RoPE, attention, SwiGLU, experts) go through ``omegalax_b200.ops.functional`` which picks
the sm_100a kernels for CUDA bf16 tensors and the PyTorch definitions otherwise.
Behavioural reference: omegalax/models/qwen3/{model,attention}.py.
"""
from __future__ import annotations

import dataclasses
import math

import torch
from torch import nn

from ...ops import functional as Fn
from ...ops import moe as moe_ops
from ...ops import reference as R
from ...parallel import tp as tp_lib
from .cache import LayerCache
from .config import Qwen3Config
from .norms import RMSNorm
from .utils import compute_positions_from_segment_ids, count_left_pads


from ...utils.profiling import scoped


class Embedding(nn.Module):
    """Token embedding table, normal(0, 0.02) init."""

    def __init__(self, num: int, dim: int, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num, dim, device=device, dtype=dtype))
        self.reset_parameters()

    def reset_parameters(self):
        if self.weight.device.type != "meta":
            nn.init.normal_(self.weight, std=0.02)

    def forward(self, ids):
        return Fn.embedding(ids, self.weight)


class Linear(nn.Module):
    """Bias-free (by default) projection, weight [out, in], lecun-normal init."""

    def __init__(self, in_dim: int, out_dim: int, bias: bool = False, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(out_dim, in_dim, device=device, dtype=dtype))
        self.bias = nn.Parameter(torch.zeros(out_dim, device=device, dtype=dtype)) if bias else None
        self.tp_sharded = False  # True when this rank holds only its tensor-parallel slice
        self.reset_parameters()

    def reset_parameters(self):
        if self.weight.device.type != "meta":
            nn.init.normal_(self.weight, std=1.0 / math.sqrt(self.weight.shape[1]))
            if self.bias is not None:
                nn.init.zeros_(self.bias)

    def forward(self, x, residual=None, tag=None):
        return Fn.linear(x, self.weight, residual=residual, bias=self.bias, tag=tag)


def left_pad_cu_seqlens(k_start, B: int, T: int) -> torch.Tensor:
    """Packed-sequence boundaries for B rows of T positions whose first ``k_start[b]`` positions are
    left padding: int32 [2B+1] = (b*T, b*T + k_start[b]) per row, then B*T.  Each row becomes two
    causal sequences, its pads and its real tokens, so a real query never sees a pad key (what the
    ``k_start`` mask of the PyTorch path does) while the kernels keep plain causal sequences.  Pad
    positions attend among themselves; nothing downstream reads them.  Built on the device."""
    if Fn.library_mode():   # the library baseline runs plain causal rows, as the reference does
        return torch.arange(B + 1, device=k_start.device, dtype=torch.int32) * T
    base = torch.arange(B, device=k_start.device, dtype=torch.int64) * T
    cu = torch.stack([base, base + k_start.to(torch.int64).clamp(0, T)], dim=1).reshape(-1)
    end = torch.full((1,), B * T, device=k_start.device, dtype=torch.int64)
    return torch.cat([cu, end]).to(torch.int32)


@dataclasses.dataclass
class ForwardCtx:
    """Per-call state shared by all layers."""
    B: int
    T: int
    sin: torch.Tensor            # [M, rot/2] fp32
    cos: torch.Tensor
    cu_seqlens: torch.Tensor     # int32 [B+1]
    segment_ids: torch.Tensor    # [B, T]
    k_start: torch.Tensor | None = None   # [B] first real key per row (left padding)
    positions: torch.Tensor | None = None
    extra: dict = dataclasses.field(default_factory=dict)


class Attention(nn.Module):
    def __init__(self, cfg: Qwen3Config, device=None, dtype=None, tp_size: int = 1):
        super().__init__()
        if cfg.num_heads % tp_size or cfg.num_kv_heads % tp_size:
            raise ValueError(f"heads ({cfg.num_heads} q / {cfg.num_kv_heads} kv) do not divide over tp_size={tp_size}")
        H, G, Kd, D = cfg.num_heads // tp_size, cfg.num_kv_heads // tp_size, cfg.head_dim, cfg.emb_dim
        self.H, self.G, self.Kd = H, G, Kd   # heads held by this tensor-parallel rank
        self.tp_size = tp_size
        self.qkv_proj = Linear(D, (H + 2 * G) * Kd, device=device, dtype=dtype)
        self.o_proj = Linear(H * Kd, D, device=device, dtype=dtype)
        self.q_norm = RMSNorm(Kd, cfg.norm_eps, device=device, dtype=dtype)
        self.k_norm = RMSNorm(Kd, cfg.norm_eps, device=device, dtype=dtype)
        self.eps = cfg.norm_eps
        self.scale = Kd ** -0.5
        self.qkv_proj.tp_sharded = self.o_proj.tp_sharded = tp_size > 1

    @scoped("attention")
    def forward(self, x, ctx: ForwardCtx, residual=None, cache: LayerCache | None = None):
        tp = tp_lib.current() if self.tp_size > 1 else None
        if tp is not None:
            x = tp_lib.all_gather_rows(x, tp)      # sequence-parallel rows -> all rows
        M = x.shape[0]
        qkv = self.qkv_proj(x, tag="qkv")
        q, k, v, _ = Fn.qk_norm_rope(qkv, self.q_norm.weight, self.k_norm.weight, ctx.sin, ctx.cos,
                                     self.H, self.G, self.Kd, eps=self.eps)
        B, T = ctx.B, ctx.T
        if cache is None:
            if Fn.use_kernels(q) or (Fn.library_mode() and q.is_cuda):
                o = Fn.flash_attention(q, k, v, ctx.cu_seqlens, T, scale=self.scale, causal=True, tag="attn")
            else:
                ks = None if ctx.k_start is None else ctx.k_start[:, None].expand(B, T)
                o = R.attention(q.reshape(B, T, self.H, self.Kd), k.reshape(B, T, self.G, self.Kd),
                                v.reshape(B, T, self.G, self.Kd), causal=True, scale=self.scale,
                                k_start=ks).reshape(M, self.H, self.Kd)
        else:
            o = self._decode(q, k, v, ctx, cache)
        o = o.reshape(M, self.H * self.Kd)
        if tp is not None:
            return tp_lib.row_parallel_linear(o, self.o_proj.weight, residual, tp)
        return self.o_proj(o, residual=residual, tag="o")

    def _decode(self, q, k, v, ctx: ForwardCtx, cache: LayerCache):
        """Append this call's K/V at the cursor and attend over the whole cache with the mask
        (key position <= query position, both relative to the row's first real token) and
        (key holds a real token).  Softmax in fp32 (reference: qwen3/attention.py:95-132)."""
        B, T = ctx.B, ctx.T
        cur = cache.cur_ind
        k4 = k.reshape(B, T, self.G, self.Kd)
        v4 = v.reshape(B, T, self.G, self.Kd)
        cache.k_cache[:, cur:cur + T] = k4.to(cache.k_cache.dtype)
        cache.v_cache[:, cur:cur + T] = v4.to(cache.v_cache.dtype)
        valid = ctx.extra["kv_valid"]  # [B, S] bool, maintained by the model
        S = cache.size
        kpos = torch.arange(S, device=q.device)[None, :]
        qpos = (cur + torch.arange(T, device=q.device))[None, :, None]
        mask = (kpos[:, None, :] <= qpos) & valid[:, None, :] & (kpos[:, None, :] >= cache.start_ind[:, None, None])
        qf = q.reshape(B, T, self.G, self.H // self.G, self.Kd).float()
        logits = torch.einsum("btgrk,bsgk->btsgr", qf, cache.k_cache.float()) * self.scale
        logits = logits.masked_fill(~mask[:, :, :, None, None], torch.finfo(torch.float32).min)
        p = torch.softmax(logits, dim=2)
        o = torch.einsum("btsgr,bsgk->btgrk", p, cache.v_cache.float())
        cache.cur_ind = cur + T
        return o.reshape(B * T, self.H, self.Kd).to(q.dtype)


class MLP(nn.Module):
    """SwiGLU feed-forward: down(silu(gate(x)) * up(x)) with gate and up fused row-wise."""

    def __init__(self, dim: int, hidden: int, device=None, dtype=None, tp_size: int = 1):
        super().__init__()
        if hidden % tp_size:
            raise ValueError(f"mlp width {hidden} does not divide over tp_size={tp_size}")
        hidden //= tp_size
        self.tp_size = tp_size
        self.gate_up_proj = Linear(dim, 2 * hidden, device=device, dtype=dtype)   # this rank's [gate | up]
        self.down_proj = Linear(hidden, dim, device=device, dtype=dtype)
        self.gate_up_proj.tp_sharded = self.down_proj.tp_sharded = tp_size > 1

    @scoped("feed_forward")
    def forward(self, x, residual=None):
        tp = tp_lib.current() if self.tp_size > 1 else None
        if tp is not None:
            h = Fn.swiglu(tp_lib.column_parallel_linear(x, self.gate_up_proj.weight, tp))
            return tp_lib.row_parallel_linear(h, self.down_proj.weight, residual, tp)
        # With a residual this call produces the decoder layer's output, whose value nothing in the
        # layer's own backward reads ("down" may then be skipped when the layer is re-run).  Without
        # one (e.g. a shared expert whose output is gated) the value is needed: no tag.
        return Fn.swiglu_linear(self.gate_up_proj(x, tag="gate_up"), self.down_proj.weight, residual,
                                tag="down" if residual is not None else None)


class MoEFeedForward(nn.Module):
    """Top-k routed SwiGLU experts with the Qwen3 load-balance loss."""

    def __init__(self, cfg: Qwen3Config, device=None, dtype=None):
        super().__init__()
        E, D, F_ = cfg.num_experts, cfg.emb_dim, cfg.moe_intermediate_size
        self.E, self.k = E, cfg.num_experts_per_tok
        self.norm_topk, self.coef = cfg.norm_topk_prob, cfg.aux_loss_coef
        self.router = Linear(D, E, device=device, dtype=dtype)
        self.experts_gate_up = nn.Parameter(torch.empty(E, 2 * F_, D, device=device, dtype=dtype))
        self.experts_down = nn.Parameter(torch.empty(E, D, F_, device=device, dtype=dtype))
        self.ep = None  # set by the expert-parallel runtime
        self.aux_group = None  # data ranks over which the load-balance statistics are taken
        self.reset_parameters()

    def reset_parameters(self):
        if self.experts_gate_up.device.type != "meta":
            nn.init.normal_(self.experts_gate_up, std=1.0 / math.sqrt(self.experts_gate_up.shape[2]))
            nn.init.normal_(self.experts_down, std=1.0 / math.sqrt(self.experts_down.shape[2]))

    @scoped("moe_feed_forward")
    def forward(self, x, residual=None):
        logits = self.router(x)
        probs, w, idx = moe_ops.route(logits, self.k, self.norm_topk)
        if self.ep is not None:
            y = self.ep.moe_mlp(x, w, idx, self.experts_gate_up, self.experts_down)
        else:
            y = moe_ops.moe_mlp(x, w, idx, self.experts_gate_up, self.experts_down)
        aux = moe_ops.load_balance_loss_qwen3(probs, idx, self.E, self.coef, self.aux_group)
        if residual is not None:
            y = y + residual
        return y, aux


class DecoderLayer(nn.Module):
    def __init__(self, cfg: Qwen3Config, layer_idx: int, device=None, dtype=None, tp_size: int = 1):
        super().__init__()
        self.input_norm = RMSNorm(cfg.emb_dim, cfg.norm_eps, device=device, dtype=dtype)
        self.attn = Attention(cfg, device=device, dtype=dtype, tp_size=tp_size)
        self.post_norm = RMSNorm(cfg.emb_dim, cfg.norm_eps, device=device, dtype=dtype)
        self.is_moe = cfg.is_moe_layer(layer_idx)
        if self.is_moe:
            self.mlp = MoEFeedForward(cfg, device=device, dtype=dtype)
        else:
            self.mlp = MLP(cfg.emb_dim, cfg.mlp_dim, device=device, dtype=dtype, tp_size=tp_size)

    def forward(self, x, ctx: ForwardCtx, cache: LayerCache | None = None):
        x = self.attn(self.input_norm(x), ctx, residual=x, cache=cache)
        h = self.post_norm(x)
        if self.is_moe:
            x, aux = self.mlp(h, residual=x)
        else:
            x, aux = self.mlp(h, residual=x), x.new_zeros((), dtype=torch.float32)
        return x, aux


def vocab_parallel_head(cfg, tp_size: int) -> bool:
    return tp_size > 1 and not cfg.tie_word_embeddings and cfg.vocab_size % (8 * tp_size) == 0


class Qwen3(nn.Module):
    """Returns the final hidden states (before lm_head) and the summed auxiliary loss; the
    lm_head is a separate projection applied by callers (loss, decode)."""

    def __init__(self, cfg: Qwen3Config, device=None, dtype=None, tp_size: int = 1):
        super().__init__()
        self.cfg = cfg
        self.tp_size = tp_size
        dtype = dtype or torch.float32
        self.embedder = Embedding(cfg.vocab_size, cfg.emb_dim, device=device, dtype=dtype)
        self.layers = nn.ModuleList(DecoderLayer(cfg, i, device=device, dtype=dtype, tp_size=tp_size)
                                    for i in range(cfg.num_layers))
        self.final_norm = RMSNorm(cfg.emb_dim, cfg.norm_eps, device=device, dtype=dtype)
        # untied head under tensor parallelism: split over the vocabulary (vocab-parallel loss)
        self.vocab_parallel = vocab_parallel_head(cfg, tp_size)
        self.lm_head = Linear(cfg.emb_dim, cfg.vocab_size // tp_size if self.vocab_parallel else cfg.vocab_size,
                              device=device, dtype=dtype)
        self.lm_head.tp_sharded = self.vocab_parallel
        self.layer_runner = None  # installed by the training engine (remat / FSDP gather)

    def make_ctx(self, token_ids, segment_ids, position_offset: int = 0, start_ind=None) -> ForwardCtx:
        B, T = token_ids.shape
        dev = token_ids.device
        if start_ind is None:
            positions = compute_positions_from_segment_ids(segment_ids)
            k_start = count_left_pads(segment_ids).to(torch.int64)
        else:
            t = torch.arange(T, device=dev, dtype=torch.int64)[None, :] + position_offset
            positions = torch.where(segment_ids != 0, t - start_ind[:, None].to(torch.int64),
                                    torch.full_like(t.expand(B, T), 2 ** 30))
            k_start = start_ind.to(torch.int64)
        sin, cos = R.rope_tables(positions.reshape(-1), self.cfg.head_dim, self.cfg.rope_theta)
        cu = left_pad_cu_seqlens(k_start, B, T)
        return ForwardCtx(B=B, T=T, sin=sin, cos=cos, cu_seqlens=cu, segment_ids=segment_ids,
                          k_start=k_start, positions=positions)

    @torch.no_grad()
    def decode_paged(self, token_ids, segment_ids, cache):
        """Prefill or one decode step against a ``PagedKVCache`` (CUDA bf16).  Only real tokens
        are processed and stored; returns the final hidden state of every sequence's last new
        token, [B, D] (zeros for sequences without a new token)."""
        from ...ops import kernels as K

        cfg = self.cfg
        B, T = token_ids.shape
        dev = token_ids.device
        real = segment_ids != 0
        counts = real.sum(-1)
        new_tokens = [int(c) for c in counts.tolist()]
        cache.reserve(new_tokens)
        seq_of = torch.arange(B, device=dev)[:, None].expand(B, T)[real].to(torch.int32)
        rank_in = (real.cumsum(-1) - 1)[real]
        start = cache.seq_lens[seq_of.long()]
        slot = (start + rank_in).to(torch.int32)
        ids = token_ids[real]
        x = self.embed(ids)
        N = x.shape[0]
        single = max(new_tokens) <= 1
        if not single and any(cache.seq_lens_host[b] > 0 and new_tokens[b] > 0 for b in range(B)):
            raise NotImplementedError("multi-token calls are only supported on an empty cache (prefill)")
        cu = torch.zeros(B + 1, dtype=torch.int32, device=dev)
        cu[1:] = counts.cumsum(0)
        sin, cos = R.rope_tables(slot, cfg.head_dim, cfg.rope_theta)
        lens_after = (cache.seq_lens + counts.to(torch.int32)).contiguous()
        rows = cache.flat_rows(seq_of, slot)
        last = (cu[1:] - 1).long().clamp_min(0)
        for li, layer in enumerate(self.layers):
            a = layer.attn
            h = layer.input_norm(x)
            qkv = a.qkv_proj(h)
            if single:
                q = K.decode_append(qkv, a.q_norm.weight, a.k_norm.weight, slot, seq_of, slot, cache.block_table,
                                    cache.page_size, cache.k_pages[li], cache.v_pages[li], a.H, a.G, a.Kd, a.Kd,
                                    cfg.rope_theta, a.eps)
                # every sequence contributes exactly one row in this mode
                qb = torch.zeros(B, a.H, a.Kd, dtype=q.dtype, device=dev)
                qb[seq_of.long()] = q
                ob = K.decode_attn(qb, cache.k_pages[li], cache.v_pages[li], cache.block_table, lens_after,
                                   cache.page_size, a.scale)
                o = ob[seq_of.long()]
            else:
                q, k, v, _ = Fn.qk_norm_rope(qkv, a.q_norm.weight, a.k_norm.weight, sin, cos, a.H, a.G, a.Kd, eps=a.eps)
                o = Fn.flash_attention(q, k, v, cu, T, scale=a.scale, causal=True)
                cache.k_pages[li].view(-1, a.G, a.Kd).index_copy_(0, rows, k)
                cache.v_pages[li].view(-1, a.G, a.Kd).index_copy_(0, rows, v.contiguous())
            x = a.o_proj(o.reshape(N, a.H * a.Kd), residual=x)
            hh = layer.post_norm(x)
            x = layer.mlp(hh, residual=x)[0] if layer.is_moe else layer.mlp(hh, residual=x)
        cache.advance(new_tokens)
        x = self.final_norm(x)
        out = torch.zeros(B, x.shape[1], dtype=x.dtype, device=dev)
        has = counts > 0
        out[has] = x[last[has]]
        return out

    def embed(self, token_ids):
        return Fn.embedding(token_ids.reshape(-1), self.embedder.weight)

    def forward(self, token_ids, segment_ids, cache=None, num_right_pads: int = 0, return_local_rows: bool = False):
        """With tensor parallelism the activations between blocks are sequence-parallel: this rank
        carries rows [r*M/tp, (r+1)*M/tp) of the flattened [B*T] token rows.  By default the final
        hidden states are gathered back to [B,T,D]; ``return_local_rows`` returns this rank's
        rows [M/tp, D] instead (the trainer computes the loss on them)."""
        B, T = token_ids.shape
        if cache is None:
            ctx = self.make_ctx(token_ids, segment_ids)
        else:
            first = cache[0]
            if first.cur_ind == 0:
                start = count_left_pads(segment_ids)
                for lc in cache:
                    lc.start_ind = start.clone()
                valid = torch.zeros(B, first.size, dtype=torch.bool, device=token_ids.device)
            else:
                valid = first._kv_valid  # type: ignore[attr-defined]
            cur = first.cur_ind
            valid = valid.clone()
            valid[:, cur:cur + T] = segment_ids != 0
            first._kv_valid = valid  # type: ignore[attr-defined]
            ctx = self.make_ctx(token_ids, segment_ids, position_offset=cur, start_ind=first.start_ind)
            ctx.extra["kv_valid"] = valid
        x = self.embed(token_ids)
        tp = tp_lib.current() if self.tp_size > 1 else None
        if tp is not None and cache is not None:
            # inference with a KV cache (this rank's kv heads): all rows on every rank
            with tp_lib.replicated_rows(tp):
                aux_total = torch.zeros((), dtype=torch.float32, device=x.device)
                for i, layer in enumerate(self.layers):
                    x, aux = layer(x, ctx, cache[i])
                    aux_total = aux_total + aux
                return self.final_norm(x).view(B, T, -1), aux_total
        if tp is not None:
            if (B * T) % tp.size:
                raise ValueError("tensor parallelism needs B*T divisible by tp_size")
            m = B * T // tp.size
            x = x[tp.rank * m:(tp.rank + 1) * m]
        aux_total = torch.zeros((), dtype=torch.float32, device=x.device)
        for i, layer in enumerate(self.layers):
            lc = None if cache is None else cache[i]
            if self.layer_runner is not None and cache is None:
                x, aux = self.layer_runner(layer, x, ctx)
            else:
                x, aux = layer(x, ctx, lc)
            aux_total = aux_total + aux
        x = self.final_norm(x)
        if tp is not None:
            if return_local_rows:
                return x, aux_total
            x = tp_lib.all_gather_rows(x, tp)
        return x.view(B, T, -1), aux_total

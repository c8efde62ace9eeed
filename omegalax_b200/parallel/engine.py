"""Sharded training state: fp32 master weights + AdamW moments sharded over the data ranks
(ZeRO-3 / FSDP), bf16 compute copies gathered one unit (decoder layer) at a time,
rematerialisation of each unit in the backward (whole, or with tagged outputs kept: fixed tag
lists or as many as the free memory allows), gradient reduce-scatter per unit (inside the
weight-gradient GEMMs where GPUs map each other's memory), expert tensors that stay with their
owner under expert parallelism, and a fused clip + AdamW + bf16 re-cast over the flat shard.

One process drives one GPU.  With a single rank every collective degenerates to a no-op
and the bf16 compute copy is simply the cast of the master buffer.

Layout.  The model is cut into *units* (embedding, each decoder layer, final norm + head).
Every parameter of a unit is split along dim 0 over the W shard ranks (parameters whose
dim 0 does not divide evenly into 16-byte aligned slices stay replicated).  A rank's slice
of all parameters of a unit is contiguous in its flat shard buffers:

    master / exp_avg / exp_avg_sq / grad   fp32  [shard_numel]     (owned)
    compute shard                          bf16  [shard_numel]     (peers read it)
    gathered unit                          bf16  per-parameter full tensors (transient)

Reference behaviour being reproduced: parameters fp32, compute bf16, optimizer state fp32
(omegalax/trainers/optim.py:11-41), every decoder layer rematerialised
(omegalax/models/qwen3/model.py:140-150), parameters born sharded
(omegalax/models/sharding_runtime.py:14-26).
"""
from __future__ import annotations

import dataclasses
import math
import os

import torch
import torch.distributed as dist
from torch import nn

from ..ops import functional as Fn
from ..ops import kernels as K

bf16 = torch.bfloat16
_TORCH_CHUNK = 1 << 26      # elements per slice of the PyTorch optimizer path (bounds its temporaries)
_SCATTER_ADD_MAX = 1 << 22  # a unit's non-GEMM gradients up to this many elements travel as NVLink reductions


# OMEGALAX_B200_POISON=1 fills every gathered-layer buffer with NaN before it is (re)filled, so a read
# of an element that no gather has written (a stale or skipped slot) turns the loss into NaN
_POISON = os.environ.get("OMEGALAX_B200_POISON", "0") == "1"


@dataclasses.dataclass
class ParamSlot:
    name: str
    param: nn.Parameter
    shape: tuple
    numel: int
    sharded: bool
    shard_numel: int      # elements this rank owns (== numel when replicated)
    shard_off: int        # offset inside the unit's shard buffers
    full_off: int         # offset inside the unit's gathered buffer
    module: nn.Module = None
    pname: str = ""
    peer: bool = False     # gradient goes through the GEMM peer-reduce epilogue
    ep: bool = False       # expert-parallel: never gathered, this rank computes with its own slice
    fused_ag: bool = False  # gathered inside its forward GEMM launch, not by the prefetch
    tp_sharded: bool = False   # differs between tensor-parallel ranks (no gradient all-reduce over tp)
    shard_world: int = 1       # number of ranks the parameter is cut over (1 when replicated) ...
    shard_rank: int = 0        # ... and which piece this rank holds
    ep_product: bool = False   # experts cut over shard group x tensor-parallel group (every rank of the job)


@dataclasses.dataclass
class Unit:
    name: str
    modules: list
    slots: list
    shard_numel: int = 0
    full_numel: int = 0
    shard_base: int = 0   # offset of the unit in the rank-wide flat shard buffers
    gathered: torch.Tensor | None = None
    full_grad: torch.Tensor | None = None
    resident: bool = False


def _align(n: int, a: int = 8) -> int:
    return (n + a - 1) // a * a


def default_units(model: nn.Module) -> list[tuple[str, list[nn.Module]]]:
    """Embedding, each decoder layer, then everything else (final norm, head, vision...)."""
    if hasattr(model, "train_units"):
        return model.train_units()
    units = []
    claimed = set()
    for name in ("embedder", "embed_tokens"):
        if hasattr(model, name):
            units.append((name, [getattr(model, name)]))
            claimed.add(name)
    if hasattr(model, "layers"):
        for i, layer in enumerate(model.layers):
            units.append((f"layers.{i}", [layer]))
        claimed.add("layers")
    rest = [m for n, m in model.named_children() if n not in claimed]
    if rest:
        units.append(("head", rest))
    return units


class TrainEngine:
    def __init__(self, model: nn.Module, *, device, shard_group=None, lr: float = 1e-4,
                 weight_decay: float = 0.01, betas=(0.9, 0.999), eps: float = 1e-8,
                 max_grad_norm: float | None = 1.0, remat: str = "full", seed: int = 0,
                 init_from_model: bool = False, comm: str = "auto", expert_parallel: bool = True,
                 ep_capacity_factor: float = 2.0, tp_group=None, fused_gather: bool = True,
                 ep_over_tp: bool = False):
        self.model = model
        self.device = torch.device(device)
        self.group = shard_group
        self.W = dist.get_world_size(shard_group) if shard_group is not None else 1
        self.rank = dist.get_rank(shard_group) if shard_group is not None else 0
        self.lr, self.wd, self.betas, self.eps = lr, weight_decay, betas, eps
        self.max_grad_norm = max_grad_norm or 0.0
        self.remat = remat
        # remat policies: "full" recomputes the whole layer; "selective" (or "save:tag,tag") keeps the
        # tagged GEMM / attention outputs from the first forward; "none" keeps everything (single rank)
        # "down!": the output of a dense layer's last projection is the layer output, which nothing
        # in that layer's backward reads, so the re-run never computes it
        if remat == "selective":
            self.remat_tags = ("qkv", "attn", "o", "gate_up", "down!")
        elif remat.startswith("save:"):
            self.remat_tags = tuple(t for t in remat[5:].split(",") if t) + ("down!",)
        elif remat == "full":
            self.remat_tags = ("down!",)
        elif remat == "auto":
            # the small attention-side tensors always; after the first optimizer step the memory that
            # is still free decides how many layers also keep the attention block's output and the
            # wide MLP activation
            self.remat_tags = ("qkv", "attn", "down!")
        else:
            self.remat_tags = ()
        self._auto = _AutoStash(("o", "gate_up")) if remat == "auto" else None
        self.step_count = 0
        self.micro_steps = 0
        self.tp_group = tp_group
        self.TP = dist.get_world_size(tp_group) if tp_group is not None else 1
        self.tp_rank = dist.get_rank(tp_group) if tp_group is not None else 0
        # router load-balance statistics over the tokens of all ranks that hold different rows (data
        # ranks, and tensor-parallel ranks with their sequence-parallel slices): one small all-reduce
        # per MoE layer, as the reference's global-batch SPMD loss does
        aux_group = shard_group if self.TP == 1 else tp_group if self.W == 1 else \
            (dist.group.WORLD if dist.get_world_size() == self.W * self.TP else None)
        if aux_group is not None:
            for mod in model.modules():
                if hasattr(mod, "aux_group"):
                    mod.aux_group = aux_group
        self.use_cuda_kernels = self.device.type == "cuda" and not Fn.library_mode()
        self.compute_dtype = bf16 if self.device.type == "cuda" else torch.float32
        if comm == "auto":
            comm = "p2p" if (self.use_cuda_kernels and self.W > 1) else "nccl"
        self.comm_kind = comm if self.W > 1 else "none"
        # expert parallelism: the peer-memory exchange kernels when GPUs can map each other's memory;
        # "a2a" asks for the library all-to-all form on any transport (NCCL baseline, CPU ranks)
        self.ep_kind = "a2a" if expert_parallel == "a2a" else ("p2p" if (expert_parallel and self.comm_kind == "p2p") else None)
        # experts over every rank of the job (shard group x tensor-parallel group) instead of the shard
        # group only: the routed experts see sequence-parallel rows, so each of the W x TP ranks brings
        # its own tokens and can own its own E / (W x TP) experts.  Library all-to-all transport only.
        self.ep_over_tp = bool(ep_over_tp) and self.TP > 1 and bool(expert_parallel)
        if self.ep_over_tp:
            if dist.get_world_size() != self.W * self.TP:
                raise ValueError("experts over the tensor-parallel group need shard group x tp group = all ranks")
            self.ep_kind = "a2a"
            self.ep_group, self.EPW, self.ep_rank = dist.group.WORLD, self.W * self.TP, self.rank * self.TP + self.tp_rank
        else:
            self.ep_group, self.EPW, self.ep_rank = shard_group, self.W, self.rank
            if self.W == 1:
                self.ep_kind = None
        self.expert_parallel = self.ep_kind is not None
        # The weight of a layer's first projection is gathered inside that projection's GEMM launch
        # instead of by the prefetch.  Every backward must re-run the forward GEMM for this to hold
        # the weight when the gradient GEMMs need it, hence only with full rematerialisation.
        self.fused_gather = bool(fused_gather) and self.comm_kind == "p2p" and remat == "full" and self.TP == 1
        self._fused_done = [None, None]
        self._ag_count = 0
        self._ag_flags = None
        self.ep_capacity_factor = ep_capacity_factor
        self._ep = None
        self._build_units()
        self._allocate()
        self._materialize(seed, init_from_model)
        self._install()

    # ------------------------------------------------------------------ construction
    def _build_units(self):
        self.units: list[Unit] = []
        seen = set()
        for uname, mods in default_units(self.model):
            slots = []
            shard_off = full_off = 0
            for mi, m in enumerate(mods):
                for pname, p in m.named_parameters():
                    if id(p) in seen:
                        continue
                    seen.add(id(p))
                    shape = tuple(p.shape)
                    numel = p.numel()
                    rows = shape[0] if len(shape) else 1
                    row_numel = numel // max(rows, 1)
                    sharded = (self.W > 1 and len(shape) >= 1 and rows % self.W == 0
                               and ((rows // self.W) * row_numel) % 8 == 0)
                    is_expert = pname.rsplit(".", 1)[-1] in ("experts_gate_up", "experts_down")
                    sw, sr = (self.W, self.rank) if sharded else (1, 0)
                    product = bool(self.ep_over_tp and is_expert and rows % self.EPW == 0
                                   and ((rows // self.EPW) * row_numel) % 8 == 0)
                    if product:
                        sharded, sw, sr = True, self.EPW, self.ep_rank
                    sn = numel // sw if sharded else numel
                    slot = ParamSlot(f"{uname}.{mi}.{pname}", p, shape, numel, sharded, sn, shard_off, full_off, m, pname)
                    slot.shard_world, slot.shard_rank, slot.ep_product = sw, sr, product
                    owner = m.get_submodule(pname.rsplit(".", 1)[0]) if "." in pname else m
                    slot.tp_sharded = bool(getattr(owner, "tp_sharded", False))
                    # expert tensors under expert parallelism are never gathered: they take no room
                    # in the gathered-layer buffers
                    slot.ep = bool(self.expert_parallel and sharded and is_expert)
                    slots.append(slot)
                    shard_off += _align(sn)
                    if not slot.ep:
                        full_off += _align(numel)
            self.units.append(Unit(uname, mods, slots, shard_off, full_off))
        base = 0
        for u in self.units:
            u.shard_base = base
            base += u.shard_numel
        self.total_shard = base

    def _allocate(self):
        dev = self.device
        n = self.total_shard
        if dev.type == "cuda":
            # fp32 master, two moments and gradients plus the compute copy: say so before the first of
            # five allocations fails somewhere in the middle
            per = 16 + (0 if (self.compute_dtype == torch.float32 and self.W == 1) else
                        (2 if self.compute_dtype == bf16 else 4))
            free = torch.cuda.mem_get_info(dev)[0]
            if n * per > free:
                raise MemoryError(
                    f"this rank's parameter shard has {n / 1e9:.2f} G elements and needs {n * per / 1e9:.1f} GB of "
                    f"optimizer state, the device has {free / 1e9:.1f} GB free: shard over more ranks "
                    f"(fsdp / expert-parallel size {self.W}, tensor-parallel size {self.TP})")
        self.master = torch.zeros(n, dtype=torch.float32, device=dev)
        self.exp_avg = torch.zeros(n, dtype=torch.float32, device=dev)
        self.exp_avg_sq = torch.zeros(n, dtype=torch.float32, device=dev)
        if self.comm_kind == "p2p":
            from . import symm

            self._symm = symm
            self._grad_buf = symm.SymmetricBuffer(n * 4, self.group)
            self.grad = self._grad_buf.view(torch.float32, n)
            self._barrier = symm.DeviceBarrier(self.group)
            self._comm_stream = torch.cuda.Stream(device=dev)
        else:
            self.grad = torch.zeros(n, dtype=torch.float32, device=dev)
        if self.compute_dtype == torch.float32 and self.W == 1:
            self.compute_shard = self.master  # CPU/fp32 path computes on the master directly
        else:
            self.compute_shard = self._alloc_compute_shard(n)
        self.norm_sq = torch.zeros(1, dtype=torch.float32, device=dev)
        if self.W > 1:
            layer_like = [u for u in self.units if u.name.startswith("layers.")]
            self._ring_numel = max((u.full_numel for u in layer_like), default=0)
            self._ring = [torch.empty(self._ring_numel, dtype=self.compute_dtype, device=dev) for _ in range(2)]
            self._ring_grad = torch.zeros(self._ring_numel, dtype=torch.float32, device=dev) if self._ring_numel else None

    def _alloc_compute_shard(self, n):
        if self.comm_kind == "p2p":
            esz = 2 if self.compute_dtype == bf16 else 4
            self._shard_buf = self._symm.SymmetricBuffer(n * esz, self.group)
            return self._shard_buf.view(self.compute_dtype, n)
        return torch.zeros(n, dtype=self.compute_dtype, device=self.device)

    def _unit_views(self, u: Unit, flat: torch.Tensor):
        return flat[u.shard_base:u.shard_base + u.shard_numel]

    def _materialize(self, seed: int, init_from_model: bool):
        """Fill the master shard: either from the values the model already holds, or by
        running each module's own initialiser on a transient fp32 copy, one unit at a time."""
        gen_devices = [self.device] if self.device.type == "cuda" else []
        for ui, u in enumerate(self.units):
            on_meta = any(s.param.device.type == "meta" for s in u.slots)
            if on_meta or not init_from_model:
                with torch.random.fork_rng(devices=gen_devices):
                    torch.manual_seed(seed * 100003 + ui)
                    for m in u.modules:
                        if on_meta:
                            m.to_empty(device=self.device)
                            for s in u.slots:  # to_empty replaces meta Parameters by new objects
                                if s.module is m:
                                    s.param = m.get_parameter(s.pname)
                        for p in m.parameters():
                            p.data = p.data.to(device=self.device, dtype=torch.float32)
                        for sub in m.modules():
                            if hasattr(sub, "reset_parameters"):
                                if getattr(sub, "tp_sharded", False):  # distinct slice per tensor-parallel rank
                                    torch.manual_seed(seed * 100003 + ui + 7919 * (self.tp_rank + 1))
                                sub.reset_parameters()
            mshard = self._unit_views(u, self.master)
            for s in u.slots:
                src = s.param.data.detach().to(device=self.device, dtype=torch.float32).reshape(-1)
                if s.sharded:
                    src = src[s.shard_rank * s.shard_numel:(s.shard_rank + 1) * s.shard_numel]
                mshard[s.shard_off:s.shard_off + s.shard_numel].copy_(src)
            for s in u.slots:  # drop the transient full-precision copy
                s.param.data = torch.empty(0, dtype=self.compute_dtype, device=self.device)
        self._refresh_compute_shard()

    def _refresh_compute_shard(self):
        if self.compute_shard is self.master:
            return
        if self.use_cuda_kernels and self.compute_dtype == bf16:
            K.cast_f32_bf16(self.master, self.compute_shard)
        else:
            self.compute_shard.copy_(self.master)

    def _install(self):
        """Point every parameter at its compute storage and attach ``main_grad``."""
        self._weights_version = 0
        self._ring_owner = [None, None]
        self._ring_event = [None, None]
        self._seg_tables = {}
        if self.comm_kind == "p2p":
            self._barrier()  # every rank has written its compute shard
        for u in self.units:
            if self.W == 1:
                cs = self._unit_views(u, self.compute_shard)
                gs = self._unit_views(u, self.grad)
                for s in u.slots:
                    shp = (s.shape[0] // s.shard_world, *s.shape[1:]) if s.ep else s.shape   # local experts only
                    s.param.data = cs[s.shard_off:s.shard_off + s.shard_numel].view(shp)
                    s.param.main_grad = gs[s.shard_off:s.shard_off + s.shard_numel].view(shp)
                if self.expert_parallel:
                    self._mark_peer_slots(u)
                u.resident = True
            else:
                if self.comm_kind == "p2p" or self.expert_parallel:
                    self._mark_peer_slots(u)
                is_layer = u.name.startswith("layers.")
                if not is_layer:  # embedding / head stay gathered between optimizer steps
                    u.gathered = torch.empty(u.full_numel, dtype=self.compute_dtype, device=self.device)
                    u.full_grad = torch.zeros(u.full_numel, dtype=torch.float32, device=self.device)
                    self._bind(u, u.gathered, u.full_grad)
                    self._all_gather(u, u.gathered)
                    u.resident = True
        if hasattr(self.model, "layer_runner"):
            self.model.layer_runner = self.run_layer
        self._layer_units = {id(u.modules[0]): u for u in self.units if u.name.startswith("layers.")}
        self._layer_by_index = {int(u.name.split(".")[1]): u for u in self.units if u.name.startswith("layers.")}

    def _bind(self, u: Unit, full: torch.Tensor, full_grad: torch.Tensor | None):
        for s in u.slots:
            if s.ep:  # this rank's experts only, straight from the shard buffers
                shp = (s.shape[0] // s.shard_world, *s.shape[1:])
                cs, gs = self._unit_views(u, self.compute_shard), self._unit_views(u, self.grad)
                s.param.data = cs[s.shard_off:s.shard_off + s.shard_numel].view(shp)
                s.param.main_grad = gs[s.shard_off:s.shard_off + s.shard_numel].view(shp)
                continue
            s.param.data = full[s.full_off:s.full_off + s.numel].view(s.shape)
            if full_grad is not None:
                s.param.main_grad = full_grad[s.full_off:s.full_off + s.numel].view(s.shape)

    def _mark_peer_slots(self, u: Unit):
        """Weights of Linear modules take their gradient through the GEMM epilogue that adds
        each row block straight into the owning rank's fp32 gradient shard over NVLink."""
        for s in u.slots:
            if s.ep:
                s.peer = True        # gradients of this rank's experts are complete locally: nothing to reduce
                owner = s.module.get_submodule(s.pname.rsplit(".", 1)[0]) if "." in s.pname else s.module
                owner.ep = _LazyEP(self, owner)
                continue
            if self.comm_kind != "p2p":
                continue
            if not (s.sharded and len(s.shape) == 2 and s.pname.endswith("weight") and s.shape[0] % 8 == 0):
                continue
            owner = s.module.get_submodule(s.pname.rsplit(".", 1)[0]) if "." in s.pname else s.module
            if type(owner).__name__ == "Embedding" and self.compute_dtype == bf16 and s.shape[1] % 2 == 0:
                # token-embedding table: gradient rows are added into the owners' shards by the embedding
                # backward itself (no full fp32 table gradient, no 2.5 GB reduce-scatter per step)
                s.peer = True
                off_bytes = (u.shard_base + s.shard_off) * 4
                s.param.peer_embed_grad = (self._grad_buf.peer_ptr_list(off_bytes), s.shape[0] // self.W)
                # a head tied to this table reaches the same shards through its weight-gradient GEMM
                s.param.peer_grad = (self._grad_buf.peer_ptr_list(off_bytes), s.shape[0] // self.W, s.shape[1])
                continue
            if type(owner).__name__ != "Linear":
                continue
            s.peer = True
            off_bytes = (u.shard_base + s.shard_off) * 4
            s.param.peer_grad = (self._grad_buf.peer_ptr_list(off_bytes), s.shape[0] // self.W, s.shape[1])
            if (self.fused_gather and u.name.startswith("layers.") and s.pname.endswith("qkv_proj.weight")
                    and (s.shape[0] // self.W) % 128 == 0 and s.shape[1] % 8 == 0 and self.compute_dtype == bf16):
                s.fused_ag = True
                s.param.ag_spec = _FusedGather(self, u, s)

    def _seg_table(self, u: Unit):
        tab = self._seg_tables.get(u.name)
        if tab is None:
            esz = 2 if self.compute_dtype == bf16 else 4
            segs = []
            for s in u.slots:
                if s.ep or s.fused_ag:
                    continue
                src = (u.shard_base + s.shard_off) * esz
                if s.sharded:
                    for r in range(self.W):
                        segs.append((r, src, (s.full_off + r * s.shard_numel) * esz, s.shard_numel * esz))
                else:
                    segs.append((self.rank, src, s.full_off * esz, _align(s.numel) * esz))
            tab = self._symm.make_copy_segments(segs, self.device)
            self._seg_tables[u.name] = tab
        return tab

    # ------------------------------------------------------------------ collectives
    def _all_gather(self, u: Unit, full: torch.Tensor):
        """Gather every parameter of the unit into its full tensor inside ``full``."""
        cs = self._unit_views(u, self.compute_shard)
        if self.W == 1:
            return
        if self.comm_kind == "p2p":
            self._symm.allgather_pull(self._shard_buf, full, self._seg_table(u))
            return
        stage = torch.empty(self.W * u.shard_numel, dtype=self.compute_dtype, device=self.device)
        dist.all_gather_into_tensor(stage, cs, group=self.group)
        st = stage.view(self.W, u.shard_numel)
        for s in u.slots:
            if s.ep:        # this rank's experts stay in the shard buffers, they have no place in `full`
                continue
            dst = full[s.full_off:s.full_off + s.numel]
            if s.sharded:
                dst.view(self.W, s.shard_numel).copy_(st[:, s.shard_off:s.shard_off + s.shard_numel])
            else:
                dst.copy_(st[self.rank, s.shard_off:s.shard_off + s.numel])

    def _reduce_scatter(self, u: Unit, full_grad: torch.Tensor):
        """Sum the unit's full fp32 gradients over ranks into this rank's grad shard."""
        gs = self._unit_views(u, self.grad)
        slots = [s for s in u.slots if not s.peer]
        if not slots:
            return
        if self.comm_kind == "p2p" and full_grad.dtype == torch.float32 \
                and sum(s.numel for s in slots) <= _SCATTER_ADD_MAX:
            self._peer_scatter_add(u, slots, full_grad)
            return
        offs, tot = [], 0
        for s in slots:
            offs.append(tot)
            tot += _align(s.shard_numel)
        stage = torch.zeros(self.W, tot, dtype=torch.float32, device=self.device)
        for s, o in zip(slots, offs):
            src = full_grad[s.full_off:s.full_off + s.numel]
            if s.sharded:
                stage[:, o:o + s.shard_numel].copy_(src.view(self.W, s.shard_numel))
            else:  # replicated parameter: every rank receives the full sum
                stage[:, o:o + s.numel].copy_(src.unsqueeze(0).expand(self.W, -1))
        out = torch.empty(tot, dtype=torch.float32, device=self.device)
        dist.reduce_scatter_tensor(out, stage.view(-1), op=dist.ReduceOp.SUM, group=self.group)
        for s, o in zip(slots, offs):
            gs[s.shard_off:s.shard_off + s.shard_numel].add_(out[o:o + s.shard_numel])
            full_grad[s.full_off:s.full_off + s.numel].zero_()

    def _peer_scatter_add(self, u: Unit, slots, full_grad: torch.Tensor):
        """Small non-GEMM gradients (norm weights, biases ...): added straight into the owners'
        gradient shards with fp32 reductions over NVLink and cleared locally, in one launch and
        without a collective, so that a layer's backward has no cross-rank synchronisation point
        (a per-layer NCCL reduce-scatter made every rank wait for the slowest one 36 times a step:
        7.8 % of the 8-GPU step).  Ordered by the end-of-backward barrier like the weight-gradient
        epilogues."""
        import ctypes

        key = ("scat", u.name)
        tab = self._seg_tables.get(key)
        if tab is None:
            rows = []
            for s in slots:
                # ScatSeg {src_off, dst_off (int64), numel, shard_numel, sharded, pad (int32)} = 4 x int64
                rows.append([s.full_off, u.shard_base + s.shard_off,
                             (s.shard_numel << 32) | s.numel, int(s.sharded)])
            tab = (torch.tensor(rows, dtype=torch.int64).to(self.device), max(s.numel for s in slots))
            self._seg_tables[key] = tab
        table, max_numel = tab
        ptrs = self._grad_buf.peer_ptr_list(0)
        arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
        from ..ops import lib

        lib.call("ob_peer_scatter_add", full_grad.data_ptr(), ctypes.cast(arr, ctypes.c_void_p), self.W,
                 table.data_ptr(), len(slots), int(max_numel), lib.stream_ptr())

    # ------------------------------------------------------------------ layer execution
    def run_layer(self, layer, x, ctx):
        u = self._layer_units[id(layer)]
        if self.remat == "none" and self.W == 1:
            return layer(x, ctx)
        return _RematLayerFn.apply(x, self, u, layer, ctx)

    def _acquire(self, u: Unit, direction: int = 1):
        """Make the unit's gathered parameters current.  With peer-memory transport the gather
        of the neighbouring layer (next in forward, previous in backward) is issued on the
        communication stream into the other ring slot so it overlaps this layer's math."""
        if u.resident:
            return
        li = int(u.name.split(".")[1])
        idx = li & 1
        self._bind(u, self._ring[idx], self._ring_grad)
        if self.comm_kind != "p2p":
            self._all_gather(u, self._ring[idx])
            return
        if self._ring_owner[idx] != (u.name, self._weights_version):
            self._issue_gather(u, idx)
        torch.cuda.current_stream().wait_event(self._ring_event[idx])
        nb = self._layer_by_index.get(li + direction)
        if nb is not None and self._ring_owner[(li + direction) & 1] != (nb.name, self._weights_version):
            self._issue_gather(nb, (li + direction) & 1)

    def _issue_gather(self, u: Unit, idx: int):
        cur = torch.cuda.current_stream()
        ready = torch.cuda.Event()
        ready.record(cur)  # the previous user of this ring slot has been enqueued before this point
        with torch.cuda.stream(self._comm_stream):
            self._comm_stream.wait_event(ready)
            if _POISON:   # debugging aid: a weight element that no gather writes shows up as NaN
                self._ring[idx].fill_(float("nan"))
            self._symm.allgather_pull(self._shard_buf, self._ring[idx], self._seg_table(u))
            ev = torch.cuda.Event()
            ev.record(self._comm_stream)
        self._ring_event[idx] = ev
        self._ring_owner[idx] = (u.name, self._weights_version)
        self._fused_done[idx] = None   # the slot's in-GEMM gathered weight belongs to the previous owner

    def _release_grads(self, u: Unit):
        """After a unit's backward: fold stray autograd grads, then reduce-scatter."""
        for s in u.slots:
            p = s.param
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(torch.float32).view(p.main_grad.shape))   # local experts: [E/W, ...]
                p.grad = None
        if self.W > 1 and not u.resident:
            self._reduce_scatter(u, self._ring_grad)

    def finish_backward(self):
        """Call once after loss.backward(): handles the units that stay resident."""
        for u in self.units:
            if u.name.startswith("layers.") and not (self.W == 1):
                continue
            for s in u.slots:
                p = s.param
                if p.grad is not None:
                    p.main_grad.add_(p.grad.to(torch.float32).view(s.shape))
                    p.grad = None
            if self.W > 1 and u.resident:
                self._reduce_scatter(u, u.full_grad)
        if self.comm_kind == "p2p":
            self._barrier()  # every peer's gradient contributions to this shard have landed
        self.micro_steps += 1

    def _tp_sync_grads(self):
        """Parameters replicated over the tensor-parallel group (norms, embeddings, router, head)
        see only this rank's sequence shard: their gradient shards are summed over tp."""
        for u in self.units:
            gs = self._unit_views(u, self.grad)
            for s in u.slots:
                if not s.tp_sharded and not s.ep_product:   # an expert that lives on one rank has its whole gradient
                    dist.all_reduce(gs[s.shard_off:s.shard_off + s.shard_numel], group=self.tp_group)

    # ------------------------------------------------------------------ optimizer
    def grad_norm_sq(self) -> torch.Tensor:
        """Squared global gradient norm (unscaled accumulated gradients) as a device scalar."""
        self.norm_sq.zero_()
        if self.TP > 1:
            # tp-sharded slices add up over tp ranks, replicated parameters count once
            rep = torch.zeros(1, dtype=torch.float32, device=self.device)
            shd = torch.zeros(1, dtype=torch.float32, device=self.device)
            for u in self.units:
                gs = self._unit_views(u, self.grad)
                for s in u.slots:
                    if not s.sharded and self.W > 1 and self.rank != 0:
                        continue
                    g = gs[s.shard_off:s.shard_off + s.shard_numel]
                    (shd if (s.tp_sharded or s.ep_product) else rep).add_((g.double() ** 2).sum().float())
            dist.all_reduce(shd, group=self.tp_group)
            self.norm_sq += rep + shd
            if self.W > 1:
                dist.all_reduce(self.norm_sq, group=self.group)
            return self.norm_sq
        if self.use_cuda_kernels:
            K.sumsq(self.grad, self.norm_sq)
        else:
            acc = torch.zeros((), dtype=torch.float64, device=self.device)
            for off in range(0, self.grad.numel(), _TORCH_CHUNK):   # bounded temporaries on large shards
                acc += (self.grad[off:off + _TORCH_CHUNK].double() ** 2).sum()
            self.norm_sq += acc.float()
        if self.W > 1:
            self._dedup_replicated_norm()
            dist.all_reduce(self.norm_sq, group=self.group)
        return self.norm_sq

    def _dedup_replicated_norm(self):
        # replicated parameters hold the same summed gradient on every rank: count them once
        for u in self.units:
            gs = self._unit_views(u, self.grad)
            for s in u.slots:
                if not s.sharded and self.rank != 0:
                    g = gs[s.shard_off:s.shard_off + s.numel]
                    self.norm_sq -= (g * g).sum()

    def optimizer_step(self, lr: float | None = None, grad_accum: int = 1) -> torch.Tensor:
        """Clip by global norm, AdamW on the fp32 shard, re-cast the compute copy, zero grads.
        Returns the pre-clip gradient norm (device scalar, already divided by grad_accum)."""
        lr = self.lr if lr is None else lr
        self.step_count += 1
        gmul = 1.0 / grad_accum
        if self.TP > 1:
            self._tp_sync_grads()
        nsq = self.grad_norm_sq()
        b1, b2 = self.betas
        if self.use_cuda_kernels:
            p16 = None if self.compute_shard is self.master else self.compute_shard
            K.adamw(self.master, self.exp_avg, self.exp_avg_sq, self.grad, p16, lr=lr, b1=b1, b2=b2,
                    eps=self.eps, wd=self.wd, step=self.step_count, grad_mul=gmul, norm_sq=nsq,
                    max_norm=self.max_grad_norm, zero_grad=True)
        else:
            mul = torch.full((), gmul, dtype=torch.float32, device=self.device)
            if self.max_grad_norm > 0:
                nrm = torch.sqrt(nsq) * gmul
                mul = mul * torch.clamp(self.max_grad_norm / (nrm + 1e-6), max=1.0).reshape(())
            bc1, bc2 = 1 - b1 ** self.step_count, 1 - b2 ** self.step_count
            for off in range(0, self.grad.numel(), _TORCH_CHUNK):   # in place, chunk-sized temporaries only
                sl = slice(off, off + _TORCH_CHUNK)
                g = self.grad[sl] * mul
                m, v, pm = self.exp_avg[sl], self.exp_avg_sq[sl], self.master[sl]
                m.mul_(b1).add_(g, alpha=1 - b1)
                v.mul_(b2).addcmul_(g, g, value=1 - b2)
                upd = (m / bc1).div_((v / bc2).sqrt_().add_(self.eps))
                pm.sub_(lr * (upd + self.wd * pm))
            self.grad.zero_()
            self._refresh_compute_shard()
        if self.W > 1:
            self._weights_version += 1
            if self.comm_kind == "p2p":
                self._barrier()  # all compute shards hold the new weights before anyone pulls
            for u in self.units:
                if u.resident:
                    self._all_gather(u, u.gathered)
        self.micro_steps = 0
        if self._auto is not None and self._auto.phase == "measure":
            self._auto.open_budget(self.device, sum(1 for u in self.units if u.name.startswith("layers.")))
        return torch.sqrt(nsq) * gmul

    # ------------------------------------------------------------------ state I/O
    def named_master_shards(self):
        """Yield (name, global shape, sharded?, fp32 shard views of master/exp_avg/exp_avg_sq)."""
        for u in self.units:
            ms = self._unit_views(u, self.master)
            m1 = self._unit_views(u, self.exp_avg)
            m2 = self._unit_views(u, self.exp_avg_sq)
            for s in u.slots:
                sl = slice(s.shard_off, s.shard_off + s.shard_numel)
                yield s, ms[sl], m1[sl], m2[sl]

    def load_full_param(self, slot: ParamSlot, value: torch.Tensor):
        """Write a full fp32 parameter value into this rank's master shard."""
        u = next(u for u in self.units if slot in u.slots)
        ms = self._unit_views(u, self.master)
        flat = value.detach().to(device=self.device, dtype=torch.float32).reshape(-1)
        if slot.sharded:
            flat = flat[slot.shard_rank * slot.shard_numel:(slot.shard_rank + 1) * slot.shard_numel]
        ms[slot.shard_off:slot.shard_off + slot.shard_numel].copy_(flat)

    def sync_compute_from_master(self):
        """After the master shards were written from outside (checkpoint restore, pretrained
        loaders): re-cast the bf16 compute shards and make every gathered copy current.  With peer
        memory the peers pull from each other's compute shards, so nobody may pull before every
        rank has finished its cast (a collective: all ranks of the shard group call this)."""
        self._refresh_compute_shard()
        if self.W > 1:
            self._weights_version += 1     # gathered layers in the ring slots are stale too
            if self.comm_kind == "p2p":
                self._barrier()
            for u in self.units:
                if u.resident:
                    self._all_gather(u, u.gathered)

    def full_param(self, slot: ParamSlot) -> torch.Tensor:
        """Assemble the full fp32 master value of a parameter (collective when sharded)."""
        u = next(u for u in self.units if slot in u.slots)
        ms = self._unit_views(u, self.master)[slot.shard_off:slot.shard_off + slot.shard_numel]
        if slot.shard_world == 1 or not slot.sharded:
            return ms.clone().view(slot.shape)
        out = torch.empty(slot.shard_world * slot.shard_numel, dtype=torch.float32, device=self.device)
        dist.all_gather_into_tensor(out, ms.contiguous(), group=self.ep_group if slot.ep_product else self.group)
        return out.view(slot.shape)


class _FusedGather:
    """Attached to a weight that is gathered inside its forward GEMM (``Fn.linear`` looks for
    ``weight.ag_spec``).  ``run`` returns None when the gathered copy in the ring slot is current,
    in which case the caller uses the plain GEMM."""

    def __init__(self, engine: "TrainEngine", unit: Unit, slot: ParamSlot):
        self.engine, self.unit, self.slot = engine, unit, slot
        off = (unit.shard_base + slot.shard_off) * 2
        self.src_ptrs = engine._shard_buf.peer_ptr_list(off)
        self.flags = None

    def run(self, x2, w, residual):
        eng, s = self.engine, self.slot
        idx = int(self.unit.name.split(".")[1]) & 1
        key = (self.unit.name, eng._weights_version)
        if eng._fused_done[idx] == key or w.shape != s.shape:
            return None
        if eng._ag_flags is None:
            eng._ag_flags = torch.zeros(eng.W, dtype=torch.int32, device=eng.device)
        rows = s.shape[0] // eng.W
        ctas = K.ag_copy_ctas(x2.shape[0], s.shape[0], s.shape[1], s.numel * 2.0)
        eng._ag_count += ctas
        y = K.gemm_ag(x2, w, self.src_ptrs, side=2, rank=eng.rank, rows_per_rank=rows, flags=eng._ag_flags,
                      target=eng._ag_count, copy_ctas=ctas, residual=residual)
        eng._fused_done[idx] = key
        return y


class _LazyEP:
    """Creates the shared expert-parallel exchange (symmetric receive buffers) on first use,
    when the number of tokens per rank is known."""

    def __init__(self, engine: "TrainEngine", module):
        self.engine, self.module = engine, module

    def moe_mlp(self, x, w, idx, gate_up_local, down_local):
        eng = self.engine
        if eng.ep_kind == "a2a":
            if eng._ep is None:
                from .ep import ExpertParallelA2A

                eng._ep = ExpertParallelA2A(eng.ep_group, self.module.E)
            return eng._ep.moe_mlp(x, w, idx, gate_up_local, down_local)
        if eng._ep is None or eng._ep.max_tokens < x.shape[0]:
            from .ep import ExpertParallel

            eng._ep = ExpertParallel(eng.group, self.module.E, x.shape[1], x.shape[0], idx.shape[1],
                                     capacity_factor=eng.ep_capacity_factor, dtype=x.dtype,
                                     reuse_buffers=(eng.remat != "none"))
            eng._ep.max_tokens = x.shape[0]
        return eng._ep.moe_mlp(x, w, idx, gate_up_local, down_local)


class _AutoStash:
    """Remat policy "auto": which layers keep which of the larger tagged outputs, decided from the
    memory the device still has after one complete step (forward, backward, optimizer) has run
    with the base policy.  The first forward after that records the extra tags layer by layer
    while the budget lasts; from then on the choice is fixed.  Tags are listed in order of value
    per byte: every layer gets the first before any layer gets the second."""

    def __init__(self, extra_tags, margin_bytes: int | None = None):
        self.extra = tuple(extra_tags)
        self.phase = "measure"          # -> "grow" (one forward) -> "done"
        self.budget = 0
        self.n_layers = 0
        self.plan = None                # tag -> number of layers that may keep it
        self.per_layer: dict[int, tuple] = {}
        gb = float(os.environ.get("OMEGALAX_B200_STASH_MARGIN_GB", "6"))
        self.margin = int(gb * (1 << 30)) if margin_bytes is None else margin_bytes

    def open_budget(self, device, n_layers: int):
        fixed = os.environ.get("OMEGALAX_B200_STASH_BUDGET_MB")   # an explicit budget instead of "what is free"
        if fixed is not None:
            self.budget = int(float(fixed) * (1 << 20))
        else:
            free = torch.cuda.mem_get_info(device)[0] if torch.device(device).type == "cuda" else 0
            self.budget = max(0, free - self.margin)
        self.n_layers = n_layers
        self.phase = "grow" if self.budget > 0 and n_layers > 0 else "done"

    def tags_for(self, idx: int, base: tuple) -> tuple:
        if idx in self.per_layer:
            return base + self.per_layer[idx]
        return base + (self.extra if self.phase == "grow" else ())

    def account(self, idx: int, stash):
        """After layer ``idx`` was recorded with every extra tag: keep what fits, drop the rest."""
        if self.phase != "grow" or idx in self.per_layer:
            return
        size = {t: 0 for t in self.extra}
        for (tag, _), v in stash.items.items():
            if tag in size:
                size[tag] += v.numel() * v.element_size()
        if self.plan is None:           # layers are alike: share the budget tag by tag
            left, self.plan = self.budget, {}
            for t in self.extra:
                n = self.n_layers if size[t] == 0 else min(self.n_layers, left // size[t])
                self.plan[t] = n
                left -= n * size[t]
        keep = []
        for t in self.extra:
            if self.plan[t] > 0 and size[t] <= self.budget:
                keep.append(t)
                self.plan[t] -= 1
                self.budget -= size[t]
            else:
                for k in [k for k in stash.items if k[0] == t]:
                    del stash.items[k]
        self.per_layer[idx] = tuple(keep)

    def close(self):
        if self.phase == "grow":
            self.phase = "done"

    def summary(self) -> dict:
        return {t: sum(1 for v in self.per_layer.values() if t in v) for t in self.extra}


class _RematLayerFn(torch.autograd.Function):
    """Run a decoder layer without keeping its activations; recompute them in backward."""

    @staticmethod
    def forward(ctx, x, engine: TrainEngine, unit: Unit, layer, fctx):
        engine._acquire(unit, +1)
        # a forward pass that no backward pass follows (evaluation) keeps nothing and decides nothing
        training = bool(ctx.needs_input_grad[0])
        tags, auto = (engine.remat_tags if training else ()), engine._auto
        is_layer = unit.name.startswith("layers.")
        if auto is not None and is_layer and training:
            idx = int(unit.name.split(".")[1])
            tags = auto.tags_for(idx, tags)
        stash = Fn._Stash(tags) if tags else None
        with torch.no_grad(), Fn.stash_scope(stash, "record"):
            y, aux = layer(x, fctx)
        if auto is not None and stash is not None and is_layer and training:
            auto.account(idx, stash)
        ctx.stash = stash
        ctx.save_for_backward(x)
        ctx.engine, ctx.unit, ctx.layer, ctx.fctx = engine, unit, layer, fctx
        return y, aux

    @staticmethod
    def backward(ctx, dy, daux):
        (x,) = ctx.saved_tensors
        engine, unit, layer, fctx = ctx.engine, ctx.unit, ctx.layer, ctx.fctx
        if engine._auto is not None:
            engine._auto.close()
        engine._acquire(unit, -1)
        with torch.enable_grad(), Fn.stash_scope(ctx.stash, "replay"):
            xin = x.detach().requires_grad_(True)
            y, aux = layer(xin, fctx)
        ctx.stash = None
        with torch.enable_grad():
            outs, grads = [y], [dy]
            if aux.requires_grad:
                outs.append(aux)
                grads.append(daux if daux is not None else torch.zeros_like(aux))
            torch.autograd.backward(outs, grads)
        engine._release_grads(unit)
        return xin.grad, None, None, None, None

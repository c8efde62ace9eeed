"""Worker functions for multi-process CPU tests (gloo).  Launched by torch.multiprocessing."""
import os

import torch
import torch.distributed as dist


def _init(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)


def fsdp_train(rank, world, port, model_id, steps, out_path, ckpt_dir=None, resume=False, aux_coef=None,
               ep_transport="auto"):
    """Train `steps` optimizer steps with FSDP over `world` CPU ranks on a fixed global batch;
    rank 0 stores the loss curve and the gathered fp32 parameters."""
    _init(rank, world, port)
    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.trainers import checkpoint_utils
    from omegalax_b200.trainers import text as trainer

    mesh_lib.set_default_mesh(None)
    mesh_lib.ensure_mesh(tp_size=1, fsdp_size=world, dp_size=1)
    tcfg = trainer.TrainConfig(seed=0, batch_size=4, seq_len=32, num_steps=100, learning_rate=1e-2, max_grad_norm=1.0,
                               ep_transport=ep_transport)
    if aux_coef is not None:   # a router loss large enough to steer the run
        import dataclasses

        from omegalax_b200.models.qwen3.config import make_config

        model_id = dataclasses.replace(make_config(model_id), aux_loss_coef=aux_coef)
    model, cfg = trainer.init_model(model_id, 0, tp_size=1, fsdp_size=world, dp_size=1, meta=True)
    opt = trainer.build_optimizer(model, tcfg, device=torch.device("cpu"))
    step = trainer.make_sft_train_step(cfg)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(1, cfg.vocab_size, (4, 32), generator=g, dtype=torch.int32)
    lm = torch.ones(4, 32, dtype=torch.int32)
    lm[:, :8] = 0
    lm[1, 20:] = 0  # uneven supervised counts across ranks
    per = 4 // world
    batch = {"token_ids_BT": tok[rank * per:(rank + 1) * per], "attention_mask_BT": torch.ones(per, 32, dtype=torch.int32),
             "loss_mask_BT": lm[rank * per:(rank + 1) * per]}
    mgr = checkpoint_utils.CheckpointManager(ckpt_dir, async_write=False) if ckpt_dir else None
    if resume:
        mgr.restore(None, opt)
    losses = []
    for i in range(steps):
        loss, m = step(opt, batch)
        losses.append(float(loss))
    if mgr is not None and not resume:
        mgr.save(steps, opt)
        mgr.close()
    names = {id(p): n for n, p in model.named_parameters()}
    full = {}
    for u in opt.units:
        for s in u.slots:
            full[names[id(s.param)]] = opt.full_param(s).clone()
    if rank == 0:
        torch.save({"losses": losses, "params": full, "grad_norm": float(opt.last_grad_norm),
                    "ep_kind": getattr(opt, "ep_kind", None)}, out_path)
    dist.barrier()
    dist.destroy_process_group()


def tp_train(rank, world, port, tp, steps, out_path, untied=False, ckpt_dir=None, resume=False, moe_aux=None,
             ep_size=0):
    """Same weights, same batch: tensor-parallel (tp) x fsdp (world/tp) run on CPU ranks."""
    _init(rank, world, port)
    import dataclasses

    from omegalax_b200.models.qwen3.config import make_config
    from omegalax_b200.models.qwen3.model import Qwen3
    from omegalax_b200.models.qwen3.tp_layout import tp_slice
    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.parallel import tp as tp_lib
    from omegalax_b200.trainers import text as trainer

    mesh_lib.set_default_mesh(None)
    tp_lib.set_current(None)
    mesh = mesh_lib.ensure_mesh(tp_size=tp, fsdp_size=world // tp, dp_size=1)
    cfg = dataclasses.replace(make_config("qwen3-smoke"), num_kv_heads=2)
    if untied:   # a separate head: split over the vocabulary under tp (vocab-parallel loss)
        cfg = dataclasses.replace(cfg, tie_word_embeddings=False)
    if moe_aux is not None:   # routed experts with a router loss large enough to steer the run
        cfg = dataclasses.replace(make_config("qwen3-smoke-moe"), aux_loss_coef=moe_aux)
    torch.manual_seed(0)
    full = Qwen3(cfg, dtype=torch.float32)                       # identical on every rank
    tcfg = trainer.TrainConfig(seed=0, batch_size=2 * (world // tp), seq_len=32, num_steps=100, learning_rate=1e-2,
                               max_grad_norm=1.0, ep_size=ep_size)
    model, cfg2 = trainer.init_model(cfg, 0, tp_size=tp, fsdp_size=world // tp, dp_size=1, meta=True)
    opt = trainer.build_optimizer(model, tcfg, device=torch.device("cpu"))
    src = dict(full.named_parameters())
    names = {id(p): n for n, p in model.named_parameters()}
    tpr = mesh.coords()["tp"]
    for u in opt.units:
        for s in u.slots:
            n = names[id(s.param)]
            opt.load_full_param(s, tp_slice(n, src[n].detach(), cfg, tp, tpr))
    opt.sync_compute_from_master()
    step = trainer.make_sft_train_step(cfg2)
    g = torch.Generator().manual_seed(0)
    nb = 2 * (world // tp)
    tok = torch.randint(1, cfg.vocab_size, (nb, 32), generator=g, dtype=torch.int32)
    lm = torch.ones(nb, 32, dtype=torch.int32)
    lm[:, :5] = 0
    di = mesh_lib.data_parallel_index()
    sl = slice(di * 2, di * 2 + 2)
    batch = {"token_ids_BT": tok[sl], "attention_mask_BT": torch.ones(2, 32, dtype=torch.int32), "loss_mask_BT": lm[sl]}
    mgr = None
    if ckpt_dir:
        from omegalax_b200.trainers import checkpoint_utils

        mgr = checkpoint_utils.CheckpointManager(ckpt_dir, async_write=False)
        if resume:
            mgr.restore(None, opt)
    losses = [float(step(opt, batch)[0]) for _ in range(steps)]
    if mgr is not None and not resume:
        mgr.save(steps, opt)
    if mgr is not None:
        mgr.close()
    if rank == 0:
        torch.save({"losses": losses, "grad_norm": float(opt.last_grad_norm),
                    "vocab_parallel": bool(getattr(model, "vocab_parallel", False)),
                    "ep": (opt.ep_kind, bool(opt.ep_over_tp), sum(s.ep_product for u in opt.units for s in u.slots))},
                   out_path)
    dist.barrier()
    tp_lib.set_current(None)
    dist.destroy_process_group()


def aux_stats(rank, world, port, out_path):
    """Load-balance losses from per-rank token slices with the group's statistics: value on each
    rank and the summed gradient of sum_r aux_r / W."""
    _init(rank, world, port)
    from omegalax_b200.ops import moe as moe_ops

    g = torch.Generator().manual_seed(0)
    E, k, M = 8, 2, 64
    logits = torch.randn(M, E, generator=g)
    per = M // world
    mine = logits[rank * per:(rank + 1) * per].clone().requires_grad_(True)
    probs = torch.softmax(mine, -1)
    idx = probs.topk(k, -1).indices
    grp = dist.group.WORLD if world > 1 else None
    a1 = moe_ops.load_balance_loss_qwen3(probs, idx, E, 0.5, grp)
    a2 = moe_ops.load_balance_loss_sq(probs, E, 0.5, grp)
    ((a1 + a2) / world).backward()
    grads = [torch.zeros_like(mine) for _ in range(world)]
    dist.all_gather(grads, mine.grad)
    if rank == 0:
        torch.save({"a1": float(a1), "a2": float(a2), "grad": torch.cat(grads)}, out_path)
    dist.barrier()
    dist.destroy_process_group()


def vl_tp_train(rank, world, port, tp, steps, out_path, moe=False):
    """Qwen3-VL on an image + text batch: the text decoder tensor-parallel over ``tp`` CPU ranks
    (vision tower, embedding replicated), same weights and batch as the tp = 1 run."""
    _init(rank, world, port)
    import numpy as np

    from omegalax_b200.models.qwen3.tp_layout import tp_slice
    from omegalax_b200.models.qwen3_vl import Qwen3VL, get_rope_index, make_vl_config
    from omegalax_b200.models.vision_common import vision_cu_seqlens
    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.parallel import tp as tp_lib
    from omegalax_b200.trainers import vlm as trainer

    IMG, VID, VSTART = 1000, 1001, 1002
    mesh_lib.set_default_mesh(None)
    tp_lib.set_current(None)
    mesh = mesh_lib.ensure_mesh(tp_size=tp, fsdp_size=world // tp, dp_size=1)
    cfg = make_vl_config("qwen3-vl-smoke-moe" if moe else "qwen3-vl-smoke")
    torch.manual_seed(0)
    full = Qwen3VL(cfg, dtype=torch.float32)                     # identical on every rank
    tcfg = trainer.TrainConfig(seed=0, batch_size=2, seq_len=24, num_steps=100, learning_rate=1e-2, max_grad_norm=1.0)
    model, cfg2 = trainer.init_model(cfg, 0, tp_size=tp, fsdp_size=world // tp, dp_size=1, meta=True)
    opt = trainer.build_optimizer(model, tcfg, device=torch.device("cpu"))
    src = dict(full.named_parameters())
    names = {id(p): n for n, p in model.named_parameters()}
    tpr = mesh.coords()["tp"]
    for u in opt.units:
        for s in u.slots:
            n = names[id(s.param)]
            opt.load_full_param(s, tp_slice(n, src[n].detach(), cfg, tp, tpr))
    opt.sync_compute_from_master()
    grid = [(1, 4, 6), (1, 4, 4)]
    nm = [t * (h // 2) * (w // 2) for t, h, w in grid]
    row0 = [7, 8, VSTART] + [IMG] * nm[0] + [1003, 9, 10, VSTART] + [IMG] * nm[1] + [1003, 11, 12, 13]
    row1 = list(range(20, 20 + 19))
    T = 24
    tok = torch.tensor([row0 + [0] * (T - len(row0)), row1 + [0] * (T - len(row1))], dtype=torch.int32)
    att = (tok != 0).to(torch.int32)
    g = torch.Generator().manual_seed(3)
    pix = torch.randn(sum(t * h * w for t, h, w in grid), 3 * 2 * 14 * 14, generator=g)
    pos, _ = get_rope_index(tok.numpy().astype(np.int64), grid, None, att.numpy(), 2, IMG, VID, VSTART)
    lm = att.clone()
    lm[:, :4] = 0
    batch = {"token_ids_BT": tok, "attention_mask_BT": att, "loss_mask_BT": lm, "pixel_values": pix,
             "image_grid_thw": grid, "vision_cu_seqlens": vision_cu_seqlens(grid),
             "position_ids_ZBT": torch.from_numpy(pos)}
    step = trainer.make_sft_train_step(cfg2)
    losses = [float(step(opt, batch)[0]) for _ in range(steps)]
    if rank == 0:
        torch.save({"losses": losses, "grad_norm": float(opt.last_grad_norm),
                    "vocab_parallel": bool(getattr(model, "vocab_parallel", False))}, out_path)
    dist.barrier()
    tp_lib.set_current(None)
    dist.destroy_process_group()


def q35_tp_train(rank, world, port, tp, steps, out_path, ckpt_dir=None, resume=False, model_id="qwen3.5-smoke"):
    """Qwen3.5 hybrid (GatedDeltaNet + gated attention, MoE or dense) with attention heads,
    linear-attention heads and MLP / shared-expert width over ``tp`` CPU ranks and
    sequence-parallel rows in between; same weights and batch as the tp = 1 run."""
    _init(rank, world, port)
    from omegalax_b200.models.qwen3_5.config import make_config
    from omegalax_b200.models.qwen3_5.model import Qwen3_5ForConditionalGeneration
    from omegalax_b200.models.qwen3_5.tp_layout import tp_slice
    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.parallel import tp as tp_lib
    from omegalax_b200.trainers import vlm as trainer

    mesh_lib.set_default_mesh(None)
    tp_lib.set_current(None)
    mesh = mesh_lib.ensure_mesh(tp_size=tp, fsdp_size=world // tp, dp_size=1)
    cfg = make_config(model_id)
    torch.manual_seed(0)
    full = Qwen3_5ForConditionalGeneration(cfg, dtype=torch.float32)      # identical on every rank
    tcfg = trainer.TrainConfig(seed=0, batch_size=2, seq_len=32, num_steps=100, learning_rate=1e-3, max_grad_norm=1.0)
    model, cfg2 = trainer.init_model(cfg, 0, tp_size=tp, fsdp_size=world // tp, dp_size=1, meta=True)
    opt = trainer.build_optimizer(model, tcfg, device=torch.device("cpu"))
    src = dict(full.named_parameters())
    names = {id(p): n for n, p in model.named_parameters()}
    tpr = mesh.coords()["tp"]
    for u in opt.units:
        for s in u.slots:
            n = names[id(s.param)]
            opt.load_full_param(s, tp_slice(n, src[n].detach(), cfg, tp, tpr))
    opt.sync_compute_from_master()
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(1, 1000, (2, 32), generator=g, dtype=torch.int32)
    tok[1, 27:] = 0                                                       # right padding on one row
    att = (tok != 0).to(torch.int32)
    lm = att.clone()
    lm[:, :5] = 0
    batch = {"token_ids_BT": tok, "attention_mask_BT": att, "loss_mask_BT": lm}
    step = trainer.make_sft_train_step(cfg2)
    mgr = None
    if ckpt_dir:
        from omegalax_b200.trainers import checkpoint_utils

        mgr = checkpoint_utils.CheckpointManager(ckpt_dir, async_write=False)
        if resume:
            mgr.restore(None, opt)
    losses = [float(step(opt, batch)[0]) for _ in range(steps)]
    if mgr is not None and not resume:
        mgr.save(steps, opt)
    if mgr is not None:
        mgr.close()
    if rank == 0:
        torch.save({"losses": losses, "grad_norm": float(opt.last_grad_norm)}, out_path)
    dist.barrier()
    tp_lib.set_current(None)
    dist.destroy_process_group()


def q35_tp_gradcheck(rank, world, port, model_id, out_path):
    """fp64 gradients of a Qwen3.5 model split over ``world`` tensor-parallel ranks (no engine):
    slices re-assembled / replicated gradients summed, against the unsplit model."""
    _init(rank, world, port)
    from omegalax_b200.models.qwen3_5.config import make_config
    from omegalax_b200.models.qwen3_5.model import Qwen3_5ForCausalLM
    from omegalax_b200.models.qwen3_5.tp_layout import tp_slice, tp_unslice
    from omegalax_b200.parallel import tp as tp_lib

    cfg = make_config(model_id).text_config
    torch.manual_seed(0)
    full = Qwen3_5ForCausalLM(cfg, dtype=torch.float64)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(1, 1000, (2, 32), generator=g, dtype=torch.int32)
    seg = torch.ones_like(tok)
    seg[1, 29:] = 0
    wt = torch.randn(cfg.hidden_size, generator=g, dtype=torch.float64)
    h, aux = full(tok, seg)
    ((h.reshape(-1, h.shape[-1]) @ wt).tanh().sum() + 100.0 * aux).backward()
    ref = {n: p.grad.clone() for n, p in full.named_parameters() if p.grad is not None}
    tp_lib.set_current(tp_lib.TPContext(dist.group.WORLD))
    m = Qwen3_5ForCausalLM(cfg, dtype=torch.float64, tp_size=world)
    src = dict(full.named_parameters())
    with torch.no_grad():
        for n, p in m.named_parameters():
            p.copy_(tp_slice(n, src[n].detach(), cfg, world, rank))
    for mod in m.modules():
        if hasattr(mod, "aux_group"):
            mod.aux_group = dist.group.WORLD
    h2, aux2 = m(tok, seg, return_local_rows=True)
    ((h2 @ wt).tanh().sum() + 100.0 * aux2 / world).backward()
    errs = {}
    for n, p in m.named_parameters():
        if n not in ref:
            continue
        if tuple(p.shape) != tuple(ref[n].shape):
            parts = [torch.zeros_like(p.grad) for _ in range(world)]
            dist.all_gather(parts, p.grad.contiguous())
            got = tp_unslice(n, parts, cfg)
        else:
            got = p.grad.clone()
            dist.all_reduce(got)
        errs[n] = float((got - ref[n]).norm() / (ref[n].norm() + 1e-30))
    if rank == 0:
        torch.save({"errs": errs, "n_ref": len(ref)}, out_path)
    dist.barrier()
    tp_lib.set_current(None)
    dist.destroy_process_group()


def vl_tp_pretrained(rank, world, port, model_dir, out_path):
    """Load a HuggingFace-format Qwen3-VL checkpoint into a tp = ``world`` engine through the
    trainer's loader; rank 0 stores every rank's master copy of two split parameters."""
    _init(rank, world, port)
    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.parallel import tp as tp_lib
    from omegalax_b200.trainers import vlm as trainer

    mesh_lib.set_default_mesh(None)
    tp_lib.set_current(None)
    mesh_lib.ensure_mesh(tp_size=world, fsdp_size=1, dp_size=1)
    tcfg = trainer.TrainConfig(seed=0, batch_size=2, seq_len=24, num_steps=10, learning_rate=1e-3)
    model, cfg = trainer.init_model(model_dir, 0, tp_size=world, fsdp_size=1, dp_size=1, meta=True)
    opt = trainer.build_optimizer(model, tcfg, device=torch.device("cpu"))
    trainer._pretrained_loader(model_dir)(opt, cfg)
    names = {id(p): n for n, p in model.named_parameters()}
    mine = {}
    for u in opt.units:
        for s in u.slots:
            n = names[id(s.param)]
            if n in ("layers.0.attn.qkv_proj.weight", "layers.1.mlp.down_proj.weight", "lm_head.weight", "final_norm.weight"):
                mine[n] = opt.full_param(s).clone()
    got = [None] * world
    dist.all_gather_object(got, mine)
    if rank == 0:
        torch.save(got, out_path)
    dist.barrier()
    tp_lib.set_current(None)
    dist.destroy_process_group()


def tp_export(rank, world, port, family, out_dir):
    """Export a tensor-parallel model (slices of a seed-0 model) to the HuggingFace format."""
    _init(rank, world, port)
    import dataclasses

    from omegalax_b200 import export
    from omegalax_b200.parallel import tp as tp_lib

    tp_lib.set_current(tp_lib.TPContext(dist.group.WORLD))
    torch.manual_seed(0)
    if family == "qwen3":
        from omegalax_b200.models.qwen3.config import make_config
        from omegalax_b200.models.qwen3.model import Qwen3 as cls
        from omegalax_b200.models.qwen3.tp_layout import tp_slice

        cfg = dataclasses.replace(make_config("qwen3-smoke"), num_kv_heads=2, tie_word_embeddings=False)
    else:
        from omegalax_b200.models.qwen3_5.config import make_config
        from omegalax_b200.models.qwen3_5.model import Qwen3_5ForConditionalGeneration as cls
        from omegalax_b200.models.qwen3_5.tp_layout import tp_slice

        cfg = make_config("qwen3.5-smoke")
    full = cls(cfg, dtype=torch.float32)
    model = cls(cfg, dtype=torch.float32, tp_size=world)
    src = dict(full.named_parameters())
    with torch.no_grad():
        for n, p in model.named_parameters():
            p.copy_(tp_slice(n, src[n].detach(), cfg, world, rank))
    export.export_model_to_hf(model, cfg, out_dir)
    dist.barrier()
    tp_lib.set_current(None)
    dist.destroy_process_group()


def tp_decode(rank, world, port, out_path, moe=False):
    """Prefill + greedy decode steps with a KV cache on a model split over ``world`` tensor-parallel
    ranks (slices of a seed-0 model); rank 0 stores the logits of every call."""
    _init(rank, world, port)
    import dataclasses

    from omegalax_b200.models.qwen3.config import make_config
    from omegalax_b200.models.qwen3.model import Qwen3
    from omegalax_b200.models.qwen3.tp_layout import tp_slice
    from omegalax_b200.parallel import tp as tp_lib
    from omegalax_b200.text import api as text_api

    tp_lib.set_current(tp_lib.TPContext(dist.group.WORLD) if world > 1 else None)
    cfg = dataclasses.replace(make_config("qwen3-smoke-moe" if moe else "qwen3-smoke"), num_kv_heads=2,
                              tie_word_embeddings=False)
    torch.manual_seed(0)
    full = Qwen3(cfg, dtype=torch.float32)
    model = Qwen3(cfg, dtype=torch.float32, tp_size=world)
    src = dict(full.named_parameters())
    with torch.no_grad():
        for n, p in model.named_parameters():
            p.copy_(tp_slice(n, src[n].detach(), cfg, world, rank))
    g = torch.Generator().manual_seed(1)
    tok = torch.randint(1, cfg.vocab_size, (2, 6), generator=g)
    tok[1, :2] = 0                                   # left padding on one row
    cache = text_api.make_cache(cfg, 2, 6, 4, dtype=torch.float32, device="cpu", tp_size=world)
    outs = []
    logits, cache, _ = text_api.decode(model, cache, tok, 0, cfg)
    outs.append(logits.clone())
    for _ in range(3):
        nxt = logits.argmax(-1, keepdim=True)
        logits, cache, _ = text_api.decode(model, cache, nxt, 0, cfg)
        outs.append(logits.clone())
    if rank == 0:
        torch.save(outs, out_path)
    dist.barrier()
    tp_lib.set_current(None)
    dist.destroy_process_group()


def checkpoint_write_failure(rank, world, port, ckpt_dir, out_path):
    """Two saves with the background writer: the first succeeds, during the second rank 1's file
    write raises.  Every rank must learn of it, the failed step must not become a checkpoint, and
    the first checkpoint must survive (max_to_keep=1 would otherwise prune it)."""
    _init(rank, world, port)
    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.trainers import checkpoint_utils
    from omegalax_b200.trainers import text as trainer

    mesh_lib.set_default_mesh(None)
    mesh_lib.ensure_mesh(tp_size=1, fsdp_size=world, dp_size=1)
    tcfg = trainer.TrainConfig(seed=0, batch_size=4, seq_len=16, num_steps=10, learning_rate=1e-2)
    model, cfg = trainer.init_model("qwen3-smoke-tiny", 0, tp_size=1, fsdp_size=world, dp_size=1, meta=True)
    opt = trainer.build_optimizer(model, tcfg, device=torch.device("cpu"))
    mgr = checkpoint_utils.CheckpointManager(ckpt_dir, max_to_keep=1, async_write=True)
    mgr.save(1, opt)
    mgr.wait_until_finished()
    ok_first = mgr.latest_step() == 1
    import safetensors.torch as st

    orig = st.save_file
    if rank == 1:
        def boom(*a, **k):
            raise OSError("disk full (injected)")
        st.save_file = boom
    mgr.save(2, opt)
    raised = False
    try:
        mgr.wait_until_finished()
    except RuntimeError:
        raised = True
    st.save_file = orig
    dist.barrier()
    res = {"ok_first": ok_first, "raised": raised, "steps": mgr.all_steps()}
    torch.save(res, f"{out_path}.{rank}")
    dist.barrier()
    dist.destroy_process_group()

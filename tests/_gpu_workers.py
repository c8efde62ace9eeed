"""Worker functions for multi-GPU tests (NCCL bootstrap, one process per GPU)."""
import os

import torch
import torch.distributed as dist


def _init(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))


def symm_primitives(rank, world, port, out_path):
    _init(rank, world, port)
    from omegalax_b200.ops import kernels as K, lib
    from omegalax_b200.parallel import symm

    dev = torch.device("cuda", rank)
    res = {}
    n = 1 << 20
    shard = symm.SymmetricBuffer(n * 2)
    mine = shard.view(torch.bfloat16, n)
    mine.copy_((torch.arange(n, device=dev) % 251 + rank * 1000).to(torch.bfloat16))
    bar = symm.DeviceBarrier()
    bar()
    full = torch.zeros(world * n, dtype=torch.bfloat16, device=dev)
    tab = symm.make_copy_segments([(r, 0, r * n * 2, n * 2) for r in range(world)], dev)
    symm.allgather_pull(shard, full, tab)
    torch.cuda.synchronize()
    want = torch.cat([(torch.arange(n, device=dev) % 251 + r * 1000).to(torch.bfloat16) for r in range(world)])
    res["allgather_ok"] = bool(torch.equal(full, want))
    # GEMM whose fp32 output rows are reduced into the owning rank's buffer
    M, N, Kd = 512, 256 * world, 384
    torch.manual_seed(1 + rank)
    a = torch.randn(M, Kd, device=dev).to(torch.bfloat16)     # this rank's activations
    dy = torch.randn(M, N, device=dev).to(torch.bfloat16)
    gbuf = symm.SymmetricBuffer((N // world) * Kd * 4)
    bar()
    K.gemm_peer_reduce(dy, a, gbuf.peer_ptr_list(0), N // world, Kd, a_mn=True, b_mn=True)
    bar()
    torch.cuda.synchronize()
    got = gbuf.view(torch.float32, (N // world) * Kd).view(N // world, Kd)
    ref_local = dy.float().t() @ a.float()                        # [N, Kd] contribution of this rank
    dist.all_reduce(ref_local)
    ref = ref_local[rank * (N // world):(rank + 1) * (N // world)]
    res["peer_reduce_err"] = float((got - ref).abs().max() / ref.abs().max())
    # the same through the CTA-pair kernel (enough tiles for every SM pair)
    M2, N2, K2 = 512, 2048 * world, 2048
    a2 = torch.randn(M2, K2, device=dev).to(torch.bfloat16)
    dy2 = torch.randn(M2, N2, device=dev).to(torch.bfloat16)
    g2 = symm.SymmetricBuffer((N2 // world) * K2 * 4)
    g2.view(torch.float32, (N2 // world) * K2).zero_()
    bar()
    K.gemm_peer_reduce(dy2, a2, g2.peer_ptr_list(0), N2 // world, K2, a_mn=True, b_mn=True)
    bar()
    torch.cuda.synchronize()
    got2 = g2.view(torch.float32, (N2 // world) * K2).view(N2 // world, K2)
    ref2 = dy2.float().t() @ a2.float()
    dist.all_reduce(ref2)
    ref2 = ref2[rank * (N2 // world):(rank + 1) * (N2 // world)]
    res["pair_peer_reduce_err"] = float((got2 - ref2).abs().max() / ref2.abs().max())
    lib.check_status()
    if rank == 0:
        torch.save(res, out_path)
    dist.barrier()
    dist.destroy_process_group()


def fsdp_train_gpu(rank, world, port, comm, steps, out_path, gbatch=4):
    _init(rank, world, port)
    import dataclasses

    from omegalax_b200.ops import lib
    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.text import api as text_api
    from omegalax_b200.trainers import text as trainer
    from omegalax_b200.trainers.optim import MixedPrecisionOptimizer

    mesh_lib.set_default_mesh(None)
    mesh = mesh_lib.ensure_mesh(tp_size=1, fsdp_size=world, dp_size=1)
    cfg = dataclasses.replace(text_api.resolve_config("Qwen/Qwen3-8B"), num_layers=3, emb_dim=512, mlp_dim=1024,
                              num_heads=4, num_kv_heads=2, vocab_size=4096)
    tcfg = trainer.TrainConfig(seed=0, batch_size=gbatch, seq_len=256, num_steps=100, learning_rate=1e-3, max_grad_norm=1.0)
    model, cfg = trainer.init_model(cfg, 0, tp_size=1, fsdp_size=world, dp_size=1, meta=True)
    group = mesh.group("shard")
    opt = MixedPrecisionOptimizer(model, device=torch.device("cuda", rank), shard_group=group, lr=1e-3,
                                  weight_decay=0.01, max_grad_norm=1.0, seed=0, comm=comm)
    step = trainer.make_sft_train_step(cfg)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(1, cfg.vocab_size, (gbatch, 256), generator=g, dtype=torch.int32)
    per = gbatch // world
    sl = slice(rank * per, (rank + 1) * per)
    batch = {"token_ids_BT": tok[sl].cuda(), "attention_mask_BT": torch.ones(per, 256, dtype=torch.int32).cuda(),
             "loss_mask_BT": torch.ones(per, 256, dtype=torch.int32).cuda()}
    losses = [float(step(opt, batch)[0]) for _ in range(steps)]
    torch.cuda.synchronize()
    lib.check_status()
    if rank == 0:
        torch.save({"losses": losses, "grad_norm": float(opt.last_grad_norm),
                    "fused_gather_ctas": int(getattr(opt, "_ag_count", 0))}, out_path)
    if world > 1:
        dist.barrier()
    dist.destroy_process_group()


def ep_train_gpu(rank, world, port, steps, out_path, gbatch=4):
    """Qwen3-MoE with experts sharded over the ranks (expert parallel) vs the same run on one GPU."""
    _init(rank, world, port)
    import dataclasses

    from omegalax_b200.ops import lib
    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.text import api as text_api
    from omegalax_b200.trainers import text as trainer
    from omegalax_b200.trainers.optim import MixedPrecisionOptimizer

    mesh_lib.set_default_mesh(None)
    mesh = mesh_lib.ensure_mesh(tp_size=1, fsdp_size=world, dp_size=1)
    cfg = dataclasses.replace(text_api.resolve_config("Qwen/Qwen3-30B-A3B-Instruct-2507"), num_layers=2, emb_dim=256,
                              mlp_dim=512, moe_intermediate_size=128, num_experts=8, num_experts_per_tok=2,
                              num_heads=2, num_kv_heads=1, vocab_size=2048)
    model, cfg = trainer.init_model(cfg, 0, tp_size=1, fsdp_size=world, dp_size=1, meta=True)
    opt = MixedPrecisionOptimizer(model, device=torch.device("cuda", rank), shard_group=mesh.group("shard"), lr=1e-3,
                                  weight_decay=0.01, max_grad_norm=1.0, seed=0)
    step = trainer.make_sft_train_step(cfg)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(1, cfg.vocab_size, (gbatch, 256), generator=g, dtype=torch.int32)
    per = gbatch // world
    sl = slice(rank * per, (rank + 1) * per)
    batch = {"token_ids_BT": tok[sl].cuda(), "attention_mask_BT": torch.ones(per, 256, dtype=torch.int32).cuda(),
             "loss_mask_BT": torch.ones(per, 256, dtype=torch.int32).cuda()}
    losses = [float(step(opt, batch)[0]) for _ in range(steps)]
    torch.cuda.synchronize()
    lib.check_status()
    if opt._ep is not None:
        opt._ep.check()
    if rank == 0:
        torch.save({"losses": losses, "used_ep": opt._ep is not None}, out_path)
    if world > 1:
        dist.barrier()
    dist.destroy_process_group()


def tp_train_gpu(rank, world, port, tp, steps, out_path, rs_mode=None):
    """Tensor parallel (sequence-parallel activations, peer-memory transport) vs one GPU, same weights."""
    _init(rank, world, port)
    if rs_mode:
        os.environ["OMEGALAX_B200_TP_RS"] = rs_mode
    import dataclasses

    from omegalax_b200.models.qwen3.model import Qwen3
    from omegalax_b200.models.qwen3.tp_layout import tp_slice
    from omegalax_b200.ops import lib
    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.parallel import tp as tp_lib
    from omegalax_b200.text import api as text_api
    from omegalax_b200.trainers import text as trainer

    mesh_lib.set_default_mesh(None)
    tp_lib.set_current(None)
    mesh = mesh_lib.ensure_mesh(tp_size=tp, fsdp_size=world // tp, dp_size=1)
    cfg = dataclasses.replace(text_api.resolve_config("Qwen/Qwen3-8B"), num_layers=2, emb_dim=512, mlp_dim=1024,
                              num_heads=4, num_kv_heads=2, vocab_size=4096)
    torch.manual_seed(0)
    full = Qwen3(cfg, dtype=torch.float32)
    tcfg = trainer.TrainConfig(seed=0, batch_size=2, seq_len=256, num_steps=100, learning_rate=1e-3, max_grad_norm=1.0)
    model, cfg2 = trainer.init_model(cfg, 0, tp_size=tp, fsdp_size=world // tp, dp_size=1, meta=True)
    opt = trainer.build_optimizer(model, tcfg, device=torch.device("cuda", rank))
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
    tok = torch.randint(1, cfg.vocab_size, (2, 256), generator=g, dtype=torch.int32).cuda()
    batch = {"token_ids_BT": tok, "attention_mask_BT": torch.ones_like(tok), "loss_mask_BT": torch.ones_like(tok)}
    losses = [float(step(opt, batch)[0]) for _ in range(steps)]
    torch.cuda.synchronize()
    lib.check_status()
    ctx = tp_lib.current()
    if rank == 0:
        torch.save({"losses": losses, "transport": ctx.transport if ctx else "none",
                    "vocab_parallel": bool(getattr(model, "vocab_parallel", False)),
                    "fused_gathers": int(getattr(ctx, "_ag_calls", 0)) if ctx else 0}, out_path)
    if world > 1:
        dist.barrier()
    tp_lib.set_current(None)
    dist.destroy_process_group()


def _load_tp_slices(opt, model, full, cfg, tp, tpr, tp_slice):
    src = dict(full.named_parameters())
    names = {id(p): n for n, p in model.named_parameters()}
    for u in opt.units:
        for s in u.slots:
            n = names[id(s.param)]
            opt.load_full_param(s, tp_slice(n, src[n].detach(), cfg, tp, tpr))
    opt.sync_compute_from_master()


def q35_tp_train_gpu(rank, world, port, tp, steps, out_path):
    """Qwen3.5 hybrid MoE: gated-attention heads, GatedDeltaNet heads and the shared expert's width
    over tp, routed experts replicated on sequence-parallel rows, vs one GPU with the same weights."""
    _init(rank, world, port)
    import dataclasses

    from omegalax_b200.models.qwen3_5.config import make_config
    from omegalax_b200.models.qwen3_5.model import Qwen3_5ForCausalLM
    from omegalax_b200.models.qwen3_5.tp_layout import tp_slice
    from omegalax_b200.ops import lib
    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.parallel import tp as tp_lib
    from omegalax_b200.trainers import text as trainer

    mesh_lib.set_default_mesh(None)
    tp_lib.set_current(None)
    mesh = mesh_lib.ensure_mesh(tp_size=tp, fsdp_size=world // tp, dp_size=1)
    cfg = dataclasses.replace(make_config("qwen3.5-smoke").text_config, hidden_size=256, vocab_size=2048,
                              num_attention_heads=4, num_key_value_heads=2, head_dim=128, linear_key_head_dim=128,
                              linear_value_head_dim=128, linear_num_key_heads=2, linear_num_value_heads=4,
                              num_experts=8, num_experts_per_tok=2, moe_intermediate_size=128,
                              shared_expert_intermediate_size=128, mrope_section=(8, 4, 4))
    torch.manual_seed(0)
    full = Qwen3_5ForCausalLM(cfg, dtype=torch.float32)
    tcfg = trainer.TrainConfig(seed=0, batch_size=2, seq_len=256, num_steps=100, learning_rate=1e-3, max_grad_norm=1.0)
    model, cfg2 = trainer.init_model(cfg, 0, tp_size=tp, fsdp_size=world // tp, dp_size=1, meta=True)
    opt = trainer.build_optimizer(model, tcfg, device=torch.device("cuda", rank))
    _load_tp_slices(opt, model, full, cfg, tp, mesh.coords()["tp"], tp_slice)
    step = trainer.make_sft_train_step(cfg2)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(1, cfg.vocab_size, (2, 256), generator=g, dtype=torch.int32).cuda()
    batch = {"token_ids_BT": tok, "attention_mask_BT": torch.ones_like(tok), "loss_mask_BT": torch.ones_like(tok)}
    losses = [float(step(opt, batch)[0]) for _ in range(steps)]
    torch.cuda.synchronize()
    lib.check_status()
    if rank == 0:
        torch.save({"losses": losses, "tp_size": int(getattr(model, "tp_size", 1))}, out_path)
    if world > 1:
        dist.barrier()
    tp_lib.set_current(None)
    dist.destroy_process_group()


def vl_tp_train_gpu(rank, world, port, tp, steps, out_path):
    """Qwen3-VL with one image per row: text decoder over tp (image rows of the second sequence
    fall into the second rank's slice), vision tower replicated, vs one GPU with the same weights."""
    _init(rank, world, port)
    import dataclasses

    import numpy as np

    from omegalax_b200.models.qwen3.tp_layout import tp_slice
    from omegalax_b200.models.qwen3_vl.config import Qwen3VLVisionConfig, make_vl_config
    from omegalax_b200.models.qwen3_vl.model import Qwen3VL, get_rope_index
    from omegalax_b200.ops import lib
    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.parallel import tp as tp_lib
    from omegalax_b200.trainers import vlm as trainer

    mesh_lib.set_default_mesh(None)
    tp_lib.set_current(None)
    mesh = mesh_lib.ensure_mesh(tp_size=tp, fsdp_size=world // tp, dp_size=1)
    vis = Qwen3VLVisionConfig(hidden_size=256, intermediate_size=512, num_heads=4, patch_size=16, temporal_patch_size=2,
                              in_channels=3, spatial_merge_size=2, out_hidden_size=256, depth=2,
                              hidden_act="gelu_pytorch_tanh", num_position_embeddings=256, deepstack_visual_indexes=(0,))
    cfg = dataclasses.replace(make_vl_config("qwen3-vl-smoke"), emb_dim=256, mlp_dim=512, num_heads=4, num_kv_heads=2,
                              head_dim=128, vocab_size=2048, mrope_section=(24, 20, 20), vision=vis)
    torch.manual_seed(0)
    full = Qwen3VL(cfg, dtype=torch.float32)
    B, T, n_img = 2, 256, 16
    tcfg = trainer.TrainConfig(seed=0, batch_size=B, seq_len=T, num_steps=100, learning_rate=1e-3, max_grad_norm=1.0)
    model, cfg2 = trainer.init_model(cfg, 0, tp_size=tp, fsdp_size=world // tp, dp_size=1, meta=True)
    dev = torch.device("cuda", rank)
    opt = trainer.build_optimizer(model, tcfg, device=dev)
    _load_tp_slices(opt, model, full, cfg, tp, mesh.coords()["tp"], tp_slice)
    step = trainer.make_sft_train_step(cfg2)
    g = torch.Generator().manual_seed(0)
    tok = torch.randint(5, 1000, (B, T), generator=g, dtype=torch.int32)
    tok[:, 0] = cfg.vision_start_token_id
    tok[:, 1:1 + n_img] = cfg.image_token_id
    grid = [(1, 8, 8)] * B
    pos, _ = get_rope_index(tok.numpy(), np.asarray(grid, dtype=np.int64), None, None, 2, cfg.image_token_id,
                            cfg.video_token_id, cfg.vision_start_token_id)
    lm = torch.ones(B, T, dtype=torch.int32)
    lm[:, :1 + n_img] = 0
    batch = {"token_ids_BT": tok.to(dev), "attention_mask_BT": torch.ones(B, T, dtype=torch.int32, device=dev),
             "loss_mask_BT": lm.to(dev), "pixel_values": torch.randn(64 * B, 3 * 2 * 16 * 16, generator=g).to(dev),
             "image_grid_thw": grid, "vision_cu_seqlens": torch.arange(B + 1, dtype=torch.int32, device=dev) * 64,
             "position_ids_ZBT": torch.from_numpy(pos).to(torch.int32).to(dev)}
    losses = [float(step(opt, batch)[0]) for _ in range(steps)]
    torch.cuda.synchronize()
    lib.check_status()
    if rank == 0:
        torch.save({"losses": losses, "vocab_parallel": bool(getattr(model, "vocab_parallel", False))}, out_path)
    if world > 1:
        dist.barrier()
    tp_lib.set_current(None)
    dist.destroy_process_group()

"""Headline benchmark: SFT training throughput of Qwen3-8B (bf16 compute, fp32 master AdamW,
FSDP over the N GPUs of one node), sequence length 4096, 8 sequences per GPU (global batch
64 at N=8, weak scaling), synthetic uniform-random token ids with a 50 % prompt-masked loss.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3

Prints one JSON line (rank 0).  ``value`` is total tokens/s over all GPUs for K optimizer
steps timed with CUDA events (max over ranks) with the batches already on the device;
``e2e`` is the same quantity through ``trainers.text.make_sft_train_step`` including the
pinned-host -> device copy of every batch and a device -> host read of every step's loss.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "sft_train_tokens_per_sec"
MODEL_ID = "Qwen/Qwen3-8B"
SEQ_LEN = 4096
SEQS_PER_GPU = 8
# --model: the headline config (default) and the other text configs that are benchmarked at 8 GPUs.
# (model id, sequence length, sequences per GPU, parallelism label at N > 1)
MODELS = {
    "qwen3-8b": (MODEL_ID, SEQ_LEN, SEQS_PER_GPU, "fsdp"),
    "qwen3-30b-a3b": ("Qwen/Qwen3-30B-A3B-Instruct-2507", 4096, 4, "ep+fsdp"),
    "qwen3.5-8l": ("qwen3.5-397b-a17b-8layer", 8192, 2, "ep+fsdp"),
    # Qwen3-VL-2B: one 448x448 image (784 patches -> 196 tokens) + text ids per sample, 4 samples per GPU
    "qwen3-vl-2b": ("Qwen/Qwen3-VL-2B-Instruct", 1220, 4, "fsdp"),
}


def qwen3_vl_2b_config():
    """Architecture of the published Qwen3-VL-2B-Instruct config.json (built-in preset: no hub access here)."""
    from omegalax_b200.models.qwen3_vl.config import make_vl_config

    return make_vl_config("Qwen/Qwen3-VL-2B-Instruct")


def vlm_batches(cfg, micro: int, T: int, n: int, seed: int):
    """Synthetic VLM micro-batches in pinned host memory: per sample <vision_start>, 196 image
    placeholders (one 448x448 image, grid [1,28,28]), then random text ids; pixels ~ N(0,1)."""
    import numpy as np
    import torch

    from omegalax_b200.models.qwen3_vl.model import get_rope_index

    g = torch.Generator().manual_seed(seed)
    out = []
    n_img = 196
    for _ in range(n):
        tok = torch.randint(1, 151000, (micro, T), generator=g, dtype=torch.int32)
        tok[:, 0] = cfg.vision_start_token_id
        tok[:, 1:1 + n_img] = cfg.image_token_id
        grid = np.tile(np.array([[1, 28, 28]], dtype=np.int64), (micro, 1))
        pos, _ = get_rope_index(tok.numpy(), grid, None, None, 2, cfg.image_token_id, cfg.video_token_id,
                                cfg.vision_start_token_id)
        lm = torch.zeros(micro, T, dtype=torch.int32)
        lm[:, T // 2:] = 1
        b = {"token_ids_BT": tok, "attention_mask_BT": torch.ones(micro, T, dtype=torch.int32), "loss_mask_BT": lm,
             "pixel_values": torch.randn(784 * micro, 3 * 2 * 16 * 16, generator=g),
             "image_grid_thw": torch.from_numpy(grid).to(torch.int32),
             "vision_cu_seqlens": torch.arange(micro + 1, dtype=torch.int32) * 784,
             "position_ids_ZBT": torch.from_numpy(pos).to(torch.int32)}
        out.append({k: v.pin_memory() for k, v in b.items()})
    return out


def reference_arm(args) -> int:
    """Run the unmodified reference (baseline/_ref, a JAX program) through its own trainer API on
    the same synthetic batches; when it cannot run here, say why in one line and exit 0."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ref

    rank0 = int(os.environ.get("RANK", "0")) == 0
    model_id, def_T, def_seqs, par = MODELS[args.model]
    why = ref.availability()
    if why is None and args.model == "qwen3-vl-2b":
        why = "the reference harness drives the text trainer only"
    if why is not None:
        if rank0:
            print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    N = max(int(os.environ.get("WORLD_SIZE", "1")), 1)
    seqs = args.seqs_per_gpu or def_seqs
    T = args.seq_len or def_T
    micro = min(args.micro_seqs or (4 if N == 1 else seqs), seqs)
    try:
        res = ref.run(model_id, N, seqs, T, micro, args.steps, args.warmup)
    except Exception as e:  # pragma: no cover - depends on the box
        if rank0:
            print(json.dumps({"impl": "reference", "unavailable": f"reference run failed: {type(e).__name__}: {e}"[:300]}))
        return 0
    if rank0:
        out = {"metric": METRIC, "value": res["value"], "unit": "tokens/s", "n_gpus": N, "steps": args.steps,
               "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "weak",
               "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
               "config": {"model": model_id, "global_batch": seqs * N, "seq_len": T, "parallelism": f"fsdp{N}",
                          "micro_batch_per_gpu": micro, "grad_accum": max(seqs // micro, 1), "timer": res["timer"]},
               "e2e": res["e2e"], "gpu_launches": 0, "final_loss": res["final_loss"]}
        print(json.dumps(out), flush=True)
    return 0


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.NamedTemporaryFile(prefix="clocks_", suffix=".csv", delete=False).name
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path).read().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for nm, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        try:
            os.unlink(self.path)
        except OSError:
            pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch_baseline"],
                    help="ours: this repository's kernels and peer-memory collectives; reference: the unmodified "
                         "reference package (baseline/_ref); torch_baseline: the same models and engine with every op "
                         "a PyTorch library call (cuBLAS, flash SDPA, eager elementwise) and NCCL collectives")
    ap.add_argument("--model", default="qwen3-8b", choices=sorted(MODELS))
    ap.add_argument("--layers", type=int, default=None, help="debug only: truncate the layer stack")
    ap.add_argument("--experts", type=int, default=None, help="debug only: shrink the expert count")
    ap.add_argument("--seqs-per-gpu", type=int, default=None)
    ap.add_argument("--micro-seqs", type=int, default=None, help="sequences per GPU per micro-batch")
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--remat", default=None, help="full | selective | save:<tags> (default depends on N)")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel degree (sequence-parallel Megatron layout); "
                                                      "the remaining N / tp ranks form the FSDP / expert-parallel group")
    ap.add_argument("--ep", type=int, default=0,
                    help="expert-parallel size: 0 = the N / tp ranks of the FSDP group; N with --tp > 1 = experts over "
                         "every rank while attention stays tensor-parallel (library all-to-all transport)")
    ap.add_argument("--ep-transport", default="auto", choices=["auto", "a2a"],
                    help="a2a: token exchange by library all_to_all instead of the peer-memory kernels")
    ap.add_argument("--kernel-table", default=None,
                    help="after the timed regions, trace one more step and write its per-kernel device times here")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.impl == "torch_baseline":   # read by ops.functional / parallel.engine at call time
        os.environ["OMEGALAX_B200_OPS"] = "library"

    import dataclasses

    import torch
    import torch.distributed as dist

    from omegalax_b200.ops import kernels as K
    from omegalax_b200.ops import lib
    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.text import api as text_api
    from omegalax_b200.trainers import text as trainer
    from omegalax_b200.trainers.perf import PEAK_TFLOPS, training_flops_per_token

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N")
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    mesh_lib.init_distributed("nccl")
    rank = mesh_lib.rank()
    N = max(world, 1)

    model_id, def_T, def_seqs, par = MODELS[args.model]
    args.seqs_per_gpu = args.seqs_per_gpu or def_seqs
    args.seq_len = args.seq_len or def_T
    is_vlm = args.model == "qwen3-vl-2b"
    cfg = qwen3_vl_2b_config() if is_vlm else text_api.resolve_config(model_id)
    if args.layers is not None:
        if hasattr(cfg, "num_layers"):
            cfg = dataclasses.replace(cfg, num_layers=args.layers)
        else:
            cfg = dataclasses.replace(cfg, num_hidden_layers=args.layers, layer_types=cfg.layer_types[:args.layers])
    if args.experts is not None:
        cfg = dataclasses.replace(cfg, num_experts=args.experts)
    # N >= 2 run the same settings (8 sequences in one micro-batch, `selective` remat) so that the scaling
    # figures compare like with like; a single GPU holds all 148 GB of fp32 state and has to run two
    # micro-batches of 4 with fewer stashed activations, which is reported in `config`.
    micro = args.micro_seqs or (4 if N == 1 else args.seqs_per_gpu)
    micro = min(micro, args.seqs_per_gpu)
    accum = args.seqs_per_gpu // micro
    T = args.seq_len
    # "auto": the small attention-side tensors are kept from the first forward, and the memory that is
    # left after one whole step decides how many layers also keep the attention block's output and the
    # wide MLP activation.  One GPU holds all fp32 state (148 GB) and has room for about 15 layers; from
    # 4 GPUs on every layer keeps them (the same as "selective").
    remat = args.remat or "auto"
    if args.model != "qwen3-8b" and args.remat is None:
        # the small-hidden models have room for the stashed attention-side outputs; the Qwen3.5 slice
        # (117 GB of expert state per GPU at 8 GPUs) recomputes whole layers
        remat = "full" if args.model == "qwen3.5-8l" else "selective"
    tcfg = trainer.TrainConfig(seed=0, batch_size=micro * N, seq_len=T, num_steps=10_000, learning_rate=1e-5,
                               weight_decay=0.01, warmup_steps=0, lr_schedule="linear", max_grad_norm=1.0,
                               grad_accum_steps=accum, remat_policy=remat, ep_size=args.ep,
                               ep_transport=args.ep_transport)
    TP = max(args.tp, 1)
    if N % TP:
        raise SystemExit(f"--tp {TP} does not divide {N} GPUs")
    FS = N // TP
    mesh = mesh_lib.ensure_mesh(tp_size=TP, fsdp_size=FS, dp_size=1)
    if is_vlm:
        from omegalax_b200.trainers import vlm as vlm_trainer

        model, cfg = vlm_trainer.init_model(cfg, 0, tp_size=TP, fsdp_size=FS, dp_size=1, meta=True)
        opt = trainer.build_optimizer(model, tcfg, device=device)
        step_fn = vlm_trainer.make_sft_train_step(cfg, pad_id=0)
    else:
        model, cfg = trainer.init_model(cfg, 0, tp_size=TP, fsdp_size=FS, dp_size=1, meta=True)
        opt = trainer.build_optimizer(model, tcfg, device=device)
        step_fn = trainer.make_sft_train_step(cfg, pad_id=0)

    # synthetic data in pinned host memory: a pool of distinct micro-batches
    # the ranks of one tensor-parallel group work on the same rows: micro * TP sequences per data rank
    drank, mrows = rank // TP, micro * TP
    g = torch.Generator().manual_seed(1234 + drank)
    pool = vlm_batches(cfg, mrows, T, 4, 1234 + drank) if is_vlm else []
    for _ in range(0 if is_vlm else 4):
        tok = torch.randint(1, cfg.vocab_size, (mrows, T), generator=g, dtype=torch.int32).pin_memory()
        lm = torch.zeros(mrows, T, dtype=torch.int32)
        lm[:, T // 2:] = 1
        pool.append({"token_ids_BT": tok, "attention_mask_BT": torch.ones(mrows, T, dtype=torch.int32).pin_memory(),
                     "loss_mask_BT": lm.pin_memory()})
    h2d_bytes = sum(v.numel() * v.element_size() for v in pool[0].values()) * accum

    def to_dev(b):   # the image grid drives host-side loops and stays on the host
        return {k: (v if k == "image_grid_thw" else v.to(device, non_blocking=True)) for k, v in b.items()}

    def barrier():
        if N > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def one_step_e2e(i):
        loss = None
        for a in range(accum):
            loss, _ = step_fn(opt, to_dev(pool[(i * accum + a) % len(pool)]))
        return float(loss.item())  # device -> host read of the step's loss

    loss_step0 = None
    for i in range(args.warmup):
        l = one_step_e2e(i)
        loss_step0 = l if loss_step0 is None else loss_step0
    # the memory-adaptive remat policy settles during the second step; with fewer than three warm-up
    # steps asked for, run the missing ones here so that the timed steps are all alike
    auto, extra_warmup = getattr(opt, "_auto", None), 0
    while auto is not None and auto.phase != "done" and extra_warmup < 3:
        one_step_e2e(args.warmup + extra_warmup)
        extra_warmup += 1
    barrier()
    lib.check_status()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    # ---- device-timed region: batches already on the device
    dev_pool = [to_dev(b) for b in pool]
    barrier()
    K.reset_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        for a in range(accum):
            step_fn(opt, dev_pool[(i * accum + a) % len(dev_pool)])
    e1.record()
    barrier()
    launches = K.launch_count()
    ms = e0.elapsed_time(e1)

    # ---- end-to-end region
    barrier()
    t0 = time.perf_counter()
    last_loss = 0.0
    for i in range(args.steps):
        last_loss = one_step_e2e(i)
    barrier()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else {}
    lib.check_status()

    if args.kernel_table:   # outside both timed regions
        from omegalax_b200.utils import profiling

        def traced():
            for a in range(accum):
                step_fn(opt, dev_pool[a % len(dev_pool)])

        rows = profiling.kernel_time_table(traced, top=60)
        if rank == 0:
            with open(args.kernel_table, "w") as f:
                f.write(profiling.format_table(rows) + "\n")

    t = torch.tensor([ms, e2e_s * 1000.0], device=device)
    if N > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    tokens_per_step = args.seqs_per_gpu * T * N
    value = tokens_per_step * args.steps / (ms / 1000.0)
    e2e_value = tokens_per_step * args.steps / (e2e_ms / 1000.0)
    fpt = training_flops_per_token(cfg, T)
    if is_vlm:  # add the vision tower (per-image FLOPs spread over the sample's tokens)
        from omegalax_b200.trainers.perf import qwen3_vl_vision_training_flops

        fpt += qwen3_vl_vision_training_flops(cfg, [(1, 28, 28)]) / T
    tflops_per_gpu = value / N * fpt / 1e12
    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": N, "steps": args.steps,
            "warmup": args.warmup + extra_warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": args.impl,
            "config": {"model": model_id if args.layers is None and args.experts is None
                       else f"{model_id}[layers={args.layers or 'all'}, experts={args.experts or 'all'}]",
                       "global_batch": args.seqs_per_gpu * N, "seq_len": T,
                       "parallelism": (f"fsdp{FS}" if par == "fsdp" else
                                       f"ep{args.ep or FS}{'(a2a)' if getattr(opt, 'ep_kind', None) == 'a2a' else ''}+fsdp{FS}")
                       + (f"+tp{TP}" if TP > 1 else ""),
                       "micro_batch_per_gpu": micro, "grad_accum": accum, "optimizer": "AdamW fp32 master",
                       "remat": remat if getattr(opt, "_auto", None) is None else
                       f"auto (save:qkv,attn; layers that also keep o / gate_up: {opt._auto.summary()})", "l2": "inputs larger than L2 (weights and activations of one step far exceed 126 MB)"},
            "tokens_per_sec_per_gpu": value / N, "tflops_per_gpu": tflops_per_gpu,
            "mfu_of_measured_burst": tflops_per_gpu / PEAK_TFLOPS["b200_measured_burst"],
            "mfu_of_nominal": tflops_per_gpu / PEAK_TFLOPS["b200"],
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches, "loss_step0": loss_step0, "final_loss": last_loss,
            "peak_mem_gb": torch.cuda.max_memory_allocated(device) / 1e9,
        }
        print(json.dumps(out), flush=True)
    if N > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())

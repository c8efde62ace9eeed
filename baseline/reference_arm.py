"""Reference arm of the benchmark: the unmodified p-doom/omegalax package, driven through its own
public API (``omegalax.trainers.text``: ``init_model`` / ``build_optimizer`` /
``make_sft_train_step``, omegalax/trainers/text.py:61-190; batch placement by
``omegalax.text.api.shard_batch_dict``, omegalax/text/api.py:87), on the same synthetic batches,
model and parallelism as the product arm.  None of this repository's models, kernels or engine
is imported here.

The reference is a JAX program.  It is expected under ``baseline/_ref`` (a ``pip install
--target`` of the reference tree) together with an importable ``jax``/``flax``/``optax``; when
any of them is missing ``run`` returns the reason and the caller prints the ``unavailable`` line.
JAX exposes no device timers, so both the "device" and the end-to-end figure are host clocks
around ``block_until_ready`` (the end-to-end one includes the per-step host -> device placement
of the batch and the device -> host read of the loss).
"""
from __future__ import annotations

import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def availability() -> str | None:
    """None when the reference can run here, else a one-line reason."""
    if not os.path.isdir(os.path.join(REF_DIR, "omegalax")):
        return ("reference not installed under baseline/_ref (its build backend hatchling and its "
                "runtime jax/flax/optax/orbax/grain/tokamax are absent from the offline wheelhouse)")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    try:
        import jax  # noqa: F401
        import flax  # noqa: F401
        import optax  # noqa: F401
        import omegalax  # noqa: F401
    except Exception as e:  # pragma: no cover - depends on the box
        return f"reference runtime missing: {type(e).__name__}: {e}"[:300]
    return None


def run(model_id: str, n_gpus: int, seqs_per_gpu: int, seq_len: int, micro: int, steps: int, warmup: int) -> dict:
    """Time the reference's SFT step.  Returns the fields of the benchmark line that depend on
    the run (value, ms_per_step, e2e, final_loss); raises on any failure."""
    import jax
    import numpy as np

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:   # one process per GPU, as the product arm is launched
        port = int(os.environ.get("MASTER_PORT", "29500")) + 17
        jax.distributed.initialize(coordinator_address=f"{os.environ.get('MASTER_ADDR', '127.0.0.1')}:{port}",
                                   num_processes=world, process_id=int(os.environ.get("RANK", "0")),
                                   local_device_ids=[int(os.environ.get("LOCAL_RANK", "0"))])
    from omegalax.distributed.mesh import ensure_mesh, mesh_rules
    from omegalax.text import api as ref_api
    from omegalax.trainers import text as ref_trainer

    accum = max(seqs_per_gpu // micro, 1)
    tcfg = ref_trainer.TrainConfig(seed=0, batch_size=micro * n_gpus, seq_len=seq_len, num_steps=10_000,
                                   learning_rate=1e-5, weight_decay=0.01, warmup_steps=0, lr_schedule="linear",
                                   max_grad_norm=1.0, grad_accum_steps=accum)
    mesh = ensure_mesh(tp_size=1, fsdp_size=n_gpus, dp_size=1)
    rng = jax.random.key(0)
    with mesh_rules(mesh):
        model, cfg = ref_trainer.init_model(model_id, rng, tp_size=1, fsdp_size=n_gpus, dp_size=1)
        opt = ref_trainer.build_optimizer(model, tcfg)
    step_fn = ref_trainer.make_sft_train_step(cfg, pad_id=0)

    rank = int(os.environ.get("RANK", "0"))
    g = np.random.default_rng(1234 + rank)
    pool = []
    for _ in range(4):
        lm = np.zeros((micro, seq_len), dtype=np.int32)
        lm[:, seq_len // 2:] = 1
        pool.append({"token_ids_BT": g.integers(1, cfg.vocab_size, (micro, seq_len), dtype=np.int32),
                     "attention_mask_BT": np.ones((micro, seq_len), dtype=np.int32), "loss_mask_BT": lm})
    h2d = sum(v.nbytes for v in pool[0].values()) * accum

    def one_step(i, placed=None):
        loss = None
        for a in range(accum):
            b = placed[(i * accum + a) % len(placed)] if placed is not None else \
                ref_api.shard_batch_dict(pool[(i * accum + a) % len(pool)], cfg, mesh)
            loss, _ = step_fn(opt, b)
        return loss

    with mesh_rules(mesh):
        for i in range(warmup):
            float(one_step(i))
        placed = [ref_api.shard_batch_dict(b, cfg, mesh) for b in pool]
        jax.block_until_ready(placed)
        t0 = time.perf_counter()
        loss = None
        for i in range(steps):
            loss = one_step(i, placed)
        jax.block_until_ready(loss)
        dev_s = time.perf_counter() - t0
        t0 = time.perf_counter()
        last = 0.0
        for i in range(steps):
            last = float(one_step(i))
        e2e_s = time.perf_counter() - t0
    tokens = seqs_per_gpu * seq_len * n_gpus * steps
    return {"value": tokens / dev_s, "ms_per_step": dev_s * 1000.0 / steps,
            "e2e": {"value": tokens / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_s * 1000.0 / steps},
            "final_loss": last, "timer": "host clock around block_until_ready (JAX exposes no device events)"}

"""Shared flag helpers for the command-line scripts: every flag is accepted with underscores
(``--tp_size``, the reference's spelling) and with dashes (``--tp-size``)."""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


class Flags(argparse.ArgumentParser):
    def define(self, name: str, default=None, help: str = "", type=None, choices=None, aliases=()):
        names = []
        for n in (name, *aliases):
            names.append(f"--{n}")
            if "_" in n:
                names.append(f"--{n.replace('_', '-')}")
        if isinstance(default, bool):
            self.add_argument(*names, dest=name, default=default, help=help,
                              type=lambda s: str(s).lower() in ("1", "true", "yes", "y"), nargs="?", const=True)
        else:
            if type is None and default is not None:
                type = default.__class__
            self.add_argument(*names, dest=name, default=default, help=help, type=type, choices=choices)


def load_tokenizer(name: str):
    if name in ("stub", "", None):
        from omegalax_b200.data.stub_tokenizer import StubTokenizer

        return StubTokenizer()
    from transformers import AutoTokenizer

    return AutoTokenizer.from_pretrained(name)


def common_train_flags(p: Flags, *, batch_size: int, workers: int, worker_buffer: int):
    p.define("model_id", "qwen3-smoke", "model id, HF repo id or checkpoint directory")
    p.define("data_path", None, "chunk-index directory built by build_sft_chunk_index.py", type=str)
    p.define("tokenizer", None, "tokenizer name or 'stub' (defaults to the model's repo id)", type=str)
    p.define("max_length", 512, "padded sequence length")
    p.define("num_steps", 100)
    p.define("batch_size", batch_size, "global batch size per micro-step")
    p.define("learning_rate", 2e-5)
    p.define("weight_decay", 0.01)
    p.define("warmup_steps", 0)
    p.define("lr_schedule", "linear", choices=["linear", "cosine", "wsd"])
    p.define("lr_end_factor", 0.0)
    p.define("lr_stable_fraction", 0.8)
    p.define("max_grad_norm", 1.0)
    p.define("grad_accum_steps", 1)
    p.define("seed", 0)
    p.define("tp_size", 1)
    p.define("fsdp_size", 1)
    p.define("dp_size", 1)
    p.define("ep_size", 0, "expert parallelism: 0 automatic (experts sharded over the fsdp ranks when peer memory is "
                           "available), 1 off, or the fsdp size")
    p.define("ep_transport", "auto", "auto: peer-memory exchange kernels when available | a2a: library all-to-all",
             choices=["auto", "a2a"])
    p.define("remat_policy", "full", "full | selective | auto (selective on as many layers as the free memory after the first step allows) | save:<tag,tag> (tags: qkv, attn, o, gate_up) | none")
    p.define("save_dir", None, type=str)
    p.define("jax_cache_dir", None, "accepted for command-line compatibility; unused", type=str)
    p.define("save_every", 50)
    p.define("log_every", 10)
    p.define("profile_dir", None, type=str)
    p.define("profile_start", 3)
    p.define("profile_end", 8)
    p.define("resume", False)
    p.define("step_deadline_s", None, "watchdog: dump all stacks and exit 124 when a step takes longer", type=float)
    p.define("heartbeat_s", None, "peers publish a heartbeat; a rank silent for this long raises PeerFailure", type=float)
    p.define("pad_id", 0)
    p.define("peak_tflops", None, "preset name (e.g. b200) or a number", type=str)
    p.define("wandb_entity", None, type=str)
    p.define("wandb_project", None, type=str)
    p.define("wandb_group", None, type=str)
    p.define("wandb_name", None, type=str)
    p.define("wandb_tags", None, type=str)
    p.define("val_data_path", None, type=str)
    p.define("val_every", None, type=int)
    p.define("val_steps", 10)
    p.define("grain_read_threads", 16, "threads that read and resolve the rows of a batch")
    p.define("grain_read_buffer_size", 500, "read-ahead (the reference counts records; here batches, capped at 8)")
    p.define("grain_workers", workers, "loader processes that build batches in turn (0: a thread of the trainer)")
    p.define("grain_worker_buffer_size", worker_buffer, "finished batches each loader process keeps ready")
    p.define("log_file", None, "JSONL metrics file", type=str)

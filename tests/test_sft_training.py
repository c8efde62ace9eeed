"""Trainer integration on CPU: one optimisation pass end to end for text, VLM text-only and
VLM multimodal batches through a real (tiny) dataset; resume reproduces the loss curve."""
import json

import numpy as np
import pytest
import torch

from omegalax_b200.data import pipeline as P
from omegalax_b200.data.collator_qwen3 import TextSFTCollator, VLMSFTCollator
from omegalax_b200.data.qwen3_encoding import make_message_length_fn
from omegalax_b200.data.stub_tokenizer import SimpleImageProcessor, StubTokenizer
from omegalax_b200.models import sharding_runtime
from omegalax_b200.parallel import mesh as mesh_lib
from omegalax_b200.trainers import text as text_trainer
from omegalax_b200.trainers import vlm as vlm_trainer


@pytest.fixture(autouse=True)
def _mesh():
    mesh_lib.set_default_mesh(None)
    yield
    mesh_lib.set_default_mesh(None)


def _dataset(tmp_path, with_images=False, n=16):
    jl = tmp_path / "d.jsonl"
    rs = np.random.RandomState(0)
    with open(jl, "w") as f:
        for s in range(n):
            user = f"question {s}"
            if with_images and s % 2 == 0:
                user = [{"type": "image", "image": rs.rand(32, 32, 3).tolist()}, {"type": "text", "text": user}]
            f.write(json.dumps({"messages": [{"role": "user", "content": user},
                                             {"role": "assistant", "content": f"answer {s} " * 3}]}) + "\n")
    tok = StubTokenizer()
    ip = SimpleImageProcessor(14, 2, 2) if with_images else None
    P.compile_jsonl_to_records(jl, tmp_path / "payload")
    P.build_chunk_index(tmp_path / "payload", tmp_path / "index", make_message_length_fn(tok, ip), max_length=96)
    return tok, ip


def test_shard_batch_dict_moves_numpy_to_tensors():
    out = sharding_runtime.shard_batch_dict({"a": np.arange(6, dtype=np.int32).reshape(2, 3)}, device="cpu")
    assert torch.is_tensor(out["a"]) and out["a"].shape == (2, 3)


def test_text_sft_trains_and_resumes_identically(tmp_path):
    tok, _ = _dataset(tmp_path)
    col = TextSFTCollator(tok, 96)
    mk = lambda: P.make_data_iterator(tmp_path / "index", batch_size=4, collator=col, seed=1, num_epochs=8, dp_index=0, dp_size=1)  # noqa: E731
    cfg = lambda n: text_trainer.TrainConfig(batch_size=4, seq_len=96, num_steps=n, learning_rate=3e-3, max_grad_norm=1.0,  # noqa: E731
                                             lr_schedule="cosine", warmup_steps=2)
    logA = tmp_path / "a.jsonl"
    text_trainer.run_sft("qwen3-smoke", cfg(6), mk(), tp_size=1, fsdp_size=1, dp_size=1, log_every=1, log_file=logA,
                         device="cpu")
    straight = [json.loads(l)["loss"] for l in logA.read_text().splitlines()]
    assert straight[-1] < straight[0]
    logB = tmp_path / "b.jsonl"
    run = tmp_path / "run"
    # same 6-step schedule, stopped after 3 steps, then resumed from the checkpoint
    mesh_lib.set_default_mesh(None)
    text_trainer.run_sft("qwen3-smoke", cfg(6), mk(), tp_size=1, fsdp_size=1, dp_size=1, log_every=1, log_file=logB,
                         device="cpu", save_dir=run, save_every=3, stop_after_step=3)
    mesh_lib.set_default_mesh(None)
    text_trainer.run_sft("qwen3-smoke", cfg(6), mk(), tp_size=1, fsdp_size=1, dp_size=1, log_every=1, log_file=logB,
                         device="cpu", save_dir=run, save_every=3, resume=True)
    resumed = [json.loads(l)["loss"] for l in logB.read_text().splitlines()]
    assert len(resumed) == 6
    assert resumed == pytest.approx(straight, rel=1e-5, abs=1e-6)
    assert (run / "config.json").exists() and (run / "000006" / "manifest.json").exists()


def test_resume_skips_a_damaged_newest_checkpoint(tmp_path):
    """Failure injected on the host: the newest step's shard file is cut short (a writer that died
    mid-copy, a full disk).  Resume warns, falls back to the step before it and retrains from
    there; with every kept step damaged it raises and names the file."""
    from omegalax_b200.trainers.checkpoint_utils import CheckpointUnreadable

    tok, _ = _dataset(tmp_path)
    col = TextSFTCollator(tok, 96)
    mk = lambda: P.make_data_iterator(tmp_path / "index", batch_size=4, collator=col, seed=1, num_epochs=8, dp_index=0, dp_size=1)  # noqa: E731
    cfg = lambda n: text_trainer.TrainConfig(batch_size=4, seq_len=96, num_steps=n, learning_rate=3e-3, max_grad_norm=1.0)  # noqa: E731
    run, log = tmp_path / "run", tmp_path / "log.jsonl"
    text_trainer.run_sft("qwen3-smoke", cfg(4), mk(), tp_size=1, fsdp_size=1, dp_size=1, log_every=1, log_file=log,
                         device="cpu", save_dir=run, save_every=2)
    first = [json.loads(l) for l in log.read_text().splitlines()]
    assert (run / "000002").exists() and (run / "000004").exists()
    shard = run / "000004" / "rank00000.safetensors"
    raw = shard.read_bytes()
    shard.write_bytes(raw[: len(raw) // 2])
    mesh_lib.set_default_mesh(None)
    log2 = tmp_path / "log2.jsonl"
    with pytest.warns(UserWarning, match="rank00000.safetensors is unreadable"):
        text_trainer.run_sft("qwen3-smoke", cfg(4), mk(), tp_size=1, fsdp_size=1, dp_size=1, log_every=1, log_file=log2,
                             device="cpu", save_dir=run, save_every=2, resume=True)
    again = [json.loads(l) for l in log2.read_text().splitlines()]
    assert [m["step"] for m in again] == [3, 4]                     # restarted after step 2, not after step 4
    assert [m["loss"] for m in again] == pytest.approx([m["loss"] for m in first[2:]], rel=1e-5, abs=1e-6)
    # now both kept steps are damaged: nothing to fall back to
    for step in ("000002", "000004"):
        f = run / step / "rank00000.safetensors"
        if f.exists():
            f.write_bytes(b"not a checkpoint")
    mesh_lib.set_default_mesh(None)
    with pytest.warns(UserWarning), pytest.raises(CheckpointUnreadable, match="rank00000.safetensors"):
        text_trainer.run_sft("qwen3-smoke", cfg(4), mk(), tp_size=1, fsdp_size=1, dp_size=1, device="cpu",
                             save_dir=run, save_every=2, resume=True)


def test_vlm_text_only_and_multimodal_steps(tmp_path):
    tok, ip = _dataset(tmp_path, with_images=True)
    col = VLMSFTCollator(tok, 96, ip)
    it = P.make_data_iterator(tmp_path / "index", batch_size=2, collator=col, seed=0, num_epochs=4, dp_index=0, dp_size=1)
    cfg = vlm_trainer.TrainConfig(batch_size=2, seq_len=96, num_steps=3, learning_rate=1e-3)
    log = tmp_path / "v.jsonl"
    from omegalax_b200.models.qwen3_vl.config import make_vl_config
    import dataclasses
    vcfg = make_vl_config("qwen3-vl-smoke")
    # the stub tokenizer's special-token ids replace the preset's
    vcfg = dataclasses.replace(vcfg, image_token_id=tok.convert_tokens_to_ids("<|image_pad|>"),
                               video_token_id=tok.convert_tokens_to_ids("<|video_pad|>"),
                               vision_start_token_id=tok.convert_tokens_to_ids("<|vision_start|>"))
    _, last = vlm_trainer.run_sft(vcfg, cfg, it, tp_size=1, fsdp_size=1, dp_size=1, log_every=1, log_file=log, device="cpu")
    losses = [json.loads(l)["loss"] for l in log.read_text().splitlines()]
    assert len(losses) == 3 and all(np.isfinite(losses))
    mesh_lib.set_default_mesh(None)
    tcol = VLMSFTCollator(tok, 96, ip)
    text_it = iter([tcol([{"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "yo"}]}] * 2)] * 3)
    _, last = vlm_trainer.run_sft("qwen3.5-smoke", vlm_trainer.TrainConfig(batch_size=2, seq_len=96, num_steps=2, learning_rate=1e-3),
                                  _Plain(text_it), tp_size=1, fsdp_size=1, dp_size=1, log_every=1, device="cpu")
    assert np.isfinite(last["loss"])


class _Plain:
    def __init__(self, it):
        self.it = it

    def __iter__(self):
        return self

    def __next__(self):
        return next(self.it)

    def get_state(self):
        return {}

    def set_state(self, s):
        pass


def test_text_cli_runs_with_watchdog_and_heartbeat_flags(tmp_path):
    """The command-line trainer end to end on CPU, with the failure-detection flags set."""
    import os
    import subprocess
    import sys

    _dataset(tmp_path)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    log = tmp_path / "m.jsonl"
    cmd = [sys.executable, os.path.join(root, "scripts", "train_text_sft.py"), "--model_id", "qwen3-smoke",
           "--data_path", str(tmp_path / "index"), "--tokenizer", "stub", "--max_length", "96", "--num_steps", "3",
           "--batch-size", "2", "--log_every", "1", "--save_every", "0", "--log_file", str(log),
           "--step_deadline_s", "120", "--heartbeat_s", "5"]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    losses = [json.loads(l)["loss"] for l in log.read_text().splitlines()]
    assert len(losses) == 3 and all(np.isfinite(losses))

"""VLM SFT entry point (Qwen3.5, Qwen3-VL); one process per GPU under torchrun."""
from __future__ import annotations

from pathlib import Path

from _flags import Flags, common_train_flags, load_tokenizer


def default_save_dir(model_id: str) -> Path:
    return Path("runs") / "vlm_sft" / model_id.replace("/", "_")


def load_image_processor(name, preprocessor_config):
    if name in (None, "", "stub"):
        from omegalax_b200.data.stub_tokenizer import SimpleImageProcessor

        return SimpleImageProcessor()
    from transformers import AutoImageProcessor

    return AutoImageProcessor.from_pretrained(preprocessor_config or name)


def main(argv=None):
    p = Flags(description=__doc__)
    common_train_flags(p, batch_size=4, workers=8, worker_buffer=4)
    p.define("processor", None, "image processor name or 'stub'", type=str)
    p.define("preprocessor_config", None, type=str)
    p.define("gc_period", 0, "run the Python garbage collector every N steps (0 = default behaviour)")
    p.define("max_vision_patches_per_sample", None, type=int)
    p.define("max_vision_images_per_sample", None, type=int)
    p.define("text_attn_backend", "sm100", choices=["sm100", "reference", "mosaic_tpu", "mosaic_gpu", "cudnn", "xla", "triton"])
    a = p.parse_args(argv)

    from omegalax_b200 import registry
    from omegalax_b200.data.collator_qwen3 import VLMSFTCollator
    from omegalax_b200.data.pipeline import (load_metadata, make_data_iterator, make_grain_multiprocessing_options,
                                             make_grain_read_options, required_epochs_for_batches)
    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.trainers import vlm as vlm_trainer
    from omegalax_b200.trainers.perf import resolve_peak_tflops

    mesh_lib.init_distributed()
    mesh_lib.ensure_mesh(tp_size=a.tp_size, fsdp_size=a.fsdp_size, dp_size=a.dp_size)
    name = a.tokenizer or registry.resolve_hf_repo_id(a.model_id)
    tok = load_tokenizer(name)
    ip = load_image_processor(a.processor or ("stub" if a.tokenizer == "stub" else name), a.preprocessor_config)
    per_rank = mesh_lib.process_local_batch_size(a.batch_size)
    if a.max_vision_patches_per_sample is not None:
        m2 = int(ip.merge_size) ** 2
        if (a.max_vision_patches_per_sample * per_rank) % m2:
            raise ValueError(f"max_vision_patches_per_sample * per-process batch must be divisible by merge_size**2 = {m2}")
    collator = VLMSFTCollator(tok, a.max_length, ip, max_vision_patches_per_sample=a.max_vision_patches_per_sample,
                              max_vision_images_per_sample=a.max_vision_images_per_sample)

    def make_iter(path, shuffle, n_batches):
        n = load_metadata(path)["num_records"]
        epochs = required_epochs_for_batches(n, per_rank, n_batches, mesh_lib.data_parallel_size())
        return make_data_iterator(path, batch_size=per_rank, collator=collator, shuffle=shuffle, seed=a.seed,
                                  num_epochs=epochs,
                                  read_options=make_grain_read_options(num_threads=a.grain_read_threads,
                                                                       prefetch_buffer_size=a.grain_read_buffer_size),
                                  multiprocessing_options=make_grain_multiprocessing_options(
                                      num_workers=a.grain_workers, per_worker_buffer_size=a.grain_worker_buffer_size))

    data_iter = make_iter(a.data_path, True, a.num_steps * a.grad_accum_steps)
    val_iter = make_iter(a.val_data_path, False, max(1, (a.num_steps // max(a.val_every or a.num_steps, 1)) * a.val_steps)) \
        if a.val_data_path else None
    cfg = vlm_trainer.TrainConfig(seed=a.seed, ep_size=a.ep_size, ep_transport=a.ep_transport, batch_size=a.batch_size, seq_len=a.max_length, num_steps=a.num_steps,
                                  learning_rate=a.learning_rate, weight_decay=a.weight_decay, warmup_steps=a.warmup_steps,
                                  lr_schedule=a.lr_schedule, lr_end_factor=a.lr_end_factor,
                                  lr_stable_fraction=a.lr_stable_fraction, max_grad_norm=a.max_grad_norm,
                                  grad_accum_steps=a.grad_accum_steps, print_every=a.log_every,
                                  remat_policy=a.remat_policy, gc_period=a.gc_period, text_attn_backend=a.text_attn_backend)
    save_dir = Path(a.save_dir) if a.save_dir else (default_save_dir(a.model_id) if a.save_every > 0 or a.resume else None)
    _, last = vlm_trainer.run_sft(a.model_id, cfg, data_iter, save_dir=save_dir, save_every=a.save_every,
                                  log_every=a.log_every, resume=a.resume, pad_id=a.pad_id,
                                  peak_tflops=resolve_peak_tflops(a.peak_tflops), tp_size=a.tp_size, fsdp_size=a.fsdp_size,
                                  dp_size=a.dp_size, profile_dir=a.profile_dir,
                                  profile_steps=(a.profile_start, a.profile_end), val_data_iter=val_iter,
                                  val_every=a.val_every, val_steps=a.val_steps, log_file=a.log_file, step_deadline_s=a.step_deadline_s, heartbeat_s=a.heartbeat_s)
    if last and mesh_lib.rank() == 0:
        print(f"finished step={int(last['step'])} loss={last['loss']:.4f}")


if __name__ == "__main__":
    main()

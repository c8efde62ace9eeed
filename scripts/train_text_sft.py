"""Text SFT entry point.  Launch one process per GPU:

    torchrun --nproc-per-node 8 scripts/train_text_sft.py --model_id Qwen/Qwen3-8B \
        --data_path data/index --fsdp_size 8 --batch_size 64 --max_length 4096
"""
from __future__ import annotations

from pathlib import Path

from _flags import Flags, common_train_flags, load_tokenizer


def default_save_dir(model_id: str) -> Path:
    return Path("runs") / "text_sft" / model_id.replace("/", "_")


def main(argv=None):
    p = Flags(description=__doc__)
    common_train_flags(p, batch_size=8, workers=0, worker_buffer=1)
    a = p.parse_args(argv)

    from omegalax_b200 import registry
    from omegalax_b200.data.collator_qwen3 import TextSFTCollator
    from omegalax_b200.data.pipeline import (load_metadata, make_data_iterator, make_grain_multiprocessing_options,
                                             make_grain_read_options, required_epochs_for_batches)
    from omegalax_b200.parallel import mesh as mesh_lib
    from omegalax_b200.trainers import text as text_trainer
    from omegalax_b200.trainers.perf import resolve_peak_tflops

    mesh_lib.init_distributed()
    mesh_lib.ensure_mesh(tp_size=a.tp_size, fsdp_size=a.fsdp_size, dp_size=a.dp_size)
    tok = load_tokenizer(a.tokenizer or registry.resolve_hf_repo_id(a.model_id))
    collator = TextSFTCollator(tok, max_length=a.max_length)
    per_rank = mesh_lib.process_local_batch_size(a.batch_size)
    if mesh_lib.rank() == 0:
        print(f"global_batch_size={a.batch_size} process_count={mesh_lib.world_size()} per_process_batch_size={per_rank}")

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
    val_iter = None
    if a.val_data_path:
        val_iter = make_iter(a.val_data_path, False, max(1, (a.num_steps // max(a.val_every or a.num_steps, 1)) * a.val_steps))
    cfg = text_trainer.TrainConfig(seed=a.seed, ep_size=a.ep_size, ep_transport=a.ep_transport, batch_size=a.batch_size, seq_len=a.max_length, num_steps=a.num_steps,
                                   learning_rate=a.learning_rate, weight_decay=a.weight_decay, warmup_steps=a.warmup_steps,
                                   lr_schedule=a.lr_schedule, lr_end_factor=a.lr_end_factor,
                                   lr_stable_fraction=a.lr_stable_fraction, max_grad_norm=a.max_grad_norm,
                                   grad_accum_steps=a.grad_accum_steps, print_every=a.log_every, remat_policy=a.remat_policy)
    save_dir = Path(a.save_dir) if a.save_dir else (default_save_dir(a.model_id) if a.save_every > 0 or a.resume else None)
    wandb_run = None
    if a.wandb_project and mesh_lib.rank() == 0:
        import wandb

        wandb_run = wandb.init(entity=a.wandb_entity, project=a.wandb_project, group=a.wandb_group, name=a.wandb_name,
                               tags=a.wandb_tags.split(",") if a.wandb_tags else None, config=vars(a))
    try:
        _, last = text_trainer.run_sft(a.model_id, cfg, data_iter, save_dir=save_dir, save_every=a.save_every,
                                       log_every=a.log_every, resume=a.resume, pad_id=a.pad_id,
                                       peak_tflops=resolve_peak_tflops(a.peak_tflops), tp_size=a.tp_size,
                                       fsdp_size=a.fsdp_size, dp_size=a.dp_size, profile_dir=a.profile_dir,
                                       profile_steps=(a.profile_start, a.profile_end), wandb_run=wandb_run,
                                       val_data_iter=val_iter, val_every=a.val_every, val_steps=a.val_steps,
                                       log_file=a.log_file, step_deadline_s=a.step_deadline_s, heartbeat_s=a.heartbeat_s)
    finally:
        if wandb_run is not None:
            wandb_run.finish()
    if last and mesh_lib.rank() == 0:
        print(f"finished step={int(last['step'])} loss={last['loss']:.4f}")


if __name__ == "__main__":
    main()

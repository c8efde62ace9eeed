"""Stage 2 of the dataset build: measure messages and pack them into <= max_length chunks.

Flags as in the reference's scripts/build_sft_chunk_index.py:16-25 (``--data_path``, ``--out_dir``,
``--model_id``, ``--tokenizer``, ``--processor``, ``--preprocessor_config``, ``--max_length``,
``--records_per_shard``, ``--overwrite``, ``--num_workers``); ``--payload_dir`` and ``--output_dir``
are accepted as other spellings of the first two, and ``stub`` names the built-in offline
tokenizer / image processor."""
from __future__ import annotations

import json

from _flags import Flags, load_tokenizer


def main(argv=None):
    p = Flags(description=__doc__)
    p.define("data_path", None, "payload-record dataset written by compile_sft_dataset.py", type=str,
             aliases=("payload_dir",))
    p.define("out_dir", None, "output directory for the chunk index", type=str, aliases=("output_dir",))
    p.define("model_id", None, "model id whose repository supplies the default tokenizer", type=str)
    p.define("tokenizer", None, "tokenizer name or path, or 'stub' (defaults to --model_id)", type=str)
    p.define("processor", None, "image processor name, 'stub', or empty for text-only data", type=str)
    p.define("preprocessor_config", None, "JSON file whose keys override the image processor's defaults", type=str)
    p.define("max_length", 512, "maximum sequence length of a chunk")
    p.define("records_per_shard", 100_000, "records per output shard")
    p.define("overwrite", False, "replace an existing output directory")
    p.define("num_workers", 2, "parallel workers for the message length measurement (0 or 1: in process)")
    a = p.parse_args(argv)
    if not a.data_path or not a.out_dir:
        p.error("--data_path and --out_dir are required")
    from omegalax_b200.data.pipeline import build_chunk_index
    from omegalax_b200.data.qwen3_encoding import make_message_length_fn
    from omegalax_b200.registry import resolve_hf_repo_id

    tok_name = a.tokenizer or (resolve_hf_repo_id(a.model_id) if a.model_id else "stub")
    if tok_name.startswith(("qwen3-smoke", "qwen3.5-smoke", "qwen3-vl-smoke")):
        tok_name = "stub"           # the smoke presets have no repository to read a tokenizer from
    tok = load_tokenizer(tok_name)
    ip = None
    if a.processor == "stub":
        from omegalax_b200.data.stub_tokenizer import SimpleImageProcessor

        ip = SimpleImageProcessor()
    elif a.processor:
        from transformers import AutoImageProcessor

        kw = json.load(open(a.preprocessor_config)) if a.preprocessor_config else {}
        ip = AutoImageProcessor.from_pretrained(a.processor, use_fast=False, **kw)
    meta = build_chunk_index(a.data_path, a.out_dir, make_message_length_fn(tok, ip), max_length=a.max_length,
                             num_workers=a.num_workers, records_per_shard=a.records_per_shard, overwrite=a.overwrite,
                             profile_metadata={"model_id": a.model_id, "tokenizer": tok_name, "processor": a.processor,
                                               "preprocessor_config": a.preprocessor_config})
    print(f"wrote {meta['num_records']} chunks (max_length={a.max_length}) to {a.out_dir}")


if __name__ == "__main__":
    main()

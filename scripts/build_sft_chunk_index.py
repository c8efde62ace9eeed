"""Stage 2 of the dataset build: measure messages and pack them into <= max_length chunks."""
from __future__ import annotations

from _flags import Flags, load_tokenizer


def main(argv=None):
    p = Flags(description=__doc__)
    p.define("payload_dir", None, type=str)
    p.define("output_dir", None, type=str)
    p.define("tokenizer", "stub")
    p.define("processor", None, "image processor name, 'stub', or empty for text-only data", type=str)
    p.define("max_length", 512)
    p.define("num_workers", 0)
    a = p.parse_args(argv)
    from omegalax_b200.data.pipeline import build_chunk_index
    from omegalax_b200.data.qwen3_encoding import make_message_length_fn

    tok = load_tokenizer(a.tokenizer)
    ip = None
    if a.processor == "stub":
        from omegalax_b200.data.stub_tokenizer import SimpleImageProcessor

        ip = SimpleImageProcessor()
    elif a.processor:
        from transformers import AutoImageProcessor

        ip = AutoImageProcessor.from_pretrained(a.processor)
    meta = build_chunk_index(a.payload_dir, a.output_dir, make_message_length_fn(tok, ip), max_length=a.max_length,
                             num_workers=a.num_workers, profile_metadata={"tokenizer": a.tokenizer, "processor": a.processor})
    print(f"wrote {meta['num_records']} chunks (max_length={a.max_length}) to {a.output_dir}")


if __name__ == "__main__":
    main()

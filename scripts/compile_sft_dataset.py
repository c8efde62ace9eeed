"""Stage 1 of the dataset build: JSONL sessions -> payload record files.

Flags as in the reference's scripts/compile_sft_dataset.py:11-15 (``--data_path``, ``--out_dir``,
``--messages_per_record``, ``--records_per_shard``, ``--overwrite``); ``--input_jsonl`` and
``--output_dir`` are accepted as other spellings of the first two."""
from __future__ import annotations

from _flags import Flags


def main(argv=None):
    p = Flags(description=__doc__)
    p.define("data_path", None, "path to the raw JSONL dataset", type=str, aliases=("input_jsonl",))
    p.define("out_dir", None, "output directory for the record shards", type=str, aliases=("output_dir",))
    p.define("messages_per_record", 128, "maximum contiguous messages stored in one payload block")
    p.define("records_per_shard", 10_000, "records per output shard")
    p.define("overwrite", False, "replace an existing output directory")
    a = p.parse_args(argv)
    if not a.data_path or not a.out_dir:
        p.error("--data_path and --out_dir are required")
    from omegalax_b200.data.pipeline import compile_jsonl_to_records

    meta = compile_jsonl_to_records(a.data_path, a.out_dir, messages_per_record=a.messages_per_record,
                                    records_per_shard=a.records_per_shard, overwrite=a.overwrite)
    print(f"wrote {meta['num_records']} records ({meta['num_sessions']} sessions) in {meta['num_shards']} shard(s) to {a.out_dir}")


if __name__ == "__main__":
    main()

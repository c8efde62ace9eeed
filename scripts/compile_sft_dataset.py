"""Stage 1 of the dataset build: JSONL sessions -> payload record files."""
from __future__ import annotations

from _flags import Flags


def main(argv=None):
    p = Flags(description=__doc__)
    p.define("input_jsonl", None, type=str)
    p.define("output_dir", None, type=str)
    p.define("messages_per_record", 64)
    p.define("records_per_shard", 4096)
    a = p.parse_args(argv)
    from omegalax_b200.data.pipeline import compile_jsonl_to_records

    meta = compile_jsonl_to_records(a.input_jsonl, a.output_dir, messages_per_record=a.messages_per_record,
                                    records_per_shard=a.records_per_shard)
    print(f"wrote {meta['num_records']} records ({meta['num_sessions']} sessions) in {meta['num_shards']} shard(s) to {a.output_dir}")


if __name__ == "__main__":
    main()

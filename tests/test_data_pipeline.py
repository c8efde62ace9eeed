"""Dataset compile / chunk index / iterator: blocking, packing across payload blocks,
checkpoint-restore of the iterator, per-rank sharding, deterministic shuffle."""
import json

import numpy as np
import pytest

from omegalax_b200.data import pipeline as P
from omegalax_b200.data import recordio as rio
from omegalax_b200.data.collator_qwen3 import TextSFTCollator
from omegalax_b200.data.qwen3_encoding import make_message_length_fn
from omegalax_b200.data.stub_tokenizer import StubTokenizer


def _write_jsonl(path, sessions=23):
    with open(path, "w") as f:
        for s in range(sessions):
            msgs = [{"role": "user" if i % 2 == 0 else "assistant", "content": f"msg {i} of {s} " * (1 + (i + s) % 3)}
                    for i in range(2 + s % 6)]
            f.write(json.dumps({"messages": msgs, "source": f"s{s}"}) + "\n")


@pytest.fixture()
def dataset(tmp_path):
    jl = tmp_path / "train.jsonl"
    _write_jsonl(jl)
    P.compile_jsonl_to_records(jl, tmp_path / "payload", messages_per_record=2, records_per_shard=7)
    tok = StubTokenizer()
    P.build_chunk_index(tmp_path / "payload", tmp_path / "index", make_message_length_fn(tok), max_length=96,
                        records_per_shard=11)
    return tmp_path, tok


@pytest.mark.parametrize("native", [True, False])
def test_record_file_roundtrip(tmp_path, native):
    p = tmp_path / "x.olrf"
    with rio.RecordWriter(p, native=native) as w:
        for i in range(50):
            w.write(bytes([i % 251]) * (i * 3))
    for rn in (True, False):
        r = rio.RecordReader(p, native=rn)
        assert len(r) == 50 and r[49] == bytes([49]) * 147 and r[0] == b""
        assert r.read_many([5, 1, 49]) == [r[5], r[1], r[49]]
    raw = bytearray(p.read_bytes())
    raw[20] ^= 0xFF  # corrupt a payload byte: the checksum must catch it
    p.write_bytes(bytes(raw))
    with pytest.raises(OSError):
        rio.RecordReader(p, native=native)[1]


def test_payload_blocks_and_metadata(dataset):
    d, _ = dataset
    meta = P.load_metadata(d / "payload")
    assert meta["num_sessions"] == 23 and meta["messages_per_record"] == 2 and meta["num_shards"] > 1
    src = P.open_source(d / "payload")
    blocks = [json.loads(src[i]) for i in range(len(src))]
    assert all(len(b["messages"]) <= 2 for b in blocks)
    b0 = [b for b in blocks if b["session_id"].endswith("000000005")]
    assert [b["block_idx"] for b in b0] == list(range(len(b0)))
    assert b0[0]["session_meta"] == {"source": "s5"}


def test_chunks_never_cross_sessions_and_respect_max_length(dataset):
    d, tok = dataset
    meta = P.load_metadata(d / "index")
    assert meta["kind"] == "chunk_index" and meta["max_length"] == 96
    src = P.open_source(d / "index")
    resolver = P.ChunkResolver(meta["payload_path"])
    fn = make_message_length_fn(tok)
    total_msgs = 0
    for i in range(len(src)):
        desc = json.loads(src[i])
        ex = resolver(desc)
        assert desc["measured_length"] <= 96
        assert sum(fn(m)["length"] for m in ex["messages"]) == desc["measured_length"]
        assert len(ex["messages"]) == desc["num_messages"]
        total_msgs += desc["num_messages"]
    assert total_msgs == sum(2 + s % 6 for s in range(23))
    assert (d / "index" / "token_stats.json").exists()


def test_single_message_longer_than_max_length_is_an_error(tmp_path):
    jl = tmp_path / "a.jsonl"
    jl.write_text(json.dumps({"messages": [{"role": "user", "content": "x" * 500}]}) + "\n")
    P.compile_jsonl_to_records(jl, tmp_path / "p")
    with pytest.raises(ValueError):
        P.build_chunk_index(tmp_path / "p", tmp_path / "i", make_message_length_fn(StubTokenizer()), max_length=64)


def test_iterator_checkpoint_restore_yields_same_next_batch(dataset):
    d, tok = dataset
    col = TextSFTCollator(tok, 96)
    mk = lambda: P.make_data_iterator(d / "index", batch_size=3, collator=col, seed=7, num_epochs=3, dp_index=0, dp_size=1)  # noqa: E731
    it = mk()
    for _ in range(4):
        next(it)
    state = json.loads(json.dumps(it.get_state()))
    want = [next(it) for _ in range(3)]
    it2 = mk()
    it2.set_state(state)
    got = [next(it2) for _ in range(3)]
    for a, b in zip(want, got):
        assert all(np.array_equal(a[k], b[k]) for k in a)


def test_ranks_see_disjoint_records_and_shuffle_is_deterministic(dataset):
    d, _ = dataset
    ident = lambda rows: [r["_omegalax_session_id"] + str(r["_omegalax_measured_length"]) + str(r["messages"][0]) for r in rows]  # noqa: E731
    seen = []
    for r in range(2):
        it = P.make_data_iterator(d / "index", batch_size=2, collator=ident, seed=5, num_epochs=1, dp_index=r, dp_size=2,
                                  prefetch=0)
        seen.append([x for b in it for x in b])
    assert not (set(seen[0]) & set(seen[1]))
    again = P.make_data_iterator(d / "index", batch_size=2, collator=ident, seed=5, num_epochs=1, dp_index=0, dp_size=2)
    assert [x for b in again for x in b] == seen[0]
    other = P.make_data_iterator(d / "index", batch_size=2, collator=ident, seed=6, num_epochs=1, dp_index=0, dp_size=2)
    assert [x for b in other for x in b] != seen[0]


def test_required_epochs():
    assert P.required_epochs_for_batches(100, 8, 10, dp_size=2) == 2
    with pytest.raises(ValueError):
        P.required_epochs_for_batches(3, 8, 1)


def test_dataset_scripts_take_the_reference_flags_and_refuse_to_overwrite(tmp_path):
    """Both build stages through their command lines, with the flag names of the reference's scripts
    (scripts/compile_sft_dataset.py:11-15, scripts/build_sft_chunk_index.py:16-25); a second run into
    the same directory is refused without --overwrite."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    jl = tmp_path / "train.jsonl"
    _write_jsonl(jl, sessions=9)
    env = dict(os.environ, PYTHONPATH=root)

    def run(script, *args):
        return subprocess.run([sys.executable, os.path.join(root, "scripts", script), *args], env=env,
                              capture_output=True, text=True, timeout=300)

    a = run("compile_sft_dataset.py", "--data_path", str(jl), "--out_dir", str(tmp_path / "payload"),
            "--messages_per_record", "2", "--records_per_shard", "5")
    assert a.returncode == 0, a.stderr
    again = run("compile_sft_dataset.py", "--data_path", str(jl), "--out_dir", str(tmp_path / "payload"))
    assert again.returncode != 0 and "Refusing to overwrite" in again.stderr
    a = run("compile_sft_dataset.py", "--data_path", str(jl), "--out_dir", str(tmp_path / "payload"), "--overwrite",
            "--messages_per_record", "2")
    assert a.returncode == 0, a.stderr
    b = run("build_sft_chunk_index.py", "--data_path", str(tmp_path / "payload"), "--out_dir", str(tmp_path / "index"),
            "--model_id", "qwen3-smoke", "--max_length", "96", "--records_per_shard", "4", "--num_workers", "2")
    assert b.returncode == 0, b.stderr
    meta = P.load_metadata(tmp_path / "index")
    assert meta["num_records"] > 0 and meta["num_shards"] > 1
    assert meta.get("profile", meta).get("model_id", "qwen3-smoke") == "qwen3-smoke"
    # the older spellings still work
    c = run("build_sft_chunk_index.py", "--payload_dir", str(tmp_path / "payload"), "--output_dir",
            str(tmp_path / "index2"), "--tokenizer", "stub", "--max-length", "96", "--num_workers", "0")
    assert c.returncode == 0, c.stderr
    assert P.load_metadata(tmp_path / "index2")["num_records"] == meta["num_records"]


def test_worker_processes_and_row_threads_yield_the_same_batches(dataset):
    """Batches come out in the same order with 0, 1 or 3 loader processes and with 1 or many row
    threads; a checkpoint taken with workers continues without them (and the other way round)."""
    d, tok = dataset
    col = TextSFTCollator(tok, max_length=96)

    def mk(**kw):
        return P.make_data_iterator(d / "index", batch_size=3, collator=col, seed=11, num_epochs=2, dp_index=0,
                                    dp_size=1, **kw)

    def drain(it, n=None):
        out = []
        for b in it:
            out.append(b["token_ids_BT"].copy())
            if n is not None and len(out) == n:
                break
        return out

    base = drain(mk(prefetch=0, read_threads=1))
    assert len(base) > 6
    for kw in (dict(read_options=P.make_grain_read_options(num_threads=8)),
               dict(multiprocessing_options=P.make_grain_multiprocessing_options(num_workers=1)),
               dict(multiprocessing_options=P.make_grain_multiprocessing_options(num_workers=3, per_worker_buffer_size=2)),
               dict(multiprocessing_options=P.make_grain_multiprocessing_options(num_workers=2, start_method="spawn"))):
        it = mk(**kw)
        got = drain(it)
        it.close()
        assert len(got) == len(base)
        assert all(np.array_equal(a, b) for a, b in zip(got, base)), kw
    # stop after 4 batches with three workers, carry the state into an in-process iterator and back
    it = mk(multiprocessing_options=P.make_grain_multiprocessing_options(num_workers=3))
    head = drain(it, 4)
    state = it.get_state()
    it.close()
    it2 = mk(prefetch=0)
    it2.set_state(state)
    mid = drain(it2, 2)
    state2 = it2.get_state()
    it3 = mk(multiprocessing_options=P.make_grain_multiprocessing_options(num_workers=2))
    it3.set_state(state2)
    tail = drain(it3)
    it3.close()
    joined = head + mid + tail
    assert len(joined) == len(base) and all(np.array_equal(a, b) for a, b in zip(joined, base))


def test_failure_in_a_loader_process_reaches_the_consumer(dataset):
    d, tok = dataset

    def bad_collator(rows):
        raise KeyError("no such field")

    it = P.make_data_iterator(d / "index", batch_size=2, collator=bad_collator, seed=1, num_epochs=1, dp_index=0,
                              dp_size=1, multiprocessing_options=P.make_grain_multiprocessing_options(num_workers=2))
    with pytest.raises(P.DataLoaderError) as ei:
        next(it)
    assert "KeyError" in str(ei.value) and "no such field" in str(ei.value)
    it.close()
    assert P.resolve_arrayrecord_paths(d / "index")[0].exists()
    assert P.load_compiled_metadata(d / "index")["kind"] == "chunk_index"


def test_a_killed_loader_process_is_reported_not_waited_for(dataset):
    """Failure injected on the host: one of the loader processes dies (here: killed by its exact
    pid).  The consumer gets a DataLoaderError for the batch that process owed, instead of blocking
    on its queue; the iterator can be rebuilt from its state."""
    import os
    import signal

    d, tok = dataset
    col = TextSFTCollator(tok, max_length=96)
    mk = lambda **kw: P.make_data_iterator(d / "index", batch_size=2, collator=col, seed=3, num_epochs=4, dp_index=0,  # noqa: E731
                                           dp_size=1, **kw)
    ref = [b["token_ids_BT"].copy() for b in mk(prefetch=0)]
    it = mk(multiprocessing_options=P.make_grain_multiprocessing_options(num_workers=2))
    got = [next(it)["token_ids_BT"].copy() for _ in range(3)]
    victim = it._procs[1]
    os.kill(victim.pid, signal.SIGKILL)
    victim.join(timeout=5)
    with pytest.raises(P.DataLoaderError, match="exited with code"):
        for _ in range(8):          # batches the dead process had already queued may still arrive
            got.append(next(it)["token_ids_BT"].copy())
    state = it.get_state()
    it.close()
    again = mk(multiprocessing_options=P.make_grain_multiprocessing_options(num_workers=2))
    again.set_state(state)
    got += [b["token_ids_BT"].copy() for b in again]
    again.close()
    assert len(got) == len(ref) and all(np.array_equal(a, b) for a, b in zip(got, ref))

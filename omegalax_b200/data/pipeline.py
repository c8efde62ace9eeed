"""SFT dataset pipeline: compile JSONL sessions into record files, build a packed chunk index,
and iterate it with a deterministic, data-parallel, checkpointable loader.

Stage 1  ``compile_jsonl_to_records``: every JSONL line is a session ``{"messages": [...], ...}``;
         it is cut into *payload blocks* of at most ``messages_per_record`` consecutive messages,
         stored as sorted-key JSON in ``part-NNNNN.olrf`` shards plus ``metadata.json``.
Stage 2  ``build_chunk_index``: every message is measured once (optionally on a process pool),
         consecutive messages of one session are packed greedily into chunks whose measured
         length stays <= ``max_length`` (never across sessions; one message that is too long is
         an error); chunk descriptors go into their own record files.
Stage 3  ``make_data_iterator``: global shuffle per epoch (seeded), sharding over the
         data-parallel ranks with the remainder dropped, random access into the payload to
         resolve each descriptor (rows of a batch on a thread pool), batching through a collator
         on a prefetch thread or on worker processes that build batches in turn, and
         ``get_state`` / ``set_state`` so that a resumed run continues with the next batch
         whatever the thread / process counts on either side.
Functional reference: omegalax/data/grain_pipeline.py (which builds on grain + array_record).
"""
from __future__ import annotations

import dataclasses
import json
import multiprocessing as mp
import queue
import threading
from pathlib import Path
from typing import Any, Callable, Iterable

import numpy as np

from .recordio import RecordWriter, ShardedRecordSource

METADATA = "metadata.json"
FORMAT_VERSION = 1


# ----------------------------------------------------------------------------- stage 1
def _dumps(obj) -> bytes:
    return json.dumps(obj, sort_keys=True, ensure_ascii=False).encode("utf-8")


class _ShardedWriter:
    def __init__(self, out_dir: Path, records_per_shard: int):
        self.dir, self.per = out_dir, records_per_shard
        self.paths: list[str] = []
        self.w: RecordWriter | None = None
        self.total = 0

    def write(self, data: bytes):
        if self.w is None or self.w.count >= self.per:
            if self.w is not None:
                self.w.close()
            name = f"part-{len(self.paths):05d}.olrf"
            self.paths.append(name)
            self.w = RecordWriter(self.dir / name)
        self.w.write(data)
        self.total += 1

    def close(self):
        if self.w is not None:
            self.w.close()
            self.w = None


def iter_payload_blocks(jsonl_path, messages_per_record: int):
    """Yield payload-block dicts for every session of a JSONL file."""
    stem = Path(jsonl_path).stem
    with open(jsonl_path, "r", encoding="utf-8") as f:
        for line_no, line in enumerate(f):
            line = line.strip()
            if not line:
                continue
            session = json.loads(line)
            if "messages" not in session or not isinstance(session["messages"], list):
                raise ValueError(f"{jsonl_path}:{line_no + 1}: session has no 'messages' list")
            meta = {k: v for k, v in session.items() if k != "messages"}
            msgs = session["messages"]
            sid = f"{stem}-{line_no:09d}"
            for b, start in enumerate(range(0, max(len(msgs), 1), messages_per_record)):
                end = min(len(msgs), start + messages_per_record)
                yield {"session_id": sid, "source_line": line_no, "block_idx": b, "message_start": start,
                       "message_end": end, "session_meta": meta, "messages": msgs[start:end]}


def _prepare_output_dir(out: Path, overwrite: bool) -> None:
    """A non-empty output directory is refused unless ``overwrite``, which empties it first
    (reference: omegalax/data/grain_pipeline.py:28-40)."""
    import shutil

    if out.exists() and any(out.iterdir()):
        if not overwrite:
            raise ValueError(f"Refusing to overwrite non-empty output directory: {out}")
        for child in out.iterdir():
            if child.is_dir() and not child.is_symlink():
                shutil.rmtree(child)
            else:
                child.unlink()
    out.mkdir(parents=True, exist_ok=True)


def compile_jsonl_to_records(jsonl_path, out_dir, *, messages_per_record: int = 64,
                             records_per_shard: int = 4096, overwrite: bool = False) -> dict:
    """Stage 1.  Returns the metadata dict that was written."""
    out = Path(out_dir)
    _prepare_output_dir(out, overwrite)
    w = _ShardedWriter(out, records_per_shard)
    sessions = set()
    for block in iter_payload_blocks(jsonl_path, messages_per_record):
        sessions.add(block["session_id"])
        w.write(_dumps(block))
    w.close()
    meta = {"version": FORMAT_VERSION, "kind": "payload", "num_records": w.total, "num_shards": len(w.paths),
            "shard_paths": w.paths, "source_path": str(jsonl_path), "messages_per_record": messages_per_record,
            "num_sessions": len(sessions)}
    (out / METADATA).write_text(json.dumps(meta, indent=2))
    return meta


compile_jsonl_to_arrayrecord = compile_jsonl_to_records  # name used by the reference scripts


def load_metadata(path) -> dict:
    mp_ = Path(path).expanduser() / METADATA
    if not mp_.exists():
        raise ValueError(f"compiled dataset metadata does not exist: {mp_}")
    return json.loads(mp_.read_text())


load_compiled_metadata = load_metadata  # name used by the reference (grain_pipeline.py:231)


def resolve_record_paths(path) -> list[Path]:
    """Shard files of a compiled dataset directory (or the one shard file that was named), checked
    for existence (reference: resolve_arrayrecord_paths, grain_pipeline.py:210-228)."""
    path = Path(path).expanduser().resolve()
    if path.is_file():
        if path.suffix != ".olrf":
            raise ValueError(f"expected a record shard (.olrf) or a dataset directory, got file: {path}")
        return [path]
    shards = [path / rel for rel in load_metadata(path)["shard_paths"]]
    if not shards:
        raise ValueError(f"no record shards found under: {path}")
    missing = [p for p in shards if not p.exists()]
    if missing:
        raise ValueError(f"missing record shard(s): {missing}")
    return shards


resolve_arrayrecord_paths = resolve_record_paths


def open_source(path) -> ShardedRecordSource:
    meta = load_metadata(path)
    return ShardedRecordSource([Path(path) / p for p in meta["shard_paths"]])


# ----------------------------------------------------------------------------- stage 2
_MEASURE_FN: Callable | None = None


def _pool_init(fn):
    global _MEASURE_FN
    _MEASURE_FN = fn


def _measure_block(raw: bytes):
    block = json.loads(raw)
    out = []
    for m in block["messages"]:
        r = _MEASURE_FN(m)
        out.append(r if isinstance(r, dict) else {"length": int(r)})
    return out


def _token_stats(lengths: list[int], max_length: int) -> dict:
    a = np.asarray(lengths, dtype=np.int64)
    if a.size == 0:
        return {"num_chunks": 0}
    return {"num_chunks": int(a.size), "total_tokens": int(a.sum()), "mean": float(a.mean()),
            "p50": float(np.percentile(a, 50)), "p90": float(np.percentile(a, 90)), "p99": float(np.percentile(a, 99)),
            "max": int(a.max()), "min": int(a.min()), "fill_ratio": float(a.sum() / (a.size * max_length))}


def build_chunk_index(payload_dir, out_dir, length_fn: Callable[[dict], Any], *, max_length: int,
                      num_workers: int = 0, records_per_shard: int = 65536, profile_metadata: dict | None = None,
                      write_token_stats: bool = True, overwrite: bool = False) -> dict:
    """Stage 2.  ``length_fn(message)`` returns a token count or a dict with ``length`` and
    optional ``vision_tokens`` / ``vision_patches`` / ``num_images``."""
    src = open_source(payload_dir)
    raws = [src[i] for i in range(len(src))]
    if num_workers and num_workers > 1:
        ctx = mp.get_context("fork")
        with ctx.Pool(num_workers, initializer=_pool_init, initargs=(length_fn,)) as pool:
            measured = pool.map(_measure_block, raws, chunksize=16)
    else:
        _pool_init(length_fn)
        measured = [_measure_block(r) for r in raws]

    out = Path(out_dir)
    _prepare_output_dir(out, overwrite)
    w = _ShardedWriter(out, records_per_shard)
    lengths: list[int] = []
    cur = None  # open chunk

    def flush():
        nonlocal cur
        if cur is not None and cur["num_messages"] > 0:
            lengths.append(cur["measured_length"])
            w.write(_dumps(cur))
        cur = None

    has_vision = False
    for rec_idx, raw in enumerate(raws):
        block = json.loads(raw)
        sid = block["session_id"]
        for off, info in enumerate(measured[rec_idx]):
            L = int(info["length"])
            if L > max_length:
                raise ValueError(f"message {block['message_start'] + off} of session {sid} measures {L} tokens, "
                                 f"more than max_length={max_length}")
            if cur is not None and (cur["session_id"] != sid or cur["measured_length"] + L > max_length):
                flush()
            if cur is None:
                cur = {"session_id": sid, "start_record_idx": rec_idx, "start_message_offset": off,
                       "end_record_idx": rec_idx, "end_message_offset": off + 1, "num_messages": 0,
                       "measured_length": 0, "vision_tokens": 0, "vision_patches": 0, "num_images": 0}
            cur["end_record_idx"], cur["end_message_offset"] = rec_idx, off + 1
            cur["num_messages"] += 1
            cur["measured_length"] += L
            for k in ("vision_tokens", "vision_patches", "num_images"):
                if info.get(k):
                    has_vision = True
                    cur[k] += int(info[k])
    flush()
    w.close()
    meta = {"version": FORMAT_VERSION, "kind": "chunk_index", "num_records": w.total, "num_shards": len(w.paths),
            "shard_paths": w.paths, "payload_path": str(Path(payload_dir).resolve()),
            "payload_num_records": len(src), "max_length": max_length, "has_vision": has_vision,
            "profile_metadata": profile_metadata or {}}
    (out / METADATA).write_text(json.dumps(meta, indent=2))
    if write_token_stats:
        (out / "token_stats.json").write_text(json.dumps(_token_stats(lengths, max_length), indent=2))
    return meta


# ----------------------------------------------------------------------------- stage 3
def required_epochs_for_batches(num_records: int, batch_size: int, num_batches: int, dp_size: int = 1) -> int:
    """Epochs needed so that every rank can draw ``num_batches`` batches (remainders dropped)."""
    per_rank = num_records // dp_size
    per_epoch = per_rank // batch_size
    if per_epoch <= 0:
        raise ValueError(f"dataset of {num_records} records cannot fill one batch of {batch_size} on {dp_size} ranks")
    return -(-num_batches // per_epoch)


class IndexSampler:
    """Deterministic global order: per-epoch permutation of all records (seed + epoch), the
    tail that does not divide by ``dp_size`` dropped, record j of the kept prefix going to
    rank j % dp_size."""

    def __init__(self, num_records: int, *, shuffle: bool, seed: int, num_epochs: int | None, dp_index: int,
                 dp_size: int):
        self.n, self.shuffle, self.seed = num_records, shuffle, seed
        self.num_epochs, self.dp_index, self.dp_size = num_epochs, dp_index, dp_size
        self.per_rank = num_records // dp_size
        self._cache: tuple[int, np.ndarray] | None = None

    def epoch_order(self, epoch: int) -> np.ndarray:
        if self._cache is not None and self._cache[0] == epoch:
            return self._cache[1]
        if self.shuffle:
            order = np.random.default_rng([self.seed, epoch]).permutation(self.n)
        else:
            order = np.arange(self.n)
        order = order[: self.per_rank * self.dp_size][self.dp_index::self.dp_size]
        self._cache = (epoch, order)
        return order

    def __len__(self):
        return self.per_rank * (self.num_epochs or 1)

    def record_at(self, position: int) -> int | None:
        """Record index of this rank's ``position``-th sample, None when exhausted."""
        if self.per_rank == 0:
            return None
        epoch, k = divmod(position, self.per_rank)
        if self.num_epochs is not None and epoch >= self.num_epochs:
            return None
        return int(self.epoch_order(epoch)[k])


def _identity(d):
    return d


class ChunkResolver:
    """Turns a chunk descriptor into the example dict a collator consumes by random access
    into the payload shards."""

    def __init__(self, payload_path):
        self.payload_path = str(payload_path)
        self._src: ShardedRecordSource | None = None

    def __getstate__(self):
        return {"payload_path": self.payload_path, "_src": None}

    def __call__(self, desc: dict) -> dict:
        if self._src is None:
            self._src = open_source(self.payload_path)
        msgs, meta = [], {}
        for rec in range(desc["start_record_idx"], desc["end_record_idx"] + 1):
            block = json.loads(self._src[rec])
            lo = desc["start_message_offset"] if rec == desc["start_record_idx"] else 0
            hi = desc["end_message_offset"] if rec == desc["end_record_idx"] else len(block["messages"])
            msgs.extend(block["messages"][lo:hi])
            meta = block.get("session_meta", meta)
        out = dict(meta) if isinstance(meta, dict) else {}
        out.update(messages=msgs, _omegalax_session_id=desc["session_id"],
                   _omegalax_measured_length=desc["measured_length"], _omegalax_num_messages=desc["num_messages"])
        return out


@dataclasses.dataclass(frozen=True)
class ReadOptions:
    """How the rows of one batch are fetched: ``num_threads`` rows are read and resolved against
    the payload at the same time (the record files are memory-mapped; the reads and the JSON
    decoding of large image payloads overlap); ``prefetch_buffer_size`` batches are kept ready
    ahead of the consumer when no worker processes are used.  (reference: grain.ReadOptions as built by
    omegalax/data/grain_pipeline.py:587-592)"""

    num_threads: int = 16
    prefetch_buffer_size: int = 2


@dataclasses.dataclass(frozen=True)
class MultiprocessingOptions:
    """``num_workers`` processes build batches in turn (worker w builds batches w, w + N, ...), each
    keeping ``per_worker_buffer_size`` finished batches ready; 0 builds them on a thread of the
    training process.  (reference: grain.MultiprocessingOptions, grain_pipeline.py:595-605)"""

    num_workers: int = 0
    per_worker_buffer_size: int = 1
    # "fork": the collator and tokenizer reach the workers by inheritance (anything works, but the
    # parent should not hold locks in other threads at that moment); "spawn" / "forkserver": they
    # are pickled into fresh interpreters (no inherited threads or CUDA state)
    start_method: str = "fork"


def make_grain_read_options(*, num_threads: int = 16, prefetch_buffer_size: int = 500) -> ReadOptions:
    """The reference's prefetch buffer counts records; here it counts batches and is capped."""
    return ReadOptions(num_threads=max(int(num_threads), 1), prefetch_buffer_size=max(2, min(int(prefetch_buffer_size), 8)))


def make_grain_multiprocessing_options(*, num_workers: int = 0, per_worker_buffer_size: int = 1,
                                       enable_profiling: bool = False, start_method: str = "fork") -> MultiprocessingOptions:
    del enable_profiling   # grain's own profiler; nothing to switch on here
    if start_method not in ("fork", "spawn", "forkserver"):
        raise ValueError(f"unknown start method {start_method!r}")
    return MultiprocessingOptions(num_workers=max(int(num_workers), 0),
                                  per_worker_buffer_size=max(int(per_worker_buffer_size), 1), start_method=start_method)


def _worker_process_main(it: "DataIterator", wid: int, nworkers: int, start: int, q, stop):
    """Body of one loader process (forked, so ``it`` is the parent's iterator object): builds the
    batches b >= start with b % nworkers == wid, in order, until the data ends or ``stop`` is set."""
    import pickle
    import traceback

    b = start + ((wid - start) % nworkers)
    pool = it._row_pool()
    try:
        while not stop.is_set():
            try:
                item = it._make_batch(b, pool)
                payload = ("ok", item)
                pickle.dumps(payload)     # a batch that cannot cross the process boundary is reported, not lost
            except BaseException as e:    # delivered to the consumer
                payload = ("err", f"{type(e).__name__}: {e}\n{traceback.format_exc()}")
            while not stop.is_set():
                try:
                    q.put((b, payload), timeout=0.1)
                    break
                except queue.Full:
                    continue
            if payload[0] == "err" or payload[1] is None:
                break
            b += nworkers
    finally:
        if pool is not None:
            pool.shutdown(wait=False)
        q.close()
        q.join_thread()


class DataLoaderError(RuntimeError):
    """A loader process failed; the message carries its traceback."""


class DataIterator:
    """Checkpointable batch iterator.  ``state`` is the number of batches handed out; restoring
    it makes the next ``next()`` return exactly the batch the saved run would have produced,
    whatever the number of threads or worker processes on either side."""

    def __init__(self, index_source, sampler: IndexSampler, transform: Callable[[dict], dict], batch_size: int,
                 batch_fn: Callable[[list], Any], *, prefetch: int = 2, read_threads: int = 4, num_workers: int = 0,
                 worker_buffer: int = 1, start_method: str = "fork"):
        self.src, self.sampler, self.transform = index_source, sampler, transform
        self.batch_size, self.batch_fn = batch_size, batch_fn
        self.prefetch, self.read_threads = max(int(prefetch), 0), max(int(read_threads), 1)
        self.num_workers, self.worker_buffer = max(int(num_workers), 0), max(int(worker_buffer), 1)
        self.start_method = start_method
        self._consumed = 0
        self._q: queue.Queue | None = None
        self._thread: threading.Thread | None = None
        self._stop = threading.Event()
        self._procs: list = []
        self._pqs: list = []
        self._pstop = None
        self._pool = None

    def __getstate__(self):     # what a spawned loader process needs: no queues, threads or children
        st = dict(self.__dict__)
        st.update(_q=None, _thread=None, _stop=None, _procs=[], _pqs=[], _pstop=None, _pool=None)
        return st

    def __setstate__(self, st):
        self.__dict__.update(st)
        self._stop = threading.Event()

    def _row_pool(self):
        if self.read_threads <= 1 or self.batch_size <= 1:
            return None
        from concurrent.futures import ThreadPoolExecutor

        return ThreadPoolExecutor(max_workers=min(self.read_threads, self.batch_size), thread_name_prefix="loader-row")

    def _row(self, rec: int):
        return self.transform(json.loads(self.src[rec]))

    def _make_batch(self, b: int, pool=None):
        recs = []
        for k in range(self.batch_size):
            rec = self.sampler.record_at(b * self.batch_size + k)
            if rec is None:
                return None
            recs.append(rec)
        rows = list(pool.map(self._row, recs)) if pool is not None else [self._row(r) for r in recs]
        return self.batch_fn(rows)

    def _worker(self, start: int, q: queue.Queue, stop: threading.Event):
        b = start
        pool = self._row_pool()
        try:
            while not stop.is_set():
                try:
                    item = self._make_batch(b, pool)
                except BaseException as e:  # delivered to the consumer
                    item = e
                while not stop.is_set():
                    try:
                        q.put((b, item), timeout=0.1)
                        break
                    except queue.Full:
                        continue
                if item is None or isinstance(item, BaseException):
                    return
                b += 1
        finally:
            if pool is not None:
                pool.shutdown(wait=False)

    def _ensure_worker(self):
        if self.num_workers > 0:
            if self._procs:
                return
            ctx = mp.get_context(self.start_method)
            self._pstop = ctx.Event()
            self._pqs = [ctx.Queue(maxsize=self.worker_buffer) for _ in range(self.num_workers)]
            for w in range(self.num_workers):
                p = ctx.Process(target=_worker_process_main, name=f"loader-{w}", daemon=True,
                                args=(self, w, self.num_workers, self._consumed, self._pqs[w], self._pstop))
                p.start()
                self._procs.append(p)
            return
        if self.prefetch == 0 or self._thread is not None:
            return
        self._stop = threading.Event()
        self._q = queue.Queue(maxsize=self.prefetch)
        self._thread = threading.Thread(target=self._worker, args=(self._consumed, self._q, self._stop), daemon=True)
        self._thread.start()

    def _shutdown(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=5)
            self._thread, self._q = None, None
        if self._procs:
            self._pstop.set()
            for q in self._pqs:          # unblock producers that wait on a full queue
                try:
                    while True:
                        q.get_nowait()
                except Exception:
                    pass
            for p in self._procs:
                p.join(timeout=5)
                if p.is_alive():
                    p.terminate()
                    p.join(timeout=2)
            for q in self._pqs:
                q.close()
                q.cancel_join_thread()
            self._procs, self._pqs, self._pstop = [], [], None
        if self._pool is not None:
            self._pool.shutdown(wait=False)
            self._pool = None

    def __iter__(self):
        return self

    def _next_from_processes(self):
        w = self._consumed % self.num_workers
        q, p = self._pqs[w], self._procs[w]
        while True:
            try:
                b, (kind, item) = q.get(timeout=1.0)
                break
            except queue.Empty:
                if not p.is_alive():
                    try:                 # it may have finished between the time-out and this check
                        b, (kind, item) = q.get(timeout=0.5)
                        break
                    except queue.Empty:
                        self._shutdown()
                        raise DataLoaderError(f"loader process {w} exited with code {p.exitcode} without a result") from None
        assert b == self._consumed, (b, self._consumed)
        if kind == "err":
            self._shutdown()
            raise DataLoaderError(f"loader process {w} failed on batch {b}:\n{item}")
        return item

    def __next__(self):
        if self.num_workers > 0:
            self._ensure_worker()
            item = self._next_from_processes()
        elif self.prefetch == 0:
            if self._pool is None:
                self._pool = self._row_pool()
            item = self._make_batch(self._consumed, self._pool)
        else:
            self._ensure_worker()
            b, item = self._q.get()
            assert b == self._consumed, (b, self._consumed)
        if isinstance(item, BaseException):
            self._shutdown()
            raise item
        if item is None:
            self._shutdown()
            raise StopIteration
        self._consumed += 1
        return item

    # ---- checkpointing
    def get_state(self) -> dict:
        return {"batches_consumed": self._consumed, "batch_size": self.batch_size, "seed": self.sampler.seed,
                "dp_index": self.sampler.dp_index, "dp_size": self.sampler.dp_size, "shuffle": self.sampler.shuffle}

    def set_state(self, state: dict) -> None:
        for k in ("batch_size", "seed", "dp_size", "shuffle"):
            if k in state and state[k] != self.get_state()[k]:
                raise ValueError(f"iterator state mismatch for '{k}': saved {state[k]}, current {self.get_state()[k]}")
        self._shutdown()
        self._consumed = int(state["batches_consumed"])

    def close(self):
        self._shutdown()

    def __del__(self):
        try:
            self._shutdown()
        except Exception:
            pass


def make_data_iterator(index_path, *, batch_size: int, collator: Callable[[list], Any] | None = None, shuffle: bool = True,
                       seed: int = 0, num_epochs: int | None = None, dp_index: int | None = None,
                       dp_size: int | None = None, prefetch: int = 2, read_threads: int = 4,
                       resolve_chunks: bool = True, read_options: ReadOptions | None = None,
                       multiprocessing_options: MultiprocessingOptions | None = None, batch_fn=None) -> DataIterator:
    """Stage 3.  ``batch_size`` is per data-parallel rank.  ``dp_index`` / ``dp_size`` default to
    this process's position in the active mesh (or its torch.distributed rank).  ``read_options`` /
    ``multiprocessing_options`` (``make_grain_read_options`` / ``make_grain_multiprocessing_options``)
    take precedence over ``prefetch`` / ``read_threads``; ``batch_fn`` is the reference's name for
    ``collator``."""
    collator = collator if batch_fn is None else batch_fn
    if collator is None:
        raise TypeError("make_data_iterator needs a collator (batch_fn)")
    if batch_size <= 0:
        raise ValueError("batch_size must be > 0")
    nworkers, wbuf, start = 0, 1, "fork"
    if read_options is not None:
        prefetch, read_threads = read_options.prefetch_buffer_size, read_options.num_threads
    if multiprocessing_options is not None:
        nworkers, wbuf = multiprocessing_options.num_workers, multiprocessing_options.per_worker_buffer_size
        start = multiprocessing_options.start_method
    from ..parallel import mesh as mesh_lib

    if dp_size is None:
        dp_size = mesh_lib.data_parallel_size()
    if dp_index is None:
        dp_index = mesh_lib.data_parallel_index()
    meta = load_metadata(index_path)
    src = open_source(index_path)
    if resolve_chunks and meta.get("kind") == "chunk_index":
        transform = ChunkResolver(meta["payload_path"])
    else:
        transform = _identity
    sampler = IndexSampler(len(src), shuffle=shuffle, seed=seed, num_epochs=num_epochs, dp_index=dp_index,
                           dp_size=dp_size)
    return DataIterator(src, sampler, transform, batch_size, collator, prefetch=prefetch, read_threads=read_threads,
                        num_workers=nworkers, worker_buffer=wbuf, start_method=start)


make_grain_iterator = make_data_iterator  # name used by the reference scripts

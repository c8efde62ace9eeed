"""Indexed record files (the on-disk container of compiled SFT datasets).

A C++ reader/writer (``csrc/recordio.cpp``, built to ``libomegalax_recordio.so`` next to this
file) memory-maps the file and gathers batches of records on a small thread pool; when the
library is not built, a pure-Python implementation of the same format is used.  Format:
magic, length+crc32 prefixed records, offset table, footer (count, table offset, magic).
"""
from __future__ import annotations

import ctypes
import mmap
import struct
import subprocess
import zlib
from pathlib import Path

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "libomegalax_recordio.so"
_MAGIC, _IDX_MAGIC = b"OLRF0001", b"OLRFIDX1"
_lib = None


def build_native(force: bool = False) -> Path | None:
    """Compile the C++ reader with g++ (a few seconds); returns the library path or None."""
    src = _HERE / "csrc" / "recordio.cpp"
    if _LIB_PATH.exists() and not force and _LIB_PATH.stat().st_mtime >= src.stat().st_mtime:
        return _LIB_PATH
    try:
        subprocess.run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-pthread", str(src), "-o", str(_LIB_PATH)],
                       check=True, capture_output=True)
    except Exception:
        return None
    return _LIB_PATH


def _native():
    global _lib
    if _lib is None:
        path = _LIB_PATH if _LIB_PATH.exists() else build_native()
        if path is None:
            _lib = False
        else:
            L = ctypes.CDLL(str(path))
            L.olrf_open.restype = ctypes.c_void_p
            L.olrf_open.argtypes = [ctypes.c_char_p]
            L.olrf_close.argtypes = [ctypes.c_void_p]
            L.olrf_num_records.restype = ctypes.c_longlong
            L.olrf_num_records.argtypes = [ctypes.c_void_p]
            L.olrf_record_len.restype = ctypes.c_longlong
            L.olrf_record_len.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
            L.olrf_read.restype = ctypes.c_longlong
            L.olrf_read.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int]
            L.olrf_read_many.restype = ctypes.c_longlong
            L.olrf_read_many.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                         ctypes.c_longlong, ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
            L.olrf_writer_open.restype = ctypes.c_void_p
            L.olrf_writer_open.argtypes = [ctypes.c_char_p]
            L.olrf_writer_append.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_longlong]
            L.olrf_writer_close.argtypes = [ctypes.c_void_p]
            _lib = L
    return _lib or None


class RecordWriter:
    def __init__(self, path, native: bool | None = None):
        self.path = str(path)
        L = _native() if native is not False else None
        self._L = L
        if L is not None:
            self._h = L.olrf_writer_open(self.path.encode())
            if not self._h:
                raise OSError(f"cannot open {self.path} for writing")
        else:
            self._f = open(self.path, "wb")
            self._f.write(_MAGIC)
            self._offsets = []
            self._pos = 8
        self.count = 0

    def write(self, data: bytes) -> None:
        if self._L is not None:
            if self._L.olrf_writer_append(self._h, data, len(data)) != 0:
                raise OSError("record append failed")
        else:
            self._offsets.append(self._pos)
            self._f.write(struct.pack("<II", len(data), zlib.crc32(data) & 0xFFFFFFFF))
            self._f.write(data)
            self._pos += 8 + len(data)
        self.count += 1

    def close(self) -> None:
        if self._L is not None:
            if self._h:
                self._L.olrf_writer_close(self._h)
                self._h = None
        elif self._f is not None:
            table = self._pos
            for o in self._offsets:
                self._f.write(struct.pack("<Q", o))
            self._f.write(struct.pack("<QQ", len(self._offsets), table))
            self._f.write(_IDX_MAGIC)
            self._f.close()
            self._f = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


class RecordReader:
    """Random access over one record file."""

    def __init__(self, path, native: bool | None = None, verify: bool = True):
        self.path = str(path)
        self.verify = verify
        self._native_arg = native
        self._open(native)

    def __getstate__(self):     # travels to another process as its path and is opened again there
        return {"path": self.path, "verify": self.verify, "native": self._native_arg}

    def __setstate__(self, st):
        self.path, self.verify, self._native_arg = st["path"], st["verify"], st["native"]
        self._open(self._native_arg)

    def _open(self, native):
        L = _native() if native is not False else None
        self._L = L
        if L is not None:
            self._h = L.olrf_open(self.path.encode())
            if not self._h:
                raise OSError(f"{self.path} is not a valid record file")
            self._n = int(L.olrf_num_records(self._h))
        else:
            self._f = open(self.path, "rb")
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
            if self._mm[:8] != _MAGIC or self._mm[-8:] != _IDX_MAGIC:
                raise OSError(f"{self.path} is not a valid record file")
            self._n, self._table = struct.unpack("<QQ", self._mm[-24:-8])

    def __len__(self) -> int:
        return self._n

    def __getitem__(self, i: int) -> bytes:
        if i < 0 or i >= self._n:
            raise IndexError(i)
        if self._L is not None:
            n = int(self._L.olrf_record_len(self._h, i))
            buf = ctypes.create_string_buffer(max(n, 1))
            rc = self._L.olrf_read(self._h, i, buf, n, int(self.verify))
            if rc == -3:
                raise OSError(f"checksum mismatch in {self.path} record {i}")
            if rc < 0:
                raise OSError(f"read failed ({rc}) in {self.path} record {i}")
            return buf.raw[:n]
        (off,) = struct.unpack("<Q", self._mm[self._table + 8 * i:self._table + 8 * i + 8])
        n, crc = struct.unpack("<II", self._mm[off:off + 8])
        data = bytes(self._mm[off + 8:off + 8 + n])
        if self.verify and (zlib.crc32(data) & 0xFFFFFFFF) != crc:
            raise OSError(f"checksum mismatch in {self.path} record {i}")
        return data

    def read_many(self, indices, threads: int = 4) -> list[bytes]:
        if self._L is None or len(indices) < 2:
            return [self[i] for i in indices]
        cnt = len(indices)
        idx = (ctypes.c_longlong * cnt)(*indices)
        total = sum(int(self._L.olrf_record_len(self._h, i)) for i in indices)
        buf = ctypes.create_string_buffer(max(total, 1))
        offs = (ctypes.c_longlong * (cnt + 1))()
        rc = self._L.olrf_read_many(self._h, idx, cnt, buf, total, offs, int(self.verify), threads)
        if rc < 0:
            raise OSError(f"batched read failed ({rc}) in {self.path}")
        raw = buf.raw
        return [raw[offs[k]:offs[k + 1]] for k in range(cnt)]

    def close(self) -> None:
        if self._L is not None:
            if self._h:
                self._L.olrf_close(self._h)
                self._h = None
        else:
            self._mm.close()
            self._f.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ShardedRecordSource:
    """Concatenation of several record files addressed by one global index."""

    def __init__(self, paths, native: bool | None = None):
        self.readers = [RecordReader(p, native=native) for p in paths]
        self.starts = [0]
        for r in self.readers:
            self.starts.append(self.starts[-1] + len(r))

    def __len__(self):
        return self.starts[-1]

    def __getitem__(self, i: int) -> bytes:
        import bisect

        if i < 0 or i >= len(self):
            raise IndexError(i)
        s = bisect.bisect_right(self.starts, i) - 1
        return self.readers[s][i - self.starts[s]]

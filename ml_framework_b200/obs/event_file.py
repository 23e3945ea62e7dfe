"""Binary event files: length-prefixed records with a checksum, an appending writer and a tolerant reader.

Reference: src/MLFramework.Visualization/Storage/{EventFileWriter.cs:30-121 (4-byte length prefix + serialised event,
write-through, append mode), EventFileReader.cs:25-170, FileStorageBackend.cs}. Record layout here (little endian):
``u32 length | u32 crc32(payload) | payload`` with the payload the event's JSON in UTF-8, after an 8-byte file magic.
The reader stops at the first truncated record (a writer that died mid-record loses only that record) and reports,
but skips, records whose checksum does not match.
"""
from __future__ import annotations

import os
import struct
import threading
import zlib
from typing import Iterator, List, Optional

from .events import Event, StorageBackend

MAGIC = b"MLFEVT1\n"
_HDR = struct.Struct("<II")
MAX_RECORD = 256 << 20


class EventFileError(RuntimeError):
    pass


class EventFileWriter:
    def __init__(self, path: str, append: bool = False):
        if not path:
            raise ValueError("path must not be empty")
        d = os.path.dirname(path)
        if d:
            os.makedirs(d, exist_ok=True)
        fresh = not (append and os.path.exists(path) and os.path.getsize(path) > 0)
        if not fresh:
            with open(path, "rb") as f:
                if f.read(len(MAGIC)) != MAGIC:
                    raise EventFileError(f"{path} is not an event file")
        self.path = path
        self._f = open(path, "ab" if not fresh else "wb")
        if fresh:
            self._f.write(MAGIC)
        self._lock = threading.Lock()
        self.records_written = 0
        self.bytes_written = 0

    def write_event(self, e: Event):
        payload = e.to_json().encode("utf-8")
        if len(payload) > MAX_RECORD:
            raise EventFileError(f"event of {len(payload)} bytes exceeds the record limit")
        rec = _HDR.pack(len(payload), zlib.crc32(payload)) + payload
        with self._lock:
            if self._f.closed:
                raise EventFileError("writer is closed")
            self._f.write(rec)
            self.records_written += 1
            self.bytes_written += len(rec)

    def write_events(self, events):
        for e in events:
            self.write_event(e)

    def flush(self, sync: bool = False):
        with self._lock:
            if not self._f.closed:
                self._f.flush()
                if sync:
                    os.fsync(self._f.fileno())

    def close(self):
        with self._lock:
            if not self._f.closed:
                self._f.flush()
                self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class EventFileReader:
    def __init__(self, path: str):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.path = path
        self.corrupt_records = 0
        self.truncated = False

    def __iter__(self) -> Iterator[Event]:
        return self.read_events()

    def read_events(self) -> Iterator[Event]:
        self.corrupt_records, self.truncated = 0, False
        with open(self.path, "rb") as f:
            if f.read(len(MAGIC)) != MAGIC:
                raise EventFileError(f"{self.path} is not an event file")
            while True:
                h = f.read(_HDR.size)
                if not h:
                    return
                if len(h) < _HDR.size:
                    self.truncated = True
                    return
                n, crc = _HDR.unpack(h)
                if n > MAX_RECORD:
                    self.truncated = True          # a damaged length: nothing after it can be trusted
                    return
                payload = f.read(n)
                if len(payload) < n:
                    self.truncated = True
                    return
                if zlib.crc32(payload) != crc:
                    self.corrupt_records += 1
                    continue
                try:
                    yield Event.from_json(payload.decode("utf-8"))
                except Exception:           # noqa: BLE001 - an undecodable record is counted, the rest is still read
                    self.corrupt_records += 1

    def read_all(self) -> List[Event]:
        return list(self.read_events())

    def count(self) -> int:
        return sum(1 for _ in self.read_events())


class BinaryFileStorageBackend(StorageBackend):
    """Storage back-end over one event file per process; rolls to a new file beyond ``max_file_bytes``."""

    def __init__(self, log_dir: str, prefix: str = "events", max_file_bytes: int = 256 << 20):
        os.makedirs(log_dir, exist_ok=True)
        self.log_dir, self.prefix, self.max_file_bytes = log_dir, prefix, max_file_bytes
        self._n = 0
        self._w: Optional[EventFileWriter] = None
        self.paths: List[str] = []
        self._roll()

    def _roll(self):
        if self._w is not None:
            self._w.close()
        p = os.path.join(self.log_dir, f"{self.prefix}.{os.getpid()}.{self._n:04d}.mlfevt")
        self._n += 1
        self._w = EventFileWriter(p)
        self.paths.append(p)

    def write(self, events):
        for e in events:
            if self._w.bytes_written >= self.max_file_bytes:
                self._roll()
            self._w.write_event(e)

    def flush(self):
        self._w.flush()

    def close(self):
        self._w.close()

    def read_all(self) -> List[Event]:
        self.flush()
        out: List[Event] = []
        for p in self.paths:
            out += EventFileReader(p).read_all()
        return out

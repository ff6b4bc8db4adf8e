"""On-disk formats either side of the decode path: safetensors payload + INSIDX01 index.

* A safetensors file is ``u64 header_len | JSON header | raw tensor bytes``; each
  header entry holds ``dtype``, ``shape`` and ``data_offsets`` relative to the
  end of the header (as read by the reference tools, tools/reference_all_layers.py:2-4).
* The Insignia index (reference writer: tools/index_safetensors.py:22-34, reader:
  src/model_file.cpp:13,22-36) is ``<8sIIQ>`` = magic ``INSIDX01``, version 1,
  tensor count, payload offset; then ``u32`` length + UTF-8 path of the payload;
  then per tensor, sorted by name, ``<HBBQQ>`` = name length, dtype code, rank,
  offset, bytes, followed by the name and ``rank`` u64 extents.

Host-only utilities (no GPU work).
"""
from __future__ import annotations

import json
import os
import struct
from typing import Iterable

import numpy as np

INDEX_MAGIC = b"INSIDX01"
# include/insignia_model.hpp:10 / tools/index_safetensors.py:8
DTYPE_CODES = {"F32": 1, "BF16": 2, "F16": 3, "U8": 4, "U32": 5, "I8": 6}
_NP = {"F32": np.float32, "BF16": np.uint16, "F16": np.float16, "U8": np.uint8, "U32": np.uint32, "I8": np.int8}


class SafetensorsWriter:
    """Streams tensors into a safetensors file without holding them all in memory.

    ``specs`` fixes names, dtypes and shapes up front (the header precedes the data);
    tensors are then appended in the same order with :meth:`write`.
    """

    def __init__(self, path: str, specs: Iterable[tuple[str, str, tuple[int, ...]]]):
        self.path = path
        header, off = {}, 0
        self._order = []
        for name, dtype, shape in specs:
            n = int(np.prod(shape, dtype=np.int64)) * np.dtype(_NP[dtype]).itemsize
            header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [off, off + n]}
            self._order.append((name, dtype, tuple(shape), n))
            off += n
        blob = json.dumps(header, separators=(",", ":")).encode()
        blob += b" " * ((8 - len(blob) % 8) % 8)
        self._f = open(path, "wb")
        self._f.write(struct.pack("<Q", len(blob)))
        self._f.write(blob)
        self._i = 0

    def write(self, name: str, array: np.ndarray) -> None:
        want, dtype, shape, n = self._order[self._i]
        if name != want:
            raise ValueError(f"expected tensor {want}, got {name}")
        a = np.ascontiguousarray(array, dtype=_NP[dtype])
        if a.nbytes != n:
            raise ValueError(f"{name}: {a.nbytes} bytes, header says {n}")
        self._f.write(memoryview(a).cast("B"))
        self._i += 1

    def close(self) -> None:
        if self._i != len(self._order):
            raise ValueError("not all tensors were written")
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        if exc[0] is None:
            self.close()
        else:
            self._f.close()


class SafetensorsReader:
    """mmap-backed reader; BF16 tensors come back as raw uint16 bit patterns."""

    def __init__(self, path: str):
        self.path = path
        with open(path, "rb") as f:
            (n,) = struct.unpack("<Q", f.read(8))
            self.header = json.loads(f.read(n))
        self.header.pop("__metadata__", None)
        self.data_start = 8 + n
        self._mm = np.memmap(path, dtype=np.uint8, mode="r")

    def names(self) -> list[str]:
        return sorted(self.header)

    def __contains__(self, name: str) -> bool:
        return name in self.header

    def get(self, name: str) -> np.ndarray:
        v = self.header[name]
        b, e = v["data_offsets"]
        raw = self._mm[self.data_start + b:self.data_start + e]
        return raw.view(_NP[v["dtype"]]).reshape(v["shape"])


def write_index(safetensors_path: str, index_path: str) -> int:
    """Writes the INSIDX01 index for a safetensors file; returns the tensor count."""
    with open(safetensors_path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
    tensors = sorted((k, v) for k, v in header.items() if k != "__metadata__")
    source = os.path.realpath(safetensors_path).encode("utf-8")
    with open(index_path, "wb") as out:
        out.write(struct.pack("<8sIIQ", INDEX_MAGIC, 1, len(tensors), 8 + n))
        out.write(struct.pack("<I", len(source)))
        out.write(source)
        for name, spec in tensors:
            raw = name.encode("utf-8")
            code = DTYPE_CODES.get(spec["dtype"])
            if code is None:
                raise ValueError(f"unsupported dtype {spec['dtype']} for {name}")
            b, e = spec["data_offsets"]
            out.write(struct.pack("<HBBQQ", len(raw), code, len(spec["shape"]), b, e - b))
            out.write(raw)
            out.write(struct.pack("<%dQ" % len(spec["shape"]), *spec["shape"]))
    return len(tensors)


def load_index(index_path: str) -> dict:
    blob = open(index_path, "rb").read()
    magic, version, count, payload = struct.unpack_from("<8sIIQ", blob, 0)
    if magic != INDEX_MAGIC or version != 1:
        raise ValueError("bad Insignia index")
    p = 24
    (path_n,) = struct.unpack_from("<I", blob, p)
    p += 4
    source = blob[p:p + path_n].decode("utf-8")
    p += path_n
    tensors = []
    for _ in range(count):
        name_n, dtype, rank, off, nbytes = struct.unpack_from("<HBBQQ", blob, p)
        p += 20
        name = blob[p:p + name_n].decode("utf-8")
        p += name_n
        shape = struct.unpack_from("<%dQ" % rank, blob, p)
        p += 8 * rank
        tensors.append({"name": name, "dtype": dtype, "shape": tuple(shape), "offset": off, "bytes": nbytes})
    return {"payload_offset": payload, "source": source, "tensors": tensors}

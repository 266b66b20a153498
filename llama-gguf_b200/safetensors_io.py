"""Reader of the safetensors container: 8 bytes little-endian header length, that many bytes of JSON (name -> dtype, shape,
data_offsets relative to the end of the header), then the raw tensor bytes.  The file is memory-mapped; tensors come out as numpy
views (BF16 / F16 as uint16 bit patterns, since numpy has no bfloat16) together with the ggml type id the library's upload takes."""
import json
import mmap
import struct

import numpy as np

F32, F16, BF16 = 0, 1, 30
_DTYPES = {"F32": (np.float32, F32), "F16": (np.uint16, F16), "BF16": (np.uint16, BF16), "I32": (np.int32, None),
           "I64": (np.int64, None)}


class SafetensorsFile:
    def __init__(self, path):
        self._f = open(path, "rb")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        if len(self._map) < 8:
            raise ValueError(f"{path}: not a safetensors file (shorter than its length field)")
        (n,) = struct.unpack("<Q", self._map[:8])
        if 8 + n > len(self._map):
            raise ValueError(f"{path}: header length {n} exceeds the file")
        self.header = json.loads(self._map[8:8 + n].decode("utf-8"))
        self.metadata = self.header.pop("__metadata__", {})
        self._base = 8 + n
        for name, e in self.header.items():
            if e["dtype"] not in _DTYPES:
                raise ValueError(f"{path}: tensor {name} has unsupported dtype {e['dtype']}")
            a, b = e["data_offsets"]
            count = int(np.prod(e["shape"], dtype=np.int64)) if e["shape"] else 1
            if b - a != count * np.dtype(_DTYPES[e["dtype"]][0]).itemsize or self._base + b > len(self._map):
                raise ValueError(f"{path}: tensor {name}: data_offsets do not fit its shape")

    def names(self):
        return list(self.header)

    def shape(self, name):
        return tuple(self.header[name]["shape"])

    def tensor(self, name):
        """(ggml type id or None for integer tables, shape, ndarray view of the mapped bytes)."""
        e = self.header[name]
        dt, gg = _DTYPES[e["dtype"]]
        a, b = e["data_offsets"]
        arr = np.frombuffer(self._map, dtype=dt, count=(b - a) // np.dtype(dt).itemsize, offset=self._base + a)
        return gg, tuple(e["shape"]), arr.reshape(e["shape"])

    def close(self):
        self._map = None
        self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        try:
            self.close()
        except BufferError:      # views of the mapping are still alive; the mapping goes with them
            pass


def bf16_bits(a):
    """float array -> bfloat16 bit patterns (round to nearest even), as uint16."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_to_f32(bits):
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def write_safetensors(path, tensors):
    """tensors: name -> ndarray (float32 -> F32, uint16 -> BF16 bit patterns, int32 -> I32).  For tests and synthetic models."""
    header, blobs, off = {}, [], 0
    for name, a in tensors.items():
        shape = list(np.shape(a))          # (a scalar keeps its empty shape: ascontiguousarray would make it [1])
        a = np.ascontiguousarray(a)
        dt = {"float32": "F32", "uint16": "BF16", "int32": "I32"}[a.dtype.name]
        raw = a.tobytes()
        header[name] = {"dtype": dt, "shape": shape, "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)

"""GGUF v3 files from Python: the reader and writer used to make and inspect model files.

Follows the layout tensomite reads and writes (src/tensomite/gguf.cr:26-66 kinds,
:156-191 writer, :297-325 parser): magic, version, tensor and key counts, typed
metadata, tensor infos with dimensions innermost first, then data aligned to
`general.alignment` (32).  Arrays of block formats are raw ggml bytes.
"""
import struct

import numpy as np

MAGIC = 0x46554747
F32, F16, Q4_0, Q4_1, Q8_0, BF16 = 0, 1, 2, 3, 8, 30
BLOCK_BYTES = {Q4_0: 18, Q4_1: 20, Q8_0: 34}
ALIGNMENT = 32


def bytes_for(kind, count):
    if kind == F32:
        return count * 4
    if kind in (F16, BF16):
        return count * 2
    return count // 32 * BLOCK_BYTES[kind]


def _string(s):
    b = s.encode()
    return struct.pack("<Q", len(b)) + b


def _value(v):
    if isinstance(v, bool):
        return struct.pack("<IB", 7, 1 if v else 0)
    if isinstance(v, int):
        return struct.pack("<II", 4, v) if 0 <= v < 2**32 else struct.pack("<Iq", 11, v)
    if isinstance(v, float):
        return struct.pack("<If", 6, v)
    if isinstance(v, str):
        return struct.pack("<I", 8) + _string(v)
    raise TypeError(type(v))


def write(path, metadata, tensors):
    """tensors: list of (name, kind, shape outermost-first, numpy array of raw bytes or float32)."""
    head = struct.pack("<IIQQ", MAGIC, 3, len(tensors), len(metadata))
    for key, value in metadata.items():
        head += _string(key) + _value(value)
    infos, offset = b"", 0
    offsets = []
    for name, kind, shape, data in tensors:
        size = bytes_for(kind, int(np.prod(shape, dtype=np.int64)))
        assert data.nbytes == size, (name, data.nbytes, size)
        infos += _string(name) + struct.pack("<I", len(shape))
        for dim in reversed(shape):
            infos += struct.pack("<Q", dim)
        infos += struct.pack("<IQ", kind, offset)
        offsets.append(offset)
        offset += (size + ALIGNMENT - 1) // ALIGNMENT * ALIGNMENT
    with open(path, "wb") as f:
        f.write(head + infos)
        pad = (-f.tell()) % ALIGNMENT
        f.write(b"\0" * pad)
        start = f.tell()
        for (name, kind, shape, data), off in zip(tensors, offsets):
            f.seek(start + off)
            f.write(np.ascontiguousarray(data).tobytes())
        end = start + offset
        f.seek(0, 2)
        if f.tell() < end:
            f.write(b"\0" * (end - f.tell()))


class File:
    """Parsed GGUF: `.metadata` dict and `.entries` name -> (kind, shape, absolute offset)."""

    def __init__(self, path):
        self.data = np.memmap(path, dtype=np.uint8, mode="r")
        self.pos = 0
        if self._u32() != MAGIC:
            raise ValueError(f"{path} is not a GGUF file")
        version = self._u32()
        if version not in (2, 3):
            raise ValueError(f"GGUF version {version} is not supported")
        tensors, keys = self._u64(), self._u64()
        self.metadata = {}
        for _ in range(keys):
            key = self._str()
            self.metadata[key] = self._val(self._u32())
        infos = []
        for _ in range(tensors):
            name = self._str()
            dims = [self._u64() for _ in range(self._u32())]
            infos.append((name, dims[::-1], self._u32(), self._u64()))
        alignment = self.metadata.get("general.alignment", 32)
        start = (self.pos + alignment - 1) // alignment * alignment
        self.entries = {name: (kind, shape, start + off) for name, shape, kind, off in infos}

    def _take(self, n):
        b = bytes(self.data[self.pos:self.pos + n])
        self.pos += n
        return b

    def _u32(self):
        return struct.unpack("<I", self._take(4))[0]

    def _u64(self):
        return struct.unpack("<Q", self._take(8))[0]

    def _str(self):
        return self._take(self._u64()).decode()

    def _val(self, t):
        fmt = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 10: "<Q", 11: "<q", 12: "<d"}
        if t in fmt:
            return struct.unpack(fmt[t], self._take(struct.calcsize(fmt[t])))[0]
        if t == 7:
            return self._take(1)[0] != 0
        if t == 8:
            return self._str()
        if t == 9:
            element = self._u32()
            return [self._val(element) for _ in range(self._u64())]
        raise ValueError(f"GGUF value type {t} is not known")

    def raw(self, name):
        kind, shape, offset = self.entries[name]
        size = bytes_for(kind, int(np.prod(shape, dtype=np.int64)))
        return kind, shape, np.array(self.data[offset:offset + size])

    def f32(self, name):
        """An F32/F16/BF16 tensor widened to float32 (gguf.cr:120-136)."""
        kind, shape, raw = self.raw(name)
        if kind == F32:
            return raw.view(np.float32).reshape(shape)
        if kind == F16:
            return raw.view(np.float16).astype(np.float32).reshape(shape)
        if kind == BF16:
            return (raw.view(np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(shape)
        raise TypeError(f"{name} is a block format")

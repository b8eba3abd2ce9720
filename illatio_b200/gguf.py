"""The GGUF container, as far as the device path needs it: header, metadata, tensor directory, and a tensor's raw
blocks from the file into device memory.

Mirrors src/gguf.lisp:10-157 (READ-GGUF, META, GGUF-TENSOR, TENSOR-BYTES, CALL-WITH-TENSOR-BYTES) and UPLOAD-GMAT
(src/cuda-dense.lisp:75-100).  All integers little-endian; versions 2 and 3.  The directory is read through the
file; tensor data stays on disk behind a memory map, and an upload streams it through a pinned staging buffer in
chunks, so a model is never held twice in host memory.  The matrices stay the file's raw blocks on the device: the
kernels multiply them as they lie (the reference's repack launches for Q8_0 and Q6_K have no counterpart here).
"""
import mmap
import os
import struct
from dataclasses import dataclass, field

import numpy as np

MAGIC = 0x46554747  # "GGUF"

# ggml tensor types: code -> (name, elements a block, bytes a block)
GGML_TYPES = {
    0: ("f32", 1, 4), 1: ("f16", 1, 2), 2: ("q4_0", 32, 18), 3: ("q4_1", 32, 20), 6: ("q5_0", 32, 22), 7: ("q5_1", 32, 24),
    8: ("q8_0", 32, 34), 9: ("q8_1", 32, 36), 10: ("q2_k", 256, 84), 11: ("q3_k", 256, 110), 12: ("q4_k", 256, 144),
    13: ("q5_k", 256, 176), 14: ("q6_k", 256, 210), 15: ("q8_k", 256, 292), 16: ("iq2_xxs", 256, 66), 17: ("iq2_xs", 256, 74),
    18: ("iq3_xxs", 256, 98), 19: ("iq1_s", 256, 50), 20: ("iq4_nl", 32, 18), 21: ("iq3_s", 256, 110), 22: ("iq2_s", 256, 82),
    23: ("iq4_xs", 256, 136), 24: ("i8", 1, 1), 25: ("i16", 1, 2), 26: ("i32", 1, 4), 27: ("i64", 1, 8), 28: ("f64", 1, 8),
    29: ("iq1_m", 256, 56), 30: ("bf16", 1, 2), 39: ("mxfp4", 32, 17),
}
TYPE_CODES = {name: code for code, (name, _, _) in GGML_TYPES.items()}

# metadata value types
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
_STRING, _ARRAY = 8, 9


class GgufError(ValueError):
    pass


@dataclass
class TensorInfo:
    name: str
    dims: tuple      # ggml order: (ne0, ne1, ...), ne0 the contiguous axis
    type: str        # ggml type name
    offset: int      # relative to the data section


@dataclass
class Gguf:
    path: str
    version: int = 0
    metadata: dict = field(default_factory=dict)
    tensors: dict = field(default_factory=dict)        # name -> TensorInfo
    tensor_order: list = field(default_factory=list)   # names in file order
    data_offset: int = 0
    alignment: int = 32

    def meta(self, key, default=None):
        """META (src/gguf.lisp:25-28)."""
        return self.metadata.get(key, default)

    def tensor(self, name, errorp=True):
        """GGUF-TENSOR (src/gguf.lisp:140-142)."""
        ti = self.tensors.get(name)
        if ti is None and errorp:
            raise GgufError("GGUF: no tensor named %r" % name)
        return ti


def type_layout(type_name):
    """(elements a block, bytes a block) of a ggml type name."""
    _, block, nbytes = GGML_TYPES[TYPE_CODES[type_name]]
    return block, nbytes


def tensor_elements(ti):
    n = 1
    for d in ti.dims:
        n *= d
    return n


def tensor_bytes(ti):
    """TENSOR-BYTES (src/gguf.lisp:53-56)."""
    block, nbytes = type_layout(ti.type)
    n = tensor_elements(ti)
    if n % block:
        raise GgufError("GGUF: tensor %s has %d elements, not a whole number of %s blocks" % (ti.name, n, ti.type))
    return n // block * nbytes


class _Reader:
    def __init__(self, f):
        self.f = f

    def take(self, n):
        b = self.f.read(n)
        if len(b) != n:
            raise GgufError("GGUF: the file ends inside its header")
        return b

    def scalar(self, fmt):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def string(self):
        n = self.scalar("<Q")
        if n > 1 << 24:
            raise GgufError("GGUF: a string of %d bytes in the header" % n)
        return self.take(n).decode("utf-8", errors="replace")

    def value(self, vtype):
        if vtype in _SCALARS:
            return self.scalar(_SCALARS[vtype])
        if vtype == _STRING:
            return self.string()
        if vtype == _ARRAY:
            etype, count = self.scalar("<I"), self.scalar("<Q")
            if etype in _SCALARS and etype != 7:
                fmt = _SCALARS[etype]
                return np.frombuffer(self.take(count * struct.calcsize(fmt)), dtype=np.dtype(fmt)).tolist()
            return [self.value(etype) for _ in range(count)]
        raise GgufError("GGUF: unknown metadata value type %d" % vtype)


def read_gguf(path):
    """READ-GGUF (src/gguf.lisp:105-138): the header, metadata and tensor directory of the file at PATH."""
    g = Gguf(path=os.fspath(path))
    with open(path, "rb") as f:
        r = _Reader(f)
        if r.scalar("<I") != MAGIC:
            raise GgufError("%s is not a GGUF file" % path)
        g.version = r.scalar("<I")
        if g.version not in (2, 3):
            raise GgufError("GGUF version %d is not supported (2 and 3 are)" % g.version)
        n_tensors, n_kv = r.scalar("<Q"), r.scalar("<Q")
        for _ in range(n_kv):
            key = r.string()
            g.metadata[key] = r.value(r.scalar("<I"))
        g.alignment = int(g.meta("general.alignment", 32))
        if g.alignment <= 0 or g.alignment & (g.alignment - 1):
            raise GgufError("GGUF: alignment %d is not a power of two" % g.alignment)
        for _ in range(n_tensors):
            name = r.string()
            nd = r.scalar("<I")
            if nd > 8:
                raise GgufError("GGUF: tensor %s has %d dimensions" % (name, nd))
            dims = tuple(r.scalar("<Q") for _ in range(nd))
            code = r.scalar("<I")
            if code not in GGML_TYPES:
                raise GgufError("GGUF: unknown ggml tensor type %d" % code)
            g.tensors[name] = TensorInfo(name, dims, GGML_TYPES[code][0], r.scalar("<Q"))
            g.tensor_order.append(name)
        pos = f.tell()
        g.data_offset = -(-pos // g.alignment) * g.alignment
    return g


def tensor_view(g, ti):
    """The raw bytes of tensor TI as a read-only numpy view of a memory map of the file."""
    total = tensor_bytes(ti)
    start = g.data_offset + ti.offset
    if start + total > os.path.getsize(g.path):
        raise GgufError("GGUF: truncated tensor %s" % ti.name)
    with open(g.path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
    return np.frombuffer(mm, dtype=np.uint8, count=total, offset=start)


def call_with_tensor_bytes(g, ti, fn, chunk=4 * 1024 * 1024):
    """CALL-WITH-TENSOR-BYTES (src/gguf.lisp:144-157): the tensor's raw bytes to FN in chunks, FN(buffer, start)."""
    v = tensor_view(g, ti)
    for pos in range(0, v.size, chunk):
        fn(v[pos:pos + chunk], pos)


# ---- writing (fixtures and tests; the reference only reads) ---------------------------------------------------
def _w_string(out, s):
    b = s.encode("utf-8")
    out += struct.pack("<Q", len(b)) + b


def _w_value(out, v):
    if isinstance(v, bool):
        out += struct.pack("<I?", 7, v)
    elif isinstance(v, int):
        out += struct.pack("<Iq", 11, v) if v < 0 else (struct.pack("<II", 4, v) if v < 1 << 32 else struct.pack("<IQ", 10, v))
    elif isinstance(v, float):
        out += struct.pack("<If", 6, v)
    elif isinstance(v, str):
        out += struct.pack("<I", _STRING)
        _w_string(out, v)
    elif isinstance(v, (list, tuple)):
        out += struct.pack("<I", _ARRAY)
        if v and all(isinstance(e, str) for e in v):
            out += struct.pack("<IQ", _STRING, len(v))
            for e in v:
                _w_string(out, e)
        elif all(isinstance(e, int) and not isinstance(e, bool) for e in v):
            out += struct.pack("<IQ", 5, len(v)) + np.asarray(v, dtype="<i4").tobytes()
        else:
            out += struct.pack("<IQ", 6, len(v)) + np.asarray(v, dtype="<f4").tobytes()
    else:
        raise TypeError("no GGUF value type for %r" % type(v))


def write_gguf(path, metadata, tensors, version=3, alignment=32):
    """A GGUF file of METADATA (a dict) and TENSORS (a list of (name, dims in ggml order, type name, bytes))."""
    out = bytearray(struct.pack("<IIQQ", MAGIC, version, len(tensors), len(metadata) + (1 if alignment != 32 else 0)))
    if alignment != 32:
        _w_string(out, "general.alignment")
        out += struct.pack("<II", 4, alignment)
    for k, v in metadata.items():
        _w_string(out, k)
        _w_value(out, v)
    offset, offsets = 0, []
    for name, dims, tname, data in tensors:
        offsets.append(offset)
        offset = -(-(offset + len(data)) // alignment) * alignment
    for (name, dims, tname, data), off in zip(tensors, offsets):
        _w_string(out, name)
        out += struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", TYPE_CODES[tname], off)
    out += b"\0" * (-len(out) % alignment)
    for (name, dims, tname, data), off in zip(tensors, offsets):
        out += bytes(data)
        out += b"\0" * (-len(data) % alignment)
    with open(path, "wb") as f:
        f.write(out)


# ---- file -> device -------------------------------------------------------------------------------------------
_QUANT = {"q8_0": 0, "q4_k": 1, "q6_k": 2, "q2_k": 3, "iq2_xxs": 4}   # the library's format codes
_DENSE = {"f32": "float32", "f16": "float16", "bf16": "bfloat16"}


def upload_tensor(g, name, device="cuda", chunk=32 * 1024 * 1024):
    """Tensor NAME's raw bytes from the file into a new uint8 device tensor, through a pinned staging buffer in
    chunks (two buffers alternate, so a chunk is read from the map while the one before is on its way)."""
    import torch
    ti = g.tensor(name)
    v = tensor_view(g, ti)
    dst = torch.empty(v.size, dtype=torch.uint8, device=device)
    stage = [torch.empty(min(chunk, max(v.size, 1)), dtype=torch.uint8).pin_memory() for _ in range(2)]
    done = [None, None]
    for i, pos in enumerate(range(0, v.size, chunk)):
        b = i & 1
        if done[b] is not None:
            done[b].synchronize()
        n = min(chunk, v.size - pos)
        stage[b][:n].numpy()[:] = v[pos:pos + n]
        dst[pos:pos + n].copy_(stage[b][:n], non_blocking=True)
        done[b] = torch.cuda.Event()
        done[b].record()
    torch.cuda.synchronize(device)
    return dst


def upload_gmat(g, name, device="cuda"):
    """UPLOAD-GMAT (src/cuda-dense.lisp:75-100) from the file: tensor NAME as a device matrix of raw blocks
    (cuda_dense.CMat: rows = ne1, cols = ne0) for the five quantized formats the kernels multiply; an unquantized
    F32 / F16 / BF16 tensor comes back as a torch tensor [ne1, ne0] (what DK-MV16 takes)."""
    import torch
    from . import cuda_dense as D
    ti = g.tensor(name)
    if len(ti.dims) != 2:
        raise GgufError("%s: %d dimensions, a matrix has two" % (name, len(ti.dims)))
    cols, rows = ti.dims
    if ti.type in _DENSE:
        raw = upload_tensor(g, name, device)
        return raw.view(getattr(torch, _DENSE[ti.type])).view(rows, cols)
    if ti.type not in _QUANT:
        raise GgufError("the device path multiplies Q8_0, Q4_K, Q6_K, Q2_K, IQ2_XXS and unquantized tensors; %s is %s" % (name, ti.type))
    block, _ = type_layout(ti.type)
    if cols % block:
        raise GgufError("%s: %d columns is not a whole number of blocks" % (name, cols))
    return D.CMat(name, _QUANT[ti.type], rows, cols, upload_tensor(g, name, device))

"""Import-only checkpoint decoders: GGUF (block dequantisation to f32) and torch pickle archives.

Reference: src/formats/gguf.rs, src/formats/pickle.rs, ``detect_format`` priority
safetensors > gguf > pickle (src/formats/mod.rs:44-95)."""
from __future__ import annotations

import io
import pickle
import struct
import zipfile
from pathlib import Path
from typing import Iterator

import numpy as np


def detect_format(path) -> tuple[str, list[Path]]:
    p = Path(path)
    if p.is_file():
        suf = p.suffix.lower()
        if suf == ".safetensors":
            return "safetensors", [p]
        if suf == ".gguf":
            return "gguf", [p]
        if suf in (".bin", ".pth", ".pt"):
            return "pickle", [p]
        raise ValueError(f"{p}: unknown checkpoint format")
    for fmt, pats in (("safetensors", ("*.safetensors",)), ("gguf", ("*.gguf",)), ("pickle", ("*.bin", "*.pth", "*.pt"))):
        files = sorted(f for pat in pats for f in p.glob(pat))
        if files:
            return fmt, files
    raise ValueError(f"{p}: no safetensors, gguf or pickle checkpoint found")


# --------------------------------------------------------------------------- GGUF
_GGUF_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}
# type id -> (block elements, block bytes)
_GGML = {0: (1, 4), 1: (1, 2), 2: (32, 18), 3: (32, 20), 6: (32, 22), 7: (32, 24), 8: (32, 34), 30: (1, 2)}


class _Rd:
    def __init__(self, buf):
        self.b, self.o = buf, 0

    def take(self, fmt):
        v = struct.unpack_from(fmt, self.b, self.o)
        self.o += struct.calcsize(fmt)
        return v[0]

    def string(self):
        n = self.take("<Q")
        s = bytes(self.b[self.o:self.o + n]).decode("utf-8", "replace")
        self.o += n
        return s

    def value(self, t):
        if t in _GGUF_SCALAR:
            return self.take(_GGUF_SCALAR[t])
        if t == 8:
            return self.string()
        if t == 9:
            et, n = self.take("<I"), self.take("<Q")
            return [self.value(et) for _ in range(n)]
        raise ValueError(f"gguf: unknown metadata type {t}")


def _dequant(t: int, raw: np.ndarray, n: int) -> np.ndarray:
    if t == 0:
        return raw.view(np.float32)[:n].copy()
    if t == 1:
        return raw.view(np.float16)[:n].astype(np.float32)
    if t == 30:
        return (raw.view(np.uint16)[:n].astype(np.uint32) << 16).view(np.float32)
    be, bb = _GGML[t]
    blk = raw.reshape(-1, bb)
    d = blk[:, 0:2].copy().view(np.float16).astype(np.float32)
    if t == 2:      # Q4_0
        qs = blk[:, 2:18]
        lo, hi = (qs & 0xF).astype(np.int8) - 8, (qs >> 4).astype(np.int8) - 8
        return (np.concatenate([lo, hi], axis=1).astype(np.float32) * d).reshape(-1)[:n]
    if t == 3:      # Q4_1
        m = blk[:, 2:4].copy().view(np.float16).astype(np.float32)
        qs = blk[:, 4:20]
        q = np.concatenate([qs & 0xF, qs >> 4], axis=1).astype(np.float32)
        return (q * d + m).reshape(-1)[:n]
    if t in (6, 7):  # Q5_0 / Q5_1
        o = 2 if t == 6 else 4
        qh = blk[:, o:o + 4].copy().view(np.uint32)
        qs = blk[:, o + 4:o + 20]
        bits = ((qh >> np.arange(32, dtype=np.uint32)[None, :]) & 1).astype(np.uint8)
        q = np.concatenate([qs & 0xF, qs >> 4], axis=1) | (bits << 4)
        if t == 6:
            return ((q.astype(np.float32) - 16.0) * d).reshape(-1)[:n]
        m = blk[:, 2:4].copy().view(np.float16).astype(np.float32)
        return (q.astype(np.float32) * d + m).reshape(-1)[:n]
    if t == 8:      # Q8_0
        return (blk[:, 2:34].view(np.int8).astype(np.float32) * d).reshape(-1)[:n]
    raise ValueError(f"gguf: tensor type {t} is not supported")


def read_gguf(path) -> tuple[dict, list[tuple[str, tuple, int, int]], np.ndarray, int]:
    buf = np.memmap(path, dtype=np.uint8, mode="r")
    r = _Rd(memoryview(buf))
    if bytes(buf[:4]) != b"GGUF":
        raise ValueError(f"{path}: not a GGUF file")
    r.o = 4
    version = r.take("<I")
    if version < 2:
        raise ValueError(f"{path}: GGUF version {version} is not supported")
    nt, nkv = r.take("<Q"), r.take("<Q")
    meta = {}
    for _ in range(nkv):
        k = r.string()
        meta[k] = r.value(r.take("<I"))
    infos = []
    for _ in range(nt):
        name = r.string()
        nd = r.take("<I")
        dims = [r.take("<Q") for _ in range(nd)]
        t, off = r.take("<I"), r.take("<Q")
        infos.append((name, tuple(reversed(dims)), t, off))
    align = int(meta.get("general.alignment", 32))
    base = (r.o + align - 1) // align * align
    return meta, infos, buf, base


def iter_gguf(path) -> Iterator[tuple[str, np.ndarray]]:
    _meta, infos, buf, base = read_gguf(path)
    for name, shape, t, off in infos:
        if t not in _GGML:
            raise ValueError(f"{path}: tensor {name!r} has unsupported ggml type {t}")
        n = int(np.prod(shape)) if shape else 1
        be, bb = _GGML[t]
        nbytes = (n + be - 1) // be * bb
        raw = np.asarray(buf[base + off:base + off + nbytes])
        yield name, _dequant(t, raw, n).reshape(shape)


# --------------------------------------------------------------------------- torch pickle
class _Storage:
    def __init__(self, dtype, key):
        self.dtype, self.key = dtype, key


_ST = {"FloatStorage": np.float32, "HalfStorage": np.float16, "DoubleStorage": np.float64,
       "BFloat16Storage": np.uint16, "LongStorage": np.int64, "IntStorage": np.int32, "ShortStorage": np.int16,
       "CharStorage": np.int8, "ByteStorage": np.uint8, "BoolStorage": np.bool_}


class _StorageType:
    def __init__(self, name):
        self.name = name


def _rebuild_tensor_v2(storage, offset, size, stride, *rest):
    return ("tensor", storage, offset, tuple(size), tuple(stride))


def _rebuild_parameter(data, *rest):
    return data


class _Unpickler(pickle.Unpickler):
    """Restricted unpickler: only the constructors a state_dict needs are allowed."""

    def find_class(self, module, name):
        if module == "torch._utils" and name == "_rebuild_tensor_v2":
            return _rebuild_tensor_v2
        if module == "torch._utils" and name in ("_rebuild_parameter", "_rebuild_parameter_with_state"):
            return _rebuild_parameter
        if module == "torch" and name in _ST:
            return _StorageType(name)
        if module == "collections" and name == "OrderedDict":
            import collections
            return collections.OrderedDict
        if module == "torch" and name == "Size":
            return tuple
        raise pickle.UnpicklingError(f"refusing to load {module}.{name} from a checkpoint pickle")

    def persistent_load(self, pid):
        # ('storage', storage_type, key, location, numel)
        if not (isinstance(pid, tuple) and pid[0] == "storage"):
            raise pickle.UnpicklingError("unknown persistent id")
        return _Storage(pid[1].name, pid[2])


def iter_pickle(path) -> Iterator[tuple[str, np.ndarray]]:
    with zipfile.ZipFile(path) as z:
        names = z.namelist()
        pkl = [n for n in names if n.endswith("data.pkl")]
        if len(pkl) != 1:
            raise ValueError(f"{path}: expected one data.pkl, found {len(pkl)}")
        prefix = pkl[0][:-len("data.pkl")]
        obj = _Unpickler(io.BytesIO(z.read(pkl[0]))).load()
        if isinstance(obj, dict) and "state_dict" in obj and isinstance(obj["state_dict"], dict):
            obj = obj["state_dict"]
        if not isinstance(obj, dict):
            raise ValueError(f"{path}: top-level pickle object is not a state dict")
        cache: dict[str, np.ndarray] = {}
        for name, t in obj.items():
            if not (isinstance(t, tuple) and t and t[0] == "tensor"):
                continue
            _, st, off, size, stride = t
            dt = _ST[st.dtype]
            if st.key not in cache:
                cache[st.key] = np.frombuffer(z.read(f"{prefix}data/{st.key}"), dtype=dt)
            flat = cache[st.key]
            a = np.lib.stride_tricks.as_strided(flat[off:], shape=size, strides=[s * flat.itemsize for s in stride]) \
                if size else flat[off:off + 1].reshape(())
            if dt == np.uint16:
                a = (np.ascontiguousarray(a).astype(np.uint32) << 16).view(np.float32)
            elif dt in (np.float16, np.float64):
                a = a.astype(np.float32)
            elif dt != np.float32:
                continue  # non-float tensors are skipped (src/ingest.rs:101-109)
            yield str(name), np.ascontiguousarray(a)

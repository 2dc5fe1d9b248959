"""Reader for torch ``.pt`` files that hold tensors in plain containers, without executing the pickle.

Reference: src/models/personaplex/voice_prompt.rs:44-360.  A ``torch.save`` file is an UNCOMPRESSED zip: ``<stem>/data.pkl`` plus one
``<stem>/data/<key>`` blob per storage, little-endian.  The pickle builds its tensors through
``torch._utils._rebuild_tensor_v2(persistent_id(("storage", <Type>Storage, key, device, numel)), offset, shape, strides, ...)``.
The stack machine below interprets exactly that surface (dicts, lists, tuples, strings, numbers, ``OrderedDict()``, tensor
rebuilds) and refuses every other callable or opcode by name: a voice file from an untrusted source can therefore construct
nothing but tensors and containers.  The device string inside the pickle (stock voices say ``cuda:0``) is ignored: storages are
read into host memory."""
from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np
import torch


def zip_entries(data) -> dict[str, memoryview]:
    """Entry name -> payload of a zip whose entries are all STORED (voice_prompt.rs:44-89)."""
    data = memoryview(data).cast("B")
    raw = bytes(data[-(1 << 16) - 22:])
    k = raw.rfind(b"PK\x05\x06")
    if k < 0:
        raise ValueError("zip: no end-of-central-directory record")
    eocd = len(data) - len(raw) + k
    n_entries, = struct.unpack_from("<H", data, eocd + 10)
    cd, = struct.unpack_from("<I", data, eocd + 16)
    if n_entries == 0xFFFF or cd == 0xFFFFFFFF:
        raise ValueError("zip: zip64 archives are not supported")
    out = {}
    for _ in range(n_entries):
        if bytes(data[cd:cd + 4]) != b"PK\x01\x02":
            raise ValueError("zip: bad central directory header")
        method, = struct.unpack_from("<H", data, cd + 10)
        csize, usize = struct.unpack_from("<II", data, cd + 20)
        name_len, extra_len, comment_len = struct.unpack_from("<HHH", data, cd + 28)
        lho, = struct.unpack_from("<I", data, cd + 42)
        name = bytes(data[cd + 46:cd + 46 + name_len]).decode("utf-8")
        if method != 0 or csize != usize:
            raise ValueError(f"zip: {name}: only STORED entries (what torch.save writes) are supported")
        if bytes(data[lho:lho + 4]) != b"PK\x03\x04":
            raise ValueError("zip: bad local header")
        lname, lextra = struct.unpack_from("<HH", data, lho + 26)
        start = lho + 30 + lname + lextra
        if start + usize > len(data):
            raise ValueError(f"zip: {name}: payload runs past the end of the file")
        out[name] = data[start:start + usize]
        cd += 46 + name_len + extra_len + comment_len
    return out


@dataclass
class TensorStub:
    storage_key: str
    storage_type: str
    numel: int
    offset: int = 0
    shape: tuple = ()
    strides: tuple = ()


class _Global(str):
    pass


_MARK = object()
_DTYPES = {"FloatStorage": torch.float32, "BFloat16Storage": torch.bfloat16, "HalfStorage": torch.float16, "DoubleStorage": torch.float64,
           "LongStorage": torch.int64, "IntStorage": torch.int32, "ShortStorage": torch.int16, "CharStorage": torch.int8,
           "ByteStorage": torch.uint8, "BoolStorage": torch.bool}


def unpickle(b) -> object:
    """Interpret the opcode surface of a tensor-container pickle (protocols 2 to 4); tensors come back as :class:`TensorStub`."""
    b = bytes(b)
    stack, memo, i = [], {}, 0

    def pop_to_mark():
        items = []
        while True:
            if not stack:
                raise ValueError("pickle: MARK not found")
            v = stack.pop()
            if v is _MARK:
                return items[::-1]
            items.append(v)
    while True:
        if i >= len(b):
            raise ValueError("pickle: ran off the end without STOP")
        op = b[i:i + 1]
        i += 1
        if op == b"\x80":                                   # PROTO
            i += 1
        elif op == b"\x95":                                 # FRAME
            i += 8
        elif op == b"}":
            stack.append({})
        elif op == b"]":
            stack.append([])
        elif op == b")":
            stack.append(())
        elif op == b"(":
            stack.append(_MARK)
        elif op == b"N":
            stack.append(None)
        elif op == b"\x88":
            stack.append(True)
        elif op == b"\x89":
            stack.append(False)
        elif op == b"K":
            stack.append(b[i]); i += 1
        elif op == b"M":
            stack.append(struct.unpack_from("<H", b, i)[0]); i += 2
        elif op == b"J":
            stack.append(struct.unpack_from("<i", b, i)[0]); i += 4
        elif op == b"\x8a":                                 # LONG1
            n = b[i]; i += 1
            stack.append(int.from_bytes(b[i:i + n], "little", signed=True)); i += n
        elif op == b"G":
            stack.append(struct.unpack_from(">d", b, i)[0]); i += 8
        elif op == b"X":
            n, = struct.unpack_from("<I", b, i); i += 4
            stack.append(b[i:i + n].decode("utf-8")); i += n
        elif op == b"\x8c":
            n = b[i]; i += 1
            stack.append(b[i:i + n].decode("utf-8")); i += n
        elif op == b"c":
            e1 = b.index(b"\n", i)
            e2 = b.index(b"\n", e1 + 1)
            stack.append(_Global(b[i:e1].decode() + " " + b[e1 + 1:e2].decode()))
            i = e2 + 1
        elif op == b"\x93":
            name, module = stack.pop(), stack.pop()
            stack.append(_Global(f"{module} {name}"))
        elif op == b"q":
            memo[b[i]] = stack[-1]; i += 1
        elif op == b"r":
            memo[struct.unpack_from("<I", b, i)[0]] = stack[-1]; i += 4
        elif op == b"\x94":
            memo[len(memo)] = stack[-1]
        elif op == b"h":
            stack.append(memo[b[i]]); i += 1
        elif op == b"j":
            stack.append(memo[struct.unpack_from("<I", b, i)[0]]); i += 4
        elif op == b"t":
            stack.append(tuple(pop_to_mark()))
        elif op in (b"\x85", b"\x86", b"\x87"):
            n = op[0] - 0x84
            items = stack[-n:]
            del stack[-n:]
            stack.append(tuple(items))
        elif op == b"a":
            v = stack.pop()
            stack[-1].append(v)
        elif op == b"e":
            items = pop_to_mark()
            stack[-1].extend(items)
        elif op == b"s":
            v, k = stack.pop(), stack.pop()
            stack[-1][k] = v
        elif op == b"u":
            kv = pop_to_mark()
            stack[-1].update(zip(kv[0::2], kv[1::2]))
        elif op == b"Q":                                    # BINPERSID
            pid = stack.pop()
            if not (isinstance(pid, tuple) and len(pid) >= 5 and pid[0] == "storage" and isinstance(pid[1], _Global)
                    and pid[1].startswith("torch ")):
                raise ValueError(f"pickle: unsupported persistent id {pid!r}")
            stack.append(TensorStub(str(pid[2]), pid[1][len("torch "):], int(pid[4])))
        elif op == b"R":
            args, fn = stack.pop(), stack.pop()
            if fn == "torch._utils _rebuild_tensor_v2":
                st = args[0]
                if not isinstance(st, TensorStub):
                    raise ValueError("pickle: _rebuild_tensor_v2 without a storage")
                stack.append(TensorStub(st.storage_key, st.storage_type, st.numel, int(args[1]), tuple(int(x) for x in args[2]),
                                        tuple(int(x) for x in args[3])))
            elif fn == "collections OrderedDict" and args == ():
                stack.append({})
            else:
                raise ValueError(f"pickle: refusing to call {fn!r}")
        elif op == b".":
            return stack.pop()
        else:
            raise ValueError(f"pickle: unsupported opcode {op!r} at byte {i - 1}")


def _materialise(obj, entries, prefix):
    if isinstance(obj, TensorStub):
        dt = _DTYPES.get(obj.storage_type)
        if dt is None:
            raise ValueError(f"unsupported storage type {obj.storage_type}")
        raw = entries.get(f"{prefix}data/{obj.storage_key}")
        if raw is None:
            raise ValueError(f"storage {obj.storage_key} is missing from the archive")
        item = torch.empty((), dtype=dt).element_size()
        if len(raw) < obj.numel * item:
            raise ValueError(f"storage {obj.storage_key}: {len(raw)} bytes for {obj.numel} elements of {item} bytes")
        span = obj.offset + (sum((d - 1) * s for d, s in zip(obj.shape, obj.strides)) + 1 if all(obj.shape) else 0)
        if span > obj.numel or any(s < 0 for s in obj.strides):
            raise ValueError(f"tensor view runs past its storage ({span} > {obj.numel})")
        flat = torch.frombuffer(bytearray(raw[:obj.numel * item]), dtype=dt) if obj.numel else torch.empty(0, dtype=dt)
        return torch.as_strided(flat, obj.shape, obj.strides, obj.offset).clone()
    if isinstance(obj, dict):
        return {k: _materialise(v, entries, prefix) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_materialise(v, entries, prefix) for v in obj)
    return obj


def load_pt(src):
    """``src``: a path or the file's bytes.  Returns the saved object with every tensor materialised on the host."""
    if isinstance(src, (bytes, bytearray, memoryview)):
        data = src
    else:
        data = np.fromfile(src, dtype=np.uint8).data
    entries = zip_entries(data)
    pkl = [n for n in entries if n.endswith("/data.pkl") or n == "data.pkl"]
    if len(pkl) != 1:
        raise ValueError(f"expected one data.pkl in the archive, found {len(pkl)}")
    prefix = pkl[0][:-len("data.pkl")]
    order = entries.get(prefix + "byteorder")
    if order is not None and bytes(order[:6]) != b"little":
        raise ValueError("big-endian save")
    return _materialise(unpickle(entries[pkl[0]]), entries, prefix)

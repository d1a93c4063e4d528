"""A small flatbuffer writer for tests: builds TFLite files without the flatbuffers package.

Objects: ``Tab([field, ...])`` (a table; None = field absent), scalars as ``("b"|"i"|"I"|"f"|..., value)`` struct codes,
``Vec(dtype, values)`` (vector of scalars), ``Vec("tables", [Tab, ...])``, ``str`` (string). Parents are written before
their children (offsets point forward)."""
import struct

import numpy as np


class Tab:
    def __init__(self, fields):
        self.fields = fields


class Vec:
    def __init__(self, kind, values):
        self.kind, self.values = kind, values


def _align(buf: bytearray, n: int):
    while len(buf) % n:
        buf.append(0)


def build(root: Tab, ident: bytes = b"TFL3") -> bytes:
    buf = bytearray(8)
    buf[4:8] = ident
    patches = []          # (position of a uoffset, object)

    def emit(obj) -> int:
        """Writes obj, returns its position."""
        if isinstance(obj, Tab):
            # inline layout: soffset to the vtable, then the present fields
            sizes = []
            for f in obj.fields:
                if f is None:
                    sizes.append(0)
                elif isinstance(f, tuple):
                    sizes.append(struct.calcsize("<" + f[0]))
                else:
                    sizes.append(4)
            # vtable first (anywhere before or after; it is found through a signed offset)
            _align(buf, 2)
            vt_pos = len(buf)
            offs, cur = [], 4
            for sz in sizes:
                if sz == 0:
                    offs.append(0)
                    continue
                cur = (cur + sz - 1) // sz * sz
                offs.append(cur)
                cur += sz
            table_size = (cur + 3) // 4 * 4
            buf.extend(struct.pack("<HH", 4 + 2 * len(sizes), table_size))
            for o in offs:
                buf.extend(struct.pack("<H", o))
            _align(buf, 8)
            pos = len(buf)
            buf.extend(bytes(table_size))
            struct.pack_into("<i", buf, pos, pos - vt_pos)
            for f, o in zip(obj.fields, offs):
                if f is None:
                    continue
                if isinstance(f, tuple):
                    struct.pack_into("<" + f[0], buf, pos + o, f[1])
                else:
                    patches.append((pos + o, f))
            return pos
        if isinstance(obj, str):
            data = obj.encode()
            _align(buf, 4)
            pos = len(buf)
            buf.extend(struct.pack("<I", len(data)) + data + b"\0")
            return pos
        if isinstance(obj, Vec):
            if obj.kind == "tables":
                _align(buf, 4)
                pos = len(buf)
                buf.extend(struct.pack("<I", len(obj.values)))
                for i, t in enumerate(obj.values):
                    patches.append((pos + 4 + 4 * i, t))
                    buf.extend(bytes(4))
                return pos
            arr = np.ascontiguousarray(np.asarray(obj.values, dtype=obj.kind))
            # the length word sits right before the (aligned) data
            while (len(buf) + 4) % max(arr.dtype.itemsize, 4 if arr.dtype.itemsize < 8 else 8, 16 if obj.kind == np.uint8 else 1):
                buf.append(0)
            pos = len(buf)
            buf.extend(struct.pack("<I", arr.size) + arr.tobytes())
            return pos
        raise TypeError(type(obj))

    root_pos = emit(root)
    struct.pack_into("<I", buf, 0, root_pos)
    while patches:
        at, obj = patches.pop(0)
        pos = emit(obj)
        struct.pack_into("<I", buf, at, pos - at)
    return bytes(buf)

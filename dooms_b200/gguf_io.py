"""GGUF files from Python: a small writer (version 3) for synthetic models, and a reader that goes through the library's own C++ reader."""
from __future__ import annotations

import ctypes as C
import struct
from pathlib import Path

import numpy as np

from . import _lib as L

_T_U32, _T_I32, _T_F32, _T_BOOL, _T_STRING, _T_ARRAY, _T_U64 = 4, 5, 6, 7, 8, 9, 10


def _s(text: str) -> bytes:
    b = text.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _kv(key: str, value) -> bytes:
    out = _s(key)
    if isinstance(value, bool):
        return out + struct.pack("<iB", _T_BOOL, int(value))
    if isinstance(value, int):
        return out + struct.pack("<iI", _T_U32, value)
    if isinstance(value, float):
        return out + struct.pack("<if", _T_F32, value)
    if isinstance(value, str):
        return out + struct.pack("<i", _T_STRING) + _s(value)
    if isinstance(value, (list, tuple)) and all(isinstance(v, int) for v in value):
        return out + struct.pack("<iiQ", _T_ARRAY, _T_I32, len(value)) + b"".join(struct.pack("<i", v) for v in value)
    if isinstance(value, (list, tuple)) and value and all(isinstance(v, float) for v in value):
        return out + struct.pack("<iiQ", _T_ARRAY, _T_F32, len(value)) + b"".join(struct.pack("<f", v) for v in value)
    if isinstance(value, (list, tuple)) and all(isinstance(v, str) for v in value):
        return out + struct.pack("<iiQ", _T_ARRAY, _T_STRING, len(value)) + b"".join(_s(v) for v in value)
    raise TypeError(f"metadata value of type {type(value)}")


class GgufWriter:
    """write(path, metadata, tensors): tensors is a list of (name, dtype, shape_row_major, producer) where producer() returns the tensor's bytes as a
    contiguous uint8 numpy array (called once, in order, so that large models stream through memory one tensor at a time)."""

    def __init__(self, alignment: int = 32):
        self.alignment = alignment

    def write(self, path: str | Path, metadata: dict, tensors: list) -> None:
        al = self.alignment
        head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(metadata) + 1)
        head += _kv("general.alignment", al)
        for k, v in metadata.items():
            head += _kv(k, v)
        infos, offset = b"", 0
        sizes = []
        for name, dtype, shape, _ in tensors:
            n = int(np.prod(shape))
            nbytes = n // L.BLOCK_ELEMS[dtype] * L.BLOCK_BYTES[dtype]
            infos += _s(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<q", d) for d in reversed(shape))
            infos += struct.pack("<iQ", L.GGML_TYPE_ID[dtype], offset)
            sizes.append(nbytes)
            offset += (nbytes + al - 1) // al * al
        with open(path, "wb") as f:
            f.write(head + infos)
            f.write(b"\0" * ((-f.tell()) % al))
            for (name, dtype, shape, producer), nbytes in zip(tensors, sizes):
                data = producer()
                data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
                if data.size != nbytes:
                    raise ValueError(f"tensor {name}: producer gave {data.size} bytes, expected {nbytes}")
                f.write(memoryview(data))
                f.write(b"\0" * ((-nbytes) % al))


class GgufFile:
    """The library's reader (GgufFile of the C++ side) behind dooms_gguf_*."""

    def __init__(self, path: str | None = None, data: bytes | None = None):
        self._h = C.c_void_p()
        self._keep = None
        lib = L.lib()
        if path is not None:
            L.check(lib.dooms_gguf_open(str(path).encode(), C.byref(self._h)))
        else:
            self._keep = C.create_string_buffer(data, len(data)) if data else None
            L.check(lib.dooms_gguf_parse(self._keep, len(data) if data else 0, C.byref(self._h)))

    def close(self):
        if self._h:
            L.lib().dooms_gguf_close(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def version(self) -> int:
        return L.lib().dooms_gguf_version(self._h)

    @property
    def alignment(self) -> int:
        return L.lib().dooms_gguf_alignment(self._h)

    def _tensor(self, t: L.GgufTensor) -> dict:
        return {"name": t.name.decode(), "dtype": t.dtype, "shape": [t.shape[i] for i in range(t.rank)], "offset": t.offset, "nbytes": t.nbytes, "data": t.data}

    def tensors(self) -> list[dict]:
        lib = L.lib()
        out = []
        for i in range(lib.dooms_gguf_tensor_count(self._h)):
            t = L.GgufTensor()
            L.check(lib.dooms_gguf_tensor_at(self._h, i, C.byref(t)))
            out.append(self._tensor(t))
        return out

    def find_tensor(self, name: str) -> dict:
        t = L.GgufTensor()
        L.check(L.lib().dooms_gguf_find_tensor(self._h, name.encode(), C.byref(t)))
        return self._tensor(t)

    def tensor_bytes(self, name: str) -> np.ndarray:
        t = self.find_tensor(name)
        return np.ctypeslib.as_array(C.cast(t["data"], C.POINTER(C.c_uint8)), shape=(t["nbytes"],)).copy()

    def get_string(self, key: str) -> str:
        v = C.c_char_p()
        L.check(L.lib().dooms_gguf_get_string(self._h, key.encode(), C.byref(v)))
        return v.value.decode()

    def get_uint(self, key: str) -> int:
        v = C.c_uint64()
        L.check(L.lib().dooms_gguf_get_uint(self._h, key.encode(), C.byref(v)))
        return v.value

    def get_int(self, key: str) -> int:
        v = C.c_int64()
        L.check(L.lib().dooms_gguf_get_int(self._h, key.encode(), C.byref(v)))
        return v.value

    def get_float(self, key: str) -> float:
        v = C.c_double()
        L.check(L.lib().dooms_gguf_get_float(self._h, key.encode(), C.byref(v)))
        return v.value

    def get_bool(self, key: str) -> bool:
        v = C.c_int32()
        L.check(L.lib().dooms_gguf_get_bool(self._h, key.encode(), C.byref(v)))
        return bool(v.value)

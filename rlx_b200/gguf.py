"""GGUF container access over include/rlxq_gguf.h: the counterpart of rlx_gguf::GgufFile for this path
(open, tensor table, scalar metadata, raw tensor bytes) plus file -> device upload."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from ._lib import check, lib


class _Tensor(C.Structure):
    _fields_ = [("ggml_type", C.c_uint32), ("scheme", C.c_int32), ("n_dims", C.c_uint32),
                ("dims", C.c_uint64 * 4), ("offset", C.c_uint64), ("bytes", C.c_uint64)]


@dataclass(frozen=True)
class GgufTensor:
    name: str
    shape: tuple          # GGML order, innermost first, verbatim (a weight W[n, k] reads (k, n))
    ggml_type: int
    scheme: int           # rlxq scheme id, or -1
    offset: int
    nbytes: int


class GgufFile:
    """GgufFile::from_path (rlx-gguf/src/lib.rs:205-209); only the header is read at open."""

    def __init__(self, path: str):
        h = C.c_void_p()
        check(lib.rlxq_gguf_open(str(path).encode(), C.byref(h)))
        self._h = h.value
        self.version = int(lib.rlxq_gguf_version(self._h))
        self.alignment = int(lib.rlxq_gguf_alignment(self._h))
        self.data_start = int(lib.rlxq_gguf_data_start(self._h))
        self.tensors: dict[str, GgufTensor] = {}
        for i in range(int(lib.rlxq_gguf_tensor_count(self._h))):
            nm = C.c_char_p()
            check(lib.rlxq_gguf_tensor_name(self._h, i, C.byref(nm)))
            t = _Tensor()
            check(lib.rlxq_gguf_find(self._h, nm.value, C.byref(t)))
            name = nm.value.decode()
            self.tensors[name] = GgufTensor(name, tuple(int(t.dims[d]) for d in range(t.n_dims)), int(t.ggml_type),
                                            int(t.scheme), int(t.offset), int(t.bytes))

    def close(self) -> None:
        h, self._h = getattr(self, "_h", None), None
        if h:
            lib.rlxq_gguf_close(h)

    __del__ = close

    def keys(self):
        return self.tensors.keys()

    def get(self, name: str):
        return self.tensors.get(name)

    def meta_u64(self, key: str) -> int:
        v = C.c_uint64()
        check(lib.rlxq_gguf_meta_u64(self._h, key.encode(), C.byref(v)))
        return v.value

    def meta_str(self, key: str) -> str:
        v = C.c_char_p()
        check(lib.rlxq_gguf_meta_str(self._h, key.encode(), C.byref(v)))
        return v.value.decode()

    def tensor_bytes(self, name: str) -> np.ndarray:
        """GgufFile::tensor_bytes (rlx-gguf/src/lib.rs:355-371) as a uint8 array."""
        t = self.tensors.get(name)
        n = t.nbytes if t else 0
        out = np.empty(n, np.uint8)
        check(lib.rlxq_gguf_read_tensor(self._h, name.encode(), out.ctypes.data, n))
        return out

    def upload(self, name: str, device=None):
        """File -> pinned staging -> device; returns a CUDA uint8 tensor holding the tensor's raw bytes."""
        import torch
        t = self.tensors.get(name)
        n = t.nbytes if t else 0
        dst = torch.empty(max(n, 1), dtype=torch.uint8, device=device or "cuda")[:n]
        with torch.cuda.device(dst.device):
            check(lib.rlxq_gguf_upload_tensor(self._h, name.encode(), dst.data_ptr(), n,
                                              torch.cuda.current_stream().cuda_stream))
        return dst

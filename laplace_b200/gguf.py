"""GGUF file -> HBM (laplace_cuda_gguf_*): the file's tensors in the on-disk block format, each GPU holding its
rows of a matrix and its experts of a stacked expert tensor. Mirrors what Laplace's GGUFContext::open
(src/gguf.cpp:217-335) and matmul_register_weights (src/matmul.h:26) do for a single host."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

from . import _lib


@dataclass
class GgufTensor:
    name: str
    type: int
    dims: tuple            # innermost first, as in the file
    kind: int              # 0 whole tensor, 1 rows split, 2 experts split
    rows: tuple            # [begin, end) of this rank
    experts: tuple         # [begin, end) of this rank
    file_offset: int
    nbytes: int
    host: int              # address of the part inside the mapping
    dev: int               # address of the part in HBM (0 before upload)

    def as_torch(self):
        """The part in HBM as a uint8 torch tensor (a view; valid until the file is closed)."""
        import torch
        from .shard import _DevMem
        if not self.dev:
            raise RuntimeError(f"{self.name}: not uploaded")
        return torch.as_tensor(_DevMem(self.dev, (self.nbytes,), "|u1"), device="cuda")


class GgufFile:
    def __init__(self, path: str, rank: int = 0, world: int = 1, replicate=()):
        self.L = _lib.load()
        keep = (C.c_char_p * max(1, len(replicate)))(*[s.encode() for s in replicate])
        h = C.c_void_p()
        rc = self.L.laplace_cuda_gguf_open(str(path).encode(), rank, world, keep, len(replicate), C.byref(h))
        if rc:
            raise RuntimeError(f"laplace_cuda_gguf_open: {self.L.laplace_cuda_last_error().decode()}")
        self.h = h

    def upload(self) -> None:
        rc = self.L.laplace_cuda_gguf_upload(self.h)
        if rc:
            raise RuntimeError(f"laplace_cuda_gguf_upload: {self.L.laplace_cuda_last_error().decode()}")

    def __len__(self) -> int:
        return self.L.laplace_cuda_gguf_tensor_count(self.h)

    def _info(self, index, name):
        info = _lib.GgufTensorInfo()
        rc = self.L.laplace_cuda_gguf_tensor(self.h, index, name.encode() if name is not None else None, C.byref(info))
        if rc == 1:
            return None
        if rc:
            raise RuntimeError(self.L.laplace_cuda_last_error().decode())
        return GgufTensor(info.name.decode(), info.type, tuple(info.dims[: max(1, info.n_dims)]), info.kind,
                          (info.row_begin, info.row_end), (info.expert_begin, info.expert_end), info.file_offset,
                          info.bytes, info.host or 0, info.dev or 0)

    def tensor(self, name: str):
        return self._info(0, name)

    def tensors(self):
        return [self._info(i, None) for i in range(len(self))]

    def meta_int(self, key: str):
        v = C.c_ulonglong()
        return v.value if self.L.laplace_cuda_gguf_meta_u64(self.h, key.encode(), C.byref(v)) == 0 else None

    def meta_float(self, key: str):
        v = C.c_double()
        return v.value if self.L.laplace_cuda_gguf_meta_f64(self.h, key.encode(), C.byref(v)) == 0 else None

    def meta_str(self, key: str):
        s = self.L.laplace_cuda_gguf_meta_str(self.h, key.encode())
        return s.decode() if s is not None else None

    def close(self) -> None:
        if self.h:
            self.L.laplace_cuda_gguf_close(self.h)
            self.h = None

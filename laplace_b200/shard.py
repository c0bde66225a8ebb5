"""Tensor-parallel split of a weight matrix along N and the one exchange step that follows it.

The reference is single-device; the split follows from its row loop (src/matmul_simd.cpp:438-448: every
output column is an independent dot product over one contiguous row of rb bytes). Each rank keeps rows
[begin, end) of every matrix (on 16-row boundaries, laplace_cuda_nsplit), computes y[:, begin:end] and the
slices are all-gathered. This module holds the host logic only; it never computes a matmul.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist


class RowShards:
    """Row ranges of an N-row matrix over `world` ranks and the gather of per-rank output slices."""

    def __init__(self, lib, N: int, rank: int, world: int):
        self.N, self.rank, self.world = int(N), int(rank), int(world)
        self.ranges = []
        for r in range(self.world):
            b, e = C.c_int(), C.c_int()
            lib.laplace_cuda_nsplit(self.N, r, self.world, C.byref(b), C.byref(e))
            self.ranges.append((b.value, e.value))
        self.begin, self.end = self.ranges[self.rank]
        self.n_loc = self.end - self.begin
        self.n_max = max(e - b for b, e in self.ranges)
        self.even = all(e - b == self.n_max for b, e in self.ranges)
        self._send = None
        self._recv = None

    def slice_rows(self, w_rows):
        """This rank's rows of a [N, rb] byte matrix (a contiguous byte range of the packed file)."""
        return w_rows[self.begin:self.end]

    def gather(self, y_loc: torch.Tensor, y_full: torch.Tensor, group=None) -> torch.Tensor:
        """All-gathers y_loc [M, n_loc] of every rank into y_full [M, N]. One collective per call.

        M == 1 with equal slices gathers straight into y_full (slices are contiguous there); otherwise
        through a padded [world, M * n_max] buffer followed by one strided copy per rank."""
        M = y_loc.shape[0]
        if y_loc.shape != (M, self.n_loc) or y_full.shape != (M, self.N):
            raise ValueError(f"gather: y_loc {tuple(y_loc.shape)} / y_full {tuple(y_full.shape)} do not match "
                             f"M={M}, n_loc={self.n_loc}, N={self.N}")
        if self.world == 1:
            y_full.copy_(y_loc)
            return y_full
        if M == 1 and self.even and y_full.is_contiguous() and y_loc.is_contiguous():
            dist.all_gather_into_tensor(y_full.view(-1), y_loc.view(-1), group=group)
            return y_full
        if self.even and y_loc.is_contiguous() and y_full.is_contiguous():
            # equal slices: gather [G, M, n_loc] and interleave the ranks' columns with one strided copy
            need = M * self.n_max
            if self._recv is None or self._recv.numel() != self.world * need or self._recv.device != y_loc.device:
                self._recv = torch.empty(self.world * need, dtype=y_loc.dtype, device=y_loc.device)
            dist.all_gather_into_tensor(self._recv, y_loc.view(-1), group=group)
            y_full.view(M, self.world, self.n_max).copy_(self._recv.view(self.world, M, self.n_max).permute(1, 0, 2))
            return y_full
        need = M * self.n_max
        if self._send is None or self._send.numel() != need or self._send.device != y_loc.device:
            self._send = torch.zeros(need, dtype=y_loc.dtype, device=y_loc.device)
            self._recv = torch.empty(self.world * need, dtype=y_loc.dtype, device=y_loc.device)
        self._send[: M * self.n_loc].view(M, self.n_loc).copy_(y_loc)
        dist.all_gather_into_tensor(self._recv, self._send, group=group)
        for r, (b, e) in enumerate(self.ranges):
            if e > b:
                y_full[:, b:e].copy_(self._recv[r * need: r * need + M * (e - b)].view(M, e - b))
        return y_full


class _DevMem:
    """A raw device allocation exposed to torch through the CUDA array interface."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 2}


class PeerGather:
    """The fused all-gather of a row-split decode matmul (laplace_cuda_gemm_allgather_dev): every rank's GEMV
    stores its slice into every rank's result buffer over NVLink and raises a step flag; `wait` makes the
    stream wait for all slices. One buffer per rank, shared with the other processes by CUDA IPC handles that
    travel over the process group (host plumbing only; no collective runs in a step)."""

    def __init__(self, lib, shards: RowShards, M: int, group=None):
        self.L, self.sh, self.M, self.group = lib, shards, int(M), group
        world, rank, N = shards.world, shards.rank, shards.N
        self.y_bytes = (4 * self.M * N * 4 + 255) & ~255      # four result slots
        self.total = self.y_bytes + 512                       # + flags[world] (256 B) + step / done counters (256 B)
        ptr = C.c_void_p()
        handle = (C.c_ubyte * 64)()
        self._check(lib.laplace_cuda_peer_alloc(self.total, C.byref(ptr), handle))
        self.own = ptr.value
        handles = [None] * world
        if world > 1:
            dist.all_gather_object(handles, bytes(handle), group=group)
        self.bases, self._opened = [], []
        for r in range(world):
            if r == rank:
                self.bases.append(self.own)
                continue
            q = C.c_void_p()
            hb = (C.c_ubyte * 64).from_buffer_copy(handles[r])
            self._check(lib.laplace_cuda_peer_open(hb, C.byref(q)))
            self.bases.append(q.value)
            self._opened.append(q.value)
        self.peer_y = (C.c_void_p * world)(*self.bases)
        self.peer_flags = (C.c_void_p * world)(*[b + self.y_bytes for b in self.bases])
        self.flags = self.own + self.y_bytes
        self.step_ctr = self.own + self.y_bytes + 256
        self.done_ctr = self.step_ctr + 4
        self.steps = 0
        if world > 1:
            dist.barrier(group=group)                         # every rank has mapped every buffer

    def _check(self, rc):
        if rc:
            raise RuntimeError(f"laplace_cuda error {rc}: {self.L.laplace_cuda_last_error().decode()}")

    def gemm(self, x: torch.Tensor, w: torch.Tensor, t: int, K: int, stream: int) -> None:
        """Enqueues this rank's slice of y = W x; results land in slot (step & 3) of every rank's buffer."""
        sh = self.sh
        self._check(self.L.laplace_cuda_gemm_allgather_dev(x.data_ptr(), w.data_ptr(), int(t), self.peer_y, self.peer_flags,
                                                          self.step_ctr, self.done_ctr, sh.rank, sh.world, sh.begin, sh.N,
                                                          self.M, K, sh.n_loc, stream))
        self.steps += 1

    def wait(self, stream: int) -> None:
        """Closes a chain of steps: announces this rank's slices of the current step and enqueues the
        (bounded) wait for all ranks' slices."""
        self._check(self.L.laplace_cuda_allgather_wait_dev(self.peer_flags, self.step_ctr, self.sh.rank, self.sh.world, stream))

    def gemm_peers(self, x: torch.Tensor, w: torch.Tensor, t: int, K: int, stream: int) -> bool:
        """Prefill (M > 8): this rank's slice of y = W x goes to slot 0 of every rank's buffer from the GEMM's own drain
        (laplace_cuda_gemm_peers_dev). False when the tensor-core kernels do not take the shape (nothing was enqueued).
        Must be followed by step_wait before the buffers are read or written again."""
        sh = self.sh
        rc = self.L.laplace_cuda_gemm_peers_dev(x.data_ptr(), w.data_ptr(), int(t), self.peer_y, sh.world, sh.begin, sh.N,
                                                self.M, K, sh.n_loc, stream)
        if rc == 1:
            return False
        self._check(rc)
        return True

    def step_wait(self, stream: int) -> None:
        """Advances this rank's step, announces it to every rank and enqueues the (bounded) wait for all ranks' slices."""
        self._check(self.L.laplace_cuda_allgather_step_wait_dev(self.peer_flags, self.step_ctr, self.sh.rank, self.sh.world, stream))

    def slot(self, which: int) -> torch.Tensor:
        """Slot `which & 3` of this rank's result buffer as a [M, N] tensor; step s (counted from 1) lands in slot s & 3."""
        mem = _DevMem(self.own + (which & 3) * self.M * self.sh.N * 4, (self.M, self.sh.N), "<f4")
        return torch.as_tensor(mem, device="cuda")

    def close(self) -> None:
        torch.cuda.synchronize()
        if self.sh.world > 1:
            dist.barrier(group=self.group)                    # nobody stores into a buffer that is being unmapped
        for q in self._opened:
            self.L.laplace_cuda_peer_close(q)
        self._opened = []
        if self.sh.world > 1:
            dist.barrier(group=self.group)
        if self.own:
            self.L.laplace_cuda_peer_free(self.own)
            self.own = 0

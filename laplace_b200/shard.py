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

"""Mixture-of-experts FFN matmuls with experts placed across GPUs.

What the reference does per token on one device (src/arch_gemma4.cpp:600-638): gate/up matmul over the token's
top-k experts (fused_moe_gemm_idx), the gated activation, down matmul with one input per expert
(fused_moe_gemm_multi), and a weighted sum of the k results. Here a batch of tokens goes through the two
expert-grouped matmuls of include/laplace_cuda.h; with more than one GPU, expert e lives on GPU e // (E / G):

    1. exchange in:  every GPU gets the tokens and the routing table of all GPUs (all-gather: at top-8 over 8 GPUs
                     two thirds of all (token, GPU) combinations are needed anyway, so this moves 1.5x the bytes of
                     a deduplicated all-to-all, needs no host round trip for split sizes and can be captured in a
                     CUDA graph);
    2. local work:   the grouped matmuls run over the full pair list with the pairs of other GPUs' experts
                     marked -1 (skipped on the device), then the weighted sum over the local experts of each token;
    3. exchange out: reduce-scatter of the per-token partial sums back to the tokens' owners.

A second exchange, `exchange="alltoall"`, is the token all-to-all proper: a token is sent ONCE to every GPU that
holds at least one of its experts (not once per expert), the partial sums come back the same way and are added in
rank order. Split sizes are data dependent, so this form synchronises with the host once per layer (the counts)
and cannot be captured in a CUDA graph; it moves fewer bytes and is the cross-check of the all-gather form.

The compute is injected: `fused_ffn` (one call of laplace_cuda_moe_ffn_dev: both matmuls, the activation and the
weighted sum) or `grouped_matmul` (two calls of laplace_cuda_moe_grouped_dev with torch glue between them), so the
exchange logic runs on CPU tensors under gloo in the tests.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist


def silu_mul(gu: torch.Tensor, inter: int) -> torch.Tensor:
    """The gated activation between the two matmuls: silu(gate) * up on a [P, 2*inter] gate/up result."""
    g, u = gu[:, :inter], gu[:, inter:]
    return (g * torch.sigmoid(g) * u).contiguous()


class ExpertParallelMoE:
    """One MoE layer's expert matmuls. `w_gate_up`: this rank's experts stacked, [E_loc * 2*inter rows];
    `w_down`: [E_loc * hidden rows]. `grouped_matmul(x, w, pair_expert, pair_row, E_loc, K, N, y)` computes
    y[p] = W[pair_expert[p]] . x[pair_row[p]] for pair_expert[p] >= 0 and leaves the other rows of y alone."""

    def __init__(self, w_gate_up, w_down, n_experts: int, top_k: int, hidden: int, inter: int,
                 grouped_matmul: Optional[Callable] = None, rank: int = 0, world: int = 1, group=None,
                 fused_ffn: Optional[Callable] = None, device_exchange: bool = False, exchange: str = "allgather"):
        if n_experts % world:
            raise ValueError(f"{n_experts} experts do not split evenly over {world} GPUs")
        if grouped_matmul is None and fused_ffn is None:
            raise ValueError("give grouped_matmul or fused_ffn")
        self.w_gate_up, self.w_down = w_gate_up, w_down
        self.E, self.k, self.H, self.I = n_experts, top_k, hidden, inter
        self.rank, self.world, self.group = rank, world, group
        self.E_loc = n_experts // world
        self.mm, self.ffn = grouped_matmul, fused_ffn
        self.device_exchange = device_exchange        # pack / unpack with the library's kernels instead of torch ops
        if exchange not in ("allgather", "alltoall"):
            raise ValueError("exchange is 'allgather' or 'alltoall'")
        self.exchange = exchange
        self.last_dispatch_rows = None                # rows this rank sent in the last all-to-all dispatch
        self._buf = {}
        self._rows_ready = None

    def _buffer(self, name, shape, dtype, device, zero=False):
        key = (name, tuple(shape), dtype, str(device))
        b = self._buf.get(key)
        if b is None:
            b = (torch.zeros if zero else torch.empty)(shape, dtype=dtype, device=device)
            self._buf[key] = b
        return b

    def _exchange_in(self, x, top_idx, top_w):
        """One all-gather of [x | expert ids (bit pattern) | weights] per token."""
        T_loc, dev = x.shape[0], x.device
        G, k, H = self.world, self.k, self.H
        if G == 1:
            return x.contiguous(), top_idx.contiguous(), top_w.contiguous()
        send = self._buffer("send", (T_loc, H + 2 * k), torch.float32, dev)
        recv = self._buffer("recv", (T_loc * G, H + 2 * k), torch.float32, dev)
        send[:, :H].copy_(x)
        send[:, H:H + k].copy_(top_idx.contiguous().view(torch.float32))
        send[:, H + k:].copy_(top_w)
        dist.all_gather_into_tensor(recv, send, group=self.group)
        return recv[:, :H].contiguous(), recv[:, H:H + k].contiguous().view(torch.int32), recv[:, H + k:].contiguous()

    def _forward_alltoall(self, x, top_idx, top_w):
        """Token all-to-all: rows [x | expert ids | weights] go once to every GPU that owns one of the token's
        experts; every GPU runs the expert FFN over what it received (other GPUs' experts marked -1) and returns one
        partial sum per received row; the owner adds the partial sums of a token in rank order."""
        T_loc, dev = x.shape[0], x.device
        G, k, H, I = self.world, self.k, self.H, self.I
        owner = torch.div(top_idx, self.E_loc, rounding_mode="floor")                            # [T_loc, k] GPU of each expert
        needs = (owner.unsqueeze(2) == torch.arange(G, device=dev).view(1, 1, G)).any(dim=1)      # [T_loc, G]
        send_counts = needs.sum(dim=0).to(torch.int64)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()                                       # the one host synchronisation
        self.last_dispatch_rows = int(sum(sc))
        # rows ordered by destination GPU, tokens in order inside a destination
        dest, tok = needs.t().nonzero(as_tuple=True)                                              # sorted by destination, then token
        row = torch.cat([x, top_idx.contiguous().view(torch.float32), top_w], dim=1)             # [T_loc, H + 2k]
        send = row.index_select(0, tok).contiguous()
        recv = torch.empty((int(sum(rc)), H + 2 * k), dtype=torch.float32, device=dev)
        dist.all_to_all_single(recv, send, output_split_sizes=rc, input_split_sizes=sc, group=self.group)
        R = recv.shape[0]
        first = self.rank * self.E_loc
        if R:
            xr = recv[:, :H].contiguous()
            idr = recv[:, H:H + k].contiguous().view(torch.int32)
            wr = recv[:, H + k:].contiguous()
            mine = (idr >= first) & (idr < first + self.E_loc)
            idx_local = torch.where(mine, idr - first, torch.full_like(idr, -1)).to(torch.int32).contiguous()
            if self.ffn is not None:
                part = self.ffn(xr, self.w_gate_up, self.w_down, idx_local, wr, self.E_loc, H, I,
                                torch.empty((R, H), dtype=torch.float32, device=dev))
            else:
                pair_expert = idx_local.reshape(-1)
                pair_row = torch.arange(R, dtype=torch.int32, device=dev).repeat_interleave(k)
                gu = torch.zeros((R * k, 2 * I), dtype=torch.float32, device=dev)
                dn = torch.zeros((R * k, H), dtype=torch.float32, device=dev)
                self.mm(xr, self.w_gate_up, pair_expert, pair_row, self.E_loc, H, 2 * I, gu)
                self.mm(silu_mul(gu, I), self.w_down, pair_expert, None, self.E_loc, I, H, dn)
                wt = (wr * mine.to(wr.dtype)).reshape(R, k, 1)
                live = torch.where(mine.reshape(R, k, 1), dn.reshape(R, k, H), torch.zeros((), dtype=dn.dtype, device=dev))
                part = (live * wt).sum(dim=1)
        else:
            part = torch.empty((0, H), dtype=torch.float32, device=dev)
        back = torch.empty((int(sum(sc)), H), dtype=torch.float32, device=dev)
        dist.all_to_all_single(back, part.contiguous(), output_split_sizes=sc, input_split_sizes=rc, group=self.group)
        # one partial sum per (token, GPU that served it), grouped by GPU: add them in rank order (reproducible)
        out = torch.zeros((T_loc, H), dtype=torch.float32, device=dev)
        start = 0
        for g in range(G):
            n = sc[g]
            if n:
                out.index_add_(0, tok[start:start + n], back[start:start + n])                   # a token appears once per GPU
            start += n
        return out

    def forward(self, x: torch.Tensor, top_idx: torch.Tensor, top_w: torch.Tensor) -> torch.Tensor:
        """x [T_loc, H] fp32, top_idx [T_loc, k] int32 (global expert ids), top_w [T_loc, k] fp32.
        Returns the layer's output for this rank's tokens, [T_loc, H]."""
        if self.exchange == "alltoall" and self.world > 1:
            return self._forward_alltoall(x, top_idx, top_w)
        T_loc, dev = x.shape[0], x.device
        G, k, H, I = self.world, self.k, self.H, self.I
        T = T_loc * G
        first = self.rank * self.E_loc
        if self.device_exchange and self.ffn is not None and G > 1:
            # one pack kernel, one all-gather, one unpack kernel (which also makes the expert ids local)
            from . import device
            send = self._buffer("send", (T_loc, H + 2 * k), torch.float32, dev)
            recv = self._buffer("recv", (T, H + 2 * k), torch.float32, dev)
            x_all = self._buffer("x_all", (T, H), torch.float32, dev)
            idx_local = self._buffer("idx_local", (T, k), torch.int32, dev)
            w_all = self._buffer("w_all", (T, k), torch.float32, dev)
            device.moe_pack(x.contiguous(), top_idx.contiguous(), top_w.contiguous(), send)
            dist.all_gather_into_tensor(recv, send, group=self.group)
            device.moe_unpack(recv, H, k, first, self.E_loc, x_all, idx_local, w_all)
            partial = self.ffn(x_all, self.w_gate_up, self.w_down, idx_local, w_all, self.E_loc, H, I,
                               self._buffer("partial", (T, H), torch.float32, dev))
            out = self._buffer("out", (T_loc, H), torch.float32, dev)
            dist.reduce_scatter_tensor(out, partial, group=self.group)
            return out
        x_all, idx_all, w_all = self._exchange_in(x, top_idx, top_w)
        # pairs of this rank's experts keep a local expert id, the others become -1
        mine = (idx_all >= first) & (idx_all < first + self.E_loc)
        idx_local = torch.where(mine, idx_all - first, torch.full_like(idx_all, -1)).to(torch.int32).contiguous()
        if self.ffn is not None:
            partial = self.ffn(x_all, self.w_gate_up, self.w_down, idx_local, w_all, self.E_loc, H, I,
                               self._buffer("partial", (T, H), torch.float32, dev))
        else:
            pair_expert = idx_local.reshape(-1)
            pair_row = self._buffer("pair_row", (T * k,), torch.int32, dev)
            if self._rows_ready != (T, k):
                pair_row.copy_(torch.arange(T, dtype=torch.int32, device=dev).repeat_interleave(k))
                self._rows_ready = (T, k)
            gu = self._buffer("gu", (T * k, 2 * I), torch.float32, dev, zero=True)
            dn = self._buffer("dn", (T * k, H), torch.float32, dev, zero=True)
            self.mm(x_all, self.w_gate_up, pair_expert, pair_row, self.E_loc, H, 2 * I, gu)
            h = silu_mul(gu, I)
            self.mm(h, self.w_down, pair_expert, None, self.E_loc, I, H, dn)
            # weighted sum over this rank's experts (rows of other ranks' pairs are never written and weigh 0)
            wt = (w_all * mine.to(w_all.dtype)).reshape(T, k, 1)
            live = torch.where(mine.reshape(T, k, 1), dn.reshape(T, k, H), torch.zeros((), dtype=dn.dtype, device=dev))
            partial = (live * wt).sum(dim=1)
        if G > 1:
            out = self._buffer("out", (T_loc, H), torch.float32, dev)
            dist.reduce_scatter_tensor(out, partial.contiguous(), group=self.group)
            return out
        return partial


def device_fused_ffn(type_gate_up: int, type_down: int, activation: int = 0) -> Callable:
    """The fused expert FFN on the GPU (laplace_cuda_moe_ffn_dev) in the signature ExpertParallelMoE expects."""
    from . import device

    def ffn(x, w_gate_up, w_down, idx_local, top_w, n_experts, hidden, inter, out):
        return device.moe_ffn(x, w_gate_up, w_down, type_gate_up, type_down, idx_local, top_w, n_experts, hidden, inter,
                              activation=activation, out=out)
    return ffn


def device_grouped_matmul(ggml_type: int) -> Callable:
    """The grouped matmul on the GPU (laplace_cuda_moe_grouped_dev) in the signature ExpertParallelMoE expects."""
    from . import device

    def mm(x, w, pair_expert, pair_row, n_experts, K, N, y):
        return device.moe_grouped(x, w, ggml_type, pair_expert, pair_row, n_experts, K, N, y=y)
    return mm


def seeded_routing(seed: int, T: int, E: int, top_k: int):
    """Router stand-in: logits ~ N(0,1) from a seed, top-k experts per token, softmax over the selected logits."""
    import numpy as np
    logits = np.random.Generator(np.random.Philox(seed)).standard_normal((T, E), dtype=np.float32)
    idx = np.argsort(-logits, axis=1)[:, :top_k].astype(np.int32)
    sel = np.take_along_axis(logits, idx, axis=1)
    ex = np.exp(sel - sel.max(axis=1, keepdims=True))
    return idx, (ex / ex.sum(axis=1, keepdims=True)).astype(np.float32)

"""Device-pointer calls into the C ABI with torch tensors as the memory owners.

torch is plumbing here: it allocates HBM, owns streams and (for multi-GPU runs)
the NCCL process group. Every function passes raw device pointers and the
current CUDA stream to the ``*_dev`` entry points of include/laplace_cuda.h.
"""
from __future__ import annotations

import numpy as np
import torch

from . import _lib
from .ggml import any_row_bytes, blocksums_per_row, row_bytes
from .matmul import LaplaceCudaError, _check

_ready_on = None


def lib(device: int | None = None):
    """Loads the library and binds it to ``device`` (default: torch's current device)."""
    global _ready_on
    L = _lib.load()
    if not torch.cuda.is_available():
        raise LaplaceCudaError(-3, "no CUDA device visible to this process; the library has no CPU path")
    dev = torch.cuda.current_device() if device is None else device
    if _ready_on is None:
        _check(L, L.laplace_cuda_init(dev))
        _ready_on = dev
        from . import matmul as _m
        _m._initialised = True
    elif _ready_on != dev:
        raise LaplaceCudaError(-3, f"library already bound to device {_ready_on}")
    return L


def _stream() -> int:
    """torch's current stream as a handle for the ABI. torch's default stream has handle 0, which the ABI
    reads as "the library's own stream", so it is passed as cudaStreamLegacy (0x1) instead."""
    h = torch.cuda.current_stream().cuda_stream
    return h if h else 1


def upload_weights(w: np.ndarray) -> torch.Tensor:
    """Copies GGUF bytes to HBM with the 16-byte read-ahead slack the kernels may touch."""
    flat = np.ascontiguousarray(w, dtype=np.uint8).reshape(-1)
    t = torch.zeros(flat.size + 64, dtype=torch.uint8, device="cuda")
    t[: flat.size].copy_(torch.from_numpy(flat))
    return t


def gemm(x: torch.Tensor, w: torch.Tensor, t: int, M: int, K: int, N: int, y: torch.Tensor | None = None) -> torch.Tensor:
    L = lib()
    assert x.dtype == torch.float32 and x.is_cuda and x.is_contiguous() and x.numel() >= M * K
    assert w.dtype == torch.uint8 and w.is_cuda and w.numel() >= N * any_row_bytes(t, K)
    if y is None:
        y = torch.empty((M, N), dtype=torch.float32, device=x.device)
    _check(L, L.laplace_cuda_gemm_dev(x.data_ptr(), w.data_ptr(), int(t), y.data_ptr(), M, K, N, _stream()))
    return y


def gemm_multi(x: torch.Tensor, ws, t: int, M: int, K: int, Ns, norm_weight: torch.Tensor | None = None, eps: float = 0.0,
               want_x_norm: bool = False):
    """Several matrices of one type against the same (optionally RMS-normalised) activation rows in one launch
    (laplace_cuda_gemm_multi_dev). Returns the list of outputs, and the normalised rows when asked for."""
    L = lib()
    assert x.dtype == torch.float32 and x.is_cuda and x.is_contiguous() and len(ws) == len(Ns)
    ys = [torch.empty((M, n), dtype=torch.float32, device=x.device) for n in Ns]
    mats = (_lib.Matrix * len(ws))(*[_lib.Matrix(w.data_ptr(), y.data_ptr(), int(n)) for w, y, n in zip(ws, ys, Ns)])
    xn = torch.empty((M, K), dtype=torch.float32, device=x.device) if want_x_norm else None
    _check(L, L.laplace_cuda_gemm_multi_dev(x.data_ptr(), norm_weight.data_ptr() if norm_weight is not None else None, float(eps),
                                            xn.data_ptr() if xn is not None else None, mats, len(ws), int(t), M, K, _stream()))
    return (ys, xn) if want_x_norm else ys


def moe_gemv(x: torch.Tensor, w: torch.Tensor, t: int, expert_idx: torch.Tensor, K: int, N: int,
             per_expert_x: bool, y: torch.Tensor | None = None) -> torch.Tensor:
    L = lib()
    n = expert_idx.numel()
    assert expert_idx.dtype == torch.int32 and expert_idx.is_cuda
    if y is None:
        y = torch.empty((n, N), dtype=torch.float32, device=x.device)
    _check(L, L.laplace_cuda_moe_gemv_dev(x.data_ptr(), w.data_ptr(), int(t), expert_idx.data_ptr(), n,
                                          y.data_ptr(), K, N, 1 if per_expert_x else 0, _stream()))
    return y


def moe_grouped(x: torch.Tensor, w: torch.Tensor, t: int, pair_expert: torch.Tensor, pair_row: torch.Tensor | None,
                n_experts_total: int, K: int, N: int, y: torch.Tensor | None = None) -> torch.Tensor:
    """y[p] = W[pair_expert[p]] . x[pair_row[p]] for every (token, expert) pair of a batch, grouped by expert on
    the device (what one fused_moe_gemm_idx / fused_moe_gemm_multi call per token computes, src/matmul.h:36-54).
    Types the grouped kernel does not take run as one expert-indexed GEMV launch per pair group of the same row."""
    L = lib()
    P = pair_expert.numel()
    assert pair_expert.dtype == torch.int32 and pair_expert.is_cuda and pair_expert.is_contiguous()
    assert pair_row is None or (pair_row.dtype == torch.int32 and pair_row.is_cuda and pair_row.numel() == P)
    assert x.dtype == torch.float32 and x.is_cuda and x.is_contiguous()
    if y is None:
        y = torch.empty((P, N), dtype=torch.float32, device=x.device)
    rc = L.laplace_cuda_moe_grouped_dev(x.data_ptr(), w.data_ptr(), int(t), pair_expert.data_ptr(),
                                        pair_row.data_ptr() if pair_row is not None else None, P, n_experts_total,
                                        y.data_ptr(), K, N, _stream())
    if rc == 1:
        # not a grouped-kernel type: the reference's own shape, one expert-indexed GEMV per input row
        rows = pair_row.cpu().tolist() if pair_row is not None else list(range(P))
        start = 0
        while start < P:
            end = start
            while end < P and rows[end] == rows[start]:
                end += 1
            moe_gemv(x[rows[start]], w, t, pair_expert[start:end], K, N, per_expert_x=False, y=y[start:end])
            start = end
        return y
    _check(L, rc)
    return y


SWIGLU, GEGLU = 0, 1


def moe_ffn(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, t_gate_up: int, t_down: int,
            top_idx: torch.Tensor, top_w: torch.Tensor, n_experts_total: int, hidden: int, inter: int,
            activation: int = SWIGLU, out: torch.Tensor | None = None, h_out: torch.Tensor | None = None,
            down_scale: torch.Tensor | None = None) -> torch.Tensor:
    """The fused expert FFN (laplace_cuda_moe_ffn_dev): out[t] = sum over the experts of token t that live here of
    top_w * down(act(gate_up(x[t]))). Raises for types the grouped kernels do not take."""
    L = lib()
    T, k = top_idx.shape
    assert top_idx.dtype == torch.int32 and top_idx.is_cuda and top_idx.is_contiguous()
    assert top_w.dtype == torch.float32 and top_w.is_cuda and top_w.is_contiguous() and top_w.shape == top_idx.shape
    assert x.dtype == torch.float32 and x.is_cuda and x.is_contiguous() and x.shape == (T, hidden)
    if out is None:
        out = torch.empty((T, hidden), dtype=torch.float32, device=x.device)
    _check(L, L.laplace_cuda_moe_ffn_dev(x.data_ptr(), w_gate_up.data_ptr(), w_down.data_ptr(), int(t_gate_up), int(t_down),
                                         top_idx.data_ptr(), top_w.data_ptr(),
                                         down_scale.data_ptr() if down_scale is not None else None, T, k, n_experts_total, hidden, inter,
                                         activation, out.data_ptr(), h_out.data_ptr() if h_out is not None else None,
                                         _stream()))
    return out


def moe_route(logits: torch.Tensor, top_k: int):
    """Softmax, top-k by repeated argmax and renormalisation of router logits [T, E] (laplace_cuda_moe_route_dev)."""
    L = lib()
    T, E = logits.shape
    assert logits.dtype == torch.float32 and logits.is_cuda and logits.is_contiguous()
    idx = torch.empty((T, top_k), dtype=torch.int32, device=logits.device)
    wts = torch.empty((T, top_k), dtype=torch.float32, device=logits.device)
    _check(L, L.laplace_cuda_moe_route_dev(logits.data_ptr(), T, E, top_k, idx.data_ptr(), wts.data_ptr(), _stream()))
    return idx, wts


def moe_pack(x: torch.Tensor, top_idx: torch.Tensor, top_w: torch.Tensor, packed: torch.Tensor) -> torch.Tensor:
    """[x | expert ids | weights] rows of this rank's tokens for the one all-gather of the expert-parallel layer."""
    L = lib()
    T, H = x.shape
    k = top_idx.shape[1]
    assert packed.shape == (T, H + 2 * k) and packed.is_contiguous() and x.is_contiguous()
    assert top_idx.is_contiguous() and top_w.is_contiguous() and top_idx.dtype == torch.int32
    _check(L, L.laplace_cuda_moe_pack_dev(x.data_ptr(), top_idx.data_ptr(), top_w.data_ptr(), T, H, k, packed.data_ptr(), _stream()))
    return packed


def moe_unpack(packed: torch.Tensor, hidden: int, top_k: int, expert_first: int, expert_count: int,
               x: torch.Tensor, idx_local: torch.Tensor, top_w: torch.Tensor) -> None:
    """Splits gathered rows into x, local expert ids (-1 = another rank's expert) and weights."""
    L = lib()
    T = packed.shape[0]
    assert packed.is_contiguous() and packed.shape[1] == hidden + 2 * top_k
    assert x.shape == (T, hidden) and idx_local.dtype == torch.int32 and idx_local.shape == (T, top_k) and top_w.shape == (T, top_k)
    _check(L, L.laplace_cuda_moe_unpack_dev(packed.data_ptr(), T, hidden, top_k, expert_first, expert_count, x.data_ptr(),
                                            idx_local.data_ptr(), top_w.data_ptr(), _stream()))


def quantize_act(x: torch.Tensor, M: int, K: int):
    """Returns (q int8 [M,K], d f32 [M,K/32], sum f32 [M,K/32], isum int16 [M,K/32,2])."""
    L = lib()
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    d = torch.empty((M, K // 32), dtype=torch.float32, device=x.device)
    s = torch.empty((M, K // 32), dtype=torch.float32, device=x.device)
    i = torch.empty((M, K // 32, 2), dtype=torch.int16, device=x.device)
    _check(L, L.laplace_cuda_quantize_act_dev(x.data_ptr(), M, K, q.data_ptr(), d.data_ptr(), s.data_ptr(),
                                              i.data_ptr(), _stream()))
    return q, d, s, i


def debug_blocksums(x: torch.Tensor, w: torch.Tensor, t: int, M: int, K: int, N: int) -> torch.Tensor:
    L = lib()
    out = torch.empty((M, N, blocksums_per_row(t, K)), dtype=torch.int32, device=x.device)
    _check(L, L.laplace_cuda_debug_blocksums_dev(x.data_ptr(), w.data_ptr(), int(t), out.data_ptr(), M, K, N, _stream()))
    return out


def dequantize(w: torch.Tensor, t: int, n: int) -> torch.Tensor:
    """dequantize(w, dst, n) of src/matmul.cpp:504 on device blocks."""
    dst = torch.empty(n, dtype=torch.float32, device=w.device)
    L = lib()
    _check(L, L.laplace_cuda_dequantize_dev(w.data_ptr(), int(t), dst.data_ptr(), n, _stream()))
    return dst


def embed_rows(w: torch.Tensor, t: int, tokens: torch.Tensor, H: int, vocab: int, scale: float = 1.0) -> torch.Tensor:
    """Token-embedding lookup (src/model.cpp:366-378): rows tokens[m] of the table, dequantized, times scale."""
    M = tokens.numel()
    dst = torch.empty((M, H), dtype=torch.float32, device=w.device)
    L = lib()
    _check(L, L.laplace_cuda_embed_rows_dev(w.data_ptr(), int(t), tokens.data_ptr(), M, H, vocab, float(scale), dst.data_ptr(), _stream()))
    return dst


def lm_head(x: torch.Tensor, w: torch.Tensor, t: int, M: int, K: int, N: int, softcap: float = 0.0) -> torch.Tensor:
    """matmul_lm_head (src/matmul.cpp:439) plus the optional logit soft-cap (src/model.cpp:399-406)."""
    y = torch.empty((M, N), dtype=torch.float32, device=x.device)
    L = lib()
    _check(L, L.laplace_cuda_lm_head_dev(x.data_ptr(), w.data_ptr(), int(t), y.data_ptr(), M, K, N, float(softcap), _stream()))
    return y


def sync() -> None:
    """Drains torch's stream and the library's, then surfaces any device-side timeout."""
    torch.cuda.synchronize()
    L = lib()
    _check(L, L.laplace_cuda_sync())

"""Expert placement across ranks (laplace_b200/moe.py) on CPU: gloo ranks, the grouped matmul played by the
oracle. The layer output of every rank's tokens must equal the reference's per-token sequence
(gate/up over the token's experts, gated activation, down, weighted sum; src/arch_gemma4.cpp:600-638)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests import synth
from laplace_b200.ggml import GGMLType, row_bytes
from laplace_b200.moe import ExpertParallelMoE, seeded_routing, silu_mul
from tests.oracle_lib import Oracle

T_TYPE = int(GGMLType.Q4_K)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_mm(orc):
    def mm(x, w, pair_expert, pair_row, n_experts, K, N, y):
        xe, pe = x.numpy(), pair_expert.numpy()
        rows = np.arange(pe.size) if pair_row is None else pair_row.numpy()
        wn = w.numpy()
        for p in range(pe.size):
            if pe[p] >= 0:
                y[p] = torch.from_numpy(orc.moe_gemv(xe[rows[p]], wn, T_TYPE, pe[p:p + 1], K, N, multi=False, mode=0)[0])
        return y
    return mm


def _inputs(E, k, H, I, T):
    w_gu = synth.weights(T_TYPE, H, E * 2 * I, seed=500, how="random")
    w_dn = synth.weights(T_TYPE, I, E * H, seed=501, how="random")
    x = synth.normal_f32(502, (T, H))
    idx, wts = seeded_routing(503, T, E, k)
    return w_gu, w_dn, x, idx, wts


def _reference_layer(orc, w_gu, w_dn, x, idx, wts, E, k, H, I):
    out = np.zeros((x.shape[0], H), dtype=np.float32)
    for tok in range(x.shape[0]):
        gu = orc.moe_gemv(x[tok], w_gu, T_TYPE, idx[tok], H, 2 * I, multi=False, mode=0)
        h = silu_mul(torch.from_numpy(gu), I).numpy()
        dn = orc.moe_gemv(h, w_dn, T_TYPE, idx[tok], I, H, multi=True, mode=0)
        out[tok] = (dn * wts[tok][:, None]).sum(axis=0)
    return out


def _worker(rank, world, port, E, k, H, I, T_loc, out_dir, exchange="allgather"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        orc = Oracle()
        T = T_loc * world
        w_gu, w_dn, x, idx, wts = _inputs(E, k, H, I, T)
        E_loc = E // world
        gu_rows, dn_rows = 2 * I * E_loc, H * E_loc
        layer = ExpertParallelMoE(torch.from_numpy(w_gu[rank * gu_rows:(rank + 1) * gu_rows].copy()),
                                  torch.from_numpy(w_dn[rank * dn_rows:(rank + 1) * dn_rows].copy()),
                                  E, k, H, I, _oracle_mm(orc), rank, world, exchange=exchange)
        sl = slice(rank * T_loc, (rank + 1) * T_loc)
        out = layer.forward(torch.from_numpy(x[sl].copy()), torch.from_numpy(idx[sl].copy()), torch.from_numpy(wts[sl].copy()))
        want = _reference_layer(orc, w_gu, w_dn, x, idx, wts, E, k, H, I)[sl]
        err = float(np.abs(out.numpy() - want).max() / (np.sqrt((want ** 2).mean()) + 1e-30))
        with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
            f.write(f"{err}\n")
        if exchange == "alltoall" and world > 1:
            # a token travels once per destination GPU, not once per expert and not to GPUs that hold none of its experts
            owners = idx[sl] // E_loc
            want_rows = sum(len(set(row.tolist())) for row in owners)
            assert layer.last_dispatch_rows == want_rows, (layer.last_dispatch_rows, want_rows)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2, 4])
def test_expert_parallel_layer(tmp_path, world):
    E, k, H, I, T_loc = 8, 3, 256, 256, 3
    assert row_bytes(T_TYPE, H) == 144
    mp.spawn(_worker, args=(world, _free_port(), E, k, H, I, T_loc, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        err = float((tmp_path / f"r{r}.txt").read_text())
        assert err < 1e-5, f"rank {r}: max-abs / RMS = {err}"


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_layer_token_alltoall(tmp_path, world):
    """The token all-to-all form of the exchange: deduplicated dispatch, partial sums added in rank order."""
    E, k, H, I, T_loc = 8, 3, 256, 256, 3
    mp.spawn(_worker, args=(world, _free_port(), E, k, H, I, T_loc, str(tmp_path), "alltoall"), nprocs=world, join=True)
    for r in range(world):
        err = float((tmp_path / f"r{r}.txt").read_text())
        assert err < 1e-5, f"rank {r}: max-abs / RMS = {err}"


def _oracle_ffn(orc):
    """The fused-FFN callable of ExpertParallelMoE played by the oracle (per-pair gate/up, SwiGLU, down, weighted sum)."""
    def ffn(x, w_gate_up, w_down, idx_local, top_w, n_experts, hidden, inter, out):
        xe, idx, wts = x.numpy(), idx_local.numpy(), top_w.numpy()
        wg, wd = w_gate_up.numpy(), w_down.numpy()
        out.zero_()
        for tok in range(idx.shape[0]):
            acc = np.zeros(hidden, dtype=np.float32)
            for j in range(idx.shape[1]):
                e = int(idx[tok, j])
                if e < 0:
                    continue
                gu = orc.moe_gemv(xe[tok], wg, T_TYPE, np.array([e], np.int32), hidden, 2 * inter, multi=False, mode=0)
                h = silu_mul(torch.from_numpy(gu), inter).numpy()
                dn = orc.moe_gemv(h, wd, T_TYPE, np.array([e], np.int32), inter, hidden, multi=True, mode=0)[0]
                acc += wts[tok, j] * dn
            out[tok] = torch.from_numpy(acc)
        return out
    return ffn


def _worker_fused(rank, world, port, E, k, H, I, T_loc, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        orc = Oracle()
        T = T_loc * world
        w_gu, w_dn, x, idx, wts = _inputs(E, k, H, I, T)
        E_loc = E // world
        gu_rows, dn_rows = 2 * I * E_loc, H * E_loc
        layer = ExpertParallelMoE(torch.from_numpy(w_gu[rank * gu_rows:(rank + 1) * gu_rows].copy()),
                                  torch.from_numpy(w_dn[rank * dn_rows:(rank + 1) * dn_rows].copy()),
                                  E, k, H, I, None, rank, world, fused_ffn=_oracle_ffn(orc))
        sl = slice(rank * T_loc, (rank + 1) * T_loc)
        out = layer.forward(torch.from_numpy(x[sl].copy()), torch.from_numpy(idx[sl].copy()), torch.from_numpy(wts[sl].copy()))
        want = _reference_layer(orc, w_gu, w_dn, x, idx, wts, E, k, H, I)[sl]
        err = float(np.abs(out.numpy() - want).max() / (np.sqrt((want ** 2).mean()) + 1e-30))
        with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
            f.write(f"{err}\n")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_expert_parallel_layer_fused_path(tmp_path, world):
    """The same layer through the fused-FFN hook (what bench.py --workload moe uses on GPUs)."""
    E, k, H, I, T_loc = 8, 3, 256, 256, 3
    mp.spawn(_worker_fused, args=(world, _free_port(), E, k, H, I, T_loc, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        err = float((tmp_path / f"r{r}.txt").read_text())
        assert err < 1e-5, f"rank {r}: max-abs / RMS = {err}"

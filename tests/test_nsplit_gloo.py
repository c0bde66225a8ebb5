"""Host logic of the N-split (tensor-parallel) path on CPU: row ranges, weight slicing, all-gather of slices.

Ranks are gloo processes; the per-rank matmul is done by the oracle here (this is a test of the split and the
exchange, not of a kernel), and the assembled result must equal the oracle's result over the whole matrix."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from laplace_b200 import _lib, ggml
from tests import synth
from laplace_b200.shard import RowShards
from tests.oracle_lib import Oracle


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, t, M, K, N, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lib = _lib.load()
        orc = Oracle()
        w = synth.weights(t, K, N, seed=77, how="random")
        x = synth.normal_f32(78, (M, K))
        sh = RowShards(lib, N, rank, world)
        w_loc = np.ascontiguousarray(sh.slice_rows(w))
        y_loc = orc.gemm(x, w_loc, t, M, K, sh.n_loc) if sh.n_loc else np.zeros((M, 0), np.float32)
        y_full = torch.full((M, N), float("nan"), dtype=torch.float32)
        sh.gather(torch.from_numpy(np.ascontiguousarray(y_loc.reshape(M, sh.n_loc))), y_full)
        want = orc.gemm(x, w, t, M, K, N).reshape(M, N)
        ok = np.array_equal(y_full.numpy(), want)
        with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
            f.write(f"{int(ok)} {sh.begin} {sh.end} {int(sh.even)}\n")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,M,N", [(2, 1, 256), (2, 3, 272), (2, 3, 256), (4, 5, 512), (3, 1, 80), (2, 1, 8), (4, 2, 1000)])
def test_split_and_gather(tmp_path, world, M, N):
    t, K = int(ggml.GGMLType.Q4_K), 512
    mp.spawn(_worker, args=(world, _free_port(), t, M, K, N, str(tmp_path)), nprocs=world, join=True)
    seen = []
    for r in range(world):
        ok, b, e, even = map(int, (tmp_path / f"r{r}.txt").read_text().split())
        assert ok == 1, f"rank {r}: gathered result differs from the whole-matrix result"
        seen.append((b, e))
    # ranges are contiguous, cover [0, N), start on 16-row boundaries
    assert seen[0][0] == 0 and seen[-1][1] == N
    for (b0, e0), (b1, e1) in zip(seen, seen[1:]):
        assert e0 == b1
    assert all(b % 16 == 0 for b, _ in seen)


def test_ranges_properties():
    lib = _lib.load()
    for N in (1, 15, 16, 17, 1024, 4096, 14336, 151936):
        for world in (1, 2, 3, 4, 8):
            rs = [RowShards(lib, N, r, world) for r in range(world)]
            assert rs[0].begin == 0 and rs[-1].end == N
            sizes = [r.n_loc for r in rs]
            assert sum(sizes) == N
            full = [s for s in sizes if s]
            assert max(sizes) - min(sizes) <= 16 + 15, (N, world, sizes)
            assert all(r.begin % 16 == 0 for r in rs)
            assert all(a.end == b.begin for a, b in zip(rs, rs[1:]))
            del full

"""The fused all-gather (peer stores + step flags) across two GPUs, one process per GPU.

Skipped on a one-GPU box; tests/test_gemv_gpu.py covers the same kernel path with a world of one."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import datetime
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=60))
    from laplace_b200 import device
    from tests import synth
    from laplace_b200.ggml import GGMLType
    from laplace_b200.shard import PeerGather, RowShards
    L = device.lib(rank)
    ok = True
    for t, M, K, N in [(GGMLType.Q4_K, 1, 4096, 2048), (GGMLType.Q6_K, 3, 512, 208), (GGMLType.Q8_0, 8, 256, 1000)]:
        w = synth.weights(t, K, N, seed=800 + M, how="random")
        sh = RowShards(L, N, rank, world)
        w_loc = device.upload_weights(np.ascontiguousarray(sh.slice_rows(w)))
        w_all = device.upload_weights(w)
        pg = PeerGather(L, sh, M)
        for step in range(1, 6):
            x = torch.from_numpy(synth.normal_f32(810 + step, (M, K))).cuda()
            pg.gemm(x, w_loc, t, K, device._stream())
            if step in (2, 5):                      # chains of steps closed by one wait
                pg.wait(device._stream())
                device.sync()
                want = device.gemm(x, w_all, t, M, K, N)
                device.sync()
                ok = ok and bool(torch.equal(pg.slot(step), want))
        pg.close()
    # prefill: the GEMM's drain stores every rank's slice into every rank's buffer; bit-identical to one GPU computing
    # the whole matrix (an N-split does not change any dot's summation... per tile; compared at the tests' tolerance)
    for t, M, K, N in [(GGMLType.Q4_K, 200, 1024, 1024), (GGMLType.Q6_K, 72, 2048, 400), (GGMLType.Q4_K, 512, 4096, 4096)]:
        w = synth.weights(t, K, N, seed=830 + M, how="random")
        sh = RowShards(L, N, rank, world)
        w_loc = device.upload_weights(np.ascontiguousarray(sh.slice_rows(w)))
        w_all = device.upload_weights(w)
        pg = PeerGather(L, sh, M)
        for rep in range(2):
            x = torch.from_numpy(synth.normal_f32(840 + rep, (M, K))).cuda()
            ok = ok and pg.gemm_peers(x, w_loc, t, K, device._stream())
            pg.step_wait(device._stream())
            device.sync()
            want = device.gemm(x, w_all, t, M, K, N)
            device.sync()
            got = pg.slot(0)
            rel = float((got - want).norm() / want.norm())
            ok = ok and rel <= 1e-5
        pg.close()
    with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
        f.write("1" if ok else "0")
    dist.barrier()
    torch.cuda.synchronize()
    os._exit(0)


def test_two_ranks(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0, f"rank process exit code {p.exitcode}"
    for r in range(2):
        assert (tmp_path / f"r{r}.txt").read_text() == "1", f"rank {r}: gathered result differs from the one-GPU result"

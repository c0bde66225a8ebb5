"""A bounded device-side wait that runs out, made on the host: the closing kernel of the fused all-gather is told
that the world has two GPUs, but the "peer's" flag array is this process's own zeroed memory that nobody raises.
The one-warp kernel gives up after its limit (a fraction of a second), records the time-out in the status word,
and returns; the context stays usable. Nothing faults, traps or spins forever."""
import ctypes as C

import numpy as np
import pytest

from laplace_b200.ggml import GGMLType
from tests import synth

pytestmark = pytest.mark.gpu


def test_peer_wait_times_out_and_the_library_recovers(oracle):
    import torch
    from laplace_b200 import device
    from laplace_b200.matmul import LaplaceCudaError
    L = device.lib()
    world, rank = 2, 0
    own_flags = torch.zeros(world, dtype=torch.int32, device="cuda")          # entry 1 would be raised by GPU 1: never happens
    fake_peer_flags = torch.zeros(world, dtype=torch.int32, device="cuda")
    step = torch.ones(1, dtype=torch.int32, device="cuda")                    # "step 1 has been sent"
    flags = (C.c_void_p * world)(own_flags.data_ptr(), fake_peer_flags.data_ptr())
    torch.cuda.synchronize()
    rc = L.laplace_cuda_allgather_wait_dev(flags, step.data_ptr(), rank, world, device._stream())
    assert rc == 0, L.laplace_cuda_last_error()
    with pytest.raises(LaplaceCudaError) as e:
        device.sync()                                                         # drains the stream, reads the status word
    assert e.value.code == -4, e.value                                        # LAPLACE_ERR_TIMEOUT
    assert int(fake_peer_flags[rank].item()) == 1                             # the announcement itself went out
    # the status word has been cleared and the context is intact: an ordinary call works and is correct
    t, M, K, N = GGMLType.Q4_K, 1, 512, 64
    w = synth.weights(t, K, N, seed=5, how="random")
    x = synth.normal_f32(6, (M, K))
    y = device.gemm(torch.from_numpy(x).cuda(), device.upload_weights(w), t, M, K, N)
    device.sync()
    ref = oracle.gemm(x, w, t, M, K, N, mode=1).astype(np.float64)
    assert np.linalg.norm(y.cpu().numpy() - ref) <= 1e-5 * np.linalg.norm(ref)

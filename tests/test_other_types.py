"""Weight types outside the int8 path (F32, F16, BF16, Q5_0, Q2_K, Q3_K, Q5_K), dequantize() for every type, the
token-embedding lookup and the LM head with its soft-cap. The reference serves these through its scalar path
(gemm_fallback, src/matmul.cpp:336-352) and dequantize (src/matmul.cpp:504-675); the checker is the reference's
own code compiled from its sources (oracle/_ref) where that exists, and always the vectors it produced
(tests/golden/other_types_golden.npz)."""
import numpy as np
import pytest

from tests import synth
from tests.oracle_lib import Reference
from tests.parity import check_close

OTHER = [0, 1, 30, 6, 10, 11, 13]
ALL = OTHER + [2, 8, 12, 14]
NAMES = {0: "F32", 1: "F16", 30: "BF16", 6: "Q5_0", 10: "Q2_K", 11: "Q3_K", 13: "Q5_K", 2: "Q4_0", 8: "Q8_0", 12: "Q4_K", 14: "Q6_K"}


def _weights(t, K, N, seed):
    if t in OTHER:
        return synth.other_type_weights(t, K, N, seed)
    return synth.weights(t, K, N, seed=seed, how="random")


def test_golden_file_matches_the_reference_build(golden_dir):
    """The stored vectors are what the reference build computes today (where it exists)."""
    if not Reference.available():
        pytest.skip("no reference build on this machine")
    r = Reference()
    z = np.load(golden_dir / "other_types_golden.npz")
    for t in ALL:
        w = z[f"w_{t}"]
        assert np.array_equal(r.dequantize(w, t, w.shape[0] * int(z["K"])), z[f"deq_{t}"]), NAMES[t]
        if t in OTHER:
            assert np.array_equal(r.matmul_rows(z["x"], w, t, z["x"].shape[0], int(z["K"]), w.shape[0]), z[f"y_{t}"]), NAMES[t]


@pytest.mark.gpu
@pytest.mark.parametrize("t", ALL)
def test_dequantize_is_bit_identical(golden_dir, t):
    import torch
    from laplace_b200 import device
    z = np.load(golden_dir / "other_types_golden.npz")
    w, K = z[f"w_{t}"], int(z["K"])
    got = device.dequantize(device.upload_weights(w), t, w.shape[0] * K)
    device.sync()
    assert np.array_equal(got.cpu().numpy(), z[f"deq_{t}"]), NAMES[t]
    if Reference.available():       # a larger, fresh case against the reference build itself
        w2 = _weights(t, 1024, 37, seed=500 + t)
        got2 = device.dequantize(device.upload_weights(w2), t, 37 * 1024)
        device.sync()
        assert np.array_equal(got2.cpu().numpy(), Reference().dequantize(w2, t, 37 * 1024)), NAMES[t]


@pytest.mark.gpu
@pytest.mark.parametrize("t", OTHER)
def test_matmul_with_fp32_activations(golden_dir, t):
    import torch
    from laplace_b200 import device
    z = np.load(golden_dir / "other_types_golden.npz")
    w, x, K = z[f"w_{t}"], z["x"], int(z["K"])
    M, N = x.shape[0], w.shape[0]
    y = device.gemm(torch.from_numpy(x).cuda(), device.upload_weights(w), t, M, K, N)
    device.sync()
    assert device.lib().laplace_cuda_last_path() == 4
    check_close(y.cpu().numpy(), z[f"y_{t}"].astype(np.float64), f"{NAMES[t]} golden")
    if Reference.available():
        r = Reference()
        for (M2, K2, N2) in ((1, 4096, 300), (8, 1024, 77), (11, 512, 40), (2, 14336, 24)):
            w2 = _weights(t, K2, N2, seed=600 + t)
            x2 = synth.normal_f32(601 + t, (M2, K2))
            y2 = device.gemm(torch.from_numpy(x2).cuda(), device.upload_weights(w2), t, M2, K2, N2)
            device.sync()
            check_close(y2.cpu().numpy(), r.matmul_rows(x2, w2, t, M2, K2, N2).astype(np.float64), f"{NAMES[t]} {M2}x{K2}x{N2}")


@pytest.mark.gpu
@pytest.mark.parametrize("t", [1, 13])
def test_host_pointer_call_takes_the_other_types(golden_dir, t):
    """laplace_cuda_gemm (what the shim binds) no longer answers "unsupported" for these types."""
    from laplace_b200 import device
    z = np.load(golden_dir / "other_types_golden.npz")
    w, x, K = np.ascontiguousarray(z[f"w_{t}"]), np.ascontiguousarray(z["x"]), int(z["K"])
    M, N = x.shape[0], w.shape[0]
    y = np.zeros((M, N), dtype=np.float32)
    L = device.lib()
    rc = L.laplace_cuda_gemm(x.ctypes.data, w.ctypes.data, t, y.ctypes.data, M, K, N)
    assert rc == 0, L.laplace_cuda_last_error()
    check_close(y, z[f"y_{t}"].astype(np.float64), f"{NAMES[t]} host call")


@pytest.mark.gpu
@pytest.mark.parametrize("t", [8, 12, 1])
def test_embedding_rows(golden_dir, t):
    import torch
    from laplace_b200 import device
    from laplace_b200.matmul import LaplaceCudaError
    z = np.load(golden_dir / "other_types_golden.npz")
    w, K = z[f"w_{t}"], int(z["K"])
    vocab = w.shape[0]
    deq = z[f"deq_{t}"].reshape(vocab, K)
    tokens = np.array([vocab - 1, 0, 3, 3, 1], dtype=np.int32)
    wd = device.upload_weights(w)
    got = device.embed_rows(wd, t, torch.from_numpy(tokens).cuda(), K, vocab, scale=1.0)
    device.sync()
    assert np.array_equal(got.cpu().numpy(), deq[tokens])
    got = device.embed_rows(wd, t, torch.from_numpy(tokens).cuda(), K, vocab, scale=22.627417)
    device.sync()
    assert np.array_equal(got.cpu().numpy(), deq[tokens] * np.float32(22.627417))
    device.embed_rows(wd, t, torch.tensor([0, vocab], dtype=torch.int32, device="cuda"), K, vocab)
    with pytest.raises(LaplaceCudaError):
        device.sync()
    device.sync()


@pytest.mark.gpu
def test_lm_head_with_soft_cap(oracle):
    """An LM head is a tall matmul (here 40,000 rows) followed by tanh(y / cap) * cap (src/model.cpp:399-406)."""
    import torch
    from laplace_b200 import device
    t, M, K, N, cap = 14, 2, 512, 40000, 30.0
    w = synth.weights(t, K, N, seed=700, how="affine")
    x = synth.normal_f32(701, (M, K)) * 40.0
    xd, wd = torch.from_numpy(x).cuda(), device.upload_weights(w)
    plain = device.lm_head(xd, wd, t, M, K, N)
    capped = device.lm_head(xd, wd, t, M, K, N, softcap=cap)
    device.sync()
    ref = oracle.gemm(x, w, t, M, K, N, mode=1, threads=8)
    check_close(plain.cpu().numpy(), ref, "lm head")
    want = np.tanh(plain.cpu().numpy().astype(np.float64) / cap) * cap
    assert np.abs(capped.cpu().numpy() - want).max() <= 4e-6 * cap
    assert np.abs(want).max() > 0.5 * cap          # the cap is actually at work on these inputs

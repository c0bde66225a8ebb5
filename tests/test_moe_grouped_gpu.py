"""GPU parity of the expert-grouped matmul against the oracle's per-token MoE GEMVs, through the C ABI.

The reference computes a mixture-of-experts layer token by token (fused_moe_gemm_idx for gate/up with one shared
input, fused_moe_gemm_multi for down with one input per selected expert, src/matmul.cpp:467-500); the grouped call
must reproduce every one of those per-token results."""
import numpy as np
import pytest

from tests import synth
from laplace_b200.ggml import GGMLType
from tests.parity import check_close

pytestmark = pytest.mark.gpu


def _routing(seed, T, E, top_k):
    """Seeded router: logits ~ N(0,1), top-k experts per token (the shape of BASELINE config 5)."""
    logits = synth.normal_f32(seed, (T, E))
    return np.argsort(-logits, axis=1)[:, :top_k].astype(np.int32)


def _run(t, x, w, pair_expert, pair_row, E, K, N):
    import torch
    from laplace_b200 import device
    pe = torch.from_numpy(np.ascontiguousarray(pair_expert, dtype=np.int32)).cuda()
    pr = None if pair_row is None else torch.from_numpy(np.ascontiguousarray(pair_row, dtype=np.int32)).cuda()
    y = device.moe_grouped(torch.from_numpy(x).cuda(), device.upload_weights(w), t, pe, pr, E, K, N)
    device.sync()
    return y.cpu().numpy(), device.lib().laplace_cuda_last_path()


@pytest.mark.parametrize("t,K", [(GGMLType.Q4_K, 512), (GGMLType.Q4_K, 768), (GGMLType.Q6_K, 2048)])
@pytest.mark.parametrize("T,E,top_k,N", [(24, 8, 2, 128), (64, 16, 4, 200), (5, 4, 1, 64)])
def test_shared_input_form(oracle, t, K, T, E, top_k, N):
    """gate/up shape: the top-k pairs of a token share its input row (fused_moe_gemm_idx per token)."""
    w = synth.weights(t, K, N * E, seed=300 + T, how="random")
    x = synth.normal_f32(301 + E, (T, K))
    top = _routing(302 + T, T, E, top_k)
    pair_expert = top.reshape(-1)
    pair_row = np.repeat(np.arange(T, dtype=np.int32), top_k)
    y, path = _run(t, x, w, pair_expert, pair_row, E, K, N)
    assert path == 3, "the grouped tensor-core path did not run"
    ref = np.concatenate([oracle.moe_gemv(x[tok], w, t, top[tok], K, N, multi=False, mode=1) for tok in range(T)])
    check_close(y, ref, f"grouped shared {t.name} T={T} E={E} k={top_k} K={K} N={N}")


@pytest.mark.parametrize("t,K", [(GGMLType.Q4_K, 768), (GGMLType.Q6_K, 2048)])
def test_per_pair_input_form(oracle, t, K):
    """down shape: every pair has its own input row (fused_moe_gemm_multi per token)."""
    T, E, top_k, N = 20, 8, 3, 256
    w = synth.weights(t, K, N * E, seed=310, how="affine")
    top = _routing(311, T, E, top_k)
    x = synth.normal_f32(312, (T * top_k, K))
    y, path = _run(t, x, w, top.reshape(-1), None, E, K, N)
    assert path == 3
    ref = np.concatenate([oracle.moe_gemv(x[tok * top_k:(tok + 1) * top_k], w, t, top[tok], K, N, multi=True, mode=1)
                          for tok in range(T)])
    check_close(y, ref, f"grouped multi {t.name}")


def test_expert_with_more_than_one_row_group(oracle):
    """One expert takes 300 pairs (three 128-row groups), one takes none, order of pairs is shuffled."""
    t, K, N, E = GGMLType.Q4_K, 512, 128, 5
    w = synth.weights(t, K, N * E, seed=320, how="random")
    pair_expert = np.concatenate([np.full(300, 3), np.full(7, 0), np.full(129, 4), np.full(1, 1)]).astype(np.int32)
    rng = np.random.default_rng(321)
    rng.shuffle(pair_expert)
    P = pair_expert.size
    x = synth.normal_f32(322, (P, K))
    y, path = _run(t, x, w, pair_expert, None, E, K, N)
    assert path == 3
    ref = oracle.moe_gemv(x, w, t, pair_expert, K, N, multi=True, mode=1, threads=8)
    check_close(y, ref, "grouped, uneven experts")


def test_grouped_equals_per_token_calls_on_device(oracle):
    """The same pairs through one grouped call and through one expert-indexed GEMV call per token."""
    import torch
    from laplace_b200 import device
    t, K, N, E, T, top_k = GGMLType.Q4_K, 1024, 192, 12, 16, 4
    w = synth.weights(t, K, N * E, seed=330, how="ref")
    x = synth.normal_f32(331, (T, K))
    top = _routing(332, T, E, top_k)
    y, _ = _run(t, x, w, top.reshape(-1), np.repeat(np.arange(T, dtype=np.int32), top_k), E, K, N)
    wd, xd = device.upload_weights(w), torch.from_numpy(x).cuda()
    per_token = [device.moe_gemv(xd[tok], wd, t, torch.from_numpy(top[tok]).cuda(), K, N, per_expert_x=False)
                 for tok in range(T)]
    device.sync()
    ref = torch.cat(per_token).cpu().numpy()
    assert np.allclose(y, ref, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("t", [GGMLType.Q8_0, GGMLType.Q4_0, GGMLType.Q6_K])
def test_other_types_run_grouped(oracle, t):
    K, N, E, T, top_k = 512, 136, 6, 21, 2
    w = synth.weights(t, K, N * E, seed=345, how="random")
    x = synth.normal_f32(346, (T, K))
    top = _routing(347, T, E, top_k)
    y, path = _run(t, x, w, top.reshape(-1), np.repeat(np.arange(T, dtype=np.int32), top_k), E, K, N)
    assert path == 3
    ref = np.concatenate([oracle.moe_gemv(x[tok], w, t, top[tok], K, N, multi=False, mode=1) for tok in range(T)])
    check_close(y, ref, f"grouped {t.name}")


def test_other_k_falls_back_to_expert_indexed_gemv(oracle):
    """K that is not a multiple of 256: no grouped kernel, the Python mirror loops the expert-indexed GEMV."""
    t, K, N, E, T, top_k = GGMLType.Q8_0, 160, 64, 6, 5, 2
    w = synth.weights(t, K, N * E, seed=340, how="random")
    x = synth.normal_f32(341, (T, K))
    top = _routing(342, T, E, top_k)
    y, path = _run(t, x, w, top.reshape(-1), np.repeat(np.arange(T, dtype=np.int32), top_k), E, K, N)
    assert path == 1
    ref = np.concatenate([oracle.moe_gemv(x[tok], w, t, top[tok], K, N, multi=False, mode=1) for tok in range(T)])
    check_close(y, ref, "grouped fallback Q8_0, K=160")


def test_bad_expert_index_is_reported():
    import torch
    from laplace_b200 import device
    from laplace_b200.matmul import LaplaceCudaError
    t, K, N, E = GGMLType.Q4_K, 512, 128, 4
    w = device.upload_weights(synth.weights(t, K, N * E, seed=350, how="random"))
    x = torch.from_numpy(synth.normal_f32(351, (3, K))).cuda()
    pe = torch.tensor([0, 9, 2], dtype=torch.int32, device="cuda")
    y = torch.zeros((3, N), dtype=torch.float32, device="cuda")
    device.moe_grouped(x, w, t, pe, None, E, K, N, y=y)
    with pytest.raises(LaplaceCudaError):
        device.sync()
    device.sync()                      # the status word is cleared by the failed sync
    assert torch.count_nonzero(y[1]).item() == 0 and torch.count_nonzero(y[0]).item() > 0


def test_negative_expert_index_skips_the_pair(oracle):
    """Pairs whose expert lives on another GPU are passed as -1: not computed, not an error."""
    import torch
    from laplace_b200 import device
    t, K, N, E = GGMLType.Q4_K, 512, 128, 4
    w = synth.weights(t, K, N * E, seed=360, how="random")
    x = synth.normal_f32(361, (6, K))
    pe = np.array([2, -1, 0, -1, -1, 3], dtype=np.int32)
    y = torch.full((6, N), 7.0, dtype=torch.float32, device="cuda")
    device.moe_grouped(torch.from_numpy(x).cuda(), device.upload_weights(w), t, torch.from_numpy(pe).cuda(), None, E, K, N, y=y)
    device.sync()
    got = y.cpu().numpy()
    live = pe >= 0
    assert np.all(got[~live] == 7.0)
    ref = oracle.moe_gemv(x[live], w, t, pe[live], K, N, multi=True, mode=1)
    check_close(got[live], ref, "grouped with skipped pairs")

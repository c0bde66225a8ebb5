"""GPU parity at the full sizes of the benchmark configurations, through the C ABI.

Four kinds of check:
  * every decode shape, small-batch shape and prefill projection against the CPU oracle (float64 mode) at
    1e-5 relative L2 / 1e-3 max-abs over RMS;
  * the same shapes with activations that the Q8 quantizer represents exactly, against the REFERENCE's own
    compiled scalar matmul (oracle/_ref/libref_matmul.so, built from the reference's sources): with such inputs
    its fp32-activation path and its int8 path are the same arithmetic up to fp32 summation order, so this pins
    the CUDA kernels to reference output at 1e-5 without going through the restatement;
  * integer block sums of the kernels that are timed (not of the debug kernel): inputs in which one 32-value
    block per row is live make every output equal scale * integer exactly, so the integer is read back from y
    bit for bit, for every block position of a super-block;
  * the fused expert FFN at 128 experts / top-8 / 256 tokens / 2048 / 768 with seeded routing.
"""
import os

import numpy as np
import pytest

from laplace_b200.ggml import GGMLType
from laplace_b200.moe import seeded_routing
from tests import synth
from tests.oracle_lib import Reference
from tests.parity import check_close

pytestmark = pytest.mark.gpu
THREADS = os.cpu_count() or 1

DECODE_SHAPES = [(4096, 4096), (4096, 1024), (4096, 14336), (14336, 4096)]
PREFILL = [("q", GGMLType.Q4_K, 4096, 4096), ("k", GGMLType.Q4_K, 4096, 1024), ("v", GGMLType.Q4_K, 4096, 1024),
           ("o", GGMLType.Q4_K, 4096, 4096), ("gate", GGMLType.Q4_K, 4096, 14336), ("up", GGMLType.Q4_K, 4096, 14336),
           ("down", GGMLType.Q6_K, 14336, 4096)]


def run_dev(t, x, w, M, K, N):
    import torch
    from laplace_b200 import device
    y = device.gemm(torch.from_numpy(x).cuda(), device.upload_weights(w), t, M, K, N)
    device.sync()
    return y.cpu().numpy(), device.lib().laplace_cuda_last_path()


def test_config1_q4_0_gemv(oracle):
    t, K, N = GGMLType.Q4_0, 4096, 4096
    w = synth.weights(t, K, N, seed=1010, how="ref")
    x = synth.normal_f32(2001, (1, K))
    y, _ = run_dev(t, x, w, 1, K, N)
    check_close(y, oracle.gemm(x, w, t, 1, K, N, mode=1, threads=THREADS), "Q4_0 4096x4096")


@pytest.mark.parametrize("t", [GGMLType.Q4_K, GGMLType.Q6_K])
@pytest.mark.parametrize("K,N", DECODE_SHAPES)
@pytest.mark.parametrize("how", ["ref", "affine"])
def test_config2_decode_shapes(oracle, t, K, N, how):
    w = synth.weights(t, K, N, seed=1020 + int(t), how=how)
    x = synth.normal_f32(2002, (1, K))
    y, path = run_dev(t, x, w, 1, K, N)
    assert path == 1
    check_close(y, oracle.gemm(x, w, t, 1, K, N, mode=1, threads=THREADS), f"{t.name} {K}x{N} {how}")


@pytest.mark.parametrize("M", [2, 4, 8])
def test_config3_small_batch(oracle, M):
    t, K, N = GGMLType.Q4_K, 4096, 14336
    w = synth.weights(t, K, N, seed=1030, how="ref")
    x = synth.normal_f32(2003 + M, (M, K))
    y, path = run_dev(t, x, w, M, K, N)
    assert path == 1
    check_close(y, oracle.gemm(x, w, t, M, K, N, mode=1, threads=THREADS), f"Q4_K M={M} 4096x14336")


@pytest.mark.parametrize("name,t,K,N", PREFILL)
def test_config4_prefill_projections(oracle, name, t, K, N):
    M = 512
    w = synth.weights(t, K, N, seed=1040 + len(name), how="ref")
    x = synth.normal_f32(2004, (M, K))
    y, path = run_dev(t, x, w, M, K, N)
    assert path == 2, "the tensor-core kernel did not run"
    check_close(y, oracle.gemm(x, w, t, M, K, N, mode=1, threads=THREADS), f"prefill {name} {t.name} 512x{K}x{N}")


@pytest.mark.skipif(not Reference.available(), reason="oracle/_ref (the reference's own code, compiled) is not present")
@pytest.mark.parametrize("t,M,K,N", [(GGMLType.Q4_0, 1, 4096, 4096), (GGMLType.Q8_0, 1, 4096, 4096),
                                     (GGMLType.Q4_K, 1, 4096, 14336), (GGMLType.Q4_K, 1, 14336, 4096),
                                     (GGMLType.Q6_K, 1, 4096, 14336), (GGMLType.Q6_K, 1, 14336, 4096),
                                     (GGMLType.Q4_K, 8, 4096, 14336), (GGMLType.Q4_K, 512, 4096, 4096),
                                     (GGMLType.Q4_K, 512, 4096, 1024), (GGMLType.Q6_K, 512, 14336, 4096),
                                     (GGMLType.Q4_0, 64, 4096, 1024), (GGMLType.Q8_0, 64, 4096, 1024)])
def test_against_the_reference_build_with_lossless_activations(t, M, K, N):
    ref = Reference()
    ref.set_threads(THREADS)
    w = synth.weights(t, K, N, seed=1050 + int(t), how="affine")
    x = synth.lossless_q8_activations(2005 + M, M, K)
    y, _ = run_dev(t, x, w, M, K, N)
    check_close(y, ref.matmul_rows(x, w, t, M, K, N), f"vs reference build, {t.name} {M}x{K}x{N}")


def test_against_stored_reference_outputs(golden_dir):
    """The same check against reference-build outputs stored by tests/golden/make_golden.py, for machines
    that have no oracle/_ref."""
    g = np.load(golden_dir / "lossless_golden.npz")
    for i in range(int(g["n_cases"])):
        t, M, K, N, wseed, xseed = (int(v) for v in g[f"l{i}_meta"])
        w = synth.weights(t, K, N, seed=wseed, how="affine")
        x = synth.lossless_q8_activations(xseed, M, K)
        y, _ = run_dev(GGMLType(t), x, w, M, K, N)
        check_close(y, g[f"l{i}_ref_y"], f"vs stored reference output, type {t} {M}x{K}x{N}")


def _expected_from_blocksums(oracle, t, w, x, sc, K, N, live):
    bs = oracle.blocksums(x, w, t, x.shape[0], K, N)
    M = x.shape[0]
    out = np.zeros((M, N), dtype=np.float32)
    for m in range(M):
        dx = np.abs(x[m, live * 32:(live + 1) * 32]).max() / np.float32(127.0)
        if t == GGMLType.Q6_K:
            v = sc[:, 0] * bs[m, :, 2 * live].astype(np.float32) + sc[:, 1] * bs[m, :, 2 * live + 1].astype(np.float32)
        elif t == GGMLType.Q4_0:
            v = bs[m, :, live].astype(np.float32) - np.float32(8.0) * np.float32(np.round(x[m] / dx).sum())
        else:
            v = sc * bs[m, :, live].astype(np.float32)
        out[m] = v * dx
    return out


@pytest.mark.parametrize("t", [GGMLType.Q4_0, GGMLType.Q8_0, GGMLType.Q4_K, GGMLType.Q6_K])
@pytest.mark.parametrize("M", [1, 4, 24])
def test_block_sums_of_the_timed_kernels_bit_exact(oracle, t, M):
    """M = 1, 4: the streaming GEMV; M = 24: the tensor-core GEMM. Every block position of a super-block (and one
    in a later super-block) is the live one in turn."""
    K, N = 2048, 136
    for live in list(range(8)) + [8 * 5 + 3, K // 32 - 1]:
        w, x1, sc = synth.single_live_block(t, K, N, 3000 + live, live)
        x = np.concatenate([x1 * np.float32(2.0 ** -(m % 5)) * (-1) ** m for m in range(M)])     # still exact in Q8
        y, path = run_dev(t, x, w, M, K, N)
        assert path == (1 if M <= 8 else 2)
        want = _expected_from_blocksums(oracle, t, w, x, sc, K, N, live)
        assert np.array_equal(y, want), f"{t.name} M={M} live block {live}: {np.abs(y - want).max()}"


def test_config5_fused_ffn_full_size(oracle):
    """128 experts, top-8, 256 tokens, hidden 2048, expert width 768, Q4_K, seeded routing: gate/up against the
    oracle's per-token expert GEMVs, the down matmul and weighted sum from the device's own activation values."""
    import torch
    from laplace_b200 import device
    t, E, k, T, H, I = GGMLType.Q4_K, 128, 8, 256, 2048, 768
    w_gu = synth.weights(t, H, E * 2 * I, seed=1060, how="ref")
    w_dn = synth.weights(t, I, E * H, seed=1061, how="ref")
    x = synth.normal_f32(2006, (T, H))
    idx, wts = seeded_routing(3000, T, E, k)
    xd, wg, wd = torch.from_numpy(x).cuda(), device.upload_weights(w_gu), device.upload_weights(w_dn)
    h_dev = torch.zeros((T * k, I), dtype=torch.float32, device="cuda")
    out = device.moe_ffn(xd, wg, wd, t, t, torch.from_numpy(idx).cuda(), torch.from_numpy(wts).cuda(), E, H, I,
                         activation=0, h_out=h_dev)
    device.sync()
    out, h_dev = out.cpu().numpy(), h_dev.cpu().numpy()
    gu = np.concatenate([oracle.moe_gemv(x[tok], w_gu, t, idx[tok], H, 2 * I, multi=False, mode=1, threads=THREADS)
                         for tok in range(T)])
    g, u = gu[:, :I].astype(np.float32), gu[:, I:].astype(np.float32)
    check_close(h_dev, (g / (np.float32(1.0) + np.exp(-g))) * u, "swiglu(gate/up), 128 experts")
    want = np.zeros((T, H), dtype=np.float64)
    for tok in range(T):
        dn = oracle.moe_gemv(h_dev[tok * k:(tok + 1) * k], w_dn, t, idx[tok], I, H, multi=True, mode=1, threads=THREADS)
        want[tok] = (dn.astype(np.float64) * wts[tok][:, None]).sum(axis=0)
    check_close(out, want, "fused FFN, 128 experts top-8 256 tokens")

"""CPU tests that pin the oracle: reference known answers, the reference test's own acceptance
check on its own seeded inputs, stored outputs of the reference's compiled code, and internal
consistency of the restatement."""
import numpy as np
import pytest

from tests import synth
from laplace_b200.ggml import GGMLType, blocksums_per_row, row_bytes
from tests.oracle_lib import ACTQ8, Reference

TYPES = [GGMLType.Q4_0, GGMLType.Q8_0, GGMLType.Q4_K, GGMLType.Q6_K]      # the types the reference's test_matmul builds
INT8_TYPES = TYPES + [GGMLType.Q5_0]                                      # every type with an int8 kernel there


def almost_equal(a, b, rel, abs_tol):
    """tests/test_util.h:33-38 of the reference."""
    diff = np.abs(a - b)
    return (diff <= abs_tol) | (diff <= rel * np.maximum(np.abs(a), np.abs(b)))


def test_fp16_known_answers(oracle):
    """The five known answers and the round trip of the reference's tests/test_matmul.cpp:252-268."""
    assert oracle.fp16_to_fp32(0x3C00) == 1.0
    assert oracle.fp16_to_fp32(0xC000) == -2.0
    assert oracle.fp16_to_fp32(0x0000) == 0.0
    assert oracle.fp16_to_fp32(0x7BFF) == 65504.0
    assert oracle.fp16_to_fp32(0x0001) == 5.9604644775390625e-08
    assert oracle.fp32_to_fp16(1.0) == 0x3C00
    assert oracle.fp32_to_fp16(-2.0) == 0xC000
    s = 31
    for _ in range(1000):                      # XorShift32(31), tests/test_util.h:47-61
        s ^= (s << 13) & 0xFFFFFFFF
        s ^= s >> 17
        s ^= (s << 5) & 0xFFFFFFFF
        h = s & 0x7FFF
        if (h & 0x7C00) == 0x7C00:
            continue
        assert oracle.fp32_to_fp16(oracle.fp16_to_fp32(h)) == h


def test_fp16_matches_reference_build(oracle, golden_dir):
    g = np.load(golden_dir / "hotpath_golden.npz")
    got = np.array([oracle.fp16_to_fp32(int(h)) for h in g["fp16_bits"]], dtype=np.float32)
    assert np.array_equal(got.view(np.uint32), g["fp16_ref_f32"].view(np.uint32))
    got16 = np.array([oracle.fp32_to_fp16(float(v)) for v in g["f32_vals"]], dtype=np.uint16)
    assert np.array_equal(got16, g["f32_ref_fp16"])
    assert np.array_equal(synth.f32_to_f16_bits(g["f32_vals"]), g["f32_ref_fp16"])


@pytest.mark.parametrize("t", TYPES)
@pytest.mark.parametrize("K,N", [(512, 1), (512, 8), (512, 33), (512, 256), (2816, 1), (2816, 8), (2816, 256), (2816, 4096)])
def test_reference_acceptance_check_on_its_own_inputs(oracle, t, K, N):
    """check_against_ref of tests/test_matmul.cpp:57-108 applied to the oracle's int8 path, with the
    x (XorShift32(7+type)) and weight blocks (seeds 17/19/23/29) that test builds."""
    if K == 2816 and t in (GGMLType.Q4_0, GGMLType.Q8_0):
        pytest.skip("the reference runs K=2816 for the K-quants only")
    x, w = oracle.testgen(t, K, N)
    wf = oracle.dequantize(w, t, K * N).reshape(N, K).astype(np.float64)
    y = oracle.gemm(x[None], w, t, 1, K, N)[0]
    y_exact = (wf @ x.astype(np.float64)).astype(np.float32)
    xq = x.reshape(-1, 32).copy()
    amax = np.abs(xq).max(axis=1, keepdims=True)
    d = (amax / np.float32(127)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d > 0, np.float32(1) / d, 0).astype(np.float32)
    r = xq * inv
    lround = np.trunc(r) + np.where(np.abs(r - np.trunc(r)) >= 0.5, np.sign(r), 0)   # lroundf
    y_q8 = (wf @ (d * lround.astype(np.float32)).reshape(-1).astype(np.float64)).astype(np.float32)
    ok = almost_equal(y, y_exact, 1e-3, 1e-3) | almost_equal(y, y_q8, 1e-3, 1e-3)
    assert ok.all(), f"{int((~ok).sum())}/{N} outputs match neither reference"


def test_batched_rows_equal_single_rows(oracle):
    """test_batched_rows of tests/test_matmul.cpp:217-250 (M=7, K=512, N=64), on the int8 path."""
    M, K, N = 7, 512, 64
    for t in (GGMLType.Q8_0, GGMLType.Q4_K):
        w = synth.random_blocks(t, K, N, seed=41 + int(t))
        x = synth.rng(42).uniform(-1, 1, size=(M, K)).astype(np.float32)
        yb = oracle.gemm(x, w, t, M, K, N)
        ys = np.stack([oracle.gemm(x[m:m + 1], w, t, 1, K, N)[0] for m in range(M)])
        assert np.array_equal(yb.view(np.uint32), ys.view(np.uint32))


def test_golden_vectors(oracle, golden_dir):
    """Stored outputs: the reference's compiled dequantize()/scalar matmul, and the oracle's own."""
    g = np.load(golden_dir / "hotpath_golden.npz")
    i = 0
    while f"c{i}_meta" in g:
        p = f"c{i}_"
        t, M, K, N = (int(v) for v in g[p + "meta"])
        w, x = g[p + "w"], g[p + "x"]
        how = str(g[p + "how"])
        assert np.array_equal(synth.weights(t, K, N, seed=9000 + i + 1, how=how), w), "synthetic weights drifted"
        assert np.array_equal(oracle.dequantize(w, t, K * N).view(np.uint32), g[p + "ref_dequant"].view(np.uint32))
        ys = oracle.gemm_scalar(x, w, t, M, K, N)
        assert np.allclose(ys, g[p + "ref_scalar_y"], rtol=1e-4, atol=1e-5), "scalar restatement vs reference build"
        assert np.array_equal(oracle.quantize(x).view(np.uint8).reshape(-1), g[p + "act"].reshape(-1))
        assert np.array_equal(oracle.blocksums(x, w, t, M, K, N), g[p + "blocksums"])
        assert np.array_equal(oracle.gemm(x, w, t, M, K, N, mode=0).view(np.uint32), g[p + "y_f32"].view(np.uint32))
        assert np.array_equal(oracle.gemm(x, w, t, M, K, N, mode=1).view(np.uint32), g[p + "y_f64"].view(np.uint32))
        # int8 path vs the reference's fp32-activation result: apart only by activation rounding
        a, b = g[p + "y_f64"].astype(np.float64), g[p + "ref_scalar_y"].astype(np.float64)
        assert np.linalg.norm(a - b) / np.linalg.norm(b) < 3e-2
        i += 1
    assert i == 12
    t, K, N, n_total = (int(v) for v in g["moe_meta"])
    yi = oracle.moe_gemv(g["moe_x"][0], g["moe_w"], t, g["moe_idx"], K, N, multi=False, mode=1)
    ym = oracle.moe_gemv(g["moe_x"], g["moe_w"], t, g["moe_idx"], K, N, multi=True, mode=1)
    assert np.array_equal(yi, g["moe_y_idx_f64"]) and np.array_equal(ym, g["moe_y_multi_f64"])
    assert np.linalg.norm(yi - g["moe_ref_scalar_idx"]) / np.linalg.norm(g["moe_ref_scalar_idx"]) < 3e-2
    assert np.linalg.norm(ym - g["moe_ref_scalar_multi"]) / np.linalg.norm(g["moe_ref_scalar_multi"]) < 3e-2


@pytest.mark.skipif(not Reference.available(), reason="oracle/_ref not built (no reference checkout here)")
@pytest.mark.parametrize("t", INT8_TYPES)
def test_against_reference_build_live(oracle, t):
    """Dequantizers bit-equal to the reference's compiled code; one-hot activations make Q8 lossless,
    so the int8 path must then reproduce single dequantized weights."""
    r = Reference()
    K, N = 512, 16
    for how in ("random", "ref", "affine"):
        w = synth.weights(t, K, N, seed=31 + int(t), how=how)
        assert np.array_equal(oracle.dequantize(w, t, K * N).view(np.uint32), r.dequantize(w, t, K * N).view(np.uint32))
    w = synth.weights(t, K, N, seed=33, how="affine")
    deq = r.dequantize(w, t, K * N).reshape(N, K)
    for k in (0, 17, 31, 32, 255, 300, 511):
        x = np.zeros((1, K), dtype=np.float32)
        x[0, k] = 127.0                                   # d = 1, q = 127: exact
        y = oracle.gemm(x, w, t, 1, K, N, mode=1)[0]
        assert np.allclose(y, 127.0 * deq[:, k].astype(np.float64), rtol=2e-6, atol=1e-9)


def test_quantizer_known_answers(oracle):
    """Ties vector of the reference's tests/test_laplace_kv.cpp:44-50 (sibling quantizer, same
    rounding rule): amax = 127 gives d = 1, and halves round to even."""
    ties = np.zeros(32, dtype=np.float32)
    ties[0] = 127.0
    ties[1:16] = np.arange(1, 16, dtype=np.float32) - 0.5
    a = oracle.quantize(ties[None])[0, 0]
    assert a["d"] == 1.0
    assert list(a["qs"][:16]) == [127, 0, 2, 2, 4, 4, 6, 6, 8, 8, 10, 10, 12, 12, 14, 14]
    assert a["sum_lo"] == 127 + sum([0, 2, 2, 4, 4, 6, 6, 8, 8, 10, 10, 12, 12, 14, 14]) and a["sum_hi"] == 0
    assert a["sum"] == float(a["sum_lo"])
    z = oracle.quantize(np.zeros((1, 32), dtype=np.float32))[0, 0]
    assert z["d"] == 0.0 and not z["qs"].any() and z["sum"] == 0.0
    n = np.ones((1, 32), dtype=np.float32)
    n[0, 5] = np.nan
    b = oracle.quantize(n)[0, 0]
    assert np.isnan(b["d"]) and not b["qs"].any()       # NaN amax -> id = 0 -> every q = 0


@pytest.mark.parametrize("t", INT8_TYPES)
def test_blocksums_rebuild_the_dot(oracle, t):
    """Scaling the integer block sums by the block scales reproduces the float64 dot."""
    M, K, N = 2, 512, 5
    w = synth.random_blocks(t, K, N, seed=55)
    x = synth.normal_f32(56, (M, K))
    bs = oracle.blocksums(x, w, t, M, K, N).astype(np.float64)
    act = oracle.quantize(x)
    y = oracle.gemm(x, w, t, M, K, N, mode=1).astype(np.float64)
    assert bs.shape == (M, N, blocksums_per_row(t, K))
    rb = row_bytes(t, K)
    f16 = lambda lo, hi: float(np.array([lo | (hi << 8)], dtype=np.uint16).view(np.float16)[0])
    for m in range(M):
        for j in range(N):
            row = w[j]
            acc = 0.0
            if t in (GGMLType.Q4_0, GGMLType.Q5_0, GGMLType.Q8_0):
                bb = rb // (K // 32)
                for b in range(K // 32):
                    dw = f16(int(row[b * bb]), int(row[b * bb + 1]))
                    acc += dw * float(act[m, b]["d"]) * bs[m, j, b]
                    if t == GGMLType.Q4_0:
                        acc -= dw * 8.0 * float(act[m, b]["sum"])
            elif t == GGMLType.Q4_K:
                for sb in range(K // 256):
                    blk = row[sb * 144:(sb + 1) * 144]
                    d, dmin = f16(int(blk[0]), int(blk[1])), f16(int(blk[2]), int(blk[3]))
                    s = blk[4:16].astype(int)
                    for jj in range(8):
                        if jj < 4:
                            sc, mn = s[jj] & 63, s[jj + 4] & 63
                        else:
                            sc = (s[jj + 4] & 0xF) | ((s[jj - 4] >> 6) << 4)
                            mn = (s[jj + 4] >> 4) | ((s[jj] >> 6) << 4)
                        a = act[m, sb * 8 + jj]
                        acc += d * sc * float(a["d"]) * bs[m, j, sb * 8 + jj] - dmin * mn * float(a["sum"])
            else:
                for sb in range(K // 256):
                    blk = row[sb * 210:(sb + 1) * 210]
                    d = f16(int(blk[208]), int(blk[209]))
                    sc = blk[192:208].view(np.int8).astype(int)
                    for g16 in range(16):
                        a = act[m, sb * 8 + g16 // 2]
                        acc += d * float(a["d"]) * sc[g16] * bs[m, j, sb * 16 + g16]
            assert abs(acc - y[m, j]) <= 1e-6 * max(1.0, abs(y[m, j])), (t, m, j, acc, y[m, j])


def test_moe_indexing(oracle):
    """Expert-indexed GEMVs equal plain GEMVs on the selected expert's slice (src/matmul_simd.cpp:506-544)."""
    t, K, N, n_total = GGMLType.Q4_K, 256, 12, 4
    w = synth.weights(t, K, N * n_total, seed=60, how="affine")
    idx = np.array([2, 2, 0], dtype=np.int32)
    x = synth.normal_f32(61, (3, K))
    yi = oracle.moe_gemv(x[0], w, t, idx, K, N, multi=False)
    ym = oracle.moe_gemv(x, w, t, idx, K, N, multi=True)
    for k, e in enumerate(idx):
        we = w[e * N:(e + 1) * N]
        assert np.array_equal(yi[k], oracle.gemm(x[0:1], we, t, 1, K, N)[0])
        assert np.array_equal(ym[k], oracle.gemm(x[k:k + 1], we, t, 1, K, N)[0])


def test_actq8_layout():
    assert ACTQ8.itemsize == 44 and ACTQ8.fields["qs"][1] == 12


def test_oracle_matches_stored_reference_outputs_on_lossless_activations(oracle, golden_dir):
    """Activations that Q8 represents exactly make the reference's compiled scalar path and its int8 path the
    same arithmetic up to fp32 summation order: the restated int8 path (both its fp32 lane-order mode and its
    float64 mode) must reproduce the reference build's stored outputs to 1e-5 relative L2."""
    g = np.load(golden_dir / "lossless_golden.npz")
    for i in range(int(g["n_cases"])):
        t, M, K, N, wseed, xseed = (int(v) for v in g[f"l{i}_meta"])
        w = synth.weights(t, K, N, seed=wseed, how="affine")
        x = synth.lossless_q8_activations(xseed, M, K)
        qa = oracle.quantize(x)
        assert np.array_equal((qa["qs"].astype(np.float32) * qa["d"][..., None]).reshape(M, K), x), "inputs are not lossless"
        ref = g[f"l{i}_ref_y"].astype(np.float64)
        for mode in (0, 1):
            y = oracle.gemm(x, w, t, M, K, N, mode=mode, threads=4).astype(np.float64)
            rel = np.linalg.norm(y - ref) / np.linalg.norm(ref)
            assert rel <= 1e-5, f"type {t} {M}x{K}x{N} mode {mode}: rel L2 {rel:.2e}"
            assert np.abs(y - ref).max() <= 1e-3 * np.sqrt(np.mean(ref ** 2))


@pytest.mark.skipif(not Reference.available(), reason="oracle/_ref not built (no reference checkout here)")
@pytest.mark.parametrize("t,M,K,N", [(GGMLType.Q4_0, 1, 4096, 4096), (GGMLType.Q4_K, 1, 4096, 14336), (GGMLType.Q6_K, 1, 14336, 4096),
                                     (GGMLType.Q8_0, 2, 4096, 1024), (GGMLType.Q4_K, 8, 4096, 14336)])
def test_oracle_matches_reference_build_live_at_benchmark_shapes(oracle, t, M, K, N):
    ref = Reference()
    ref.set_threads(4)
    w = synth.weights(t, K, N, seed=31 + int(t), how="affine")
    x = synth.lossless_q8_activations(32 + M, M, K)
    want = ref.matmul_rows(x, w, t, M, K, N).astype(np.float64)
    y = oracle.gemm(x, w, t, M, K, N, mode=1, threads=4).astype(np.float64)
    assert np.linalg.norm(y - want) / np.linalg.norm(want) <= 1e-5

"""Regenerates tests/golden/hotpath_golden.npz, lossless_golden.npz and other_types_golden.npz. Run where the reference checkout is present:

    make -C oracle all ref && python tests/golden/make_golden.py

The file pins two things for machines that have no reference checkout:
  * outputs of the reference's OWN code (oracle/_ref/libref_matmul.so, built
    from its sources): dequantize(), the scalar fp32-activation matmul_rows,
    and its fp16 conversions, on small seeded inputs; and (lossless_golden.npz) its
    matmul_rows on mid-size inputs whose activations Q8 represents exactly;
  * outputs of the C restatement of its int8 path (liboracle_q8.so) on the same
    inputs: quantized activation blocks, integer block sums, fp32 (lane-order)
    and float64 results, so that a later edit of the oracle cannot drift
    silently and GPU tests can compare against stored vectors.
Inputs are regenerated from seeds by tests.synth and are stored too.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tests import synth  # noqa: E402
from tests.oracle_lib import Oracle, Reference  # noqa: E402

CASES = [  # (type, how, M, K, N, seed)
    (2, "random", 2, 512, 8, 1), (2, "ref", 1, 512, 5, 2), (2, "affine", 1, 256, 4, 3),
    (8, "random", 2, 512, 8, 4), (8, "ref", 1, 512, 5, 5), (8, "affine", 1, 256, 4, 6),
    (12, "random", 2, 512, 8, 7), (12, "ref", 1, 768, 5, 8), (12, "affine", 1, 256, 4, 9),
    (14, "random", 2, 512, 8, 10), (14, "ref", 1, 768, 5, 11), (14, "affine", 1, 256, 4, 12),
]


def main():
    o, r = Oracle(), Reference()
    out = {}
    hs = np.concatenate([np.array([0x3C00, 0xC000, 0x0000, 0x7BFF, 0x0001, 0x8000, 0x7C00, 0x03FF, 0x0400], dtype=np.uint16),
                         synth.rng(77).integers(0, 0x7C00, size=1000, dtype=np.uint16)])
    out["fp16_bits"] = hs
    out["fp16_ref_f32"] = np.array([r.lib.ref_fp16_to_fp32(int(h)) for h in hs], dtype=np.float32)
    fs = np.concatenate([synth.normal_f32(78, 500, 1.0), synth.normal_f32(79, 500, 1e-5),
                         np.array([1.0, -2.0, 65504.0, 65520.0, 1e9, 6e-8, 2.98e-8, 0.1], dtype=np.float32)])
    out["f32_vals"] = fs
    out["f32_ref_fp16"] = np.array([r.lib.ref_fp32_to_fp16(float(v)) for v in fs], dtype=np.uint16)
    for i, (t, how, M, K, N, seed) in enumerate(CASES):
        w = synth.weights(t, K, N, seed=9000 + seed, how=how)
        x = synth.normal_f32(9100 + seed, (M, K))
        p = f"c{i}_"
        out[p + "meta"] = np.array([t, M, K, N], dtype=np.int64)
        out[p + "how"] = np.array(how)
        out[p + "w"] = w
        out[p + "x"] = x
        out[p + "ref_dequant"] = r.dequantize(w, t, K * N)
        out[p + "ref_scalar_y"] = r.matmul_rows(x, w, t, M, K, N)
        out[p + "act"] = o.quantize(x).view(np.uint8)
        out[p + "blocksums"] = o.blocksums(x, w, t, M, K, N)
        out[p + "y_f32"] = o.gemm(x, w, t, M, K, N, mode=0)
        out[p + "y_f64"] = o.gemm(x, w, t, M, K, N, mode=1)
    # expert-indexed calls (the reference's scalar fall-back path, src/matmul.cpp:469-499)
    t, K, N, n_total = 12, 256, 6, 5
    w = synth.weights(t, K, N * n_total, seed=9500, how="affine")
    idx = np.array([3, 0, 4], dtype=np.int32)
    x = synth.normal_f32(9501, (3, K))
    out["moe_w"], out["moe_idx"], out["moe_x"] = w, idx, x
    out["moe_meta"] = np.array([t, K, N, n_total], dtype=np.int64)
    out["moe_ref_scalar_idx"] = r.moe(x[0], w, t, idx, n_total, K, N, multi=False)
    out["moe_ref_scalar_multi"] = r.moe(x, w, t, idx, n_total, K, N, multi=True)
    out["moe_y_idx_f64"] = o.moe_gemv(x[0], w, t, idx, K, N, multi=False, mode=1)
    out["moe_y_multi_f64"] = o.moe_gemv(x, w, t, idx, K, N, multi=True, mode=1)
    path = Path(__file__).with_name("hotpath_golden.npz")
    np.savez_compressed(path, **out)
    print(path, path.stat().st_size, "bytes")
    lossless(r)
    other_types(r)


# Reference-build outputs for activations that Q8 represents exactly (tests.synth.lossless_q8_activations): with
# those the reference's scalar fp32-activation path and its int8 path are the same arithmetic up to fp32
# summation order, so implementations of the int8 path are held to these vectors at 1e-5. Weights and
# activations are regenerated from the stored seeds; only the reference's outputs are stored.
LOSSLESS_CASES = [  # (type, M, K, N, weight seed, activation seed)
    (2, 1, 4096, 512, 9601, 9701), (8, 1, 4096, 256, 9602, 9702), (12, 1, 4096, 1024, 9603, 9703),
    (14, 1, 4096, 512, 9604, 9704), (12, 8, 4096, 512, 9605, 9705), (12, 64, 2048, 256, 9606, 9706),
    (14, 64, 2048, 256, 9607, 9707), (2, 40, 1024, 128, 9608, 9708), (8, 40, 1024, 128, 9609, 9709),
    (12, 1, 14336, 128, 9610, 9710), (14, 1, 14336, 128, 9611, 9711),
    (6, 1, 4096, 512, 9612, 9712), (6, 40, 1024, 128, 9613, 9713),
]


def lossless(r):
    out = {"n_cases": np.array(len(LOSSLESS_CASES))}
    for i, (t, M, K, N, ws, xs) in enumerate(LOSSLESS_CASES):
        w = synth.weights(t, K, N, seed=ws, how="affine")
        x = synth.lossless_q8_activations(xs, M, K)
        out[f"l{i}_meta"] = np.array([t, M, K, N, ws, xs], dtype=np.int64)
        out[f"l{i}_ref_y"] = r.matmul_rows(x, w, t, M, K, N)
    path = Path(__file__).with_name("lossless_golden.npz")
    np.savez_compressed(path, **out)
    print(path, path.stat().st_size, "bytes")


# Reference-build outputs for the weight types outside the int8 path and for dequantize() of every type
# (other_types_golden.npz): weight bytes, dequantized values, and matmul_rows (scalar path, fp32 activations).
def other_types(r):
    K, N, M = 512, 24, 3
    out = {"K": np.array(K), "x": synth.normal_f32(8801, (M, K))}
    for t in (0, 1, 30, 6, 10, 11, 13, 2, 8, 12, 14):
        w = synth.other_type_weights(t, K, N, seed=8810 + t) if t in (0, 1, 30, 6, 10, 11, 13) else synth.weights(t, K, N, seed=8810 + t, how="random")
        w = np.ascontiguousarray(w)
        out[f"w_{t}"] = w
        out[f"deq_{t}"] = r.dequantize(w, t, N * K)
        if t in (0, 1, 30, 6, 10, 11, 13):
            out[f"y_{t}"] = r.matmul_rows(out["x"], w, t, M, K, N)
    path = Path(__file__).with_name("other_types_golden.npz")
    np.savez_compressed(path, **out)
    print(path, path.stat().st_size, "bytes")


if __name__ == "__main__":
    main()

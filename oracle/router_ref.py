"""CPU restatement of the reference's expert selection for one token - TEST INFRASTRUCTURE ONLY.

Follows Laplace src/arch_gemma4.cpp:547-565 operation for operation in fp32: softmax over the router logits
(running maximum, exp(l - max) summed in index order, division by the sum), then top_k times the largest
remaining probability (strict '>' comparison: the first index wins among equal values; a selected entry is
replaced by -1e30), then the selected probabilities divided by their sum (added in selection order). The combine
weight of a pair is top_w * down_scale[expert] (:634-638). Only tests and the benchmark's checker import this;
the product never does.

Parity pin: the reference holds no vectors for this block; the restatement is anchored by the properties its code
implies (weights sum to 1, indices distinct, ordering by probability, first-index tie rule), which
tests/test_moe_router.py checks on the CPU.
"""
import numpy as np


def route(logits: np.ndarray, top_k: int):
    """logits [T, E] float32 -> (top_idx [T, top_k] int32, top_w [T, top_k] float32)."""
    logits = np.asarray(logits, dtype=np.float32)
    T, E = logits.shape
    top_idx = np.zeros((T, top_k), dtype=np.int32)
    top_w = np.zeros((T, top_k), dtype=np.float32)
    f32 = np.float32
    for t in range(T):
        l = logits[t].copy()
        maxl = l[0]
        for e in range(1, E):
            if l[e] > maxl:
                maxl = l[e]
        p = np.exp((l - maxl).astype(np.float32)).astype(np.float32)      # element-wise, as std::exp(float)
        suml = f32(0.0)
        for e in range(E):
            suml = f32(suml + p[e])
        p = (p / suml).astype(np.float32)
        for k in range(top_k):
            best = 0
            for e in range(1, E):
                if p[e] > p[best]:
                    best = e
            top_idx[t, k] = best
            top_w[t, k] = p[best]
            p[best] = f32(-1e30)
        wsum = f32(0.0)
        for k in range(top_k):
            wsum = f32(wsum + top_w[t, k])
        for k in range(top_k):
            top_w[t, k] = f32(top_w[t, k] / wsum)
    return top_idx, top_w

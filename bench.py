#!/usr/bin/env python3
"""Benchmark of the packed polynomial transcendental hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (one "step"): the isolated FP16 function sweep at the HBM endpoint, N = 2^28 elements per function
and per GPU -- polynomial sigmoid D3, tanh D4, SiLU D3, fractional exp2 (hinge) and paired sin/cos (D5/D6
half turn) -- on seeded synthetic inputs already resident in HBM.  `value` is elements/s over the whole job
(all functions, all GPUs).  Every function is also run in its native special-function-unit form and, at the
L2-resident endpoint N = 2^20, in both forms; those numbers, the SwiGLU and B3 lines ride along in
`functions` / `extras`.  `e2e` is the same sweep through the public `spline_ops` API from pinned HOST buffers
with both PCIe copies inside the timed region.  Prints ONE JSON line on rank 0.

`--impl reference` times the CPU path instead: this repository's exact packed-arithmetic emulator (the port of
the reference's programs used as the parity oracle) with all host threads on a bounded sample of the sweep.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

N_HBM = 1 << 28
N_L2 = 1 << 20
SEED = 1234
NOMINAL_HBM_GBS = 8000.0
# dram__bytes_read + dram__bytes_write of the sigmoid kernel per 2^28-element launch, scaled from the 2^26 capture
SIGMOID_TRAFFIC_BYTES_PER_LAUNCH = int(4 * 134.225152e6 + (4 * 134.217728e6 - (134.217728e6 - 82.393088e6)))


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


# ------------------------------------------------------------------------------------ CPU arm

def cpu_sample_inputs(n):
    import numpy as np
    rng = np.random.default_rng(SEED)
    u8 = rng.uniform(-8, 8, n).astype(np.float16).view(np.uint16)
    frac = rng.uniform(0, 1, n).astype(np.float16).view(np.uint16)
    ang = rng.uniform(-math.pi, math.pi, n).astype(np.float32)
    return u8, frac, ang


def cpu_sweep(oracle, inputs):
    """One pass of the sweep on the CPU emulator; returns elements processed."""
    u8, frac, ang = inputs
    oracle.unary(oracle.find_program("SIGMOID_FWD_D3", 0), u8)
    oracle.unary(oracle.find_program("TANH_FWD_D4", 0), u8)
    oracle.unary(oracle.find_program("SWISH_FWD_D3", 0), u8)
    oracle.exp2_hinge(frac, 0)
    oracle.sincos_packed("d5_d6_half_turn_fp16", ang)
    return 5 * u8.size


def cpu_baseline(sample_elems=1 << 22, budget_s=12.0):
    from oracle import oracle
    oracle.build()
    threads = oracle.set_threads(os.cpu_count() or 1)     # torchrun exports OMP_NUM_THREADS=1
    inputs = cpu_sample_inputs(sample_elems)
    cpu_sweep(oracle, inputs)
    t0 = time.perf_counter()
    done, passes = 0, 0
    while time.perf_counter() - t0 < budget_s and passes < 8:
        done += cpu_sweep(oracle, inputs)
        passes += 1
    dt = time.perf_counter() - t0
    return {"value": done / dt, "unit": "elements/s", "cores": threads, "kind": "port",
            "sample": f"{passes} passes of the 5-function sweep at 2^{int(math.log2(sample_elems))} elements per "
                      f"function, exact packed-FMA emulator (OpenMP, all host threads)"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle
    oracle.build()
    threads = oracle.set_threads(os.cpu_count() or 1)     # torchrun exports OMP_NUM_THREADS=1
    n = 1 << 21
    inputs = cpu_sample_inputs(n)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_sweep(oracle, inputs)
    t0 = time.perf_counter()
    done = 0
    for _ in range(args.steps):
        done += cpu_sweep(oracle, inputs)
    dt = time.perf_counter() - t0
    value = done / dt
    line = {
        "impl": "reference", "metric": "elements_per_s_fp16_function_sweep", "value": value, "unit": "elements/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "elements/s", "cores": threads, "kind": "port",
                         "sample": f"each step = the 5-function sweep at 2^21 elements per function (bounded "
                                   f"sample of the 2^28 workload), exact packed-FMA emulator, all host threads"},
        "e2e": {"value": value, "unit": "elements/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus):
    return {"workload": "BASELINE config[1]: isolated FP16 function sweep, HBM endpoint N=2^28 per function "
                        "(sigmoid D3, tanh D4, SiLU D3, exp2 hinge, sin/cos D5/D6), polynomial vs native SFU",
            "elements_per_function_per_gpu": N_HBM, "functions": 5, "sharding": f"{n_gpus} x independent element ranges",
            "l2": "inputs of 512 MiB..1 GiB per function exceed the 126 MB L2; no flush needed"}


# ------------------------------------------------------------------------------------ GPU arm

class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            self.thread.join(timeout=2)
        return False

    def summary(self):
        sm, reasons, sm_max = [], set(), None
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                sm_max = float(r[2])
            except (ValueError, IndexError):
                continue
            names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
            for name, flag in zip(names, r[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": sm_max, "reasons": sorted(reasons),
                "samples": len(sm)}


def make_inputs(torch, device, n, rank):
    """Seeded per-rank inputs: the global stream of rank r starts at element r*n of the same generator."""
    g = torch.Generator(device=device)
    g.manual_seed(SEED + 7919 * rank)
    u8 = (torch.rand(n, device=device, generator=g) * 16 - 8).to(torch.float16)
    frac = torch.rand(n, device=device, generator=g).to(torch.float16)
    ang = (torch.rand(n, device=device, generator=g) * (2 * math.pi) - math.pi).contiguous()
    return u8, frac, ang


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist
    from fast_polynomial_transcendentals_b200 import _lib, spline_ops
    from fast_polynomial_transcendentals_b200.pipeline import HostPipeline

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    from fast_polynomial_transcendentals_b200.pipeline import bind_host_thread_to_device_node
    all_cpus = os.sched_getaffinity(0)
    host_binding = bind_host_thread_to_device_node(local) if world > 1 else None   # pinned buffers local to the GPU
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    lib = _lib.load()
    ctx = {"stream": torch.cuda.current_stream().cuda_stream}
    S = lambda: ctx["stream"]  # kernels read the launch stream at call time (graph capture swaps it)
    hbm_peak, _, peak_kind = measured_peaks()

    u8, frac, ang = make_inputs(torch, device, N_HBM, rank)
    out16 = torch.empty(N_HBM, dtype=torch.float16, device=device)
    out_sc = torch.empty(2, N_HBM, dtype=torch.float16, device=device)

    def k_unary(fn, degree, x, out, n):
        return lambda: _lib.check("fpt_unary", lib.fpt_unary(out.data_ptr(), x.data_ptr(), n, fn, 0, degree, 0, 0, S()))

    def k_exp2(variant, x, out, n):
        return lambda: _lib.check("fpt_exp2_fraction", lib.fpt_exp2_fraction(out.data_ptr(), x.data_ptr(), n, variant, 1, S()))

    def k_sincos(variant, x, out, n):
        return lambda: _lib.check("fpt_sincos", lib.fpt_sincos(out.data_ptr(), x.data_ptr(), n, variant, 0, S()))

    def sweep(n, poly):
        o16, osc = out16[:n], out_sc.view(-1)[: 2 * n]
        return [
            ("sigmoid", 4, k_unary(0, 3 if poly else 0, u8[:n], o16, n)),
            ("tanh", 4, k_unary(1, 4 if poly else 0, u8[:n], o16, n)),
            ("silu", 4, k_unary(2, 3 if poly else 0, u8[:n], o16, n)),
            ("exp2", 4, k_exp2(1 if poly else 0, frac[:n], o16, n)),
            ("sincos", 8, k_sincos(3 if poly else 10, ang[:n], osc, n)),
        ]

    def barrier(collective):
        if collective and world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def time_sweep(kernels, steps, warmup, collective=False):
        """Per-kernel CUDA-event durations inside a back-to-back loop; returns (total ms, {name: avg ms})."""
        for _ in range(warmup):
            for _, _, k in kernels:
                k()
        barrier(collective)
        marks = [[torch.cuda.Event(enable_timing=True) for _ in range(len(kernels) + 1)] for _ in range(steps)]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for s in range(steps):
            marks[s][0].record()
            for i, (_, _, k) in enumerate(kernels):
                k()
                marks[s][i + 1].record()
        stop.record()
        barrier(collective)
        total = start.elapsed_time(stop)
        per = {}
        for i, (name, _, _) in enumerate(kernels):
            per[name] = sum(marks[s][i].elapsed_time(marks[s][i + 1]) for s in range(steps)) / steps
        return total, per

    def time_graph(kernels, launches=20, rounds=15):
        """Kernel-side time of small launches: every kernel is captured `launches` times into its own CUDA graph and
        the replay is timed, so that host launch cost stays outside the measurement.  Returns {name: avg ms}."""
        side = torch.cuda.Stream(device)
        per = {}
        for name, _, k in kernels:
            saved = ctx["stream"]
            ctx["stream"] = side.cuda_stream
            try:
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    for _ in range(3):
                        k()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=side):
                        for _ in range(launches):
                            k()
                torch.cuda.current_stream().wait_stream(side)
            finally:
                ctx["stream"] = saved
            graph.replay()
            torch.cuda.synchronize()
            times = []
            for _ in range(rounds):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                graph.replay()
                b.record()
                torch.cuda.synchronize()
                times.append(a.elapsed_time(b) / launches)
            times.sort()
            per[name] = times[len(times) // 2]
        return per

    # ---- headline: polynomial sweep at the HBM endpoint, with clock sampling
    poly_hbm = sweep(N_HBM, True)
    with ClockSampler(local) as clocks:
        total_ms, per_poly = time_sweep(poly_hbm, args.steps, args.warmup, collective=True)
    if world > 1:
        t = torch.tensor([total_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    elements_per_step = 5 * N_HBM * world
    value = elements_per_step * args.steps / (total_ms * 1e-3)
    gpu_launches = len(poly_hbm) * args.steps * world   # whole job: every rank launches the same five kernels per step

    # ---- e2e through the public API with host buffers: every rank its own sweep, whole-job value = all ranks'
    # elements over the slowest rank's time
    if world > 1:
        dist.barrier()
    e2e = bench_e2e(torch, spline_ops, HostPipeline, device)
    if host_binding:
        e2e["host_binding"] = host_binding
        os.sched_setaffinity(0, all_cpus)      # the CPU legs below use every core again
    if world > 1:
        t = torch.tensor([e2e["ms_per_step"]], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e["ms_per_step"] = float(t.item())
        e2e["value"] = world * 5 * e2e["elements_per_function"] / (e2e["ms_per_step"] * 1e-3)
        e2e["h2d_bytes_per_step"] *= world
        e2e["d2h_bytes_per_step"] *= world
        e2e["path"] += f"; {world} ranks at once, slowest rank's time"

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ---- rank 0 only: native twins, L2 endpoint, SwiGLU / B3 lines, e2e, CPU baseline
    _, per_native = time_sweep(sweep(N_HBM, False), max(3, args.steps // 2), 3)
    functions = {}
    for name, bytes_per, _ in poly_hbm:
        gbs = bytes_per * N_HBM / (per_poly[name] * 1e-3) / 1e9
        functions[name] = {
            "poly_elements_per_s": N_HBM / (per_poly[name] * 1e-3), "native_elements_per_s": N_HBM / (per_native[name] * 1e-3),
            "poly_ms": per_poly[name], "native_ms": per_native[name], "poly_gbs": gbs,
            "frac_of_measured_hbm": gbs / hbm_peak, "frac_of_nominal_8tbs": gbs / NOMINAL_HBM_GBS,
            "algorithmic_bytes_per_element": bytes_per,
        }
    l2 = {}
    l2_poly = time_graph(sweep(N_L2, True))
    l2_native = time_graph(sweep(N_L2, False))
    for name in l2_poly:
        l2[name] = {"poly_us": l2_poly[name] * 1e3, "native_us": l2_native[name] * 1e3,
                    "speedup_vs_native": l2_native[name] / l2_poly[name]}
    # ALU-bound probe: 16 evaluations per load at the L2 endpoint
    alu = {}
    for name, fn, deg in (("sigmoid", 0, 3), ("tanh", 1, 4), ("silu", 2, 3)):
        ks = [(kind, 4, (lambda d=d: _lib.check("fpt_unary_repeat", lib.fpt_unary_repeat(
            out16.data_ptr(), u8.data_ptr(), N_L2, fn, 0, d, 0, 0, 16, S())))) for kind, d in (("poly", deg), ("native", 0))]
        t = time_graph(ks)
        alu[name] = {"poly_us": t["poly"] * 1e3, "native_us": t["native"] * 1e3, "speedup_vs_native": t["native"] / t["poly"]}
    ks = [(kind, 4, (lambda v=v: _lib.check("fpt_exp2_fraction", lib.fpt_exp2_fraction(
        out16.data_ptr(), frac.data_ptr(), N_L2, v, 16, S())))) for kind, v in (("poly", 1), ("native", 0))]
    t = time_graph(ks)
    alu["exp2"] = {"poly_us": t["poly"] * 1e3, "native_us": t["native"] * 1e3, "speedup_vs_native": t["native"] / t["poly"]}
    ks = [(kind, 8, (lambda v=v: _lib.check("fpt_sincos", lib.fpt_sincos(
        out_sc.data_ptr(), ang.data_ptr(), N_L2, v, 16, S())))) for kind, v in (("poly", 3), ("native", 10))]
    t = time_graph(ks)
    alu["sincos"] = {"poly_us": t["poly"] * 1e3, "native_us": t["native"] * 1e3, "speedup_vs_native": t["native"] / t["poly"]}

    extras = {"l2_resident_2^20": l2, "alu_bound_16_evals_per_load_2^20": alu,
              "l2_timing": "CUDA-graph replay of 20 launches per kernel, median of 15 replays (no host launch cost)"}
    del u8, frac, ang, out16, out_sc
    torch.cuda.empty_cache()
    extras["swiglu_bf16"] = bench_swiglu(torch, lib, _lib, device, S, hbm_peak, time_sweep)
    extras["b3_config1"] = bench_b3(torch, lib, _lib, device, S, time_graph)
    extras["attention_fwd_bf16"] = bench_attention(torch, lib, _lib, device, S, time_sweep)

    cpu = cpu_baseline()
    dominant = functions["sigmoid"]
    line = {
        "metric": "elements_per_s_fp16_function_sweep", "value": value, "unit": "elements/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": workload_config(world),
        "roofline": {"bound": "hbm", "achieved": dominant["poly_gbs"], "peak": hbm_peak, "unit": "GB/s",
                     "frac": dominant["poly_gbs"] / hbm_peak, "traffic": SIGMOID_TRAFFIC_BYTES_PER_LAUNCH,
                     "traffic_source": "ncu capture at 2^26 elements (dram read 134.23 MB, write 82.39 MB = algorithmic minus "
                                       "what stays dirty in L2), reads scaled x4, the L2-resident remainder kept constant",
                     "algorithmic_bytes": 4 * N_HBM, "peak_kind": f"of {peak_kind}",
                     "kernel": "stream_kernel<UnaryOp<fp16, ODD_HALF, 3>> (sigmoid D3), 4 algorithmic bytes per element "
                               "x 2^28 elements per launch", "frac_of_nominal_8tbs": dominant["poly_gbs"] / NOMINAL_HBM_GBS},
        "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": gpu_launches, "clocks": clocks.summary(),
        "functions": functions, "extras": extras,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def bench_swiglu(torch, lib, _lib, device, S, hbm_peak, time_sweep):
    out = {}
    g = torch.Generator(device=device)
    g.manual_seed(SEED)
    for name, rows, hidden in (("B1_dense_16384x14336", 16384, 14336), ("B4_routed_131072x1408", 131072, 1408)):
        packed = (torch.randn(rows, 2 * hidden, device=device, generator=g) * 1.5).to(torch.bfloat16)
        gate, up = packed[:, :hidden].contiguous(), packed[:, hidden:].contiguous()
        o = torch.empty_like(gate)
        n = rows * hidden
        ks = [
            ("flat_poly", 6, lambda: _lib.check("fpt_swish_mul", lib.fpt_swish_mul(o.data_ptr(), gate.data_ptr(), up.data_ptr(), n, 3, 1, 0, S()))),
            ("flat_native", 6, lambda: _lib.check("fpt_swish_mul", lib.fpt_swish_mul(o.data_ptr(), gate.data_ptr(), up.data_ptr(), n, 0, 1, 0, S()))),
            ("packed_poly", 6, lambda: _lib.check("fpt_swish_mul_packed", lib.fpt_swish_mul_packed(o.data_ptr(), packed.data_ptr(), rows, hidden, 3, 1, 0, S()))),
            ("packed_native", 6, lambda: _lib.check("fpt_swish_mul_packed", lib.fpt_swish_mul_packed(o.data_ptr(), packed.data_ptr(), rows, hidden, 0, 1, 0, S()))),
        ]
        _, t = time_sweep(ks, 10, 3)
        out[name] = {k: {"ms": v, "elements_per_s": n / (v * 1e-3), "gbs": 6 * n / (v * 1e-3) / 1e9,
                         "frac_of_measured_hbm": 6 * n / (v * 1e-3) / 1e9 / hbm_peak} for k, v in t.items()}
        del packed, gate, up, o
    torch.cuda.empty_cache()
    return out


def bench_b3(torch, lib, _lib, device, S, time_graph):
    n = 1 << 24
    g = torch.Generator(device=device)
    g.manual_seed(SEED)
    x = (torch.rand(n, device=device, generator=g) * 32 - 16).to(torch.bfloat16)
    o = torch.empty_like(x)
    ks = [("b3_direct_poly", 4, lambda: _lib.check("fpt_b3_sigmoid_direct", lib.fpt_b3_sigmoid_direct(o.data_ptr(), None, x.data_ptr(), n, 0, 12, S()))),
          ("sigmoid_native", 4, lambda: _lib.check("fpt_unary", lib.fpt_unary(o.data_ptr(), x.data_ptr(), n, 0, 0, 0, 1, 0, S())))]
    t = time_graph(ks)
    return {k: {"us": v * 1e3, "elements_per_s": n / (v * 1e-3)} for k, v in t.items()} | {"n": n, "regime": "64 MiB touched: L2 resident"}


def bench_attention(torch, lib, _lib, device, S, time_sweep):
    """Configurations 4 and 5 of the baseline (plus the reference's published S=4096 shape), forward only."""
    import ctypes
    _, tensor_peak, _ = measured_peaks()
    out = {}
    g = torch.Generator(device=device)
    g.manual_seed(SEED)
    D = 128
    # last field: exp2 routing frequency (0 = every exponential on the SFU; f = four of every f keys on the FMA pipe)
    shapes = (("config4_causal_gqa_softcap50_tanhD4_B4_S8192_Hq32_Hkv8", 4, 8192, 32, 8, 0, 1, 50.0, 12, 0),
              ("config5_sigmoid_direct_B2_S16384_H32", 2, 16384, 32, 32, 1, 0, 0.0, 14, 0),
              ("published_shape_softcap30_B1_S4096_Hq32_Hkv8", 1, 4096, 32, 8, 0, 1, 30.0, 12, 0),
              ("published_shape_sigmoid_B1_S4096_Hq32_Hkv8_causal", 1, 4096, 32, 8, 1, 1, 0.0, 12, 0),
              ("control_plain_softmax_B4_S8192_Hq32_Hkv8_causal", 4, 8192, 32, 8, 2, 1, 0.0, 12, 0),
              ("routed_exp2_d3_freq32_softmax_B4_S8192_Hq32_Hkv8_causal", 4, 8192, 32, 8, 2, 1, 0.0, 12, 32),
              ("routed_exp2_d3_freq12_softmax_B4_S8192_Hq32_Hkv8_causal", 4, 8192, 32, 8, 2, 1, 0.0, 12, 12))
    for name, B, Sq, Hq, Hk, mode, causal, cap, log2_n, route in shapes:
        q = torch.randn(B, Sq, Hq, D, device=device, generator=g).to(torch.bfloat16)
        k = torch.randn(B, Sq, Hk, D, device=device, generator=g).to(torch.bfloat16)
        v = torch.randn(B, Sq, Hk, D, device=device, generator=g).to(torch.bfloat16)
        o = torch.empty_like(q)
        lse = torch.empty(B, Hq, Sq, device=device)
        status = torch.zeros(1, dtype=torch.int32, device=device)
        arr = lambda t: (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
        sq, sk, sv, so = arr(q), arr(k), arr(v), arr(o)
        ks = [("attn", 0, lambda: _lib.check("fpt_attention_fwd_routed", lib.fpt_attention_fwd_routed(
            o.data_ptr(), lse.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), B, Sq, Hq, Hk, D, sq, sk, sv, so, mode,
            causal, 1.0 / math.sqrt(D), cap, log2_n, 0, route, status.data_ptr(), S())))]
        _, t = time_sweep(ks, 5, 2)
        if int(status.item()) != 0:
            raise RuntimeError(f"attention kernel reported status {int(status.item()) & 0xffffffff:#x}")
        flops = 4.0 * B * Hq * Sq * Sq * D * (0.5 if causal else 1.0)
        tf = flops / (t["attn"] * 1e-3) / 1e12
        out[name] = {"ms": t["attn"], "tflops": tf, "frac_of_measured_bf16_peak": tf / tensor_peak,
                     "flops_convention": "4*B*Hq*S^2*D, halved when causal"}
        if route == 0 and name.startswith(("config", "control")):
            # backward of the same shape: dQ and dK/dV kernels plus the delta pre-pass, forward output as input
            dout = torch.randn(B, Sq, Hq, D, device=device, generator=g).to(torch.bfloat16)
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            need = int(lib.fpt_attention_bwd_workspace_bytes(B, Sq, Hq))
            workspace = torch.empty(need, dtype=torch.uint8, device=device)
            sdo = arr(dout)
            kb = [("bwd", 0, lambda: _lib.check("fpt_attention_bwd", lib.fpt_attention_bwd(
                dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                o.data_ptr(), lse.data_ptr(), workspace.data_ptr(), need, B, Sq, Hq, Hk, D, sq, sk, sv, so, sdo, mode, causal,
                1.0 / math.sqrt(D), cap, log2_n, 0, status.data_ptr(), S())))]
            _, tb = time_sweep(kb, 3, 2)
            if int(status.item()) != 0:
                raise RuntimeError(f"attention backward reported status {int(status.item()) & 0xffffffff:#x}")
            tfb = 2.5 * flops / (tb["bwd"] * 1e-3) / 1e12
            out[name]["backward"] = {"ms": tb["bwd"], "tflops": tfb, "frac_of_measured_bf16_peak": tfb / tensor_peak,
                                     "flops_convention": "5 matrix products = 2.5 x the forward count (7 are executed: S and "
                                                         "dP are recomputed in the dQ and in the dK/dV kernel)"}
            del dout, dq, dk, dv, workspace
        del q, k, v, o, lse
    torch.cuda.empty_cache()
    return out


def bench_e2e(torch, spline_ops, HostPipeline, device):
    """The sweep from pinned host memory through spline_ops: chunked H2D -> kernel -> D2H on three streams."""
    n = 1 << 26          # per function; bounded so that the default run stays within minutes
    chunk = 1 << 23
    g = torch.Generator()
    g.manual_seed(SEED)
    host_u8 = (torch.rand(n, generator=g) * 16 - 8).to(torch.float16).pin_memory()
    host_frac = torch.rand(n, generator=g).to(torch.float16).pin_memory()
    host_ang = (torch.rand(n, generator=g) * (2 * math.pi) - math.pi).pin_memory()
    host_out = torch.empty(n, dtype=torch.float16).pin_memory()
    host_sc = torch.empty(2 * n, dtype=torch.float16).pin_memory()
    unary_pipe = HostPipeline(device, [(torch.float16, 1)], [(torch.float16, 1)], chunk)
    # sin/cos keeps the two planes of a chunk adjacent in the device buffer; the host copy de-interleaves per chunk
    sincos_pipe = HostPipeline(device, [(torch.float32, 1)], [(torch.float16, 2)], chunk)

    def run_once():
        launches = 0
        for op, src in ((spline_ops.sigmoid_fwd_d3, host_u8), (spline_ops.tanh_fwd_d4, host_u8),
                        (spline_ops.swish_fwd_d3, host_u8), (spline_ops.exp2_fraction, host_frac)):
            def fn(ins, outs, m, op=op):
                outs[0].copy_(op(ins[0]))
            launches += 2 * unary_pipe.run(fn, [src], [host_out], n)
        def fn_sc(ins, outs, m):
            outs[0].copy_(spline_ops.sincos_d5_d6_half_turn_fp16(ins[0]).view(-1))
        launches += 2 * sincos_pipe.run(fn_sc, [host_ang], [host_sc], n)
        unary_pipe.synchronize()
        sincos_pipe.synchronize()
        return launches

    run_once()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    reps = 2
    for _ in range(reps):
        run_once()
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / reps
    h2d = 4 * n * 2 + n * 4
    d2h = 4 * n * 2 + 2 * n * 2
    return {"value": 5 * n / dt, "unit": "elements/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "elements_per_function": n, "ms_per_step": dt * 1e3,
            "path": "spline_ops.* on pinned host buffers, 2^23-element chunks, H2D / kernel / D2H on three streams; "
                    "sin/cos results are returned chunk by chunk as [cos | sin] blocks"}


def run_profile_case(args):
    """A small fixed case of ONE kernel for profiler captures: `--profile-case NAME --profile-n ELEMENTS`."""
    import torch
    from fast_polynomial_transcendentals_b200 import _lib
    lib = _lib.load()
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    stream = torch.cuda.current_stream().cuda_stream
    n = args.profile_n
    g = torch.Generator(device=device)
    g.manual_seed(SEED)
    case = args.profile_case
    if case in ("sigmoid", "tanh", "silu", "sigmoid_native"):
        x = (torch.rand(n, device=device, generator=g) * 16 - 8).to(torch.float16)
        o = torch.empty_like(x)
        fn, deg = {"sigmoid": (0, 3), "tanh": (1, 4), "silu": (2, 3), "sigmoid_native": (0, 0)}[case]
        run = lambda: _lib.check("fpt_unary", lib.fpt_unary(o.data_ptr(), x.data_ptr(), n, fn, 0, deg, 0, 0, stream))
    elif case.startswith("rep16_"):
        # ALU-bound probes at an L2-resident size (use --profile-n 1048576): 16 evaluations per loaded element, polynomial
        # and native twin of each function, to read FMA-pipe against XU-pipe (MUFU) use
        name = case[len("rep16_"):]
        if name in ("sigmoid", "tanh", "silu", "sigmoid_native", "tanh_native", "silu_native"):
            x = (torch.rand(n, device=device, generator=g) * 16 - 8).to(torch.float16)
            o = torch.empty_like(x)
            fn, deg = {"sigmoid": (0, 3), "tanh": (1, 4), "silu": (2, 3), "sigmoid_native": (0, 0), "tanh_native": (1, 0),
                       "silu_native": (2, 0)}[name]
            run = lambda: _lib.check("fpt_unary_repeat", lib.fpt_unary_repeat(o.data_ptr(), x.data_ptr(), n, fn, 0, deg, 0, 0, 16, stream))
        elif name in ("exp2", "exp2_native"):
            x = torch.rand(n, device=device, generator=g).to(torch.float16).clamp_(max=0.9995)
            o = torch.empty_like(x)
            variant = 1 if name == "exp2" else 0
            run = lambda: _lib.check("fpt_exp2_fraction", lib.fpt_exp2_fraction(o.data_ptr(), x.data_ptr(), n, variant, 16, stream))
        elif name in ("sincos", "sincos_native"):
            x = torch.rand(n, device=device, generator=g) * (2 * math.pi) - math.pi
            o = torch.empty(2, n, dtype=torch.float16, device=device)
            variant = 3 if name == "sincos" else 10
            run = lambda: _lib.check("fpt_sincos", lib.fpt_sincos(o.data_ptr(), x.data_ptr(), n, variant, 16, stream))
        else:
            raise SystemExit(f"unknown profile case {case}")
    elif case == "sincos":
        x = torch.rand(n, device=device, generator=g) * (2 * math.pi) - math.pi
        o = torch.empty(2, n, dtype=torch.float16, device=device)
        run = lambda: _lib.check("fpt_sincos", lib.fpt_sincos(o.data_ptr(), x.data_ptr(), n, 3, 0, stream))
    elif case in ("swiglu", "swiglu_packed"):
        hidden = 1408
        rows = n // hidden
        packed = (torch.randn(rows, 2 * hidden, device=device, generator=g) * 1.5).to(torch.bfloat16)
        gate, up = packed[:, :hidden].contiguous(), packed[:, hidden:].contiguous()
        o = torch.empty_like(gate)
        if case == "swiglu":
            run = lambda: _lib.check("fpt_swish_mul", lib.fpt_swish_mul(o.data_ptr(), gate.data_ptr(), up.data_ptr(), rows * hidden, 3, 1, 0, stream))
        else:
            run = lambda: _lib.check("fpt_swish_mul_packed", lib.fpt_swish_mul_packed(o.data_ptr(), packed.data_ptr(), rows, hidden, 3, 1, 0, stream))
    elif case in ("attn_softcap", "attn_sigmoid", "attn_softmax", "attn_softmax_full", "attn_softcap_full"):
        import ctypes
        B, S, Hq, Hk, D = 1, n, 32, 8, 128      # --profile-n is the sequence length here
        mode = {"attn_softcap": 0, "attn_sigmoid": 1, "attn_softmax": 2, "attn_softmax_full": 2, "attn_softcap_full": 0}[case]
        causal = 0 if mode == 1 or case.endswith("_full") else 1   # "_full": every key tile, no mask
        q = torch.randn(B, S, Hq, D, device=device, generator=g).to(torch.bfloat16)
        k = torch.randn(B, S, Hk, D, device=device, generator=g).to(torch.bfloat16)
        v = torch.randn(B, S, Hk, D, device=device, generator=g).to(torch.bfloat16)
        o = torch.empty_like(q)
        lse = torch.empty(B, Hq, S, device=device)
        status = torch.zeros(1, dtype=torch.int32, device=device)
        arr = lambda t: (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
        run = lambda: _lib.check("fpt_attention_fwd", lib.fpt_attention_fwd(
            o.data_ptr(), lse.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), B, S, Hq, Hk, D, arr(q), arr(k), arr(v),
            arr(o), mode, causal, 1.0 / math.sqrt(D), 50.0, 12, status.data_ptr(), stream))
    elif case in ("attn_bwd_softmax", "attn_bwd_softcap", "attn_bwd_sigmoid"):
        import ctypes
        B, S, Hq, Hk, D = 1, n, 32, 8, 128      # --profile-n is the sequence length; no mask
        mode = {"attn_bwd_softcap": 0, "attn_bwd_sigmoid": 1, "attn_bwd_softmax": 2}[case]
        mk = lambda h: torch.randn(B, S, h, D, device=device, generator=g).to(torch.bfloat16)
        q, k, v, dout = mk(Hq), mk(Hk), mk(Hk), mk(Hq)
        o = torch.empty_like(q)
        lse = torch.empty(B, Hq, S, device=device)
        status = torch.zeros(1, dtype=torch.int32, device=device)
        arr = lambda t: (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
        _lib.check("fpt_attention_fwd", lib.fpt_attention_fwd(
            o.data_ptr(), lse.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), B, S, Hq, Hk, D, arr(q), arr(k), arr(v),
            arr(o), mode, 0, 1.0 / math.sqrt(D), 50.0, 12, status.data_ptr(), stream))
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        need = int(lib.fpt_attention_bwd_workspace_bytes(B, S, Hq))
        workspace = torch.empty(need, dtype=torch.uint8, device=device)
        run = lambda: _lib.check("fpt_attention_bwd", lib.fpt_attention_bwd(
            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
            lse.data_ptr(), workspace.data_ptr(), need, B, S, Hq, Hk, D, arr(q), arr(k), arr(v), arr(o), arr(dout), mode, 0,
            1.0 / math.sqrt(D), 50.0, 12, 0, status.data_ptr(), stream))
    else:
        raise SystemExit(f"unknown profile case {case}")
    for _ in range(args.steps):
        run()
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": case, "n": n, "launches": args.steps}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--profile-case", default=None, help="run only one small kernel case (for ncu captures)")
    ap.add_argument("--profile-n", type=int, default=1 << 26)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.profile_case:
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()

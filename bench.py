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

`--impl reference` times the reference's CPU path instead, on the host cores: (i) PyTorch's native CPU functions on
the same seeded inputs with every host thread, and (ii) the reference's own vectorised packed-arithmetic replays
(its fitters' split-rounded Horner in numpy float16, its polynomial sin/cos in torch), each step a bounded sample of
2^24 elements per function.  The exact single-rounding emulator this repository uses as its parity oracle is timed
beside them as a third leg and reported, not counted into the value.

`--compare-reference-kernels` (a separate invocation, 1 GPU) times this library's kernels next to the reference's own
kernels where those have been compiled into oracle/_ref (`make -C oracle ref`), same inputs, same protocol.
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


def measured_sustained_tflops():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text()).get("bf16_tflops_sustained", 1400.0))
    return 1400.0


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


# ------------------------------------------------------------------------------------ CPU arm

CPU_FUNCTIONS = ("sigmoid", "tanh", "silu", "exp2", "sincos")


def cpu_sample_inputs(n):
    import numpy as np
    rng = np.random.default_rng(SEED)
    u8 = rng.uniform(-8, 8, n).astype(np.float16)
    frac = rng.uniform(0, 1, n).astype(np.float16)
    ang = rng.uniform(-math.pi, math.pi, n).astype(np.float32)
    return u8, frac, ang


def host_threads():
    """Every core this process may use (torchrun exports OMP_NUM_THREADS=1, which the CPU legs override)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


class CpuLegs:
    """The three CPU legs over one set of seeded inputs; every leg returns {function: seconds} for one pass.

    (i)   torch_native: torch.sigmoid / tanh / F.silu / exp2 on fp16 tensors, torch.sin + torch.cos on fp32 angles,
          intra-op threads = every host core (the reference's isolated sweep compares against these PyTorch natives,
          scripts/benchmark_report_function_speed.py:112-134, there on the GPU);
    (ii)  reference_replay: the reference's own CPU arithmetic for the polynomial programs: split-rounded fp16 Horner
          (autonumerics_zero/evolution/fit_all_degrees.py:59-96) for sigmoid D3, tanh D4, SiLU D3 in numpy, the array cut
          into one slice per host core and the slices run on a thread pool (numpy's element-wise loops release the
          interpreter lock; the reference itself calls the function on one thread), polynomial_sincos
          (src/sfu_repro/rope/polynomial_sincos.py:138-165) in torch with every core; the reference has no CPU evaluator
          of the exp2 hinge, so that function has no entry;
    (iii) exact_emulator: this repository's single-rounding soft-float port (OpenMP, every core)."""

    def __init__(self, n_native, n_replay, n_emulator):
        import numpy as np
        import torch
        self.np, self.torch = np, torch
        self.threads = host_threads()
        torch.set_num_threads(self.threads)
        self.n = {"torch_native": n_native, "reference_replay": n_replay, "exact_emulator": n_emulator}
        u8, frac, ang = cpu_sample_inputs(max(n_native, n_replay, n_emulator))
        self.u8, self.frac, self.ang = u8, frac, ang
        self.t_u8, self.t_frac, self.t_ang = (torch.from_numpy(a[:n_native]) for a in (u8, frac, ang))
        self.oracle = None

    @staticmethod
    def _timed(fn):
        t0 = time.perf_counter()
        fn()
        return time.perf_counter() - t0

    def torch_native(self):
        torch, F = self.torch, self.torch.nn.functional
        return {"sigmoid": self._timed(lambda: torch.sigmoid(self.t_u8)), "tanh": self._timed(lambda: torch.tanh(self.t_u8)),
                "silu": self._timed(lambda: F.silu(self.t_u8)), "exp2": self._timed(lambda: torch.exp2(self.t_frac)),
                "sincos": self._timed(lambda: (torch.sin(self.t_ang), torch.cos(self.t_ang)))}

    def reference_replay(self):
        from fast_polynomial_transcendentals_b200.sfu_repro.rope.polynomial_sincos import polynomial_sincos
        from oracle import reference_replays
        from concurrent.futures import ThreadPoolExecutor
        n = self.n["reference_replay"]
        ang = self.torch.from_numpy(self.ang[:n])
        slices = self.np.array_split(self.u8[:n], self.threads)

        def replay(name):
            with ThreadPoolExecutor(self.threads) as pool:
                list(pool.map(lambda part: reference_replays.activation_replay_fp16(name, part), slices))
        out = {name: self._timed(lambda name=name: replay(name)) for name in ("sigmoid", "tanh", "silu")}
        out["sincos"] = self._timed(lambda: polynomial_sincos(ang, accurate_reduction=False))
        return out

    def exact_emulator(self):
        if self.oracle is None:
            from oracle import oracle
            oracle.build()
            oracle.set_threads(self.threads)
            self.oracle = oracle
        o, n, np = self.oracle, self.n["exact_emulator"], self.np
        u8, frac, ang = self.u8[:n].view(np.uint16), self.frac[:n].view(np.uint16), self.ang[:n]
        return {"sigmoid": self._timed(lambda: o.unary(o.find_program("SIGMOID_FWD_D3", 0), u8)),
                "tanh": self._timed(lambda: o.unary(o.find_program("TANH_FWD_D4", 0), u8)),
                "silu": self._timed(lambda: o.unary(o.find_program("SWISH_FWD_D3", 0), u8)),
                "exp2": self._timed(lambda: o.exp2_hinge(frac, 0)),
                "sincos": self._timed(lambda: o.sincos_packed("d5_d6_half_turn_fp16", ang))}

    def cores(self, leg):
        return self.threads

    def summarise(self, leg, passes):
        """passes: list of {function: seconds}.  Median seconds per function -> elements/s per function and for the leg."""
        n = self.n[leg]
        per = {}
        for fn in passes[0]:
            ts = sorted(p[fn] for p in passes)
            per[fn] = n / ts[len(ts) // 2]
        total_s = sum(n / v for v in per.values())
        return {"elements_per_s": len(per) * n / total_s, "per_function_elements_per_s": per, "functions": len(per),
                "elements_per_function": n, "passes": len(passes), "cores": self.cores(leg)}


def cpu_baseline():
    """Bounded CPU legs for the GPU arm's line: about 10-20 s of CPU work on rank 0."""
    legs = CpuLegs(1 << 24, 1 << 22, 1 << 22)
    out = {}
    for leg, passes in (("torch_native", 4), ("reference_replay", 1), ("exact_emulator", 2)):
        fn = getattr(legs, leg)
        if leg != "reference_replay":
            fn()
        out[leg] = legs.summarise(leg, [fn() for _ in range(passes)])
    done = sum(out[leg]["functions"] * out[leg]["elements_per_function"] for leg in ("torch_native", "reference_replay"))
    spent = sum(out[leg]["functions"] * out[leg]["elements_per_function"] / out[leg]["elements_per_s"]
                for leg in ("torch_native", "reference_replay"))
    return {"value": done / spent, "unit": "elements/s", "cores": legs.threads, "kind": "port",
            "sample": "the reference's CPU path restated: torch CPU natives (5 functions, 2^24 fp16 / fp32 elements each, all "
                      "host threads) + the reference's vectorised replays (split-rounded fp16 Horner for sigmoid / tanh / "
                      "SiLU in numpy, polynomial_sincos in torch; 2^22 elements each); value = all their elements over all "
                      "their time; the exact single-rounding emulator (2^22 per function) rides in `legs` and is not counted",
            "legs": out}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n = 1 << 24
    legs = CpuLegs(n, n, 1 << 21)
    counted = ("torch_native", "reference_replay")
    for _ in range(max(1, min(args.warmup, 2))):
        legs.torch_native()
    legs.reference_replay()
    passes = {leg: [] for leg in counted}
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for leg in counted:
            passes[leg].append(getattr(legs, leg)())
    dt = time.perf_counter() - t0
    detail = {leg: legs.summarise(leg, passes[leg]) for leg in counted}
    emulator = legs.exact_emulator()
    detail["exact_emulator"] = legs.summarise("exact_emulator", [legs.exact_emulator(), emulator])
    elements_per_step = sum(detail[leg]["functions"] for leg in counted) * n
    value = elements_per_step * args.steps / dt
    sample = (f"each step = torch CPU natives (sigmoid, tanh, SiLU, exp2 on fp16; sin + cos on fp32) and the reference's "
              f"vectorised replays (split-rounded fp16 Horner for sigmoid D3 / tanh D4 / SiLU D3, polynomial_sincos), 2^24 "
              f"elements per function (a bounded sample of the 2^28 workload); value = elements of both legs over the "
              f"wall time of the step loop")
    line = {
        "impl": "reference", "metric": "elements_per_s_fp16_function_sweep", "value": value, "unit": "elements/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": "elements/s", "cores": legs.threads, "kind": "port", "sample": sample,
                         "legs": detail},
        "e2e": {"value": value, "unit": "elements/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus):
    return {"workload": "BASELINE config[1]: isolated FP16 function sweep, HBM endpoint N=2^28 per function "
                        "(sigmoid D3, tanh D4, SiLU D3, exp2 hinge, sin/cos D5/D6), polynomial vs native SFU",
            "elements_per_function_per_gpu": N_HBM, "functions": 5,
            "sharding": f"headline: {n_gpus} x independent 2^28-element ranges (weak scaling); the partitioning of ONE seeded "
                        "problem by element ranges, expert groups and (batch, head) blocks is timed under extras.sharded",
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

    # the headline buffers are needed again only on rank 0 (native twins, L2 endpoint); free them elsewhere
    if rank != 0:
        del u8, frac, ang, out16, out_sc, poly_hbm
        torch.cuda.empty_cache()

    # ---- e2e through the public API with host buffers: every rank its own 2^28-element sweep, whole-job value = all
    # ranks' elements over the slowest rank's time; beside it the same copies with no kernel between them
    if world > 1:
        dist.barrier()
    e2e = bench_e2e(torch, spline_ops, HostPipeline, device, max(5, args.steps), lambda: barrier(True))
    if host_binding:
        e2e["host_binding"] = host_binding
        os.sched_setaffinity(0, all_cpus)      # the CPU legs below use every core again
    if world > 1:
        t = torch.tensor([e2e["ms_per_step"], e2e["copy_only"]["ms_per_step"]], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e["ms_per_step"], e2e["copy_only"]["ms_per_step"] = float(t[0].item()), float(t[1].item())
        e2e["h2d_bytes_per_step"] *= world
        e2e["d2h_bytes_per_step"] *= world
        e2e["path"] += f"; {world} ranks at once, slowest rank's time"
    e2e["value"] = world * 5 * e2e["elements_per_function"] / (e2e["ms_per_step"] * 1e-3)
    copy = e2e["copy_only"]
    copy["value"] = world * 5 * e2e["elements_per_function"] / (copy["ms_per_step"] * 1e-3)
    copy["gbs_per_direction_per_rank"] = e2e["h2d_bytes_per_step"] / world / (copy["ms_per_step"] * 1e-3) / 1e9
    e2e["fraction_of_copy_only_rate"] = copy["ms_per_step"] / e2e["ms_per_step"]

    # ---- the partitioning of one seeded problem over the ranks (all ranks take part)
    sharded = bench_sharded(torch, dist, lib, _lib, device, rank, world, hbm_peak, measured_peaks()[1])

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
    extras["gate_up_swiglu_bf16"] = bench_gate_up(torch, lib, _lib, device, S, time_sweep)
    extras["b3_config1"] = bench_b3(torch, lib, _lib, device, S, time_graph)
    extras["attention_fwd_bf16"] = bench_attention(torch, lib, _lib, device, S, time_sweep)
    extras["sharded"] = sharded

    cpu = cpu_baseline() if world == 1 else None     # the host cores are timed alone, not beside other ranks' work
    dominant = functions["sigmoid"]
    line = {
        "metric": "elements_per_s_fp16_function_sweep", "value": value, "unit": "elements/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": workload_config(world),
        "impl": "ours", "roofline": {"bound": "hbm", "achieved": dominant["poly_gbs"], "peak": hbm_peak, "unit": "GB/s",
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


# ---- one seeded problem, addressed by GLOBAL element index, so that a shard is a slice of the same tensor at every N

def hashed_uniform(torch, lo, hi, stream_id, device, chunk=1 << 26):
    """U[0,1) fp32 for global indices [lo, hi): a 32-bit integer hash of (index, stream), generated in chunks."""
    out = torch.empty(hi - lo, dtype=torch.float32, device=device)
    for a in range(lo, hi, chunk):
        b = min(hi, a + chunk)
        x = torch.arange(a, b, device=device, dtype=torch.int64)
        x = (x * 2654435761 + (SEED + 7919 * stream_id) * 40503) & 0xFFFFFFFF
        for _ in range(2):
            x = ((x ^ (x >> 16)) * 0x45D9F3B) & 0xFFFFFFFF
        x = x ^ (x >> 16)
        out[a - lo:b - lo] = x.to(torch.float32) * (1.0 / 4294967296.0)
    return out


def hashed_normal(torch, index, stream_id, std=1.0):
    """N(0, std^2) fp32 for a tensor of global int64 indices (Box-Muller on two hashed uniforms)."""
    def u(salt):
        x = (index * 2654435761 + (SEED + 7919 * stream_id + salt) * 40503) & 0xFFFFFFFF
        for _ in range(2):
            x = ((x ^ (x >> 16)) * 0x45D9F3B) & 0xFFFFFFFF
        x = x ^ (x >> 16)
        return (x.to(torch.float32) + 0.5) * (1.0 / 4294967296.0)
    return torch.sqrt(-2.0 * torch.log(u(1))) * torch.cos(6.283185307179586 * u(2)) * std


def bits_checksum(torch, t):
    """Integer sum of the 16-bit patterns of a tensor (order-independent, so shard sums add up to the whole)."""
    return int(t.contiguous().view(torch.int16).sum(dtype=torch.int64).item())


class L2Flush:
    """Overwrites a buffer larger than the L2 between timed launches whose working set is not itself larger."""

    def __init__(self, torch, device, nbytes=256 << 20):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)

    def __call__(self):
        self.buf.zero_()


def time_launch(torch, fn, reps, flush=None, warm=2):
    """Median CUDA-event duration (ms) of fn() over `reps` launches, an L2 flush before each when given."""
    for _ in range(warm):
        fn()
    times = []
    for _ in range(reps):
        if flush:
            flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]


def gather_floats(torch, dist, world, device, values):
    t = torch.tensor(values, dtype=torch.float64, device=device)
    if world == 1:
        return [list(values)]
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return [o.tolist() for o in out]


def gather_ints(torch, dist, world, device, values):
    t = torch.tensor(values, dtype=torch.int64, device=device)
    if world == 1:
        return [list(values)]
    out = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return [o.tolist() for o in out]


def bench_sharded(torch, dist, lib, _lib, device, rank, world, hbm_peak, tensor_peak):
    """north_star's partitioning of ONE seeded problem over the N ranks: contiguous element ranges (function sweep,
    2^30 elements per function in total: strong scaling), expert groups over the Zipf token counts (B4 SwiGLU), (batch,
    kv-head group) blocks (attention configurations 4 and 5, the latter with its fused RoPE prologue).  Inputs are a
    function of the GLOBAL element index, so a shard holds the same values at every N; each shard's output checksum is
    gathered, their sum is the checksum of the whole output (equal at every N), and rank 0 recomputes the last rank's
    shard to show that a shard does not depend on who computes it.  No collective touches the data."""
    import ctypes

    import numpy as np
    from fast_polynomial_transcendentals_b200 import sharding
    stream = torch.cuda.current_stream().cuda_stream
    flush = L2Flush(torch, device)
    out = {"generator": "inputs are hashes of the global element index (seed 1234): shards are slices of one tensor"}

    # ---- (1) function sweep, contiguous element ranges of 2^30 elements per function
    total = 1 << 30

    def sweep_shard(r):
        lo, hi = sharding.element_range(total, r, world)
        n = hi - lo
        u8 = (hashed_uniform(torch, lo, hi, 1, device) * 16 - 8).to(torch.float16)
        frac = hashed_uniform(torch, lo, hi, 2, device).to(torch.float16)
        ang = hashed_uniform(torch, lo, hi, 3, device) * (2 * math.pi) - math.pi
        o16 = torch.empty(n, dtype=torch.float16, device=device)
        osc = torch.empty(2, n, dtype=torch.float16, device=device)
        kernels = [("sigmoid", lambda: lib.fpt_unary(o16.data_ptr(), u8.data_ptr(), n, 0, 0, 3, 0, 0, stream), o16),
                   ("tanh", lambda: lib.fpt_unary(o16.data_ptr(), u8.data_ptr(), n, 1, 0, 4, 0, 0, stream), o16),
                   ("silu", lambda: lib.fpt_unary(o16.data_ptr(), u8.data_ptr(), n, 2, 0, 3, 0, 0, stream), o16),
                   ("exp2", lambda: lib.fpt_exp2_fraction(o16.data_ptr(), frac.data_ptr(), n, 1, 1, stream), o16),
                   ("sincos", lambda: lib.fpt_sincos(osc.data_ptr(), ang.data_ptr(), n, 3, 0, stream), osc)]
        return n, kernels

    n, kernels = sweep_shard(rank)
    ms, sums = [], []
    for name, k, result in kernels:
        def run(k=k, name=name):
            _lib.check(name, k())
        ms.append(time_launch(torch, run, 5, flush if n * 4 < (192 << 20) else None))
        sums.append(bits_checksum(torch, result))
    del kernels
    torch.cuda.empty_cache()
    all_ms = gather_floats(torch, dist, world, device, ms)
    all_sums = gather_ints(torch, dist, world, device, sums)
    recheck = None
    if world > 1 and rank == 0:        # the last rank's shard, recomputed here
        _, other = sweep_shard(world - 1)
        redo = []
        for name, k, result in other:
            _lib.check(name, k())
            redo.append(bits_checksum(torch, result))
        recheck = redo == all_sums[world - 1]
        del other
        torch.cuda.empty_cache()
    names = ("sigmoid", "tanh", "silu", "exp2", "sincos")
    makespan = sum(max(all_ms[r][i] for r in range(world)) for i in range(5))
    out["function_sweep_2^30_total"] = {
        "scaling": "strong: 2^30 elements per function in total, contiguous element ranges of 2^30/N per GPU",
        "per_function_ms_max_over_ranks": {nm: max(all_ms[r][i] for r in range(world)) for i, nm in enumerate(names)},
        "elements_per_s": 5 * total / (makespan * 1e-3),
        "checksum_total_per_function": {nm: sum(all_sums[r][i] for r in range(world)) for i, nm in enumerate(names)},
        "last_shard_recomputed_on_rank0_equal": recheck}

    # ---- (2) B4 routed experts: 131072 expert-sorted rows x 1408, experts sharded in contiguous groups
    rows_total, hidden, experts = 16384 * 8, 1408, 64
    counts = sharding.zipf_expert_counts(rows_total, experts)

    def b4_shard(r):
        shard = sharding.expert_group(counts, r, world)
        nrows = shard.last_row - shard.first_row
        idx = torch.arange(shard.first_row * hidden, shard.last_row * hidden, device=device, dtype=torch.int64)
        gate = hashed_normal(torch, idx, 11, 1.5).to(torch.bfloat16)
        up = hashed_normal(torch, idx, 12, 1.5).to(torch.bfloat16)
        del idx
        o = torch.empty_like(gate)
        nel = nrows * hidden
        return shard, nrows, o, (lambda: _lib.check("fpt_swish_mul", lib.fpt_swish_mul(
            o.data_ptr(), gate.data_ptr(), up.data_ptr(), nel, 3, 1, 0, stream)))

    shard, nrows, o, run = b4_shard(rank)
    b4_ms = time_launch(torch, run, 7, flush)
    b4_sum = bits_checksum(torch, o)
    del o, run
    torch.cuda.empty_cache()
    per_ms = [v[0] for v in gather_floats(torch, dist, world, device, [b4_ms])]
    per_rows = [v[0] for v in gather_ints(torch, dist, world, device, [nrows])]
    per_sum = [v[0] for v in gather_ints(torch, dist, world, device, [b4_sum])]
    recheck = None
    if world > 1 and rank == 0:
        _, _, o2, run2 = b4_shard(world - 1)
        run2()
        recheck = bits_checksum(torch, o2) == per_sum[world - 1]
        del o2, run2
        torch.cuda.empty_cache()
    out["b4_routed_experts_131072x1408"] = {
        "experts_per_gpu": experts // world if experts % world == 0 else f"{experts}/{world}",
        "rows_per_gpu": per_rows, "ms_per_gpu": per_ms, "makespan_ms": max(per_ms),
        "imbalance_rows_max_over_mean": max(per_rows) / (sum(per_rows) / world),
        "elements_per_s": rows_total * hidden / (max(per_ms) * 1e-3),
        "gbs_aggregate": 6 * rows_total * hidden / (max(per_ms) * 1e-3) / 1e9,
        "frac_of_measured_hbm_per_gpu_at_makespan": 6 * max(per_rows) * hidden / (max(per_ms) * 1e-3) / 1e9 / hbm_peak,
        "token_counts": "seeded Zipf(1.1) weights over a seeded permutation of 64 experts, multinomial of 131072 assignments",
        "timing": "median of 7 launches, 256 MiB written between launches (a shard can be smaller than the L2)",
        "checksum_total": sum(per_sum), "last_shard_recomputed_on_rank0_equal": recheck}

    # ---- (2b) the same experts with their input projections: out = SwiGLU(x W_gate^T, x W_up^T) in one kernel per GPU
    dim = 2048
    offsets_all = np.concatenate([[0], np.cumsum(counts)])

    def b4_projection_shard(r):
        sh = sharding.expert_group(counts, r, world)
        n_local = sh.last_row - sh.first_row
        e_local = sh.last_expert - sh.first_expert
        x = torch.empty(max(n_local, 1), dim, dtype=torch.bfloat16, device=device)
        wg = torch.empty(e_local, hidden, dim, dtype=torch.bfloat16, device=device)
        wu = torch.empty_like(wg)
        for e in range(sh.first_expert, sh.last_expert):      # values are functions of the GLOBAL row / expert index
            r0, r1 = int(offsets_all[e]), int(offsets_all[e + 1])
            if r1 > r0:
                idx = torch.arange(r0 * dim, r1 * dim, device=device, dtype=torch.int64)
                x[r0 - sh.first_row:r1 - sh.first_row] = hashed_normal(torch, idx, 21, 1.0).view(r1 - r0, dim).to(torch.bfloat16)
            idx = torch.arange(e * hidden * dim, (e + 1) * hidden * dim, device=device, dtype=torch.int64)
            wg[e - sh.first_expert] = hashed_normal(torch, idx, 22, dim ** -0.5).view(hidden, dim).to(torch.bfloat16)
            wu[e - sh.first_expert] = hashed_normal(torch, idx, 23, dim ** -0.5).view(hidden, dim).to(torch.bfloat16)
        ends = torch.tensor(offsets_all[sh.first_expert + 1:sh.last_expert + 1] - sh.first_row, dtype=torch.int32, device=device)
        o = torch.zeros(max(n_local, 1), hidden, dtype=torch.bfloat16, device=device)
        gstatus = torch.zeros(1, dtype=torch.int32, device=device)

        def run():
            if n_local:
                _lib.check("fpt_gate_up_swiglu", lib.fpt_gate_up_swiglu(
                    o.data_ptr(), x.data_ptr(), wg.data_ptr(), wu.data_ptr(), n_local, dim, hidden, dim, dim, hidden * dim, hidden,
                    ends.data_ptr(), e_local, 3, 0, 0, gstatus.data_ptr(), stream))
        return n_local, o, run, gstatus, (x, wg, wu, ends)

    nloc, o, run, gstatus, keep = b4_projection_shard(rank)
    gu_ms = time_launch(torch, run, 7, flush)
    if int(gstatus.item()) != 0:
        raise RuntimeError(f"fpt_gate_up_swiglu reported status {int(gstatus.item()) & 0xffffffff:#x}")
    gu_sum = bits_checksum(torch, o[:nloc]) if nloc else 0
    del o, run, keep
    torch.cuda.empty_cache()
    per_ms = [v[0] for v in gather_floats(torch, dist, world, device, [gu_ms])]
    per_sum = [v[0] for v in gather_ints(torch, dist, world, device, [gu_sum])]
    recheck = None
    if world > 1 and rank == 0:
        n2, o2, run2, _, keep2 = b4_projection_shard(world - 1)
        run2()
        recheck = (bits_checksum(torch, o2[:n2]) if n2 else 0) == per_sum[world - 1]
        del o2, run2, keep2
        torch.cuda.empty_cache()
    flops = 2.0 * rows_total * dim * 2 * hidden
    out["b4_routed_experts_with_projections_131072x2048_to_1408"] = {
        "rows_per_gpu": per_rows, "ms_per_gpu": per_ms, "makespan_ms": max(per_ms),
        "tflops_aggregate": flops / (max(per_ms) * 1e-3) / 1e12,
        "tflops_busiest_gpu": 2.0 * max(per_rows) * dim * 2 * hidden / (max(per_ms) * 1e-3) / 1e12,
        "kernel": "fpt_gate_up_swiglu, one launch per GPU over its expert group (grouped, pairs of CTAs)",
        "checksum_total": sum(per_sum), "last_shard_recomputed_on_rank0_equal": recheck}

    # ---- (3) attention, (batch, kv-head group) blocks
    D = 128
    arr = lambda t: (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
    status = torch.zeros(1, dtype=torch.int32, device=device)

    def block_tensor(b, h0, h1, heads_total, S, stream_id):
        """[1, S, h1-h0, D] bf16 slice of the global [B, S, heads_total, D] tensor"""
        s_i = torch.arange(S, device=device, dtype=torch.int64).view(S, 1, 1)
        h_i = torch.arange(h0, h1, device=device, dtype=torch.int64).view(1, -1, 1)
        d_i = torch.arange(D, device=device, dtype=torch.int64).view(1, 1, D)
        idx = ((b * S + s_i) * heads_total + h_i) * D + d_i
        return hashed_normal(torch, idx, stream_id).to(torch.bfloat16).unsqueeze(0)

    def attention_shard(r, B, S, Hq, Hk, mode, causal, cap, log2_n, with_rope):
        group = Hq // Hk
        work = []
        for blk in sharding.attention_blocks(B, Hq, Hk, r, world):
            h0, h1 = blk.first_q_head, blk.last_q_head
            q = block_tensor(blk.batch, h0, h1, Hq, S, 21)
            k = block_tensor(blk.batch, h0 // group, h1 // group, Hk, S, 22)
            v = block_tensor(blk.batch, h0 // group, h1 // group, Hk, S, 23)
            o = torch.empty_like(q)
            lse = torch.empty(1, h1 - h0, S, device=device)
            work.append((q, k, v, o, lse))
        inc = None
        if with_rope:
            freqs = 500000.0 ** (-np.arange(0, D, 2, dtype=np.float64) / D)
            inc = torch.from_numpy(np.round(freqs * 2.0 ** 32 / (2 * math.pi)).astype(np.int64).astype(np.uint32)
                                   .view(np.int32)).to(device)
            rotated = [(torch.empty(1, q.shape[2], S, D, dtype=q.dtype, device=device),
                        torch.empty(1, k.shape[2], S, D, dtype=k.dtype, device=device)) for q, k, *_ in work]

        def rope():
            for (q, k, *_), (qr, kr) in zip(work, rotated):
                _lib.check("fpt_rope_apply", lib.fpt_rope_apply(qr.data_ptr(), kr.data_ptr(), q.data_ptr(), k.data_ptr(),
                                                                inc.data_ptr(), 1, S, q.shape[2], k.shape[2], D, 0, 1, stream))

        def attend():
            for i, (q, k, v, o, lse) in enumerate(work):
                if with_rope:       # the rotation writes (batch, head, seq, dim); the attention reads it through strides
                    q, k = rotated[i][0].permute(0, 2, 1, 3), rotated[i][1].permute(0, 2, 1, 3)
                _lib.check("fpt_attention_fwd", lib.fpt_attention_fwd(
                    o.data_ptr(), lse.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), 1, S, q.shape[2], k.shape[2], D,
                    arr(q), arr(k), arr(v), arr(o), mode, causal, 1.0 / math.sqrt(D), cap, log2_n, status.data_ptr(), stream))
        return work, (rope if with_rope else None), attend

    for name, B, S, Hq, Hk, mode, causal, cap, log2_n, with_rope in (
            ("config4_causal_gqa_softcap50_tanhD4_B4_S8192_Hq32_Hkv8", 4, 8192, 32, 8, 0, 1, 50.0, 12, False),
            ("config5_rope_sigmoid_direct_B2_S16384_H32", 2, 16384, 32, 32, 1, 0, 0.0, 14, True)):
        work, rope, attend = attention_shard(rank, B, S, Hq, Hk, mode, causal, cap, log2_n, with_rope)
        rope_ms = time_launch(torch, rope, 3) if rope else 0.0
        attn_ms = time_launch(torch, attend, 5)
        if int(status.item()) != 0:
            raise RuntimeError(f"attention kernel reported status {int(status.item()) & 0xffffffff:#x}")
        csum = sum(bits_checksum(torch, w[3]) for w in work)
        units = sum(w[0].shape[2] for w in work)
        del work, rope, attend
        torch.cuda.empty_cache()
        per = gather_floats(torch, dist, world, device, [attn_ms, rope_ms])
        sums = [v[0] for v in gather_ints(torch, dist, world, device, [csum])]
        heads = [v[0] for v in gather_ints(torch, dist, world, device, [units])]
        recheck = None
        if world > 1 and rank == 0:
            work2, rope2, attend2 = attention_shard(world - 1, B, S, Hq, Hk, mode, causal, cap, log2_n, with_rope)
            if rope2:
                rope2()
            attend2()
            recheck = sum(bits_checksum(torch, w[3]) for w in work2) == sums[world - 1]
            del work2, rope2, attend2
            torch.cuda.empty_cache()
        flops = 4.0 * B * Hq * S * S * D * (0.5 if causal else 1.0)
        makespan = max(p[0] for p in per)
        with_rope_ms = max(p[0] + p[1] for p in per)
        out[name] = {"q_heads_per_gpu": heads, "attention_ms_per_gpu": [p[0] for p in per], "rope_ms_per_gpu": [p[1] for p in per],
                     "makespan_ms": makespan, "tflops_aggregate": flops / (makespan * 1e-3) / 1e12,
                     "tflops_per_gpu": flops / world / (makespan * 1e-3) / 1e12,
                     "frac_of_measured_bf16_peak_per_gpu": flops / world / (makespan * 1e-3) / 1e12 / tensor_peak,
                     "tflops_aggregate_with_rope_prologue": flops / (with_rope_ms * 1e-3) / 1e12 if with_rope else None,
                     "timing": "median of 5 passes over the rank's blocks (bursts, not power-capped)",
                     "checksum_total": sum(sums), "last_shard_recomputed_on_rank0_equal": recheck}
    return out


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


def gate_up_forms(torch, lib, _lib, time_sweep, call, flops):
    """The forms of the projection kernel on one problem: one CTA with 128- or 256-row tiles, pairs of CTAs with one or two
    hidden tiles per row tile (the latter where the number of hidden tiles is even; otherwise it runs as the former).  Each
    is timed inside one back-to-back loop over the three (clocks as in a training step) and as isolated launches 50 ms
    apart (clocks at their maximum): TFLOP/s for both."""
    forms = (("one_cta_128_rows", 128, 0, 0), ("one_cta_256_rows", 256, 0, 0), ("cta_pair_one_hidden_tile", 0, 1, 0),
             ("cta_pair_two_hidden_tiles", 0, 1, 1))

    def with_form(rows, pair, wide):
        def run():
            _lib.check("fpt_set_tuning", lib.fpt_set_tuning(b"gate_up_tile_rows", rows))
            _lib.check("fpt_set_tuning", lib.fpt_set_tuning(b"gate_up_cta_pair", pair))
            _lib.check("fpt_set_tuning", lib.fpt_set_tuning(b"gate_up_pair_wide", wide))
            call()
        return run
    try:
        _, together = time_sweep([(name, 0, with_form(rows, pair, wide)) for name, rows, pair, wide in forms], 15, 2)
        alone = {}
        for name, rows, pair, wide in forms:
            run = with_form(rows, pair, wide)
            run()
            torch.cuda.synchronize()
            times = []
            for _ in range(5):
                time.sleep(0.05)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                run()
                b.record()
                torch.cuda.synchronize()
                times.append(a.elapsed_time(b))
            alone[name] = sorted(times)[len(times) // 2]
    finally:
        _lib.check("fpt_set_tuning", lib.fpt_set_tuning(b"gate_up_tile_rows", 0))
        _lib.check("fpt_set_tuning", lib.fpt_set_tuning(b"gate_up_cta_pair", -1))
        _lib.check("fpt_set_tuning", lib.fpt_set_tuning(b"gate_up_pair_wide", 0))
    return {name: {"back_to_back_ms": together[name], "back_to_back_tflops": flops / (together[name] * 1e-3) / 1e12,
                   "isolated_ms": alone[name], "isolated_tflops": flops / (alone[name] * 1e-3) / 1e12} for name, *_ in forms}


def bench_gate_up(torch, lib, _lib, device, S, time_sweep):
    """The projection that feeds the SwiGLU with the activation in its epilogue (`fpt_gate_up_swiglu`) next to the two-step
    path it replaces, at the B1 and B4 sizes: library matrix product(s) writing [gate | up], then this library's SwiGLU
    kernel reading them back.  The candidates alternate inside one timed loop, so that they meet the same clocks."""
    import ctypes
    _, tensor_peak, _ = measured_peaks()
    sustained = measured_sustained_tflops()
    vp = ctypes.c_void_p
    status = torch.zeros(1, dtype=torch.int32, device=device)
    g = torch.Generator(device=device)
    g.manual_seed(SEED)
    out = {"timing": "20 rounds of [fused, products, activation] back to back (about 0.1 s: clocks as in a training step)"}

    def fused_call(o, x, wg, wu, rows, dim, hidden, group_stride, ends, groups):
        return lambda: _lib.check("fpt_gate_up_swiglu", lib.fpt_gate_up_swiglu(
            o.data_ptr(), x.data_ptr(), wg.data_ptr(), wu.data_ptr(), rows, dim, hidden, dim, dim, group_stride, hidden,
            vp(ends.data_ptr()) if ends is not None else None, groups, 3, 0, 0, status.data_ptr(), S()))

    # B1: Llama-3-8B feed-forward, 16384 tokens
    rows, dim, hidden = 16384, 4096, 14336
    x = torch.randn(rows, dim, device=device, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * hidden, dim, device=device, generator=g) * dim ** -0.5).to(torch.bfloat16)
    o = torch.empty(rows, hidden, dtype=torch.bfloat16, device=device)
    packed = torch.empty(rows, 2 * hidden, dtype=torch.bfloat16, device=device)
    ks = [("fused", 0, fused_call(o, x, w[:hidden], w[hidden:], rows, dim, hidden, 0, None, 1)),
          ("matmul", 0, lambda: torch.matmul(x, w.T, out=packed)),
          ("packed_swiglu", 0, lambda: _lib.check("fpt_swish_mul_packed", lib.fpt_swish_mul_packed(
              o.data_ptr(), packed.data_ptr(), rows, hidden, 3, 1, 0, S())))]
    _, t = time_sweep(ks, 20, 3)
    flops = 2.0 * rows * dim * 2 * hidden
    two_step = t["matmul"] + t["packed_swiglu"]
    out["B1_dense_16384x4096_to_14336"] = {
        "fused_ms": t["fused"], "fused_tflops": flops / (t["fused"] * 1e-3) / 1e12,
        "fused_frac_of_measured_bf16_peak": flops / (t["fused"] * 1e-3) / 1e12 / tensor_peak,
        "fused_frac_of_sustained_bf16_peak": flops / (t["fused"] * 1e-3) / 1e12 / sustained,
        "library_matmul_ms": t["matmul"], "library_matmul_tflops": flops / (t["matmul"] * 1e-3) / 1e12,
        "packed_swiglu_ms": t["packed_swiglu"], "two_step_ms": two_step, "fused_speedup_vs_two_step": two_step / t["fused"],
        "intermediate_bytes_not_written": rows * 2 * hidden * 2}
    out["B1_dense_16384x4096_to_14336"]["forms"] = gate_up_forms(
        torch, lib, _lib, time_sweep, fused_call(o, x, w[:hidden], w[hidden:], rows, dim, hidden, 0, None, 1), flops)
    del x, w, o, packed
    torch.cuda.empty_cache()

    # B4: 64 routed experts, Zipf(1.1) token counts, 131072 rows
    rows, dim, hidden, groups = 131072, 2048, 1408, 64
    x = torch.randn(rows, dim, device=device, generator=g).to(torch.bfloat16)
    wg = (torch.randn(groups, hidden, dim, device=device, generator=g) * dim ** -0.5).to(torch.bfloat16)
    wu = (torch.randn(groups, hidden, dim, device=device, generator=g) * dim ** -0.5).to(torch.bfloat16)
    weights = 1.0 / torch.arange(1, groups + 1, dtype=torch.float64) ** 1.1
    counts = torch.multinomial(weights / weights.sum(), rows, replacement=True,
                               generator=torch.Generator().manual_seed(SEED)).bincount(minlength=groups)
    ends = torch.cumsum(counts, 0).to(torch.int32).to(device)
    o = torch.empty(rows, hidden, dtype=torch.bfloat16, device=device)
    entry = {}
    ks = [("fused", 0, fused_call(o, x, wg, wu, rows, dim, hidden, hidden * dim, ends, groups))]
    if hasattr(torch, "_grouped_mm"):
        held = {}
        def products():
            held["gate"] = torch._grouped_mm(x, wg.transpose(-2, -1), offs=ends)
            held["up"] = torch._grouped_mm(x, wu.transpose(-2, -1), offs=ends)
        products()
        ks += [("grouped_mm_x2", 0, products),
               ("flat_swiglu", 0, lambda: _lib.check("fpt_swish_mul", lib.fpt_swish_mul(
                   o.data_ptr(), held["gate"].data_ptr(), held["up"].data_ptr(), rows * hidden, 3, 1, 0, S())))]
    _, t = time_sweep(ks, 20, 3)
    flops = 2.0 * rows * dim * 2 * hidden
    entry = {"fused_ms": t["fused"], "fused_tflops": flops / (t["fused"] * 1e-3) / 1e12,
             "fused_frac_of_measured_bf16_peak": flops / (t["fused"] * 1e-3) / 1e12 / tensor_peak,
             "fused_frac_of_sustained_bf16_peak": flops / (t["fused"] * 1e-3) / 1e12 / sustained,
             "rows_of_largest_and_smallest_expert": [int(counts.max()), int(counts.min())],
             "intermediate_bytes_not_written": rows * 2 * hidden * 2}
    if "grouped_mm_x2" in t:
        two_step = t["grouped_mm_x2"] + t["flat_swiglu"]
        entry |= {"library_grouped_mm_x2_ms": t["grouped_mm_x2"], "flat_swiglu_ms": t["flat_swiglu"], "two_step_ms": two_step,
                  "fused_speedup_vs_two_step": two_step / t["fused"]}
    # the whole expert feed-forward: fused input projections + SwiGLU, then the projection back as the same kernel's raw
    # epilogue (a plain grouped product), against three library grouped products with the activation kernel between
    w2 = (torch.randn(groups, dim, hidden, device=device, generator=g) * hidden ** -0.5).to(torch.bfloat16)
    y = torch.empty(rows, dim, dtype=torch.bfloat16, device=device)
    half = dim // 2

    def ours_mlp():
        fused_call(o, x, wg, wu, rows, dim, hidden, hidden * dim, ends, groups)()
        _lib.check("fpt_gate_up_swiglu", lib.fpt_gate_up_swiglu(
            y.data_ptr(), o.data_ptr(), w2.data_ptr(), w2[:, half:].data_ptr(), rows, hidden, half, hidden, hidden, dim * hidden, dim,
            vp(ends.data_ptr()), groups, 3, 0, 1, status.data_ptr(), S()))
    ks = [("ours", 0, ours_mlp)]
    if hasattr(torch, "_grouped_mm"):
        def library_mlp():
            gt = torch._grouped_mm(x, wg.transpose(-2, -1), offs=ends)
            ut = torch._grouped_mm(x, wu.transpose(-2, -1), offs=ends)
            _lib.check("fpt_swish_mul", lib.fpt_swish_mul(o.data_ptr(), gt.data_ptr(), ut.data_ptr(), rows * hidden, 3, 1, 0, S()))
            return torch._grouped_mm(o, w2.transpose(-2, -1), offs=ends)
        ks.append(("library", 0, library_mlp))
    _, tm = time_sweep(ks, 15, 3)
    mlp_flops = 2.0 * rows * dim * 3 * hidden
    entry["expert_feed_forward"] = {"ours_ms": tm["ours"], "ours_tflops": mlp_flops / (tm["ours"] * 1e-3) / 1e12,
                                    "what": "two launches of fpt_gate_up_swiglu: projections + SwiGLU, then the projection back (raw epilogue)"}
    if "library" in tm:
        entry["expert_feed_forward"] |= {"library_ms": tm["library"], "speedup_vs_library": tm["library"] / tm["ours"],
                                         "library": "three torch._grouped_mm with this library's SwiGLU kernel between"}
    del w2, y
    entry["forms"] = gate_up_forms(torch, lib, _lib, time_sweep,
                                   fused_call(o, x, wg, wu, rows, dim, hidden, hidden * dim, ends, groups), flops)
    out["B4_routed_131072x2048_to_1408_x64_experts"] = entry
    if int(status.item()) != 0:
        raise RuntimeError(f"fpt_gate_up_swiglu reported status {int(status.item()) & 0xffffffff:#x}")
    del x, wg, wu, o
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
    """Configurations 4 and 5 of the baseline and the reference's two published S=4096 shapes, every polynomial
    score-mod next to its native special-function twin (the reference's B2 / B3 pairs, src/sfu_repro/fa4.py:650-709),
    the plain soft-max control with the routed software exponentials of B5 (:724-752), forward and backward."""
    import ctypes
    _, tensor_peak, _ = measured_peaks()
    sustained = measured_sustained_tflops()
    out = {"published_gb200_speedups_poly_over_native": {"B2_softcap_S4096_fwd_bwd": 2.05, "B3_sigmoid_S4096_fwd_bwd": 1.07,
           "source": "evidence/report-data/b1_b4_100_iteration_phase_probes_gb200.json rows 1-2 (631.4 -> 307.5 us, 395.1 -> 368.0 us)"}}
    g = torch.Generator(device=device)
    g.manual_seed(SEED)
    D = 128
    arr = lambda t: (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2))
    status = torch.zeros(1, dtype=torch.int32, device=device)
    # variants: (label, mode, exp2 backend, forward route, backward route, softcap_grad)
    softcap_pair = (("poly", 0, 0, 0, 0, 0), ("native", 3, 0, 0, 0, 1))
    sigmoid_pair = (("poly", 1, 0, 0, 0, 0), ("native", 4, 0, 0, 0, 0))
    routed = (("native", 2, 0, 0, 0, 0), ("d2_safe_fwd12_bwd32", 2, 2, 12, 32, 0), ("pwl2_safe_f16_fwd12_bwd32", 2, 3, 12, 32, 0),
              ("d3_fwd12_bwd32", 2, 0, 12, 32, 0), ("d3_fwd32_bwd32", 2, 0, 32, 32, 0))
    shapes = (("config4_causal_gqa_softcap50_tanhD4_B4_S8192_Hq32_Hkv8", 4, 8192, 32, 8, 1, 50.0, 12, softcap_pair, True),
              ("config5_sigmoid_direct_B2_S16384_H32", 2, 16384, 32, 32, 0, 0.0, 14, sigmoid_pair, True),
              ("published_shape_softcap30_B1_S4096_Hq32_Hkv8", 1, 4096, 32, 8, 1, 30.0, 12, softcap_pair, True),
              ("published_shape_sigmoid_B1_S4096_Hq32_Hkv8_causal", 1, 4096, 32, 8, 1, 0.0, 12, sigmoid_pair, True),
              ("control_plain_softmax_B4_S8192_Hq32_Hkv8_causal_and_routed_exp2", 4, 8192, 32, 8, 1, 0.0, 12, routed, True))
    for name, B, Sq, Hq, Hk, causal, cap, log2_n, variants, with_backward in shapes:
        q = torch.randn(B, Sq, Hq, D, device=device, generator=g).to(torch.bfloat16)
        k = torch.randn(B, Sq, Hk, D, device=device, generator=g).to(torch.bfloat16)
        v = torch.randn(B, Sq, Hk, D, device=device, generator=g).to(torch.bfloat16)
        dout = torch.randn(B, Sq, Hq, D, device=device, generator=g).to(torch.bfloat16)
        o = torch.empty_like(q)
        lse = torch.empty(B, Hq, Sq, device=device)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        need = int(lib.fpt_attention_bwd_fused_workspace_bytes(B, Sq, Hq))     # large enough for either form of the backward
        workspace = torch.empty(need, dtype=torch.uint8, device=device)
        sq, sk, sv, so, sdo = arr(q), arr(k), arr(v), arr(o), arr(dout)
        flops = 4.0 * B * Hq * Sq * Sq * D * (0.5 if causal else 1.0)
        entry = {"flops_convention": "forward 4*B*Hq*S^2*D, halved when causal; backward 2.5 x that (5 matrix products counted; the "
                                     "two-pass form executes 7: S and dP are recomputed in the dQ and in the dK/dV kernel)"}
        for label, mode, backend, route, route_bwd, grad in variants:
            fwd = [("attn", 0, lambda: _lib.check("fpt_attention_fwd_routed", lib.fpt_attention_fwd_routed(
                o.data_ptr(), lse.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), B, Sq, Hq, Hk, D, sq, sk, sv, so, mode,
                causal, 1.0 / math.sqrt(D), cap, log2_n, backend, route, status.data_ptr(), S())))]
            _, t = time_sweep(fwd, 5, 2)
            tf = flops / (t["attn"] * 1e-3) / 1e12
            entry[label] = {"ms": t["attn"], "tflops": tf, "frac_of_measured_bf16_peak": tf / tensor_peak,
                            "frac_of_sustained_bf16_peak": tf / sustained}
            if label == "poly" and route == 0:
                # the same forward on pairs of CTAs (cta_group::2, opt-in), in the short loop above and in a loop long enough
                # to meet the power cap (launches back to back for about a third of a second)
                long_runs = max(20, int(300.0 / t["attn"]))
                pair_entry = {}
                for key, use_pair in (("single_cta", 0), ("cta_pair", 1)):
                    _lib.check("fpt_set_tuning", lib.fpt_set_tuning(b"attention_cta_pair", use_pair))
                    try:
                        _, ts_ = time_sweep(fwd, 5, 2)
                        _, tl_ = time_sweep(fwd, long_runs, 2)
                    finally:
                        _lib.check("fpt_set_tuning", lib.fpt_set_tuning(b"attention_cta_pair", 0))
                    pair_entry[key] = {"short_loop_tflops": flops / (ts_["attn"] * 1e-3) / 1e12,
                                       "long_loop_tflops": flops / (tl_["attn"] * 1e-3) / 1e12, "long_loop_launches": long_runs}
                entry[label]["forward_on_cta_pairs"] = pair_entry
            if with_backward:
                bwd = [("bwd", 0, lambda: _lib.check("fpt_attention_bwd_routed", lib.fpt_attention_bwd_routed(
                    dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                    o.data_ptr(), lse.data_ptr(), workspace.data_ptr(), need, B, Sq, Hq, Hk, D, sq, sk, sv, so, sdo, mode, causal,
                    1.0 / math.sqrt(D), cap, log2_n, grad, backend, route_bwd, status.data_ptr(), S())))]
                _, tb = time_sweep(bwd, 3, 2)
                tfb = 2.5 * flops / (tb["bwd"] * 1e-3) / 1e12
                entry[label]["backward"] = {"ms": tb["bwd"], "tflops": tfb, "frac_of_measured_bf16_peak": tfb / tensor_peak,
                                            "frac_of_sustained_bf16_peak": tfb / sustained,
                                            "form": "single pass, 5 matrix products, dQ accumulated in fp32 by reduce-add copies "
                                                    "(the default when the workspace holds the fp32 dQ buffer)"}
                if label in ("poly", "native") and route_bwd == 0:
                    # the deterministic form: two passes, 7 products, no additions in memory (tuning key off)
                    _lib.check("fpt_set_tuning", lib.fpt_set_tuning(b"attention_bwd_fused", 0))
                    try:
                        _, ts = time_sweep(bwd, 3, 2)
                    finally:
                        _lib.check("fpt_set_tuning", lib.fpt_set_tuning(b"attention_bwd_fused", 1))
                    entry[label]["backward_two_passes"] = {"ms": ts["bwd"], "tflops": 2.5 * flops / (ts["bwd"] * 1e-3) / 1e12,
                                                           "single_pass_speedup": ts["bwd"] / tb["bwd"]}
            if int(status.item()) != 0:
                raise RuntimeError(f"attention kernel reported status {int(status.item()) & 0xffffffff:#x} in {name}/{label}")
        base = entry["native"]
        for label, *_ in variants:
            if label == "native":
                continue
            e = entry[label]
            e["speedup_vs_native"] = base["ms"] / e["ms"]
            if "backward" in e:
                e["backward"]["speedup_vs_native"] = base["backward"]["ms"] / e["backward"]["ms"]
                e["fwd_bwd_speedup_vs_native"] = (base["ms"] + base["backward"]["ms"]) / (e["ms"] + e["backward"]["ms"])
        out[name] = entry
        del q, k, v, dout, o, lse, dq, dk, dv, workspace
    torch.cuda.empty_cache()
    return out


def bench_e2e(torch, spline_ops, HostPipeline, device, steps, barrier):
    """The sweep from pinned host memory through spline_ops at the headline size (2^28 elements per function): chunked
    H2D -> kernel -> D2H on three streams, `steps` timed repetitions.  Beside it the same chunked copies with no kernel
    between them: what the host's copy path delivers when this many ranks use it at once."""
    n = N_HBM
    chunk = 1 << 23
    g = torch.Generator(device=device)
    g.manual_seed(SEED)

    def pinned_from_device(make):
        t = make()
        host = torch.empty(t.shape, dtype=t.dtype).pin_memory()
        host.copy_(t)
        return host
    host_u8 = pinned_from_device(lambda: (torch.rand(n, device=device, generator=g) * 16 - 8).to(torch.float16))
    host_frac = pinned_from_device(lambda: torch.rand(n, device=device, generator=g).to(torch.float16))
    host_ang = pinned_from_device(lambda: torch.rand(n, device=device, generator=g) * (2 * math.pi) - math.pi)
    torch.cuda.empty_cache()
    host_out = torch.empty(n, dtype=torch.float16).pin_memory()
    host_sc = torch.empty(2 * n, dtype=torch.float16).pin_memory()
    unary_pipe = HostPipeline(device, [(torch.float16, 1)], [(torch.float16, 1)], chunk)
    # sin/cos keeps the two planes of a chunk adjacent in the device buffer; the host copy de-interleaves per chunk
    sincos_pipe = HostPipeline(device, [(torch.float32, 1)], [(torch.float16, 2)], chunk)

    def run_once(compute=True):
        for op, src in ((spline_ops.sigmoid_fwd_d3, host_u8), (spline_ops.tanh_fwd_d4, host_u8),
                        (spline_ops.swish_fwd_d3, host_u8), (spline_ops.exp2_fraction, host_frac)):
            def fn(ins, outs, m, op=op):
                if compute:
                    outs[0].copy_(op(ins[0]))
            unary_pipe.run(fn, [src], [host_out], n)
        def fn_sc(ins, outs, m):
            if compute:
                outs[0].copy_(spline_ops.sincos_d5_d6_half_turn_fp16(ins[0]).view(-1))
        sincos_pipe.run(fn_sc, [host_ang], [host_sc], n)
        unary_pipe.synchronize()
        sincos_pipe.synchronize()

    def timed(compute, reps):
        run_once(compute)
        barrier()
        t0 = time.perf_counter()
        for _ in range(reps):
            run_once(compute)
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / reps
    dt = timed(True, steps)
    dt_copy = timed(False, max(3, steps // 4))
    h2d = 4 * n * 2 + n * 4
    d2h = 4 * n * 2 + 2 * n * 2
    return {"value": 5 * n / dt, "unit": "elements/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "elements_per_function": n, "ms_per_step": dt * 1e3, "steps": steps,
            "path": "spline_ops.* on pinned host buffers, 2^23-element chunks, H2D / kernel / D2H on three streams; "
                    "sin/cos results are returned chunk by chunk as [cos | sin] blocks",
            "copy_only": {"ms_per_step": dt_copy * 1e3, "steps": max(3, steps // 4),
                          "what": "the same pinned H2D and D2H copies, same chunks and streams, no kernel"}}


def run_compare_reference_kernels(args):
    """This library's kernels next to the reference's own kernels (compiled from the reference's sources with its flags
    into oracle/_ref by `make -C oracle ref`) on the same GPU, same inputs, same timing protocol: median over 7 rounds of
    the mean of back-to-back launches; L2-resident sizes also as CUDA-graph replays (no host launch cost) and as eager
    calls through the Python operator surface.  Prints one JSON line {"compare_reference_kernels": [rows]}."""
    import ctypes

    import numpy as np
    import torch
    from fast_polynomial_transcendentals_b200 import _lib, spline_ops
    path = ROOT / "oracle" / "_ref" / "libref_spline_kernels.so"
    if not path.exists():
        print(json.dumps({"compare_reference_kernels": "unavailable: oracle/_ref/libref_spline_kernels.so is not built"}))
        return
    ref_kernels = ctypes.CDLL(str(path))
    lib = _lib.load()
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    vp, ci = ctypes.c_void_p, ctypes.c_int
    rows = []

    def timed(fn, reps, rounds=7, graph=False):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        runner = fn
        if graph:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(g, stream=side):
                    for _ in range(reps):
                        fn(side.cuda_stream)
            torch.cuda.current_stream().wait_stream(side)
            runner = g.replay
        times = []
        for _ in range(rounds):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            if graph:
                runner()
            else:
                for _ in range(reps):
                    fn()
            b.record()
            torch.cuda.synchronize()
            times.append(a.elapsed_time(b) / reps)
        times.sort()
        return times[len(times) // 2]

    def ref(symbol, *a):
        f = getattr(ref_kernels, symbol)
        f.restype = None
        conv = [vp(x.data_ptr()) if hasattr(x, "data_ptr") else ci(int(x)) for x in a]
        return lambda s=None: f(*conv, vp(s or torch.cuda.current_stream().cuda_stream))

    def ours(name, *a):
        f = getattr(lib, name)
        return lambda s=None: f(*a, s or torch.cuda.current_stream().cuda_stream)

    def row(what, t_ref, t_our, nbytes=None):
        r = {"what": what, "ref_ms": t_ref, "ours_ms": t_our, "ours_over_ref_speed": t_ref / t_our}
        if nbytes:
            r.update(ref_gbs=nbytes / t_ref / 1e6, ours_gbs=nbytes / t_our / 1e6)
        rows.append(r)

    n = 1 << 28
    x = (torch.rand(n, device=device) * 16 - 8).to(torch.float16)
    o = torch.empty_like(x)
    for fn_name, fn, degree in (("sigmoid", 0, 3), ("tanh", 1, 4), ("swish", 2, 3), ("gelu", 4, 5)):
        row(f"{fn_name}_fwd_d{degree}_fp16_2^28", timed(ref(f"launch_{fn_name}_fwd_d{degree}_kernel", o, x, n), 10),
            timed(ours("fpt_unary", o.data_ptr(), x.data_ptr(), n, fn, 0, degree, 0, 0), 10), 4 * n)
    row("swish_native_fp16_2^28", timed(ref("launch_swish_fwd_native_kernel", o, x, n), 10),
        timed(ours("fpt_unary", o.data_ptr(), x.data_ptr(), n, 2, 0, 0, 0, 0), 10), 4 * n)
    t_torch = timed(lambda s=None: torch.sigmoid(x, out=o), 10)
    rows.append({"what": "torch_sigmoid_fp16_2^28", "torch_ms": t_torch, "torch_gbs": 4 * n / t_torch / 1e6})
    go = torch.randn(n, device=device).to(torch.float16)
    for fn_name, fn, degree in (("sigmoid", 0, 4), ("swish", 2, 3)):
        row(f"{fn_name}_bwd_d{degree}_fp16_2^28", timed(ref(f"launch_{fn_name}_bwd_d{degree}_kernel", o, go, x, n), 10),
            timed(ours("fpt_binary_bwd", o.data_ptr(), go.data_ptr(), x.data_ptr(), n, fn, degree, 0, 0), 10), 6 * n)
    del go
    for m in (1 << 20, 1 << 22):     # L2-resident: eager C-ABI calls, graph replays, and the Python operator surface
        xs, os_ = x[:m], o[:m]
        e = {"what": f"sigmoid_fwd_d3_fp16_{m}"}
        e["ref_us"] = timed(ref("launch_sigmoid_fwd_d3_kernel", os_, xs, m), 200) * 1e3
        e["ours_us"] = timed(ours("fpt_unary", os_.data_ptr(), xs.data_ptr(), m, 0, 0, 3, 0, 0), 200) * 1e3
        e["ours_native_us"] = timed(ours("fpt_unary", os_.data_ptr(), xs.data_ptr(), m, 0, 0, 0, 0, 0), 200) * 1e3
        e["torch_native_us"] = timed(lambda s=None: torch.sigmoid(xs, out=os_), 200) * 1e3
        e["ours_python_op_us"] = timed(lambda s=None: spline_ops.sigmoid_fwd_d3(xs), 200) * 1e3
        e["ours_python_op_path"] = spline_ops.binding_kind()
        e["torch_native_allocating_us"] = timed(lambda s=None: torch.sigmoid(xs), 200) * 1e3
        e["ref_graph_us"] = timed(ref("launch_sigmoid_fwd_d3_kernel", os_, xs, m), 50, graph=True) * 1e3
        e["ours_graph_us"] = timed(ours("fpt_unary", os_.data_ptr(), xs.data_ptr(), m, 0, 0, 3, 0, 0), 50, graph=True) * 1e3
        e["ours_native_graph_us"] = timed(ours("fpt_unary", os_.data_ptr(), xs.data_ptr(), m, 0, 0, 0, 0, 0), 50, graph=True) * 1e3
        rows.append(e)
    m = 1 << 27
    ang = torch.rand(m, device=device) * 6.2831853 - 3.14159265
    sc = torch.empty(2, m, dtype=torch.float16, device=device)
    row("sincos_d5_d6_half_turn_fp16_2^27", timed(ref("launch_sincos_d5_d6_half_turn_fp16", sc, ang, m), 10),
        timed(ours("fpt_sincos", sc.data_ptr(), ang.data_ptr(), m, 3, 0), 10), 8 * m)
    row("sincos_native_fp16_2^27", timed(ref("launch_sincos_native_fp16", sc, ang, m), 10),
        timed(ours("fpt_sincos", sc.data_ptr(), ang.data_ptr(), m, 10, 0), 10), 8 * m)
    del x, o, ang, sc
    torch.cuda.empty_cache()
    for name, r, h in (("B1_16384x14336", 16384, 14336), ("B4_131072x1408", 131072, 1408)):
        packed = (torch.randn(r, 2 * h, device=device) * 1.5).to(torch.bfloat16)
        gate, up = packed[:, :h].contiguous(), packed[:, h:].contiguous()
        out = torch.empty_like(gate)
        nn = r * h
        row(f"swiglu_flat_d3_bf16_{name}", timed(ref("launch_swish_mul_fwd_d3_kernel_bf16", out, gate, up, nn), 10),
            timed(ours("fpt_swish_mul", out.data_ptr(), gate.data_ptr(), up.data_ptr(), nn, 3, 1, 0), 10), 6 * nn)
        row(f"swiglu_packed_d3_bf16_{name}", timed(ref("launch_swish_mul_packed_fwd_d3_kernel_bf16", out, packed, r, h), 10),
            timed(ours("fpt_swish_mul_packed", out.data_ptr(), packed.data_ptr(), r, h, 3, 1, 0), 10), 6 * nn)
        go = torch.randn(r, h, device=device).to(torch.bfloat16)
        gp = torch.empty_like(packed)
        row(f"swiglu_packed_bwd_d3_bf16_{name}", timed(ref("launch_swish_mul_packed_bwd_d3_kernel_bf16", gp, go, packed, r, h), 10),
            timed(ours("fpt_swish_mul_packed_bwd", gp.data_ptr(), go.data_ptr(), packed.data_ptr(), r, h, 3, 1, 0), 10), 10 * nn)
        del packed, gate, up, out, go, gp
        torch.cuda.empty_cache()
    B, S, H, D = 2, 16384, 32, 128
    q = torch.randn(B, S, H, D, device=device).to(torch.float16)
    k = torch.randn(B, S, H, D, device=device).to(torch.float16)
    qo, ko = torch.empty(B, H, S, D, dtype=q.dtype, device=device), torch.empty(B, H, S, D, dtype=q.dtype, device=device)
    freqs = 500000.0 ** (-np.arange(0, D, 2, dtype=np.float64) / D)
    inc = torch.from_numpy(np.round(freqs * 2.0 ** 32 / (2 * math.pi)).astype(np.int64).astype(np.uint32).view(np.int32)).to(device)
    row("rope_apply_d5_d6_fp16_B2_S16384_H32_D128",
        timed(ref("launch_rope_apply_fixed_half_turn_d5_d6_fp16", qo, ko, q, k, inc, B, S, H, H, D), 10),
        timed(ours("fpt_rope_apply", qo.data_ptr(), ko.data_ptr(), q.data_ptr(), k.data_ptr(), inc.data_ptr(), B, S, H, H, D, 0, 0), 10),
        4 * q.numel() * 2)
    print(json.dumps({"compare_reference_kernels": rows}), flush=True)


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
    elif case in ("attn_softcap", "attn_sigmoid", "attn_softmax", "attn_softmax_full", "attn_softcap_full",
                  "attn_softcap_native_full", "attn_sigmoid_native"):
        import ctypes
        B, S, Hq, Hk, D = 1, n, 32, 8, 128      # --profile-n is the sequence length here
        mode = {"attn_softcap": 0, "attn_sigmoid": 1, "attn_softmax": 2, "attn_softmax_full": 2, "attn_softcap_full": 0,
                "attn_softcap_native_full": 3, "attn_sigmoid_native": 4}[case]
        causal = 0 if mode in (1, 4) or case.endswith("_full") else 1   # "_full": every key tile, no mask
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
    elif case in ("attn_bwd_softmax", "attn_bwd_softcap", "attn_bwd_sigmoid",
                  "attn_bwd_single_pass_softmax", "attn_bwd_single_pass_softcap", "attn_bwd_single_pass_sigmoid"):
        import ctypes
        B, S, Hq, Hk, D = 1, n, 32, 8, 128      # --profile-n is the sequence length; no mask
        single_pass = "_single_pass_" in case   # the workspace decides: with the fp32 dQ buffer the single-pass kernel runs
        mode = {"softcap": 0, "sigmoid": 1, "softmax": 2}[case.rsplit("_", 1)[1]]
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
        need = int((lib.fpt_attention_bwd_fused_workspace_bytes if single_pass else lib.fpt_attention_bwd_workspace_bytes)(B, S, Hq))
        workspace = torch.empty(need, dtype=torch.uint8, device=device)
        run = lambda: _lib.check("fpt_attention_bwd", lib.fpt_attention_bwd(
            dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
            lse.data_ptr(), workspace.data_ptr(), need, B, S, Hq, Hk, D, arr(q), arr(k), arr(v), arr(o), arr(dout), mode, 0,
            1.0 / math.sqrt(D), 50.0, 12, 0, status.data_ptr(), stream))
    elif case in ("gate_up_dense", "gate_up_grouped", "gate_up_dense_pair"):
        if case.endswith("_pair"):                      # pairs of CTAs (the default form), asked for by name
            _lib.check("fpt_set_tuning", lib.fpt_set_tuning(b"gate_up_cta_pair", 1))
            case = "gate_up_dense"
        elif case == "gate_up_dense":                   # one CTA per tile of 256 rows
            _lib.check("fpt_set_tuning", lib.fpt_set_tuning(b"gate_up_cta_pair", 0))
        # --profile-n is the number of rows; dim 4096 -> hidden 3584 (dense) or 16 groups of dim 2048 -> hidden 1408
        rows = n
        dim, hidden, groups = (4096, 3584, 1) if case == "gate_up_dense" else (2048, 1408, 16)
        x = torch.randn(rows, dim, device=device, generator=g).to(torch.bfloat16)
        wg = (torch.randn(groups, hidden, dim, device=device, generator=g) * dim ** -0.5).to(torch.bfloat16)
        wu = (torch.randn(groups, hidden, dim, device=device, generator=g) * dim ** -0.5).to(torch.bfloat16)
        o = torch.empty(rows, hidden, dtype=torch.bfloat16, device=device)
        status = torch.zeros(1, dtype=torch.int32, device=device)
        ends = torch.linspace(rows / groups, rows, groups).to(torch.int32).to(device) if groups > 1 else None
        run = lambda: _lib.check("fpt_gate_up_swiglu", lib.fpt_gate_up_swiglu(
            o.data_ptr(), x.data_ptr(), wg.data_ptr(), wu.data_ptr(), rows, dim, hidden, dim, dim, hidden * dim, hidden,
            ends.data_ptr() if ends is not None else None, groups, 3, 0, 0, status.data_ptr(), stream))
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
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--compare-reference-kernels", action="store_true",
                    help="time this library's kernels next to the reference's compiled kernels (oracle/_ref), 1 GPU")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.profile_case:
        run_profile_case(args)
    elif args.compare_reference_kernels:
        run_compare_reference_kernels(args)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()

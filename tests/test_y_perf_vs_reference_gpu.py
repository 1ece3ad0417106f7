"""GPU: throughput of our kernels next to the reference's own kernels (compiled from the reference sources into
oracle/_ref with the reference's flags) on the same B200, same inputs, same timing protocol.  Writes the table as
perf_vs_reference.json into the directory named by FPT_PERF_OUT (default: a scratch folder at the repository root)
and asserts only that we are not slower than the reference beyond noise."""
import ctypes
import json
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def timed(fn, reps, rounds=7, graph=False):
    import torch
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    runner = fn
    if graph:  # replay `reps` launches from one CUDA graph: no host launch cost inside the timed region
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


def test_throughput_next_to_reference_kernels(fpt, cuda, ref_kernels):
    import torch
    lib = fpt.load()
    vp, ci = ctypes.c_void_p, ctypes.c_int
    rows = []

    def ref(symbol, *args):
        f = getattr(ref_kernels, symbol)
        f.restype = None
        conv = [vp(a.data_ptr()) if hasattr(a, "data_ptr") else ci(int(a)) for a in args]
        return lambda s=None: f(*conv, vp(s or torch.cuda.current_stream().cuda_stream))

    def ours(name, *args):
        f = getattr(lib, name)
        return lambda s=None: f(*args, s or torch.cuda.current_stream().cuda_stream)

    # HBM endpoint, fp16 unary
    n = 1 << 28
    x = (torch.rand(n, device=cuda) * 16 - 8).to(torch.float16)
    o = torch.empty_like(x)
    for fn_name, fn, degree in (("sigmoid", 0, 3), ("tanh", 1, 4), ("swish", 2, 3), ("gelu", 4, 5)):
        t_ref = timed(ref(f"launch_{fn_name}_fwd_d{degree}_kernel", o, x, n), 10)
        t_our = timed(ours("fpt_unary", o.data_ptr(), x.data_ptr(), n, fn, 0, degree, 0, 0), 10)
        rows.append({"what": f"{fn_name}_fwd_d{degree}_fp16_2^28", "ref_ms": t_ref, "ours_ms": t_our,
                     "ref_gbs": 4 * n / t_ref / 1e6, "ours_gbs": 4 * n / t_our / 1e6})
    t_ref = timed(ref("launch_swish_fwd_native_kernel", o, x, n), 10)
    t_our = timed(ours("fpt_unary", o.data_ptr(), x.data_ptr(), n, 2, 0, 0, 0, 0), 10)
    rows.append({"what": "swish_native_fp16_2^28", "ref_ms": t_ref, "ours_ms": t_our})
    t_torch = timed(lambda s=None: torch.sigmoid(x, out=o), 10)
    rows.append({"what": "torch_sigmoid_fp16_2^28", "torch_ms": t_torch, "torch_gbs": 4 * n / t_torch / 1e6})
    go = torch.randn(n, device=cuda).to(torch.float16)
    for fn_name, fn, degree in (("sigmoid", 0, 4), ("swish", 2, 3)):
        t_ref = timed(ref(f"launch_{fn_name}_bwd_d{degree}_kernel", o, go, x, n), 10)
        t_our = timed(ours("fpt_binary_bwd", o.data_ptr(), go.data_ptr(), x.data_ptr(), n, fn, degree, 0, 0), 10)
        rows.append({"what": f"{fn_name}_bwd_d{degree}_fp16_2^28", "ref_ms": t_ref, "ours_ms": t_our,
                     "ref_gbs": 6 * n / t_ref / 1e6, "ours_gbs": 6 * n / t_our / 1e6})
    del go
    # L2-resident endpoints: eager calls and graph replays (kernel-side time without host launch cost)
    for m in (1 << 20, 1 << 22):
        xs, os_ = x[:m], o[:m]
        entry = {"what": f"sigmoid_fwd_d3_fp16_{m}"}
        entry["ref_us"] = timed(ref("launch_sigmoid_fwd_d3_kernel", os_, xs, m), 200) * 1e3
        entry["ours_us"] = timed(ours("fpt_unary", os_.data_ptr(), xs.data_ptr(), m, 0, 0, 3, 0, 0), 200) * 1e3
        entry["ours_native_us"] = timed(ours("fpt_unary", os_.data_ptr(), xs.data_ptr(), m, 0, 0, 0, 0, 0), 200) * 1e3
        entry["torch_native_us"] = timed(lambda s=None: torch.sigmoid(xs, out=os_), 200) * 1e3
        entry["ref_graph_us"] = timed(ref("launch_sigmoid_fwd_d3_kernel", os_, xs, m), 50, graph=True) * 1e3
        entry["ours_graph_us"] = timed(ours("fpt_unary", os_.data_ptr(), xs.data_ptr(), m, 0, 0, 3, 0, 0), 50, graph=True) * 1e3
        entry["ours_native_graph_us"] = timed(ours("fpt_unary", os_.data_ptr(), xs.data_ptr(), m, 0, 0, 0, 0, 0), 50, graph=True) * 1e3
        rows.append(entry)
    # sin/cos at 2^27 angles
    m = 1 << 27
    ang = (torch.rand(m, device=cuda) * 6.2831853 - 3.14159265)
    sc = torch.empty(2, m, dtype=torch.float16, device=cuda)
    t_ref = timed(ref("launch_sincos_d5_d6_half_turn_fp16", sc, ang, m), 10)
    t_our = timed(ours("fpt_sincos", sc.data_ptr(), ang.data_ptr(), m, 3, 0), 10)
    rows.append({"what": "sincos_d5_d6_half_turn_fp16_2^27", "ref_ms": t_ref, "ours_ms": t_our,
                 "ref_gbs": 8 * m / t_ref / 1e6, "ours_gbs": 8 * m / t_our / 1e6})
    t_ref = timed(ref("launch_sincos_native_fp16", sc, ang, m), 10)
    t_our = timed(ours("fpt_sincos", sc.data_ptr(), ang.data_ptr(), m, 10, 0), 10)
    rows.append({"what": "sincos_native_fp16_2^27", "ref_ms": t_ref, "ours_ms": t_our})
    del x, o, ang, sc
    torch.cuda.empty_cache()
    # SwiGLU bf16
    for name, r, h in (("B1_16384x14336", 16384, 14336), ("B4_131072x1408", 131072, 1408)):
        packed = (torch.randn(r, 2 * h, device=cuda) * 1.5).to(torch.bfloat16)
        g, u = packed[:, :h].contiguous(), packed[:, h:].contiguous()
        out = torch.empty_like(g)
        nn = r * h
        t_ref = timed(ref("launch_swish_mul_fwd_d3_kernel_bf16", out, g, u, nn), 10)
        t_our = timed(ours("fpt_swish_mul", out.data_ptr(), g.data_ptr(), u.data_ptr(), nn, 3, 1, 0), 10)
        rows.append({"what": f"swiglu_flat_d3_bf16_{name}", "ref_ms": t_ref, "ours_ms": t_our,
                     "ref_gbs": 6 * nn / t_ref / 1e6, "ours_gbs": 6 * nn / t_our / 1e6})
        t_ref = timed(ref("launch_swish_mul_packed_fwd_d3_kernel_bf16", out, packed, r, h), 10)
        t_our = timed(ours("fpt_swish_mul_packed", out.data_ptr(), packed.data_ptr(), r, h, 3, 1, 0), 10)
        rows.append({"what": f"swiglu_packed_d3_bf16_{name}", "ref_ms": t_ref, "ours_ms": t_our,
                     "ref_gbs": 6 * nn / t_ref / 1e6, "ours_gbs": 6 * nn / t_our / 1e6})
        go = torch.randn(r, h, device=cuda).to(torch.bfloat16)
        gp = torch.empty_like(packed)
        t_ref = timed(ref("launch_swish_mul_packed_bwd_d3_kernel_bf16", gp, go, packed, r, h), 10)
        t_our = timed(ours("fpt_swish_mul_packed_bwd", gp.data_ptr(), go.data_ptr(), packed.data_ptr(), r, h, 3, 1, 0), 10)
        rows.append({"what": f"swiglu_packed_bwd_d3_bf16_{name}", "ref_ms": t_ref, "ours_ms": t_our,
                     "ref_gbs": 10 * nn / t_ref / 1e6, "ours_gbs": 10 * nn / t_our / 1e6})
        del packed, g, u, out, go, gp
        torch.cuda.empty_cache()
    # fused RoPE, configuration-5 shape in fp16 (reference dtype)
    B, S, H, D = 2, 16384, 32, 128
    q = torch.randn(B, S, H, D, device=cuda).to(torch.float16)
    k = torch.randn(B, S, H, D, device=cuda).to(torch.float16)
    qo, ko = torch.empty(B, H, S, D, dtype=q.dtype, device=cuda), torch.empty(B, H, S, D, dtype=q.dtype, device=cuda)
    import math
    import numpy as np
    freqs = 500000.0 ** (-np.arange(0, D, 2, dtype=np.float64) / D)
    inc = torch.from_numpy(np.round(freqs * 2.0 ** 32 / (2 * math.pi)).astype(np.int64).astype(np.uint32).view(np.int32)).to(cuda)
    t_ref = timed(ref("launch_rope_apply_fixed_half_turn_d5_d6_fp16", qo, ko, q, k, inc, B, S, H, H, D), 10)
    t_our = timed(ours("fpt_rope_apply", qo.data_ptr(), ko.data_ptr(), q.data_ptr(), k.data_ptr(), inc.data_ptr(),
                       B, S, H, H, D, 0, 0), 10)
    by = 4 * q.numel() * 2
    rows.append({"what": "rope_apply_d5_d6_fp16_B2_S16384_H32_D128", "ref_ms": t_ref, "ours_ms": t_our,
                 "ref_gbs": by / t_ref / 1e6, "ours_gbs": by / t_our / 1e6})
    import os
    out_dir = Path(os.environ.get("FPT_PERF_OUT", ROOT / "gpurun_out"))
    out_dir.mkdir(exist_ok=True)
    (out_dir / "perf_vs_reference.json").write_text(json.dumps(rows, indent=1))
    for row in rows:
        print(json.dumps(row))
    for row in rows:
        if "ref_ms" in row and "ours_ms" in row:
            assert row["ours_ms"] <= 1.10 * row["ref_ms"], row

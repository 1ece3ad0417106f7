"""Generates include/fpt_b200_compat.h and csrc/fpt_compat_launch.cpp: `launch_*` entry points with the reference's
names, argument order and `void` return (reference: autonumerics_zero/spline_ops/spline_ops.cpp:14-288), each a thin
call into the status-returning `fpt_*` C ABI.  A maintainer can link the reference's torch-facing C++ against
libfpt_b200_compat.so instead of compiling its own .cu files.

    python fast_polynomial_transcendentals_b200/csrc/gen_compat_launch.py
"""
from pathlib import Path

HERE = Path(__file__).resolve().parent
S = "cudaStream_t s"
FUNCS = {"sigmoid": "FPT_FN_SIGMOID", "tanh": "FPT_FN_TANH", "swish": "FPT_FN_SWISH", "gelu": "FPT_FN_GELU"}
SUFFIXES = {"": ("FPT_FP16", "FPT_SRC_CURRENT"), "_bf16": ("FPT_BF16", "FPT_SRC_CURRENT"),
            "_bf16_sollya": ("FPT_BF16", "FPT_SRC_SOLLYA")}

entries: list[tuple[str, str, str]] = []   # (name, parameter list, call expression)


def add(name: str, params: str, call: str) -> None:
    entries.append((name, params, call))


# unary forward / gradient products, degrees 3..6, three coefficient tables
for fn, code in FUNCS.items():
    for suffix, (dt, src) in SUFFIXES.items():
        if suffix == "_bf16_sollya" and fn == "tanh":
            continue   # the reference ships no Sollya tanh launchers
        for d in (3, 4, 5, 6):
            add(f"launch_{fn}_fwd_d{d}_kernel{suffix}", f"void* out, const void* in, int size, {S}",
                f"fpt_unary(out, in, size, {code}, FPT_FWD, {d}, {dt}, {src}, s)")
            add(f"launch_{fn}_bwd_d{d}_kernel{suffix}", f"void* gi, const void* go, const void* in, int size, {S}",
                f"fpt_binary_bwd(gi, go, in, size, {code}, {d}, {dt}, {src}, s)")

# SwiGLU: flat and packed, forward and backward; degree 0 = the SFU control
for suffix, (dt, src) in SUFFIXES.items():
    degrees = [("native", 0)] if suffix != "_bf16_sollya" else []
    degrees += [(f"d{d}", d) for d in (3, 4, 5, 6)]
    for tag, d in degrees:
        add(f"launch_swish_mul_fwd_{tag}_kernel{suffix}", f"void* out, const void* gate, const void* up, int size, {S}",
            f"fpt_swish_mul(out, gate, up, size, {d}, {dt}, {src}, s)")
        add(f"launch_swish_mul_bwd_{tag}_kernel{suffix}",
            f"void* grad_gate, void* grad_up, const void* grad_out, const void* gate, const void* up, int size, {S}",
            f"fpt_swish_mul_bwd(grad_gate, grad_up, grad_out, gate, up, size, {d}, {dt}, {src}, s)")
        add(f"launch_swish_mul_packed_fwd_{tag}_kernel{suffix}",
            f"void* out, const void* packed, int rows, int hidden_size, {S}",
            f"fpt_swish_mul_packed(out, packed, rows, hidden_size, {d}, {dt}, {src}, s)")
        add(f"launch_swish_mul_packed_bwd_{tag}_kernel{suffix}",
            f"void* grad_packed, const void* grad_out, const void* packed, int rows, int hidden_size, {S}",
            f"fpt_swish_mul_packed_bwd(grad_packed, grad_out, packed, rows, hidden_size, {d}, {dt}, {src}, s)")
for suffix, dt in (("", "FPT_FP16"), ("_bf16", "FPT_BF16")):
    add(f"launch_swish_fwd_native_kernel{suffix}", f"void* out, const void* in, int size, {S}",
        f"fpt_unary(out, in, size, FPT_FN_SWISH, FPT_FWD, 0, {dt}, FPT_SRC_CURRENT, s)")
    add(f"launch_swish_bwd_native_kernel{suffix}", f"void* gi, const void* go, const void* in, int size, {S}",
        f"fpt_binary_bwd(gi, go, in, size, FPT_FN_SWISH, 0, {dt}, FPT_SRC_CURRENT, s)")
    for fn in ("sigmoid", "tanh"):
        add(f"launch_{fn}_bwd_alg_kernel{suffix}", f"void* gi, const void* go, const void* y, int size, {S}",
            f"fpt_bwd_algebraic(gi, go, y, size, {FUNCS[fn]}, {dt}, s)")

# FP16 composites
for fn in ("sigmoid", "tanh", "swish"):
    code = FUNCS[fn]
    add(f"launch_{fn}_fwd_hybrid_kernel", f"void* out, const void* in, int size, {S}",
        f"fpt_unary_hybrid(out, in, size, {code}, s)")
    add(f"launch_{fn}_bwd_hybrid_kernel", f"void* gi, const void* go, const void* in, int size, {S}",
        f"fpt_binary_bwd_hybrid(gi, go, in, size, {code}, s)")
    add(f"launch_{fn}_fused_kernel", f"void* y_out, void* gi_out, const void* x_in, const void* go_in, int size, {S}",
        f"fpt_fused_fwd_bwd(y_out, gi_out, x_in, go_in, size, {code}, s)")
for name, fn, variant in (("sigmoid_fwd_deriv_alg", "sigmoid", "FPT_DERIV_ALGEBRAIC"),
                          ("sigmoid_fwd_deriv_poly", "sigmoid", "FPT_DERIV_POLY"),
                          ("tanh_fwd_deriv_alg", "tanh", "FPT_DERIV_ALGEBRAIC"),
                          ("tanh_fwd_deriv_poly", "tanh", "FPT_DERIV_POLY"),
                          ("swish_fwd_deriv", "swish", "FPT_DERIV_SHARED_SIGMOID"),
                          ("swish_fwd_deriv_poly", "swish", "FPT_DERIV_POLY")):
    add(f"launch_{name}_kernel", f"void* y, void* dy, const void* x, int size, {S}",
        f"fpt_fwd_deriv(y, dy, x, size, {FUNCS[fn]}, {variant}, s)")
add("launch_multiply_kernel", f"void* out, const void* a, const void* b, int size, {S}",
    "fpt_multiply(out, a, b, size, FPT_FP16, s)")

# paired sin/cos: fp32 family, packed 16-bit family, plain and repeated-evaluation probes
F32 = ("native", "d3_d4", "d3_d4_cycle", "d3_d4_magic_bias", "d5_d4_half_turn_ls", "d5_d4_half_turn_sollya",
       "d5_d4_half_turn_sollya_fast", "d5_d4", "d7_d6")
for i, v in enumerate(F32):
    add(f"launch_sincos_{v}_f32", f"void* out, const void* in, int size, {S}", f"fpt_sincos_f32(out, in, size, {i}, 0, s)")
    add(f"launch_sincos_{v}_compute_f32", f"void* out, const void* in, int size, int iterations, {S}",
        f"fpt_sincos_f32(out, in, size, {i}, positive(iterations), s)")
PACKED = {"d3_d4_quarter_turn_fp16": 0, "d3_d4_half_turn_fp16": 1, "d5_d4_half_turn_fp16": 2, "d5_d6_half_turn_fp16": 3,
          "d7_d6_half_turn_fp16": 4, "d3_d4_bf16": 5, "d3_d4_quarter_turn_bf16": 6, "d3_d4_half_turn_bf16": 7,
          "d5_d6_half_turn_bf16": 8, "d5_d4_half_turn_fp16_bf16": 9, "native_fp16": 10, "native_bf16": 11}
for v, i in PACKED.items():
    add(f"launch_sincos_{v}", f"void* out, const void* in, int size, {S}", f"fpt_sincos(out, in, size, {i}, 0, s)")
    add(f"launch_sincos_{v}_compute", f"void* out, const void* in, int size, int iterations, {S}",
        f"fpt_sincos(out, in, size, {i}, positive(iterations), s)")

# RoPE tables and fused rotation
for name, param, kind in (("native", "frequencies", "FPT_ROPE_NATIVE"), ("fixed_d3_d4", "phase_increments", "FPT_ROPE_QUARTER_TURN_D3_D4"),
                          ("fixed_half_turn_d5_d6", "phase_increments", "FPT_ROPE_HALF_TURN_D5_D6")):
    add(f"launch_rope_sincos_{name}_fp16", f"void* out, const void* {param}, int sequence_length, int frequency_count, {S}",
        f"fpt_rope_table(out, {param}, sequence_length, frequency_count, {kind}, 0, s)")
    add(f"launch_rope_sincos_{name}_fp16_compute",
        f"void* out, const void* {param}, int sequence_length, int frequency_count, int iterations, {S}",
        f"fpt_rope_table(out, {param}, sequence_length, frequency_count, {kind}, positive(iterations), s)")
add("launch_rope_sincos_fixed_lut_fp16",
    f"void* out, const void* phase_increments, const void* phase_table, int sequence_length, int frequency_count, {S}",
    "fpt_rope_table_lut(out, phase_increments, phase_table, sequence_length, frequency_count, 0, s)")
add("launch_rope_sincos_fixed_lut_fp16_compute",
    f"void* out, const void* phase_increments, const void* phase_table, int sequence_length, int frequency_count, "
    f"int iterations, {S}",
    "fpt_rope_table_lut(out, phase_increments, phase_table, sequence_length, frequency_count, positive(iterations), s)")
for name, param, kind in (("cached", "rope_table", "FPT_ROPE_CACHED"), ("native", "frequencies", "FPT_ROPE_NATIVE"),
                          ("fixed_half_turn_d5_d6", "phase_increments", "FPT_ROPE_HALF_TURN_D5_D6")):
    add(f"launch_rope_apply_{name}_fp16",
        f"void* q_out, void* k_out, const void* q, const void* k, const void* {param}, int batch_size, int sequence_length, "
        f"int q_head_count, int k_head_count, int head_dim, {S}",
        f"fpt_rope_apply(q_out, k_out, q, k, {param}, batch_size, sequence_length, q_head_count, k_head_count, head_dim, "
        f"{kind}, FPT_FP16, s)")

HEADER_TOP = '''/* Generated by fast_polynomial_transcendentals_b200/csrc/gen_compat_launch.py -- do not edit.
 *
 * The reference's C++ <-> CUDA boundary, name for name (reference: autonumerics_zero/spline_ops/spline_ops.cpp:14-288):
 * `extern "C" void launch_*(pointers..., int sizes..., cudaStream_t)`, raw device pointers owned by the caller,
 * no return value.  Each entry forwards to the status-returning fpt_* function of fpt_b200.h.  A rejected
 * argument or a launch error cannot be returned through `void`; it is kept per host thread and read with
 * fpt_compat_last_status() (0 = ok), which also clears it.  Link libfpt_b200_compat.so in place of the
 * reference's own spline_kernels.cu / spline_kernels_bf16.cu / sincos_kernels.cu objects. */
#ifndef FPT_B200_COMPAT_H
#define FPT_B200_COMPAT_H

#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

int fpt_compat_last_status(void);
int fpt_compat_symbol_count(void);

'''

HEADER_END = '''
#ifdef __cplusplus
}
#endif
#endif
'''

SOURCE_TOP = '''// Generated by fast_polynomial_transcendentals_b200/csrc/gen_compat_launch.py -- do not edit.
// launch_* entry points with the reference's names and argument order, forwarding to the fpt_* C ABI.
#include "../../include/fpt_b200.h"
#include "../../include/fpt_b200_compat.h"

namespace {
thread_local int g_last_status = 0;
inline void keep(int status) {
    if (status != 0 && g_last_status == 0) g_last_status = status;
}
// the repeated-evaluation launchers of the reference run zero evaluations for iterations <= 0 and so write zeros;
// here iterations == 0 means "plain evaluation", so non-positive counts are rejected instead
inline int positive(int iterations) { return iterations > 0 ? iterations : -1; }
}  // namespace

extern "C" int fpt_compat_last_status(void) {
    const int s = g_last_status;
    g_last_status = 0;
    return s;
}
'''


def main() -> None:
    names = [e[0] for e in entries]
    assert len(names) == len(set(names)), "duplicate symbol"
    header = HEADER_TOP + "".join(f"void {n}({p});\n" for n, p, _ in entries) + HEADER_END
    source = SOURCE_TOP + f"extern \"C\" int fpt_compat_symbol_count(void) {{ return {len(entries)}; }}\n\n"
    source += "".join(f"extern \"C\" void {n}({p}) {{\n    keep({c});\n}}\n" for n, p, c in entries)
    (HERE.parent.parent / "include" / "fpt_b200_compat.h").write_text(header)
    (HERE / "fpt_compat_launch.cpp").write_text(source)
    print(len(entries), "entry points")


if __name__ == "__main__":
    main()

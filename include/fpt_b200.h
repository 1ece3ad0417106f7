/*
 * fpt_b200 -- C ABI of the B200 (sm_100a) packed polynomial transcendental library.
 *
 * Drop-in boundary: the reference separates its torch-facing C++ (spline_ops.cpp)
 * from its CUDA kernels by `extern "C" void launch_*(void* out, const void* in, ...,
 * int size, cudaStream_t)` launchers (reference: autonumerics_zero/spline_ops/
 * spline_ops.cpp:14-288).  This library offers that boundary twice:
 *
 *   1. the `fpt_*` entry points below: one entry point per operator family, the
 *      program selected by (function, direction, degree, dtype, coefficient
 *      source) instead of by symbol name; 64-bit sizes; an `int` status return
 *      (0 ok, negative = rejected argument, positive = cudaError_t);
 *   2. the reference's own `launch_*` symbols with the reference's exact
 *      signatures (declared in fpt_b200_compat.h), thin shims over (1), so the
 *      reference's spline_ops.cpp links against this library unchanged.
 *
 * Conventions: every pointer is a device pointer owned by the caller; 16-bit data
 * are fp16 or bf16 bit patterns according to `dtype`; work is enqueued on `stream`
 * of the CURRENT device and the call returns without synchronising; no entry
 * point allocates device memory.  All entry points may be called concurrently
 * from several host threads and for several devices.
 */
#ifndef FPT_B200_H
#define FPT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* fpt_stream_t; /* == cudaStream_t */

/* status codes (positive values are cudaError_t) */
#define FPT_OK 0
#define FPT_ERR_NULL_POINTER (-1)
#define FPT_ERR_BAD_SIZE (-2)
#define FPT_ERR_MISALIGNED (-3)      /* pointer not aligned to the element size / required vector width */
#define FPT_ERR_UNKNOWN_PROGRAM (-4) /* no program for (function, direction, degree, dtype, source) */
#define FPT_ERR_BAD_ENUM (-5)
#define FPT_ERR_UNSUPPORTED_SHAPE (-6)
#define FPT_ERR_NO_DEVICE (-7)       /* no CUDA device, or not compute capability 10.x */
#define FPT_ERR_DEVICE_TIMEOUT (-8)  /* a bounded device-side wait ran out (attention kernel status word) */
#define FPT_ERR_SCRATCH_TOO_SMALL (-9) /* the problem needs more than the library's fixed scratch array holds */

enum { FPT_FP16 = 0, FPT_BF16 = 1 };
enum { FPT_SRC_CURRENT = 0, FPT_SRC_SOLLYA = 1 };
enum { FPT_FN_SIGMOID = 0, FPT_FN_TANH = 1, FPT_FN_SWISH = 2, FPT_FN_ERF = 3, FPT_FN_GELU = 4 };
enum { FPT_FWD = 0, FPT_BWD = 1 };
/* degree: 3..6 selects the polynomial of that degree; 0 selects the native special-function-unit
 * (MUFU) control that shares the same memory code. */

const char* fpt_status_string(int status);
/* library / build identification, e.g. "fpt_b200 sm_100a" */
const char* fpt_version(void);

/* ---- program table (reference: spline_structs_odd.cuh:14-1047, spline_structs_odd_bf16.cuh:11-1006,
 *      spline_structs_sollya_bf16.cuh:14-852) ------------------------------------------------------ */
int fpt_program_count(void);
/* name_out receives e.g. "SIGMOID_FWD_D3"; coeffs7 receives the seven 16-bit coefficient slots. */
int fpt_program_info(int index, char* name_out, int name_capacity, int* dtype, int* source, int* shape,
                     int* degree, uint16_t* clamp, uint16_t* coeffs7);

/* ---- unary activations: out = F(in)
 *      replaces launch_{sigmoid,tanh,swish,gelu}_fwd_d{3..6}_kernel[_bf16[_sollya]] and
 *      launch_swish_fwd_native_kernel[_bf16] (reference: spline_kernels.cu:49-64,544-571,1177-1250;
 *      spline_kernels_bf16.cu:57-72,636-668).  direction FPT_BWD evaluates the derivative program F'(in). */
int fpt_unary(void* out, const void* in, int64_t n, int function, int direction, int degree, int dtype,
              int source, fpt_stream_t stream);
/* `repeats` evaluations per loaded element, each fed back as the next input (val <- F(val)); the
 * ALU-bound probe of the reference's repeated-evaluation benchmarks (benchmark_bfloat16_sollya.cu:70-82). */
int fpt_unary_repeat(void* out, const void* in, int64_t n, int function, int direction, int degree, int dtype,
                     int source, int repeats, fpt_stream_t stream);

/* ---- gradient products: grad_in = grad_out * F'(x)
 *      replaces launch_{sigmoid,tanh,swish,gelu}_bwd_d{3..6}_kernel[_bf16[_sollya]],
 *      launch_swish_bwd_native_kernel[_bf16] (reference: spline_kernels.cu:66-90,573-607). */
int fpt_binary_bwd(void* grad_in, const void* grad_out, const void* x, int64_t n, int function, int degree,
                   int dtype, int source, fpt_stream_t stream);
/* grad_in = grad_out * g(y) with y the saved forward output: sigmoid y(1-y), tanh 1-y^2
 *      replaces launch_{sigmoid,tanh}_bwd_alg_kernel[_bf16] (reference: spline_structs_odd.cuh:668-682). */
int fpt_bwd_algebraic(void* grad_in, const void* grad_out, const void* y, int64_t n, int function, int dtype,
                      fpt_stream_t stream);

/* ---- FP16 composites of the degree-3 forward programs (sigmoid, tanh, SiLU), fp16 only like the reference's
 *      replaces launch_{sigmoid,tanh}_fwd_deriv_{alg,poly}_kernel, launch_swish_fwd_deriv[_poly]_kernel,
 *      launch_{sigmoid,tanh,swish}_fused_kernel, launch_multiply_kernel and the six launch_*_{fwd,bwd}_hybrid_kernel
 *      (reference: autonumerics_zero/spline_ops/spline_kernels.cu:776-1027 kernels, :1394-1480 launchers).
 *      fpt_fwd_deriv: y = F_D3(x) and the derivative saved for backward, dy =
 *        FPT_DERIV_ALGEBRAIC      y(1-y) / 1-y^2 from y            (sigmoid, tanh)
 *        FPT_DERIV_POLY           the D4 derivative program of x    (sigmoid, tanh, SiLU)
 *        FPT_DERIV_SHARED_SIGMOID s = sigmoid_D3(x): y = x s, dy = s(1 + x(1-s))   (SiLU)
 *      Every length takes the same arithmetic (the reference's fallback for short or ragged arrays multiplies
 *      the algebraic derivative by y once more and drops the tail of `multiply`; neither is reproduced).
 *      fpt_fused_fwd_bwd: y = F_D3(x), grad_in = grad_out * (algebraic derivative of y; SiLU: D4 program of x).
 *      fpt_multiply: out = a * b (one rounding), fp16 or bf16.
 *      fpt_unary_hybrid / fpt_binary_bwd_hybrid: of every four packed words (16 bytes) the first is evaluated on
 *      the special-function unit (packed ex2 / rcp / tanh), the other three by the D3 (forward) or D4 (derivative)
 *      program; as in the reference the routing applies when n is a multiple of 8 and n >= 8192, otherwise (and
 *      for unaligned pointers) every lane is polynomial. */
enum { FPT_DERIV_ALGEBRAIC = 0, FPT_DERIV_POLY = 1, FPT_DERIV_SHARED_SIGMOID = 2 };
int fpt_fwd_deriv(void* y, void* dy, const void* x, int64_t n, int function, int variant, fpt_stream_t stream);
int fpt_fused_fwd_bwd(void* y, void* grad_in, const void* x, const void* grad_out, int64_t n, int function,
                      fpt_stream_t stream);
int fpt_multiply(void* out, const void* a, const void* b, int64_t n, int dtype, fpt_stream_t stream);
int fpt_unary_hybrid(void* out, const void* in, int64_t n, int function, fpt_stream_t stream);
int fpt_binary_bwd_hybrid(void* grad_in, const void* grad_out, const void* x, int64_t n, int function,
                          fpt_stream_t stream);

/* ---- SwiGLU: out = swish(gate) * up over flat arrays (B4 routed experts, B1 unpacked)
 *      replaces launch_swish_mul_fwd_{native,d3..d6}_kernel[_bf16[_sollya]]
 *      (reference: spline_kernels.cu:137-158,609-642; spline_kernels_bf16.cu:143-164,705-739). */
int fpt_swish_mul(void* out, const void* gate, const void* up, int64_t n, int degree, int dtype, int source,
                  fpt_stream_t stream);
/* grad_gate = (grad_out*up)*swish'(gate), grad_up = grad_out*swish(gate)
 *      replaces launch_swish_mul_bwd_* (reference: spline_kernels.cu:183-245; bf16 D3/current uses the
 *      shared-sigmoid form of spline_kernels_bf16.cu:255-341). */
int fpt_swish_mul_bwd(void* grad_gate, void* grad_up, const void* grad_out, const void* gate, const void* up,
                      int64_t n, int degree, int dtype, int source, fpt_stream_t stream);

/* ---- packed SwiGLU (B1 dense FFN): packed [rows, 2*hidden] = [gate | up] -> out [rows, hidden]
 *      replaces launch_swish_mul_packed_fwd_{native,d3..d6}_kernel[_bf16[_sollya]]
 *      (reference: spline_kernels.cu:247-351,700-733; spline_kernels_bf16.cu:421-503,838-883). */
int fpt_swish_mul_packed(void* out, const void* packed, int64_t rows, int64_t hidden, int degree, int dtype,
                         int source, fpt_stream_t stream);
/* grad_packed [rows, 2*hidden] from grad_out [rows, hidden] and packed
 *      replaces launch_swish_mul_packed_bwd_* (reference: spline_kernels.cu:418-494,735-769). */
int fpt_swish_mul_packed_bwd(void* grad_packed, const void* grad_out, const void* packed, int64_t rows,
                             int64_t hidden, int degree, int dtype, int source, fpt_stream_t stream);

/* ---- gate / up projection with the SwiGLU in its epilogue (the step before the activation, B1 and B4):
 *      out[r, h] = swish(sum_k x[r, k] w_gate[g, h, k]) * (sum_k x[r, k] w_up[g, h, k]),  g = the group of row r
 *      on the tensor cores (bf16 operands, fp32 accumulation), each product rounded to bf16 before the same packed
 *      program as fpt_swish_mul: the [rows, 2*hidden] intermediate of
 *      `w_in(x)` -> launch_swish_mul_packed_fwd_* (reference: src/sfu_repro/torchtitan/plugin.py:238-239, the fused
 *      gate / up feed-forward) and of `_grouped_mm(x, w1)`, `_grouped_mm(x, w3)` -> launch_swish_mul_fwd_*
 *      (reference: plugin.py:294-310, the routed experts) is never written.
 *      x [rows, dim] with row stride x_ld; w_gate, w_up [groups, hidden, dim] with row stride w_ld and group stride
 *      w_group_stride (a packed [2*hidden, dim] weight is w_gate = w, w_up = w + hidden*w_ld, groups = 1); out
 *      [rows, hidden] (or [rows, 2*hidden] = [gate | up] with FPT_GATE_UP_RAW: the products alone, for callers that
 *      keep them for a backward pass) with row stride out_ld; all strides in elements, all tensors bf16.
 *      group_ends (device memory, int32, cumulative row counts: the `offs` of a grouped matrix product) may be NULL
 *      when groups == 1; rows beyond the last end are left untouched.  hidden must be a multiple of 128, dim and the
 *      strides multiples of 8, groups <= 256.  degree 0 = the special-function twin, 3 = the cubic program.
 *      `status` as in the attention entry points (a zeroed device word, non-zero afterwards = a bounded wait ran
 *      out and `out` is invalid). */
enum { FPT_GATE_UP_SWIGLU = 0, FPT_GATE_UP_RAW = 1 };
int fpt_gate_up_swiglu(void* out, const void* x, const void* w_gate, const void* w_up, int64_t rows, int64_t dim,
                       int64_t hidden, int64_t x_ld, int64_t w_ld, int64_t w_group_stride, int64_t out_ld,
                       const int32_t* group_ends, int64_t groups, int degree, int source, int epilogue, void* status,
                       fpt_stream_t stream);

/* ---- B3 sigmoid attention score-mod, isolated: prob = p(score) ~ sigmoid(score - log n), bf16 out
 *      Direct piecewise cubic on the raw score with the deployed n = 4096 constants shifted to
 *      n = 2^log2_n (reference: scripts/audit_b3_deployed_fit.py:341-366 for the arithmetic,
 *      extras/paper/manuscript/main.tex:1042-1117 for the instruction sequence and immediates).
 *      `scores` is bf16, or fp32 when scores_are_f32 != 0 (rounded to bf16 first, as in the attention kernel).
 *      `grad` may be NULL; otherwise it receives prob * (intercept + slope*clamp(score)), the coupled
 *      derivative of the deployed pair. */
int fpt_b3_sigmoid_direct(void* prob, void* grad, const void* scores, int64_t n, int scores_are_f32,
                          int log2_n, fpt_stream_t stream);
/* The same evaluator in a chosen instruction order.  FPT_B3_DEPLOYED_ORDER is fpt_b3_sigmoid_direct: clamp to
 * [-6, 6], row selected before the cubic, floor by a separate maximum (reference: extras/paper/manuscript/
 * main.tex:1042-1072).  FPT_B3_SELECT_LATE is the order the attention kernels of this library run: both rows'
 * cubics, one select afterwards, upper clamp only, floor folded into the last multiply-add.  Probabilities are the
 * same bits for every input; the gradient may differ in the sign of a zero below the lower clamp and nowhere else. */
enum { FPT_B3_DEPLOYED_ORDER = 0, FPT_B3_SELECT_LATE = 1 };
int fpt_b3_sigmoid_direct_variant(void* prob, void* grad, const void* scores, int64_t n, int scores_are_f32,
                                  int log2_n, int variant, fpt_stream_t stream);

/* ---- fractional exp2 on packed fp16, x in [0, 1)
 *      replaces FractionalNative / FractionalPwl2Hinge of the reference's stand-alone benchmark
 *      (reference: autonumerics_zero/cuda_benchmarks/benchmark_exp2_pwl2.cu:53-99, 200-259).
 *      `repeats` >= 1 evaluations per element, fed back through x <- v/2 - 1/2. */
enum { FPT_EXP2_NATIVE = 0, FPT_EXP2_HINGE_LEAST_SQUARES = 1, FPT_EXP2_HINGE_ENDPOINT = 2 };
int fpt_exp2_fraction(void* out, const void* in, int64_t n, int variant, int repeats, fpt_stream_t stream);

/* ---- full-range fp32 2^a on the FMA pipe: a' = max(a, -127), n = floor(a') through a round-down magic-constant add,
 *      f = a' - n, then a cubic in f (FPT_EXP2_FULL_D3, relative error 8.8e-5) or a continuous two-piece line
 *      (FPT_EXP2_FULL_PWL2, 2.1e-2), n added to the exponent field
 *      replaces FullDegree3 / FullPwl2Hinge of the reference's benchmark, operation for operation (reference:
 *      autonumerics_zero/cuda_benchmarks/benchmark_exp2_pwl2.cu:106-198); these are the software exponentials the
 *      attention kernel routes a share of its soft-max lanes through.  in/out: fp32 [n], 16-byte aligned; a <= 127.
 *      One difference: the two-piece line clamps at -126, not -127 (its p starts below 1, so at n = -127 the
 *      reference's bit arithmetic wraps into a NaN pattern; -inf is a regular input of a masked soft-max).
 *      FPT_EXP2_FULL_D2_SAFE ("d2_safe") and FPT_EXP2_FULL_PWL2_SAFE_F16 ("pwl2_safe_f16") keep the same reduction and
 *      reconstruction and change the fractional evaluator to the two endpoint-preserving fits of the reference
 *      (reference: extras/paper/manuscript/appendix_exp2.tex:18-33 and :74-80): p = 1 + a f + (1 - a) f^2 with
 *      a = 0.6602339719 in fp32 (relative error 2.7e-3), and p = 1 + A f + C max(f - 1/2, 0) on a packed fp16 pair with
 *      A = 0.7978515625, C = 0.40380859375 (1.1e-2).  Both give p(0) = 1 and p(1) = 2 exactly; both clamp at -127. */
enum { FPT_EXP2_FULL_D3 = 0, FPT_EXP2_FULL_PWL2 = 1, FPT_EXP2_FULL_D2_SAFE = 2, FPT_EXP2_FULL_PWL2_SAFE_F16 = 3 };
int fpt_exp2_full_f32(void* out, const void* in, int64_t n, int variant, fpt_stream_t stream);

/* ---- paired sin/cos: fp32 angles [n] -> out [2, n] 16-bit, cos plane first
 *      replaces launch_sincos_*_{fp16,bf16}[_compute] (reference: sincos_kernels.cu:527-975 evaluators,
 *      1084-1240 kernels).  iterations == 0: one evaluation; iterations > 0: the repeated-evaluation probe
 *      (sums of `iterations` evaluations, angle <- fma(angle, 1 - 2^-24, 2^-13) between them). */
enum {
    FPT_SINCOS_D3_D4_QUARTER_TURN_FP16 = 0,
    FPT_SINCOS_D3_D4_HALF_TURN_FP16 = 1,
    FPT_SINCOS_D5_D4_HALF_TURN_FP16 = 2,
    FPT_SINCOS_D5_D6_HALF_TURN_FP16 = 3,
    FPT_SINCOS_D7_D6_HALF_TURN_FP16 = 4,
    FPT_SINCOS_D3_D4_BF16 = 5,
    FPT_SINCOS_D3_D4_QUARTER_TURN_BF16 = 6,
    FPT_SINCOS_D3_D4_HALF_TURN_BF16 = 7,
    FPT_SINCOS_D5_D6_HALF_TURN_BF16 = 8,
    FPT_SINCOS_D5_D4_HALF_TURN_FP16_BF16 = 9,
    FPT_SINCOS_VARIANT_COUNT = 10,
    FPT_SINCOS_NATIVE_FP16 = 10,
    FPT_SINCOS_NATIVE_BF16 = 11
};
int fpt_sincos(void* out, const void* angles, int64_t n, int variant, int iterations, fpt_stream_t stream);

/* ---- paired sin/cos in fp32: fp32 angles [n] -> out [2, n] fp32, cos plane first
 *      replaces launch_sincos_*_f32 and launch_sincos_*_compute_f32 (reference: sincos_kernels.cu:24-118 reducers,
 *      :120-406 evaluators, :980-1082 kernels, :2125-2357 launchers).  iterations as in fpt_sincos. */
enum {
    FPT_SINCOS_F32_NATIVE = 0,
    FPT_SINCOS_F32_D3_D4 = 1,
    FPT_SINCOS_F32_D3_D4_CYCLE = 2,
    FPT_SINCOS_F32_D3_D4_MAGIC_BIAS = 3,
    FPT_SINCOS_F32_D5_D4_HALF_TURN_LS = 4,
    FPT_SINCOS_F32_D5_D4_HALF_TURN_SOLLYA = 5,
    FPT_SINCOS_F32_D5_D4_HALF_TURN_SOLLYA_FAST = 6,
    FPT_SINCOS_F32_D5_D4 = 7,
    FPT_SINCOS_F32_D7_D6 = 8
};
int fpt_sincos_f32(void* out, const void* angles, int64_t n, int variant, int iterations, fpt_stream_t stream);

/* ---- RoPE tables: table [2, seq, freq_count] fp16 (cos plane, then sin plane)
 *      replaces launch_rope_sincos_{native,fixed_d3_d4,fixed_half_turn_d5_d6}_fp16[_compute]
 *      (reference: sincos_kernels.cu:1242-1348, 1387-1480).  params: int32 Q0.32 phase increments
 *      [freq_count] (round(freq * 2^32 / 2pi)), or fp32 frequencies for FPT_ROPE_NATIVE. */
enum { FPT_ROPE_HALF_TURN_D5_D6 = 0, FPT_ROPE_QUARTER_TURN_D3_D4 = 1, FPT_ROPE_NATIVE = 2, FPT_ROPE_CACHED = 3 };
int fpt_rope_table(void* table, const void* params, int64_t seq, int64_t freq_count, int kind, int iterations,
                   fpt_stream_t stream);

/* ---- RoPE table by look-up: phase_table [128, 2] fp16 = (sin, cos) of 2*pi*i/128; the top phase bits pick an entry,
 *      the remainder drives one first-order step in fp16
 *      replaces launch_rope_sincos_fixed_lut_fp16[_compute] (reference: sincos_kernels.cu:1350-1385 evaluator,
 *      :1482-1502 and :1894-1928 kernels).  iterations as in fpt_rope_table. */
int fpt_rope_table_lut(void* table, const void* phase_increments, const void* phase_table, int64_t seq,
                       int64_t freq_count, int iterations, fpt_stream_t stream);

/* ---- fused RoPE rotation + transpose: q [B,S,Hq,D], k [B,S,Hk,D] -> q_out [B,Hq,S,D], k_out [B,Hk,S,D]
 *      replaces launch_rope_apply_{fixed_half_turn_d5_d6,native,cached}_fp16
 *      (reference: sincos_kernels.cu:1504-1754).  Interleaved (even, odd) pairs; one parameter per pair:
 *      params [D/2] increments or frequencies, or for FPT_ROPE_CACHED a table [2, S, D/2] fp16.
 *      dtype FPT_FP16 is the reference's form.  FPT_BF16 reads and writes bf16 around the same fp16
 *      rotation (input widened exactly and rounded to fp16, result rounded once to bf16). */
int fpt_rope_apply(void* q_out, void* k_out, const void* q, const void* k, const void* params, int64_t batch,
                   int64_t seq, int64_t q_heads, int64_t k_heads, int64_t head_dim, int kind, int dtype,
                   fpt_stream_t stream);

/* ---- fused RoPE from a cached table WITHOUT a caller-provided table (no counterpart in the reference)
 *      Same result as fpt_rope_table followed by fpt_rope_apply(kind = FPT_ROPE_CACHED), for callers that may not
 *      allocate device memory (a plugin inside a serving loop whose host owns all device memory, a real-time path
 *      that must stay off the allocator, a user without a device allocator): the [2, seq, head_dim/2] fp16 table
 *      lives in a fixed 4 MiB array inside the library, held by every GPU that loads it until the process exits.
 *      Limit: seq * head_dim <= fpt_rope_static_table_capacity() (2^21, e.g. 16384 x 128); larger problems are
 *      rejected with FPT_ERR_SCRATCH_TOO_SMALL.  The call allocates nothing.  The first call on a device looks up
 *      the array's device address (cudaGetSymbolAddress); make that first call before any stream capture.
 *      All calls share the one array: two calls whose kernels may overlap on the GPU (different streams) race on
 *      it; calls on one stream are safe.  table_kind: FPT_ROPE_HALF_TURN_D5_D6 or FPT_ROPE_QUARTER_TURN_D3_D4.
 *      Every argument is checked before anything is enqueued: after an error return the array holds what the last
 *      successful call left in it.  The looked-up address is kept per device for the life of the process; a program
 *      that calls cudaDeviceReset must not use this entry point on that device afterwards. */
int64_t fpt_rope_static_table_capacity(void);
int fpt_rope_apply_static_table(void* q_out, void* k_out, const void* q, const void* k, const void* phase_increments,
                                int64_t batch, int64_t seq, int64_t q_heads, int64_t k_heads, int64_t head_dim,
                                int table_kind, int dtype, fpt_stream_t stream);

/* ---- attention forward with a polynomial score-mod, bf16, head_dim 128, any sequence length
 *      replaces the forward of the patched FlashAttention interface that the reference drives through
 *      `_flash_attn_fwd(q, k, v, softmax_scale=, causal=, softcap=, score_mod=, sigmoid_attention=, ...) -> (out, lse)`
 *      (reference: src/sfu_repro/fa4.py:755-826, wrapper :899-948, canonical configurations :650-709).
 *      q [B,S,Hq,D], k / v [B,S,Hkv,D], out [B,S,Hq,D]: logical (batch, seq, head, dim) tensors addressed through
 *      `*_strides` = element strides of (batch, seq, head); dim is contiguous.  Grouped-query attention:
 *      kv head = q head / (Hq / Hkv).  lse fp32 [B,Hq,S] (may be NULL; unused in sigmoid mode).
 *      mode FPT_ATTN_SOFTCAP_TANH:  softmax(softcap * tanhD4_bf16(score*scale/softcap)), the B2 score-mod
 *      mode FPT_ATTN_SIGMOID_DIRECT: P = direct piecewise cubic sigmoid of bf16(score*scale) scaled for n = 2^log2_n
 *                                    keys (B3), O = P V without normalisation
 *      mode FPT_ATTN_SOFTMAX:        plain softmax (control)
 *      mode FPT_ATTN_SOFTCAP_NATIVE: the native twin of FPT_ATTN_SOFTCAP_TANH: softmax(softcap * tanh(score*scale/softcap))
 *                                    with the special-function unit's fp32 tanh (the reference's softcap_backend =
 *                                    "native", src/sfu_repro/fa4.py:650-659), same kernel otherwise
 *      mode FPT_ATTN_SIGMOID_NATIVE: the native twin of FPT_ATTN_SIGMOID_DIRECT: P = 1 / (1 + 2^(log2_n - score*scale*
 *                                    log2 e)) = sigmoid(score*scale - ln 2^log2_n) through ex2 and rcp (the reference's
 *                                    sigmoid_variant = "sfu", src/sfu_repro/fa4.py:686-692), O = P V
 *      status: one zero-initialised device word; non-zero after the launch means a bounded device-side wait ran
 *      out (bit 31 set, low bits tell where) and the output is invalid. */
enum { FPT_ATTN_SOFTCAP_TANH = 0, FPT_ATTN_SIGMOID_DIRECT = 1, FPT_ATTN_SOFTMAX = 2, FPT_ATTN_SOFTCAP_NATIVE = 3,
       FPT_ATTN_SIGMOID_NATIVE = 4 };
int fpt_attention_fwd(void* out, void* lse, const void* q, const void* k, const void* v, int64_t batch, int64_t seq,
                      int64_t q_heads, int64_t kv_heads, int64_t head_dim, const int64_t* q_strides,
                      const int64_t* k_strides, const int64_t* v_strides, const int64_t* out_strides, int mode,
                      int causal, float scale, float softcap, int log2_n, void* status, fpt_stream_t stream);

/* ---- the same forward with the soft-max exponentials partly routed to the FMA pipe
 *      replaces the exp2_emu_backend / exp2_emu_freq routing of the reference's attention interface
 *      (reference: src/sfu_repro/fa4.py:34-47 backends, :724-752 routed configurations, forward kwargs :790-807):
 *      exp2_emu_freq 0 keeps every exponential on the special-function unit; f in {8, 12, 16, 32} sends four of
 *      every f keys of a row through a software exponential of fpt_exp2_full_f32 instead (one half, third, quarter,
 *      eighth): exp2_emu_backend FPT_EXP2_FULL_D3 ("d3") in both polynomial soft-max modes; FPT_EXP2_FULL_PWL2
 *      ("pwl2"), FPT_EXP2_FULL_D2_SAFE ("d2_safe") and FPT_EXP2_FULL_PWL2_SAFE_F16 ("pwl2_safe_f16") in
 *      FPT_ATTN_SOFTMAX.  The sigmoid modes have no soft-max exponential and FPT_ATTN_SOFTCAP_NATIVE is the all-native
 *      control: they accept frequency 0 only. */
int fpt_attention_fwd_routed(void* out, void* lse, const void* q, const void* k, const void* v, int64_t batch,
                             int64_t seq, int64_t q_heads, int64_t kv_heads, int64_t head_dim,
                             const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                             const int64_t* out_strides, int mode, int causal, float scale, float softcap, int log2_n,
                             int exp2_emu_backend, int exp2_emu_freq, void* status, fpt_stream_t stream);

/* ---- attention backward for the same three modes, bf16, head_dim 128, any sequence length
 *      replaces the backward of the patched FlashAttention interface the reference drives through
 *      `flash_attn_bwd(q, k, v, out, dout, lse, softmax_scale, causal, softcap, score_mod=, score_mod_bwd=,
 *      sigmoid_attention=, ...) -> (dq, dk, dv)` (reference: src/sfu_repro/fa4.py:828-859).
 *      q, k, v, out, dout: (batch, seq, head, dim) tensors through element strides as in the forward; lse fp32
 *      [B,Hq,S] from the forward; dq [B,S,Hq,D], dk / dv [B,S,Hkv,D] contiguous bf16 outputs.
 *      Soft-max modes need out, lse and a workspace of fpt_attention_bwd_workspace_bytes() (16-byte aligned);
 *      FPT_ATTN_SIGMOID_DIRECT and FPT_ATTN_SIGMOID_NATIVE need none of the three (NULL accepted): dS = dP * p(x) * (intercept + slope*clamp(x)),
 *      the coupled derivative of the direct cubic.  softcap_grad picks d tanh_poly / dx for FPT_ATTN_SOFTCAP_TANH:
 *      the derivative of the polynomial itself (zero where the input is clamped or the output saturated), or
 *      1 - t^2 of its value.  status as in the forward.
 *      Two forms, chosen by the size of the workspace the caller passes:
 *        one pass (workspace >= fpt_attention_bwd_fused_workspace_bytes, in every mode, unless tuning key
 *          "attention_bwd_fused" is set to 0): one kernel for dK, dV and dQ, 5 matrix products per tile pair.  The block
 *          of a key tile also forms the partial dQ of every query tile it streams and adds it into an fp32
 *          [B, Hq, S, 128] buffer inside the workspace with reduce-add copies; a last pass scales and rounds it to bf16.
 *          The order of those fp32 additions is not fixed, so the last bit of a dQ element can differ from run to run
 *          (dK and dV are deterministic, and the same bits as in the two-pass form).  Measured on B200: 1.4-1.65x the
 *          two-pass form;
 *        two passes (workspace >= fpt_attention_bwd_workspace_bytes; none needed in the sigmoid modes): one launch for dQ,
 *          one for dK and dV, each recomputing S and dP: 7 matrix products per tile pair, no atomics, deterministic.
 *          A caller who needs run-to-run identical dQ passes the smaller workspace or sets the tuning key to 0. */
enum { FPT_SOFTCAP_GRAD_ANALYTICAL = 0, FPT_SOFTCAP_GRAD_ONE_MINUS_T2 = 1 };
int64_t fpt_attention_bwd_workspace_bytes(int64_t batch, int64_t seq, int64_t q_heads);
int64_t fpt_attention_bwd_fused_workspace_bytes(int64_t batch, int64_t seq, int64_t q_heads);
int fpt_attention_bwd(void* dq, void* dk, void* dv, const void* dout, const void* q, const void* k, const void* v,
                      const void* out, const void* lse, void* workspace, int64_t workspace_bytes, int64_t batch,
                      int64_t seq, int64_t q_heads, int64_t kv_heads, int64_t head_dim, const int64_t* q_strides,
                      const int64_t* k_strides, const int64_t* v_strides, const int64_t* out_strides,
                      const int64_t* dout_strides, int mode, int causal, float scale, float softcap, int log2_n,
                      int softcap_grad, void* status, fpt_stream_t stream);

/* The same backward with the soft-max exponentials of the recomputed probabilities partly routed to the FMA pipe
 *      replaces exp2_emu_freq_bwd of the reference's attention interface (reference: src/sfu_repro/fa4.py:724-752, the
 *      retained routed configurations use forward frequency 12 and backward frequency 32; backward kwargs :828-859).
 *      FPT_ATTN_SOFTMAX only; frequencies 0, 8, 12, 16, 32: four of every f columns of each 64-column half of a score
 *      tile take the software exponential exp2_emu_backend (any FPT_EXP2_FULL_* value).  The native twins take
 *      softcap_grad as given for FPT_ATTN_SOFTCAP_NATIVE (1 - t^2 is what they compute) and need neither out nor lse
 *      for FPT_ATTN_SIGMOID_NATIVE (dS = dP p (1 - p)). */
int fpt_attention_bwd_routed(void* dq, void* dk, void* dv, const void* dout, const void* q, const void* k, const void* v,
                             const void* out, const void* lse, void* workspace, int64_t workspace_bytes, int64_t batch,
                             int64_t seq, int64_t q_heads, int64_t kv_heads, int64_t head_dim, const int64_t* q_strides,
                             const int64_t* k_strides, const int64_t* v_strides, const int64_t* out_strides,
                             const int64_t* dout_strides, int mode, int causal, float scale, float softcap, int log2_n,
                             int softcap_grad, int exp2_emu_backend, int exp2_emu_freq, void* status, fpt_stream_t stream);

/* ---- diagnostic: one 128x128x128 bf16 tile through the tensor-core building blocks of the attention kernel
 *      (no counterpart in the reference).  a, b: bf16 [128,128] row-major; c: fp32 [128,128];
 *      mode 0: c = a * b^T (both operands K-major in shared memory); mode 1: c = a * b (a staged in tensor memory,
 *      b an MN-major shared-memory operand); mode 2: c = a^T * b (a stored to shared memory by the threads in the swizzled
 *      panel layout and read as an MN-major A operand, b MN-major: the form the fused attention backward uses for dQ).
 *      status: one zero-initialised device word; non-zero afterwards means a
 *      bounded device-side wait ran out. */
int fpt_selftest_umma(void* c, const void* a, const void* b, int mode, void* status, fpt_stream_t stream);

/* ---- diagnostic: the bounded device-side wait of the attention kernels, run on a barrier nobody arrives on
 *      (no counterpart in the reference).  One thread waits at most limit_ns (1 us .. 1 ms) on an mbarrier of its own;
 *      the kernel uses no TMA, no tensor memory and no tensor-core operation, so nothing is in flight when it gives up.
 *      status: one device word, as in the attention entry points: zero before the call; afterwards 0x80000000 | where.
 *      A call whose status word is already non-zero does not wait at all (the attention kernels' behaviour for blocks
 *      that start after a timeout).  report: three device words: [0] 1 = timed out, 2 = skipped, 3 = wait succeeded;
 *      [1], [2] = nanoseconds waited (low, high). */
int fpt_selftest_bounded_wait(void* status, void* report, int64_t limit_ns, int where, fpt_stream_t stream);

/* ---- launch knobs for benchmarks (process-wide; defaults are the measured-best values) -------- */
/* key "blocks_per_sm": persistent-grid cap (0 = one block per tile); key "streaming": -1 auto, 0, 1;
 * key "attention_split": 1 (default) lets the attention forward use its column-split score-mod warps where the mode
 * allows (soft-cap with cap*log2(e) <= 98), 0 forces the one-thread-per-row layout, 2 uses the column-split layout for
 * the sigmoid mode as well (measured no faster; kept for comparison runs);
 * key "attention_raster": order in which attention blocks are handed out: 0 heads fastest, 1 row blocks of one head
 * fastest, -1 (default) the measured-best choice per kernel (forward and backward: rows when nothing is masked and the
 * streamed tensors exceed 64 MB, heads otherwise);
 * key "rope_heads_per_block": heads of Q and of K that one block of the fused RoPE rotates (default 8; 0 = all heads);
 * key "attention_bwd_fused": 1 (default) lets the attention backward take its one-pass form when the workspace allows, 0
 * keeps the deterministic two-pass form whatever the workspace, 2 is 1 with sixteen score-mod warps per block in every mode
 * (the default uses sixteen for the polynomial soft-cap with the analytical derivative and eight elsewhere; same results);
 * key "attention_cta_pair": 1 runs the attention forward on pairs of CTAs (clusters of two, tcgen05 cta_group::2: one
 * 256-row product per pair, every K and V tile split between the two SMs) wherever two blocks share their K / V (two
 * query heads of one K / V group; two row blocks of one head without a mask), 0 (default) never: same bits; 0.85-1.00x the
 * single-CTA speed;
 * key "gate_up_cta_pair": 1 runs fpt_gate_up_swiglu on pairs of CTAs (clusters of two, tcgen05 cta_group::2: one product of
 * 256 rows whose weight tile is split over the two SMs), 0 on single CTAs, -1 (default) on pairs unless
 * "gate_up_tile_rows" names a height;
 * key "gate_up_pair_wide": 1 gives a pair two hidden tiles per row tile (a 256 x 256 output tile) where the number of hidden
 * tiles is even, 0 (default) one: measured slower (no accumulator left to alternate);
 * key "gate_up_tile_rows": rows per tile of the single-CTA forms, 128 or 256; 0 (default) = 256 for one group (both halves
 * of a tile share every weight tile: fewer bytes per product, which under the power cap is the faster form), 128 for
 * grouped problems (a ragged group wastes less of a smaller tile). */
int fpt_set_tuning(const char* key, int value);
int fpt_get_tuning(const char* key, int* value);

#ifdef __cplusplus
}
#endif
#endif /* FPT_B200_H */

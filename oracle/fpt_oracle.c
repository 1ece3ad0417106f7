/*
 * TEST INFRASTRUCTURE ONLY -- CPU restatement of the reference's packed
 * polynomial programs, evaluated with the exact single-rounding lane model of
 * fpt_softfloat.h.  Tests, the smoke check and the bench's CPU-baseline leg use
 * it as the checker; the shipped library never links or loads it.
 *
 * What each block follows in the reference (paths inside the reference project):
 *   activation programs   autonumerics_zero/spline_ops/spline_structs_odd.cuh:14-1047,
 *                         spline_structs_odd_bf16.cuh:11-1006, spline_structs_sollya_bf16.cuh:14-852
 *   element-wise wrappers autonumerics_zero/spline_ops/spline_kernels.cu:49-494,
 *                         spline_kernels_bf16.cu:57-608
 *   B3 direct sigmoid     scripts/audit_b3_deployed_fit.py:341-366 and the PTX listing in
 *                         extras/paper/manuscript/main.tex:1042-1117 (PTX NaN/zero rules are used)
 *   fractional exp2       autonumerics_zero/cuda_benchmarks/benchmark_exp2_pwl2.cu:53-99
 *   paired sin/cos        autonumerics_zero/spline_ops/sincos_kernels.cu:24-127, 527-975
 *   RoPE tables / apply   autonumerics_zero/spline_ops/sincos_kernels.cu:1242-1348, 1409-1480, 1504-1612
 */
#include "fpt_oracle.h"
#include "fpt_softfloat.h"

#include <stdlib.h>

/* ------------------------------------------------------------- threading */

#ifdef _OPENMP
#include <omp.h>
#endif

/* Number of OpenMP threads the loops below use from now on (n <= 0: leave as is); returns the count in effect.
 * Launchers such as torchrun export OMP_NUM_THREADS=1, which would otherwise silently make the timed CPU legs scalar. */
int fpt_oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

/* ------------------------------------------------------------------ table */

enum { SH_ODD_HALF, SH_ODD, SH_ODD_SAT, SH_SWISH, SH_XMUL_HALF, SH_EVEN, SH_ALG_SIG, SH_ALG_TANH };
enum { DT_FP16 = 0, DT_BF16 = 1 };
enum { SRC_CURRENT = 0, SRC_SOLLYA = 1 };

typedef struct {
    const char* name; int dtype; int source; int shape; int degree; uint16_t clamp; uint16_t c[7];
} program_row;

#define FPT_PROGRAM(NAME, DT, SRC, SHAPE, DEG, CLAMP, C0, C1, C2, C3, C4, C5, C6) \
    { #NAME, DT_##DT, SRC_##SRC, SH_##SHAPE, DEG, CLAMP, { C0, C1, C2, C3, C4, C5, C6 } },
static const program_row k_programs[] = {
#include "../fast_polynomial_transcendentals_b200/csrc/fpt_program_table.inc"
};
#undef FPT_PROGRAM
static const int k_program_count = (int)(sizeof(k_programs) / sizeof(k_programs[0]));

int fpt_oracle_program_count(void) { return k_program_count; }

int fpt_oracle_find_program(const char* name, int dtype, int source) {
    for (int i = 0; i < k_program_count; ++i)
        if (k_programs[i].dtype == dtype && k_programs[i].source == source && !strcmp(k_programs[i].name, name))
            return i;
    return -1;
}

int fpt_oracle_program_info(int program, char* name_out, int name_cap, int* dtype, int* source,
                            int* shape, int* degree, uint16_t* clamp, uint16_t* coeffs7) {
    if (program < 0 || program >= k_program_count) return -1;
    const program_row* p = &k_programs[program];
    if (name_out && name_cap > 0) { strncpy(name_out, p->name, (size_t)name_cap - 1); name_out[name_cap - 1] = 0; }
    if (dtype) *dtype = p->dtype;
    if (source) *source = p->source;
    if (shape) *shape = p->shape;
    if (degree) *degree = p->degree;
    if (clamp) *clamp = p->clamp;
    if (coeffs7) memcpy(coeffs7, p->c, sizeof(p->c));
    return 0;
}

/* ---------------------------------------------------------- lane programs */

static inline uint16_t const_half(sf_format f) { return f == SF_FP16 ? 0x3800u : 0x3f00u; }
static inline uint16_t const_one(sf_format f) { return f == SF_FP16 ? 0x3c00u : 0x3f80u; }

static uint16_t eval_lane(const program_row* p, uint16_t x) {
    const sf_format f = p->dtype == DT_FP16 ? SF_FP16 : SF_BF16;
    if (p->shape == SH_ALG_SIG) return sf_mul(f, x, sf_sub(f, const_one(f), x));
    if (p->shape == SH_ALG_TANH) return sf_sub(f, const_one(f), sf_mul(f, x, x));
    const uint16_t sign = x & 0x8000u;
    const uint16_t a = x & 0x7fffu;
    const uint16_t t = sf_min(f, a, p->clamp);
    const int d = p->degree;
    if (p->shape == SH_EVEN) {
        uint16_t r = sf_fma(f, t, p->c[d], p->c[d - 1]);
        for (int k = d - 2; k >= 0; --k) r = sf_fma(f, t, r, p->c[k]);
        return r;
    }
    /* h = t*(c1 + t*(c2 + ... )) with slot k = c(k+1) */
    uint16_t h = sf_fma(f, t, p->c[d - 1], p->c[d - 2]);
    for (int k = d - 3; k >= 0; --k) h = sf_fma(f, t, h, p->c[k]);
    h = sf_mul(f, t, h);
    switch (p->shape) {
    case SH_ODD: return h ^ sign;
    case SH_ODD_SAT: return sf_min(f, h, const_one(f)) ^ sign;
    case SH_ODD_HALF: return sf_add(f, const_half(f), h ^ sign);
    case SH_XMUL_HALF: return sf_mul(f, x, sf_add(f, const_half(f), h ^ sign));
    case SH_SWISH: return sf_fma(f, a, h, sf_mul(f, const_half(f), x));
    default: return SF_CANONICAL_NAN;
    }
}

uint16_t fpt_oracle_eval_lane(int program, uint16_t x) {
    if (program < 0 || program >= k_program_count) return SF_CANONICAL_NAN;
    return eval_lane(&k_programs[program], x);
}

static inline sf_format prog_format(int program) {
    return k_programs[program].dtype == DT_FP16 ? SF_FP16 : SF_BF16;
}

void fpt_oracle_unary(int program, const uint16_t* in, uint16_t* out, int64_t n) {
    const program_row* p = &k_programs[program];
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = eval_lane(p, in[i]);
}

/* y <- F(y) applied `repeats` times (the activation feedback probe) */
void fpt_oracle_unary_repeat(int program, const uint16_t* in, uint16_t* out, int64_t n, int repeats) {
    const program_row* p = &k_programs[program];
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        uint16_t v = in[i];
        for (int r = 0; r < repeats; ++r) v = eval_lane(p, v);
        out[i] = v;
    }
}

void fpt_oracle_binary_bwd(int program, const uint16_t* grad_out, const uint16_t* x, uint16_t* grad_in, int64_t n) {
    const program_row* p = &k_programs[program];
    const sf_format f = prog_format(program);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) grad_in[i] = sf_mul(f, grad_out[i], eval_lane(p, x[i]));
}

void fpt_oracle_swiglu(int program, const uint16_t* gate, const uint16_t* up, uint16_t* out, int64_t n) {
    const program_row* p = &k_programs[program];
    const sf_format f = prog_format(program);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = sf_mul(f, eval_lane(p, gate[i]), up[i]);
}

void fpt_oracle_swiglu_packed(int program, const uint16_t* packed, uint16_t* out, int64_t rows, int64_t hidden) {
    const program_row* p = &k_programs[program];
    const sf_format f = prog_format(program);
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const uint16_t* g = packed + r * 2 * hidden;
        const uint16_t* u = g + hidden;
        uint16_t* o = out + r * hidden;
        for (int64_t c = 0; c < hidden; ++c) o[c] = sf_mul(f, eval_lane(p, g[c]), u[c]);
    }
}

void fpt_oracle_swiglu_bwd(int fwd_program, int bwd_program, const uint16_t* grad_out, const uint16_t* gate,
                           const uint16_t* up, uint16_t* grad_gate, uint16_t* grad_up, int64_t n) {
    const program_row* pf = &k_programs[fwd_program];
    const program_row* pb = &k_programs[bwd_program];
    const sf_format f = prog_format(fwd_program);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        grad_gate[i] = sf_mul(f, sf_mul(f, grad_out[i], up[i]), eval_lane(pb, gate[i]));
        grad_up[i] = sf_mul(f, grad_out[i], eval_lane(pf, gate[i]));
    }
}

/* BF16 D3 backward that derives swish and swish' from one sigmoid evaluation:
 * sig = sigmoid_d3(x); swish = x*sig; swish' = fma(swish, 1 - sig, sig)
 * (spline_kernels_bf16.cu:255-341). `sigmoid_program` is SIGMOID_FWD_D3 bf16. */
void fpt_oracle_swiglu_bwd_shared_sigmoid(int sigmoid_program, const uint16_t* grad_out, const uint16_t* gate,
                                          const uint16_t* up, uint16_t* grad_gate, uint16_t* grad_up, int64_t n) {
    const program_row* ps = &k_programs[sigmoid_program];
    const sf_format f = prog_format(sigmoid_program);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        uint16_t sig = eval_lane(ps, gate[i]);
        uint16_t swish = sf_mul(f, gate[i], sig);
        uint16_t deriv = sf_fma(f, swish, sf_sub(f, const_one(f), sig), sig);
        grad_gate[i] = sf_mul(f, sf_mul(f, grad_out[i], up[i]), deriv);
        grad_up[i] = sf_mul(f, grad_out[i], swish);
    }
}

/* ------------------------------------------------------- B3 direct sigmoid */

/* Deployed n = 4096 constants (bf16 patterns, already scaled by 2^-12).
 * Row 1 is selected where x >= 1.25.  A different sequence length 2^k shifts
 * every forward coefficient by 2^-(k-12), exact in bf16. */
static const uint16_t k_b3_row0[4] = { 0x3980, 0x3987, 0x3909, 0x37e8 }; /* c0..c3, x <  1.25 */
static const uint16_t k_b3_row1[4] = { 0xbb09, 0x3b8c, 0xbb11, 0x3a09 }; /* c0..c3, x >= 1.25 */
static const uint16_t k_b3_grad0[2] = { 0x3f80, 0xbc10 };                /* intercept, slope */
static const uint16_t k_b3_grad1[2] = { 0x3f81, 0xbb38 };

static inline uint16_t bf16_scale_pow2(uint16_t x, int down) { /* exact while the result stays normal */
    return (uint16_t)(x - ((uint16_t)down << 7));
}

static void b3_lane(uint16_t x, int log2_n, uint16_t* value, uint16_t* grad) {
    const sf_format f = SF_BF16;
    const int row = sf_ge(f, x, 0x3fa0u);
    uint16_t c = sf_min(f, x, 0x40c0u);
    c = sf_max(f, c, 0xc0c0u);
    const uint16_t* k = row ? k_b3_row1 : k_b3_row0;
    const int down = log2_n - 12;
    uint16_t v = bf16_scale_pow2(k[3], down);
    v = sf_fma(f, c, v, bf16_scale_pow2(k[2], down));
    v = sf_fma(f, c, v, bf16_scale_pow2(k[1], down));
    v = sf_fma(f, c, v, bf16_scale_pow2(k[0], down));
    v = sf_max(f, v, 0x0000u);
    *value = v;
    if (grad) {
        const uint16_t* g = row ? k_b3_grad1 : k_b3_grad0;
        *grad = sf_mul(f, v, sf_fma(f, c, g[1], g[0]));
    }
}

void fpt_oracle_b3_direct_bf16(const uint16_t* scores, uint16_t* prob, uint16_t* grad, int64_t n, int log2_n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) b3_lane(scores[i], log2_n, &prob[i], grad ? &grad[i] : NULL);
}

void fpt_oracle_b3_direct_f32(const float* scores, uint16_t* prob, uint16_t* grad, int64_t n, int log2_n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i)
        b3_lane(sf_from_float(SF_BF16, scores[i]), log2_n, &prob[i], grad ? &grad[i] : NULL);
}

/* ------------------------------------------------ FP16/BF16 composite helpers */

/* one rounded product per lane (reference: multiply_vec_kernel, spline_kernels.cu:1009-1027) */
void fpt_oracle_multiply(const uint16_t* a, const uint16_t* b, uint16_t* out, int64_t n, int dtype) {
    const sf_format f = dtype ? SF_BF16 : SF_FP16;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = sf_mul(f, a[i], b[i]);
}

/* one fused multiply-add per lane: the form a compiler may contract `c + a*b` into */
void fpt_oracle_fma16(const uint16_t* a, const uint16_t* b, const uint16_t* c, uint16_t* out, int64_t n, int dtype) {
    const sf_format f = dtype ? SF_BF16 : SF_FP16;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = sf_fma(f, a[i], b[i], c[i]);
}

/* SiLU forward with the derivative from one shared sigmoid (reference: fwd_deriv_swish_kernel,
 * spline_kernels.cu:981-1006): s given, y = x*s, dy = s * fma(x, 1 - s, 1). */
void fpt_oracle_swish_shared_sigmoid(const uint16_t* x, const uint16_t* s, uint16_t* y, uint16_t* dy, int64_t n, int dtype) {
    const sf_format f = dtype ? SF_BF16 : SF_FP16;
    const uint16_t one = dtype ? 0x3f80u : 0x3c00u;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        y[i] = sf_mul(f, x[i], s[i]);
        dy[i] = sf_mul(f, s[i], sf_fma(f, x[i], sf_sub(f, one, s[i]), one));
    }
}

/* --------------------------------------------------------- fractional exp2 */

/* set 0: least-squares constants compiled into the reference benchmark
 * set 1: endpoint-preserving constants of the paper appendix (p(0)=1, p(1)=2) */
static const uint16_t k_exp2_sets[2][3] = { { 0x3a91, 0x3bea, 0x357b }, { 0x3a62, 0x3c00, 0x3676 } };

static inline uint16_t exp2_hinge_lane(uint16_t x, int set) {
    const sf_format f = SF_FP16;
    uint16_t hinge = sf_max(f, sf_sub(f, x, 0x3800u), 0x0000u);
    uint16_t base = sf_fma(f, x, k_exp2_sets[set][0], k_exp2_sets[set][1]);
    return sf_fma(f, hinge, k_exp2_sets[set][2], base);
}

void fpt_oracle_exp2_hinge(const uint16_t* in, uint16_t* out, int64_t n, int set) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = exp2_hinge_lane(in[i], set);
}

/* r evaluations per element with the benchmark's feedback x <- fma(v, 0.5, -0.5) */
void fpt_oracle_exp2_hinge_repeat(const uint16_t* in, uint16_t* out, int64_t n, int set, int repeats) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        uint16_t x = in[i], v = 0;
        for (int r = 0; r < repeats; ++r) {
            v = exp2_hinge_lane(x, set);
            x = sf_fma(SF_FP16, v, 0x3800u, 0xb800u);
        }
        out[i] = v;
    }
}

/* Full-range fp32 2^a of the reference's routed soft-max exponentials (reference:
 * autonumerics_zero/cuda_benchmarks/benchmark_exp2_pwl2.cu:106-198, FullDegree3 and FullPwl2Hinge), restated operation
 * by operation: clamp at -127, floor through a round-DOWN add of 1.5*2^23, fraction in [0,1), a cubic (variant 0) or
 * a continuous two-piece line (variant 1) in the fraction, and the integer part added to the exponent field.  Every
 * step is a single IEEE-754 binary32 operation, so the device result can be compared bit for bit. */
#include <fenv.h>

static inline float add_round_down(float a, float b) {
    /* nearest sum, its exact error by the two-sum identity (every step volatile binary32), one step down if the
     * nearest sum lies above the exact one */
    volatile float r = a + b;
    volatile float bb = r - a;
    volatile float t = r - bb;
    volatile float ea = a - t;
    volatile float eb = b - bb;
    volatile float err = ea + eb;
    float out = r;
    if (err < 0.0f) out = nextafterf(out, -INFINITY);
    return out;
}

static inline float exp2_full_lane(float a, int variant) {
    volatile float xr, n, f, p;   /* volatile: no step may be fused or reassociated */
    union { float f; uint32_t u; } pb, xb, r;
    /* max(a, floor) with the NaN-dropping rule of PTX max.  The cubic has p >= 1, so -127 ends at bit pattern 0; the
     * two-piece line starts at p = 0.989 < 1, whose exponent field would wrap below -126 (the reference's sequence,
     * floor -127 for both, is only used above that): the device clamps that kind at -126 and so does this. */
    const float floor_value = variant == 1 ? -126.0f : -127.0f;   /* variants 2 and 3 have p(0) = 1 exactly, like the cubic */
    if (!(a >= floor_value)) a = floor_value;
    if (fabsf(a) < 1.17549435e-38f) a = copysignf(0.0f, a);   /* .ftz on every device step: subnormal inputs are zero */
    xr = add_round_down(a, 12582912.0f);
    n = xr - 12582912.0f;
    f = a - n;
    if (variant == 0) {
        p = fmaf(f, 0.07711908966302872f, 0.22756439447402954f);
        p = fmaf(p, f, 0.6951461434364319f);
        p = fmaf(p, f, 1.0f);
    } else if (variant == 1) {
        volatile float h = f - 0.5f;
        if (!(h > 0.0f)) h = 0.0f;
        p = fmaf(f, 0.820852518081665f, 0.9894611835479736f);
        p = fmaf(h, 0.34246066212654114f, p);
    } else if (variant == 2) {
        /* endpoint-preserving quadratic p = 1 + a f + (1 - a) f^2, a = 0.6602339719 (reference:
         * extras/paper/manuscript/appendix_exp2.tex:28-33), two fp32 multiply-adds */
        p = fmaf(f, 0.3397660281f, 0.6602339719f);
        p = fmaf(p, f, 1.0f);
    } else {
        /* endpoint-preserving two-piece line on an fp16 lane, p = 1 + A f + C max(f - 1/2, 0) with the packed fp16
         * constants A = 0.7978515625, C = 0.40380859375 (reference: extras/paper/manuscript/appendix_exp2.tex:23-27,
         * 74-76): f rounded to fp16, hinge by subtract and maximum, two fp16 multiply-adds, widened to fp32 */
        const uint16_t fh = sf_from_float(SF_FP16, f);
        const uint16_t hinge = sf_max(SF_FP16, sf_sub(SF_FP16, fh, 0x3800u), 0x0000u);
        uint16_t ph = sf_fma(SF_FP16, fh, 0x3a62u, 0x3c00u);
        ph = sf_fma(SF_FP16, hinge, 0x3676u, ph);
        p = sf_to_float(SF_FP16, ph);
    }
    pb.f = p; xb.f = xr;
    r.u = pb.u + (xb.u << 23);
    return r.f;
}

void fpt_oracle_exp2_full_f32(const float* in, float* out, int64_t n, int variant) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) out[i] = exp2_full_lane(in[i], variant);
}

/* ------------------------------------------------------------ paired sincos */

typedef struct {
    int reducer;         /* 0 two-term quarter turn (int convert), 1 one-term quarter turn (magic bias),
                            2 one-term half turn (magic bias) */
    int eval_fmt;        /* lane format of the Horner evaluation */
    int out_fmt;         /* lane format of the stored result */
    int n_sin, n_cos;    /* number of coefficients in r^2 */
    float sin_c[4];      /* lowest order first: sin = r*(s0 + s1 r^2 + ...) */
    float cos_c[4];      /* cos = c0 + c1 r^2 + ... */
} sincos_variant;

static const sincos_variant k_sincos[FPT_SINCOS_VARIANT_COUNT] = {
    /* FP16 */
    [FPT_SINCOS_D3_D4_QUARTER_TURN_FP16] = { 1, SF_FP16, SF_FP16, 2, 3, { 0.9990234375f, -0.1602783203125f }, { 1.0f, -0.499755859375f, 0.040435791015625f } },
    [FPT_SINCOS_D3_D4_HALF_TURN_FP16] = { 2, SF_FP16, SF_FP16, 2, 3, { 0.98876953125f, -0.14501953125f }, { 0.99951171875f, -0.496337890625f, 0.037200927734375f } },
    [FPT_SINCOS_D5_D4_HALF_TURN_FP16] = { 2, SF_FP16, SF_FP16, 3, 3, { 0.99951171875f, -0.16552734375f, 0.0074920654296875f }, { 0.99951171875f, -0.49560546875f, 0.036773681640625f } },
    [FPT_SINCOS_D5_D6_HALF_TURN_FP16] = { 2, SF_FP16, SF_FP16, 3, 4, { 0.99951171875f, -0.16552734375f, 0.0074920654296875f }, { 1.0f, -0.499755859375f, 0.041412353515625f, -0.0012674331665039062f } },
    [FPT_SINCOS_D7_D6_HALF_TURN_FP16] = { 2, SF_FP16, SF_FP16, 4, 4, { 1.0f, -0.1666259765625f, 0.00829315185546875f, -0.00018227100372314453f }, { 1.0f, -0.499755859375f, 0.041412353515625f, -0.0012674331665039062f } },
    /* BF16 */
    [FPT_SINCOS_D3_D4_BF16] = { 0, SF_BF16, SF_BF16, 2, 3, { 0.99903142452239990234375f, -0.16034401953220367431640625f }, { 0.999990046024322509765625f, -0.4997082054615020751953125f, 0.0403986163437366485595703125f } },
    [FPT_SINCOS_D3_D4_QUARTER_TURN_BF16] = { 1, SF_BF16, SF_BF16, 2, 3, { 1.0f, -0.162109375f }, { 1.0f, -0.5f, 0.041015625f } },
    [FPT_SINCOS_D3_D4_HALF_TURN_BF16] = { 2, SF_BF16, SF_BF16, 2, 3, { 0.98828125f, -0.1455078125f }, { 1.0f, -0.49609375f, 0.037109375f } },
    [FPT_SINCOS_D5_D6_HALF_TURN_BF16] = { 2, SF_BF16, SF_BF16, 3, 4, { 1.0f, -0.166015625f, 0.007598876953125f }, { 1.0f, -0.5f, 0.04150390625f, -0.00125885009765625f } },
    [FPT_SINCOS_D5_D4_HALF_TURN_FP16_BF16] = { 2, SF_FP16, SF_BF16, 3, 3, { 0.99951171875f, -0.16552734375f, 0.0074920654296875f }, { 0.99951171875f, -0.49560546875f, 0.036773681640625f } },
};

int fpt_oracle_sincos_is_bf16(int variant) { return k_sincos[variant].out_fmt == SF_BF16; }

/* Range reduction in fp32, every step a single correctly rounded operation. */
static void reduce_angle(int reducer, float angle, float* reduced, unsigned* quadrant_or_sign) {
    if (reducer == 0) {
        const float prod = angle * 0.63661977236758134308f;
        /* cvt.rni.s32.f32 then cvt.rn.f32.s32: the trip through an integer turns -0 into +0
         * (saturation of huge angles is not modelled) */
        const float q = (float)(int)nearbyintf(prod);
        float r = fmaf(q, -1.57079625129699707031f, angle);
        r = fmaf(q, -7.54978941586159635335e-08f, r);
        *reduced = r;
        *quadrant_or_sign = (unsigned)(int)q & 3u;
    } else if (reducer == 1) {
        const float biased = fmaf(angle, 0.63661977236758134308f, 12582912.0f);
        const float q = biased - 12582912.0f;
        *reduced = fmaf(q, -1.57079637050628662109375f, angle);
        *quadrant_or_sign = sf_fbits(biased);
    } else {
        const float biased = fmaf(angle, 0.31830988618379067154f, 12582912.0f);
        const float h = biased - 12582912.0f;
        *reduced = fmaf(h, -3.1415927410125732421875f, angle);
        *quadrant_or_sign = (sf_fbits(biased) & 1u) << 15; /* lane sign bit */
    }
}

static void sincos_lane(const sincos_variant* v, float angle, uint16_t* cos_out, uint16_t* sin_out) {
    const sf_format f = (sf_format)v->eval_fmt;
    float rf; unsigned qs;
    reduce_angle(v->reducer, angle, &rf, &qs);
    const uint16_t r = sf_from_float(f, rf);
    const uint16_t r2 = sf_mul(f, r, r);
    uint16_t s = sf_fma(f, sf_from_float(f, v->sin_c[v->n_sin - 1]), r2, sf_from_float(f, v->sin_c[v->n_sin - 2]));
    for (int k = v->n_sin - 3; k >= 0; --k) s = sf_fma(f, s, r2, sf_from_float(f, v->sin_c[k]));
    s = sf_mul(f, r, s);
    uint16_t c = sf_fma(f, sf_from_float(f, v->cos_c[v->n_cos - 1]), r2, sf_from_float(f, v->cos_c[v->n_cos - 2]));
    for (int k = v->n_cos - 3; k >= 0; --k) c = sf_fma(f, c, r2, sf_from_float(f, v->cos_c[k]));
    if (v->reducer == 2) {
        s ^= (uint16_t)qs; c ^= (uint16_t)qs;
    } else {
        const unsigned q = qs;
        if (q & 1u) { uint16_t t = s; s = c; c = t; }
        s ^= (uint16_t)((q & 2u) << 14);
        c ^= (uint16_t)(((q + 1u) & 2u) << 14);
    }
    if (v->out_fmt != v->eval_fmt) { /* fp16 result widened to fp32, then rounded to bf16 */
        s = sf_from_float((sf_format)v->out_fmt, sf_to_float(f, s));
        c = sf_from_float((sf_format)v->out_fmt, sf_to_float(f, c));
    }
    *sin_out = s; *cos_out = c;
}

void fpt_oracle_sincos_packed(int variant, const float* angles, uint16_t* cos_out, uint16_t* sin_out, int64_t n) {
    const sincos_variant* v = &k_sincos[variant];
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) sincos_lane(v, angles[i], &cos_out[i], &sin_out[i]);
}

/* `iterations` evaluations per angle; sums accumulated in the lane format,
 * probe <- fma(probe, 1 - 2^-24, 2^-13) between evaluations. */
void fpt_oracle_sincos_packed_compute(int variant, const float* angles, uint16_t* cos_out, uint16_t* sin_out,
                                      int64_t n, int iterations) {
    const sincos_variant* v = &k_sincos[variant];
    const sf_format f = (sf_format)v->out_fmt;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        float probe = angles[i];
        uint16_t cs = 0, ss = 0;
        for (int it = 0; it < iterations; ++it) {
            uint16_t c, s;
            sincos_lane(v, probe, &c, &s);
            cs = sf_add(f, cs, c);
            ss = sf_add(f, ss, s);
            probe = fmaf(probe, 0.999999940395355224609375f, 0.0001220703125f);
        }
        cos_out[i] = cs; sin_out[i] = ss;
    }
}

/* ------------------------------------------------------- fp32 paired sincos */

/* The fp32 family (reference: sincos_kernels.cu:24-118 reducers and quadrant restore, :129-406 evaluators):
 * range reduction, Horner in r^2 and sign / swap restore, every step one binary32 operation.  Variants:
 * 1 D3/D4 quarter turn, two-term pi/2, integer conversion   2 D3/D4 in turns with symmetry folding
 * 3 D3/D4 quarter turn, two-term, magic bias                4 D5/D4 half turn, least squares
 * 5 D5/D4 half turn, Sollya                                 6 the same with one-term pi
 * 7 D5/D4 quarter turn                                      8 D7/D6 quarter turn            (0 = native: no oracle) */
typedef struct { int reducer; int n_sin, n_cos; float sin_c[4]; float cos_c[4]; } sincos_f32_variant;
enum { RED_QUARTER_CVT = 0, RED_CYCLE = 1, RED_QUARTER_MAGIC2 = 2, RED_HALF_MAGIC2 = 3, RED_HALF_MAGIC1 = 4 };

static const sincos_f32_variant k_sincos_f32[9] = {
    [1] = { RED_QUARTER_CVT, 2, 3, { 0.99903142452239990234375f, -0.16034401953220367431640625f },
            { 0.999990046024322509765625f, -0.4997082054615020751953125f, 0.0403986163437366485595703125f } },
    [2] = { RED_CYCLE, 2, 3, { 6.277099609375f, -39.77336883544921875f },
            { 0.999990046024322509765625f, -19.7276897430419921875f, 62.96308135986328125f } },
    [3] = { RED_QUARTER_MAGIC2, 2, 3, { 0.99903142452239990234375f, -0.16034401953220367431640625f },
            { 0.999990046024322509765625f, -0.4997082054615020751953125f, 0.0403986163437366485595703125f } },
    [4] = { RED_HALF_MAGIC2, 3, 3, { 0.999771416187286376953125f, -0.16582702100276947021484375f, 0.00757423602044582366943359375f },
            { 0.999579489231109619140625f, -0.4963922202587127685546875f, 0.0372092612087726593017578125f } },
    [5] = { RED_HALF_MAGIC2, 3, 3, { 0.999696791172027587890625f, -0.1656731069087982177734375f, 0.0075143859721720218658447265625f },
            { 0.9994032382965087890625f, -0.495580852031707763671875f, 0.03679168224334716796875f } },
    [6] = { RED_HALF_MAGIC1, 3, 3, { 0.999696791172027587890625f, -0.1656731069087982177734375f, 0.0075143859721720218658447265625f },
            { 0.9994032382965087890625f, -0.495580852031707763671875f, 0.03679168224334716796875f } },
    [7] = { RED_QUARTER_CVT, 3, 3, { 0.9999962449073792f, -0.16661198437213898f, 0.008137642405927181f },
            { 0.999993085861206f, -0.499763548374176f, 0.04051213711500168f } },
    [8] = { RED_QUARTER_CVT, 4, 4, { 1.0f, -0.1666664183139801f, 0.00833179522305727f, -0.00019484198128338903f },
            { 1.0f, -0.49999886751174927f, 0.041656624525785446f, -0.0013605882413685322f } },
};

static inline float f32_xor(float v, unsigned sign) {
    uint32_t u = sf_fbits(v) ^ sign;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

static void sincos_f32_lane(const sincos_f32_variant* v, float angle, float* cos_out, float* sin_out) {
    volatile float r = 0.0f, r2, sp, cp;   /* volatile: each step stays a separate rounded operation */
    unsigned sin_sign = 0, cos_sign = 0;
    int swap = 0;
    if (v->reducer == RED_QUARTER_CVT || v->reducer == RED_QUARTER_MAGIC2) {
        unsigned q;
        volatile float qf;
        if (v->reducer == RED_QUARTER_CVT) {
            volatile float prod = angle * 0.63661977236758134308f;
            const int qi = (int)nearbyintf(prod);
            qf = (float)qi;
            q = (unsigned)qi;
        } else {
            volatile float biased = fmaf(angle, 0.63661977236758134308f, 12582912.0f);
            qf = biased - 12582912.0f;
            q = sf_fbits(biased);
        }
        r = fmaf(qf, -1.57079625129699707031f, angle);
        r = fmaf(qf, -7.54978941586159635335e-08f, r);
        swap = (int)(q & 1u);
        sin_sign = (q & 2u) << 30;
        cos_sign = ((q + 1u) & 2u) << 30;
    } else if (v->reducer == RED_HALF_MAGIC2 || v->reducer == RED_HALF_MAGIC1) {
        volatile float biased = fmaf(angle, 0.31830988618379067154f, 12582912.0f);
        volatile float h = biased - 12582912.0f;
        if (v->reducer == RED_HALF_MAGIC2) {
            r = fmaf(h, -3.141592502593994140625f, angle);
            r = fmaf(h, -1.50995788317231927067e-07f, r);
        } else {
            r = fmaf(h, -3.1415927410125732421875f, angle);
        }
        sin_sign = cos_sign = (sf_fbits(biased) & 1u) << 31;
    } else {
        volatile float cycles = angle * 0.15915494309189533577f;
        volatile float wrapped = cycles - nearbyintf(cycles);
        sin_sign = sf_fbits(wrapped) & 0x80000000u;
        volatile float a = fabsf(wrapped);
        const int outer = a > 0.25f;
        if (outer) a = 0.5f - a;
        swap = a > 0.125f;
        if (swap) a = 0.25f - a;
        r = a;
        cos_sign = (unsigned)outer << 31;
    }
    r2 = r * r;
    sp = fmaf(v->sin_c[v->n_sin - 1], r2, v->sin_c[v->n_sin - 2]);
    for (int k = v->n_sin - 3; k >= 0; --k) sp = fmaf(sp, r2, v->sin_c[k]);
    sp = r * sp;
    cp = fmaf(v->cos_c[v->n_cos - 1], r2, v->cos_c[v->n_cos - 2]);
    for (int k = v->n_cos - 3; k >= 0; --k) cp = fmaf(cp, r2, v->cos_c[k]);
    const float sm = swap ? cp : sp, cm = swap ? sp : cp;
    *sin_out = f32_xor(sm, sin_sign);
    *cos_out = f32_xor(cm, cos_sign);
}

/* out [2, n]: cos plane then sin plane.  iterations == 0: one evaluation; > 0: the repeated-evaluation probe
 * (sums of `iterations` evaluations, probe <- fma(probe, 1 - 2^-24, 2^-13) between them). */
int fpt_oracle_sincos_f32(int variant, const float* angles, float* out, int64_t n, int iterations) {
    if (variant < 1 || variant > 8) return -1;
    const sincos_f32_variant* v = &k_sincos_f32[variant];
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        if (iterations <= 0) {
            sincos_f32_lane(v, angles[i], &out[i], &out[n + i]);
        } else {
            volatile float cs = 0.0f, ss = 0.0f, probe = angles[i];
            for (int it = 0; it < iterations; ++it) {
                float c, s2;
                sincos_f32_lane(v, probe, &c, &s2);
                cs = cs + c;
                ss = ss + s2;
                probe = fmaf(probe, 0.999999940395355224609375f, 0.0001220703125f);
            }
            out[i] = cs; out[n + i] = ss;
        }
    }
    return 0;
}

/* ------------------------------------------------------------------- RoPE */

static inline uint16_t f16c(float x) { return sf_from_float(SF_FP16, x); }

/* Q0.32 phase -> (cos, sin) in fp16, half-turn residual, sin D5 / cos D6 */
static void rope_half_turn_d5_d6(uint32_t position, uint32_t increment, uint16_t* cos_out, uint16_t* sin_out) {
    const sf_format f = SF_FP16;
    const uint32_t phase = position * increment;
    const int16_t q15 = (int16_t)(uint16_t)(phase >> 15);
    const uint16_t hi = (uint16_t)(phase >> 16);
    const uint16_t sign = (uint16_t)((hi ^ (uint16_t)(hi << 1)) & 0x8000u);
    const uint16_t r = sf_mul(f, sf_from_double(f, (double)q15), f16c(0x1p-15f));
    const uint16_t r2 = sf_mul(f, r, r);
    uint16_t s = sf_fma(f, f16c(0.072021484375f), r2, f16c(-0.64208984375f));
    s = sf_fma(f, s, r2, f16c(1.5703125f));
    s = sf_mul(f, r, s);
    uint16_t c = sf_fma(f, f16c(-0.0190887451171875f), r2, f16c(0.25244140625f));
    c = sf_fma(f, c, r2, f16c(-1.2333984375f));
    c = sf_fma(f, c, r2, f16c(1.0f));
    *sin_out = s ^ sign; *cos_out = c ^ sign;
}

/* Q0.32 phase, quarter-turn residual, sin D3 / cos D4 */
static void rope_quarter_turn_d3_d4(uint32_t position, uint32_t increment, uint16_t* cos_out, uint16_t* sin_out) {
    const sf_format f = SF_FP16;
    const uint32_t phase = position * increment;
    const uint32_t quadrant = (phase + 0x20000000u) >> 30;
    const int32_t residual = (int32_t)(phase - (quadrant << 30));
    const int16_t q15 = (int16_t)(residual >> 14);
    const uint16_t r = sf_mul(f, sf_from_double(f, (double)q15), f16c(0x1p-15f));
    const uint16_t r2 = sf_mul(f, r, r);
    uint16_t s = sf_fma(f, f16c(-0.07763671875f), r2, f16c(0.78466796875f));
    s = sf_mul(f, r, s);
    uint16_t c = sf_fma(f, f16c(0.01538848876953125f), r2, f16c(-0.308349609375f));
    c = sf_fma(f, c, r2, f16c(1.0f));
    if (quadrant & 1u) { uint16_t t = s; s = c; c = t; }
    s ^= (uint16_t)((quadrant & 2u) << 14);
    c ^= (uint16_t)(((quadrant + 1u) & 2u) << 14);
    *sin_out = s; *cos_out = c;
}

/* table layout [2, S, F]: cos plane first, then sin plane */
void fpt_oracle_rope_table(int kind, const uint32_t* increments, uint16_t* table, int64_t seq, int64_t freq_count) {
    uint16_t* cos_plane = table;
    uint16_t* sin_plane = table + seq * freq_count;
#pragma omp parallel for schedule(static)
    for (int64_t p = 0; p < seq; ++p)
        for (int64_t j = 0; j < freq_count; ++j) {
            if (kind == FPT_ROPE_HALF_TURN_D5_D6)
                rope_half_turn_d5_d6((uint32_t)p, increments[j], &cos_plane[p * freq_count + j], &sin_plane[p * freq_count + j]);
            else
                rope_quarter_turn_d3_d4((uint32_t)p, increments[j], &cos_plane[p * freq_count + j], &sin_plane[p * freq_count + j]);
        }
}

/* Table-lookup RoPE sin/cos (reference: evaluate_rope_phase_lut_fp16, sincos_kernels.cu:1350-1385): the 7 top
 * phase bits (rounded) pick (sin, cos) of a 128-entry table, the signed remainder becomes an fp16 angle delta and
 * one first-order step follows: sin = fma(delta, cos_b, sin_b), cos = fma(-delta, sin_b, cos_b).
 * lut: 128 words, low half sin, high half cos.  iterations > 0: sums over positions p, p+1, ... in fp16. */
static void rope_lut_lane(uint32_t position, uint32_t inc, const uint32_t* lut, uint16_t* cos_out, uint16_t* sin_out) {
    const sf_format f = SF_FP16;
    const uint32_t phase = position * inc;
    const uint32_t index = ((phase + (1u << 24)) >> 25) & 127u;
    const int32_t residual = (int32_t)(phase - (index << 25));
    volatile float radians = (float)residual * 0x1.921fb6p-30f;
    const uint16_t delta = sf_from_float(f, radians);
    const uint16_t sin_b = (uint16_t)(lut[index] & 0xffffu), cos_b = (uint16_t)(lut[index] >> 16);
    *sin_out = sf_fma(f, delta, cos_b, sin_b);
    *cos_out = sf_fma(f, delta ^ 0x8000u, sin_b, cos_b);
}

void fpt_oracle_rope_table_lut(const uint32_t* increments, const uint32_t* lut, uint16_t* table, int64_t seq,
                               int64_t freq_count, int iterations) {
    uint16_t* cos_plane = table;
    uint16_t* sin_plane = table + seq * freq_count;
#pragma omp parallel for schedule(static)
    for (int64_t p = 0; p < seq; ++p)
        for (int64_t j = 0; j < freq_count; ++j) {
            uint16_t c, s;
            if (iterations <= 0) {
                rope_lut_lane((uint32_t)p, increments[j], lut, &c, &s);
            } else {
                c = s = 0;
                for (int it = 0; it < iterations; ++it) {
                    uint16_t c1, s1;
                    rope_lut_lane((uint32_t)p + (uint32_t)it, increments[j], lut, &c1, &s1);
                    c = sf_add(SF_FP16, c, c1);
                    s = sf_add(SF_FP16, s, s1);
                }
            }
            cos_plane[p * freq_count + j] = c;
            sin_plane[p * freq_count + j] = s;
        }
}

/* Rotate interleaved (even, odd) pairs of one [B,S,H,D] tensor and write it
 * transposed as [B,H,S,D].  even' = fma(-sin, odd, cos*even), odd' = fma(sin, even, cos*odd).
 * out_fmt: 0 keeps fp16 (reference layout and dtype); 1 reads/writes bf16 by converting the
 * input exactly to fp32 -> fp16 (RNE) before the rotation and the fp16 result to bf16 (RNE) after. */
static void rope_apply_one(const uint16_t* in, uint16_t* out, const uint32_t* increments, int64_t B, int64_t S,
                           int64_t H, int64_t D, int io_bf16) {
    const sf_format f = SF_FP16;
#pragma omp parallel for collapse(2) schedule(static)
    for (int64_t b = 0; b < B; ++b)
        for (int64_t s = 0; s < S; ++s)
            for (int64_t j = 0; j < D / 2; ++j) {
                uint16_t c, sn;
                rope_half_turn_d5_d6((uint32_t)s, increments[j], &c, &sn);
                for (int64_t h = 0; h < H; ++h) {
                    const uint16_t* src = in + (((b * S + s) * H + h) * D) + 2 * j;
                    uint16_t* dst = out + (((b * H + h) * S + s) * D) + 2 * j;
                    uint16_t e = src[0], o = src[1];
                    if (io_bf16) { e = sf_from_float(f, sf_to_float(SF_BF16, e)); o = sf_from_float(f, sf_to_float(SF_BF16, o)); }
                    uint16_t re = sf_fma(f, sn ^ 0x8000u, o, sf_mul(f, c, e));
                    uint16_t ro = sf_fma(f, sn, e, sf_mul(f, c, o));
                    if (io_bf16) { re = sf_from_float(SF_BF16, sf_to_float(f, re)); ro = sf_from_float(SF_BF16, sf_to_float(f, ro)); }
                    dst[0] = re; dst[1] = ro;
                }
            }
}

void fpt_oracle_rope_apply(const uint16_t* q, const uint16_t* k, const uint32_t* increments, uint16_t* q_out,
                           uint16_t* k_out, int64_t B, int64_t S, int64_t Hq, int64_t Hk, int64_t D, int io_bf16) {
    rope_apply_one(q, q_out, increments, B, S, Hq, D, io_bf16);
    rope_apply_one(k, k_out, increments, B, S, Hk, D, io_bf16);
}

/* -------------------------------------------------------------- attention */

static inline float bf16f(uint16_t x) { return sf_ffrom((uint32_t)x << 16); }

/* fp32 reference attention for selected query rows of one (batch, q_head).
 * Layout (B,S,H,D) bf16.  mode 0: causal softmax with tanh soft-cap through the
 * bf16 TANH_FWD_D4 program: s' = cap * tanhD4(bf16(s*scale/cap)); probabilities in
 * fp32, rounded to bf16 before P.V.  mode 1: sigmoid attention, p = B3direct(bf16(s*scale))
 * with the 2^-log2_n scaling, no mask unless `causal`, O = P.V without normalisation.
 * mode 2: plain softmax (no soft-cap).  Output fp32 [n_rows, D]. */
void fpt_oracle_attention_rows(const uint16_t* q, const uint16_t* k, const uint16_t* v, float* out,
                               int64_t B, int64_t S, int64_t Hq, int64_t Hk, int64_t D, int64_t b, int64_t hq,
                               const int64_t* rows, int64_t n_rows, int mode, int causal, float scale,
                               float softcap, int log2_n) {
    (void)B;
    const int64_t hk = hq / (Hq / Hk);
    const int tanh_prog = fpt_oracle_find_program("TANH_FWD_D4", DT_BF16, SRC_CURRENT);
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t ri = 0; ri < n_rows; ++ri) {
        const int64_t i = rows[ri];
        const int64_t limit = causal ? i + 1 : S;
        float* sc = (float*)malloc((size_t)limit * sizeof(float));
        const uint16_t* qi = q + ((b * S + i) * Hq + hq) * D;
        float row_max = -INFINITY;
        for (int64_t j = 0; j < limit; ++j) {
            const uint16_t* kj = k + ((b * S + j) * Hk + hk) * D;
            float acc = 0.f;
            for (int64_t d = 0; d < D; ++d) acc += bf16f(qi[d]) * bf16f(kj[d]);
            float s = acc * scale;
            if (mode == 0) {
                uint16_t xb = sf_from_float(SF_BF16, s / softcap);
                s = softcap * bf16f(fpt_oracle_eval_lane(tanh_prog, xb));
            } else if (mode == 1) {
                uint16_t p, xb = sf_from_float(SF_BF16, s);
                b3_lane(xb, log2_n, &p, NULL);
                s = bf16f(p);
            } else if (mode == 3) {            /* native control of mode 0: exact tanh in fp32, no polynomial */
                s = softcap * tanhf(s / softcap);
            } else if (mode == 4) {            /* native control of mode 1: exact sigmoid(s - log n), rounded to bf16 */
                const double bias = (double)log2_n * 0.69314718055994530942;
                s = bf16f(sf_from_float(SF_BF16, (float)(1.0 / (1.0 + exp(bias - (double)s)))));
            }
            sc[j] = s;
            if (s > row_max) row_max = s;
        }
        const int unnormalised = mode == 1 || mode == 4;
        double denom = 0.0;
        if (!unnormalised) {
            for (int64_t j = 0; j < limit; ++j) { sc[j] = expf(sc[j] - row_max); denom += sc[j]; }
        }
        float* o = out + ri * D;
        for (int64_t d = 0; d < D; ++d) o[d] = 0.f;
        for (int64_t j = 0; j < limit; ++j) {
            const float p = unnormalised ? sc[j] : bf16f(sf_from_float(SF_BF16, sc[j]));
            const uint16_t* vj = v + ((b * S + j) * Hk + hk) * D;
            for (int64_t d = 0; d < D; ++d) o[d] += p * bf16f(vj[d]);
        }
        if (!unnormalised) for (int64_t d = 0; d < D; ++d) o[d] = (float)(o[d] / denom);
        free(sc);
    }
}

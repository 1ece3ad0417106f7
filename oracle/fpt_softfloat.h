/*
 * TEST INFRASTRUCTURE ONLY -- exact software model of the packed 16-bit lane
 * arithmetic that the GPU kernels execute (one lane of HFMA2 / HMUL2 / HADD2 /
 * HMNMX2 on fp16 and bf16).  Nothing in the shipped library includes this file.
 *
 * Contract (one lane):
 *   fma  : a*b+c computed exactly, rounded ONCE to nearest-even in the lane format
 *   mul / add / sub : one nearest-even rounding
 *   subnormals are kept (packed 16-bit arithmetic has no flush-to-zero mode),
 *   overflow goes to infinity, every NaN result is the canonical 0x7fff,
 *   min / max follow PTX `min/max.{f16x2,bf16x2}` without `.NaN`: a single NaN
 *   operand is dropped, two NaNs give the canonical NaN, and -0 < +0.
 *
 * Method: both formats convert exactly to double.  A product of two lane values
 * has at most 22 significant bits and is exact in double.  The sum p + c may
 * need more than 53 bits, so it is formed with round-to-odd (sticky) in double
 * and only then rounded to the 11-bit or 8-bit target, which is a correct
 * single rounding because 53 >= 2*11 + 2.
 */
#ifndef FPT_SOFTFLOAT_H
#define FPT_SOFTFLOAT_H

#include <math.h>
#include <stdint.h>
#include <string.h>

typedef enum { SF_FP16 = 0, SF_BF16 = 1 } sf_format;

#define SF_CANONICAL_NAN 0x7fffu

static inline uint64_t sf_dbits(double d) { uint64_t u; memcpy(&u, &d, 8); return u; }
static inline double sf_dfrom(uint64_t u) { double d; memcpy(&d, &u, 8); return d; }
static inline uint32_t sf_fbits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float sf_ffrom(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

static inline int sf_is_nan(sf_format f, uint16_t x) {
    return f == SF_FP16 ? ((x & 0x7c00u) == 0x7c00u && (x & 0x03ffu))
                        : ((x & 0x7f80u) == 0x7f80u && (x & 0x007fu));
}

/* exact widening */
static inline double sf_to_double(sf_format f, uint16_t x) {
    if (f == SF_BF16) return (double)sf_ffrom((uint32_t)x << 16);
    int sign = x >> 15, e = (x >> 10) & 31, m = x & 1023;
    double v;
    if (e == 31) v = m ? NAN : INFINITY;
    else if (e == 0) v = ldexp((double)m, -24);
    else v = ldexp((double)(m + 1024), e - 25);
    return sign ? -v : v;
}

/* one nearest-even rounding of a double into the lane format */
static inline uint16_t sf_from_double(sf_format f, double d) {
    const int p = f == SF_FP16 ? 11 : 8;
    const int emin = f == SF_FP16 ? -14 : -126;
    const int emax = f == SF_FP16 ? 15 : 127;
    const int mbits = p - 1;
    const int bias = emax;
    if (isnan(d)) return SF_CANONICAL_NAN;
    uint16_t sign = (uint16_t)((sf_dbits(d) >> 63) << 15);
    double a = fabs(d);
    uint16_t inf = (uint16_t)(sign | (f == SF_FP16 ? 0x7c00u : 0x7f80u));
    if (isinf(a)) return inf;
    if (a == 0.0) return sign;
    int e2;
    (void)frexp(a, &e2);            /* a = m * 2^e2, m in [0.5, 1) */
    int e = e2 - 1;
    if (e < emin) e = emin;
    double q = rint(ldexp(a, mbits - e)); /* default rounding mode: nearest even */
    if (q == ldexp(1.0, p)) { q = ldexp(1.0, p - 1); e += 1; }
    if (e > emax) return inf;
    uint32_t qi = (uint32_t)q;
    if (qi < (1u << mbits)) return (uint16_t)(sign | qi);       /* subnormal / zero */
    return (uint16_t)(sign | ((uint32_t)(e + bias) << mbits) | (qi - (1u << mbits)));
}

/* a + b in double with round-to-odd, so that a later narrowing rounds once */
static inline double sf_add_sticky(double a, double b) {
    double s = a + b;
    if (!isfinite(s) || !isfinite(a) || !isfinite(b)) return s;
    double bb = s - a;
    double err = (a - (s - bb)) + (b - bb);
    if (err != 0.0) {
        uint64_t u = sf_dbits(s);
        if (!(u & 1u)) {
            if ((err > 0.0) == (s > 0.0)) u += 1; else u -= 1;
            s = sf_dfrom(u);
        }
    }
    return s;
}

static inline uint16_t sf_fma(sf_format f, uint16_t a, uint16_t b, uint16_t c) {
    if (sf_is_nan(f, a) || sf_is_nan(f, b) || sf_is_nan(f, c)) return SF_CANONICAL_NAN;
    double p = sf_to_double(f, a) * sf_to_double(f, b);           /* exact, or NaN for inf*0 */
    return sf_from_double(f, sf_add_sticky(p, sf_to_double(f, c)));
}
static inline uint16_t sf_mul(sf_format f, uint16_t a, uint16_t b) {
    if (sf_is_nan(f, a) || sf_is_nan(f, b)) return SF_CANONICAL_NAN;
    return sf_from_double(f, sf_to_double(f, a) * sf_to_double(f, b));
}
static inline uint16_t sf_add(sf_format f, uint16_t a, uint16_t b) {
    if (sf_is_nan(f, a) || sf_is_nan(f, b)) return SF_CANONICAL_NAN;
    return sf_from_double(f, sf_add_sticky(sf_to_double(f, a), sf_to_double(f, b)));
}
static inline uint16_t sf_sub(sf_format f, uint16_t a, uint16_t b) {
    return sf_add(f, a, (uint16_t)(b ^ 0x8000u));
}
/* ordered key: total order on non-NaN patterns with -0 < +0 */
static inline int32_t sf_key(uint16_t x) { return (x & 0x8000u) ? -(int32_t)(x & 0x7fffu) - 1 : (int32_t)x; }
static inline uint16_t sf_min(sf_format f, uint16_t a, uint16_t b) {
    int na = sf_is_nan(f, a), nb = sf_is_nan(f, b);
    if (na && nb) return SF_CANONICAL_NAN;
    if (na) return b;
    if (nb) return a;
    return sf_key(a) <= sf_key(b) ? a : b;
}
static inline uint16_t sf_max(sf_format f, uint16_t a, uint16_t b) {
    int na = sf_is_nan(f, a), nb = sf_is_nan(f, b);
    if (na && nb) return SF_CANONICAL_NAN;
    if (na) return b;
    if (nb) return a;
    return sf_key(a) >= sf_key(b) ? a : b;
}
/* ordered >= : false when either side is NaN; -0 == +0 */
static inline int sf_ge(sf_format f, uint16_t a, uint16_t b) {
    if (sf_is_nan(f, a) || sf_is_nan(f, b)) return 0;
    return sf_to_double(f, a) >= sf_to_double(f, b);
}
/* cvt.rn.{f16,bf16}.f32 */
static inline uint16_t sf_from_float(sf_format f, float x) { return sf_from_double(f, (double)x); }
static inline float sf_to_float(sf_format f, uint16_t x) { return (float)sf_to_double(f, x); }

#endif

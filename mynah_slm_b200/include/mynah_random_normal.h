/* Counter-based normal random numbers: value = f(seed, tensor key, element index).
 *
 * The random-weights mode fills tensors with this function, on the device (a kernel) and on the host (the
 * folder writer); a test's plain implementation evaluates it element by element. All three give the same
 * bits, because the function uses only operations that IEEE 754 rounds exactly (add, multiply, divide, square
 * root in double, never fused) in one fixed order, and no library logarithm or cosine:
 *
 *   z      = mix64(state + (index + 1) * 0x9E3779B97F4A7C15)            (the splitmix64 output function)
 *   u1     = (high 32 bits of z + 1) / 2^32   in (0, 1]
 *   u2     = (low 32 bits of z) / 2^32        in [0, 1)
 *   normal = sqrt(-2 ln u1) * cos(2 pi u2)                              (Box-Muller, the cosine branch only)
 *   ln     : u1 = m * 2^e with m in [sqrt(1/2), sqrt(2)); ln m = 2 s (1 + s^2/3 + ... + s^24/25), s = (m-1)/(m+1)
 *   cos    : quadrant of u2 taken exactly (u2 is a multiple of 2^-32), the angle folded to [0, pi/4], Taylor
 *            polynomials of sine and cosine to x^19 and x^18
 *   state  = mix64(seed + 0x9E3779B97F4A7C15) ^ tensor key              (the key: FNV-1a of the tensor's name)
 *
 * The value stored is (float)(mean + std * normal), then rounded to bfloat16 (nearest, ties to even) when the
 * tensor is bfloat16. The reference has no random-weights mode (mynah-slm .github/workflows/build.yml:10-13).
 */
#ifndef MYNAH_RANDOM_NORMAL_H
#define MYNAH_RANDOM_NORMAL_H

#include <stdint.h>
#include <string.h>

#if defined(__CUDA_ARCH__)
#define MYNAH_RN_FN __device__ __forceinline__
#define MYNAH_RN_MUL(a, b) __dmul_rn((a), (b))
#define MYNAH_RN_ADD(a, b) __dadd_rn((a), (b))
#define MYNAH_RN_DIV(a, b) __ddiv_rn((a), (b))
#define MYNAH_RN_SQRT(a) __dsqrt_rn((a))
#define MYNAH_RN_BITS(d) __double_as_longlong((d))
#define MYNAH_RN_FROM_BITS(i) __longlong_as_double((i))
#else
#define MYNAH_RN_FN static inline
#define MYNAH_RN_MUL(a, b) ((a) * (b))       /* compile host code with -ffp-contract=off */
#define MYNAH_RN_ADD(a, b) ((a) + (b))
#define MYNAH_RN_DIV(a, b) ((a) / (b))
#define MYNAH_RN_SQRT(a) __builtin_sqrt((a))
static inline long long mynah_rn_bits(double d) { long long i; memcpy(&i, &d, 8); return i; }
static inline double mynah_rn_from_bits(long long i) { double d; memcpy(&d, &i, 8); return d; }
#define MYNAH_RN_BITS(d) mynah_rn_bits((d))
#define MYNAH_RN_FROM_BITS(i) mynah_rn_from_bits((i))
#endif

#define MYNAH_RN_GAMMA 0x9E3779B97F4A7C15ull

MYNAH_RN_FN uint64_t mynah_rn_mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

MYNAH_RN_FN uint64_t mynah_rn_state(uint64_t seed, uint64_t tensor_key) {
    return mynah_rn_mix64(seed + MYNAH_RN_GAMMA) ^ tensor_key;
}

/* ln(u) for u = k / 2^32, k in [1, 2^32]. */
MYNAH_RN_FN double mynah_rn_log(double u) {
    const long long bits = MYNAH_RN_BITS(u);
    int e = (int)((bits >> 52) & 0x7ff) - 1022;                                   /* u = m * 2^e, m in [1/2, 1) */
    double m = MYNAH_RN_FROM_BITS((bits & 0x000fffffffffffffll) | 0x3fe0000000000000ll);
    if (m < 0.70710678118654752440) {
        m = MYNAH_RN_MUL(m, 2.0);
        e -= 1;
    }
    const double s = MYNAH_RN_DIV(MYNAH_RN_ADD(m, -1.0), MYNAH_RN_ADD(m, 1.0));
    const double s2 = MYNAH_RN_MUL(s, s);
    double p = 1.0 / 25.0;
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, s2), 1.0 / 23.0);
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, s2), 1.0 / 21.0);
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, s2), 1.0 / 19.0);
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, s2), 1.0 / 17.0);
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, s2), 1.0 / 15.0);
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, s2), 1.0 / 13.0);
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, s2), 1.0 / 11.0);
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, s2), 1.0 / 9.0);
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, s2), 1.0 / 7.0);
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, s2), 1.0 / 5.0);
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, s2), 1.0 / 3.0);
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, s2), 1.0);
    const double ln_m = MYNAH_RN_MUL(MYNAH_RN_MUL(2.0, s), p);
    return MYNAH_RN_ADD(MYNAH_RN_MUL((double)e, 0.69314718055994530942), ln_m);
}

/* sin(x) and cos(x) for x in [0, pi/4]. */
MYNAH_RN_FN double mynah_rn_sin_poly(double x) {
    const double x2 = MYNAH_RN_MUL(x, x);
    double p = -1.0 / 121645100408832000.0;                                       /* -1/19! */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), 1.0 / 355687428096000.0);               /*  1/17! */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), -1.0 / 1307674368000.0);                /* -1/15! */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), 1.0 / 6227020800.0);                    /*  1/13! */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), -1.0 / 39916800.0);                     /* -1/11! */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), 1.0 / 362880.0);                        /*  1/9!  */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), -1.0 / 5040.0);                         /* -1/7!  */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), 1.0 / 120.0);                           /*  1/5!  */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), -1.0 / 6.0);                            /* -1/3!  */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), 1.0);
    return MYNAH_RN_MUL(x, p);
}

MYNAH_RN_FN double mynah_rn_cos_poly(double x) {
    const double x2 = MYNAH_RN_MUL(x, x);
    double p = -1.0 / 6402373705728000.0;                                         /* -1/18! */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), 1.0 / 20922789888000.0);                /*  1/16! */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), -1.0 / 87178291200.0);                  /* -1/14! */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), 1.0 / 479001600.0);                     /*  1/12! */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), -1.0 / 3628800.0);                      /* -1/10! */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), 1.0 / 40320.0);                         /*  1/8!  */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), -1.0 / 720.0);                          /* -1/6!  */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), 1.0 / 24.0);                            /*  1/4!  */
    p = MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), -1.0 / 2.0);                            /* -1/2!  */
    return MYNAH_RN_ADD(MYNAH_RN_MUL(p, x2), 1.0);
}

/* cos(2 pi k / 2^32) for k in [0, 2^32). */
MYNAH_RN_FN double mynah_rn_cos_turn(uint32_t k) {
    const uint32_t quadrant = k >> 30;
    const double g = (double)(k & 0x3fffffffu) * (1.0 / 1073741824.0);            /* in [0, 1), exact */
    const int fold = g > 0.5;
    const double a = MYNAH_RN_MUL(fold ? MYNAH_RN_ADD(1.0, -g) : g, 1.57079632679489661923);   /* in [0, pi/4] */
    const double sa = mynah_rn_sin_poly(a), ca = mynah_rn_cos_poly(a);
    const double c = fold ? sa : ca;                                              /* cos(g pi/2) */
    const double s = fold ? ca : sa;                                              /* sin(g pi/2) */
    return quadrant == 0 ? c : quadrant == 1 ? -s : quadrant == 2 ? -c : s;
}

/* The standard normal number of element `index` under `state`. */
MYNAH_RN_FN double mynah_rn_normal(uint64_t state, uint64_t index) {
    const uint64_t z = mynah_rn_mix64(state + (index + 1) * MYNAH_RN_GAMMA);
    const double u1 = MYNAH_RN_MUL(MYNAH_RN_ADD((double)(uint32_t)(z >> 32), 1.0), 1.0 / 4294967296.0);
    const double r = MYNAH_RN_SQRT(MYNAH_RN_MUL(-2.0, mynah_rn_log(u1)));
    return MYNAH_RN_MUL(r, mynah_rn_cos_turn((uint32_t)z));
}

/* (float)(mean + std * normal). */
MYNAH_RN_FN float mynah_rn_value(uint64_t state, uint64_t index, double mean, double std) {
    return (float)MYNAH_RN_ADD(mean, MYNAH_RN_MUL(std, mynah_rn_normal(state, index)));
}

/* float -> bfloat16 bits, nearest, ties to even (the values here are finite). */
MYNAH_RN_FN uint16_t mynah_rn_bf16_bits(float v) {
    uint32_t u;
#if defined(__CUDA_ARCH__)
    u = __float_as_uint(v);
#else
    memcpy(&u, &v, 4);
#endif
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

#endif

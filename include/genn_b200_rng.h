/* genn_b200_rng.h - the random streams of the B200 backend.
 *
 * Part of the library's contract: PROCEDURAL connectivity, device-side
 * initialisation and the stochastic built-in models (PoissonExp, Poisson) draw
 * from a counter-based Philox4x32-10 generator (Salmon, Moraes, Dror, Shaw:
 * "Parallel random numbers: as easy as 1, 2, 3", SC'11) keyed on the model
 * seed, so any element's draws can be regenerated anywhere from
 * (seed, stream, element, time step) with no stored generator state.  The
 * reference keeps an XORWOW state per neuron and a cuRAND Philox state it
 * skips ahead per thread (backendCUDAHIP.cc:270-289); its CPU backend draws
 * from std::mt19937 (generateRunner.cc:101-136).  Neither sequence is
 * reproduced here: results that depend on random draws agree with the
 * reference statistically, not bit for bit.
 *
 * Everything below is integer arithmetic or single IEEE-754 operations
 * (explicit fma, correctly rounded sqrt and divide), so host C and device
 * CUDA code produce identical bits.  Compiles as C99, C++ and CUDA.
 */
#ifndef GENN_B200_RNG_H
#define GENN_B200_RNG_H

#include <stdint.h>
#include <math.h>
#include <string.h>

#if defined(__CUDACC__)
#define B200_HD __host__ __device__ __forceinline__
#else
#define B200_HD static inline
#endif

#if defined(__CUDA_ARCH__)
#define B200_FMUL(a, b) __fmul_rn((a), (b))
#define B200_FADD(a, b) __fadd_rn((a), (b))
#define B200_FSUB(a, b) __fsub_rn((a), (b))
#define B200_FMAF(a, b, c) __fmaf_rn((a), (b), (c))
#define B200_FSQRT(a) __fsqrt_rn((a))
#define B200_FDIV(a, b) __fdiv_rn((a), (b))
#else
/* volatile-free: strict IEEE evaluation is guaranteed by building host code
 * with -ffp-contract=off (each operation below is a single rounding). */
#define B200_FMUL(a, b) ((float)((float)(a) * (float)(b)))
#define B200_FADD(a, b) ((float)((float)(a) + (float)(b)))
#define B200_FSUB(a, b) ((float)((float)(a) - (float)(b)))
#define B200_FMAF(a, b, c) fmaf((a), (b), (c))
#define B200_FSQRT(a) sqrtf((a))
#define B200_FDIV(a, b) ((float)((float)(a) / (float)(b)))
#endif

typedef struct b200_philox_out { uint32_t x[4]; } b200_philox_out;

#define B200_PHILOX_M0 0xD2511F53u
#define B200_PHILOX_M1 0xCD9E8D57u
#define B200_PHILOX_W0 0x9E3779B9u
#define B200_PHILOX_W1 0xBB67AE85u

/* Philox4x32 with 10 rounds: counter c[4], key k[2]. */
B200_HD b200_philox_out b200_philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                           uint32_t k0, uint32_t k1)
{
    for(int r = 0; r < 10; r++) {
        const uint64_t p0 = (uint64_t)B200_PHILOX_M0 * c0;
        const uint64_t p1 = (uint64_t)B200_PHILOX_M1 * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        const uint32_t n1 = (uint32_t)p1;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        const uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += B200_PHILOX_W0;
        k1 += B200_PHILOX_W1;
    }
    b200_philox_out o;
    o.x[0] = c0; o.x[1] = c1; o.x[2] = c2; o.x[3] = c3;
    return o;
}

/* A stream of 32-bit draws for one (stream, element, time step).  Simulation
 * draws use counter {element, stream, timestep[31:0], timestep[46:32]<<16 | block};
 * initialisation draws use {element[31:0], stream, element[63:32], 0x80000000 | block}. */
typedef struct b200_rng {
    uint32_t c0, c1, c2, c3, k0, k1;
    uint32_t have;             /* unread words left */
    uint32_t w0, w1, w2, w3;   /* unread words, next one in w0 */
} b200_rng;

B200_HD b200_rng b200_rng_sim(uint64_t seed, uint32_t stream, uint32_t element, uint64_t timestep)
{
    b200_rng r;
    r.c0 = element; r.c1 = stream; r.c2 = (uint32_t)timestep;
    r.c3 = ((uint32_t)(timestep >> 32) & 0x7FFFu) << 16;
    r.k0 = (uint32_t)seed; r.k1 = (uint32_t)(seed >> 32);
    r.have = 0;
    r.w0 = r.w1 = r.w2 = r.w3 = 0;
    return r;
}

B200_HD b200_rng b200_rng_init(uint64_t seed, uint32_t stream, uint64_t element)
{
    b200_rng r;
    r.c0 = (uint32_t)element; r.c1 = stream; r.c2 = (uint32_t)(element >> 32);
    r.c3 = 0x80000000u;
    r.k0 = (uint32_t)seed; r.k1 = (uint32_t)(seed >> 32);
    r.have = 0;
    r.w0 = r.w1 = r.w2 = r.w3 = 0;
    return r;
}

B200_HD uint32_t b200_rng_u32(b200_rng *r)
{
    if(r->have == 0) {
        const b200_philox_out o = b200_philox4x32_10(r->c0, r->c1, r->c2, r->c3, r->k0, r->k1);
        r->w0 = o.x[0]; r->w1 = o.x[1]; r->w2 = o.x[2]; r->w3 = o.x[3];
        r->c3 += 1u;
        r->have = 4;
    }
    r->have -= 1;
    {
        const uint32_t out = r->w0;     /* shift instead of indexing: stays in registers */
        r->w0 = r->w1; r->w1 = r->w2; r->w2 = r->w3;
        return out;
    }
}

/* The four words one (stream, element) pair owns for time steps 4j..4j+3:
 * step t uses word t & 3 of the block with counter
 * {element, stream, (t>>2)[31:0], (t>>34)[14:0]<<16}.  A kernel that stays
 * resident across steps computes the block once every four steps. */
B200_HD b200_philox_out b200_rng_step_block(uint64_t seed, uint32_t stream, uint32_t element, uint64_t timestep)
{
    const uint64_t blk = timestep >> 2;
    return b200_philox4x32_10(element, stream, (uint32_t)blk, ((uint32_t)(blk >> 32) & 0x7FFFu) << 16,
                              (uint32_t)seed, (uint32_t)(seed >> 32));
}

B200_HD uint32_t b200_rng_step_word(const b200_philox_out *blk, uint64_t timestep)
{
    const uint32_t j = (uint32_t)timestep & 3u;
    return (j == 0) ? blk->x[0] : (j == 1) ? blk->x[1] : (j == 2) ? blk->x[2] : blk->x[3];
}

/* Uniform in (0, 1): 23 random bits centred in their cell, exact in fp32. */
B200_HD float b200_u32_to_uniform(uint32_t x)
{
    return B200_FMUL(B200_FADD((float)(x >> 9), 0.5f), 1.1920928955078125e-07f);
}

B200_HD float b200_rng_uniform(b200_rng *r)
{
    return b200_u32_to_uniform(b200_rng_u32(r));
}

/* Poisson variate by inversion of the CDF with ONE uniform: sequential search
 * n = 0, 1, 2... until the cumulative probability passes u.  exp_minus_lambda
 * and lambda are supplied pre-rounded to fp32.  Single IEEE operations only. */
B200_HD uint32_t b200_poisson_inverse(float u, float exp_minus_lambda, float lambda)
{
    uint32_t n = 0;
    float p = exp_minus_lambda;
    float s = p;
    while(u > s && n < 64u) {
        n++;
        p = B200_FDIV(B200_FMUL(p, lambda), (float)n);
        s = B200_FADD(s, p);
    }
    return n;
}

/* Natural logarithm for x in (0, 1], built from single IEEE operations so
 * host and device agree bitwise: x = m * 2^e with m in [sqrt(1/2), sqrt(2)),
 * log(m) = 2 atanh(s), s = (m-1)/(m+1), odd series in s to s^9. */
B200_HD float b200_logf(float x)
{
    uint32_t bits;
#if defined(__CUDA_ARCH__)
    bits = __float_as_uint(x);
#else
    memcpy(&bits, &x, sizeof(bits));
#endif
    int e = (int)(bits >> 23) - 127;
    uint32_t mant = (bits & 0x007FFFFFu) | 0x3F800000u;
    float m;
#if defined(__CUDA_ARCH__)
    m = __uint_as_float(mant);
#else
    memcpy(&m, &mant, sizeof(m));
#endif
    if(m > 1.41421356f) {
        m = B200_FMUL(m, 0.5f);
        e += 1;
    }
    const float s = B200_FDIV(B200_FSUB(m, 1.0f), B200_FADD(m, 1.0f));
    const float s2 = B200_FMUL(s, s);
    float p = 0.2222222222f;                 /* 2/9 */
    p = B200_FMAF(p, s2, 0.2857142857f);     /* 2/7 */
    p = B200_FMAF(p, s2, 0.4f);              /* 2/5 */
    p = B200_FMAF(p, s2, 0.6666666667f);     /* 2/3 */
    p = B200_FMAF(p, s2, 2.0f);
    const float lm = B200_FMUL(p, s);
    return B200_FMAF((float)e, 0.6931471805599453f, lm);
}

/* exp(x) for x <= 0 from single IEEE operations: x = n*ln2 + r with
 * |r| <= ln2/2 (two-constant reduction), degree-6 polynomial, exact scaling. */
B200_HD float b200_expf(float x)
{
    if(x < -87.0f) return 0.0f;
    const float nf = rintf(B200_FMUL(x, 1.4426950408889634f));
    float r = B200_FMAF(nf, -0.693145751953125f, x);          /* ln2 high part (exact product) */
    r = B200_FMAF(nf, -1.4286068203094172e-06f, r);           /* ln2 low part */
    float p = 1.3888888889e-03f;                              /* 1/720 */
    p = B200_FMAF(p, r, 8.3333333333e-03f);
    p = B200_FMAF(p, r, 4.1666666667e-02f);
    p = B200_FMAF(p, r, 1.6666666667e-01f);
    p = B200_FMAF(p, r, 0.5f);
    p = B200_FMAF(p, r, 1.0f);
    p = B200_FMAF(p, r, 1.0f);
    const int n = (int)nf;
    const uint32_t sbits = (uint32_t)(n + 127) << 23;         /* n >= -126 here */
    float scale;
#if defined(__CUDA_ARCH__)
    scale = __uint_as_float(sbits);
#else
    memcpy(&scale, &sbits, sizeof(scale));
#endif
    return B200_FMUL(p, scale);
}

/* sin and cos of 2*pi*u for u in [0, 1): octant reduction then polynomials on
 * [-pi/4, pi/4]; single IEEE operations only. */
B200_HD void b200_sincos2pif(float u, float *s, float *c)
{
    const float t = B200_FMUL(u, 8.0f);              /* octants */
    int q = (int)t;                                   /* 0..7 */
    q = (q + 1) >> 1;                                 /* nearest quarter turn 0..4 */
    const float r = B200_FMUL(B200_FSUB(u, B200_FMUL((float)q, 0.25f)), 6.283185307179586f);
    const float r2 = B200_FMUL(r, r);
    float sp = -1.9841269841e-04f;                    /* -1/7! */
    sp = B200_FMAF(sp, r2, 8.3333333333e-03f);        /*  1/5! */
    sp = B200_FMAF(sp, r2, -1.6666666667e-01f);       /* -1/3! */
    sp = B200_FMAF(B200_FMUL(sp, r2), r, r);
    float cp = 2.4801587302e-05f;                     /*  1/8! */
    cp = B200_FMAF(cp, r2, -1.3888888889e-03f);       /* -1/6! */
    cp = B200_FMAF(cp, r2, 4.1666666667e-02f);        /*  1/4! */
    cp = B200_FMAF(cp, r2, -0.5f);
    cp = B200_FMAF(cp, r2, 1.0f);
    switch(q & 3) {
    case 0: *s = sp;  *c = cp;  break;
    case 1: *s = cp;  *c = -sp; break;
    case 2: *s = -sp; *c = -cp; break;
    default: *s = -cp; *c = sp; break;
    }
}

/* Standard normal by Box-Muller from two uniforms; the second variate of the
 * pair is discarded so a draw never depends on earlier calls. */
B200_HD float b200_rng_normal(b200_rng *r)
{
    const float u1 = b200_rng_uniform(r);
    const float u2 = b200_rng_uniform(r);
    const float rad = B200_FSQRT(B200_FMUL(-2.0f, b200_logf(u1)));
    float s, c;
    b200_sincos2pif(u2, &s, &c);
    (void)s;
    return B200_FMUL(rad, c);
}

#endif /* GENN_B200_RNG_H */

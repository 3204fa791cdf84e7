/*
 * srf_canon_math.h -- the library's definition of its float elementary functions.
 *
 * The reference calls atan2f / asinf / cosf / sinf / __expf / __logf from the CUDA
 * math library inside its march and compositing kernels
 * (internal/utils/common_device.h:434-446,510-518, internal/render/ray_marcher.cu:246,
 * internal/sampler/occupancy_sampler.cu:320-322).  That library is documented only by
 * error bounds (atan2f, asinf, cosf: <= 2 ulp), so no CPU code can reproduce its bits.
 * To make "which grid cell does this sample fall in" a question with ONE answer on the
 * host and on the GPU, every elementary function used on the hot path is defined here
 * from IEEE-754 correctly-rounded primitives only (+, -, *, /, sqrt, fma, rint,
 * int<->float conversion).  The same source is compiled by gcc (-ffp-contract=off) and
 * by nvcc (-fmad=false); fused operations appear only where fmaf() is written.
 * Measured maximum errors against float64 libm (tests/test_canon_math.py):
 * atan2f 1.7 ulp, asinf 1.6 ulp, sinf/cosf 1.3 ulp on |x| <= 256, expf 0.9 ulp,
 * logf 1 ulp -- all inside the CUDA library's own documented bounds.
 *
 * Header-only, C++11, no dependencies.  Usable from host and device code.
 */
#ifndef SRF_CANON_MATH_H_
#define SRF_CANON_MATH_H_

#include <math.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define SRF_HD __host__ __device__ __forceinline__
#else
#define SRF_HD inline
#endif

SRF_HD float srf_u32_as_f32(uint32_t u) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f; memcpy(&f, &u, 4); return f;
#endif
}
SRF_HD uint32_t srf_f32_as_u32(float f) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u; memcpy(&u, &f, 4); return u;
#endif
}

/* float -> int with the semantics of the GPU's cvt.rzi.s32.f32: truncate, NaN -> 0,
 * saturate.  The reference's `(p * n).cast<int>()` compiles to that instruction. */
SRF_HD int srf_f2i_rz(float f) {
#if defined(__CUDA_ARCH__)
    return __float2int_rz(f);
#else
    if (f != f) return 0;
    if (f >= 2147483648.0f) return 2147483647;
    if (f <= -2147483648.0f) return (-2147483647 - 1);
    return (int)f;
#endif
}

/*
 * SRF_CANON_PLAIN (host builds of the test oracle only): every fused multiply-add written in this header and in
 * the including file becomes a separate multiply and add, and the elementary functions below become the C
 * library's.  That is the arithmetic a host compile of the reference's own source performs
 * (-ffp-contract=off), so a test oracle built this way can be compared bit for bit with such a compile:
 * a check of that test oracle's control flow, statement order and association order, independent of the
 * elementary-function definitions.
 */
#if defined(SRF_CANON_PLAIN)
#if defined(__CUDACC__)
#error "SRF_CANON_PLAIN is a host-only test mode"
#endif
static inline float srf_plain_fmaf(float a, float b, float c) { return a * b + c; }
static inline double srf_plain_fma(double a, double b, double c) { return a * b + c; }
#define fmaf(a, b, c) srf_plain_fmaf((a), (b), (c))
#define fma(a, b, c) srf_plain_fma((a), (b), (c))
#endif

/* atan(a) for a in [0,1]: a + a*s*P(s), s = a*a, P of degree 8. */
SRF_HD float srf_atan_unit(float a) {
    const float s = a * a;
    float r = -0.00244703121f;
    r = fmaf(r, s, 0.013750284f);
    r = fmaf(r, s, -0.0362701751f);
    r = fmaf(r, s, 0.0628436059f);
    r = fmaf(r, s, -0.0867317095f);
    r = fmaf(r, s, 0.110379942f);
    r = fmaf(r, s, -0.142791107f);
    r = fmaf(r, s, 0.199997663f);
    r = fmaf(r, s, -0.333333313f);
    r = r * s;
    return fmaf(r, a, a);
}

/* atan2f for finite arguments; atan2(0,0) = 0.  Result in (-pi, pi]. */
SRF_HD float srf_atan2f(float y, float x) {
    const float ax = fabsf(x), ay = fabsf(y);
    const float mx = fmaxf(ax, ay), mn = fminf(ax, ay);
    const float a = (mx == 0.0f) ? 0.0f : mn / mx;
    float r = srf_atan_unit(a);
    if (ay > ax) r = (1.57079637f - r) + (-4.37113883e-08f);
    if (x < 0.0f) r = (3.14159274f - r) + (-8.74227766e-08f);
    return (y < 0.0f) ? -r : r;
}

/* asin(x) core on [0, 0.5]: x + x*s*P(s), s = x*x supplied by the caller. */
SRF_HD float srf_asin_core(float x, float s) {
    float r = 0.0338057466f;
    r = fmaf(r, s, 0.0170778595f);
    r = fmaf(r, s, 0.0311161559f);
    r = fmaf(r, s, 0.0445980318f);
    r = fmaf(r, s, 0.0750009865f);
    r = fmaf(r, s, 0.166666657f);
    r = r * s;
    return fmaf(r, x, x);
}

/* asinf; |x| > 1 gives NaN as the C library does. */
SRF_HD float srf_asinf(float x) {
    const float ax = fabsf(x);
    float r;
    if (ax <= 0.5f) {
        r = srf_asin_core(ax, ax * ax);
    } else if (ax <= 1.0f) {
        const float z = (1.0f - ax) * 0.5f;            /* both operations exact */
        const float q = sqrtf(z);
        const float t = srf_asin_core(q, z);
        r = fmaf(-2.0f, t, 1.57079637f) + (-4.37113883e-08f);
    } else {
        r = srf_u32_as_f32(0x7fc00000u);
    }
    return (x < 0.0f) ? -r : r;
}

/* sin and cos together.  Three-term Cody-Waite reduction by pi/2; accurate for
 * |x| <= 256 (the largest angle the inverse sinusoidal warp produces for grids up to
 * 4096 cells across), defined -- with growing error -- up to 65536, NaN beyond. */
SRF_HD void srf_sincosf(float x, float* sn, float* cs) {
    if (!(fabsf(x) <= 65536.0f)) {
        *sn = *cs = srf_u32_as_f32(0x7fc00000u);
        return;
    }
    const float k = rintf(x * 0.636619747f);
    float r = fmaf(-k, 1.5703125f, x);
    r = fmaf(-k, 0.000483751297f, r);
    r = fmaf(-k, 7.54979013e-08f, r);
    const int q = srf_f2i_rz(k) & 3;
    const float s = r * r;
    float ps = 2.72499642e-06f;
    ps = fmaf(ps, s, -0.00019840087f);
    ps = fmaf(ps, s, 0.00833333191f);
    ps = fmaf(ps, s, -0.166666672f);
    const float sr = fmaf(ps * s, r, r);
    float pc = -2.73009874e-07f;
    pc = fmaf(pc, s, 2.48005999e-05f);
    pc = fmaf(pc, s, -0.00138888881f);
    pc = fmaf(pc, s, 0.0416666679f);
    const float cr = fmaf(pc * s, s, fmaf(s, -0.5f, 1.0f));
    const float a = (q & 1) ? cr : sr;
    const float b = (q & 1) ? sr : cr;
    *sn = (q & 2) ? -a : a;
    *cs = ((q + 1) & 2) ? -b : b;
}
SRF_HD float srf_sinf(float x) { float s, c; srf_sincosf(x, &s, &c); return s; }
SRF_HD float srf_cosf(float x) { float s, c; srf_sincosf(x, &s, &c); return c; }

/* expf.  Overflows to +inf above 88.72, underflows to 0 below -104. */
SRF_HD float srf_expf(float x) {
    if (x != x) return x;
    if (x > 88.7228394f) return srf_u32_as_f32(0x7f800000u);
    if (x < -104.0f) return 0.0f;
    const float k = rintf(x * 1.44269502f);
    float r = fmaf(-k, 0.693115234f, x);
    r = fmaf(-k, 3.19461833e-05f, r);
    float p = 0.00019900444f;
    p = fmaf(p, r, 0.0013934545f);
    p = fmaf(p, r, 0.00833329745f);
    p = fmaf(p, r, 0.0416664556f);
    p = fmaf(p, r, 0.166666672f);
    p = fmaf(p, r, 0.5f);
    const float e = fmaf(p * r, r, r) + 1.0f;
    const int ki = srf_f2i_rz(k);
    const int k1 = ki >> 1, k2 = ki - k1;               /* both in [-76, 65] */
    const float s1 = srf_u32_as_f32((uint32_t)(k1 + 127) << 23);
    const float s2 = srf_u32_as_f32((uint32_t)(k2 + 127) << 23);
    return (e * s1) * s2;
}

/* logf for positive normal x. */
SRF_HD float srf_logf(float x) {
    const uint32_t ux = srf_f32_as_u32(x);
    const int32_t i = (int32_t)(ux - 0x3f3504f3u);
    const int32_t e = i >> 23;
    const float m = srf_u32_as_f32(ux - ((uint32_t)e << 23));   /* [sqrt(.5), sqrt(2)) */
    const float f = m - 1.0f;
    float p = -0.0810155869f;
    p = fmaf(p, f, 0.127123073f);
    p = fmaf(p, f, -0.129722387f);
    p = fmaf(p, f, 0.142021745f);
    p = fmaf(p, f, -0.166422471f);
    p = fmaf(p, f, 0.200014681f);
    p = fmaf(p, f, -0.25000298f);
    p = fmaf(p, f, 0.333333284f);
    const float f2 = f * f;
    const float r = fmaf(p * f, f2, fmaf(f2, -0.5f, f));
    return fmaf((float)e, 0.693147182f, r);
}

/*
 * SRF_CANON_CUDA_MATH (a test-only build of the kernels, never the shipped library): the canonical names map to the
 * CUDA math library's functions the reference calls -- atan2f, asinf, sinf, cosf, and the fast intrinsics __expf /
 * __logf -- so that, compiled with nvcc's default -fmad=true, the kernels compute what a CUDA build of the
 * reference's expressions computes.  The tests measure how far the shipped (canonical) results are from that.
 */
#if defined(SRF_CANON_CUDA_MATH) && defined(__CUDACC__)
static __host__ __device__ __forceinline__ float srf_cm_atan2f(float y, float x) { return atan2f(y, x); }
static __host__ __device__ __forceinline__ float srf_cm_asinf(float x) { return asinf(x); }
static __host__ __device__ __forceinline__ float srf_cm_sinf(float x) { return sinf(x); }
static __host__ __device__ __forceinline__ float srf_cm_cosf(float x) { return cosf(x); }
static __host__ __device__ __forceinline__ void srf_cm_sincosf(float x, float* s, float* c) { *s = sinf(x); *c = cosf(x); }
static __host__ __device__ __forceinline__ float srf_cm_expf(float x) {
#if defined(__CUDA_ARCH__) && !defined(SRF_CANON_CUDA_MATH_ACCURATE_EXP)
    return __expf(x);      /* the reference's choice; SRF_CANON_CUDA_MATH_ACCURATE_EXP swaps in expf to isolate its effect */
#else
    return expf(x);
#endif
}
static __host__ __device__ __forceinline__ float srf_cm_logf(float x) {
#if defined(__CUDA_ARCH__) && !defined(SRF_CANON_CUDA_MATH_ACCURATE_EXP)
    return __logf(x);
#else
    return logf(x);
#endif
}
#define srf_atan2f srf_cm_atan2f
#define srf_asinf srf_cm_asinf
#define srf_sinf srf_cm_sinf
#define srf_cosf srf_cm_cosf
#define srf_sincosf srf_cm_sincosf
#define srf_expf srf_cm_expf
#define srf_logf srf_cm_logf
#endif

#if defined(SRF_CANON_PLAIN)
/* the C library's functions under the canonical names (the definitions above stay compiled but unused) */
static inline float srf_plain_atan2f(float y, float x) { return atan2f(y, x); }
static inline float srf_plain_asinf(float x) { return asinf(x); }
static inline float srf_plain_sinf(float x) { return sinf(x); }
static inline float srf_plain_cosf(float x) { return cosf(x); }
static inline void srf_plain_sincosf(float x, float* s, float* c) { *s = sinf(x); *c = cosf(x); }
static inline float srf_plain_expf(float x) { return expf(x); }
static inline float srf_plain_logf(float x) { return logf(x); }
#define srf_atan2f srf_plain_atan2f
#define srf_asinf srf_plain_asinf
#define srf_sinf srf_plain_sinf
#define srf_cosf srf_plain_cosf
#define srf_sincosf srf_plain_sincosf
#define srf_expf srf_plain_expf
#define srf_logf srf_plain_logf
#endif

/* 1 / (1 + exp(-x)), the shape of tiny-cuda-nn's logistic(). */
SRF_HD float srf_logisticf(float x) { return 1.0f / (1.0f + srf_expf(-x)); }

/* Dot product of two 3-vectors the way Eigen reduces three terms, t0 + (t1 + t2), with both additions fused
 * into multiply-adds: fma(a0,b0, fma(a1,b1, a2*b2)).  The reference's dot(), norm(), normalized() and 3x3
 * matrix-vector products all reduce in this order (Eigen's unrolled scalar reduction splits [0,n) into
 * [0,n/2) and [n/2,n)). */
SRF_HD float srf_dot3f(float a0, float b0, float a1, float b1, float a2, float b2) {
    return fmaf(a0, b0, fmaf(a1, b1, a2 * b2));
}
/* Euclidean length: sqrt of the dot product above. */
SRF_HD float srf_norm3f(float x, float y, float z) {
    return sqrtf(srf_dot3f(x, x, y, y, z, z));
}

#endif /* SRF_CANON_MATH_H_ */

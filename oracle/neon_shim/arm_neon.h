/*
 * Minimal <arm_neon.h> stand-in for building the FastConv Winograd sources on an
 * x86_64 host.  TEST INFRASTRUCTURE ONLY: it exists so that the unmodified
 * reference translation units (winoF63ZC/winoF63ZC.cpp, winoF63ZC/TensorGEMMZC.cpp,
 * utility/helper.cpp, ...) can be compiled into the checker library under
 * oracle/_ref/.  Nothing shipped by the product includes this header.
 *
 * The types are GCC vector types so the reference's own `+ - *` operator
 * expressions compile unchanged and evaluate lane-wise in IEEE binary32.
 * vfmaq_f32 is one fused multiply-add per lane (fmaf), as on aarch64; every
 * other multiply/add stays unfused when the build passes -ffp-contract=off.
 */
#ifndef FASTCONV_ORACLE_NEON_SHIM_H_
#define FASTCONV_ORACLE_NEON_SHIM_H_

#include <math.h>
#include <string.h>

typedef float float32x4_t __attribute__((vector_size(16)));
typedef float float32x2_t __attribute__((vector_size(8)));
typedef struct { float32x4_t val[2]; } float32x4x2_t;

static inline float32x4_t vld1q_f32(const float *p) {
    float32x4_t v;
    memcpy(&v, p, sizeof v);
    return v;
}
static inline void vst1q_f32(float *p, float32x4_t v) { memcpy(p, &v, sizeof v); }
static inline void vst1_f32(float *p, float32x2_t v) { memcpy(p, &v, sizeof v); }
static inline float32x4_t vdupq_n_f32(float x) {
    float32x4_t v = {x, x, x, x};
    return v;
}
static inline float32x4_t vaddq_f32(float32x4_t a, float32x4_t b) { return a + b; }
static inline float32x4_t vsubq_f32(float32x4_t a, float32x4_t b) { return a - b; }
/* acc + a*b, fused, per lane */
static inline float32x4_t vfmaq_f32(float32x4_t acc, float32x4_t a, float32x4_t b) {
    float32x4_t r;
    for (int i = 0; i < 4; ++i) r[i] = fmaf(a[i], b[i], acc[i]);
    return r;
}
/* acc + a*b, two roundings, per lane */
static inline float32x4_t vmlaq_f32(float32x4_t acc, float32x4_t a, float32x4_t b) {
    return acc + a * b;
}
static inline float32x2_t vget_low_f32(float32x4_t v) {
    float32x2_t r = {v[0], v[1]};
    return r;
}
static inline float32x2_t vget_high_f32(float32x4_t v) {
    float32x2_t r = {v[2], v[3]};
    return r;
}
static inline float32x4_t vcombine_f32(float32x2_t lo, float32x2_t hi) {
    float32x4_t r = {lo[0], lo[1], hi[0], hi[1]};
    return r;
}
/* 2x2 transposes of (a,b): val[0] = (a0 b0 a2 b2), val[1] = (a1 b1 a3 b3) */
static inline float32x4x2_t vtrnq_f32(float32x4_t a, float32x4_t b) {
    float32x4x2_t r;
    float32x4_t e = {a[0], b[0], a[2], b[2]};
    float32x4_t o = {a[1], b[1], a[3], b[3]};
    r.val[0] = e;
    r.val[1] = o;
    return r;
}
static inline float32x4_t vmlaq_lane_f32(float32x4_t acc, float32x4_t a, float32x2_t b, const int lane) {
    return acc + a * vdupq_n_f32(b[lane]);
}
static inline float32x4_t vmlaq_laneq_f32(float32x4_t acc, float32x4_t a, float32x4_t b, const int lane) {
    return acc + a * vdupq_n_f32(b[lane]);
}
static inline float32x4_t vfmaq_laneq_f32(float32x4_t acc, float32x4_t a, float32x4_t b, const int lane) {
    return vfmaq_f32(acc, a, vdupq_n_f32(b[lane]));
}

#endif

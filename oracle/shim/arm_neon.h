/* Scalar/GCC-vector stand-in for the 13 NEON intrinsics full_trained_egg.c uses,
 * so that the reference's CPU functions compile unmodified on x86-64.
 * Test/baseline infrastructure only. */
#ifndef EGG_SHIM_ARM_NEON_H
#define EGG_SHIM_ARM_NEON_H
#include <stdint.h>
#include <string.h>
typedef int8_t   int8x16_t  __attribute__((vector_size(16)));
typedef int8_t   int8x8_t   __attribute__((vector_size(8)));
typedef uint8_t  uint8x16_t __attribute__((vector_size(16)));
typedef int16_t  int16x8_t  __attribute__((vector_size(16)));
typedef uint16_t uint16x8_t __attribute__((vector_size(16)));
typedef int32_t  int32x4_t  __attribute__((vector_size(16)));
typedef uint32_t uint32x4_t __attribute__((vector_size(16)));

static inline int32x4_t vdupq_n_s32(int32_t v) { return (int32x4_t){v, v, v, v}; }
static inline int8x16_t vld1q_s8(const int8_t *p) { int8x16_t r; memcpy(&r, p, 16); return r; }
static inline int8x8_t vget_low_s8(int8x16_t a) { int8x8_t r; memcpy(&r, &a, 8); return r; }
static inline int8x8_t vget_high_s8(int8x16_t a) { int8x8_t r; memcpy(&r, (const char *)&a + 8, 8); return r; }
static inline int16x8_t vmull_s8(int8x8_t a, int8x8_t b) {
    return __builtin_convertvector(a, int16x8_t) * __builtin_convertvector(b, int16x8_t);
}
static inline int32x4_t vpadalq_s16(int32x4_t acc, int16x8_t v) {
    for (int i = 0; i < 4; i++) acc[i] += (int32_t)v[2 * i] + (int32_t)v[2 * i + 1];
    return acc;
}
static inline int32_t vaddvq_s32(int32x4_t a) { return a[0] + a[1] + a[2] + a[3]; }
static inline int8x16_t vabsq_s8(int8x16_t a) {
    int8x16_t r; for (int i = 0; i < 16; i++) r[i] = (int8_t)(a[i] < 0 ? -a[i] : a[i]); return r;
}
static inline uint8x16_t vreinterpretq_u8_s8(int8x16_t a) { uint8x16_t r; memcpy(&r, &a, 16); return r; }
static inline int32x4_t vreinterpretq_s32_u32(uint32x4_t a) { int32x4_t r; memcpy(&r, &a, 16); return r; }
static inline uint16x8_t vpaddlq_u8(uint8x16_t a) {
    uint16x8_t r; for (int i = 0; i < 8; i++) r[i] = (uint16_t)((uint16_t)a[2 * i] + (uint16_t)a[2 * i + 1]); return r;
}
static inline uint32x4_t vpaddlq_u16(uint16x8_t a) {
    uint32x4_t r; for (int i = 0; i < 4; i++) r[i] = (uint32_t)a[2 * i] + (uint32_t)a[2 * i + 1]; return r;
}
static inline int32x4_t vaddq_s32(int32x4_t a, int32x4_t b) { return a + b; }
#endif

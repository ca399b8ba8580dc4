// mathx_dev.cuh — device restatement of the reference's scalar math
// (src/core/mathx.c:37-147, the WR_MATH_APPROX=1 bodies).
//
// RoPE parity is bit-for-bit, so every operation is a separately rounded
// IEEE multiply/add/divide (the __f*_rn intrinsics are never contracted
// into FMA) in the reference's evaluation order.  The reference's sin/cos
// are truncated Taylor series after a repeated +-2*pi reduction; they are
// reproduced as they are, including their error near +-pi, because the
// KV-cache bytes must equal the reference's.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "rope_reduce.h"

namespace wrmath {

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float dvd(float a, float b) { return __fdiv_rn(a, b); }

constexpr float kLn2 = 0.6931471805599453f;
constexpr float kPi = 3.14159265358979f;
constexpr float kTwoPi = 6.28318530717958f;

// src/core/mathx.c:37-57
__device__ inline float exp_ref(float x)
{
    if (x < -88.0f) return 0.0f;
    if (x > 88.0f) return 1e38f;
    int k = __float2int_rz(add(dvd(x, kLn2), (x >= 0.0f) ? 0.5f : -0.5f));
    float r = sub(x, mul((float)k, kLn2));
    float r2 = mul(r, r);
    float e = add(1.0f, r);
    e = add(e, mul(r2, 0.5f));
    e = add(e, mul(mul(r2, r), 1.0f / 6.0f));
    e = add(e, mul(mul(r2, r2), 1.0f / 24.0f));
    e = add(e, mul(mul(mul(r2, r2), r), 1.0f / 120.0f));
    if (k >= -126 && k <= 127) e = __uint_as_float(__float_as_uint(e) + ((uint32_t)k << 23));
    return e;
}

// src/core/mathx.c:72-86
__device__ inline float log_ref(float x)
{
    if (x <= 0.0f) return -1e38f;
    uint32_t u = __float_as_uint(x);
    int e = (int)((u >> 23) & 0xFFu) - 127;
    float m = __uint_as_float((u & 0x007FFFFFu) | 0x3F800000u);
    float t = dvd(sub(m, 1.0f), add(m, 1.0f));
    float t2 = mul(t, t);
    float s = add(1.0f / 5.0f, mul(t2, 1.0f / 7.0f));
    s = add(1.0f / 3.0f, mul(t2, s));
    s = add(1.0f, mul(t2, s));
    float lnm = mul(mul(2.0f, t), s);
    return add(lnm, mul((float)e, kLn2));
}

// src/core/mathx.c:98-110
__device__ inline float sqrt_ref(float x)
{
    if (x <= 0.0f) return 0.0f;
    float g = __uint_as_float((__float_as_uint(x) + 0x3f800000u) >> 1);
#pragma unroll
    for (int i = 0; i < 4; ++i) g = mul(0.5f, add(g, dvd(x, g)));
    return g;
}

// src/core/mathx.c:124-127: the reduction is a float loop whose rounding
// accumulates, so it is run as written (fmodf would not give the same bits).
//
// wr_reduce_pi (rope_reduce.h) returns the bits of that loop without running
// its thousands of dependent subtractions.
__device__ inline float reduce_pi(float x) { return wr_reduce_pi(x); }

// src/core/mathx.c:124-147 after reduction; both series share x2.
__device__ inline void sincos_ref(float angle, float &sn, float &cs)
{
    float x = reduce_pi(angle);
    float x2 = mul(x, x);
    float x3 = mul(x2, x);
    float x5 = mul(x3, x2);
    float x7 = mul(x5, x2);
    sn = sub(add(sub(x, mul(x3, 1.0f / 6.0f)), mul(x5, 1.0f / 120.0f)), mul(x7, 1.0f / 5040.0f));
    float x4 = mul(x2, x2);
    float x6 = mul(x4, x2);
    cs = sub(add(sub(1.0f, mul(x2, 0.5f)), mul(x4, 1.0f / 24.0f)), mul(x6, 1.0f / 720.0f));
}

// cos/sin of pair j at absolute position pos (src/core/kernels.c:1400-1405).
__device__ inline void rope_angle(uint32_t pos, uint32_t j, uint32_t hd, float ln_theta, float &sn,
                                  float &cs)
{
    float exponent = dvd((float)(2u * j), (float)hd);
    float powv = exp_ref(mul(exponent, ln_theta));
    float angle = dvd((float)pos, powv);
    sincos_ref(angle, sn, cs);
}

}  // namespace wrmath

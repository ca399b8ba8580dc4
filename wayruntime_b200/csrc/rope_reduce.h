// rope_reduce.h — the reference's sin/cos range reduction in closed form.
//
// The reference reduces an angle with `while (x > pi) x -= 2*pi` in float
// (src/core/mathx.c:124-127, :137-140).  Every subtraction rounds, the error
// accumulates, and the KV-cache bytes depend on the exact result, so the loop
// cannot be replaced by fmodf.  It can be replaced by integer arithmetic:
// while x stays inside one binade [2^e, 2^(e+1)), e >= 4, x is an integer
// multiple X of u = 2^(e-23) and the rounded subtraction lowers X by the same
// integer D_e every time (2*pi in float is C * 2^-21 with C odd, so C / 2^(e-2)
// is never a rounding tie for e >= 4).  So all the steps that stay in the
// binade collapse into one division; the step that leaves the binade is done
// as a real float subtraction, and below 16 the loop runs as written (at most
// three more steps).  Bit-identical to the loop for every finite x >= 0; the
// CPU test suite checks it against the loop over all positions in use.
//
// Plain C/C++ with no CUDA intrinsics on the host side, so that the same
// source is compiled by the host compiler for that test.
#pragma once

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define WR_HD __host__ __device__ __forceinline__
#else
#define WR_HD static inline
#endif

WR_HD uint32_t wr_f2u(float f)
{
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
#endif
}
WR_HD float wr_u2f(uint32_t u)
{
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f;
    memcpy(&f, &u, 4);
    return f;
#endif
}
WR_HD float wr_fsub(float a, float b)
{
#if defined(__CUDA_ARCH__)
    return __fsub_rn(a, b);
#else
    return a - b;
#endif
}
WR_HD float wr_fadd(float a, float b)
{
#if defined(__CUDA_ARCH__)
    return __fadd_rn(a, b);
#else
    return a + b;
#endif
}

// Result of `while (x > pi) x -= 2pi; while (x < -pi) x += 2pi;` in float.
WR_HD float wr_reduce_pi(float x)
{
    const float kPi = 3.14159265358979f, kTwoPi = 6.28318530717958f;
    const uint32_t kC = 13176795u;           // significand of kTwoPi: kTwoPi = kC * 2^-21
    while (x >= 16.0f) {
        const uint32_t bits = wr_f2u(x);
        const uint32_t e = (bits >> 23) - 127u;            // >= 4
        const uint32_t k = e - 2u;
        if (k < 24u) {
            const uint32_t q = kC >> k, r = kC & ((1u << k) - 1u);
            const uint32_t d = q + ((r > (1u << (k - 1u))) ? 1u : 0u);
            if (d == 0u) break;                            // 2pi below half an ulp: x no longer moves
            uint32_t X = (bits & 0x007FFFFFu) | 0x00800000u;
            // steps whose exact difference stays inside this binade
            const uint32_t n = (X > 0x00800000u) ? (X - 0x00800001u) / d : 0u;
            X -= n * d;
            x = wr_u2f((bits & 0xFF800000u) | (X & 0x007FFFFFu));
        } else {
            break;
        }
        x = wr_fsub(x, kTwoPi);                            // the step that may leave the binade
    }
    while (x > kPi) {
        const float y = wr_fsub(x, kTwoPi);
        if (y == x) break;                                 // (x stuck: the reference would spin forever)
        x = y;
    }
    while (x < -kPi) x = wr_fadd(x, kTwoPi);
    return x;
}

/* Host check of the closed-form range reduction (wayruntime_b200/csrc/rope_reduce.h)
 * against the float loop it replaces (src/core/mathx.c:124-127 in the reference).
 * Built and run by tests/test_rope_reduce.py; prints the number of mismatches. */
#include <stdio.h>
#include <stdint.h>
#include <string.h>

#include "rope_reduce.h"
#include "wr_oracle.h"

static float loop_reduce(float x)
{
    const float pi = 3.14159265358979f, two_pi = 6.28318530717958f;
    while (x > pi) x -= two_pi;
    while (x < -pi) x += two_pi;
    return x;
}

static uint32_t bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

int main(void)
{
    unsigned long long checked = 0, bad = 0;
    /* 1. every RoPE angle of the positions in use: theta in {1e4, 5e5, 1e6}, hd 128 and 64 */
    const float thetas[3] = { 10000.0f, 500000.0f, 1000000.0f };
    const uint32_t hds[2] = { 128, 64 };
    for (int ti = 0; ti < 3; ti++) {
        float lnb = wro_log(thetas[ti]);
        for (int hi = 0; hi < 2; hi++) {
            uint32_t hd = hds[hi];
            for (uint32_t j = 0; j < hd / 2; j++) {
                float powv = wro_exp(((float)(2 * j) / (float)hd) * lnb);
                for (uint32_t pos = 0; pos < 40000; pos++) {
                    float a = (float)pos / powv;
                    if (bits(loop_reduce(a)) != bits(wr_reduce_pi(a))) bad++;
                    checked++;
                }
            }
        }
    }
    /* 2. a stride through every float in [3, 2^18) */
    for (uint32_t u = bits(3.0f); u < bits(262144.0f); u += 2039) {
        float x; memcpy(&x, &u, 4);
        if (bits(loop_reduce(x)) != bits(wr_reduce_pi(x))) bad++;
        checked++;
    }
    /* 3. binade edges */
    for (int e = 2; e < 20; e++)
        for (int d = -40; d <= 40; d++) {
            uint32_t u = bits((float)(1u << e)) + (uint32_t)d;
            float x; memcpy(&x, &u, 4);
            if (bits(loop_reduce(x)) != bits(wr_reduce_pi(x))) bad++;
            checked++;
        }
    printf("checked %llu mismatches %llu\n", checked, bad);
    return bad ? 1 : 0;
}

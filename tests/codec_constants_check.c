/* Exhaustive check of the two identities the kernels' per-block constants rest on (csrc/common.cuh):
 *   RN(d / 15)  ==  q + RN((d - 15 q) * c)   with c = RN(1/15), q = RN(d * c)         for 2^-100 <= d <= 2^100
 *   RN(1 / u)   ==  two Newton steps from any start within 3 ulp of it                 for 2^-100 <= u <= 2^100,
 *                   except where the mantissa bits of u are all ones
 * over every float of the range (1.68e9 values).  Prints the numbers of mismatches; exit status 0 when there are none.
 * Build: gcc -O2 -march=native (hardware FMA makes it fast; fmaf is exact either way). */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

int main(void) {
    const float c = 1.0f / 15.0f;
    const uint32_t lo = f2u(ldexpf(1.0f, -100)), hi = f2u(ldexpf(1.0f, 100));
    unsigned long long bad_div = 0, bad_rcp = 0, bad_rcp_ones = 0;
    for (uint32_t b = lo; b <= hi; ++b) {
        const float x = u2f(b);
        const float q = x * c;
        if (fmaf(fmaf(-15.0f, q, x), c, q) != x / 15.0f) ++bad_div;
        const float rr = 1.0f / x;
        for (int k = -3; k <= 3; ++k) {
            float y = u2f(f2u(rr) + k);
            float e = fmaf(-x, y, 1.0f);
            y = fmaf(y, e, y);
            e = fmaf(-x, y, 1.0f);
            y = fmaf(y, e, y);
            if (y != rr) { if ((b & 0x7FFFFFu) == 0x7FFFFFu) ++bad_rcp_ones; else ++bad_rcp; }
        }
    }
    printf("div15 mismatches %llu, reciprocal mismatches %llu (mantissa of all ones: %llu)\n", bad_div, bad_rcp, bad_rcp_ones);
    return (bad_div == 0 && bad_rcp == 0) ? 0 : 1;
}

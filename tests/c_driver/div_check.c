/* Checks the three-operation division by a constant that the attention kernels use for scores / sqrtf(head_dim)
 * (div_by_const in csrc/mma_common.cuh: y = x * rc; q = fma(fma(-y, c, x), rc, y) with rc = 1.0f / c) against IEEE
 * division, bit for bit, over the floats x = bits(first + k * stride) with 1e-30 < |x| < 1e30 (outside that range
 * the kernels divide).  Usage: div_check <stride> ; stride 1 is every float (about a minute on a few cores).
 * Prints the number of mismatches per constant; exit code 1 if any. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

int main(int argc, char **argv) {
    const long long stride = argc > 1 ? atoll(argv[1]) : 61;
    const float cs[4] = {sqrtf(32.0f), sqrtf(64.0f), sqrtf(96.0f), sqrtf(128.0f)};
    int fail = 0;
    for (int ci = 0; ci < 4; ++ci) {
        const float c = cs[ci], rc = 1.0f / c;
        long long bad = 0, seen = 0;
        for (long long u = ci; u < (1ll << 32); u += stride) {
            const uint32_t b = (uint32_t)u;
            float x;
            memcpy(&x, &b, 4);
            const float ax = fabsf(x);
            if (!(ax > 1e-30f && ax < 1e30f)) continue;
            const float want = x / c;
            const float y = x * rc;
            const float got = fmaf(fmaf(-y, c, x), rc, y);
            ++seen;
            if (memcmp(&want, &got, 4) != 0) ++bad;
        }
        printf("c = sqrtf(%d): %lld values, %lld mismatches\n", (int)lrintf(c * c), seen, bad);
        if (bad) fail = 1;
    }
    return fail;
}

// Exhaustive check of the packers' division for 16-bit weights (BlockDivider in
// metalops_b200/csrc/q4b_quantize.cu): for EVERY scale d (1e-30 <= d <= 1e30) and value v (|v| <= 16.5 d)
// of fp16, or of bf16 when an argument is given, the 4-bit code that the reference's pipeline
// (packages/metalcore/src/metalcore/quantization.py:341-350: w / d, + 8, round, clamp, each op rounded to
// the weight's dtype) gives through IEEE division equals the one through v * r corrected once by fma,
// r the correctly rounded reciprocal of d.  Exit status 0 when no pair differs.
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
static float h2f(uint16_t h) {
    uint32_t s = (h >> 15) & 1, e = (h >> 10) & 31, m = h & 1023, u;
    if (e == 0) { if (m == 0) u = s << 31; else { int k = 0; while (!(m & 1024)) { m <<= 1; ++k; } m &= 1023; u = (s << 31) | ((uint32_t)(113 - k) << 23) | (m << 13); } }
    else if (e == 31) u = (s << 31) | 0x7F800000u | (m << 13);
    else u = (s << 31) | ((e + 112) << 23) | (m << 13);
    float f; memcpy(&f, &u, 4); return f;
}
static float b2f(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }
static uint16_t f2h(float f) {   // round to nearest even, fp16 (no NaN/inf inputs here)
    uint32_t u; memcpy(&u, &f, 4);
    uint32_t s = (u >> 16) & 0x8000; int e = (int)((u >> 23) & 255) - 127 + 15; uint32_t m = u & 0x7FFFFF;
    if (e >= 31) return (uint16_t)(s | 0x7C00);
    if (e <= 0) { if (e < -10) return (uint16_t)s; m |= 0x800000; int sh = 14 - e; uint32_t r = m >> sh, rem = m & ((1u << sh) - 1), half = 1u << (sh - 1);
        if (rem > half || (rem == half && (r & 1))) ++r; return (uint16_t)(s | r); }
    uint32_t r = (uint32_t)e << 10 | (m >> 13), rem = m & 0x1FFF;
    if (rem > 0x1000 || (rem == 0x1000 && (r & 1))) ++r; return (uint16_t)(s | r);
}
static uint16_t f2b(float f) { uint32_t u; memcpy(&u, &f, 4); uint32_t r = u >> 16, rem = u & 0xFFFF; if (rem > 0x8000 || (rem == 0x8000 && (r & 1))) ++r; return (uint16_t)r; }
static int nib(float t, int bf) {
    t = bf ? b2f(f2b(t)) : h2f(f2h(t));
    t = t + 8.0f;
    t = bf ? b2f(f2b(t)) : h2f(f2h(t));
    float r = nearbyintf(t);
    if (r < 0) r = 0; if (r > 15) r = 15;
    return (int)r;
}
int main(int argc, char **argv) {
    int bf = argc > 1;
    long bad = 0, n = 0;
    for (uint32_t di = 1; di < 0x8000; ++di) {
        float d = bf ? b2f((uint16_t)di) : h2f((uint16_t)di);
        if (!(d > 0) || isinf(d) || isnan(d)) continue;
        if (d < 1e-30f || d > 1e30f) continue;
        float r = 1.0f / d;
        for (uint32_t vi = 0; vi < 0x10000; ++vi) {
            float v = bf ? b2f((uint16_t)vi) : h2f((uint16_t)vi);
            if (isnan(v) || isinf(v)) continue;
            if (fabsf(v) > 16.5f * d) continue;         // |v| <= amax, d = RN(amax / 7), denormal d included
            float q = v * r;
            float e = fmaf(-q, d, v);
            float q1 = fmaf(e, r, q);
            float ref = v / d;
            ++n;
            /* equal quotients need no second look */
            if (memcmp(&q1, &ref, 4) != 0 && nib(q1, bf) != nib(ref, bf)) { if (bad < 5) printf("mismatch v=%a d=%a fast=%a ref=%a\n", v, d, q1, ref); ++bad; }
        }
    }
    printf("%s: %ld pairs, %ld mismatches\n", bf ? "bf16" : "fp16", n, bad);
    return bad != 0;
}

/* CPU twin of the device exp (trs_exp in pytorch-rs_b200/csrc/pointwise_plan.cpp), same operations in the same
 * order with the C library's fmaf, swept against glibc's expf -- the function the reference calls
 * (pytorch-rs src/tensor.rs:2398-2400 -> f32::exp -> libm expf).  Test infrastructure only.
 *
 *   exp_sweep <stride>     checks every <stride>-th float32 bit pattern in [-104.5, 89.5]; stride 1 = all 2.2e9
 *
 * Prints "max_ulp <d> equal <n> off_by_one <n> worse <n>" and the constants it used. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

static inline float as_float(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static inline uint32_t as_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

#define LOG2E 1.44269502f
#define MAGIC 12582912.0f
#define LN2_HI (-0.693145752f)
#define LN2_LO (-1.42860677e-06f)
static const uint32_t COEFF[4] = {0x3ab6da3fu, 0x3c091dc9u, 0x3d2aaa2fu, 0x3e2aaa47u};

static float polynomial(float r) {
    float q = as_float(COEFF[0]);
    q = fmaf(q, r, as_float(COEFF[1]));
    q = fmaf(q, r, as_float(COEFF[2]));
    q = fmaf(q, r, as_float(COEFF[3]));
    q = fmaf(q, r, 0.5f);
    q = fmaf(q, r, 1.0f);
    return fmaf(q, r, 1.0f);
}

static float exp_slow(float x) {
    const float t = x < -110.0f ? -110.0f : (x > 90.0f ? 90.0f : x);
    const float j = fmaf(t, LOG2E, MAGIC) - MAGIC;
    float r = fmaf(j, LN2_HI, t);
    r = fmaf(j, LN2_LO, r);
    const float p = polynomial(r);
    const int ji = isnan(j) ? 0 : (int)j;          /* the device conversion gives 0 for NaN */
    const int h = ji >> 1;
    const float s1 = as_float((uint32_t)(h + 127) << 23), s2 = as_float((uint32_t)(ji - h + 127) << 23);
    return (p * s1) * s2;
}

static float exp_twin(float x) {
    if (!(fabsf(x) <= 87.0f)) return exp_slow(x);
    const float m = fmaf(x, LOG2E, MAGIC);
    const float j = m - MAGIC;
    float r = fmaf(j, LN2_HI, x);
    r = fmaf(j, LN2_LO, r);
    return as_float(as_bits(polynomial(r)) + (as_bits(m) << 23));
}

static long long ulp_distance(float a, float b) {
    int32_t ia = (int32_t)as_bits(a), ib = (int32_t)as_bits(b);
    if (ia < 0) ia = (int32_t)0x80000000 - ia;
    if (ib < 0) ib = (int32_t)0x80000000 - ib;
    long long d = (long long)ia - ib;
    return d < 0 ? -d : d;
}

/* The twin over an array, for the GPU test that compares the device function with it bit for bit. */
void exp_twin_array(const float* x, float* y, long long n) {
    for (long long i = 0; i < n; ++i) y[i] = exp_twin(x[i]);
}

int main(int argc, char** argv) {
    const uint32_t stride = argc > 1 ? (uint32_t)strtoul(argv[1], 0, 10) : 64;
    const uint32_t ranges[2][2] = {{0u, as_bits(89.5f)}, {0x80000000u, as_bits(-104.5f)}};
    long long max_d = 0, count[3] = {0, 0, 0};
    for (int s = 0; s < 2; ++s)
        for (uint64_t u = ranges[s][0]; u <= ranges[s][1]; u += stride ? stride : 1) {
            const float x = as_float((uint32_t)u);
            const long long d = ulp_distance(expf(x), exp_twin(x));
            if (d > max_d) max_d = d;
            count[d > 2 ? 2 : d] += 1;
        }
    const float specials[] = {0.0f, -0.0f, 1e-45f, -1e-45f, INFINITY, -INFINITY, 89.0f, -104.0f, 88.72283f, -103.972f};
    int specials_ok = 1;
    for (unsigned i = 0; i < sizeof specials / sizeof specials[0]; ++i)
        specials_ok &= as_bits(expf(specials[i])) == as_bits(exp_twin(specials[i]));
    specials_ok &= isnan(exp_twin(NAN)) != 0;
    printf("max_ulp %lld equal %lld off_by_one %lld worse %lld specials_ok %d\n", max_d, count[0], count[1], count[2], specials_ok);
    printf("constants %a %a %a %a 0x%08x 0x%08x 0x%08x 0x%08x\n", (double)LOG2E, (double)MAGIC, (double)LN2_HI, (double)LN2_LO,
           COEFF[0], COEFF[1], COEFF[2], COEFF[3]);
    return 0;
}

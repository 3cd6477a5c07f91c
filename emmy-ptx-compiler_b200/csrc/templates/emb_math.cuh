// Single-precision exp, log and tanh for sm_100a kernels, built from the SFU's ex2/lg2
// approximations and FMA polynomials.
//
// They take the place of the reference's PTX routines (emmy_ptx/mathlib.py:92-209: exp and
// tanh measured at <= 2 ulp, log at <= 1 ulp) and keep the same accuracy class; the
// polynomials were fitted for this file (least squares at Chebyshev nodes, coefficients
// rounded to float) and are evaluated with FMAs.
#pragma once

namespace emb {

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float ex2_approx_ftz(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// e^x = 2^j * 2^f, j = round(x * log2 e) clamped so that 2^j is a normal number, and
// f = x * log2 e - j from two FMAs against log2 e split in two floats, so f carries almost no
// rounding error even near |x| = 88. 2^f comes from the SFU on a small argument (where its
// absolute error is smallest); outside the clamp f simply grows and the SFU saturates to
// 0 or inf, and the last multiply rounds into the subnormal range.
__device__ __forceinline__ float exp_f32(float x) {
    const float log2e_hi = 1.44269502162933349609375f;  // float(log2 e)
    const float log2e_lo = 1.925963033500011e-08f;      // log2 e - log2e_hi
    float j = rintf(x * log2e_hi);
    j = fminf(fmaxf(j, -126.0f), 126.0f);
    float f = fmaf(x, log2e_hi, -j);
    f = fmaf(x, log2e_lo, f);
    float p = ex2_approx(f);
    float scale = __int_as_float((static_cast<int>(j) + 127) << 23);
    return p * scale;  // a NaN reaches the result through f (the clamp drops it from j only)
}

// 2^f for |f| <= 1/2 on the FMA pipe alone (no SFU): degree-6 polynomial, < 1 ulp. For kernels
// whose exponentials would otherwise saturate the SFU (16 results per clock per SM).
__device__ __forceinline__ float ex2_poly(float f) {
    float p = 0.00015469732170458883f;
    p = fmaf(p, f, 0.0013400432653725147f);
    p = fmaf(p, f, 0.00961802527308464f);
    p = fmaf(p, f, 0.05550327152013779f);
    p = fmaf(p, f, 0.24022650718688965f);
    p = fmaf(p, f, 0.6931471824645996f);
    return fmaf(p, f, 1.0f);
}

// 2^t for t <= 0 (softmax weights), all on the FMA/ALU pipes: split t = j + f with
// |f| <= 1/2, polynomial for 2^f, exponent-field add for 2^j. Results below 2^-125 flush to 0.
__device__ __forceinline__ float ex2_neg_fma(float t) {
    float tc = fmaxf(t, -125.0f);  // keeps the exponent field positive
    float j = rintf(tc);
    float f = tc - j;
    float p = ex2_poly(f);
    float r = __int_as_float(__float_as_int(p) + (static_cast<int>(j) << 23));
    return t < -125.0f ? 0.0f : r;
}

// ---- two floats at a time (sm_100 has packed f32x2 FMA and ADD: half the issue slots) ----

__device__ __forceinline__ unsigned long long pack_f2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_f2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long add_f2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// 2^t for two values t <= ~8 on the FMA and integer pipes only: round t to an integer with the
// magic-number add, cubic for 2^f on |f| <= 1/2 (2.1e-4 relative, finer than the f16 the softmax
// weights are rounded to), exponent-field add. For kernels whose exponentials saturate the SFU.
__device__ __forceinline__ void ex2_poly3_pair(float t0, float t1, float& p0, float& p1) {
    const float magic = 12582912.0f;  // 1.5 * 2^23: adding it leaves round(t) in the low mantissa bits
    t0 = fmaxf(t0, -125.0f);
    t1 = fmaxf(t1, -125.0f);
    const unsigned long long t = pack_f2(t0, t1);
    const unsigned long long one = pack_f2(1.0f, 1.0f);
    const unsigned long long shifted = add_f2(t, pack_f2(magic, magic));
    const unsigned long long j = add_f2(shifted, pack_f2(-magic, -magic));
    const unsigned long long f = fma_f2(j, pack_f2(-1.0f, -1.0f), t);
    // 2^f = 1 + f (c1 + f (c2 + f c3)): exact at f = 0, so a weight of 2^0 is exactly 1
    unsigned long long p = fma_f2(pack_f2(0.055838342756032944f, 0.055838342756032944f), f,
                                  pack_f2(0.24203594028949738f, 0.24203594028949738f));
    p = fma_f2(p, f, pack_f2(0.6931367516517639f, 0.6931367516517639f));
    p = fma_f2(p, f, one);
    float s0, s1, q0, q1;
    unpack_f2(shifted, s0, s1);
    unpack_f2(p, q0, q1);
    p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(s0) << 23));
    p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(s1) << 23));
}

// tanh: below 0.6 an odd polynomial x + x^3 P(x^2) (0.75 ulp in the fit's float emulation);
// above, 1 - 2 / (e^(2|x|) + 1) with x's sign.
__device__ __forceinline__ float tanh_f32(float x) {
    float a = fabsf(x);
    float s = x * x;
    float p = 0.002373300027102232f;
    p = fmaf(p, s, -0.00841234065592289f);
    p = fmaf(p, s, 0.021789031103253365f);
    p = fmaf(p, s, -0.05396164208650589f);
    p = fmaf(p, s, 0.13333313167095184f);
    p = fmaf(p, s, -0.3333333432674408f);
    float small = fmaf(x * s, p, x);
    float e = exp_f32(a + a);
    float big = copysignf(1.0f - 2.0f * __frcp_rn(e + 1.0f), x);
    float r = copysignf(a < 0.6f ? fabsf(small) : fabsf(big), x);  // tanh is odd: tanh(-0) = -0
    return x == x ? r : x;
}

// log: x = m * 2^e with m in [sqrt(1/2), sqrt(2)); log x = e ln2 + log1p(m - 1), the latter
// f + f^2 P(f) (0.82 ulp in the fit's float emulation); ln2 split so that e * ln2_hi is exact.
__device__ __forceinline__ float log_f32(float x) {
    if (!(x > 0.0f)) return x == 0.0f ? -__int_as_float(0x7f800000) : (x != x ? x : __int_as_float(0x7fc00000));
    if (x == __int_as_float(0x7f800000)) return x;
    float bias = 0.0f;
    if (x < 1.1754943508222875e-38f) {  // subnormal: scale into the normal range
        x *= 8388608.0f;
        bias = -23.0f;
    }
    int i = __float_as_int(x) - 0x3f3504f3;  // bits of sqrt(1/2)
    int e = i >> 23;
    float m = __int_as_float((i & 0x007fffff) + 0x3f3504f3);
    float f = m - 1.0f;
    float p = -0.07866667956113815f;
    p = fmaf(p, f, 0.12821748852729797f);
    p = fmaf(p, f, -0.131016343832016f);
    p = fmaf(p, f, 0.1418900042772293f);
    p = fmaf(p, f, -0.1662759929895401f);
    p = fmaf(p, f, 0.2000196874141693f);
    p = fmaf(p, f, -0.2500077188014984f);
    p = fmaf(p, f, 0.33333322405815125f);
    p = fmaf(p, f, -0.4999999701976776f);
    float ef = static_cast<float>(e) + bias;
    float r = fmaf(f * f, p, f);
    r = fmaf(ef, 1.4286067653e-06f, r);  // ln2 - ln2_hi
    return fmaf(ef, 0.693145751953125f, r);  // ln2_hi: 15 significant bits
}

// tanh-form GELU, 0.5 x (1 + tanh(c (x + k x^3))), with the SFU's tanh.approx: about 2^-11
// relative error, for epilogues whose output is bf16 or narrower.
__device__ __forceinline__ float gelu_tanh_fast(float x) {
    float u = 0.7978845608028654f * fmaf(0.044715f * x * x, x, x);
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
    float hx = 0.5f * x;
    return fmaf(hx, t, hx);
}

}  // namespace emb

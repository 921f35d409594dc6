// Arithmetic shared by the attention forward kernels.
#pragma once
#include <cuda_runtime.h>

namespace gm {

constexpr int POLY_PER_8 = 2;     // of every 8 exponentials, how many run on the FMA pipe instead of MUFU

// 2^x for x <= 0 on the FMA pipe: split x into integer and fraction, cubic minimax polynomial for 2^frac (max relative
// error about 1e-4, below bf16 resolution), exponent added through the float's bit pattern.  The MUFU unit evaluates
// only 16 exponentials per clock per SM and also executes the float -> bf16 conversions; evaluating a part of every row
// here takes that much off its pipe.  Measured on the 16 x 2048 x 12 x 64 window-1024 case: 0, 1 and 2 of 8 give the same
// time, 3 of 8 is 6 % slower and 4 of 8 10 % slower (the polynomial costs nine instructions, and the softmax warps are short
// of issue slots before they are short of MUFU throughput).
__device__ __forceinline__ float exp2_poly(float x) {
    x = fmaxf(x, -125.f);
    const float shifted = x + 12582912.f;                       // 1.5 * 2^23: the integer part lands in the low mantissa bits
    const float xi = shifted - 12582912.f;
    const float f = x - xi;                                     // f in [-0.5, 0.5]
    float pl = fmaf(f, 0.0555041086f, 0.2402265069f);
    pl = fmaf(pl, f, 0.6931471806f);
    pl = fmaf(pl, f, 1.0f);
    return __int_as_float(__float_as_int(pl) + (__float_as_int(shifted) << 23));
}

// ---- packed fp32 pairs (sm_100 add / mul / fma .f32x2): one instruction for two scores -----------------------------------------
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
// exp2_poly on a pair: the clamp and the exponent insertion stay per element, the five float operations are packed
__device__ __forceinline__ uint64_t exp2_poly2(uint64_t x2) {
    float x0, x1;
    unpack2(x2, x0, x1);
    x2 = pack2(fmaxf(x0, -125.f), fmaxf(x1, -125.f));
    const uint64_t shifted = add2(x2, pack2(12582912.f, 12582912.f));
    const uint64_t xi = add2(shifted, pack2(-12582912.f, -12582912.f));
    const uint64_t f = fma2(xi, pack2(-1.f, -1.f), x2);
    uint64_t pl = fma2(f, pack2(0.0555041086f, 0.0555041086f), pack2(0.2402265069f, 0.2402265069f));
    pl = fma2(pl, f, pack2(0.6931471806f, 0.6931471806f));
    pl = fma2(pl, f, pack2(1.0f, 1.0f));
    float p0, p1, s0, s1;
    unpack2(pl, p0, p1);
    unpack2(shifted, s0, s1);
    return pack2(__int_as_float(__float_as_int(p0) + (__float_as_int(s0) << 23)), __int_as_float(__float_as_int(p1) + (__float_as_int(s1) << 23)));
}

__device__ __forceinline__ float tanh_approx(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace gm

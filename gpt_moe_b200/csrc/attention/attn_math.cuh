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

__device__ __forceinline__ float tanh_approx(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace gm

// MXFP8 quantisation pieces shared by the stand-alone quantisers (gemm/gemm_mxfp8.cu) and by the producer kernels that
// emit a quantised copy next to their bf16 output (fused/*.cu, attention/*.cu).
//
// Format: e4m3 payload, one UE8M0 (power-of-two) scale per 32 consecutive elements of the contraction dimension.
//   scale   = smallest power of two >= amax / 448, taken by integer rounding of the fp32 bit pattern
//             (reference model/linear/fp8/custom/quantization.py:5-13), exponent byte 127 (scale 1) for an all-zero block
//   payload = round-to-nearest-even, saturating, of value / scale
// Scales are stored as 512-byte records, one per (128-row block, 128-wide K block): the byte of (row r, k-group g) of a
// record sits at (r % 32) * 16 + (r / 32) * 4 + g, which is the shared-memory image `tcgen05.cp 32x128b.warpx4` expects,
// so the GEMM moves a record global -> shared -> TMEM without touching it.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace gm {

constexpr int SF_RECORD_BYTES = 512;

__device__ __forceinline__ uint32_t e8m0_from_amax(float amax) {
    if (amax == 0.f) return 127u;
    uint32_t bits = __float_as_uint(amax * (1.f / 448.f));
    bits = (bits + 0x007FFFFFu) & 0x7F800000u;
    uint32_t e = bits >> 23;
    return e < 1u ? 1u : (e > 254u ? 254u : e);
}
__device__ __forceinline__ float inv_scale_from_e8m0(uint32_t e) { return __uint_as_float((254u - e) << 23); }

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(a), "f"(b));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(c), "f"(d));
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// byte offset of the scale of (row, k_group) in a scale array whose rows are `k_blocks` 128-wide K blocks long
__device__ __forceinline__ long long sf_offset(long long row, int k_group, int k_blocks) {
    const long long rb = row >> 7;
    const int r = static_cast<int>(row & 127);
    return (rb * k_blocks + (k_group >> 2)) * SF_RECORD_BYTES + (r & 31) * 16 + (r >> 5) * 4 + (k_group & 3);
}

// A 32-element block spread over `LANES_PER_BLOCK` adjacent lanes (aligned to that count), each holding N consecutive values
// (LANES_PER_BLOCK * N == 32).  Every lane of the warp must call this (the amax travels by full-warp shuffles); lanes whose
// values are not to be stored pass zeros and ignore the result.  Returns this lane's N payload bytes packed little-endian
// in `out` (N / 4 words) and the block's exponent byte.
template <int N>
__device__ __forceinline__ uint32_t quantize_block_lanes(const float (&v)[N], uint32_t (&out)[N / 4]) {
    static_assert(N == 4 || N == 8 || N == 16 || N == 32, "values per lane");
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < N; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 1; o < 32 / N; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const uint32_t e8 = e8m0_from_amax(amax);
    const float inv = inv_scale_from_e8m0(e8);
#pragma unroll
    for (int i = 0; i < N / 4; ++i) out[i] = pack_e4m3x4(v[4 * i] * inv, v[4 * i + 1] * inv, v[4 * i + 2] * inv, v[4 * i + 3] * inv);
    return e8;
}

// values as the bf16 tensor next to the quantised copy holds them (the quantised copy equals quantise(bf16 output) bit for bit)
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

}  // namespace gm

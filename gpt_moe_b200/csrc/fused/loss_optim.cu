// Streaming fp32 cross-entropy over bf16 logits (forward + in-place gradient), AdamW, and the element-wise
// parts of Muon (momentum / Nesterov / bf16 pack, and the scaled weight update).
//
// Reference counterparts: `model/cross_entropy.py:12-69` (online-softmax CE, fp32 statistics, int64 row
// offsets), `model/loss.py:11-60` (gradients computed during the forward pass),
// `optimizers/polar_prepare.py:8-35` (momentum + Nesterov + bf16 pack), `optimizers/polar_express.py:325-377`
// (final update into fp32 master weights), torch's fused AdamW (`model/gpt.py:284-293`).
#include "../common/ptx.cuh"
#include "../kernels_decl.h"
#include <algorithm>

namespace gm {

// 2^x on the special-function unit (the softmax needs no more than its 2-ulp accuracy)
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// One block per row.  loss[row] = logsumexp(logits) - logits[target]; logits are overwritten by
// (softmax - onehot) * (*grad_scale) in bf16, zeros for ignored rows.  64-bit row offsets.
__global__ void __launch_bounds__(512)
ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets, float* __restrict__ loss,
                  const float* __restrict__ grad_scale, int vocab, long long row_stride, long long ignore_index, int write_grad) {
    __shared__ float red_m[16], red_s[16];
    const long long row = blockIdx.x;
    __nv_bfloat16* p = logits + row * row_stride;
    long long tgt = targets[row];
    if (!GM_IN_BOUNDS(tgt == ignore_index || (tgt >= 0 && tgt < vocab), 905)) tgt = ignore_index;      // checked build: the row is ignored
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int vec = vocab / 8;
    if (tgt == ignore_index) {
        if (threadIdx.x == 0) loss[row] = 0.f;
        if (write_grad) {
            for (int i = threadIdx.x; i < vec; i += blockDim.x) reinterpret_cast<uint4*>(p)[i] = make_uint4(0, 0, 0, 0);
            for (int i = vec * 8 + threadIdx.x; i < vocab; i += blockDim.x) p[i] = __float2bfloat16(0.f);
        }
        return;
    }
    float m = -INFINITY, s = 0.f;
    auto push = [&](float v) {
        if (v > m) { s = s * __expf(m - v) + 1.f; m = v; } else { s += __expf(v - m); }
    };
    for (int i = threadIdx.x; i < vec; i += blockDim.x) {
        const uint4 raw = reinterpret_cast<const uint4*>(p)[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h[e]); push(f.x); push(f.y); }
    }
    for (int i = vec * 8 + threadIdx.x; i < vocab; i += blockDim.x) push(__bfloat162float(p[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
        const float mm = fmaxf(m, m2);
        s = (m == -INFINITY ? 0.f : s * __expf(m - mm)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mm));
        m = mm;
    }
    if (lane == 0) { red_m[warp] = m; red_s[warp] = s; }
    __syncthreads();
    float gm_ = red_m[0], gs = red_s[0];
    for (int w = 1; w < nwarps; ++w) {
        const float mm = fmaxf(gm_, red_m[w]);
        gs = (gm_ == -INFINITY ? 0.f : gs * __expf(gm_ - mm)) + (red_m[w] == -INFINITY ? 0.f : red_s[w] * __expf(red_m[w] - mm));
        gm_ = mm;
    }
    const float lse = gm_ + __logf(gs);
    if (threadIdx.x == 0) loss[row] = lse - __bfloat162float(p[tgt]);
    if (!write_grad) return;
    __syncthreads();     // every thread has read what it needs of the row before it is overwritten
    const float scale = *grad_scale;
    for (int i = threadIdx.x; i < vec; i += blockDim.x) {
        uint4 raw = reinterpret_cast<const uint4*>(p)[i];
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
        uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            const int c = i * 8 + 2 * e;
            const float g0 = (__expf(f.x - lse) - (c == tgt ? 1.f : 0.f)) * scale;
            const float g1 = (__expf(f.y - lse) - (c + 1 == tgt ? 1.f : 0.f)) * scale;
            w[e] = pack_bf16x2(g0, g1);
        }
        reinterpret_cast<uint4*>(p)[i] = raw;
    }
    for (int i = vec * 8 + threadIdx.x; i < vocab; i += blockDim.x)
        p[i] = __float2bfloat16((__expf(__bfloat162float(p[i]) - lse) - (i == tgt ? 1.f : 0.f)) * scale);
}

// Same computation for rows that fit in registers (vocab <= 512 * CE_MAXV * 8 and a multiple of 8): every thread keeps its
// CE_MAXV 16-byte pieces of the row, so the row is read from memory once, the maximum is found without exponentials, and
// the two exponentials per element (sum, gradient) carry no data-dependent branch.
constexpr int CE_MAXV = 13;

__global__ void __launch_bounds__(512)
ce_fwd_bwd_reg_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ targets, float* __restrict__ loss,
                      const float* __restrict__ grad_scale, int vocab, long long row_stride, long long ignore_index, int write_grad) {
    __shared__ float red[16];
    __shared__ float bcast;
    const long long row = blockIdx.x;
    uint4* p = reinterpret_cast<uint4*>(logits + row * row_stride);
    long long tgt = targets[row];
    if (!GM_IN_BOUNDS(tgt == ignore_index || (tgt >= 0 && tgt < vocab), 905)) tgt = ignore_index;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int vec = vocab / 8;
    if (tgt == ignore_index) {
        if (threadIdx.x == 0) loss[row] = 0.f;
        if (write_grad)
            for (int i = threadIdx.x; i < vec; i += 512) p[i] = make_uint4(0, 0, 0, 0);
        return;
    }
    uint4 raw[CE_MAXV];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < CE_MAXV; ++j) {
        const int i = threadIdx.x + j * 512;
        raw[j] = make_uint4(0xff80ff80u, 0xff80ff80u, 0xff80ff80u, 0xff80ff80u);          // bf16 -inf pairs: neutral for max and sum
        if (i < vec) raw[j] = p[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h[e]); m = fmaxf(m, fmaxf(f.x, f.y)); }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = red[0];
#pragma unroll
        for (int w = 1; w < 16; ++w) t = fmaxf(t, red[w]);
        bcast = t;
    }
    __syncthreads();
    const float gmax = bcast;
    float s = 0.f;
    constexpr float LOG2E = 1.4426950408889634f;
    const float mb = gmax * LOG2E;
#pragma unroll
    for (int j = 0; j < CE_MAXV; ++j) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            s += ex2_approx(fmaf(f.x, LOG2E, -mb)) + ex2_approx(fmaf(f.y, LOG2E, -mb));
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    __syncthreads();                                      // red / bcast are reused
    if (lane == 0) red[warp] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 16; ++w) t += red[w];
        bcast = t;
    }
    __syncthreads();
    const float lse = gmax + __logf(bcast);
    if (threadIdx.x == 0) loss[row] = lse - __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[tgt]);
    if (!write_grad) return;
    __syncthreads();                                      // the target logit has been read before the row is overwritten
    const float scale = *grad_scale;
    const float lb = lse * LOG2E;
    const int tvec = static_cast<int>(tgt >> 3), tsub = static_cast<int>(tgt & 7);
#pragma unroll
    for (int j = 0; j < CE_MAXV; ++j) {
        const int i = threadIdx.x + j * 512;
        if (i >= vec) continue;
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
        float g[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            g[2 * e] = ex2_approx(fmaf(f.x, LOG2E, -lb));
            g[2 * e + 1] = ex2_approx(fmaf(f.y, LOG2E, -lb));
        }
        if (i == tvec) g[tsub] -= 1.f;
        uint4 o;
        o.x = pack_bf16x2(g[0] * scale, g[1] * scale); o.y = pack_bf16x2(g[2] * scale, g[3] * scale);
        o.z = pack_bf16x2(g[4] * scale, g[5] * scale); o.w = pack_bf16x2(g[6] * scale, g[7] * scale);
        p[i] = o;
    }
}

void launch_ce_fwd_bwd(void* logits, const long long* targets, float* loss, const float* grad_scale, int rows, int vocab,
                       long long row_stride, long long ignore_index, int write_grad, cudaStream_t s) {
    if (vocab % 8 == 0 && vocab / 8 <= 512 * CE_MAXV && row_stride % 8 == 0) {
        ce_fwd_bwd_reg_kernel<<<rows, 512, 0, s>>>(static_cast<__nv_bfloat16*>(logits), targets, loss, grad_scale, vocab, row_stride,
                                                   ignore_index, write_grad);
        return;
    }
    ce_fwd_bwd_kernel<<<rows, 512, 0, s>>>(static_cast<__nv_bfloat16*>(logits), targets, loss, grad_scale, vocab, row_stride,
                                           ignore_index, write_grad);
}

// ---- AdamW ---------------------------------------------------------------------------------------------
// p, g fp32; moments fp32 or bf16.  Decoupled weight decay; bias corrections passed in.  Optionally refreshes a
// bf16 copy of the parameter (the GEMM operand) in the same pass.
template <typename TM>
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p, const float* __restrict__ g, TM* __restrict__ m, TM* __restrict__ v,
             __nv_bfloat16* __restrict__ p_bf16, long long n, float lr, float beta1, float beta2, float eps, float wd,
             float bc1, float bc2_sqrt, float grad_scale) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const float grad = g[i] * grad_scale;
        float mi, vi;
        if constexpr (sizeof(TM) == 4) { mi = m[i]; vi = v[i]; } else { mi = __bfloat162float(m[i]); vi = __bfloat162float(v[i]); }
        mi = beta1 * mi + (1.f - beta1) * grad;
        vi = beta2 * vi + (1.f - beta2) * grad * grad;
        if constexpr (sizeof(TM) == 4) { m[i] = mi; v[i] = vi; } else { m[i] = __float2bfloat16(mi); v[i] = __float2bfloat16(vi); }
        float w = p[i] * (1.f - lr * wd);
        w -= lr / bc1 * mi / (sqrtf(vi) / bc2_sqrt + eps);
        p[i] = w;
        if (p_bf16) p_bf16[i] = __float2bfloat16(w);
    }
}

void launch_adamw(float* p, const float* g, void* m, void* v, bool moments_bf16, void* p_bf16, long long n, float lr, float beta1,
                  float beta2, float eps, float wd, float bc1, float bc2_sqrt, float grad_scale, cudaStream_t s) {
    const int blocks = static_cast<int>(std::min<long long>((n + 255) / 256, 2368LL));
    if (moments_bf16)
        adamw_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(p, g, static_cast<__nv_bfloat16*>(m), static_cast<__nv_bfloat16*>(v),
                                                           static_cast<__nv_bfloat16*>(p_bf16), n, lr, beta1, beta2, eps, wd, bc1, bc2_sqrt, grad_scale);
    else
        adamw_kernel<float><<<blocks, 256, 0, s>>>(p, g, static_cast<float*>(m), static_cast<float*>(v),
                                                   static_cast<__nv_bfloat16*>(p_bf16), n, lr, beta1, beta2, eps, wd, bc1, bc2_sqrt, grad_scale);
}

// ---- Muon element-wise stages -----------------------------------------------------------------------------
// For matrix i of a same-shape bucket (pointer tables on the device):
//   buf = momentum*buf + g ;  u = nesterov ? g + momentum*buf : buf ;  packed[i] = bf16(u), transposed if tall
// and per-matrix sum of squares of bf16(u) (for the Frobenius normalisation) accumulated into sumsq[i].
// 32x32 tiles through shared memory keep both the row-major reads and the (possibly transposed) writes coalesced.
__global__ void __launch_bounds__(256)
muon_prepare_kernel(const float* const* __restrict__ grads, float* const* __restrict__ bufs, __nv_bfloat16* __restrict__ packed,
                    float* __restrict__ sumsq, int rows, int cols, long long g_stride, long long b_stride, float momentum,
                    int nesterov, int transpose, float grad_scale) {
    __shared__ float tile[32][33];
    __shared__ float part[8];
    const int mat = blockIdx.z;
    const float* g = grads[mat];
    float* buf = bufs[mat];
    __nv_bfloat16* out = packed + static_cast<long long>(mat) * rows * cols;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    float local = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + ty + 8 * i, c = c0 + tx;
        float u = 0.f;
        if (r < rows && c < cols) {
            const float grad = g[r * g_stride + c] * grad_scale;
            float b = buf[r * b_stride + c] * momentum;
            b = b + grad;
            buf[r * b_stride + c] = b;
            u = __bfloat162float(__float2bfloat16(nesterov ? fmaf(momentum, b, grad) : b));
            if (!transpose) out[static_cast<long long>(r) * cols + c] = __float2bfloat16(u);
        }
        tile[ty + 8 * i][tx] = u;
        local += u * u;
    }
    if (transpose) {
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = c0 + ty + 8 * i, r = r0 + tx;          // out is [cols][rows]
            if (r < rows && c < cols) out[static_cast<long long>(c) * rows + r] = __float2bfloat16(tile[tx][ty + 8 * i]);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    if (tx == 0) part[ty] = local;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
        for (int w = 0; w < 8; ++w) t += part[w];
        atomicAdd(&sumsq[mat], t);
    }
}

// x[i] *= 1 / (sqrt(sumsq[mat]) * 1.02 + 1e-6)   (spectral norm <= 1 before the first iteration)
__global__ void __launch_bounds__(256)
muon_normalize_kernel(__nv_bfloat16* __restrict__ packed, const float* __restrict__ sumsq, long long per_matrix) {
    const int mat = blockIdx.y;
    const float inv = 1.f / (sqrtf(sumsq[mat]) * 1.02f + 1e-6f);
    uint4* x = reinterpret_cast<uint4*>(packed + mat * per_matrix);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < per_matrix / 8; i += static_cast<long long>(gridDim.x) * blockDim.x) {
        uint4 raw = x[i];
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            h[e] = __floats2bfloat162_rn(f.x * inv, f.y * inv);
        }
        x[i] = raw;
    }
}

// W[i] += alpha * O[i] (O bf16, stored transposed when the matrix is tall); optionally refresh the bf16 copy of W
__global__ void __launch_bounds__(256)
muon_apply_kernel(float* const* __restrict__ weights, __nv_bfloat16* const* __restrict__ weights_bf16,
                  const __nv_bfloat16* __restrict__ update, int rows, int cols, long long w_stride, float alpha, int transpose) {
    __shared__ float tile[32][33];
    const int mat = blockIdx.z;
    float* w = weights[mat];
    __nv_bfloat16* wb = weights_bf16 ? weights_bf16[mat] : nullptr;
    const __nv_bfloat16* o = update + static_cast<long long>(mat) * rows * cols;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    if (transpose) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = c0 + ty + 8 * i, r = r0 + tx;          // update is [cols][rows]
            tile[ty + 8 * i][tx] = (r < rows && c < cols) ? __bfloat162float(o[static_cast<long long>(c) * rows + r]) : 0.f;
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + ty + 8 * i, c = c0 + tx;
        if (r < rows && c < cols) {
            const float upd = transpose ? tile[tx][ty + 8 * i] : __bfloat162float(o[static_cast<long long>(r) * cols + c]);
            const float nw = w[r * w_stride + c] + alpha * upd;
            w[r * w_stride + c] = nw;
            if (wb) wb[r * w_stride + c] = __float2bfloat16(nw);
        }
    }
}

void launch_muon_prepare(const float* const* grads, float* const* bufs, void* packed, float* sumsq, int n_mats, int rows, int cols,
                         long long g_stride, long long b_stride, float momentum, int nesterov, int transpose, float grad_scale,
                         cudaStream_t s) {
    const long long n = static_cast<long long>(rows) * cols;
    dim3 grid((cols + 31) / 32, (rows + 31) / 32, n_mats);
    muon_prepare_kernel<<<grid, 256, 0, s>>>(grads, bufs, static_cast<__nv_bfloat16*>(packed), sumsq, rows, cols, g_stride, b_stride,
                                             momentum, nesterov, transpose, grad_scale);
    dim3 grid2(static_cast<unsigned>(std::min<long long>((n / 8 + 255) / 256, 592LL)), n_mats);
    muon_normalize_kernel<<<grid2, 256, 0, s>>>(static_cast<__nv_bfloat16*>(packed), sumsq, n);
}

void launch_muon_normalize(void* packed, const float* sumsq, int n_mats, long long per_matrix, cudaStream_t s) {
    dim3 grid(static_cast<unsigned>(std::min<long long>((per_matrix / 8 + 255) / 256, 592LL)), n_mats);
    muon_normalize_kernel<<<grid, 256, 0, s>>>(static_cast<__nv_bfloat16*>(packed), sumsq, per_matrix);
}

void launch_muon_apply(float* const* weights, void* const* weights_bf16, const void* update, int n_mats, int rows, int cols,
                       long long w_stride, float alpha, int transpose, cudaStream_t s) {
    dim3 grid((cols + 31) / 32, (rows + 31) / 32, n_mats);
    muon_apply_kernel<<<grid, 256, 0, s>>>(weights, reinterpret_cast<__nv_bfloat16* const*>(weights_bf16),
                                           static_cast<const __nv_bfloat16*>(update), rows, cols, w_stride, alpha, transpose);
}

// dst_bf16 = bf16(src_fp32)  (compute copies of weights; n elements)
__global__ void __launch_bounds__(256) cast_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
    for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
        if (i + 4 <= n) {
            const float4 f = *reinterpret_cast<const float4*>(src + i);
            uint2 o;
            o.x = pack_bf16x2(f.x, f.y);
            o.y = pack_bf16x2(f.z, f.w);
            *reinterpret_cast<uint2*>(dst + i) = o;
        } else {
            for (long long j = i; j < n; ++j) dst[j] = __float2bfloat16(src[j]);
        }
    }
}
void launch_cast_bf16(const float* src, void* dst, long long n, cudaStream_t s) {
    const int blocks = static_cast<int>(std::min<long long>((n / 4 + 255) / 256 + 1, 2368LL));
    cast_bf16_kernel<<<blocks, 256, 0, s>>>(src, static_cast<__nv_bfloat16*>(dst), n);
}

GM_DEFINE_BOUNDS_READER(loss)

}  // namespace gm

// Memory-bound row kernels: RMSNorm (forward / backward, optionally fused with the residual update) and
// RoPE + per-head QK-norm (forward / backward).  One warp owns one row; statistics are fp32.
//
// Reference counterparts: `model/linear/fp8/custom/rms_norm.py:14-91` (RMSNorm gain / backward),
// `model/attention/qk_norm_rope.py:21-150` (RoPE -> QK-norm -> clamped learned scale),
// `experiments/057-fused-attention-residual-rmsnorm.patch` (residual + RMSNorm).
#include "../common/ptx.cuh"
#include "../common/mxfp8.cuh"
#include "../kernels_decl.h"

namespace gm {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T> __device__ __forceinline__ void store4(T* p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
    uint2 raw;
    raw.x = pack_bf16x2(v.x, v.y);
    raw.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = raw;
}

constexpr int NORM_WARPS = 8;
// A row of d elements is covered by d/128 chunks of 128 (32 lanes x 4); the chunk count is a template
// parameter so the per-lane row copy stays in registers.  Supported: d = 128*{1,2,4,6,8,12,16} (up to 2048).

// x_new = alpha*x + beta*branch (when branch != nullptr; written to x_out), y = rmsnorm(x_new) * w
// yq / ysf (optional): the MXFP8 copy of y (e4m3 + scale records of the bf16 values stored), so the projection that consumes y
// needs no quantisation pass (reference: RMSNorm writing the FP8 layouts directly, model/linear/fp8/custom/rms_norm.py:23-55).
// A lane holds 4 consecutive columns per chunk: a 32-column block is 8 adjacent lanes.
template <typename TX, int MAX_CHUNKS>
__global__ void __launch_bounds__(NORM_WARPS * 32)
rmsnorm_fwd_kernel(const TX* __restrict__ x, const __nv_bfloat16* __restrict__ branch, const float* __restrict__ alpha,
                   const float* __restrict__ beta, TX* __restrict__ x_out, const float* __restrict__ w,
                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, uint8_t* __restrict__ yq, uint8_t* __restrict__ ysf,
                   int rows, int d, float eps) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * NORM_WARPS + (threadIdx.x >> 5);
    if (row >= rows) return;                       // whole warps leave together: a warp owns one row
    const int chunks = d >> 7;
    const float a = alpha ? *alpha : 1.f, b = beta ? *beta : 1.f;
    float4 v[MAX_CHUNKS];
    float ss = 0.f;
    const long long base = static_cast<long long>(row) * d;
#pragma unroll
    for (int c = 0; c < MAX_CHUNKS; ++c) {
        if (c < chunks) {
            const int col = (c * 32 + lane) * 4;
            float4 t = load4<TX>(x + base + col);
            if (branch) {
                const float4 r = load4<__nv_bfloat16>(branch + base + col);
                t.x = a * t.x + b * r.x; t.y = a * t.y + b * r.y; t.z = a * t.z + b * r.z; t.w = a * t.w + b * r.w;
                store4<TX>(x_out + base + col, t);
            }
            v[c] = t;
            ss += t.x * t.x + t.y * t.y + t.z * t.z + t.w * t.w;
        }
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / d + eps);
    if (lane == 0 && rstd) rstd[row] = r;
#pragma unroll
    for (int c = 0; c < MAX_CHUNKS; ++c) {
        if (c < chunks) {
            const int col = (c * 32 + lane) * 4;
            float4 g = w ? *reinterpret_cast<const float4*>(w + col) : make_float4(1.f, 1.f, 1.f, 1.f);
            const float4 o = make_float4(v[c].x * r * g.x, v[c].y * r * g.y, v[c].z * r * g.z, v[c].w * r * g.w);
            store4<__nv_bfloat16>(y + base + col, o);
            if (yq != nullptr) {
                const float q4[4] = {round_bf16(o.x), round_bf16(o.y), round_bf16(o.z), round_bf16(o.w)};
                uint32_t out[1];
                const uint32_t e8 = quantize_block_lanes<4>(q4, out);
                *reinterpret_cast<uint32_t*>(yq + base + col) = out[0];
                if ((lane & 7) == 0) ysf[sf_offset(row, col >> 5, d >> 7)] = static_cast<uint8_t>(e8);
            }
        }
    }
}

// dx = rstd * (w*dy - xhat * mean(w*dy*xhat)) (+ dres), dw partial per block (deterministic two-pass reduce).
template <typename TX, int MAX_CHUNKS>
__global__ void __launch_bounds__(NORM_WARPS * 32)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const TX* __restrict__ x, const float* __restrict__ w,
                   const float* __restrict__ rstd, const TX* __restrict__ dres, TX* __restrict__ dx,
                   float* __restrict__ dw_partial, int rows, int d) {
    extern __shared__ float smem_dw[];      // [NORM_WARPS][d]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int chunks = d >> 7;
    float4 acc[MAX_CHUNKS];
#pragma unroll
    for (int c = 0; c < MAX_CHUNKS; ++c) acc[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int row = blockIdx.x * NORM_WARPS + warp; row < rows; row += gridDim.x * NORM_WARPS) {
        const long long base = static_cast<long long>(row) * d;
        const float r = rstd[row];
        // one dependent memory phase per row: x, dy and the residual gradient are all requested before the row reduction
        float4 xh[MAX_CHUNKS], e[MAX_CHUNKS];
        uint2 dyraw[MAX_CHUNKS];
        float dot = 0.f;
#pragma unroll
        for (int c = 0; c < MAX_CHUNKS; ++c) {
            if (c < chunks) {
                const int col = (c * 32 + lane) * 4;
                xh[c] = load4<TX>(x + base + col);
                dyraw[c] = *reinterpret_cast<const uint2*>(dy + base + col);
                if (dres) e[c] = load4<TX>(dres + base + col);
            }
        }
#pragma unroll
        for (int c = 0; c < MAX_CHUNKS; ++c) {
            if (c < chunks) {
                const int col = (c * 32 + lane) * 4;
                const float2 d01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dyraw[c].x));
                const float2 d23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dyraw[c].y));
                const float4 wv = w ? *reinterpret_cast<const float4*>(w + col) : make_float4(1.f, 1.f, 1.f, 1.f);
                xh[c] = make_float4(xh[c].x * r, xh[c].y * r, xh[c].z * r, xh[c].w * r);
                acc[c].x += d01.x * xh[c].x; acc[c].y += d01.y * xh[c].y; acc[c].z += d23.x * xh[c].z; acc[c].w += d23.y * xh[c].w;
                dot += d01.x * wv.x * xh[c].x + d01.y * wv.y * xh[c].y + d23.x * wv.z * xh[c].z + d23.y * wv.w * xh[c].w;
            }
        }
        dot = warp_sum(dot) / d;
#pragma unroll
        for (int c = 0; c < MAX_CHUNKS; ++c) {
            if (c < chunks) {
                const int col = (c * 32 + lane) * 4;
                const float2 d01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dyraw[c].x));
                const float2 d23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dyraw[c].y));
                const float4 wv = w ? *reinterpret_cast<const float4*>(w + col) : make_float4(1.f, 1.f, 1.f, 1.f);
                float4 o = make_float4(r * (d01.x * wv.x - xh[c].x * dot), r * (d01.y * wv.y - xh[c].y * dot),
                                       r * (d23.x * wv.z - xh[c].z * dot), r * (d23.y * wv.w - xh[c].w * dot));
                if (dres) { o.x += e[c].x; o.y += e[c].y; o.z += e[c].z; o.w += e[c].w; }
                store4<TX>(dx + base + col, o);
            }
        }
    }
    if (dw_partial == nullptr) return;
#pragma unroll
    for (int c = 0; c < MAX_CHUNKS; ++c) {
        if (c < chunks) *reinterpret_cast<float4*>(smem_dw + warp * d + (c * 32 + lane) * 4) = acc[c];
    }
    __syncthreads();
    for (int col = threadIdx.x; col < d; col += blockDim.x) {
        float s = 0.f;
#pragma unroll
        for (int wi = 0; wi < NORM_WARPS; ++wi) s += smem_dw[wi * d + col];
        dw_partial[static_cast<long long>(blockIdx.x) * d + col] = s;
    }
}

// out[col] = sum over rows of partial[row][col]  (second pass of the deterministic column reductions).
// Each block owns 32 columns; 32 warps stride over the rows (four independent loads in flight per thread) and combine
// through shared memory in a fixed order.
constexpr int COLSUM_WARPS = 32;
__global__ void __launch_bounds__(COLSUM_WARPS * 32)
column_sum_kernel(const float* __restrict__ partial, float* __restrict__ out, int rows, int cols, int accumulate) {
    __shared__ float red[COLSUM_WARPS][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int col = blockIdx.x * 32 + tx;
    float s = 0.f;
    if (col < cols) {
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        int r = ty;
        for (; r + 3 * COLSUM_WARPS < rows; r += 4 * COLSUM_WARPS) {
            s0 += partial[static_cast<long long>(r) * cols + col];
            s1 += partial[static_cast<long long>(r + COLSUM_WARPS) * cols + col];
            s2 += partial[static_cast<long long>(r + 2 * COLSUM_WARPS) * cols + col];
            s3 += partial[static_cast<long long>(r + 3 * COLSUM_WARPS) * cols + col];
        }
        for (; r < rows; r += COLSUM_WARPS) s0 += partial[static_cast<long long>(r) * cols + col];
        s = (s0 + s1) + (s2 + s3);
    }
    red[ty][tx] = s;
    __syncthreads();
    if (ty == 0 && col < cols) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < COLSUM_WARPS; ++w) t += red[w][tx];
        out[col] = accumulate ? out[col] + t : t;
    }
}

// out[0] = sum of partial[0 .. n)  (the one-column case: every thread takes a strided share, fixed combination order)
__global__ void __launch_bounds__(1024)
vector_sum_kernel(const float* __restrict__ partial, float* __restrict__ out, int n) {
    __shared__ float red[32];
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += 1024) s += partial[i];
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = warp_sum(red[threadIdx.x]);
        if (threadIdx.x == 0) *out = t;
    }
}

// Backward of x_new = x + beta * branch with respect to the branch and beta:
//   dbranch = bf16(beta * dxn),  partial[block] = sum(dxn * branch)   (fixed-order block partials)
__global__ void __launch_bounds__(256)
residual_bwd_kernel(const float* __restrict__ dxn, const __nv_bfloat16* __restrict__ branch, const float* __restrict__ beta,
                    __nv_bfloat16* __restrict__ dbranch, float* __restrict__ partial, long long n) {
    __shared__ float red[8];
    const float b = *beta;
    float dot = 0.f;
    for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
        const float4 g = *reinterpret_cast<const float4*>(dxn + i);
        const float4 r = load4<__nv_bfloat16>(branch + i);
        dot += g.x * r.x + g.y * r.y + g.z * r.z + g.w * r.w;
        store4<__nv_bfloat16>(dbranch + i, make_float4(b * g.x, b * g.y, b * g.z, b * g.w));
    }
    dot = warp_sum(dot);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = dot;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += red[w];
        partial[blockIdx.x] = t;
    }
}

int residual_bwd_blocks(long long n) { return static_cast<int>(n / 4 / 256 + 1 < 1184 ? n / 4 / 256 + 1 : 1184); }

void launch_residual_bwd(const float* dxn, const void* branch, const float* beta, void* dbranch, float* partial, float* dbeta,
                         long long n, cudaStream_t s) {
    const int blocks = residual_bwd_blocks(n);
    residual_bwd_kernel<<<blocks, 256, 0, s>>>(dxn, static_cast<const __nv_bfloat16*>(branch), beta, static_cast<__nv_bfloat16*>(dbranch), partial, n);
    vector_sum_kernel<<<1, 1024, 0, s>>>(partial, dbeta, blocks);
}

bool norm_dim_supported(int d) {
    const int c = d / 128;
    return d % 128 == 0 && (c == 1 || c == 2 || c == 4 || c == 6 || c == 8 || c == 12 || c == 16);
}

#define GM_DISPATCH_CHUNKS(d, CALL)        \
    switch ((d) / 128) {                   \
        case 1: { CALL(1); } break;        \
        case 2: { CALL(2); } break;        \
        case 4: { CALL(4); } break;        \
        case 6: { CALL(6); } break;        \
        case 8: { CALL(8); } break;        \
        case 12: { CALL(12); } break;      \
        case 16: { CALL(16); } break;      \
        default: return false;             \
    }

bool launch_rmsnorm_fwd(const void* x, bool x_fp32, const void* branch, const float* alpha, const float* beta, void* x_out,
                        const float* w, void* y, float* rstd, void* yq, void* ysf, int rows, int d, float eps, cudaStream_t s) {
    if (!norm_dim_supported(d)) return false;
    const int blocks = (rows + NORM_WARPS - 1) / NORM_WARPS;
#define GM_FWD(C)                                                                                                              \
    if (x_fp32)                                                                                                                \
        rmsnorm_fwd_kernel<float, C><<<blocks, NORM_WARPS * 32, 0, s>>>(                                                       \
            static_cast<const float*>(x), static_cast<const __nv_bfloat16*>(branch), alpha, beta, static_cast<float*>(x_out), w, \
            static_cast<__nv_bfloat16*>(y), rstd, static_cast<uint8_t*>(yq), static_cast<uint8_t*>(ysf), rows, d, eps);         \
    else                                                                                                                       \
        rmsnorm_fwd_kernel<__nv_bfloat16, C><<<blocks, NORM_WARPS * 32, 0, s>>>(                                               \
            static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(branch), alpha, beta,                      \
            static_cast<__nv_bfloat16*>(x_out), w, static_cast<__nv_bfloat16*>(y), rstd, static_cast<uint8_t*>(yq),            \
            static_cast<uint8_t*>(ysf), rows, d, eps);
    GM_DISPATCH_CHUNKS(d, GM_FWD)
#undef GM_FWD
    return true;
}

int rmsnorm_bwd_blocks(int rows) { return min(1184, (rows + NORM_WARPS - 1) / NORM_WARPS); }

bool launch_rmsnorm_bwd(const void* dy, const void* x, bool x_fp32, const float* w, const float* rstd, const void* dres, void* dx,
                        float* dw_partial, float* dw, int dw_accumulate, int rows, int d, cudaStream_t s) {
    if (!norm_dim_supported(d)) return false;
    const int blocks = rmsnorm_bwd_blocks(rows);
    const size_t smem = dw_partial ? static_cast<size_t>(NORM_WARPS) * d * sizeof(float) : 0;
#define GM_BWD(C)                                                                                                              \
    if (x_fp32) {                                                                                                              \
        auto k = rmsnorm_bwd_kernel<float, C>;                                                                                 \
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));    \
        k<<<blocks, NORM_WARPS * 32, smem, s>>>(static_cast<const __nv_bfloat16*>(dy), static_cast<const float*>(x), w, rstd,  \
                                                static_cast<const float*>(dres), static_cast<float*>(dx), dw_partial, rows, d); \
    } else {                                                                                                                   \
        auto k = rmsnorm_bwd_kernel<__nv_bfloat16, C>;                                                                         \
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));    \
        k<<<blocks, NORM_WARPS * 32, smem, s>>>(static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x), w, rstd, \
                                                static_cast<const __nv_bfloat16*>(dres), static_cast<__nv_bfloat16*>(dx), dw_partial, rows, d); \
    }
    GM_DISPATCH_CHUNKS(d, GM_BWD)
#undef GM_BWD
    if (dw_partial) column_sum_kernel<<<(d + 31) / 32, COLSUM_WARPS * 32, 0, s>>>(dw_partial, dw, blocks, d, dw_accumulate);
    return true;
}

void launch_column_sum(const float* partial, float* out, int rows, int cols, int accumulate, cudaStream_t s) {
    column_sum_kernel<<<(cols + 31) / 32, COLSUM_WARPS * 32, 0, s>>>(partial, out, rows, cols, accumulate);
}

// ---- RoPE + QK-norm ---------------------------------------------------------------------------------------
// Rows are (token, head) vectors of D elements inside a [tokens, row_stride] matrix (the packed QKV GEMM output):
// element (t, h, i) sits at t*row_stride + h*D + i.  The first `q_heads` heads use q_scale, the next `k_heads`
// heads use k_scale.  pos = t % seq_len indexes the cos/sin tables [seq_len, D/2].
// forward:  r = rope(x);  g = rsqrt(mean|sum(r^2) + eps);  y = r * g * clamp(scale[h])
// backward: dr = g*s*(dy - r * g^2 * mean|sum(dy*r));  dx = rope^T(dr);  dscale[h] += sum(dy * r * g) inside the clamp range
// A lane owns four rotation pairs (16 bytes) of one head, so a head of D elements takes D/8 lanes and a warp works on
// 256/D heads of a token at once; statistics are reduced inside the head's lane group.  Forward also copies `copy_cols`
// trailing columns (the value heads of a packed QKV row) from x to out; backward may run in place (out == dy): every
// element is read by the lane that later writes it.
template <int D>
__device__ __forceinline__ float head_sum(float v) {
#pragma unroll
    for (int o = D / 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int D, bool BWD>
__global__ void __launch_bounds__(256)
rope_qknorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* dy, __nv_bfloat16* out,
                   const float* __restrict__ cos_t, const float* __restrict__ sin_t, const float* __restrict__ q_scale,
                   const float* __restrict__ k_scale, float* __restrict__ dscale_partial, long long tokens, int seq_len,
                   int q_heads, int k_heads, long long x_stride, long long o_stride, float eps, int rms, float smin, float smax,
                   int copy_cols, const float* __restrict__ dq32, long long dq_stride, uint8_t* __restrict__ mxq, uint8_t* __restrict__ mxsf,
                   int mx_width) {
    constexpr int PAIRS = D / 2;
    constexpr int LANES = D / 8;                 // lanes per head
    constexpr int HEADS_PER_WARP = 32 / LANES;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane / LANES, li = lane % LANES;
    const int heads = q_heads + k_heads;
    const int groups = (heads + HEADS_PER_WARP - 1) / HEADS_PER_WARP;
    const long long total = tokens * groups;
    const bool has_norm = q_scale != nullptr;
    __shared__ float ds_smem[8][64];
    if (BWD) {
        for (int i = threadIdx.x; i < 8 * 64; i += blockDim.x) (&ds_smem[0][0])[i] = 0.f;
        __syncthreads();
    }
    for (long long idx = static_cast<long long>(blockIdx.x) * 8 + warp; idx < total; idx += static_cast<long long>(gridDim.x) * 8) {
        const long long t = idx / groups;
        const int h = static_cast<int>(idx - t * groups) * HEADS_PER_WARP + sub;
        const bool live = h < heads;
        const int pos = static_cast<int>(t % seq_len);
        float c[4] = {1.f, 1.f, 1.f, 1.f}, sn[4] = {0.f, 0.f, 0.f, 0.f};
        if (cos_t) {
            const float4 cv = *reinterpret_cast<const float4*>(cos_t + pos * PAIRS + li * 4);
            const float4 sv = *reinterpret_cast<const float4*>(sin_t + pos * PAIRS + li * 4);
            c[0] = cv.x; c[1] = cv.y; c[2] = cv.z; c[3] = cv.w;
            sn[0] = sv.x; sn[1] = sv.y; sn[2] = sv.z; sn[3] = sv.w;
        }
        uint4 xraw = make_uint4(0, 0, 0, 0), graw = make_uint4(0, 0, 0, 0);
        if (live) {
            xraw = *reinterpret_cast<const uint4*>(x + t * x_stride + h * D + li * 8);
            if (BWD && !(dq32 != nullptr && h < q_heads)) graw = *reinterpret_cast<const uint4*>(dy + t * o_stride + h * D + li * 8);
        }
        const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xraw);
        const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&graw);
        float r1[4], r2[4], g1[4], g2[4];
        float ss = 0.f, dot = 0.f;
        // backward: query-head gradients may arrive as fp32 (the attention backward's dQ accumulator) instead of bf16 rows
        const bool g_fp32 = BWD && dq32 != nullptr && live && h < q_heads;
        float4 ga = make_float4(0.f, 0.f, 0.f, 0.f), gb = ga;
        if (g_fp32) {
            ga = *reinterpret_cast<const float4*>(dq32 + t * dq_stride + h * D + li * 8);
            gb = *reinterpret_cast<const float4*>(dq32 + t * dq_stride + h * D + li * 8 + 4);
        }
        const float gq[8] = {ga.x, ga.y, ga.z, ga.w, gb.x, gb.y, gb.z, gb.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 xf = __bfloat1622float2(xp[i]);
            r1[i] = xf.x * c[i] - xf.y * sn[i];
            r2[i] = xf.x * sn[i] + xf.y * c[i];
            ss += r1[i] * r1[i] + r2[i] * r2[i];
            if (BWD) {
                const float2 gf = __bfloat1622float2(gp[i]);
                g1[i] = g_fp32 ? gq[2 * i] : gf.x;
                g2[i] = g_fp32 ? gq[2 * i + 1] : gf.y;
                dot += g1[i] * r1[i] + g2[i] * r2[i];
            }
        }
        const float raw = !live ? 1.f : h < q_heads ? (q_scale ? q_scale[h] : 1.f) : (k_scale ? k_scale[h - q_heads] : 1.f);
        const float sc = fminf(fmaxf(raw, smin), smax);
        float gain = 1.f, mult = 1.f;
        if (has_norm) {
            ss = head_sum<D>(ss);
            gain = rsqrtf((rms ? ss / D : ss) + eps);
            mult = gain * sc;
        }
        uint4 oraw;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&oraw);
        if (BWD) {
            dot = head_sum<D>(dot);
            if (has_norm && live && li == 0 && raw >= smin && raw <= smax) ds_smem[warp][h] += dot * gain;
            const float coef = has_norm ? gain * gain * (rms ? dot / D : dot) : 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float d1 = mult * (g1[i] - r1[i] * coef), d2 = mult * (g2[i] - r2[i] * coef);
                op[i] = __floats2bfloat162_rn(d1 * c[i] + d2 * sn[i], -d1 * sn[i] + d2 * c[i]);
            }
            if (live) *reinterpret_cast<uint4*>(out + t * x_stride + h * D + li * 8) = oraw;
            if (mxq != nullptr) {
                // MXFP8 copy of the packed gradient row (the operand of the projection's input-gradient GEMM): a lane's 8
                // values are a quarter of a 32-column block, the 4 lanes of a block are adjacent
                float v8[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float2 f = __bfloat1622float2(op[i]);
                    v8[2 * i] = live ? f.x : 0.f; v8[2 * i + 1] = live ? f.y : 0.f;
                }
                uint32_t o2[2];
                const uint32_t e8 = quantize_block_lanes<8>(v8, o2);
                if (live) {
                    const int col = h * D + li * 8;
                    *reinterpret_cast<uint2*>(mxq + t * mx_width + col) = make_uint2(o2[0], o2[1]);
                    if ((lane & 3) == 0) mxsf[sf_offset(t, col >> 5, (mx_width + 127) >> 7)] = static_cast<uint8_t>(e8);
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) op[i] = __floats2bfloat162_rn(r1[i] * mult, r2[i] * mult);
            if (live) *reinterpret_cast<uint4*>(out + t * o_stride + h * D + li * 8) = oraw;
        }
    }
    if (!BWD && copy_cols > 0) {
        const int vecs = copy_cols / 8;
        const long long n = tokens * vecs;
        for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x) {
            const long long t = i / vecs;
            const int v = static_cast<int>(i - t * vecs);
            *reinterpret_cast<uint4*>(out + t * o_stride + heads * D + v * 8) = *reinterpret_cast<const uint4*>(x + t * x_stride + heads * D + v * 8);
        }
    }
    if (BWD && mxq != nullptr && copy_cols > 0) {
        // the trailing (value) columns of the gradient row pass through unchanged: only their quantised copy is produced here
        const int vecs = copy_cols / 8;
        const long long n = tokens * vecs;
        for (long long base = static_cast<long long>(blockIdx.x) * blockDim.x + (threadIdx.x & ~31); base < n; base += static_cast<long long>(gridDim.x) * blockDim.x) {
            const long long i = base + lane;
            const bool active = i < n;
            const long long t = active ? i / vecs : 0;
            const int col = heads * D + (active ? static_cast<int>(i - t * vecs) * 8 : 0);
            float v8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (active) {
                const uint4 raw = *reinterpret_cast<const uint4*>(dy + t * o_stride + col);
                const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(hp[e]); v8[2 * e] = f.x; v8[2 * e + 1] = f.y; }
            }
            uint32_t o2[2];
            const uint32_t e8 = quantize_block_lanes<8>(v8, o2);
            if (active) {
                *reinterpret_cast<uint2*>(mxq + t * mx_width + col) = make_uint2(o2[0], o2[1]);
                if ((lane & 3) == 0) mxsf[sf_offset(t, col >> 5, (mx_width + 127) >> 7)] = static_cast<uint8_t>(e8);
            }
        }
    }
    if (BWD && dscale_partial) {
        __syncthreads();
        for (int h = threadIdx.x; h < heads; h += blockDim.x) {
            float s = 0.f;
#pragma unroll
            for (int wi = 0; wi < 8; ++wi) s += ds_smem[wi][h];
            dscale_partial[static_cast<long long>(blockIdx.x) * heads + h] = s;
        }
    }
}

int rope_blocks(long long tokens, int heads) {
    const long long want = (tokens * ((heads + 3) / 4) + 7) / 8;      // at least 4 heads of a token per warp pass for every supported head size
    return static_cast<int>(want < 2368 ? want : 2368);
}

bool launch_rope_qknorm(bool bwd, int D, const void* x, const void* dy, void* out, const float* cos_t, const float* sin_t,
                        const float* q_scale, const float* k_scale, float* dscale_partial, long long tokens, int seq_len,
                        int q_heads, int k_heads, long long x_stride, long long o_stride, float eps, int rms, float smin,
                        float smax, int copy_cols, const float* dq32, long long dq_stride, void* gq, void* gsf, int gq_width,
                        cudaStream_t s) {
    if (q_heads + k_heads > 64) return false;
    const int blocks = rope_blocks(tokens, q_heads + k_heads);
#define GM_ROPE(DD)                                                                                                            \
    if (bwd)                                                                                                                   \
        rope_qknorm_kernel<DD, true><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy), \
            static_cast<__nv_bfloat16*>(out), cos_t, sin_t, q_scale, k_scale, dscale_partial, tokens, seq_len, q_heads, k_heads,  \
            x_stride, o_stride, eps, rms, smin, smax, copy_cols, dq32, dq_stride, static_cast<uint8_t*>(gq),                   \
            static_cast<uint8_t*>(gsf), gq_width);                                                                             \
    else                                                                                                                       \
        rope_qknorm_kernel<DD, false><<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), nullptr,                     \
            static_cast<__nv_bfloat16*>(out), cos_t, sin_t, q_scale, k_scale, nullptr, tokens, seq_len, q_heads, k_heads,        \
            x_stride, o_stride, eps, rms, smin, smax, copy_cols, nullptr, 0, nullptr, nullptr, 0);
    switch (D) {
        case 32: GM_ROPE(32); break;
        case 64: GM_ROPE(64); break;
        case 128: GM_ROPE(128); break;
        default: return false;
    }
#undef GM_ROPE
    return true;
}

}  // namespace gm

// Mixture-of-experts data movement: counted top-k routing into a padded expert-major layout, row gather,
// gated combine (forward / backward) and the expert activation (forward / backward).
//
// Layout produced by routing: the S = M*k (token, slot) pairs are bucketed by expert, order inside a bucket
// is the original slot order (stable, no atomics decide placement), and every bucket is padded to a multiple
// of 256 rows (SEG_PAD).  Consequences: the 256-row tile of a CTA pair of the GEMM never straddles two experts, the
// weight-gradient GEMM can contract over whole padded segments, and pad rows are written as zeros so they contribute nothing.
//   dest[slot]        row of the packed buffer that holds this (token, slot)
//   src_of_row[row]   slot stored in that row, -1 for pad rows
//   seg_ends[e]       cumulative padded end of expert e;  counts[e] the true row count
//   tile_expert[t]    expert of the t-th 128-row tile;  meta[0] = number of tiles, meta[1] = padded rows
// Reference counterparts: `model/feedforward/routing.py:12-96` (histogram -> prefix -> stable permutation),
// `model/linear/fp8/custom/grouped.py:57-72` (per-expert padding to 128), `experiments/053-fused-expert-output-combine.patch`.
#include "../common/ptx.cuh"
#include "../common/mxfp8.cuh"
#include "../kernels_decl.h"

namespace gm {

constexpr int ROUTE_CHUNK = 1024;
constexpr int MAX_EXPERTS = 128;
constexpr int SEG_PAD = 256;

__global__ void __launch_bounds__(ROUTE_CHUNK)
route_count_kernel(const long long* __restrict__ idx, int* __restrict__ chunk_hist, int slots, int experts) {
    __shared__ int hist[MAX_EXPERTS];
    for (int e = threadIdx.x; e < experts; e += blockDim.x) hist[e] = 0;
    __syncthreads();
    const int slot = blockIdx.x * ROUTE_CHUNK + threadIdx.x;
    if (slot < slots) {
        const int e = static_cast<int>(idx[slot]);
        if (GM_IN_BOUNDS(e >= 0 && e < experts, 901)) atomicAdd(&hist[e], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) chunk_hist[blockIdx.x * experts + e] = hist[e];
}

// single block: per-expert prefix over chunks, padded segment plan, tile table, pad rows marked -1
__global__ void __launch_bounds__(128)
route_plan_kernel(const int* __restrict__ chunk_hist, int* __restrict__ chunk_start, int* __restrict__ counts,
                  int* __restrict__ seg_ends, int* __restrict__ tile_expert, int* __restrict__ meta,
                  int* __restrict__ src_of_row, int chunks, int experts) {
    __shared__ int cnt[MAX_EXPERTS], pstart[MAX_EXPERTS + 1];
    const int e = threadIdx.x;
    if (e < experts) {
        int c = 0;
        for (int ch = 0; ch < chunks; ++ch) c += chunk_hist[ch * experts + e];
        cnt[e] = c;
        counts[e] = c;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int i = 0; i < experts; ++i) {
            pstart[i] = acc;
            acc += (cnt[i] + SEG_PAD - 1) / SEG_PAD * SEG_PAD;
            seg_ends[i] = acc;
        }
        pstart[experts] = acc;
        meta[0] = acc / 128;
        meta[1] = acc;
    }
    __syncthreads();
    if (e < experts) {
        int run = pstart[e];
        for (int ch = 0; ch < chunks; ++ch) {
            chunk_start[ch * experts + e] = run;
            run += chunk_hist[ch * experts + e];
        }
        for (int r = pstart[e] + cnt[e]; r < pstart[e + 1]; ++r) src_of_row[r] = -1;
        for (int t = pstart[e] / 128; t < pstart[e + 1] / 128; ++t) tile_expert[t] = e;
    }
}

__global__ void __launch_bounds__(ROUTE_CHUNK)
route_place_kernel(const long long* __restrict__ idx, const int* __restrict__ chunk_start, int* __restrict__ dest,
                   int* __restrict__ src_of_row, int slots, int experts) {
    __shared__ int warp_count[32][MAX_EXPERTS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < 32 * MAX_EXPERTS; i += blockDim.x) (&warp_count[0][0])[i] = 0;
    __syncthreads();
    const int slot = blockIdx.x * ROUTE_CHUNK + threadIdx.x;
    int e = slot < slots ? static_cast<int>(idx[slot]) : experts;           // `experts` = sentinel for idle lanes
    if (!GM_IN_BOUNDS(e >= 0 && e <= experts, 901)) e = experts;           // checked build: an id out of range places nothing
    const unsigned same = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(same & ((1u << lane) - 1u));
    if (e < experts && rank == 0) warp_count[warp][e] = __popc(same);
    __syncthreads();
    if (threadIdx.x < experts) {           // exclusive prefix over the 32 warps, per expert
        int run = 0;
        for (int w = 0; w < 32; ++w) {
            const int c = warp_count[w][threadIdx.x];
            warp_count[w][threadIdx.x] = run;
            run += c;
        }
    }
    __syncthreads();
    if (e < experts) {
        const int row = chunk_start[blockIdx.x * experts + e] + warp_count[warp][e] + rank;
        dest[slot] = row;
        src_of_row[row] = slot;
    }
}

bool launch_route(const long long* idx, int slots, int experts, int* chunk_hist, int* chunk_start, int* counts, int* seg_ends,
                  int* tile_expert, int* meta, int* dest, int* src_of_row, cudaStream_t s) {
    if (experts > MAX_EXPERTS || slots < 0) return false;
    // slots == 0 (an expert-parallel rank that received no rows this step): the plan alone yields empty segments and zero tiles
    const int chunks = (slots + ROUTE_CHUNK - 1) / ROUTE_CHUNK;
    if (chunks > 0) route_count_kernel<<<chunks, ROUTE_CHUNK, 0, s>>>(idx, chunk_hist, slots, experts);
    route_plan_kernel<<<1, 128, 0, s>>>(chunk_hist, chunk_start, counts, seg_ends, tile_expert, meta, src_of_row, chunks, experts);
    if (chunks > 0) route_place_kernel<<<chunks, ROUTE_CHUNK, 0, s>>>(idx, chunk_start, dest, src_of_row, slots, experts);
    return true;
}

__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(h[i]);
        v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
    uint4 o;
    o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]); o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
    return o;
}

// Every kernel below that writes a bf16 matrix feeding an MXFP8 GEMM can emit the quantised copy in the same pass (`q`, `sf`
// non-null): e4m3 payload + scale records of exactly the bf16 values it stores, so the GEMM operand never costs a pass of its
// own (reference: gather + activation + quantise in one kernel, model/linear/fp8/custom/grouped.py:15-84).  A thread holds 8
// consecutive elements, so a 32-element block is 4 adjacent lanes.

// packed[row] = hidden[src_of_row[row] / k] (zeros for pad rows); one warp per row, 16-byte vectors
__global__ void __launch_bounds__(256)
gather_rows_kernel(const __nv_bfloat16* __restrict__ hidden, const int* __restrict__ src_of_row, const int* __restrict__ meta,
                   __nv_bfloat16* __restrict__ packed, uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int d, int top_k, int cap_rows,
                   int tokens) {
    const int lane = threadIdx.x & 31;
    const int total = min(meta[1], cap_rows);
    const int vecs = d / 8, k_blocks = (d + 127) >> 7;
    for (int row = blockIdx.x * 8 + (threadIdx.x >> 5); row < total; row += gridDim.x * 8) {
        int src = src_of_row[row];
        if (!GM_IN_BOUNDS(src < 0 || src / top_k < tokens, 902)) src = -1;                    // checked build: treated as a pad row
        uint4* out = reinterpret_cast<uint4*>(packed + static_cast<long long>(row) * d);
        const uint4* in = reinterpret_cast<const uint4*>(hidden + static_cast<long long>(src < 0 ? 0 : src / top_k) * d);
        for (int base = 0; base < vecs; base += 32) {                  // warp-uniform trip count: the quantiser shuffles
            const int i = base + lane;
            const bool active = i < vecs;
            const uint4 raw = (active && src >= 0) ? in[i] : make_uint4(0, 0, 0, 0);
            if (active) out[i] = raw;
            if (q != nullptr) {
                float v[8];
                unpack8(raw, v);
                uint32_t o[2];
                const uint32_t e8 = quantize_block_lanes<8>(v, o);
                if (active) {
                    *reinterpret_cast<uint2*>(q + static_cast<long long>(row) * d + i * 8) = make_uint2(o[0], o[1]);
                    if ((lane & 3) == 0) sf[sf_offset(row, i >> 2, k_blocks)] = static_cast<uint8_t>(e8);
                }
            }
        }
    }
}

void launch_gather_rows(const void* hidden, const int* src_of_row, const int* meta, void* packed, void* q, void* sf, int d, int top_k,
                        int cap_rows, int tokens, cudaStream_t s) {
    gather_rows_kernel<<<1184, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(hidden), src_of_row, meta,
                                            static_cast<__nv_bfloat16*>(packed), static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), d, top_k,
                                            cap_rows, tokens);
}

// out[t] = sum_k gates[t,k] * y[dest[t*k+k']]   (fp32 accumulation, bf16 result); one warp per token
__global__ void __launch_bounds__(256)
combine_fwd_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ dest, const float* __restrict__ gates,
                   __nv_bfloat16* __restrict__ out, int tokens, int d, int top_k, int y_rows) {
    const int lane = threadIdx.x & 31;
    for (int t = blockIdx.x * 8 + (threadIdx.x >> 5); t < tokens; t += gridDim.x * 8) {
        for (int i = lane; i < d / 8; i += 32) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int k = 0; k < top_k; ++k) {
                const float g = gates ? gates[t * top_k + k] : 1.f;
                const int row = dest[t * top_k + k];
                if (!GM_IN_BOUNDS(row >= 0 && row < y_rows, 903)) continue;
                const uint4 raw = *reinterpret_cast<const uint4*>(y + static_cast<long long>(row) * d + i * 8);
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(h[e]);
                    acc[2 * e] += g * f.x;
                    acc[2 * e + 1] += g * f.y;
                }
            }
            uint4 o;
            o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
            o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
            *reinterpret_cast<uint4*>(out + static_cast<long long>(t) * d + i * 8) = o;
        }
    }
}

// per packed row: dy[row] = gate * dout[token] (zeros for pad rows), dgate[slot] = <dout[token], y[row]>
__global__ void __launch_bounds__(256)
combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y, const int* __restrict__ src_of_row,
                   const float* __restrict__ gates, const int* __restrict__ meta, __nv_bfloat16* __restrict__ dy,
                   float* __restrict__ dgates, uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int d, int top_k, int cap_rows,
                   int tokens) {
    const int lane = threadIdx.x & 31;
    const int total = min(meta[1], cap_rows);
    const int vecs = d / 8, k_blocks = (d + 127) >> 7;
    for (int row = blockIdx.x * 8 + (threadIdx.x >> 5); row < total; row += gridDim.x * 8) {
        int src = src_of_row[row];
        if (!GM_IN_BOUNDS(src < 0 || src / top_k < tokens, 904)) src = -1;
        const bool live = src >= 0;
        uint4* o = reinterpret_cast<uint4*>(dy + static_cast<long long>(row) * d);
        const float g = live ? gates[src] : 0.f;
        const uint4* gin = reinterpret_cast<const uint4*>(dout + static_cast<long long>(live ? src / top_k : 0) * d);
        const uint4* yin = reinterpret_cast<const uint4*>(y + static_cast<long long>(row) * d);
        float dot = 0.f;
        for (int base = 0; base < vecs; base += 32) {
            const int i = base + lane;
            const bool active = i < vecs;
            uint4 w = make_uint4(0, 0, 0, 0);
            if (active && live) {
                const uint4 a = gin[i], b = yin[i];
                const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
                const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
                uint32_t* wp = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 fa = __bfloat1622float2(ha[e]), fb = __bfloat1622float2(hb[e]);
                    dot += fa.x * fb.x + fa.y * fb.y;
                    wp[e] = pack_bf16x2(g * fa.x, g * fa.y);
                }
            }
            if (active) o[i] = w;
            if (q != nullptr) {
                float v[8];
                unpack8(w, v);                                       // the bf16 values just stored
                uint32_t out[2];
                const uint32_t e8 = quantize_block_lanes<8>(v, out);
                if (active) {
                    *reinterpret_cast<uint2*>(q + static_cast<long long>(row) * d + i * 8) = make_uint2(out[0], out[1]);
                    if ((lane & 3) == 0) sf[sf_offset(row, i >> 2, k_blocks)] = static_cast<uint8_t>(e8);
                }
            }
        }
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, s);
        if (lane == 0 && live) dgates[src] = dot;
    }
}

void launch_combine_fwd(const void* y, const int* dest, const float* gates, void* out, int tokens, int d, int top_k, int y_rows, cudaStream_t s) {
    combine_fwd_kernel<<<1184, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(y), dest, gates, static_cast<__nv_bfloat16*>(out), tokens, d, top_k, y_rows);
}
void launch_combine_bwd(const void* dout, const void* y, const int* src_of_row, const float* gates, const int* meta, void* dy,
                        float* dgates, void* q, void* sf, int d, int top_k, int cap_rows, int tokens, cudaStream_t s) {
    combine_bwd_kernel<<<1184, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(y), src_of_row,
                                            gates, meta, static_cast<__nv_bfloat16*>(dy), dgates, static_cast<uint8_t*>(q),
                                            static_cast<uint8_t*>(sf), d, top_k, cap_rows, tokens);
}

// ---- activations ---------------------------------------------------------------------------------------
// kind: 0 gelu (erf), 1 relu, 2 relu^2, 3 silu, 4 swiglu (pre = [gate | up], gate first).
__device__ __forceinline__ float act_fwd(int kind, float x) {
    switch (kind) {
        case 0: return 0.5f * x * (1.f + erff(x * 0.70710678118f));
        case 1: return fmaxf(x, 0.f);
        case 2: { const float r = fmaxf(x, 0.f); return r * r; }
        default: return x / (1.f + __expf(-x));
    }
}
__device__ __forceinline__ float act_grad(int kind, float x) {
    switch (kind) {
        case 0: return 0.5f * (1.f + erff(x * 0.70710678118f)) + x * 0.3989422804f * __expf(-0.5f * x * x);
        case 1: return x > 0.f ? 1.f : 0.f;
        case 2: return 2.f * fmaxf(x, 0.f);
        default: { const float s = 1.f / (1.f + __expf(-x)); return s * (1.f + x * (1.f - s)); }
    }
}

// rows limited by meta[1] when meta != nullptr (padded expert rows), else by `rows`.  A thread handles 8 consecutive
// elements (16-byte loads and stores); SWIGLU is a template parameter so the common case carries no per-element switch.
// store 8 quantised values of one thread (a quarter of a 32-element block) + the block's scale byte from its first lane
__device__ __forceinline__ void emit_quantized8(const uint4& stored, bool active, uint8_t* q, uint8_t* sf, long long row, int col, int width,
                                                int k_blocks) {
    float v[8];
    unpack8(stored, v);
    uint32_t out[2];
    const uint32_t e8 = quantize_block_lanes<8>(v, out);
    if (active) {
        *reinterpret_cast<uint2*>(q + row * width + col) = make_uint2(out[0], out[1]);
        if ((threadIdx.x & 3) == 0) sf[sf_offset(row, col >> 5, k_blocks)] = static_cast<uint8_t>(e8);
    }
}

template <bool SWIGLU>
__global__ void __launch_bounds__(256)
activation_fwd_kernel(const __nv_bfloat16* __restrict__ pre, __nv_bfloat16* __restrict__ act, const int* __restrict__ meta,
                      uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int rows, int h, int kind) {
    const int total = meta ? min(meta[1], rows) : rows;
    const int per_row = h / 8;
    const long long n = static_cast<long long>(total) * per_row;
    const int in_w = SWIGLU ? 2 * h : h;
    const int k_blocks = (h + 127) >> 7;
    // warp-uniform trip count (the quantiser shuffles inside 4-lane groups; h % 32 == 0 keeps a group inside one row)
    for (long long base = blockIdx.x * static_cast<long long>(blockDim.x) + (threadIdx.x & ~31); base < n; base += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long i = base + (threadIdx.x & 31);
        const bool active = i < n;
        const long long r = active ? i / per_row : 0;
        const int c = active ? static_cast<int>(i - r * per_row) * 8 : 0;
        uint4 stored = make_uint4(0, 0, 0, 0);
        if (active) {
            float a[8], o[8];
            unpack8(*reinterpret_cast<const uint4*>(pre + r * in_w + c), a);
            if (SWIGLU) {
                float u[8];
                unpack8(*reinterpret_cast<const uint4*>(pre + r * in_w + h + c), u);
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = a[j] / (1.f + __expf(-a[j])) * u[j];
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = act_fwd(kind, a[j]);
            }
            stored = pack8(o);
            *reinterpret_cast<uint4*>(act + r * h + c) = stored;
        }
        if (q != nullptr) emit_quantized8(stored, active, q, sf, r, c, h, k_blocks);
    }
}

template <bool SWIGLU>
__global__ void __launch_bounds__(256)
activation_bwd_kernel(const __nv_bfloat16* __restrict__ dact, const __nv_bfloat16* __restrict__ pre, __nv_bfloat16* __restrict__ dpre,
                      const int* __restrict__ meta, uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int rows, int h, int kind) {
    const int total = meta ? min(meta[1], rows) : rows;
    const int per_row = h / 8;
    const long long n = static_cast<long long>(total) * per_row;
    const int in_w = SWIGLU ? 2 * h : h;
    const int k_blocks = (in_w + 127) >> 7;
    for (long long base = blockIdx.x * static_cast<long long>(blockDim.x) + (threadIdx.x & ~31); base < n; base += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long i = base + (threadIdx.x & 31);
        const bool active = i < n;
        const long long r = active ? i / per_row : 0;
        const int c = active ? static_cast<int>(i - r * per_row) * 8 : 0;
        uint4 s0 = make_uint4(0, 0, 0, 0), s1 = s0;
        if (active) {
            float g[8], a[8], d0[8];
            unpack8(*reinterpret_cast<const uint4*>(dact + r * h + c), g);
            unpack8(*reinterpret_cast<const uint4*>(pre + r * in_w + c), a);
            if (SWIGLU) {
                float u[8], d1[8];
                unpack8(*reinterpret_cast<const uint4*>(pre + r * in_w + h + c), u);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float sg = 1.f / (1.f + __expf(-a[j]));
                    d0[j] = g[j] * u[j] * sg * (1.f + a[j] * (1.f - sg));      // d/d(gate): up * silu'(gate)
                    d1[j] = g[j] * a[j] * sg;                                    // d/d(up):   silu(gate)
                }
                s1 = pack8(d1);
                *reinterpret_cast<uint4*>(dpre + r * in_w + h + c) = s1;
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) d0[j] = g[j] * act_grad(kind, a[j]);
            }
            s0 = pack8(d0);
            *reinterpret_cast<uint4*>(dpre + r * in_w + c) = s0;
        }
        if (q != nullptr) {
            emit_quantized8(s0, active, q, sf, r, c, in_w, k_blocks);
            if (SWIGLU) emit_quantized8(s1, active, q, sf, r, h + c, in_w, k_blocks);
        }
    }
}

void launch_activation_fwd(const void* pre, void* act, const int* meta, void* q, void* sf, int rows, int h, int kind, cudaStream_t s) {
    auto* qp = static_cast<uint8_t*>(q);
    auto* sp = static_cast<uint8_t*>(sf);
    if (kind == 4)
        activation_fwd_kernel<true><<<2368, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(pre), static_cast<__nv_bfloat16*>(act), meta, qp, sp, rows, h, kind);
    else
        activation_fwd_kernel<false><<<2368, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(pre), static_cast<__nv_bfloat16*>(act), meta, qp, sp, rows, h, kind);
}
void launch_activation_bwd(const void* dact, const void* pre, void* dpre, const int* meta, void* q, void* sf, int rows, int h, int kind,
                           cudaStream_t s) {
    auto* qp = static_cast<uint8_t*>(q);
    auto* sp = static_cast<uint8_t*>(sf);
    if (kind == 4)
        activation_bwd_kernel<true><<<2368, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dact), static_cast<const __nv_bfloat16*>(pre),
                                                         static_cast<__nv_bfloat16*>(dpre), meta, qp, sp, rows, h, kind);
    else
        activation_bwd_kernel<false><<<2368, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(dact), static_cast<const __nv_bfloat16*>(pre),
                                                          static_cast<__nv_bfloat16*>(dpre), meta, qp, sp, rows, h, kind);
}

GM_DEFINE_BOUNDS_READER(moe)

}  // namespace gm

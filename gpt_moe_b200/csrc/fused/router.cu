// The MoE router after its (tiny) logits GEMM, as one forward and one backward kernel: fp32 softmax over the experts,
// top-k selection, gate weights, and the statistics of the Switch-style load-balance loss.
//
//   probs  = softmax(float(logits))                                            [tokens, E]
//   top-k  = the k largest logits (ties: lowest expert index)
//   gates  = probs[top]                      for k = 1 or full-softmax gating
//          = softmax(logits[top])            otherwise (renormalised over the selection)
//   balance = E * sum_e (count_e / (tokens * k)) * (sum_t probs[t, e] / tokens)
// Reference: model/feedforward/moe.py:55-88 (router linear -> .float() -> topk -> gates -> balance loss), done there with
// a chain of torch ops.  One warp owns a token; lane l holds experts l, l + 32, l + 64, l + 96 (E <= 128).  The per-expert
// sums are reduced deterministically: per-block partials in shared memory (fixed warp order), then a column sum.
// Backward recomputes the probabilities from the saved logits:
//   d probs[e]  = dgate (chosen experts, gather form) + dbalance * E * f_e / tokens
//   d logits    = probs * (d probs - <probs, d probs>)  (+ the renormalised-gate softmax backward on the chosen logits)
#include "../common/ptx.cuh"
#include "../kernels_decl.h"

namespace gm {

constexpr int ROUTER_WARPS = 8;
constexpr int ROUTER_MAX_E = 128;
constexpr int ROUTER_MAX_K = 8;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_add(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// register arrays are indexed through these (a run-time subscript would send them to local memory)
__device__ __forceinline__ float get4(const float (&a)[4], int j) { return j == 0 ? a[0] : j == 1 ? a[1] : j == 2 ? a[2] : a[3]; }
__device__ __forceinline__ void set4(float (&a)[4], int j, float v) {
#pragma unroll
    for (int i = 0; i < 4; ++i) if (i == j) a[i] = v;
}
__device__ __forceinline__ void add4(float (&a)[4], int j, float v) {
#pragma unroll
    for (int i = 0; i < 4; ++i) if (i == j) a[i] += v;
}

// logits of one token into the lanes: z[j] = logit of expert lane + 32 j (-inf beyond E)
template <typename T>
__device__ __forceinline__ void load_row(const T* row, int experts, int lane, float (&z)[4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int e = lane + 32 * j;
        z[j] = e < experts ? to_f32<T>(row[e]) : -INFINITY;
    }
}

// the k largest of the warp's values, ties to the lowest index; sel_idx / sel_val are identical on every lane
__device__ __forceinline__ void select_top_k(const float (&z)[4], int lane, int top_k, int (&sel_idx)[ROUTER_MAX_K], float (&sel_val)[ROUTER_MAX_K]) {
    float w[4] = {z[0], z[1], z[2], z[3]};
#pragma unroll
    for (int s = 0; s < ROUTER_MAX_K; ++s) {
        if (s >= top_k) break;
        float best = w[0];
        int best_e = lane;
#pragma unroll
        for (int j = 1; j < 4; ++j)
            if (w[j] > best) { best = w[j]; best_e = lane + 32 * j; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ov > best || (ov == best && oe < best_e)) { best = ov; best_e = oe; }
        }
        sel_idx[s] = best_e;
        sel_val[s] = best;
        if ((best_e & 31) == lane) set4(w, best_e >> 5, -INFINITY);      // taken: out of the next rounds
    }
}

template <typename T>
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
router_fwd_kernel(const T* __restrict__ logits, long long* __restrict__ top_idx, float* __restrict__ gates, float* __restrict__ prob_partial,
                  float* __restrict__ count_partial, int tokens, int experts, int top_k, int renormalise) {
    __shared__ float psum[ROUTER_WARPS][ROUTER_MAX_E];
    __shared__ float csum[ROUTER_WARPS][ROUTER_MAX_E];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float pacc[4] = {0.f, 0.f, 0.f, 0.f}, cacc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int t = blockIdx.x * ROUTER_WARPS + warp; t < tokens; t += gridDim.x * ROUTER_WARPS) {
        float z[4];
        load_row<T>(logits + static_cast<long long>(t) * experts, experts, lane, z);
        const float m = warp_max(fmaxf(fmaxf(z[0], z[1]), fmaxf(z[2], z[3])));
        float p[4], s = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) { p[j] = z[j] == -INFINITY ? 0.f : expf(z[j] - m); s += p[j]; }
        const float inv = 1.f / warp_add(s);
#pragma unroll
        for (int j = 0; j < 4; ++j) { p[j] *= inv; pacc[j] += p[j]; }
        int sel_idx[ROUTER_MAX_K];
        float sel_val[ROUTER_MAX_K];
        select_top_k(z, lane, top_k, sel_idx, sel_val);
        float denom = 0.f;
        if (renormalise) {
#pragma unroll
            for (int s2 = 0; s2 < ROUTER_MAX_K; ++s2)
                if (s2 < top_k) denom += expf(sel_val[s2] - sel_val[0]);      // sel_val[0] is the maximum of the selection
        }
#pragma unroll
        for (int s2 = 0; s2 < ROUTER_MAX_K; ++s2) {
            if (s2 >= top_k) break;
            const int e = sel_idx[s2];
            if ((e & 31) == lane) {
                add4(cacc, e >> 5, 1.f);
                const float g = renormalise ? expf(sel_val[s2] - sel_val[0]) / denom : get4(p, e >> 5);
                top_idx[static_cast<long long>(t) * top_k + s2] = e;
                gates[static_cast<long long>(t) * top_k + s2] = g;
            }
        }
    }
    if (prob_partial == nullptr) return;
#pragma unroll
    for (int j = 0; j < 4; ++j) { psum[warp][lane + 32 * j] = pacc[j]; csum[warp][lane + 32 * j] = cacc[j]; }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        float a = 0.f, b = 0.f;
#pragma unroll
        for (int w = 0; w < ROUTER_WARPS; ++w) { a += psum[w][e]; b += csum[w][e]; }
        prob_partial[static_cast<long long>(blockIdx.x) * experts + e] = a;
        count_partial[static_cast<long long>(blockIdx.x) * experts + e] = b;
    }
}

// balance = E * sum_e (counts[e] / slots) * (prob_sums[e] / tokens); one block, fixed order
__global__ void __launch_bounds__(128)
router_balance_kernel(const float* __restrict__ prob_sums, const float* __restrict__ counts, float* __restrict__ balance, int tokens, int experts,
                      int top_k) {
    __shared__ float red[ROUTER_MAX_E];
    const int e = threadIdx.x;
    red[e] = e < experts ? (counts[e] / (static_cast<float>(tokens) * top_k)) * (prob_sums[e] / tokens) : 0.f;
    __syncthreads();
    if (e == 0) {
        float s = 0.f;
        for (int i = 0; i < experts; ++i) s += red[i];
        *balance = s * experts;
    }
}

template <typename T>
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
router_bwd_kernel(const T* __restrict__ logits, const long long* __restrict__ top_idx, const float* __restrict__ dgates,
                  const float* __restrict__ dbalance, const float* __restrict__ counts, T* __restrict__ dlogits, int tokens, int experts,
                  int top_k, int renormalise) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // d balance / d probs[t, e] = dbalance * E * f_e / tokens, the same for every token
    float bal[4] = {0.f, 0.f, 0.f, 0.f};
    if (dbalance != nullptr) {
        const float k = *dbalance * experts / (static_cast<float>(tokens) * top_k) / tokens;
#pragma unroll
        for (int j = 0; j < 4; ++j) { const int e = lane + 32 * j; bal[j] = e < experts ? k * counts[e] : 0.f; }
    }
    for (int t = blockIdx.x * ROUTER_WARPS + warp; t < tokens; t += gridDim.x * ROUTER_WARPS) {
        float z[4];
        load_row<T>(logits + static_cast<long long>(t) * experts, experts, lane, z);
        const float m = warp_max(fmaxf(fmaxf(z[0], z[1]), fmaxf(z[2], z[3])));
        float p[4], s = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) { p[j] = z[j] == -INFINITY ? 0.f : expf(z[j] - m); s += p[j]; }
        const float inv = 1.f / warp_add(s);
        float dp[4], direct[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 4; ++j) { p[j] *= inv; dp[j] = bal[j]; }
        if (dgates != nullptr) {
            int idx[ROUTER_MAX_K];
            float dg[ROUTER_MAX_K], zs[ROUTER_MAX_K];
#pragma unroll
            for (int s2 = 0; s2 < ROUTER_MAX_K; ++s2) {
                if (s2 < top_k) {
                    idx[s2] = static_cast<int>(top_idx[static_cast<long long>(t) * top_k + s2]);
                    if (!GM_IN_BOUNDS(idx[s2] >= 0 && idx[s2] < experts, 906)) idx[s2] = 0;
                    dg[s2] = dgates[static_cast<long long>(t) * top_k + s2];
                    zs[s2] = __shfl_sync(0xffffffffu, get4(z, (idx[s2] >> 5) & 3), idx[s2] & 31);
                }
            }
            if (renormalise) {
                // g = softmax(zs): d zs = g * (dg - <g, dg>), straight onto the chosen logits
                float zmax = zs[0];
#pragma unroll
                for (int s2 = 1; s2 < ROUTER_MAX_K; ++s2) if (s2 < top_k) zmax = fmaxf(zmax, zs[s2]);
                float g[ROUTER_MAX_K], den = 0.f, dot = 0.f;
#pragma unroll
                for (int s2 = 0; s2 < ROUTER_MAX_K; ++s2) if (s2 < top_k) { g[s2] = expf(zs[s2] - zmax); den += g[s2]; }
#pragma unroll
                for (int s2 = 0; s2 < ROUTER_MAX_K; ++s2) if (s2 < top_k) { g[s2] /= den; dot += g[s2] * dg[s2]; }
#pragma unroll
                for (int s2 = 0; s2 < ROUTER_MAX_K; ++s2)
                    if (s2 < top_k && (idx[s2] & 31) == lane) add4(direct, idx[s2] >> 5, g[s2] * (dg[s2] - dot));
            } else {
#pragma unroll
                for (int s2 = 0; s2 < ROUTER_MAX_K; ++s2)
                    if (s2 < top_k && (idx[s2] & 31) == lane) add4(dp, idx[s2] >> 5, dg[s2]);
            }
        }
        float inner = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) inner += p[j] * dp[j];
        inner = warp_add(inner);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int e = lane + 32 * j;
            if (e < experts) dlogits[static_cast<long long>(t) * experts + e] = from_f32<T>(p[j] * (dp[j] - inner) + direct[j]);
        }
    }
}

int router_blocks(int tokens) { return min(592, (tokens + ROUTER_WARPS - 1) / ROUTER_WARPS); }

bool launch_router_fwd(const void* logits, bool bf16, long long* top_idx, float* gates, float* prob_partial, float* count_partial,
                       float* prob_sums, float* counts, float* balance, int tokens, int experts, int top_k, int renormalise, cudaStream_t s) {
    if (experts > ROUTER_MAX_E || top_k > ROUTER_MAX_K || top_k > experts || tokens <= 0) return false;
    const int blocks = router_blocks(tokens);
    if (bf16)
        router_fwd_kernel<__nv_bfloat16><<<blocks, ROUTER_WARPS * 32, 0, s>>>(static_cast<const __nv_bfloat16*>(logits), top_idx, gates, prob_partial,
                                                                             count_partial, tokens, experts, top_k, renormalise);
    else
        router_fwd_kernel<float><<<blocks, ROUTER_WARPS * 32, 0, s>>>(static_cast<const float*>(logits), top_idx, gates, prob_partial, count_partial,
                                                                     tokens, experts, top_k, renormalise);
    if (prob_partial != nullptr) {
        launch_column_sum(prob_partial, prob_sums, blocks, experts, 0, s);
        launch_column_sum(count_partial, counts, blocks, experts, 0, s);
        router_balance_kernel<<<1, 128, 0, s>>>(prob_sums, counts, balance, tokens, experts, top_k);
    }
    return true;
}

bool launch_router_bwd(const void* logits, bool bf16, const long long* top_idx, const float* dgates, const float* dbalance, const float* counts,
                       void* dlogits, int tokens, int experts, int top_k, int renormalise, cudaStream_t s) {
    if (experts > ROUTER_MAX_E || top_k > ROUTER_MAX_K || tokens <= 0) return false;
    const int blocks = router_blocks(tokens);
    if (bf16)
        router_bwd_kernel<__nv_bfloat16><<<blocks, ROUTER_WARPS * 32, 0, s>>>(static_cast<const __nv_bfloat16*>(logits), top_idx, dgates, dbalance,
                                                                             counts, static_cast<__nv_bfloat16*>(dlogits), tokens, experts, top_k,
                                                                             renormalise);
    else
        router_bwd_kernel<float><<<blocks, ROUTER_WARPS * 32, 0, s>>>(static_cast<const float*>(logits), top_idx, dgates, dbalance, counts,
                                                                     static_cast<float*>(dlogits), tokens, experts, top_k, renormalise);
    return true;
}

GM_DEFINE_BOUNDS_READER(router)

}  // namespace gm

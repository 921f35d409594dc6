// Expert-parallel dispatch and combine fused with their all-to-all over NVLink peer memory.
//
// Experts are sharded over the W ranks of a group (rank r owns experts [r * E_local, (r + 1) * E_local)).  Every rank maps
// the others' receive / return buffers (symmetric allocation), so the all-to-all of token rows is not a separate
// collective: the kernel that gathers a token's row STORES it into the owner's receive buffer at its final position in
// the owner's padded expert-major layout (dispatch), and the kernel that applies the gates LOADS the expert outputs
// straight from the owners' return buffers (combine).  Nothing is staged or sorted on the way.
//
//   ep_push_counts   this rank's per-expert slot counts are stored into row `me` of every rank's count table
//   ep_plan          (one block) from the full W x E table every rank derives, identically, the owners' layouts:
//                    segment of expert e in its owner's buffer = rows of source 0, source 1, ..., padded to 256;
//                    emits my_base[e] (first row of MY rows for expert e) and this rank's own plan
//                    (segment ends, valid ends, tile -> local expert table, tile / row totals)
//   ep_zero_pads     zero the pad rows of the local receive buffer (between a segment's valid end and its padded end)
//   ep_dispatch      one warp per (token, slot): row -> owner's buffer, optionally scaled by the gate (backward: dY = g * dOut)
//                    and with the dot product against a saved row (backward: dGate)
//   ep_combine       one warp per token: sum over its slots of gate * row loaded from the owner's return buffer;
//                    optionally keeps the loaded rows (needed for dGate)
// Ordering across ranks comes from barriers the caller issues between the phases; no kernel here waits on a peer.
// Only plain loads and stores touch peer memory.  The reference keeps every expert on every rank
// (model/feedforward/moe.py:30) and has no counterpart.
#include "../common/ptx.cuh"
#include "../kernels_decl.h"

#include <algorithm>

namespace gm {

constexpr int EP_MAX_RANKS = 16;
constexpr int EP_MAX_EXPERTS = 128;
constexpr int EP_SEG_PAD = 256;           // same unit as the local routing: a CTA pair of the GEMM owns 256 rows of one expert
struct EpDeltas { long long d[EP_MAX_RANKS]; };

__global__ void ep_push_counts_kernel(const int* __restrict__ counts, int* __restrict__ table, EpDeltas peers, int world, int me, int experts) {
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= experts) return;
    const int c = counts[e];
    for (int r = 0; r < world; ++r)
        *reinterpret_cast<int*>(reinterpret_cast<char*>(table + me * experts + e) + peers.d[r]) = c;
}

// plan[0 .. E)                      my_base
// local_plan: seg_ends[E_local], valid_ends[E_local]; tile_expert[cap / 128]; meta = {tiles, padded rows}
__global__ void __launch_bounds__(EP_MAX_EXPERTS)
ep_plan_kernel(const int* __restrict__ table, int* __restrict__ my_base, int* __restrict__ seg_ends, int* __restrict__ valid_ends,
               int* __restrict__ tile_expert, int* __restrict__ meta, int world, int me, int experts, int per_rank, int cap_rows,
               int* __restrict__ status) {
    __shared__ int total[EP_MAX_EXPERTS], before[EP_MAX_EXPERTS], start[EP_MAX_EXPERTS];
    const int e = threadIdx.x;
    if (e < experts) {
        int t = 0, b = 0;
        for (int s = 0; s < world; ++s) {
            const int c = table[s * experts + e];
            if (s < me) b += c;
            t += c;
        }
        total[e] = t;
        before[e] = b;
    }
    __syncthreads();
    if (e < experts) {
        const int first = e / per_rank * per_rank;
        int s = 0;
        for (int j = first; j < e; ++j) s += (total[j] + EP_SEG_PAD - 1) / EP_SEG_PAD * EP_SEG_PAD;
        start[e] = s;
        my_base[e] = s + before[e];
    }
    __syncthreads();
    const int lo = me * per_rank;
    if (e < per_rank) {
        const int g = lo + e;
        const int padded = (total[g] + EP_SEG_PAD - 1) / EP_SEG_PAD * EP_SEG_PAD;
        seg_ends[e] = min(start[g] + padded, cap_rows);
        valid_ends[e] = min(start[g] + total[g], cap_rows);
        for (int t = start[g] / 128; t < (start[g] + padded) / 128 && t < cap_rows / 128; ++t) tile_expert[t] = e;
    }
    if (e == 0) {
        const int last = lo + per_rank - 1;
        int rows = start[last] + (total[last] + EP_SEG_PAD - 1) / EP_SEG_PAD * EP_SEG_PAD;
        if (rows > cap_rows) { atomicExch(status, 501); rows = cap_rows / EP_SEG_PAD * EP_SEG_PAD; }
        meta[0] = rows / 128;
        meta[1] = rows;
    }
}

__global__ void __launch_bounds__(256)
ep_zero_pads_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ seg_ends, const int* __restrict__ valid_ends, int d) {
    const int j = blockIdx.y;
    const int lo = valid_ends[j], hi = seg_ends[j];
    const int lane = threadIdx.x & 31;
    for (int row = lo + blockIdx.x * 8 + (threadIdx.x >> 5); row < hi; row += gridDim.x * 8) {
        uint4* out = reinterpret_cast<uint4*>(buf + static_cast<long long>(row) * d);
        for (int i = lane; i < d / 8; i += 32) out[i] = make_uint4(0, 0, 0, 0);
    }
}

// slot i = (token i / k, choice i % k) with expert idx[i]; `dest[i]` is the slot's position in this rank's own padded
// expert-major order and `local_seg_ends` the ends of those segments, so dest[i] - start(e) counts the slot among this
// rank's slots for the expert.
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(const __nv_bfloat16* __restrict__ src, const long long* __restrict__ idx, const int* __restrict__ dest,
                   const int* __restrict__ local_seg_ends, const int* __restrict__ my_base, const float* __restrict__ gates,
                   const __nv_bfloat16* __restrict__ saved_rows, float* __restrict__ dgates, __nv_bfloat16* __restrict__ recv,
                   int* __restrict__ route_row, EpDeltas peers, int slots, int d, int top_k, int per_rank, int cap_rows,
                   int* __restrict__ status) {
    const int lane = threadIdx.x & 31;
    for (int i = blockIdx.x * 8 + (threadIdx.x >> 5); i < slots; i += gridDim.x * 8) {
        const int e = static_cast<int>(idx[i]);
        const int within = dest[i] - (e ? local_seg_ends[e - 1] : 0);
        const int row = my_base[e] + within;
        if (route_row && lane == 0) route_row[i] = row;
        const uint4* in = reinterpret_cast<const uint4*>(src + static_cast<long long>(i / top_k) * d);
        const float g = gates ? gates[i] : 1.f;
        float dot = 0.f;
        const bool in_range = row < cap_rows;
        if (!in_range && lane == 0) atomicExch(status, 502);
        uint4* out = reinterpret_cast<uint4*>(reinterpret_cast<char*>(recv + static_cast<long long>(row) * d) + peers.d[e / per_rank]);
        const uint4* sv = saved_rows ? reinterpret_cast<const uint4*>(saved_rows + static_cast<long long>(i) * d) : nullptr;
        for (int c = lane; c < d / 8; c += 32) {
            uint4 raw = in[c];
            if (gates) {
                __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
                uint4 s4 = sv ? sv[c] : make_uint4(0, 0, 0, 0);
                const __nv_bfloat162* s = reinterpret_cast<const __nv_bfloat162*>(&s4);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 f = __bfloat1622float2(h[q]);
                    const float2 y = __bfloat1622float2(s[q]);
                    dot += f.x * y.x + f.y * y.y;
                    h[q] = __floats2bfloat162_rn(f.x * g, f.y * g);
                }
            }
            if (in_range) out[c] = raw;
        }
        if (dgates) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
            if (lane == 0) dgates[i] = dot;
        }
    }
}

__global__ void __launch_bounds__(256)
ep_combine_kernel(const __nv_bfloat16* __restrict__ ret, const long long* __restrict__ idx, const int* __restrict__ route_row,
                  const float* __restrict__ gates, __nv_bfloat16* __restrict__ out, __nv_bfloat16* __restrict__ keep_rows, EpDeltas peers,
                  int tokens, int d, int top_k, int per_rank, int cap_rows) {
    const int lane = threadIdx.x & 31;
    for (int t = blockIdx.x * 8 + (threadIdx.x >> 5); t < tokens; t += gridDim.x * 8) {
        for (int c = lane; c < d / 8; c += 32) {
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int k = 0; k < top_k; ++k) {
                const int i = t * top_k + k;
                const int row = route_row[i];
                uint4 raw = make_uint4(0, 0, 0, 0);
                if (row < cap_rows)
                    raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(ret + static_cast<long long>(row) * d + c * 8) +
                                                          peers.d[static_cast<int>(idx[i]) / per_rank]);
                if (keep_rows) *reinterpret_cast<uint4*>(keep_rows + static_cast<long long>(i) * d + c * 8) = raw;
                const float g = gates ? gates[i] : 1.f;
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float2 f = __bfloat1622float2(h[q]);
                    acc[2 * q] += g * f.x;
                    acc[2 * q + 1] += g * f.y;
                }
            }
            uint4 o;
            o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
            o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
            *reinterpret_cast<uint4*>(out + static_cast<long long>(t) * d + c * 8) = o;
        }
    }
}

static bool ep_deltas(EpDeltas& out, const long long* deltas, int world) {
    if (world < 1 || world > EP_MAX_RANKS) return false;
    for (int i = 0; i < EP_MAX_RANKS; ++i) out.d[i] = i < world ? deltas[i] : 0;
    return true;
}

bool launch_ep_push_counts(const int* counts, int* table, const long long* deltas, int world, int me, int experts, cudaStream_t s) {
    EpDeltas p;
    if (!ep_deltas(p, deltas, world) || experts > EP_MAX_EXPERTS) return false;
    ep_push_counts_kernel<<<1, EP_MAX_EXPERTS, 0, s>>>(counts, table, p, world, me, experts);
    return true;
}

bool launch_ep_plan(const int* table, int* my_base, int* seg_ends, int* valid_ends, int* tile_expert, int* meta, int world, int me,
                    int experts, int per_rank, int cap_rows, int* status, cudaStream_t s) {
    if (experts > EP_MAX_EXPERTS || world > EP_MAX_RANKS || per_rank * world != experts) return false;
    ep_plan_kernel<<<1, EP_MAX_EXPERTS, 0, s>>>(table, my_base, seg_ends, valid_ends, tile_expert, meta, world, me, experts, per_rank, cap_rows, status);
    return true;
}

void launch_ep_zero_pads(void* buf, const int* seg_ends, const int* valid_ends, int per_rank, int d, cudaStream_t s) {
    ep_zero_pads_kernel<<<dim3(4, per_rank), 256, 0, s>>>(static_cast<__nv_bfloat16*>(buf), seg_ends, valid_ends, d);
}

bool launch_ep_dispatch(const void* src, const long long* idx, const int* dest, const int* local_seg_ends, const int* my_base,
                        const float* gates, const void* saved_rows, float* dgates, void* recv, int* route_row, const long long* deltas,
                        int world, int slots, int d, int top_k, int per_rank, int cap_rows, int* status, cudaStream_t s) {
    EpDeltas p;
    if (!ep_deltas(p, deltas, world) || d % 8) return false;
    const int blocks = std::min((slots + 7) / 8, 148 * 8);
    if (blocks > 0)
        ep_dispatch_kernel<<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(src), idx, dest, local_seg_ends, my_base, gates,
                                                  static_cast<const __nv_bfloat16*>(saved_rows), dgates, static_cast<__nv_bfloat16*>(recv),
                                                  route_row, p, slots, d, top_k, per_rank, cap_rows, status);
    return true;
}

bool launch_ep_combine(const void* ret, const long long* idx, const int* route_row, const float* gates, void* out, void* keep_rows,
                       const long long* deltas, int world, int tokens, int d, int top_k, int per_rank, int cap_rows, cudaStream_t s) {
    EpDeltas p;
    if (!ep_deltas(p, deltas, world) || d % 8) return false;
    const int blocks = std::min((tokens + 7) / 8, 148 * 8);
    if (blocks > 0)
        ep_combine_kernel<<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(ret), idx, route_row, gates, static_cast<__nv_bfloat16*>(out),
                                                 static_cast<__nv_bfloat16*>(keep_rows), p, tokens, d, top_k, per_rank, cap_rows);
    return true;
}

}  // namespace gm

// Optimizer kernels fused with their collectives over NVLink peer memory.
//
// Every rank maps every other rank's gradient / weight buffers (symmetric allocation: the same offset means the same
// tensor on every GPU), so a kernel reaches a peer's copy as `local pointer + delta[rank]`.  Three kernels replace
// "reduce-scatter, optimizer, all-gather":
//   rs_muon_prepare   the owner of a matrix SUMS that matrix's gradient straight out of all ranks' buffers (plain P2P
//                     loads = the reduce-scatter), averages, applies momentum / Nesterov, packs bf16 (transposed when
//                     tall) and accumulates the Frobenius norm — the input of Polar Express
//   muon_apply_push   W_master += alpha * O on the owner, and the refreshed bf16 GEMM copy is STORED into every rank's
//                     weight buffer (P2P stores = the all-gather); nothing is staged
//   adamw_sharded     each rank owns a slice of the flat AdamW parameters: sum of all ranks' gradients for the slice,
//                     AdamW on the slice, new fp32 values stored into every rank's parameter buffer
// Cross-rank ordering (gradients complete before they are read, pushes complete before the next forward) is provided by
// barriers between the kernels, issued by the engine.  No multicast / cluster loads are used on peer memory.
// The reference has no counterpart: its DDP all-reduces every gradient and then repeats the full optimizer on every
// rank (train.py:213-215, optimizers/muon.py:147-224).
#include "../common/ptx.cuh"
#include "../kernels_decl.h"

namespace gm {

constexpr int MAX_RANKS = 16;
struct PeerDeltas { long long d[MAX_RANKS]; };

__device__ __forceinline__ float4 ld_peer4(const float* p, long long delta) {
    return *reinterpret_cast<const float4*>(reinterpret_cast<const char*>(p) + delta);
}

// Sum of the same float4 on every rank, added in rank order.  The loads of up to eight ranks are issued before any of them
// is consumed, so a thread keeps eight NVLink requests in flight instead of one.
__device__ __forceinline__ float4 sum_peers4(const float* p, const PeerDeltas& peers, int world) {
    if (world == 1) return ld_peer4(p, peers.d[0]);          // one GPU: a plain load, no batch of predicated slots
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int base = 0; base < world; base += 8) {
        float4 t[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
            t[k] = (base + k < world) ? ld_peer4(p, peers.d[base + k]) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < 8; ++k) { s.x += t[k].x; s.y += t[k].y; s.z += t[k].z; s.w += t[k].w; }
    }
    return s;
}

// bf16 wire format: every rank keeps a bf16 shadow of its gradient buffer (same element offsets); a peer's contribution is
// read from its shadow (half the NVLink bytes), this rank's own from its fp32 buffer; the sum is formed in fp32 in rank order.
__device__ __forceinline__ float4 ld_peer4_bf16(const __nv_bfloat16* p, long long delta) {
    const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const char*>(p) + delta);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ float4 sum_peers4_bf16(const float* own, const __nv_bfloat16* shadow, const PeerDeltas& peers, int world) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int base = 0; base < world; base += 8) {
        float4 t[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (base + k >= world) t[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            else if (peers.d[base + k] == 0) t[k] = *reinterpret_cast<const float4*>(own);
            else t[k] = ld_peer4_bf16(shadow, peers.d[base + k]);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) { s.x += t[k].x; s.y += t[k].y; s.z += t[k].z; s.w += t[k].w; }
    }
    return s;
}

// tile: 32 rows x 128 columns, 256 threads; thread (tx, ty) owns columns 4*tx..4*tx+3 of rows ty, ty+8, ty+16, ty+24
// `shadow_gap` != 0 selects the bf16 wire: the bf16 shadow of gradient element i of this rank's flat buffer sits at
// shadow_base + i, where shadow_base - grad_base (in bytes, through `shadow_gap` and the element index) is uniform; `peers`
// then holds the deltas of the SHADOW buffers.
__global__ void __launch_bounds__(256)
rs_muon_prepare_kernel(const float* const* __restrict__ grads, float* const* __restrict__ bufs, __nv_bfloat16* __restrict__ packed,
                       float* __restrict__ sumsq, int rows, int cols, long long g_stride, long long b_stride, float momentum,
                       int nesterov, int transpose, PeerDeltas peers, int world, float inv_world,
                       const float* grad_base, const __nv_bfloat16* shadow_base) {
    __shared__ float tile[32][132];
    __shared__ float part[8];
    const int mat = blockIdx.z;
    const float* g = grads[mat];
    float* buf = bufs[mat];
    __nv_bfloat16* out = packed + static_cast<long long>(mat) * rows * cols;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c0 = blockIdx.x * 128, r0 = blockIdx.y * 32;
    float local = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + ty + 8 * i, c = c0 + 4 * tx;
        float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < rows && c < cols) {
            const float* gp = g + r * g_stride + c;
            float4 s = shadow_base ? sum_peers4_bf16(gp, shadow_base + (gp - grad_base), peers, world) : sum_peers4(gp, peers, world);
            s.x *= inv_world; s.y *= inv_world; s.z *= inv_world; s.w *= inv_world;
            float4 b = *reinterpret_cast<const float4*>(buf + r * b_stride + c);
            b.x = b.x * momentum + s.x; b.y = b.y * momentum + s.y; b.z = b.z * momentum + s.z; b.w = b.w * momentum + s.w;
            *reinterpret_cast<float4*>(buf + r * b_stride + c) = b;
            if (nesterov) { u.x = fmaf(momentum, b.x, s.x); u.y = fmaf(momentum, b.y, s.y); u.z = fmaf(momentum, b.z, s.z); u.w = fmaf(momentum, b.w, s.w); }
            else u = b;
            const __nv_bfloat162 lo = __floats2bfloat162_rn(u.x, u.y), hi = __floats2bfloat162_rn(u.z, u.w);
            const float2 flo = __bfloat1622float2(lo), fhi = __bfloat1622float2(hi);
            u = make_float4(flo.x, flo.y, fhi.x, fhi.y);               // the rounded values are what Polar Express sees
            if (!transpose) {
                uint2 w;
                w.x = *reinterpret_cast<const uint32_t*>(&lo);
                w.y = *reinterpret_cast<const uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(out + static_cast<long long>(r) * cols + c) = w;
            }
        }
        tile[ty + 8 * i][4 * tx] = u.x; tile[ty + 8 * i][4 * tx + 1] = u.y; tile[ty + 8 * i][4 * tx + 2] = u.z; tile[ty + 8 * i][4 * tx + 3] = u.w;
        local += u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
    }
    if (transpose) {
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const int c = c0 + ty + 8 * i, r = r0 + tx;              // out is [cols][rows]
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

__global__ void __launch_bounds__(256)
muon_apply_push_kernel(float* const* __restrict__ weights, __nv_bfloat16* const* __restrict__ weights_bf16,
                       const __nv_bfloat16* __restrict__ update, int rows, int cols, long long w_stride, long long wb_stride,
                       float alpha, int transpose, PeerDeltas peers, int world) {
    __shared__ float tile[128][33];
    const int mat = blockIdx.z;
    float* w = weights[mat];
    __nv_bfloat16* wb = weights_bf16[mat];
    const __nv_bfloat16* o = update + static_cast<long long>(mat) * rows * cols;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c0 = blockIdx.x * 128, r0 = blockIdx.y * 32;
    if (transpose) {                                                 // update is [cols][rows]: stage the 128 x 32 block
        if ((rows & 3) == 0) {                                       // 8-byte loads: four consecutive rows of one column
            const int r4 = (threadIdx.x & 7) * 4, cl0 = threadIdx.x >> 3;          // 8 threads cover 32 rows; 32 columns per pass
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int cl = cl0 + 32 * i, c = c0 + cl, r = r0 + r4;
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (c < cols && r < rows) {
                    const uint2 raw = *reinterpret_cast<const uint2*>(o + static_cast<long long>(c) * rows + r);
                    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                    v = make_float4(a.x, a.y, b.x, b.y);
                }
                tile[cl][r4] = v.x; tile[cl][r4 + 1] = v.y; tile[cl][r4 + 2] = v.z; tile[cl][r4 + 3] = v.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int c = c0 + ty + 8 * i, r = r0 + tx;
                tile[ty + 8 * i][tx] = (r < rows && c < cols) ? __bfloat162float(o[static_cast<long long>(c) * rows + r]) : 0.f;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int rl = ty + 8 * i, r = r0 + rl, c = c0 + 4 * tx;
        if (r < rows && c < cols) {
            float4 upd;
            if (transpose) {
                upd = make_float4(tile[4 * tx][rl], tile[4 * tx + 1][rl], tile[4 * tx + 2][rl], tile[4 * tx + 3][rl]);
            } else {
                const uint2 raw = *reinterpret_cast<const uint2*>(o + static_cast<long long>(r) * cols + c);
                const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                upd = make_float4(a.x, a.y, b.x, b.y);
            }
            float4 cur = *reinterpret_cast<const float4*>(w + r * w_stride + c);
            cur.x += alpha * upd.x; cur.y += alpha * upd.y; cur.z += alpha * upd.z; cur.w += alpha * upd.w;
            *reinterpret_cast<float4*>(w + r * w_stride + c) = cur;
            uint2 q;
            q.x = pack_bf16x2(cur.x, cur.y);
            q.y = pack_bf16x2(cur.z, cur.w);
            char* dst = reinterpret_cast<char*>(wb + r * wb_stride + c);
            for (int k = 0; k < world; ++k) *reinterpret_cast<uint2*>(dst + peers.d[k]) = q;      // local copy and every peer's copy
        }
    }
}

// slice [lo, lo + n) of the flat AdamW parameter / gradient buffers (n and lo multiples of 4)
template <typename TM>
__global__ void __launch_bounds__(256)
adamw_sharded_kernel(float* __restrict__ params, const float* __restrict__ grads, TM* __restrict__ m, TM* __restrict__ v,
                     const float* __restrict__ decay, long long lo, long long n, float lr, float beta1, float beta2, float eps,
                     float bc1, float bc2_sqrt, PeerDeltas gpeers, PeerDeltas ppeers, int world, float inv_world) {
    for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
        const float* gp = grads + lo + i;
        const float4 g = sum_peers4(gp, gpeers, world);
        const float gg[4] = {g.x * inv_world, g.y * inv_world, g.z * inv_world, g.w * inv_world};
        float4 pw = *reinterpret_cast<const float4*>(params + lo + i);
        float pp[4] = {pw.x, pw.y, pw.z, pw.w};
        const float4 wd4 = *reinterpret_cast<const float4*>(decay + lo + i);      // per-element weight decay (0 for no-decay groups)
        const float wd[4] = {wd4.x, wd4.y, wd4.z, wd4.w};
        // the four moments of this thread travel as one 16-byte (fp32) or 8-byte (bf16) access each way
        float mm[4], vv[4];
        if constexpr (sizeof(TM) == 4) {
            const float4 m4 = *reinterpret_cast<const float4*>(m + i), v4 = *reinterpret_cast<const float4*>(v + i);
            mm[0] = m4.x; mm[1] = m4.y; mm[2] = m4.z; mm[3] = m4.w;
            vv[0] = v4.x; vv[1] = v4.y; vv[2] = v4.z; vv[3] = v4.w;
        } else {
            const uint2 mr = *reinterpret_cast<const uint2*>(m + i), vr = *reinterpret_cast<const uint2*>(v + i);
            const float2 m01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&mr.x)), m23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&mr.y));
            const float2 v01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vr.x)), v23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&vr.y));
            mm[0] = m01.x; mm[1] = m01.y; mm[2] = m23.x; mm[3] = m23.y;
            vv[0] = v01.x; vv[1] = v01.y; vv[2] = v23.x; vv[3] = v23.y;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float mi = beta1 * mm[e] + (1.f - beta1) * gg[e];
            const float vi = beta2 * vv[e] + (1.f - beta2) * gg[e] * gg[e];
            mm[e] = mi; vv[e] = vi;
            float x = pp[e] * (1.f - lr * wd[e]);
            x -= lr / bc1 * mi / (sqrtf(vi) / bc2_sqrt + eps);
            pp[e] = x;
        }
        if constexpr (sizeof(TM) == 4) {
            *reinterpret_cast<float4*>(m + i) = make_float4(mm[0], mm[1], mm[2], mm[3]);
            *reinterpret_cast<float4*>(v + i) = make_float4(vv[0], vv[1], vv[2], vv[3]);
        } else {
            uint2 mo, vo;
            mo.x = pack_bf16x2(mm[0], mm[1]); mo.y = pack_bf16x2(mm[2], mm[3]);
            vo.x = pack_bf16x2(vv[0], vv[1]); vo.y = pack_bf16x2(vv[2], vv[3]);
            *reinterpret_cast<uint2*>(m + i) = mo;
            *reinterpret_cast<uint2*>(v + i) = vo;
        }
        const float4 nw = make_float4(pp[0], pp[1], pp[2], pp[3]);
        char* dst = reinterpret_cast<char*>(params + lo + i);
        for (int k = 0; k < world; ++k) *reinterpret_cast<float4*>(dst + ppeers.d[k]) = nw;
    }
}

static PeerDeltas make_deltas(const long long* deltas, int world) {
    PeerDeltas p;
    for (int i = 0; i < MAX_RANKS; ++i) p.d[i] = i < world ? deltas[i] : 0;
    return p;
}

bool launch_rs_muon_prepare(const float* const* grads, float* const* bufs, void* packed, float* sumsq, int n_mats, int rows, int cols,
                            long long g_stride, long long b_stride, float momentum, int nesterov, int transpose,
                            const long long* peer_deltas, int world, const float* grad_base, const void* shadow_base, cudaStream_t s) {
    if (world > MAX_RANKS || cols % 4) return false;
    if (n_mats == 0) return true;
    dim3 grid((cols + 127) / 128, (rows + 31) / 32, n_mats);
    rs_muon_prepare_kernel<<<grid, 256, 0, s>>>(grads, bufs, static_cast<__nv_bfloat16*>(packed), sumsq, rows, cols, g_stride, b_stride,
                                                momentum, nesterov, transpose, make_deltas(peer_deltas, world), world, 1.f / world,
                                                grad_base, static_cast<const __nv_bfloat16*>(shadow_base));
    return true;
}

bool launch_muon_apply_push(float* const* weights, void* const* weights_bf16, const void* update, int n_mats, int rows, int cols,
                            long long w_stride, long long wb_stride, float alpha, int transpose, const long long* peer_deltas, int world,
                            cudaStream_t s) {
    if (world > MAX_RANKS || cols % 4) return false;
    dim3 grid((cols + 127) / 128, (rows + 31) / 32, n_mats);
    muon_apply_push_kernel<<<grid, 256, 0, s>>>(weights, reinterpret_cast<__nv_bfloat16* const*>(weights_bf16),
                                                static_cast<const __nv_bfloat16*>(update), rows, cols, w_stride, wb_stride, alpha, transpose,
                                                make_deltas(peer_deltas, world), world);
    return true;
}

bool launch_adamw_sharded(float* params, const float* grads, void* m, void* v, bool moments_bf16, const float* decay, long long lo,
                          long long n, float lr, float beta1, float beta2, float eps, float bc1, float bc2_sqrt,
                          const long long* grad_deltas, const long long* param_deltas, int world, cudaStream_t s) {
    if (world > MAX_RANKS || (n % 4) || (lo % 4)) return false;
    if (n == 0) return true;
    const int blocks = static_cast<int>((n / 4 + 255) / 256 < 1184 ? (n / 4 + 255) / 256 : 1184);
    const PeerDeltas gp = make_deltas(grad_deltas, world), pp = make_deltas(param_deltas, world);
    if (moments_bf16)
        adamw_sharded_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(params, grads, static_cast<__nv_bfloat16*>(m), static_cast<__nv_bfloat16*>(v),
                                                                   decay, lo, n, lr, beta1, beta2, eps, bc1, bc2_sqrt, gp, pp, world, 1.f / world);
    else
        adamw_sharded_kernel<float><<<blocks, 256, 0, s>>>(params, grads, static_cast<float*>(m), static_cast<float*>(v), decay, lo, n, lr,
                                                           beta1, beta2, eps, bc1, bc2_sqrt, gp, pp, world, 1.f / world);
    return true;
}

// ---- cross-rank readiness flags and barrier -------------------------------------------------------------------------------
// flags[slot * world + src] on every rank holds the last step for which rank `src` has finished producing the data of `slot`
// (the gradients of one transformer block).  flag_signal publishes this rank's value to every rank after a system-scope
// fence; flag_wait polls this rank's own copy until every source has reached `value`.  The value is a kernel argument or,
// when `value_word` is given, read from device memory (a step counter bumped on the device: the launches then carry no
// host state and can be replayed from a CUDA graph).  The poll is bounded: when the budget runs out the kernel records
// code 601 in the status word and returns, so a missing peer fails the step instead of hanging the GPU.  Kernels that
// wait for one another always run on different GPUs.
__global__ void flag_signal_kernel(int* flags, PeerDeltas peers, int world, int index, int value, const int* value_word) {
    const int r = threadIdx.x;
    if (r < world) {
        const int v = value_word ? *value_word : value;
        __threadfence_system();
        *reinterpret_cast<volatile int*>(reinterpret_cast<char*>(flags + index) + peers.d[r]) = v;
    }
}

__global__ void flag_wait_kernel(const int* flags, int first, int world, int value, const int* value_word, int* status) {
    const int r = threadIdx.x;
    if (r < world) {
        const int v = value_word ? *value_word : value;
        const volatile int* f = flags + first + r;
        const long long start = clock64();
        while (*f < v) {
            if (clock64() - start > kWaitBudgetCycles) { atomicExch(status, 601); break; }
            __nanosleep(256);
        }
    }
    __threadfence_system();
}

__global__ void bump_word_kernel(int* word) { *word += 1; }

// Barrier across the ranks of a symmetric flag table, as ONE launch per rank: everything this rank queued on the stream before
// it is complete when the kernel starts; thread r publishes this rank's next epoch into slot `me` of rank r's table
// (system-scope fence first, so this rank's earlier peer stores are visible before the flag), then waits until rank r's
// epoch has arrived in this rank's own table.  The epoch lives in device memory (`epoch_word`, bumped here), so the launch
// carries no host state.  The wait is bounded like every wait in this code base: status 601 and return when a peer does
// not arrive within the budget.
__global__ void peer_barrier_kernel(int* flags, PeerDeltas peers, int world, int me, int* epoch_word, int* status, long long budget) {
    __shared__ int epoch;
    if (threadIdx.x == 0) { epoch = *epoch_word + 1; *epoch_word = epoch; }
    __syncthreads();
    const int r = threadIdx.x;
    if (r < world) {
        __threadfence_system();
        *reinterpret_cast<volatile int*>(reinterpret_cast<char*>(flags + me) + peers.d[r]) = epoch;
        const volatile int* f = flags + r;
        const long long start = clock64();
        while (*f < epoch) {
            if (clock64() - start > budget) { atomicExch(status, 601); break; }
            __nanosleep(128);
        }
    }
    __threadfence_system();
}

bool launch_flag_signal(int* flags, const long long* deltas, int world, int index, int value, const int* value_word, cudaStream_t s) {
    if (world > MAX_RANKS) return false;
    flag_signal_kernel<<<1, 32, 0, s>>>(flags, make_deltas(deltas, world), world, index, value, value_word);
    return true;
}

bool launch_flag_wait(const int* flags, int first, int world, int value, const int* value_word, int* status, cudaStream_t s) {
    if (world > MAX_RANKS) return false;
    flag_wait_kernel<<<1, 32, 0, s>>>(flags, first, world, value, value_word, status);
    return true;
}

void launch_bump_word(int* word, cudaStream_t s) { bump_word_kernel<<<1, 1, 0, s>>>(word); }

bool launch_peer_barrier(int* flags, const long long* deltas, int world, int me, int* epoch_word, int* status, long long budget_cycles,
                         cudaStream_t s) {
    if (world > MAX_RANKS || me < 0 || me >= world) return false;
    peer_barrier_kernel<<<1, 32, 0, s>>>(flags, make_deltas(deltas, world), world, me, epoch_word, status,
                                         budget_cycles > 0 ? budget_cycles : kWaitBudgetCycles);
    return true;
}

}  // namespace gm

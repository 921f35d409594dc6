// Absorbed-weight decode for multi-head latent attention: new tokens attend over the LATENT cache directly.
//
//   score[b, h, t, s] = (q_latent[b,t,h,:] . latent[b,s,:] + q_rope[b,t,h,:] . rope[b,s,:]) * key_gain[b,s,kv(h)] * scale
//   (optional soft-capping cap * tanh(score / cap); causal: s <= start + t; optional window: start + t - s <= W)
//   context[b, t, h, :] = sum_s softmax_s(score) * latent[b, s, :]                        (latent space, fp32)
// Every head of a token reads the same latent rows (keys and values are both the latent cache), so the kernel is bound by
// reading the cache once; the work is organised around that:
//   * split-K: grid = (splits, new tokens, batch); a CTA walks its share of the cache in tiles of 32 positions staged in
//     shared memory (one coalesced pass over the cache per CTA), keeps an online softmax per head, and writes an
//     un-normalised partial context + (max, sum) per head; a second kernel merges the splits by their log-sum-exp;
//   * shared tile loads: the 8 warps of a CTA own H / 8 heads each and all read the staged tile; inside a warp the heads are
//     processed together on each latent row a lane has loaded (the "paired-head" form: one load, two or more heads);
//   * lane = slice of the latent dimension (r / 32 consecutive values) for both products, so the row slice a lane loads
//     serves the score and the value accumulation; scores are completed by a warp butterfly, lane k keeps position k's.
// Reference: the Triton kernels `_mla_decode_kernel` / `_mla_decode_merge_kernel` (experiments/073-mla-current-kv768.patch:456-673)
// and the paired-head variant (experiments/051-paired-head-mla-decode.patch).
#include "../common/ptx.cuh"
#include "../kernels_decl.h"

namespace gm {

constexpr int MD_TILE = 32;          // cache positions per tile = lanes of a warp
constexpr int MD_WARPS = 8;

struct MlaDecodeParams {
    const float* q_latent;           // [B, T, H, r]
    const float* q_rope;             // [B, T, H, dr]
    const __nv_bfloat16* latent;     // [B, S, r]   (row pitch r, batch stride given)
    const __nv_bfloat16* rope;       // [B, S, dr]
    const __nv_bfloat16* key_gain;   // [B, S, Hkv]
    long long latent_bs, rope_bs, gain_bs;      // batch strides in elements
    float* part_ctx;                 // [B, T, H, splits, r]  un-normalised partial contexts
    float* part_ml;                  // [B, T, H, splits, 2]  running max (of base-e scores) and sum
    int B, T, H, Hkv, r, dr, S, splits, start, window;
    float scale, softcap;
};

__device__ __forceinline__ float wsum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float wmax(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// CHUNK = r / 32 latent values per lane (multiple of 8); HPW = heads per warp (H = 8 * HPW)
template <int CHUNK, int HPW>
__global__ void __launch_bounds__(MD_WARPS * 32)
mla_decode_split_kernel(const MlaDecodeParams p) {
    extern __shared__ __align__(16) uint8_t md_smem[];
    const int r = CHUNK * 32;
    __nv_bfloat16* lat_s = reinterpret_cast<__nv_bfloat16*>(md_smem);                       // [32][r]
    __nv_bfloat16* rope_s = lat_s + MD_TILE * r;                                            // [32][dr]
    float* gain_s = reinterpret_cast<float*>(rope_s + MD_TILE * p.dr);                      // [32][Hkv]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int split = blockIdx.x, t = blockIdx.y, b = blockIdx.z;
    const int qpos = p.start + t;
    const int hi = min(p.S - 1, qpos);                                                      // last visible position
    const int lo = p.window >= 0 ? max(0, qpos - p.window) : 0;                             // first visible position
    // the visible range is divided into `splits` runs of whole tiles
    const int first_tile = lo / MD_TILE, last_tile = hi / MD_TILE;
    const int tiles = hi >= lo ? last_tile - first_tile + 1 : 0;
    const int per = (tiles + p.splits - 1) / p.splits;
    const int tile_begin = first_tile + split * per, tile_end = min(first_tile + tiles, tile_begin + per);

    // this lane's slice of the queries of the warp's heads
    float ql[HPW][CHUNK], qr[HPW][2];
#pragma unroll
    for (int j = 0; j < HPW; ++j) {
        const int h = warp * HPW + j;
        const float* q = p.q_latent + ((static_cast<long long>(b) * p.T + t) * p.H + h) * r + lane * CHUNK;
#pragma unroll
        for (int i = 0; i < CHUNK; i += 4) {
            const float4 v = *reinterpret_cast<const float4*>(q + i);
            ql[j][i] = v.x; ql[j][i + 1] = v.y; ql[j][i + 2] = v.z; ql[j][i + 3] = v.w;
        }
        const float* qrp = p.q_rope + ((static_cast<long long>(b) * p.T + t) * p.H + h) * p.dr;
        qr[j][0] = 2 * lane < p.dr ? qrp[2 * lane] : 0.f;
        qr[j][1] = 2 * lane + 1 < p.dr ? qrp[2 * lane + 1] : 0.f;
    }
    float m[HPW], l[HPW], acc[HPW][CHUNK];
#pragma unroll
    for (int j = 0; j < HPW; ++j) {
        m[j] = -INFINITY; l[j] = 0.f;
#pragma unroll
        for (int i = 0; i < CHUNK; ++i) acc[j][i] = 0.f;
    }
    const int group = p.H / p.Hkv;

    for (int tile = tile_begin; tile < tile_end; ++tile) {
        const int s0 = tile * MD_TILE;
        __syncthreads();                                   // the previous tile has been consumed
        // stage the tile: 16-byte pieces, rows beyond the cache length are zero
        {
            const int vec_per_row = r / 8;
            for (int i = threadIdx.x; i < MD_TILE * vec_per_row; i += blockDim.x) {
                const int row = i / vec_per_row, v = i - row * vec_per_row;
                uint4 raw = make_uint4(0, 0, 0, 0);
                if (s0 + row < p.S) raw = *reinterpret_cast<const uint4*>(p.latent + b * p.latent_bs + static_cast<long long>(s0 + row) * r + v * 8);
                *reinterpret_cast<uint4*>(lat_s + row * r + v * 8) = raw;
            }
            for (int i = threadIdx.x; i < MD_TILE * p.dr; i += blockDim.x) {
                const int row = i / p.dr, c = i - row * p.dr;
                rope_s[i] = s0 + row < p.S ? p.rope[b * p.rope_bs + static_cast<long long>(s0 + row) * p.dr + c] : __float2bfloat16(0.f);
            }
            for (int i = threadIdx.x; i < MD_TILE * p.Hkv; i += blockDim.x) {
                const int row = i / p.Hkv, c = i - row * p.Hkv;
                gain_s[i] = s0 + row < p.S ? __bfloat162float(p.key_gain[b * p.gain_bs + static_cast<long long>(s0 + row) * p.Hkv + c]) : 0.f;
            }
        }
        __syncthreads();
        // scores: lane k ends up with position s0 + k's score for each of the warp's heads
        float sc[HPW];
#pragma unroll
        for (int j = 0; j < HPW; ++j) sc[j] = 0.f;
        for (int key = 0; key < MD_TILE; ++key) {
            float lat[CHUNK];
#pragma unroll
            for (int i = 0; i < CHUNK; i += 8) {
                const uint4 raw = *reinterpret_cast<const uint4*>(lat_s + key * r + lane * CHUNK + i);
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h2[e]); lat[i + 2 * e] = f.x; lat[i + 2 * e + 1] = f.y; }
            }
            float rp0 = 0.f, rp1 = 0.f;
            if (2 * lane < p.dr) {
                const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(rope_s + key * p.dr + 2 * lane));
                rp0 = f.x; rp1 = f.y;
            }
#pragma unroll
            for (int j = 0; j < HPW; ++j) {
                float part = qr[j][0] * rp0 + qr[j][1] * rp1;
#pragma unroll
                for (int i = 0; i < CHUNK; ++i) part = fmaf(ql[j][i], lat[i], part);
                part = wsum(part);
                if (lane == key) sc[j] = part;
            }
        }
        const int pos = s0 + lane;
        const bool visible = pos >= lo && pos <= hi;
        float pr[HPW];
#pragma unroll
        for (int j = 0; j < HPW; ++j) {
            const int h = warp * HPW + j;
            float s = sc[j] * gain_s[lane * p.Hkv + h / group] * p.scale;
            if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
            s = visible ? s : -INFINITY;
            const float m_new = fmaxf(m[j], wmax(s));
            const float corr = m_new == -INFINITY ? 1.f : expf(m[j] - m_new);          // m = -inf: nothing accumulated yet
            pr[j] = visible ? expf(s - m_new) : 0.f;
            l[j] = l[j] * corr + wsum(pr[j]);
            m[j] = m_new;
#pragma unroll
            for (int i = 0; i < CHUNK; ++i) acc[j][i] *= corr;
        }
        // values: the same latent rows, weighted by the probabilities
        for (int key = 0; key < MD_TILE; ++key) {
            float pk[HPW];
            bool any = false;
#pragma unroll
            for (int j = 0; j < HPW; ++j) { pk[j] = __shfl_sync(0xffffffffu, pr[j], key); any = any || pk[j] != 0.f; }
            if (!any) continue;                                                              // uniform across the warp
#pragma unroll
            for (int i = 0; i < CHUNK; i += 8) {
                const uint4 raw = *reinterpret_cast<const uint4*>(lat_s + key * r + lane * CHUNK + i);
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(h2[e]);
#pragma unroll
                    for (int j = 0; j < HPW; ++j) {
                        acc[j][i + 2 * e] = fmaf(pk[j], f.x, acc[j][i + 2 * e]);
                        acc[j][i + 2 * e + 1] = fmaf(pk[j], f.y, acc[j][i + 2 * e + 1]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int j = 0; j < HPW; ++j) {
        const int h = warp * HPW + j;
        const long long row = ((static_cast<long long>(b) * p.T + t) * p.H + h) * p.splits + split;
        float* out = p.part_ctx + row * r + lane * CHUNK;
#pragma unroll
        for (int i = 0; i < CHUNK; i += 4) *reinterpret_cast<float4*>(out + i) = make_float4(acc[j][i], acc[j][i + 1], acc[j][i + 2], acc[j][i + 3]);
        if (lane == 0) { p.part_ml[row * 2] = m[j]; p.part_ml[row * 2 + 1] = l[j]; }
    }
}

// context[row, :] = sum_i part[row, i, :] * exp(m_i - M) / sum_i l_i * exp(m_i - M);  one warp per (b, t, h) row
__global__ void __launch_bounds__(256)
mla_decode_merge_kernel(const float* __restrict__ part_ctx, const float* __restrict__ part_ml, float* __restrict__ context, long long rows,
                        int splits, int r) {
    const int lane = threadIdx.x & 31;
    const long long row = blockIdx.x * 8LL + (threadIdx.x >> 5);
    if (row >= rows) return;
    float big = -INFINITY;
    for (int i = 0; i < splits; ++i) big = fmaxf(big, part_ml[(row * splits + i) * 2]);
    float denom = 0.f;
    for (int i = 0; i < splits; ++i) {
        const float mi = part_ml[(row * splits + i) * 2];
        if (mi != -INFINITY) denom += part_ml[(row * splits + i) * 2 + 1] * expf(mi - big);
    }
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    for (int c = lane; c < r; c += 32) {
        float s = 0.f;
        for (int i = 0; i < splits; ++i) {
            const float mi = part_ml[(row * splits + i) * 2];
            if (mi != -INFINITY) s += part_ctx[(row * splits + i) * r + c] * expf(mi - big);
        }
        context[row * r + c] = s * inv;
    }
}

template <int CHUNK, int HPW>
static void launch_split(const MlaDecodeParams& p, cudaStream_t s) {
    const size_t smem = static_cast<size_t>(MD_TILE) * (CHUNK * 32 + p.dr) * 2 + static_cast<size_t>(MD_TILE) * p.Hkv * 4;
    auto k = mla_decode_split_kernel<CHUNK, HPW>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    k<<<dim3(p.splits, p.T, p.B), MD_WARPS * 32, smem, s>>>(p);
}

int mla_decode_splits(int B, int T, int S) {
    const int tiles = (S + MD_TILE - 1) / MD_TILE;
    int want = (2 * 148 + B * T - 1) / (B * T);            // about two CTAs per SM
    want = want < 1 ? 1 : (want > 32 ? 32 : want);
    return want < tiles ? want : (tiles < 1 ? 1 : tiles);
}

bool mla_decode_supported(int H, int Hkv, int r, int dr) {
    const int chunk = r / 32, hpw = H / MD_WARPS;
    // chunk * hpw accumulators and as many query values per lane stay in registers: at most 64 of each
    return r % 256 == 0 && (chunk == 8 || chunk == 16 || chunk == 24 || chunk == 32) && H % MD_WARPS == 0 && (hpw == 1 || hpw == 2 || hpw == 4) &&
           chunk * hpw <= 64 && Hkv >= 1 && H % Hkv == 0 && dr % 2 == 0 && dr <= 64 && dr >= 2;
}

bool launch_mla_decode(const float* q_latent, const float* q_rope, const void* latent, const void* rope, const void* key_gain,
                       long long latent_bs, long long rope_bs, long long gain_bs, float* part_ctx, float* part_ml, float* context, int B, int T,
                       int H, int Hkv, int r, int dr, int S, int splits, int start, int window, float scale, float softcap, cudaStream_t s) {
    if (!mla_decode_supported(H, Hkv, r, dr) || B <= 0 || T <= 0 || S <= 0 || splits < 1) return false;
    MlaDecodeParams p;
    p.q_latent = q_latent; p.q_rope = q_rope;
    p.latent = static_cast<const __nv_bfloat16*>(latent); p.rope = static_cast<const __nv_bfloat16*>(rope);
    p.key_gain = static_cast<const __nv_bfloat16*>(key_gain);
    p.latent_bs = latent_bs; p.rope_bs = rope_bs; p.gain_bs = gain_bs;
    p.part_ctx = part_ctx; p.part_ml = part_ml;
    p.B = B; p.T = T; p.H = H; p.Hkv = Hkv; p.r = r; p.dr = dr; p.S = S; p.splits = splits; p.start = start; p.window = window;
    p.scale = scale; p.softcap = softcap;
    const int chunk = r / 32, hpw = H / MD_WARPS;
    if (chunk == 8) {
        if (hpw == 1) launch_split<8, 1>(p, s); else if (hpw == 2) launch_split<8, 2>(p, s); else launch_split<8, 4>(p, s);
    } else if (chunk == 16) {
        if (hpw == 1) launch_split<16, 1>(p, s); else if (hpw == 2) launch_split<16, 2>(p, s); else launch_split<16, 4>(p, s);
    } else if (chunk == 24) {
        if (hpw == 1) launch_split<24, 1>(p, s); else launch_split<24, 2>(p, s);
    } else {
        if (hpw == 1) launch_split<32, 1>(p, s); else launch_split<32, 2>(p, s);
    }
    const long long rows = static_cast<long long>(B) * T * H;
    mla_decode_merge_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, s>>>(part_ctx, part_ml, context, rows, splits, r);
    return true;
}

}  // namespace gm

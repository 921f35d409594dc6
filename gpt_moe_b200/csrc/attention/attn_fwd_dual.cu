// Causal sliding-window attention forward for sm_100a, 64-wide heads, two query tiles per CTA.
//
// One CTA owns 256 query rows of one (batch, head) as two tiles of 128 rows (A: q0.., B: q0 + 128..) and walks the key
// tiles either of them can see.  Both query tiles read the same key / value tiles from one four-deep shared-memory ring,
// so every key and value tile crosses from L2 once per 256 query rows, and the softmax of one query tile runs while the
// tensor core works on the other:
//   warps 0-3   softmax of tile A: thread = query row, running maximum / sum in registers, P written to TMEM as packed bf16 pairs
//   warps 4-7   the same for tile B
//   warp  8, 9  MMA issue for tile A and for tile B (one thread each):  S_x = Q_x K^T  (M128 N128 K64),
//               O_x += P_x V  (M128 N64 K128, A from TMEM).  A thread serving both tiles in turn spent 1850 clocks per
//               (query tile, key tile) - eight N = 64 instructions 960, four N = 128 instructions 275, four commits 130 each,
//               waits on complete barriers 100 each - against 512 clocks of tensor-core work, so each tile has its own
//               thread, the descriptors are formed once and advanced by adding to their address field, and one commit per
//               step announces both the PV product of the step and the S product of the next one.  (The kernel time did
//               not change with that alone: the softmax of a tile, 1700 clocks, is the longer part of its chain.)
//   warp  10    TMA loads (one thread): Q once, then the K and V tile of a ring stage as it comes free
// O stays in TMEM for the whole CTA and the PV product accumulates into it.  The running maximum a row's exponentials are
// taken against is only moved when the row's maximum has grown by more than 2^8 since it was last moved; then (rarely
// after the first tiles) the row's O is rescaled in TMEM by its softmax thread.  The stale reference only changes the
// common factor of numerator and denominator, which cancels in O / l.
// TMEM: S_A 0-127, S_B 128-255, P_A 256-319, P_B 320-383, O_A 384-447, O_B 448-511 (one CTA per SM).
// A ring stage is released by the softmax warps: a tile's users each arrive once they have seen their PV product of that tile
// complete (a tile only one query tile reads gets both arrivals from it), so the two query tiles may drift apart by up to
// the depth of the ring.  The launcher sends document-masked calls to the single-tile kernel, whose key range is per tile.
// Reference counterpart: FlexAttention with the causal + sliding-window BlockMask (model/gpt.py:311-687,
// model/attention/self_attention.py:250-255); here the window test is exact per token in every tile.
#include "../common/ptx.cuh"
#include "../common/mxfp8.cuh"
#include "attn.h"
#include "attn_math.cuh"

namespace gm {

constexpr int DU_BM = 128, DU_BN = 128, DU_D = 64;
constexpr int DU_THREADS = 352;
constexpr int DU_STAGES = 4;
constexpr int DU_TILE_BYTES = 128 * 64 * 2;             // a 128 x 64 bf16 tile (one 128-byte-swizzled TMA box)
constexpr uint32_t DU_TMEM_COLS = 512;
constexpr uint32_t DU_COL_S = 0, DU_COL_P = 256, DU_COL_O = 384;
constexpr int DU_POLY_PER_8 = 2;                         // exponentials of every 8 evaluated as a polynomial on the FMA pipe (0 or an even number;
                                                         // 232 us with 2, 241 us with 0 on 16 x 2048 tokens, 12 heads, window 1024)
constexpr float DU_RESCALE_STEP = 8.f;                   // log2 units the row maximum may outgrow its reference before O is rescaled

// Capping and masking of 32 scores (columns kv0 .. kv0 + 31 of the key tile) in place.
template <bool MASK, bool CAP>
__device__ __forceinline__ void dual_prepare32(uint32_t (&v32)[32], int kv0, int qpos, int window, float cap_a, float cap_b) {
    if (!(MASK || CAP)) return;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        float v = __uint_as_float(v32[i]);
        if (CAP) v = cap_a * tanh_approx(v * cap_b);
        if (MASK) {
            const int kpos = kv0 + i;
            v = (kpos > qpos || qpos - kpos > window) ? -INFINITY : v;
        }
        v32[i] = __float_as_uint(v);
    }
}

__device__ __forceinline__ void dual_max32(const uint32_t (&v32)[32], float (&mx)[4]) {
#pragma unroll
    for (int i = 0; i < 32; i += 2) mx[(i >> 1) & 3] = max3(mx[(i >> 1) & 3], __uint_as_float(v32[i]), __uint_as_float(v32[i + 1]));
}

// Exponentials of 32 prepared scores against `base`, packed to bf16 pairs and stored to 16 P columns.  The scores are taken
// two at a time: scale-and-shift, the polynomial and the row sum are packed f32x2 instructions (the softmax warps are short of
// issue slots, not of arithmetic throughput); of every 8 exponentials DU_POLY_PER_8 use the polynomial.
__device__ __forceinline__ void dual_exp32(const uint32_t (&v32)[32], uint32_t p_addr, uint64_t c2, uint64_t neg_base2, uint64_t (&sum2)[2]) {
    static_assert(DU_POLY_PER_8 % 2 == 0, "pairs of scores share one form of the exponential");
    uint32_t packed[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
        const uint64_t arg = fma2(pack2(__uint_as_float(v32[i]), __uint_as_float(v32[i + 1])), c2, neg_base2);
        uint64_t e;
        if (i % 8 < DU_POLY_PER_8) {
            e = exp2_poly2(arg);
        } else {
            float a0, a1;
            unpack2(arg, a0, a1);
            e = pack2(exp2f(a0), exp2f(a1));
        }
        sum2[(i >> 1) & 1] = add2(sum2[(i >> 1) & 1], e);
        float e0, e1;
        unpack2(e, e0, e1);
        packed[i >> 1] = pack_bf16x2(e0, e1);
    }
    tmem_st_32x32b_x16(p_addr, packed);
}

// Softmax of one thread's query row against one key tile (128 scores).  The first pass reads all four 32-column chunks at
// once and keeps the first two in registers; the second pass re-reads the other two from TMEM while the exponentials of the
// first two are being formed (a thread has 168 registers: 128 scores plus the packed results do not fit).
// Masking: on a tile that touches the diagonal or the window edge (`edge_tile`) each 32-key chunk is classified for the
// warp's 32 query rows as FULL (every row sees every key: the plain path), EMPTY (no row sees any key: no arithmetic, zeros
// stored to P) or PARTIAL (the token-exact test per element).  The class is the same for all lanes of a warp, so the
// branches do not diverge; a warp meets one partial chunk in the diagonal tile and one in the window-edge tile, and
// everything else runs the unmasked code, which therefore stays resident in the instruction cache.
constexpr int CHUNK_FULL = 0, CHUNK_PARTIAL = 1, CHUNK_EMPTY = 2;

template <bool CAP>
__device__ __forceinline__ void dual_prepare_chunk(uint32_t (&v32)[32], int cls, int kv0, int qpos, int window, float cap_a, float cap_b) {
    if (cls == CHUNK_PARTIAL) dual_prepare32<true, CAP>(v32, kv0, qpos, window, cap_a, cap_b);
    else dual_prepare32<false, CAP>(v32, kv0, qpos, window, cap_a, cap_b);
}

__device__ __forceinline__ void dual_zero16(uint32_t p_addr) {
    uint32_t zeros[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) zeros[i] = 0u;
    tmem_st_32x32b_x16(p_addr, zeros);
}

template <bool CAP>
__device__ __forceinline__ void dual_softmax_tile(uint32_t s_addr, uint32_t p_addr, uint32_t o_addr, int kv0, int qpos, int warp_q0, int window,
                                                  bool edge_tile, float c, float& m_ref, float& l, bool first, float cap_a, float cap_b) {
    int cls[4] = {CHUNK_FULL, CHUNK_FULL, CHUNK_FULL, CHUNK_FULL};
    if (edge_tile) {
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            const int k_lo = kv0 + 32 * cc, k_hi = k_lo + 31, q_lo = warp_q0, q_hi = warp_q0 + 31;
            const bool empty = k_lo > q_hi || q_lo - k_hi > window;
            const bool full = k_hi <= q_lo && q_hi - k_lo <= window;
            cls[cc] = empty ? CHUNK_EMPTY : (full ? CHUNK_FULL : CHUNK_PARTIAL);
        }
    }
    uint32_t s0[32], s1[32];
    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    {
        uint32_t s2[32], s3[32];
        tmem_ld_32x32b_x32(s_addr, s0);
        tmem_ld_32x32b_x32(s_addr + 32, s1);
        tmem_ld_32x32b_x32(s_addr + 64, s2);
        tmem_ld_32x32b_x32(s_addr + 96, s3);
        tmem_ld_wait();
        if (cls[0] != CHUNK_EMPTY) { dual_prepare_chunk<CAP>(s0, cls[0], kv0, qpos, window, cap_a, cap_b); dual_max32(s0, mx); }
        if (cls[1] != CHUNK_EMPTY) { dual_prepare_chunk<CAP>(s1, cls[1], kv0 + 32, qpos, window, cap_a, cap_b); dual_max32(s1, mx); }
        if (cls[2] != CHUNK_EMPTY) { dual_prepare_chunk<CAP>(s2, cls[2], kv0 + 64, qpos, window, cap_a, cap_b); dual_max32(s2, mx); }
        if (cls[3] != CHUNK_EMPTY) { dual_prepare_chunk<CAP>(s3, cls[3], kv0 + 96, qpos, window, cap_a, cap_b); dual_max32(s3, mx); }
    }
    const float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * c;
    const bool grow = m_tile > m_ref + DU_RESCALE_STEP;       // also true for the first finite maximum (m_ref = -inf)
    if (__any_sync(0xffffffffu, grow)) {
        const float alpha = grow ? exp2f(m_ref - m_tile) : 1.f;
        if (!first) {                 // the previous PV product is complete: the commit that announced this S came after it
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                uint32_t o[32];
                tmem_ld_32x32b_x32(o_addr + hh * 32, o);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                tmem_st_32x32b_x16(o_addr + hh * 32, *reinterpret_cast<uint32_t(*)[16]>(&o[0]));
                tmem_st_32x32b_x16(o_addr + hh * 32 + 16, *reinterpret_cast<uint32_t(*)[16]>(&o[16]));
            }
        }
        l *= alpha;
        if (grow) m_ref = m_tile;
    }
    const float base = m_ref == -INFINITY ? 0.f : m_ref;       // a row may have no visible key yet
    const uint64_t c2 = pack2(c, c), neg_base2 = pack2(-base, -base);
    uint64_t sum2[2] = {0ull, 0ull};                        // two packed pairs of partial row sums (bit pattern of 0.f, 0.f)
    uint32_t s2[32];
    tmem_ld_32x32b_x32(s_addr + 64, s2);
    if (cls[0] != CHUNK_EMPTY) dual_exp32(s0, p_addr, c2, neg_base2, sum2); else dual_zero16(p_addr);
    tmem_ld_wait();
    tmem_ld_32x32b_x32(s_addr + 96, s0);
    if (cls[1] != CHUNK_EMPTY) dual_exp32(s1, p_addr + 16, c2, neg_base2, sum2); else dual_zero16(p_addr + 16);
    if (cls[2] != CHUNK_EMPTY) {
        dual_prepare_chunk<CAP>(s2, cls[2], kv0 + 64, qpos, window, cap_a, cap_b);
        dual_exp32(s2, p_addr + 32, c2, neg_base2, sum2);
    } else {
        dual_zero16(p_addr + 32);
    }
    tmem_ld_wait();
    if (cls[3] != CHUNK_EMPTY) {
        dual_prepare_chunk<CAP>(s0, cls[3], kv0 + 96, qpos, window, cap_a, cap_b);
        dual_exp32(s0, p_addr + 48, c2, neg_base2, sum2);
    } else {
        dual_zero16(p_addr + 48);
    }
    float t0, t1, t2, t3;
    unpack2(sum2[0], t0, t1);
    unpack2(sum2[1], t2, t3);
    l += (t0 + t1) + (t2 + t3);
}

template <bool CAPPED>
__global__ void __launch_bounds__(DU_THREADS, 1)
attn_fwd_dual_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sq = smem;                                   // two query tiles
    uint8_t* sk = sq + 2 * DU_TILE_BYTES;                 // DU_STAGES key tiles
    uint8_t* sv = sk + DU_STAGES * DU_TILE_BYTES;         // DU_STAGES value tiles
    uint64_t* bars = reinterpret_cast<uint64_t*>(sv + DU_STAGES * DU_TILE_BYTES);
    uint64_t* bar_q = bars + 0;
    uint64_t* bar_s = bars + 1;                           // [2] S_x complete (and every product of tile x issued before it)
    uint64_t* bar_p = bars + 3;                           // [2] P_x written, S_x consumed (128 arrivals)
    uint64_t* bar_o = bars + 5;                           // [2] last PV product of tile x complete
    uint64_t* bar_full = bars + 7;                        // [STAGES] key and value tile landed
    uint64_t* bar_free = bar_full + DU_STAGES;            // [STAGES] both query tiles are done with the stage (2 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_free + DU_STAGES);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y, batch = blockIdx.z;
    const int q0 = blockIdx.x * 2 * DU_BM;
    const int window = p.window_ptr ? min(max(*p.window_ptr, 0), p.seq_len) : p.window;
    const int row0 = batch * p.seq_len;
    // key tiles (units of 128 keys) of each query tile: from the tile holding the first key its first row sees to its diagonal tile
    const int first_a = q0 - window, first_b = q0 + DU_BM - window;
    const int lo_a = first_a > 0 ? first_a / DU_BN : 0, lo_b = first_b > 0 ? first_b / DU_BN : 0;
    const int hi_a = q0 / DU_BN;                                // B's diagonal tile is hi_a + 1
    const int kv_head = head / p.group;                       // grouped-query attention: several q heads share a kv head
    const int q_col = p.q_col0 + head * DU_D, k_col = p.k_col0 + kv_head * DU_D, v_col = p.v_col0 + kv_head * DU_D;

    if (threadIdx.x == 0) {
        mbar_init(bar_q, 1);
        for (int x = 0; x < 2; ++x) { mbar_init(&bar_s[x], 1); mbar_init(&bar_p[x], 128); mbar_init(&bar_o[x], 1); }
        for (int st = 0; st < DU_STAGES; ++st) { mbar_init(&bar_full[st], 1); mbar_init(&bar_free[st], 2); }
        fence_barrier_init();
    }
    if (warp == 8) { tmem_alloc(tmem_slot, DU_TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 10) {
        if (lane == 0) {
            mbar_expect_tx(bar_q, 2 * DU_TILE_BYTES);
            tma_load_3d(sq, &tmap_q, bar_q, q_col, row0 + q0, 0);
            tma_load_3d(sq + DU_TILE_BYTES, &tmap_q, bar_q, q_col, row0 + q0 + DU_BM, 0);
            const int total = hi_a + 1 - lo_a + 1;                // key tiles lo_a .. hi_a + 1
            for (int u = 0; u < total; ++u) {
                const int st = u % DU_STAGES, use = u / DU_STAGES;
                const int key_row = row0 + (lo_a + u) * DU_BN;
                if (use > 0 && !mbar_wait(&bar_free[st], (use - 1) & 1)) { atomicExch(p.status, 211); break; }
                mbar_expect_tx(&bar_full[st], 2 * DU_TILE_BYTES);
                tma_load_3d(sk + st * DU_TILE_BYTES, &tmap_k, &bar_full[st], k_col, key_row, 0);
                tma_load_3d(sv + st * DU_TILE_BYTES, &tmap_v, &bar_full[st], v_col, key_row, 0);
            }
        }
    } else if (warp >= 8) {
        if (lane == 0) {
            const int x = warp - 8;
            const int n_x = x == 0 ? hi_a - lo_a + 1 : hi_a + 1 - lo_b + 1;
            const int u0 = x == 0 ? 0 : lo_b - lo_a;              // ring position of this tile's first key tile
            constexpr uint32_t idesc_s = make_idesc_bf16(DU_BM, DU_BN, false, false);
            constexpr uint32_t idesc_pv = make_idesc_bf16(DU_BM, DU_D, false, true);
            // descriptors of the first K-slice of Q_x, of ring stage 0 of K and of V; the address field counts 16-byte units, so a
            // stage is 1024 units further, a 16-column slice of a K-major tile 2 units, a 16-key slice of the MN-major V tile 128 units
            const uint64_t q_desc = make_smem_desc(smem_u32(sq) + x * DU_TILE_BYTES, 16, 1024);
            const uint64_t k_desc = make_smem_desc(smem_u32(sk), 16, 1024);
            const uint64_t v_desc = make_smem_desc(smem_u32(sv), DU_BN * 128, 1024);
            const uint32_t tmem_s = tmem_base + DU_COL_S + x * DU_BN, tmem_p = tmem_base + DU_COL_P + x * (DU_BN / 2);
            const uint32_t tmem_o = tmem_base + DU_COL_O + x * DU_D;
            auto issue_s = [&](int u) -> bool {
                const int st = u % DU_STAGES;
                if (!mbar_wait(&bar_full[st], (u / DU_STAGES) & 1)) return false;
                tc_fence_after();
                const uint64_t kd = k_desc + st * (DU_TILE_BYTES >> 4);
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) umma_f16(tmem_s, q_desc + k4 * 2, kd + k4 * 2, idesc_s, k4 != 0);
                umma_commit(&bar_s[x]);
                return true;
            };
            if (!mbar_wait(bar_q, 0) || !issue_s(u0)) { atomicExch(p.status, 213); ok = false; }
            for (int i = 0; i < n_x && ok; ++i) {
                if (!mbar_wait(&bar_p[x], i & 1)) { atomicExch(p.status, 215); ok = false; break; }
                tc_fence_after();
                const uint64_t vd = v_desc + ((u0 + i) % DU_STAGES) * (DU_TILE_BYTES >> 4);   // landed: S of this tile waited for the stage
#pragma unroll
                for (int k8 = 0; k8 < DU_BN / 16; ++k8)
                    umma_f16_ta(tmem_o, tmem_p + k8 * 8, vd + k8 * 128, idesc_pv, (i | k8) != 0);      // 16 keys = 8 packed columns
                if (i + 1 < n_x) {
                    if (!issue_s(u0 + i + 1)) { atomicExch(p.status, 217); ok = false; }
                } else {
                    umma_commit(&bar_o[x]);
                }
            }
        }
    } else {
        const int x = warp >> 2, quad = warp & 3;            // query tile; TMEM lanes 32*quad..+31
        const int r = quad * 32 + lane;
        const int q0x = q0 + x * DU_BM;
        const int qpos = q0x + r;
        const int lo_x = x == 0 ? lo_a : lo_b;
        const int n_x = q0x / DU_BN - lo_x + 1;
        const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
        const uint32_t s_addr = tmem_base + lane_off + DU_COL_S + x * DU_BN;
        const uint32_t p_addr = tmem_base + lane_off + DU_COL_P + x * (DU_BN / 2);
        const uint32_t o_addr = tmem_base + lane_off + DU_COL_O + x * DU_D;
        const float c = p.scale_log2e;
        constexpr bool capped = CAPPED;
        const float cap_a = capped ? p.softcap / p.scale : 0.f, cap_b = capped ? p.scale / p.softcap : 0.f;
        float m_ref = -INFINITY, l = 0.f;
        for (int i = 0; i < n_x && ok; ++i) {
            const int tile = lo_x + i;
            const int kv0 = tile * DU_BN;
            if (!mbar_wait(&bar_s[x], i & 1)) { atomicExch(p.status, 218); ok = false; break; }
            tc_fence_after();
            if (i > 0 && r == 0) {
                // this S was committed after the PV product of the previous key tile: tile x is done with that ring stage.  A key
                // tile the other query tile does not read (before B's first, after A's diagonal) gets both arrivals from here
                const int done = tile - 1;
                uint64_t* fb = &bar_free[(done - lo_a) % DU_STAGES];
                mbar_arrive(fb);
                if (x == 0 ? done < lo_b : done > hi_a) mbar_arrive(fb);
            }
            // tiles strictly inside the band need no mask; the diagonal tile and the tile at the window edge do
            const bool need_mask = (kv0 + DU_BN - 1 > q0x) || (q0x + DU_BM - 1 - kv0 > window);
            dual_softmax_tile<capped>(s_addr, p_addr, o_addr, kv0, qpos, q0x + quad * 32, window, need_mask, c, m_ref, l, i == 0, cap_a, cap_b);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(&bar_p[x]);
        }
        if (ok && !mbar_wait(&bar_o[x], 0)) { atomicExch(p.status, 220); ok = false; }
        if (ok) {
            tc_fence_after();
            float o[DU_D];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) tmem_ld_32x32b_x32(o_addr + hh * 32, *reinterpret_cast<uint32_t(*)[32]>(&o[32 * hh]));
            tmem_ld_wait();
            const float inv = 1.f / l;
            const long long token = static_cast<long long>(row0) + qpos;
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out) + token * p.out_stride + head * DU_D;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                uint4 w;
                w.x = pack_bf16x2(o[8 * q] * inv, o[8 * q + 1] * inv);
                w.y = pack_bf16x2(o[8 * q + 2] * inv, o[8 * q + 3] * inv);
                w.z = pack_bf16x2(o[8 * q + 4] * inv, o[8 * q + 5] * inv);
                w.w = pack_bf16x2(o[8 * q + 6] * inv, o[8 * q + 7] * inv);
                *reinterpret_cast<uint4*>(out + 8 * q) = w;
            }
            if (p.out_q != nullptr) {
                // the thread's 64 output columns are two MXFP8 blocks of the token-major row: quantise the bf16 values just stored
                // (reference: attention output quantised straight from its own layout, model/linear/fp8/custom/output_projection.py:16-49)
                const int width = p.heads * DU_D;
#pragma unroll
                for (int blk = 0; blk < 2; ++blk) {
                    float amax = 0.f;
#pragma unroll
                    for (int i = 0; i < 32; ++i) { o[32 * blk + i] = round_bf16(o[32 * blk + i] * inv); amax = fmaxf(amax, fabsf(o[32 * blk + i])); }
                    const uint32_t e8 = e8m0_from_amax(amax);
                    const float qs = inv_scale_from_e8m0(e8);
                    const int col = head * DU_D + 32 * blk;
                    uint8_t* dst = p.out_q + token * width + col;
                    const float* ob = o + 32 * blk;
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        uint4 w;
                        w.x = pack_e4m3x4(ob[16 * q] * qs, ob[16 * q + 1] * qs, ob[16 * q + 2] * qs, ob[16 * q + 3] * qs);
                        w.y = pack_e4m3x4(ob[16 * q + 4] * qs, ob[16 * q + 5] * qs, ob[16 * q + 6] * qs, ob[16 * q + 7] * qs);
                        w.z = pack_e4m3x4(ob[16 * q + 8] * qs, ob[16 * q + 9] * qs, ob[16 * q + 10] * qs, ob[16 * q + 11] * qs);
                        w.w = pack_e4m3x4(ob[16 * q + 12] * qs, ob[16 * q + 13] * qs, ob[16 * q + 14] * qs, ob[16 * q + 15] * qs);
                        *reinterpret_cast<uint4*>(dst + 16 * q) = w;
                    }
                    p.out_sf[sf_offset(token, col >> 5, (width + 127) >> 7)] = static_cast<uint8_t>(e8);
                }
            }
            // natural-log LSE of the scaled scores, layout [batch, head, seq]; m_ref is the reference the sum l was taken against
            p.lse[(static_cast<long long>(batch) * p.heads + head) * p.seq_len + qpos] = m_ref * 0.69314718056f + __logf(l);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        if (*reinterpret_cast<volatile int*>(p.status) != 0) {    // a wait gave up: let MMAs and copies in flight drain before the columns are freed
            const long long start = clock64();
            while (clock64() - start < 200000) {}
        }
        tc_fence_after();
        tmem_dealloc(tmem_base, DU_TMEM_COLS);
    }
}

bool attn_fwd_dual_supported(const AttnParams& p) {
    return p.qk_dim == 64 && p.doc_start == nullptr && p.seq_len % (2 * DU_BM) == 0;
}

template <bool CAPPED>
static cudaError_t launch_dual_variant(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, cudaStream_t stream) {
    constexpr int smem = (2 + 2 * DU_STAGES) * DU_TILE_BYTES + 1024 + 256;
    auto kernel = attn_fwd_dual_kernel<CAPPED>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    dim3 grid(p.seq_len / (2 * DU_BM), p.heads, p.batch);
    kernel<<<grid, DU_THREADS, smem, stream>>>(tq, tk, tv, p);
    return cudaGetLastError();
}

cudaError_t launch_attn_fwd_dual(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, cudaStream_t stream) {
    return p.softcap > 0.f ? launch_dual_variant<true>(tq, tk, tv, p, stream) : launch_dual_variant<false>(tq, tk, tv, p, stream);
}

}  // namespace gm

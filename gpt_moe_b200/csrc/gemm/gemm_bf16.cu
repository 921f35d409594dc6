// Persistent, warp-specialised bf16 GEMM for sm_100a: D = alpha * A * B^T (+ beta * C) (+ D).
//
// CTAs run as pairs (a cluster of two on neighbouring SMs, tcgen05 cta_group::2).  A pair walks a list of
// 256 x 256 output tiles: each CTA owns 128 of the rows and stages only HALF of the B tile, the tensor cores of
// both SMs read both halves, so a CTA pulls 32 KB instead of 48 KB through L2 per 128 x 256 x 64 block of work -
// the main loop of a one-CTA kernel is bound by exactly that traffic.  Roles inside each CTA:
//   warp 0  : TMA producer   - fills a 5-stage ring of {A 128x64, B 128x64} bf16 tiles (128B swizzle); the
//                              bytes of both CTAs are counted on the leader's (even CTA's) barrier
//   warp 1  : MMA issuer     - leader CTA only: one thread issues tcgen05.mma (M256 N256 K16) into one of
//                              two TMEM accumulators (2 x 256 columns in each CTA), commits to both CTAs
//   warps 2-9: epilogue      - tcgen05.ld the finished accumulator (thread = row; two warps per TMEM lane
//                              quadrant split the columns), scale / add C, convert, stage 128-byte-swizzled
//                              slabs in one of two shared-memory buffers and hand them to TMA (store, or
//                              reduce-add for fp32 accumulation and split-K); overlaps the next tile's main
//                              loop.  TMA clips rows/columns outside the tensor.
// Operands may be K-major ([rows, K] with K contiguous) or MN-major ([K, rows] with rows
// contiguous); both are read straight from row-major tensors by TMA, so forward (X W^T), input
// gradient (dY W) and weight gradient (dY^T X) all run without a transposed copy.
//
// Three tile enumerations share the kernel:
//   DENSE     (optionally batched over z)                      - projections, LM head, Polar Express
//             symmetric results (X X^T, A A with A symmetric): only the tiles on or above the diagonal are computed, the
//             epilogue stores every off-diagonal tile a second time transposed (the reference's triangle-and-mirror
//             kernels, optimizers/polar_express.py:60-121 and :155-230)
//   GROUPED_M rows of A belong to experts; tile -> expert table on the device picks B's z slice
//             (expert segments are padded to 128 rows, so a tile never straddles two experts)
//   GROUPED_K one output matrix per expert, contraction over that expert's (padded) row segment
//             - the expert weight gradient; empty experts get exact zeros
// Reference counterparts: Triton `_grouped_mm_kernel` (model/linear/default/grouped.py:12-70) and the
// cuBLAS calls behind every F.linear (model/linear/linear.py:23).
#include "../common/ptx.cuh"
#include "gemm.h"

#include <cuda.h>

namespace gm {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 5;
constexpr int BN_HALF = BN / 2;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN_HALF * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int GEMM_THREADS = 320;           // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue
constexpr int GROUP_M = 4;               // in pair tiles (256 rows each)
constexpr uint32_t TMEM_COLS = 512;
constexpr int STAGING_BYTES = 2 * BM * 128;      // two slabs of [128 rows][128 bytes]; the staging area holds two such buffers

struct TileCoord {
    int m0, n0;        // element offsets of the tile in the output
    int az, bz, dz;    // z (batch / expert) coordinates for A, B, D
    int k_begin, k_blocks;
    int m_limit, n_limit;
    bool store_zeros;  // no contraction work at all for this output tile: write zeros unless accumulating
};

// Work is enumerated in PAIR tiles (two vertically adjacent 128-row tiles, one per CTA of the pair); `m_tiles` counts
// the 128-row tiles rounded up to an even number.
__device__ __forceinline__ int total_tiles(const GemmParams& p, int& m_tiles, int& n_tiles) {
    n_tiles = (p.N + BN - 1) / BN;
    if (p.mode == GEMM_GROUPED_M) {
        m_tiles = (*p.num_m_tiles + 1) & ~1;
        return m_tiles / 2 * n_tiles;
    }
    m_tiles = ((p.M + BM - 1) / BM + 1) & ~1;
    if (p.symmetric) return n_tiles * (n_tiles + 1) / 2 * p.batch;      // M == N: pair tiles (i, j) with i <= j
    return m_tiles / 2 * n_tiles * p.batch * p.split_k;
}

__device__ __forceinline__ TileCoord tile_coord(const GemmParams& p, int tile, int cta_rank, int m_tiles, int n_tiles) {
    TileCoord t;
    int split = 0;
    if (p.mode != GEMM_GROUPED_M && p.split_k > 1) {
        split = tile % p.split_k;
        tile /= p.split_k;
    }
    const int m_pairs = m_tiles / 2;
    const int per_batch = p.symmetric ? n_tiles * (n_tiles + 1) / 2 : m_pairs * n_tiles;
    const int z = (p.mode == GEMM_GROUPED_M) ? 0 : tile / per_batch;
    int r = tile - z * per_batch;
    int mt, nt;
    if (p.symmetric) {
        // row i of the upper triangle holds n_tiles - i tiles
        int i = 0;
        while (r >= n_tiles - i) { r -= n_tiles - i; ++i; }
        mt = 2 * i + cta_rank;
        nt = i + r;
    } else {
        // grouped raster: GROUP_M pair-rows share their column sweep so A tiles stay in L2
        const int group = r / (GROUP_M * n_tiles);
        const int first_m = group * GROUP_M;
        const int rows_in_group = min(GROUP_M, m_pairs - first_m);
        r -= group * GROUP_M * n_tiles;
        mt = 2 * (first_m + r % rows_in_group) + cta_rank;
        nt = r / rows_in_group;
    }
    t.m0 = mt * BM;
    t.n0 = nt * BN;
    t.m_limit = p.M;
    t.n_limit = p.N;
    t.k_begin = 0;
    t.k_blocks = (p.K + BK - 1) / BK;
    t.az = t.bz = t.dz = z;
    if (p.mode == GEMM_GROUPED_M) {
        t.az = 0;
        t.dz = 0;
        t.bz = p.tile_expert[mt & ~1];          // both tiles of a pair belong to one expert (segments are padded to 256 rows)
        t.m_limit = *p.num_m_tiles * BM;
    } else if (p.mode == GEMM_GROUPED_K) {
        const int begin = z == 0 ? 0 : p.seg_ends[z - 1];
        t.az = t.bz = 0;
        t.k_begin = begin;
        t.k_blocks = (p.seg_ends[z] - begin) / BK;
    }
    t.store_zeros = t.k_blocks == 0;
    if (p.split_k > 1) {          // contiguous share of the K blocks; partial results meet in a TMA reduce-add
        const int per = (t.k_blocks + p.split_k - 1) / p.split_k;
        const int first = min(split * per, t.k_blocks);
        const int count = min(per, t.k_blocks - first);
        t.k_begin += first * BK;
        t.k_blocks = count;
        t.store_zeros = false;
    }
    return t;
}

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_d, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* staging = smem + STAGES * STAGE_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(staging + 2 * STAGING_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta_rank = static_cast<int>(cluster_ctarank());     // 0 = leader of the pair
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        // acc_empty of the leader collects one arrival per epilogue warp of each of the two CTAs (a remote arrival per thread
        // would put 256 messages per tile on the cluster's shared-memory network)
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 16); }
        fence_barrier_init();
        tma_prefetch_desc(&tmap_a);
        tma_prefetch_desc(&tmap_b);
        tma_prefetch_desc(&tmap_d);
    }
    if (warp == 1) { tmem_alloc_pair(tmem_slot, TMEM_COLS); tmem_relinquish_pair(); }
    tc_fence_before();
    cluster_sync_all();                                            // both CTAs' barriers exist before either signals the other
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    int m_tiles, n_tiles;
    const int tiles = total_tiles(p, m_tiles, n_tiles);
    const int first_tile = blockIdx.x >> 1, tile_step = gridDim.x >> 1;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0; uint32_t ph = 0;
            for (int tile = first_tile; tile < tiles && ok; tile += tile_step) {
                const TileCoord t = tile_coord(p, tile, cta_rank, m_tiles, n_tiles);
                for (int kb = 0; kb < t.k_blocks; ++kb) {
                    if (!mbar_wait(&empty[s], ph ^ 1)) { atomicExch(p.status, 101); ok = false; break; }
                    if (cta_rank == 0) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);      // both CTAs' copies land on the leader's barrier
                    uint8_t* a_dst = smem + s * STAGE_BYTES;
                    uint8_t* b_dst = a_dst + A_BYTES;
                    const int k = t.k_begin + kb * BK;
                    const int bn0 = t.n0 + cta_rank * BN_HALF;                          // this CTA stages its half of the B tile
                    if (A_MN) {
                        for (int i = 0; i < BM / 64; ++i) tma_load_3d_pair(a_dst + i * (64 * BK * 2), &tmap_a, &full[s], t.m0 + 64 * i, k, t.az);
                    } else {
                        tma_load_3d_pair(a_dst, &tmap_a, &full[s], k, t.m0, t.az);
                    }
                    if (B_MN) {
                        for (int i = 0; i < BN_HALF / 64; ++i) tma_load_3d_pair(b_dst + i * (64 * BK * 2), &tmap_b, &full[s], bn0 + 64 * i, k, t.bz);
                    } else {
                        tma_load_3d_pair(b_dst, &tmap_b, &full[s], k, bn0, t.bz);
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && cta_rank == 0) {
            constexpr uint32_t idesc = make_idesc_bf16(2 * BM, BN, A_MN, B_MN);
            // K-major: 8-row groups are 1024 B apart, 16 K-elements = 32 B.  MN-major: 64-element column slabs are
            // BK*128 B apart (leading offset), 8-K-row groups 1024 B apart, 16 K-rows = 2048 B.
            constexpr uint32_t a_lbo = A_MN ? BK * 128 : 16, b_lbo = B_MN ? BK * 128 : 16;
            constexpr uint32_t a_kstep = A_MN ? 2048 : 32, b_kstep = B_MN ? 2048 : 32;
            int s = 0; uint32_t ph = 0; int acc = 0; uint32_t acc_ph = 0;
            for (int tile = first_tile; tile < tiles && ok; tile += tile_step) {
                const TileCoord t = tile_coord(p, tile, cta_rank, m_tiles, n_tiles);
                if (t.k_blocks == 0) continue;
                if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1)) { atomicExch(p.status, 102); ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < t.k_blocks; ++kb) {
                    if (!mbar_wait(&full[s], ph)) { atomicExch(p.status, 103); ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
                    for (int k4 = 0; k4 < BK / 16; ++k4) {
                        const uint64_t adesc = make_smem_desc(a_addr + k4 * a_kstep, a_lbo, 1024);
                        const uint64_t bdesc = make_smem_desc(b_addr + k4 * b_kstep, b_lbo, 1024);
                        umma_f16_pair(d_tmem, adesc, bdesc, idesc, (kb | k4) != 0);
                    }
                    umma_commit_pair(&empty[s]);
                    if (++s == STAGES) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                umma_commit_pair(&acc_full[acc]);
                if (++acc == 2) { acc = 0; acc_ph ^= 1; }
            }
        }
    } else {
        // Eight epilogue warps: TMEM lanes 32*quad .. 32*quad+31 are readable by warps with warp % 4 == quad, so two warps share
        // a lane quadrant and split the columns of every round between them (half 0: first slab, half 1: second slab).
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;
        const int row_in_tile = quad * 32 + lane;
        const bool leader = threadIdx.x == 64;      // first epilogue thread issues the TMA stores
        const int elem = p.out_fp32 ? 4 : 2;
        const int chunks_per_round = p.out_fp32 ? 2 : 4;          // 32-column accumulator chunks staged per round
        const int my_chunks = chunks_per_round / 2;               // per warp half
        const int rounds = (BN / 32) / chunks_per_round;
        const int cols_per_slab = 128 / elem;
        const bool reduce = p.accumulate || p.split_k > 1;
        const int sw = row_in_tile & 7;
        int acc = 0; uint32_t acc_ph = 0;
        uint32_t stores = 0;                                       // committed store groups: selects the staging buffer
        for (int tile = first_tile; tile < tiles && ok; tile += tile_step) {
            const TileCoord t = tile_coord(p, tile, cta_rank, m_tiles, n_tiles);
            const bool have_acc = t.k_blocks != 0;
            if (!have_acc && !(t.store_zeros && !p.accumulate)) continue;      // nothing to add, nothing to clear
            const int row = t.m0 + row_in_tile;
            const bool row_ok = row < t.m_limit;
            float alpha = p.alpha, beta = p.beta;
            if (p.batch_sumsq != nullptr) {                   // an operand is an un-normalised Muon update: scale the result instead
                const float inv = 1.f / (sqrtf(p.batch_sumsq[t.dz]) * 1.02f + 1e-6f);
                if (p.scale_mode == 2) alpha *= inv * inv;
                else { alpha *= inv; beta *= inv; }
            }
            const bool mirror = p.symmetric && t.n0 != t.m0 - cta_rank * BM;      // off-diagonal pair tile (uniform across the pair)
            if (have_acc) {
                if (!mbar_wait(&acc_full[acc], acc_ph)) { atomicExch(p.status, 104); ok = false; break; }
                tc_fence_after();
            }
            for (int round = 0; round < rounds; ++round) {
                const int round_col0 = t.n0 + round * chunks_per_round * 32;
                if (round_col0 >= t.n_limit) break;                           // uniform across the CTA
                uint8_t* buf = staging + (stores & 1) * STAGING_BYTES;
                // the store that read this buffer two rounds ago must have finished reading it
                if (leader) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                asm volatile("bar.sync 1, 256;" ::: "memory");
                uint32_t r[2][32];
                if (have_acc) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        if (j < my_chunks) {
                            const int chunk = round * chunks_per_round + half * my_chunks + j;
                            tmem_ld_32x32b_x32(tmem_base + acc * BN + chunk * 32 + (static_cast<uint32_t>(quad * 32) << 16), r[j]);
                        }
                    }
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 2; ++j)
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[j][i] = 0u;
                }
                if (have_acc && round == rounds - 1) {                        // accumulator fully read: release it early
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(&acc_empty[acc], 0);
                }
                uint8_t* slab_row = buf + half * (BM * 128) + row_in_tile * 128;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    if (j >= my_chunks) break;
                    const int col0 = round_col0 + (half * my_chunks + j) * 32;
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[j][i]) * alpha;
                    if (p.C != nullptr && row_ok && col0 < t.n_limit) {
                        const __nv_bfloat16* c = reinterpret_cast<const __nv_bfloat16*>(p.C) +
                            static_cast<long long>(t.dz) * p.c_batch_stride + static_cast<long long>(row) * p.ldc + col0;
                        if (col0 + 32 <= t.n_limit) {
#pragma unroll
                            for (int i = 0; i < 32; i += 8) {
                                const uint4 q = *reinterpret_cast<const uint4*>(c + i);
                                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const float2 f = __bfloat1622float2(h[e]);
                                    v[i + 2 * e] += beta * f.x;
                                    v[i + 2 * e + 1] += beta * f.y;
                                }
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (col0 + i < t.n_limit) v[i] += beta * __bfloat162float(c[i]);
                        }
                    }
                    if (mirror) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[j][i] = __float_as_uint(v[i]);      // kept for the transposed store below
                    }
                    // 16-byte pieces of this thread's row go to piece index (i ^ row%8) of the 128-byte slab row
                    if (p.out_fp32) {
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            *reinterpret_cast<float4*>(slab_row + ((q ^ sw) << 4)) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                    } else {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint4 o;
                            o.x = pack_bf16x2(v[8 * q], v[8 * q + 1]);
                            o.y = pack_bf16x2(v[8 * q + 2], v[8 * q + 3]);
                            o.z = pack_bf16x2(v[8 * q + 4], v[8 * q + 5]);
                            o.w = pack_bf16x2(v[8 * q + 6], v[8 * q + 7]);
                            *reinterpret_cast<uint4*>(slab_row + (((j * 4 + q) ^ sw) << 4)) = o;
                        }
                    }
                }
                fence_proxy_async();
                asm volatile("bar.sync 1, 256;" ::: "memory");                 // slabs complete and visible to the async proxy
                if (leader) {
                    for (int sl = 0; sl < 2; ++sl) {
                        const int col = round_col0 + sl * cols_per_slab;
                        if (col >= t.n_limit || t.m0 >= t.m_limit) break;
                        const uint32_t src = smem_u32(buf + sl * (BM * 128));
                        if (reduce) {
                            asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.bulk_group [%0, {%2, %3, %4}], [%1];"
                                         ::"l"(&tmap_d), "r"(src), "r"(col), "r"(t.m0), "r"(t.dz) : "memory");
                        } else {
                            asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                                         ::"l"(&tmap_d), "r"(src), "r"(col), "r"(t.m0), "r"(t.dz) : "memory");
                        }
                    }
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                ++stores;
                if (mirror) {
                    // The same 128 x 128 block goes out transposed (bf16 only): element (row, c) of this round lands in row c of
                    // the transposed block, and 64 of this CTA's rows make one 128-byte slab row, so the two slabs are the
                    // column ranges [m0, m0 + 64) and [m0 + 64, m0 + 128) of the mirrored tile.
                    uint8_t* tbuf = staging + (stores & 1) * STAGING_BYTES;
                    if (leader) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                    asm volatile("bar.sync 1, 256;" ::: "memory");
                    uint8_t* tcol = tbuf + (row_in_tile >> 6) * (BM * 128) + (row_in_tile & 7) * 2;
                    const int piece = (row_in_tile & 63) >> 3;
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int cl = (half * 2 + j) * 32 + i;
                            *reinterpret_cast<__nv_bfloat16*>(tcol + cl * 128 + ((piece ^ (i & 7)) << 4)) =
                                __float2bfloat16_rn(__uint_as_float(r[j][i]));
                        }
                    }
                    fence_proxy_async();
                    asm volatile("bar.sync 1, 256;" ::: "memory");
                    if (leader) {
                        for (int sl = 0; sl < 2; ++sl) {
                            const int col = t.m0 + sl * 64;
                            if (col >= t.n_limit || round_col0 >= t.m_limit) break;
                            const uint32_t src = smem_u32(tbuf + sl * (BM * 128));
                            asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                                         ::"l"(&tmap_d), "r"(src), "r"(col), "r"(round_col0), "r"(t.dz) : "memory");
                        }
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                    ++stores;
                }
            }
            if (have_acc) {
                // tiles narrower than BN leave the round loop early: the accumulator is released here in that case
                const int rounds_done = min(rounds, (t.n_limit - t.n0 + chunks_per_round * 32 - 1) / (chunks_per_round * 32));
                if (rounds_done < rounds) { tc_fence_before(); __syncwarp(); if (lane == 0) mbar_arrive_cluster(&acc_empty[acc], 0); }
                if (++acc == 2) { acc = 0; acc_ph ^= 1; }
            }
        }
        if (leader) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    // common teardown: every path (including a timed-out wait) reaches it, so TMEM is always released
    tc_fence_before();
    cluster_sync_all();                       // the partner no longer reads this CTA's shared memory or signals its barriers
    if (warp == 1) {
        if (*reinterpret_cast<volatile int*>(p.status) != 0) {
            // a wait gave up: give any TMA copy still in flight time to land before the CTA's smem is recycled
            const long long start = clock64();
            while (clock64() - start < 200000) {}
        }
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

constexpr int GEMM_SMEM_BYTES = STAGES * STAGE_BYTES + 2 * STAGING_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;

template <bool A_MN, bool B_MN>
static cudaError_t launch_variant(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const GemmParams& p, int sms,
                                  cudaStream_t stream) {
    auto kernel = gemm_bf16_kernel<A_MN, B_MN>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms & ~1);
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = GEMM_SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, ta, tb, td, p);
}

cudaError_t launch_gemm_bf16(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const GemmParams& p, bool a_mn,
                             bool b_mn, int sms, cudaStream_t stream) {
    if (a_mn) return b_mn ? launch_variant<true, true>(ta, tb, td, p, sms, stream) : launch_variant<true, false>(ta, tb, td, p, sms, stream);
    return b_mn ? launch_variant<false, true>(ta, tb, td, p, sms, stream) : launch_variant<false, false>(ta, tb, td, p, sms, stream);
}

}  // namespace gm

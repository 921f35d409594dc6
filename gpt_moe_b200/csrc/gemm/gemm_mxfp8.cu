// Block-scaled MXFP8 GEMM for sm_100a: D[M,N] (bf16) = alpha * A[M,K] * B[N,K]^T with e4m3 operands and one UE8M0
// (power-of-two) scale per 32 consecutive K elements of every row of A and of B, multiplied in by the tensor core
// (tcgen05.mma kind::mxf8f6f4.block_scale), fp32 accumulation in TMEM.
//
// CTAs run as pairs (cluster of two, tcgen05 cta_group::2) on 256 x 256 output tiles, like the bf16 kernel: each CTA owns
// 128 of the rows and stages only HALF of the B tile, so a CTA pulls 32 KB of operands through L2 per 128 x 256 x 128 block
// of work; at the e4m3 rate (twice bf16) a one-CTA 128 x 128 tile is bound by exactly that traffic.  Roles per CTA:
//   warp 0   : TMA producer - 4-stage ring of {A 128x128, B-half 128x128} e4m3 tiles (128B swizzle) plus the scale records
//              of the stage: this CTA's 128 A rows (512 B) and ALL 256 B rows (2 x 512 B; every CTA applies the scales of
//              the whole B tile to its own accumulator rows); the bytes of both CTAs land on the leader's barrier
//   warp 1   : MMA issuer (leader CTA) - per stage: three tcgen05.cp (scale records -> TMEM, both CTAs at once), then four
//              M256 N256 K32 block-scaled MMAs whose scale-factor ids select the K group's byte of the records
//   warps 2-9: epilogue - the accumulator fills 256 of the 512 TMEM columns and the scale factors need columns of their
//              own, so there is ONE accumulator: the eight warps read all of it into registers (4 x 32 columns per thread),
//              hand it back to the MMA warp at once, and then convert / stage / TMA-store while the next tile's main
//              loop already runs
// Scale layout in global memory: one 512-byte record per (128-row block, 128-wide K block), byte (r % 32) * 16 +
// (r / 32) * 4 + g for row r and K group g: the image `tcgen05.cp 32x128b.warpx4` wants, moved by TMA as a row of a
// [records, 128] 32-bit tensor.  In TMEM the scales of 128 rows take 4 columns (row r: lane r % 32, column r / 32).
// Dense (optionally batched) and grouped-M (expert rows padded to 256, tile -> expert table on the device) enumerations.
// Reference counterparts: DeepGEMM `fp8_gemm_nt` (model/linear/fp8/custom/dense.py:142-150) and the Triton block-scaled
// grouped kernel (model/linear/fp8/custom/grouped.py:136-225), which use 128-element blocks on SM120.
#include "../common/ptx.cuh"
#include "../common/mxfp8.cuh"
#include "gemm.h"

#include <cuda.h>

namespace gm {

constexpr int FM = 128, FN = 256, FK = 128, FSTAGES = 4;
constexpr int FN_HALF = FN / 2;
constexpr int FA_BYTES = FM * FK, FB_BYTES = FN_HALF * FK, SF_BYTES = SF_RECORD_BYTES;
constexpr int FSTAGE_TX = FA_BYTES + FB_BYTES + 3 * SF_BYTES;        // bytes one CTA receives per stage
constexpr int FSTAGE_BYTES = 34 * 1024;                                // stage pitch: tiles stay 1024-byte aligned
constexpr int F_THREADS = 320;
constexpr int F_STAGING = 2 * FM * 128;                                // one staging buffer: two slabs of [128 rows][128 bytes]
constexpr uint32_t F_TMEM_COLS = 512;
constexpr uint32_t COL_SFA = 256, COL_SFB = 264;                       // after the 256-column accumulator
constexpr int F_GROUP_M = 4;                                           // raster: pair rows that share a column sweep

__device__ __forceinline__ uint64_t make_sf_desc(uint32_t smem_addr) {
    // no-swizzle descriptor of a 32-row x 16-byte scale record: 8-row core matrices 128 bytes apart
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>(128 >> 4) << 32;
    d |= 1ull << 46;
    return d;
}

__device__ __forceinline__ void umma_mxf8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate) : "memory");
}
// shared -> TMEM copy of a 512-byte scale record in BOTH CTAs of the pair (each from its own shared memory, same offset)
__device__ __forceinline__ void tmem_cp_sf_pair(uint32_t taddr, uint64_t s_desc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(s_desc) : "memory");
}

struct FTile { int m0, n0, bz, z, m_limit; };

__device__ __forceinline__ int f_total_tiles(const Mxfp8Params& p, int& m_pairs, int& n_tiles) {
    n_tiles = (p.N + FN - 1) / FN;
    m_pairs = p.grouped ? (*p.num_m_tiles + 1) / 2 : (p.M + 2 * FM - 1) / (2 * FM);
    return m_pairs * n_tiles * (p.grouped ? 1 : p.batch);
}

__device__ __forceinline__ FTile f_tile(const Mxfp8Params& p, int tile, int cta_rank, int m_pairs, int n_tiles) {
    const int per = m_pairs * n_tiles;
    FTile t;
    t.z = p.grouped ? 0 : tile / per;
    int r = tile - t.z * per;
    const int group = r / (F_GROUP_M * n_tiles);
    const int first_m = group * F_GROUP_M;
    const int rows = min(F_GROUP_M, m_pairs - first_m);
    r -= group * F_GROUP_M * n_tiles;
    const int mt = 2 * (first_m + r % rows) + cta_rank;
    t.m0 = mt * FM;
    t.n0 = (r / rows) * FN;
    t.bz = p.grouped ? p.tile_expert[mt & ~1] : t.z;       // expert segments are padded to 256 rows: one expert per pair
    t.m_limit = p.grouped ? *p.num_m_tiles * FM : p.M;
    return t;
}

__global__ void __launch_bounds__(F_THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_d, const __grid_constant__ CUtensorMap tmap_sfa,
                  const __grid_constant__ CUtensorMap tmap_sfb, const Mxfp8Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* staging = smem + FSTAGES * FSTAGE_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(staging + 2 * F_STAGING);
    uint64_t* empty = full + FSTAGES;
    uint64_t* acc_full = empty + FSTAGES;
    uint64_t* acc_empty = acc_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta_rank = static_cast<int>(cluster_ctarank());
    if (threadIdx.x == 0) {
        for (int s = 0; s < FSTAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 16);                                // one arrival per epilogue warp of each CTA, on the leader's barrier
        fence_barrier_init();
        tma_prefetch_desc(&tmap_a); tma_prefetch_desc(&tmap_b); tma_prefetch_desc(&tmap_d);
        tma_prefetch_desc(&tmap_sfa); tma_prefetch_desc(&tmap_sfb);
    }
    if (warp == 1) { tmem_alloc_pair(tmem_slot, F_TMEM_COLS); tmem_relinquish_pair(); }
    tc_fence_before();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    int m_pairs, n_tiles;
    const int tiles = f_total_tiles(p, m_pairs, n_tiles);
    const int k_blocks = (p.K + FK - 1) / FK;
    const int first_tile = blockIdx.x >> 1, tile_step = gridDim.x >> 1;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0; uint32_t ph = 0;
            for (int tile = first_tile; tile < tiles && ok; tile += tile_step) {
                const FTile t = f_tile(p, tile, cta_rank, m_pairs, n_tiles);
                // record index of (row block, K block 0) in the [records, 128 words] scale tensors
                const int sfa_rec = (t.z * p.sfa_row_blocks + t.m0 / 128) * k_blocks;
                const int sfb_rec = (t.bz * p.sfb_row_blocks + t.n0 / 128) * k_blocks;
                const bool second_b = t.n0 / 128 + 1 < p.sfb_row_blocks;     // the tile's upper 128 columns exist at all
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&empty[s], ph ^ 1)) { atomicExch(p.status, 401); ok = false; break; }
                    if (cta_rank == 0) mbar_expect_tx(&full[s], 2 * FSTAGE_TX);
                    uint8_t* a_dst = smem + s * FSTAGE_BYTES;
                    uint8_t* b_dst = a_dst + FA_BYTES;
                    uint8_t* sf_dst = b_dst + FB_BYTES;
                    tma_load_3d_pair(a_dst, &tmap_a, &full[s], kb * FK, t.m0, t.z);
                    tma_load_3d_pair(b_dst, &tmap_b, &full[s], kb * FK, t.n0 + cta_rank * FN_HALF, t.bz);
                    // rows beyond the tensors (last row block of A, a B tile narrower than 256) read as zeros: their products are clipped
                    tma_load_3d_pair(sf_dst, &tmap_sfa, &full[s], 0, sfa_rec + kb, 0);
                    tma_load_3d_pair(sf_dst + SF_BYTES, &tmap_sfb, &full[s], 0, sfb_rec + kb, 0);
                    tma_load_3d_pair(sf_dst + 2 * SF_BYTES, &tmap_sfb, &full[s], 0, second_b ? sfb_rec + k_blocks + kb : sfb_rec + kb, 0);
                    if (++s == FSTAGES) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && cta_rank == 0) {
            constexpr uint32_t idesc = make_idesc_mxf8(2 * FM, FN);
            int s = 0; uint32_t ph = 0; uint32_t acc_ph = 0;
            for (int tile = first_tile; tile < tiles && ok; tile += tile_step) {
                if (!mbar_wait(acc_empty, acc_ph ^ 1)) { atomicExch(p.status, 402); ok = false; break; }
                tc_fence_after();
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&full[s], ph)) { atomicExch(p.status, 403); ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * FSTAGE_BYTES), b_addr = a_addr + FA_BYTES, sf_addr = b_addr + FB_BYTES;
                    tmem_cp_sf_pair(tmem_base + COL_SFA, make_sf_desc(sf_addr));
                    tmem_cp_sf_pair(tmem_base + COL_SFB, make_sf_desc(sf_addr + SF_BYTES));
                    tmem_cp_sf_pair(tmem_base + COL_SFB + 4, make_sf_desc(sf_addr + 2 * SF_BYTES));
#pragma unroll
                    for (int g = 0; g < FK / 32; ++g) {
                        const uint64_t adesc = make_smem_desc(a_addr + g * 32, 16, 1024);
                        const uint64_t bdesc = make_smem_desc(b_addr + g * 32, 16, 1024);
                        const uint32_t id = idesc | (static_cast<uint32_t>(g) << 29) | (static_cast<uint32_t>(g) << 4);
                        umma_mxf8_pair(tmem_base, adesc, bdesc, id, tmem_base + COL_SFA, tmem_base + COL_SFB, (kb | g) != 0);
                    }
                    umma_commit_pair(&empty[s]);
                    if (++s == FSTAGES) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                umma_commit_pair(acc_full);
                acc_ph ^= 1;
            }
        }
    } else {
        // Eight epilogue warps; warps with warp % 4 == quad read TMEM lanes 32*quad..32*quad+31.  Thread = accumulator row; the
        // two warps of a quadrant take the two 64-column halves of every 128-column round.
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;
        const int row_in_tile = quad * 32 + lane;
        const bool leader = threadIdx.x == 64;
        const int sw = row_in_tile & 7;
        uint32_t acc_ph = 0;
        uint32_t stores = 0;
        for (int tile = first_tile; tile < tiles && ok; tile += tile_step) {
            const FTile t = f_tile(p, tile, cta_rank, m_pairs, n_tiles);
            if (!mbar_wait(acc_full, acc_ph)) { atomicExch(p.status, 404); ok = false; break; }
            tc_fence_after();
            acc_ph ^= 1;
            uint32_t r[2][2][32];                                  // [round][chunk of this half][column]
#pragma unroll
            for (int round = 0; round < 2; ++round)
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    tmem_ld_32x32b_x32(tmem_base + (round * 4 + half * 2 + j) * 32 + (static_cast<uint32_t>(quad * 32) << 16), r[round][j]);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty, 0);     // the accumulator is free: the next tile's MMAs may start
#pragma unroll
            for (int round = 0; round < 2; ++round) {
                const int round_col0 = t.n0 + round * 128;
                if (round_col0 >= p.N) break;                      // uniform across the CTA
                uint8_t* buf = staging + (stores & 1) * F_STAGING;
                if (leader) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                asm volatile("bar.sync 1, 256;" ::: "memory");
                uint8_t* slab_row = buf + half * (FM * 128) + row_in_tile * 128;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        uint4 o;
                        o.x = pack_bf16x2(__uint_as_float(r[round][j][8 * q]) * p.alpha, __uint_as_float(r[round][j][8 * q + 1]) * p.alpha);
                        o.y = pack_bf16x2(__uint_as_float(r[round][j][8 * q + 2]) * p.alpha, __uint_as_float(r[round][j][8 * q + 3]) * p.alpha);
                        o.z = pack_bf16x2(__uint_as_float(r[round][j][8 * q + 4]) * p.alpha, __uint_as_float(r[round][j][8 * q + 5]) * p.alpha);
                        o.w = pack_bf16x2(__uint_as_float(r[round][j][8 * q + 6]) * p.alpha, __uint_as_float(r[round][j][8 * q + 7]) * p.alpha);
                        *reinterpret_cast<uint4*>(slab_row + (((j * 4 + q) ^ sw) << 4)) = o;
                    }
                }
                fence_proxy_async();
                asm volatile("bar.sync 1, 256;" ::: "memory");
                if (leader) {
                    for (int sl = 0; sl < 2; ++sl) {
                        const int col = round_col0 + sl * 64;
                        if (col >= p.N || t.m0 >= t.m_limit) break;
                        asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                                     ::"l"(&tmap_d), "r"(smem_u32(buf + sl * (FM * 128))), "r"(col), "r"(t.m0), "r"(t.z) : "memory");
                    }
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                ++stores;
            }
        }
        if (leader) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    // common teardown: every path (including a timed-out wait) reaches it, so TMEM is always released
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        if (*reinterpret_cast<volatile int*>(p.status) != 0) {
            const long long start = clock64();
            while (clock64() - start < 200000) {}
        }
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, F_TMEM_COLS);
    }
}

constexpr int F_SMEM = FSTAGES * FSTAGE_BYTES + 2 * F_STAGING + 1024 + 256;

cudaError_t launch_gemm_mxfp8(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const CUtensorMap& tsfa,
                              const CUtensorMap& tsfb, const Mxfp8Params& p, int sms, cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F_SMEM);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms & ~1);
    cfg.blockDim = dim3(F_THREADS);
    cfg.dynamicSmemBytes = F_SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, gemm_mxfp8_kernel, ta, tb, td, tsfa, tsfb, p);
}

// ---- quantisation -------------------------------------------------------------------------------------------------------
// x[rows, cols] bf16 (row pitch ld) -> q[rows, cols] e4m3 + scales; one thread per 32-element block.
// rows beyond `rows_limit` (device-side, optional) are skipped.
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, uint8_t* __restrict__ sf, long long rows, int cols,
                     long long ld, const int* __restrict__ rows_limit) {
    const int groups = cols >> 5;
    const int k_blocks = (cols + 127) >> 7;
    const long long limit = rows_limit ? min(static_cast<long long>(*rows_limit), rows) : rows;
    const long long total = limit * groups;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long row = i / groups;
        const int g = static_cast<int>(i - row * groups);
        const uint4* src = reinterpret_cast<const uint4*>(x + row * ld + g * 32);
        float v[32];
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 raw = src[j];
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(h[e]);
                v[8 * j + 2 * e] = f.x; v[8 * j + 2 * e + 1] = f.y;
                amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
            }
        }
        const uint32_t e8 = e8m0_from_amax(amax);
        const float inv = inv_scale_from_e8m0(e8);
        uint4* dst = reinterpret_cast<uint4*>(q + row * cols + g * 32);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            uint4 o;
            o.x = pack_e4m3x4(v[16 * j] * inv, v[16 * j + 1] * inv, v[16 * j + 2] * inv, v[16 * j + 3] * inv);
            o.y = pack_e4m3x4(v[16 * j + 4] * inv, v[16 * j + 5] * inv, v[16 * j + 6] * inv, v[16 * j + 7] * inv);
            o.z = pack_e4m3x4(v[16 * j + 8] * inv, v[16 * j + 9] * inv, v[16 * j + 10] * inv, v[16 * j + 11] * inv);
            o.w = pack_e4m3x4(v[16 * j + 12] * inv, v[16 * j + 13] * inv, v[16 * j + 14] * inv, v[16 * j + 15] * inv);
            dst[j] = o;
        }
        sf[sf_offset(row, g, k_blocks)] = static_cast<uint8_t>(e8);
    }
}

// Both quantised copies of a weight in one pass over it: w[rows, cols] bf16 (batched over z) ->
//   q  [rows, cols] e4m3, scales per 32 consecutive columns (the forward GEMM contracts over the columns), and
//   qt [cols, rows] e4m3 = the transpose, scales per 32 consecutive ORIGINAL rows (the input-gradient GEMM contracts over them).
// Block = 32 rows x 128 columns, 256 threads.  Row layout: thread (tx, ty) holds columns 4*tx..4*tx+3 of rows ty, ty+8, ty+16,
// ty+24, a 32-column block is 8 adjacent lanes (shuffle reduction).  The values also go to a shared-memory tile, from which
// thread (col = t / 2, half = t % 2) reads 16 rows of one column: the column's 32 rows are the pair's two halves (one
// shuffle), and each thread stores 16 consecutive bytes of the transposed copy (a pair of lanes fills a 32-byte sector).
__global__ void __launch_bounds__(256)
quantize_weight_dual_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q, uint8_t* __restrict__ sf, uint8_t* __restrict__ qt,
                            uint8_t* __restrict__ sft, int rows, int cols, long long batch_stride, long long sf_batch_stride,
                            long long sft_batch_stride) {
    __shared__ __align__(16) float tile[32][132];
    const int z = blockIdx.z;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c0 = blockIdx.x * 128, r0 = blockIdx.y * 32;
    const int c = c0 + 4 * tx;
    const __nv_bfloat16* src = w + z * batch_stride;
    const int kb_row = (cols + 127) >> 7, kb_col = (rows + 127) >> 7;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + ty + 8 * i;
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        if (r < rows && c < cols) {
            const uint2 raw = *reinterpret_cast<const uint2*>(src + static_cast<long long>(r) * cols + c);
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
            const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
            v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
        }
        *reinterpret_cast<float4*>(&tile[ty + 8 * i][4 * tx]) = make_float4(v[0], v[1], v[2], v[3]);
        uint32_t out[1];
        const uint32_t e8 = quantize_block_lanes<4>(v, out);
        if (r < rows && c < cols) {
            *reinterpret_cast<uint32_t*>(q + z * batch_stride + static_cast<long long>(r) * cols + c) = out[0];
            if ((tx & 7) == 0) sf[z * sf_batch_stride + sf_offset(r, c >> 5, kb_row)] = static_cast<uint8_t>(e8);
        }
    }
    __syncthreads();
    const int col = threadIdx.x >> 1, hf = threadIdx.x & 1;
    float u[16];
    float amax = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) { u[k] = tile[hf * 16 + k][col]; amax = fmaxf(amax, fabsf(u[k])); }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    const uint32_t e8 = e8m0_from_amax(amax);
    const float inv = inv_scale_from_e8m0(e8);
    if (c0 + col < cols && r0 + hf * 16 < rows) {
        uint4 o;
        o.x = pack_e4m3x4(u[0] * inv, u[1] * inv, u[2] * inv, u[3] * inv);
        o.y = pack_e4m3x4(u[4] * inv, u[5] * inv, u[6] * inv, u[7] * inv);
        o.z = pack_e4m3x4(u[8] * inv, u[9] * inv, u[10] * inv, u[11] * inv);
        o.w = pack_e4m3x4(u[12] * inv, u[13] * inv, u[14] * inv, u[15] * inv);
        *reinterpret_cast<uint4*>(qt + z * batch_stride + static_cast<long long>(c0 + col) * rows + r0 + hf * 16) = o;
        if (hf == 0) sft[z * sft_batch_stride + sf_offset(c0 + col, r0 >> 5, kb_col)] = static_cast<uint8_t>(e8);
    }
}

void launch_quantize_rows(const void* x, void* q, void* sf, long long rows, int cols, long long ld, const int* rows_limit, cudaStream_t s) {
    const long long total = rows * (cols / 32);
    const int blocks = static_cast<int>(total / 256 + 1 < 4736 ? total / 256 + 1 : 4736);
    quantize_rows_kernel<<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), rows,
                                                cols, ld, rows_limit);
}

void launch_quantize_weight_dual(const void* w, void* q, void* sf, void* qt, void* sft, int batch, int rows, int cols, long long sf_batch_stride,
                                 long long sft_batch_stride, cudaStream_t s) {
    dim3 grid((cols + 127) / 128, (rows + 31) / 32, batch);
    quantize_weight_dual_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(w), static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf),
                                                     static_cast<uint8_t*>(qt), static_cast<uint8_t*>(sft), rows, cols,
                                                     static_cast<long long>(rows) * cols, sf_batch_stride, sft_batch_stride);
}

}  // namespace gm

// Block-scaled MXFP8 GEMM for sm_100a: D[M,N] (bf16) = A[M,K] * B[N,K]^T with e4m3 operands and one UE8M0
// (power-of-two) scale per 32 consecutive K elements of every row of A and of B, multiplied in by the tensor core
// (tcgen05.mma kind::mxf8f6f4.block_scale), fp32 accumulation in TMEM.
//
// Same persistent, warp-specialised structure as the bf16 kernel (TMA ring -> tcgen05 -> TMEM -> staged TMA store)
// with 128 x 128 output tiles, 128-element K blocks (four K=32 MMAs) and, per stage, the scale factors of the tile:
//   global scale layout: for every 128-row block and every 128-wide K block one 512-byte record; inside a record the
//   byte of (row r, k-group g) sits at (r % 32) * 16 + (r / 32) * 4 + g.  That is exactly the image tcgen05.cp
//   (32x128b.warpx4) wants in shared memory: one bulk copy per record, one tcgen05.cp per record into 4 TMEM columns,
//   and the MMA of k-group g selects byte g through the scale-factor ids of the instruction descriptor.
// Dense (optionally batched) and grouped-M (expert rows, tile -> expert table on the device) enumerations.
// Reference counterparts: DeepGEMM `fp8_gemm_nt` (model/linear/fp8/custom/dense.py:142-150) and the Triton block-scaled
// grouped kernel (model/linear/fp8/custom/grouped.py:136-225), which use 128-element blocks on SM120.
#include "../common/ptx.cuh"
#include "gemm.h"

#include <cuda.h>

namespace gm {

constexpr int FM = 128, FN = 128, FK = 128, FSTAGES = 5;
constexpr int FA_BYTES = FM * FK, FB_BYTES = FN * FK, SF_BYTES = 512;
constexpr int FSTAGE_BYTES = FA_BYTES + FB_BYTES + 2 * SF_BYTES;
constexpr int F_THREADS = 192;
constexpr int F_STAGING = 2 * FM * 128;
constexpr uint32_t F_TMEM_COLS = 512;
constexpr uint32_t COL_SFA = 256, COL_SFB = 260;      // after the two 128-column accumulators
constexpr int F_GROUP_M = 8;

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// no-swizzle descriptor of a 32-row x 16-byte scale record: 8-row core matrices 128 bytes apart
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
    d |= static_cast<uint64_t>(128 >> 4) << 32;
    d |= 1ull << 46;
    return d;
}

__device__ __forceinline__ void umma_mxf8_bs(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                             uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], p;\n\t}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate) : "memory");
}

struct FTile { int m0, n0, bz, m_limit; };

__device__ __forceinline__ int f_total_tiles(const Mxfp8Params& p, int& m_tiles, int& n_tiles) {
    n_tiles = (p.N + FN - 1) / FN;
    m_tiles = p.grouped ? *p.num_m_tiles : (p.M + FM - 1) / FM;
    return m_tiles * n_tiles * (p.grouped ? 1 : p.batch);
}

__device__ __forceinline__ FTile f_tile(const Mxfp8Params& p, int tile, int m_tiles, int n_tiles, int& z) {
    const int per = m_tiles * n_tiles;
    z = p.grouped ? 0 : tile / per;
    int r = tile - z * per;
    const int group = r / (F_GROUP_M * n_tiles);
    const int first_m = group * F_GROUP_M;
    const int rows = min(F_GROUP_M, m_tiles - first_m);
    r -= group * F_GROUP_M * n_tiles;
    FTile t;
    const int mt = first_m + r % rows;
    t.m0 = mt * FM;
    t.n0 = (r / rows) * FN;
    t.bz = p.grouped ? p.tile_expert[mt] : z;
    t.m_limit = p.grouped ? m_tiles * FM : p.M;
    return t;
}

__global__ void __launch_bounds__(F_THREADS, 1)
gemm_mxfp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ CUtensorMap tmap_d, const Mxfp8Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* staging = smem + FSTAGES * FSTAGE_BYTES;
    uint64_t* full = reinterpret_cast<uint64_t*>(staging + F_STAGING);
    uint64_t* empty = full + FSTAGES;
    uint64_t* acc_full = empty + FSTAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < FSTAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 128); }
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, F_TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    int m_tiles, n_tiles;
    const int tiles = f_total_tiles(p, m_tiles, n_tiles);
    const int k_blocks = (p.K + FK - 1) / FK;
    const int a_row_blocks = p.sfa_row_blocks, b_row_blocks = p.sfb_row_blocks;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0; uint32_t ph = 0;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                int z;
                const FTile t = f_tile(p, tile, m_tiles, n_tiles, z);
                const uint8_t* sfa = p.sfa + ((static_cast<long long>(z) * a_row_blocks + t.m0 / FM) * k_blocks) * SF_BYTES;
                const uint8_t* sfb = p.sfb + ((static_cast<long long>(t.bz) * b_row_blocks + t.n0 / FN) * k_blocks) * SF_BYTES;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&empty[s], ph ^ 1)) { atomicExch(p.status, 401); ok = false; break; }
                    mbar_expect_tx(&full[s], FSTAGE_BYTES);
                    uint8_t* a_dst = smem + s * FSTAGE_BYTES;
                    uint8_t* b_dst = a_dst + FA_BYTES;
                    tma_load_3d(a_dst, &tmap_a, &full[s], kb * FK, t.m0, z);
                    tma_load_3d(b_dst, &tmap_b, &full[s], kb * FK, t.n0, t.bz);
                    bulk_load(b_dst + FB_BYTES, sfa + kb * SF_BYTES, SF_BYTES, &full[s]);
                    bulk_load(b_dst + FB_BYTES + SF_BYTES, sfb + kb * SF_BYTES, SF_BYTES, &full[s]);
                    if (++s == FSTAGES) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_mxf8(FM, FN);
            int s = 0; uint32_t ph = 0; int acc = 0; uint32_t acc_ph = 0;
            for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
                if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1)) { atomicExch(p.status, 402); ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * FN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait(&full[s], ph)) { atomicExch(p.status, 403); ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + s * FSTAGE_BYTES), b_addr = a_addr + FA_BYTES, sf_addr = b_addr + FB_BYTES;
                    tmem_cp_32x128b_warpx4(tmem_base + COL_SFA, make_sf_desc(sf_addr));
                    tmem_cp_32x128b_warpx4(tmem_base + COL_SFB, make_sf_desc(sf_addr + SF_BYTES));
#pragma unroll
                    for (int g = 0; g < FK / 32; ++g) {
                        const uint64_t adesc = make_smem_desc(a_addr + g * 32, 16, 1024);
                        const uint64_t bdesc = make_smem_desc(b_addr + g * 32, 16, 1024);
                        const uint32_t id = idesc | (static_cast<uint32_t>(g) << 29) | (static_cast<uint32_t>(g) << 4);
                        umma_mxf8_bs(d_tmem, adesc, bdesc, id, tmem_base + COL_SFA, tmem_base + COL_SFB, (kb | g) != 0);
                    }
                    umma_commit(&empty[s]);
                    if (++s == FSTAGES) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                umma_commit(&acc_full[acc]);
                if (++acc == 2) { acc = 0; acc_ph ^= 1; }
            }
        }
    } else {
        const int quad = warp & 3;
        const int row_in_tile = quad * 32 + lane;
        const bool leader = threadIdx.x == 64;
        uint8_t* my_row = staging + row_in_tile * 128;
        const int sw = row_in_tile & 7;
        int acc = 0; uint32_t acc_ph = 0;
        for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
            int z;
            const FTile t = f_tile(p, tile, m_tiles, n_tiles, z);
            if (!mbar_wait(&acc_full[acc], acc_ph)) { atomicExch(p.status, 404); ok = false; break; }
            tc_fence_after();
            if (leader) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                uint32_t r[32];
                tmem_ld_32x32b_x32(tmem_base + acc * FN + cc * 32 + (static_cast<uint32_t>(quad * 32) << 16), r);
                tmem_ld_wait();
                uint8_t* slab = my_row + (cc >> 1) * (FM * 128);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint4 o;
                    o.x = pack_bf16x2(__uint_as_float(r[8 * q]) * p.alpha, __uint_as_float(r[8 * q + 1]) * p.alpha);
                    o.y = pack_bf16x2(__uint_as_float(r[8 * q + 2]) * p.alpha, __uint_as_float(r[8 * q + 3]) * p.alpha);
                    o.z = pack_bf16x2(__uint_as_float(r[8 * q + 4]) * p.alpha, __uint_as_float(r[8 * q + 5]) * p.alpha);
                    o.w = pack_bf16x2(__uint_as_float(r[8 * q + 6]) * p.alpha, __uint_as_float(r[8 * q + 7]) * p.alpha);
                    *reinterpret_cast<uint4*>(slab + ((((cc & 1) * 4 + q) ^ sw) << 4)) = o;
                }
            }
            tc_fence_before();
            mbar_arrive(&acc_empty[acc]);
            fence_proxy_async();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (leader) {
                for (int sl = 0; sl < 2; ++sl) {
                    const int col = t.n0 + sl * 64;
                    if (col >= p.N) break;
                    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                                 ::"l"(&tmap_d), "r"(smem_u32(staging + sl * (FM * 128))), "r"(col), "r"(t.m0), "r"(z) : "memory");
                }
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
        if (leader) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        if (*reinterpret_cast<volatile int*>(p.status) != 0) {
            const long long start = clock64();
            while (clock64() - start < 200000) {}
        }
        tc_fence_after();
        tmem_dealloc(tmem_base, F_TMEM_COLS);
    }
}

constexpr int F_SMEM = FSTAGES * FSTAGE_BYTES + F_STAGING + 1024 + 256;

cudaError_t launch_gemm_mxfp8(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const Mxfp8Params& p, int sms,
                              cudaStream_t stream) {
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_mxfp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F_SMEM);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    gemm_mxfp8_kernel<<<sms, F_THREADS, F_SMEM, stream>>>(ta, tb, td, p);
    return cudaGetLastError();
}

// ---- quantisation -------------------------------------------------------------------------------------------------------
// UE8M0 exponent byte of the smallest power of two >= amax / 448 (integer rounding of the fp32 bit pattern), 127 for amax == 0.
__device__ __forceinline__ uint32_t e8m0_from_amax(float amax) {
    if (amax == 0.f) return 127u;
    uint32_t bits = __float_as_uint(amax * (1.f / 448.f));
    bits = (bits + 0x007FFFFFu) & 0x7F800000u;
    uint32_t e = bits >> 23;
    return e < 1u ? 1u : (e > 254u ? 254u : e);
}
__device__ __forceinline__ float inv_scale_from_e8m0(uint32_t e) { return __uint_as_float((254u - e) << 23); }

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(a), "f"(b));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(c), "f"(d));
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

__device__ __forceinline__ long long sf_offset(long long row, int k_group, int k_blocks) {
    const long long rb = row >> 7;
    const int r = static_cast<int>(row & 127);
    return (rb * k_blocks + (k_group >> 2)) * SF_BYTES + (r & 31) * 16 + (r >> 5) * 4 + (k_group & 3);
}

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

// w[rows, cols] bf16 (batched over z) -> q[cols, rows] e4m3 = transposed copy, scaled in groups of 32 along the ORIGINAL row index
// (the contraction dimension of the input-gradient GEMM).  Block = 32 x 32 tile through shared memory.
__global__ void __launch_bounds__(256)
quantize_transposed_kernel(const __nv_bfloat16* __restrict__ w, uint8_t* __restrict__ q, uint8_t* __restrict__ sf, int rows, int cols,
                           long long batch_stride_in, long long batch_stride_q, long long batch_stride_sf) {
    __shared__ float tile[32][33];
    const int z = blockIdx.z;
    const int r0 = blockIdx.y * 32, c0 = blockIdx.x * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const __nv_bfloat16* src = w + z * batch_stride_in;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + ty + 8 * i, c = c0 + tx;
        tile[ty + 8 * i][tx] = (r < rows && c < cols) ? __bfloat162float(src[static_cast<long long>(r) * cols + c]) : 0.f;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int c = c0 + threadIdx.x;                     // output row (original column); its 32 values run along original rows
        if (c < cols) {
            float amax = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(tile[j][threadIdx.x]));
            const uint32_t e8 = e8m0_from_amax(amax);
            const float inv = inv_scale_from_e8m0(e8);
            uint4* dst = reinterpret_cast<uint4*>(q + z * batch_stride_q + static_cast<long long>(c) * rows + r0);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint4 o;
                o.x = pack_e4m3x4(tile[16 * j][threadIdx.x] * inv, tile[16 * j + 1][threadIdx.x] * inv, tile[16 * j + 2][threadIdx.x] * inv, tile[16 * j + 3][threadIdx.x] * inv);
                o.y = pack_e4m3x4(tile[16 * j + 4][threadIdx.x] * inv, tile[16 * j + 5][threadIdx.x] * inv, tile[16 * j + 6][threadIdx.x] * inv, tile[16 * j + 7][threadIdx.x] * inv);
                o.z = pack_e4m3x4(tile[16 * j + 8][threadIdx.x] * inv, tile[16 * j + 9][threadIdx.x] * inv, tile[16 * j + 10][threadIdx.x] * inv, tile[16 * j + 11][threadIdx.x] * inv);
                o.w = pack_e4m3x4(tile[16 * j + 12][threadIdx.x] * inv, tile[16 * j + 13][threadIdx.x] * inv, tile[16 * j + 14][threadIdx.x] * inv, tile[16 * j + 15][threadIdx.x] * inv);
                dst[j] = o;
            }
            const int k_blocks = (rows + 127) >> 7;
            sf[z * batch_stride_sf + sf_offset(c, r0 >> 5, k_blocks)] = static_cast<uint8_t>(e8);
        }
    }
}

void launch_quantize_rows(const void* x, void* q, void* sf, long long rows, int cols, long long ld, const int* rows_limit, cudaStream_t s) {
    const long long total = rows * (cols / 32);
    const int blocks = static_cast<int>(total / 256 + 1 < 4736 ? total / 256 + 1 : 4736);
    quantize_rows_kernel<<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), rows,
                                                cols, ld, rows_limit);
}

void launch_quantize_transposed(const void* w, void* q, void* sf, int batch, int rows, int cols, long long sf_batch_stride, cudaStream_t s) {
    dim3 grid((cols + 31) / 32, (rows + 31) / 32, batch);
    quantize_transposed_kernel<<<grid, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(w), static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf),
                                                    rows, cols, static_cast<long long>(rows) * cols, static_cast<long long>(rows) * cols, sf_batch_stride);
}

}  // namespace gm

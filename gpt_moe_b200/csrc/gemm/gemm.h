// Host-visible interface of the tcgen05 GEMM kernels.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gm {

enum GemmMode : int { GEMM_DENSE = 0, GEMM_GROUPED_M = 1, GEMM_GROUPED_K = 2 };

struct GemmParams {
    int M, N, K;                 // per-problem output rows, output columns, contraction length
    int batch;                   // DENSE: batched problems; GROUPED_K: number of experts
    int mode;
    void* D;                     // output, bf16 or fp32
    long long ldd, d_batch_stride;
    const void* C;               // optional bf16 addend: D = alpha*acc + beta*C
    long long ldc, c_batch_stride;
    float alpha, beta;
    int out_fp32, accumulate;    // accumulate: D += result (fp32 output only)
    int split_k;                 // >1: the K loop is shared by this many CTAs per tile, partials meet in a TMA reduce-add (fp32 output)
    const int* tile_expert;      // GROUPED_M: expert of each 128-row tile
    const int* num_m_tiles;      // GROUPED_M: number of 128-row tiles (device scalar)
    const int* seg_ends;         // GROUPED_K: cumulative padded row ends per expert
    int symmetric;               // DENSE, M == N, bf16 output: the result is known to be symmetric (X X^T); only tiles on or above the
                                 // diagonal are computed and every off-diagonal tile is also stored transposed
    const float* batch_sumsq;    // DENSE, optional: per-batch sum of squares; s = 1 / (sqrt(sumsq[z]) * 1.02 + 1e-6) is Muon's Frobenius
    int scale_mode;              // normalisation of an operand, folded into the epilogue: 1 -> alpha * s and beta * s, 2 -> alpha * s * s
    int* status;                 // device word; kernels write a non-zero code if a bounded wait gives up
};

// Encode a 3-D tiled tensor map over a row-major bf16 tensor [batch, rows, cols] (cols contiguous) with a
// {box_cols, box_rows, 1} box and 128-byte swizzle.  Returns false if the driver entry point is unavailable
// or rejects the arguments.
bool make_tensor_map_bf16(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t batch,
                          uint64_t row_stride_elems, uint64_t batch_stride_elems, uint32_t box_cols, uint32_t box_rows);
bool make_tensor_map(CUtensorMap* out, const void* base, int elem_bytes, uint64_t cols, uint64_t rows, uint64_t batch,
                     uint64_t row_stride_bytes, uint64_t batch_stride_bytes, uint32_t box_cols, uint32_t box_rows,
                     int swizzle_bytes);

cudaError_t launch_gemm_bf16(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const GemmParams& p, bool a_mn,
                             bool b_mn, int sms, cudaStream_t stream);

// Block-scaled MXFP8 GEMM: D[M,N] (bf16) = alpha * A[M,K] B[N,K]^T, e4m3 operands, UE8M0 scales per 32 elements of K.
// Scales are stored as 512-byte records [row block of 128][K block of 128]; byte (r % 32) * 16 + (r / 32) * 4 + g of a record
// belongs to row r of the block and the g-th group of 32 inside the K block.
struct Mxfp8Params {
    int M, N, K;
    int batch;                   // dense: batched problems
    int grouped;                 // 1: A rows are expert-major padded segments, B is [E, N, K]
    const uint8_t* sfa;          // [batch, sfa_row_blocks, K/128, 512]
    const uint8_t* sfb;          // [batch or E, sfb_row_blocks, K/128, 512]
    int sfa_row_blocks, sfb_row_blocks;
    float alpha;
    const int* tile_expert;
    const int* num_m_tiles;
    int* status;
};

// tsfa / tsfb: maps over the scale arrays seen as [records, 128] 32-bit words (one 512-byte record per row), box {128, 1}
cudaError_t launch_gemm_mxfp8(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const CUtensorMap& tsfa,
                              const CUtensorMap& tsfb, const Mxfp8Params& p, int sms, cudaStream_t stream);
// x [rows, cols] bf16 with row pitch ld -> q [rows, cols] e4m3 and scale records; rows at or beyond *rows_limit (optional,
// device) are left untouched.  cols must be a multiple of 32.
void launch_quantize_rows(const void* x, void* q, void* sf, long long rows, int cols, long long ld, const int* rows_limit, cudaStream_t s);
// w [batch, rows, cols] bf16 -> q [batch, rows, cols] e4m3 with scales along the columns AND qt [batch, cols, rows] e4m3 (the
// transpose) with scales along the original rows, in one pass.  rows and cols must be multiples of 32.
void launch_quantize_weight_dual(const void* w, void* q, void* sf, void* qt, void* sft, int batch, int rows, int cols, long long sf_batch_stride,
                                 long long sft_batch_stride, cudaStream_t s);

}  // namespace gm

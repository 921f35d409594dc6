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

}  // namespace gm

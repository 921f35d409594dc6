// Declarations of the launchers defined in the .cu files (raw pointers, explicit stream).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace gm {

// fused/norm_rope.cu
bool norm_dim_supported(int d);
bool launch_rmsnorm_fwd(const void* x, bool x_fp32, const void* branch, const float* alpha, const float* beta, void* x_out,
                        const float* w, void* y, float* rstd, int rows, int d, float eps, cudaStream_t s);
int rmsnorm_bwd_blocks(int rows);
bool launch_rmsnorm_bwd(const void* dy, const void* x, bool x_fp32, const float* w, const float* rstd, const void* dres, void* dx,
                        float* dw_partial, float* dw, int dw_accumulate, int rows, int d, cudaStream_t s);
void launch_column_sum(const float* partial, float* out, int rows, int cols, int accumulate, cudaStream_t s);
int rope_blocks(long long tokens, int heads);
bool launch_rope_qknorm(bool bwd, int D, const void* x, const void* dy, void* out, const float* cos_t, const float* sin_t,
                        const float* q_scale, const float* k_scale, float* dscale_partial, long long tokens, int seq_len,
                        int q_heads, int k_heads, long long x_stride, long long o_stride, float eps, int rms, float smin,
                        float smax, cudaStream_t s);

}  // namespace gm

// Declarations of the launchers defined in the .cu files (raw pointers, explicit stream).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace gm {

// fused/norm_rope.cu
bool norm_dim_supported(int d);
bool launch_rmsnorm_fwd(const void* x, bool x_fp32, const void* branch, const float* alpha, const float* beta, void* x_out,
                        const float* w, void* y, float* rstd, void* yq, void* ysf, int rows, int d, float eps, cudaStream_t s);
int rmsnorm_bwd_blocks(int rows);
bool launch_rmsnorm_bwd(const void* dy, const void* x, bool x_fp32, const float* w, const float* rstd, const void* dres, void* dx,
                        float* dw_partial, float* dw, int dw_accumulate, int rows, int d, cudaStream_t s);
int residual_bwd_blocks(long long n);
void launch_residual_bwd(const float* dxn, const void* branch, const float* beta, void* dbranch, float* partial, float* dbeta,
                         long long n, cudaStream_t s);
void launch_column_sum(const float* partial, float* out, int rows, int cols, int accumulate, cudaStream_t s);
int rope_blocks(long long tokens, int heads);
bool launch_rope_qknorm(bool bwd, int D, const void* x, const void* dy, void* out, const float* cos_t, const float* sin_t,
                        const float* q_scale, const float* k_scale, float* dscale_partial, long long tokens, int seq_len,
                        int q_heads, int k_heads, long long x_stride, long long o_stride, float eps, int rms, float smin,
                        float smax, int copy_cols, const float* dq32, long long dq_stride, void* gq, void* gsf, int gq_width,
                        cudaStream_t s);

// fused/moe.cu
bool launch_route(const long long* idx, int slots, int experts, int* chunk_hist, int* chunk_start, int* counts, int* seg_ends,
                  int* tile_expert, int* meta, int* dest, int* src_of_row, cudaStream_t s);
// q / sf (optional, every launcher below that has them): MXFP8 copy of the bf16 matrix the kernel writes, emitted in the same pass
void launch_gather_rows(const void* hidden, const int* src_of_row, const int* meta, void* packed, void* q, void* sf, int d, int top_k,
                        int cap_rows, int tokens, cudaStream_t s);
// gates == nullptr: unit gates
void launch_combine_fwd(const void* y, const int* dest, const float* gates, void* out, int tokens, int d, int top_k, int y_rows, cudaStream_t s);
void launch_combine_bwd(const void* dout, const void* y, const int* src_of_row, const float* gates, const int* meta, void* dy,
                        float* dgates, void* q, void* sf, int d, int top_k, int cap_rows, int tokens, cudaStream_t s);
// bounds-checked build: first recorded code of each translation unit (0 = none; reading clears it); always 0 in the normal build
int read_bounds_moe();
int read_bounds_loss();
int read_bounds_router();
void launch_activation_fwd(const void* pre, void* act, const int* meta, void* q, void* sf, int rows, int h, int kind, cudaStream_t s);
void launch_activation_bwd(const void* dact, const void* pre, void* dpre, const int* meta, void* q, void* sf, int rows, int h, int kind,
                           cudaStream_t s);

// attention/mla_decode.cu
int mla_decode_splits(int B, int T, int S);
bool mla_decode_supported(int H, int Hkv, int r, int dr);
bool launch_mla_decode(const float* q_latent, const float* q_rope, const void* latent, const void* rope, const void* key_gain,
                       long long latent_bs, long long rope_bs, long long gain_bs, float* part_ctx, float* part_ml, float* context, int B, int T,
                       int H, int Hkv, int r, int dr, int S, int splits, int start, int window, float scale, float softcap, cudaStream_t s);

// fused/router.cu
int router_blocks(int tokens);
bool launch_router_fwd(const void* logits, bool bf16, long long* top_idx, float* gates, float* prob_partial, float* count_partial,
                       float* prob_sums, float* counts, float* balance, int tokens, int experts, int top_k, int renormalise, cudaStream_t s);
bool launch_router_bwd(const void* logits, bool bf16, const long long* top_idx, const float* dgates, const float* dbalance, const float* counts,
                       void* dlogits, int tokens, int experts, int top_k, int renormalise, cudaStream_t s);

// fused/loss_optim.cu
void launch_ce_fwd_bwd(void* logits, const long long* targets, float* loss, const float* grad_scale, int rows, int vocab,
                       long long row_stride, long long ignore_index, int write_grad, cudaStream_t s);
void launch_adamw(float* p, const float* g, void* m, void* v, bool moments_bf16, void* p_bf16, long long n, float lr, float beta1,
                  float beta2, float eps, float wd, float bc1, float bc2_sqrt, float grad_scale, cudaStream_t s);
void launch_muon_prepare(const float* const* grads, float* const* bufs, void* packed, float* sumsq, int n_mats, int rows, int cols,
                         long long g_stride, long long b_stride, float momentum, int nesterov, int transpose, float grad_scale,
                         cudaStream_t s);
void launch_muon_apply(float* const* weights, void* const* weights_bf16, const void* update, int n_mats, int rows, int cols,
                       long long w_stride, float alpha, int transpose, cudaStream_t s);
void launch_cast_bf16(const float* src, void* dst, long long n, cudaStream_t s);

void launch_muon_normalize(void* packed, const float* sumsq, int n_mats, long long per_matrix, cudaStream_t s);

// comm/fused_comm.cu
bool launch_rs_muon_prepare(const float* const* grads, float* const* bufs, void* packed, float* sumsq, int n_mats, int rows, int cols,
                            long long g_stride, long long b_stride, float momentum, int nesterov, int transpose,
                            const long long* peer_deltas, int world, const float* grad_base, const void* shadow_base, cudaStream_t s);
bool launch_muon_apply_push(float* const* weights, void* const* weights_bf16, const void* update, int n_mats, int rows, int cols,
                            long long w_stride, long long wb_stride, float alpha, int transpose, const long long* peer_deltas, int world,
                            cudaStream_t s);
bool launch_adamw_sharded(float* params, const float* grads, void* m, void* v, bool moments_bf16, const float* decay, long long lo,
                          long long n, float lr, float beta1, float beta2, float eps, float bc1, float bc2_sqrt,
                          const long long* grad_deltas, const long long* param_deltas, int world, cudaStream_t s);

bool launch_flag_signal(int* flags, const long long* deltas, int world, int index, int value, const int* value_word, cudaStream_t s);
bool launch_flag_wait(const int* flags, int first, int world, int value, const int* value_word, int* status, cudaStream_t s);
void launch_bump_word(int* word, cudaStream_t s);
bool launch_peer_barrier(int* flags, const long long* deltas, int world, int me, int* epoch_word, int* status, long long budget_cycles,
                         cudaStream_t s);

// ---- expert-parallel dispatch / combine over peer memory (comm/ep_comm.cu) -------------------------------------------
bool launch_ep_push_counts(const int* counts, int* table, const long long* deltas, int world, int me, int experts, cudaStream_t s);
bool launch_ep_plan(const int* table, int* my_base, int* seg_ends, int* valid_ends, int* tile_expert, int* meta, int world, int me,
                    int experts, int per_rank, int cap_rows, int* status, cudaStream_t s);
void launch_ep_zero_pads(void* buf, const int* seg_ends, const int* valid_ends, int per_rank, int d, cudaStream_t s);
bool launch_ep_dispatch(const void* src, const long long* idx, const int* dest, const int* local_seg_ends, const int* my_base,
                        const float* gates, const void* saved_rows, float* dgates, void* recv, int* route_row, const long long* deltas,
                        int world, int slots, int d, int top_k, int per_rank, int cap_rows, int* status, cudaStream_t s);
bool launch_ep_combine(const void* ret, const long long* idx, const int* route_row, const float* gates, void* out, void* keep_rows,
                       const long long* deltas, int world, int tokens, int d, int top_k, int per_rank, int cap_rows, cudaStream_t s);

// csrc/bench/mma_issue.cu: clocks to issue / to complete `count` chained tcgen05.mma instructions of one shape (see the file)
cudaError_t launch_mma_issue(int shape, long long* out, int count, int* status, cudaStream_t s);

}  // namespace gm

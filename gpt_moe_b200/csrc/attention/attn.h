// Host-visible interface of the tcgen05 attention kernels (value heads 64 wide; query/key heads 64 or 128 wide).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace gm {

struct AttnParams {
    int batch, heads, seq_len;      // q heads
    int group;                      // q heads per kv head
    int qk_dim;                     // width of a query / key head: 64 or 128
    int q_col0, k_col0, v_col0;     // first column of head 0 inside each tensor map
    int window;                     // inclusive look-back W (a query sees keys q-W..q); >= seq_len means plain causal
    const int* window_ptr;          // optional device-resident window (overrides `window`; clamped to [0, seq_len] by the kernels), so
                                    // that a window-schedule step is a write to that word and a captured launch stays valid
    const int* doc_start;           // optional [batch * seq]: position (inside its sequence) of the first token of each token's document;
                                    // a query then sees keys max(q - W, doc_start[q]) .. q (documents are contiguous runs of tokens)
    float scale_log2e;              // softmax scale * log2(e)
    float scale;                    // softmax scale
    float softcap;                  // > 0: logits are soft-capped, z = softcap * tanh(scale * s / softcap), before the softmax
    void* out;                      // forward: O [tokens, heads*64] bf16
    long long out_stride;
    uint8_t* out_q;                 // optional MXFP8 copy of O (row pitch heads*64): e4m3 payload ...
    uint8_t* out_sf;                // ... and its scale records (the output projection's GEMM operand, written by the epilogue)
    float* lse;                     // [batch, heads, seq] natural-log LSE of the scaled scores
    // backward
    const float* delta;             // [batch, heads, seq] rowsum(dO * O)
    float* dq_accum;                // [tokens, heads*qk_dim] fp32, zero-initialised; reduced into by TMA
    void* dk;                       // [tokens, kv_heads*qk_dim] bf16; dv is [tokens, kv_heads*64] with its own pitch
    void* dv;
    long long dkv_stride, dv_stride;
    int* status;
    int single_tile;                // 1 keeps the call on the basic kernel of its direction: one query tile per CTA (forward),
                                    // score and gradient products in program order (backward)
};

cudaError_t launch_attn_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, cudaStream_t stream);

// Forward with two query tiles per CTA (attn_fwd_dual.cu): 64-wide heads, no document masking, sequence length a multiple of 256.
// launch_attn_fwd picks it when it applies and `single_tile` is 0.
bool attn_fwd_dual_supported(const AttnParams& p);
cudaError_t launch_attn_fwd_dual(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, cudaStream_t stream);

// Backward with the next tile's score products issued ahead of the current gradient products (attn_bwd_pipe.cu): 64-wide heads.
// launch_attn_bwd picks it when it applies and `single_tile` is 0.
cudaError_t launch_attn_bwd_pipe(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                                 const CUtensorMap& tdq, const AttnParams& p, cudaStream_t stream);

cudaError_t launch_attn_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                            const CUtensorMap& tdq, const AttnParams& p, const void* d_out, const void* out, long long do_stride,
                            long long o_stride, float* delta, cudaStream_t stream);

}  // namespace gm

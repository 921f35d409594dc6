// Bindings of the non-GEMM kernels: tensors in, raw pointers out.  Shape/dtype checks live here so the
// kernels can assume aligned, contiguous data.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "guarded_alloc.h"
#include "kernels.h"
#include "kernels_decl.h"

namespace gm {
namespace {

#define GM_CHECK(cond, msg) TORCH_CHECK(cond, "gpt_moe_b200: ", msg)
using torch::Tensor;
using OptTensor = c10::optional<Tensor>;

cudaStream_t stream() { return at::cuda::getCurrentCUDAStream().stream(); }
const float* fptr(const OptTensor& t) { return t.has_value() ? t->data_ptr<float>() : nullptr; }
void check_bf16(const Tensor& t, const char* name) {
    GM_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.is_contiguous(), std::string(name) + " must be a contiguous CUDA bf16 tensor");
}
// MXFP8 copy of a [rows, cols] matrix: e4m3 payload (uint8 [rows, cols]) and scale records (uint8 [ceil(rows/128) * ceil(cols/128) * 512]).
// The scale array is not cleared: every byte that belongs to a row the producer writes is written by it, the others belong to
// rows the GEMM clips.
struct QuantOut { Tensor q, sf; uint8_t* qp = nullptr; uint8_t* sp = nullptr; };
QuantOut alloc_quant(bool wanted, int64_t rows, int64_t cols, const Tensor& like) {
    QuantOut o;
    if (!wanted) return o;
    GM_CHECK(cols % 32 == 0, "MXFP8 copy: the row width must be a multiple of 32");
    auto opt = like.options().dtype(torch::kUInt8);
    o.q = gm::out_empty({rows, cols}, opt);
    o.sf = gm::out_empty({((rows + 127) / 128) * ((cols + 127) / 128) * 512}, opt);
    o.qp = o.q.data_ptr<uint8_t>();
    o.sp = o.sf.data_ptr<uint8_t>();
    return o;
}

// y = rmsnorm(x_new) * w with x_new = alpha*x + beta*branch when a branch is given.  Returns (y, rstd, x_new) and, with
// `quantize`, the MXFP8 copy of y as two more tensors (payload, scale records).
std::vector<Tensor> rmsnorm_fwd(const Tensor& x, const OptTensor& w, double eps, const OptTensor& branch, const OptTensor& alpha,
                                const OptTensor& beta, bool quantize) {
    c10::cuda::CUDAGuard guard(x.device());
    GM_CHECK(x.is_cuda() && x.is_contiguous(), "rmsnorm input must be contiguous");
    GM_CHECK(x.scalar_type() == torch::kFloat32 || x.scalar_type() == torch::kBFloat16, "rmsnorm input must be fp32 or bf16");
    const int d = x.size(-1);
    const int rows = x.numel() / d;
    GM_CHECK(norm_dim_supported(d), "rmsnorm width must be 128*{1,2,4,6,8,12,16}");
    Tensor y = gm::out_empty(x.sizes(), x.options().dtype(torch::kBFloat16));
    Tensor rstd = gm::out_empty({rows}, x.options().dtype(torch::kFloat32));
    Tensor x_new = x;
    if (branch.has_value()) {
        check_bf16(*branch, "branch");
        x_new = gm::out_empty_like(x);
    }
    QuantOut qo = alloc_quant(quantize, rows, d, x);
    launch_rmsnorm_fwd(x.data_ptr(), x.scalar_type() == torch::kFloat32, branch.has_value() ? branch->data_ptr() : nullptr,
                       fptr(alpha), fptr(beta), x_new.data_ptr(), fptr(w), y.data_ptr(), rstd.data_ptr<float>(), qo.qp, qo.sp, rows, d,
                       static_cast<float>(eps), stream());
    if (quantize) return {y, rstd, x_new, qo.q, qo.sf};
    return {y, rstd, x_new};
}

// Returns (dx, dw).  dx = norm backward (+ dres when given), same dtype as x.
std::vector<Tensor> rmsnorm_bwd(const Tensor& dy, const Tensor& x, const OptTensor& w, const Tensor& rstd, const OptTensor& dres) {
    c10::cuda::CUDAGuard guard(x.device());
    check_bf16(dy, "dy");
    const int d = x.size(-1);
    const int rows = x.numel() / d;
    Tensor dx = gm::out_empty_like(x);
    Tensor dw, partial;
    if (w.has_value()) {
        dw = gm::out_empty({d}, x.options().dtype(torch::kFloat32));
        partial = gm::out_empty({rmsnorm_bwd_blocks(rows), d}, x.options().dtype(torch::kFloat32));
    }
    GM_CHECK(launch_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), x.scalar_type() == torch::kFloat32, fptr(w), rstd.data_ptr<float>(),
                                dres.has_value() ? dres->data_ptr() : nullptr, dx.data_ptr(),
                                w.has_value() ? partial.data_ptr<float>() : nullptr, w.has_value() ? dw.data_ptr<float>() : nullptr, 0,
                                rows, d, stream()), "unsupported rmsnorm width");
    return {dx, dw};
}

// backward of x_new = x + beta*branch: returns (dbranch bf16, dbeta fp32[1])
std::vector<Tensor> residual_bwd(const Tensor& dxn, const Tensor& branch, const Tensor& beta) {
    c10::cuda::CUDAGuard guard(dxn.device());
    GM_CHECK(dxn.scalar_type() == torch::kFloat32 && dxn.is_contiguous() && dxn.numel() % 4 == 0, "dxn must be contiguous fp32");
    check_bf16(branch, "branch");
    GM_CHECK(beta.scalar_type() == torch::kFloat32 && beta.numel() == 1, "beta must be one fp32 value");
    Tensor dbranch = gm::out_empty_like(branch);
    Tensor partial = gm::out_empty({residual_bwd_blocks(dxn.numel())}, dxn.options());
    Tensor dbeta = gm::out_empty({1}, dxn.options());
    launch_residual_bwd(dxn.data_ptr<float>(), branch.data_ptr(), beta.data_ptr<float>(), dbranch.data_ptr(), partial.data_ptr<float>(),
                        dbeta.data_ptr<float>(), dxn.numel(), stream());
    return {dbranch, dbeta};
}

// qkv: [tokens, row_stride] bf16 holding q heads then k heads (then anything else) of width D each.
// forward writes rotated+normalised q,k into `out` (same layout; may alias a separate buffer)
// `copy_cols` trailing columns after the q and k heads (the value heads of a packed row) are copied from x to out as they are
void rope_qknorm_fwd(const Tensor& x, Tensor& out, const OptTensor& cos_t, const OptTensor& sin_t, const OptTensor& q_scale,
                     const OptTensor& k_scale, int64_t seq_len, int64_t q_heads, int64_t k_heads, int64_t head_dim, double eps,
                     bool rms, double smin, double smax, int64_t copy_cols) {
    c10::cuda::CUDAGuard guard(x.device());
    GM_CHECK(x.scalar_type() == torch::kBFloat16 && x.stride(-1) == 1 && out.stride(-1) == 1, "rope_qknorm needs bf16 rows");
    GM_CHECK(copy_cols % 8 == 0 && ((q_heads + k_heads) * head_dim) % 8 == 0 && x.stride(0) % 8 == 0 && out.stride(0) % 8 == 0 &&
             (q_heads + k_heads) * head_dim + copy_cols <= x.size(-1), "rope_qknorm: pass-through columns must be 16-byte aligned");
    const long long tokens = x.size(0);
    GM_CHECK(launch_rope_qknorm(false, head_dim, x.data_ptr(), nullptr, out.data_ptr(), fptr(cos_t), fptr(sin_t), fptr(q_scale),
                                fptr(k_scale), nullptr, tokens, seq_len, q_heads, k_heads, x.stride(0), out.stride(0),
                                static_cast<float>(eps), rms, static_cast<float>(smin), static_cast<float>(smax), copy_cols, nullptr, 0,
                                nullptr, nullptr, 0, stream()),
             "unsupported head size for rope_qknorm");
}

// backward: dx written into `dx` (layout of x) for the q and k heads; returns dscale [q_heads + k_heads] (fp32)
// `dq32` (optional, fp32 [tokens, q_heads * head_dim]): gradients of the query heads in full precision; when given, the query
// columns of `dy` are not read.
// `quantize`: also return the MXFP8 copy (payload, scale records) of the whole gradient row of width dx.size(1) — the rotated /
// normalised heads as written here plus the trailing columns of dy (value-head gradients) that pass through unchanged.
std::vector<Tensor> rope_qknorm_bwd(const Tensor& x, const Tensor& dy, Tensor& dx, const OptTensor& cos_t, const OptTensor& sin_t,
                                    const OptTensor& q_scale, const OptTensor& k_scale, int64_t seq_len, int64_t q_heads, int64_t k_heads,
                                    int64_t head_dim, double eps, bool rms, double smin, double smax, const OptTensor& dq32, bool quantize) {
    c10::cuda::CUDAGuard guard(x.device());
    const long long tokens = x.size(0);
    const int heads = q_heads + k_heads;
    const int blocks = rope_blocks(tokens, heads);
    Tensor partial = gm::out_empty({blocks, heads}, x.options().dtype(torch::kFloat32));
    GM_CHECK(x.stride(0) == dx.stride(0), "dx must share x's row stride");
    if (dq32.has_value())
        GM_CHECK(dq32->scalar_type() == torch::kFloat32 && dq32->is_contiguous() && dq32->numel() == tokens * q_heads * head_dim,
                 "dq32 must be a contiguous fp32 [tokens, q_heads * head_dim] tensor");
    const int width = dx.size(1);
    const int copy_cols = quantize ? width - heads * static_cast<int>(head_dim) : 0;
    if (quantize) GM_CHECK(dx.data_ptr() == dy.data_ptr() && width % 32 == 0 && copy_cols >= 0 && copy_cols % 32 == 0 && head_dim % 32 == 0,
                           "rope_qknorm_bwd with an MXFP8 copy runs in place on the full packed gradient rows");
    QuantOut qo = alloc_quant(quantize, tokens, width, x);
    GM_CHECK(launch_rope_qknorm(true, head_dim, x.data_ptr(), dy.data_ptr(), dx.data_ptr(), fptr(cos_t), fptr(sin_t), fptr(q_scale),
                                fptr(k_scale), partial.data_ptr<float>(), tokens, seq_len, q_heads, k_heads, x.stride(0),
                                dy.stride(0), static_cast<float>(eps), rms, static_cast<float>(smin), static_cast<float>(smax), copy_cols,
                                dq32.has_value() ? dq32->data_ptr<float>() : nullptr, dq32.has_value() ? q_heads * head_dim : 0,
                                qo.qp, qo.sp, width, stream()),
             "unsupported head size for rope_qknorm");
    Tensor dscale = gm::out_empty({heads}, partial.options());
    launch_column_sum(partial.data_ptr<float>(), dscale.data_ptr<float>(), blocks, heads, 0, stream());
    if (quantize) return {dscale, qo.q, qo.sf};
    return {dscale};
}

// Router after the logits GEMM: (top_idx int64 [T, k], gates fp32 [T, k]) and, with `want_balance`, (balance fp32 [1], counts fp32 [E]).
// renormalise: gates = softmax over the selected logits; otherwise the full-softmax probability of each selected expert.
std::vector<Tensor> router_fwd(const Tensor& logits, int64_t top_k, bool renormalise, bool want_balance) {
    c10::cuda::CUDAGuard guard(logits.device());
    GM_CHECK(logits.is_cuda() && logits.dim() == 2 && logits.is_contiguous() &&
             (logits.scalar_type() == torch::kBFloat16 || logits.scalar_type() == torch::kFloat32), "router logits: contiguous [tokens, experts] bf16 or fp32");
    const int tokens = logits.size(0), experts = logits.size(1);
    auto f32 = logits.options().dtype(torch::kFloat32);
    Tensor top_idx = gm::out_empty({tokens, top_k}, logits.options().dtype(torch::kInt64));
    Tensor gates = gm::out_empty({tokens, top_k}, f32);
    Tensor partial, sums, balance;
    if (want_balance) {
        partial = gm::out_empty({2, router_blocks(tokens), experts}, f32);
        sums = gm::out_empty({2, experts}, f32);
        balance = gm::out_empty({1}, f32);
    }
    GM_CHECK(launch_router_fwd(logits.data_ptr(), logits.scalar_type() == torch::kBFloat16, top_idx.data_ptr<int64_t>() ? reinterpret_cast<long long*>(top_idx.data_ptr<int64_t>()) : nullptr,
                               gates.data_ptr<float>(), want_balance ? partial[0].data_ptr<float>() : nullptr,
                               want_balance ? partial[1].data_ptr<float>() : nullptr, want_balance ? sums[0].data_ptr<float>() : nullptr,
                               want_balance ? sums[1].data_ptr<float>() : nullptr, want_balance ? balance.data_ptr<float>() : nullptr, tokens,
                               experts, top_k, renormalise, stream()),
             "router kernel: at most 128 experts, top-k at most 8");
    if (want_balance) return {top_idx, gates, balance, sums[1]};
    return {top_idx, gates};
}

// d logits from d gates (optional), d balance (optional, fp32 [1]) and the expert counts of the forward pass.
Tensor router_bwd(const Tensor& logits, const Tensor& top_idx, const OptTensor& dgates, const OptTensor& dbalance, const OptTensor& counts,
                  bool renormalise) {
    c10::cuda::CUDAGuard guard(logits.device());
    const int tokens = logits.size(0), experts = logits.size(1), top_k = top_idx.size(1);
    if (dgates.has_value()) GM_CHECK(dgates->scalar_type() == torch::kFloat32 && dgates->is_contiguous() && dgates->numel() == static_cast<int64_t>(tokens) * top_k, "dgates: contiguous fp32 [tokens, k]");
    if (dbalance.has_value()) GM_CHECK(dbalance->scalar_type() == torch::kFloat32 && dbalance->numel() == 1 && counts.has_value(), "dbalance: one fp32 value, with the forward's counts");
    Tensor dlogits = gm::out_empty_like(logits);
    GM_CHECK(launch_router_bwd(logits.data_ptr(), logits.scalar_type() == torch::kBFloat16, reinterpret_cast<const long long*>(top_idx.data_ptr<int64_t>()),
                               fptr(dgates), fptr(dbalance), fptr(counts), dlogits.data_ptr(), tokens, experts, top_k, renormalise, stream()),
             "router kernel: at most 128 experts, top-k at most 8");
    return dlogits;
}

// Absorbed-weight MLA decode over the latent cache (see attention/mla_decode.cu).  q_latent [B,T,H,r] fp32, q_rope [B,T,H,dr] fp32,
// latent [B,S,r] / rope [B,S,dr] / key_gain [B,S,Hkv] bf16 (views of a longer cache are fine: only the batch stride may differ from
// the packed one).  window < 0: none.  Returns the context in latent space [B,T,H,r] fp32.
Tensor mla_decode(const Tensor& q_latent, const Tensor& q_rope, const Tensor& latent, const Tensor& rope, const Tensor& key_gain,
                  int64_t start, double scale, double softcap, int64_t window) {
    c10::cuda::CUDAGuard guard(q_latent.device());
    GM_CHECK(q_latent.scalar_type() == torch::kFloat32 && q_rope.scalar_type() == torch::kFloat32 && q_latent.is_contiguous() && q_rope.is_contiguous() &&
             q_latent.dim() == 4 && q_rope.dim() == 4, "mla_decode: contiguous fp32 queries [B, T, H, r] and [B, T, H, dr]");
    const int B = q_latent.size(0), T = q_latent.size(1), H = q_latent.size(2), r = q_latent.size(3), dr = q_rope.size(3);
    const int S = latent.size(1), Hkv = key_gain.size(2);
    for (const Tensor* c : {&latent, &rope, &key_gain})
        GM_CHECK(c->is_cuda() && c->scalar_type() == torch::kBFloat16 && c->dim() == 3 && c->size(0) == B && c->size(1) == S && c->stride(2) == 1 &&
                 c->stride(1) == c->size(2), "mla_decode: bf16 cache tensors [B, S, width] with packed rows");
    GM_CHECK(latent.size(2) == r && rope.size(2) == dr && mla_decode_supported(H, Hkv, r, dr),
             "mla_decode: latent rank 256/512/768/1024, 8/16/32 heads (rank/32 * heads/8 <= 64), rope width even and <= 64");
    const int splits = mla_decode_splits(B, T, S);
    Tensor part_ctx = gm::out_empty({B, T, H, splits, r}, q_latent.options());
    Tensor part_ml = gm::out_empty({B, T, H, splits, 2}, q_latent.options());
    Tensor context = gm::out_empty({B, T, H, r}, q_latent.options());
    GM_CHECK(launch_mla_decode(q_latent.data_ptr<float>(), q_rope.data_ptr<float>(), latent.data_ptr(), rope.data_ptr(), key_gain.data_ptr(),
                               latent.stride(0), rope.stride(0), key_gain.stride(0), part_ctx.data_ptr<float>(), part_ml.data_ptr<float>(),
                               context.data_ptr<float>(), B, T, H, Hkv, r, dr, S, splits, start, window, static_cast<float>(scale),
                               static_cast<float>(softcap), stream()), "mla_decode: unsupported shape");
    return context;
}

// (issue clocks, completion clocks) of `count` chained tcgen05.mma instructions of shape code `shape` (csrc/bench/mma_issue.cu)
std::vector<int64_t> mma_issue_bench(int64_t shape, int64_t count) {
    GM_CHECK(count > 0 && count % 4 == 0 && count <= 4096, "mma_issue_bench: count must be a multiple of 4, at most 4096");
    auto out = gm::out_zeros({2}, torch::TensorOptions().dtype(torch::kInt64).device(torch::kCUDA));
    cudaError_t e = launch_mma_issue(static_cast<int>(shape), reinterpret_cast<long long*>(out.data_ptr<int64_t>()), static_cast<int>(count),
                                     status_word(out.device().index()), stream());
    GM_CHECK(e == cudaSuccess, cudaGetErrorString(e));
    auto host = out.cpu();
    return {host[0].item<int64_t>(), host[1].item<int64_t>()};
}

bool mla_decode_ok(int64_t H, int64_t Hkv, int64_t r, int64_t dr) { return mla_decode_supported(H, Hkv, r, dr); }

// Counted routing.  Returns (dest[S], src_of_row[cap], seg_ends[E], counts[E], tile_expert[cap/128], meta[2]).
std::vector<Tensor> route(const Tensor& top_idx, int64_t experts) {
    c10::cuda::CUDAGuard guard(top_idx.device());
    GM_CHECK(top_idx.is_cuda() && top_idx.scalar_type() == torch::kInt64 && top_idx.is_contiguous(), "top_idx must be contiguous int64");
    const int slots = top_idx.numel();
    const int cap = (slots + 255) / 256 * 256 + experts * 256;      // every expert segment is padded to 256 rows
    const int chunks = (slots + 1023) / 1024;
    auto opt = top_idx.options().dtype(torch::kInt32);
    Tensor hist = gm::out_empty({2, chunks > 0 ? chunks : 1, experts}, opt);
    Tensor dest = gm::out_empty({slots}, opt), src = gm::out_empty({cap}, opt);
    Tensor seg = gm::out_empty({experts}, opt), counts = gm::out_empty({experts}, opt);
    Tensor tiles = gm::out_empty({cap / 128}, opt), meta = gm::out_empty({2}, opt);      // entries beyond meta[0] are never read
    GM_CHECK(launch_route(top_idx.data_ptr<int64_t>() ? reinterpret_cast<const long long*>(top_idx.data_ptr<int64_t>()) : nullptr, slots,
                          experts, hist[0].data_ptr<int>(), hist[1].data_ptr<int>(), counts.data_ptr<int>(), seg.data_ptr<int>(),
                          tiles.data_ptr<int>(), meta.data_ptr<int>(), dest.data_ptr<int>(), src.data_ptr<int>(), stream()),
             "routing supports at most 128 experts");      // zero slots are fine: every segment is then empty
    return {dest, src, seg, counts, tiles, meta};
}

std::vector<Tensor> gather_rows(const Tensor& hidden, const Tensor& src_of_row, const Tensor& meta, int64_t top_k, bool quantize) {
    c10::cuda::CUDAGuard guard(hidden.device());
    check_bf16(hidden, "hidden");
    const int d = hidden.size(-1);
    GM_CHECK(d % 8 == 0, "row width must be a multiple of 8");
    const int cap = src_of_row.numel();
    Tensor packed = gm::out_empty({cap, d}, hidden.options());
    QuantOut qo = alloc_quant(quantize, cap, d, hidden);
    launch_gather_rows(hidden.data_ptr(), src_of_row.data_ptr<int>(), meta.data_ptr<int>(), packed.data_ptr(), qo.qp, qo.sp, d, top_k, cap,
                       hidden.numel() / d, stream());
    if (quantize) return {packed, qo.q, qo.sf};
    return {packed};
}

// gates: fp32 [tokens, k], or none for unit gates (then `top_k` says how many rows each token sums)
Tensor combine_fwd(const Tensor& y, const Tensor& dest, const OptTensor& gates, int64_t top_k_if_no_gates) {
    c10::cuda::CUDAGuard guard(y.device());
    check_bf16(y, "y");
    if (gates.has_value()) GM_CHECK(gates->scalar_type() == torch::kFloat32 && gates->is_contiguous(), "gates must be contiguous fp32");
    const int top_k = gates.has_value() ? gates->size(1) : static_cast<int>(top_k_if_no_gates);
    GM_CHECK(top_k >= 1 && dest.numel() % top_k == 0, "combine_fwd: slots must be a multiple of top_k");
    const int tokens = dest.numel() / top_k, d = y.size(-1);
    Tensor out = gm::out_empty({tokens, d}, y.options());
    launch_combine_fwd(y.data_ptr(), dest.data_ptr<int>(), fptr(gates), out.data_ptr(), tokens, d, top_k, y.numel() / d, stream());
    return out;
}

std::vector<Tensor> combine_bwd(const Tensor& dout, const Tensor& y, const Tensor& src_of_row, const Tensor& gates, const Tensor& meta, bool quantize) {
    c10::cuda::CUDAGuard guard(y.device());
    check_bf16(dout, "dout");
    check_bf16(y, "y");
    const int top_k = gates.size(1), d = y.size(-1), cap = src_of_row.numel();
    Tensor dy = gm::out_empty_like(y);
    Tensor dgates = gm::out_empty_like(gates);                     // every (token, slot) has exactly one live row that writes it
    QuantOut qo = alloc_quant(quantize, cap, d, y);
    launch_combine_bwd(dout.data_ptr(), y.data_ptr(), src_of_row.data_ptr<int>(), gates.data_ptr<float>(), meta.data_ptr<int>(),
                       dy.data_ptr(), dgates.data_ptr<float>(), qo.qp, qo.sp, d, top_k, cap, dout.numel() / d, stream());
    if (quantize) return {dy, dgates, qo.q, qo.sf};
    return {dy, dgates};
}

int act_kind(const std::string& name) {
    if (name == "gelu") return 0;
    if (name == "relu") return 1;
    if (name == "relu2") return 2;
    if (name == "silu") return 3;
    if (name == "swiglu") return 4;
    GM_CHECK(false, "unsupported activation function: " + name);
    return -1;
}

std::vector<Tensor> activation_fwd(const Tensor& pre, const std::string& name, const OptTensor& meta, bool quantize) {
    c10::cuda::CUDAGuard guard(pre.device());
    check_bf16(pre, "pre");
    const int kind = act_kind(name);
    const int in_w = pre.size(-1), h = kind == 4 ? in_w / 2 : in_w;
    const int rows = pre.numel() / in_w;
    GM_CHECK(h % 8 == 0 && pre.is_contiguous(), "activation width must be a multiple of 8 (16-byte vectors) and rows contiguous");
    auto sizes = pre.sizes().vec();
    sizes.back() = h;
    Tensor act = gm::out_empty(sizes, pre.options());
    GM_CHECK(!quantize || h % 32 == 0, "activation with an MXFP8 copy: width must be a multiple of 32");
    QuantOut qo = alloc_quant(quantize, rows, h, pre);
    launch_activation_fwd(pre.data_ptr(), act.data_ptr(), meta.has_value() ? meta->data_ptr<int>() : nullptr, qo.qp, qo.sp, rows, h, kind, stream());
    if (quantize) return {act, qo.q, qo.sf};
    return {act};
}

std::vector<Tensor> activation_bwd(const Tensor& dact, const Tensor& pre, const std::string& name, const OptTensor& meta, bool quantize) {
    c10::cuda::CUDAGuard guard(pre.device());
    check_bf16(dact, "dact");
    const int kind = act_kind(name);
    const int in_w = pre.size(-1), h = kind == 4 ? in_w / 2 : in_w;
    const int rows = pre.numel() / in_w;
    GM_CHECK(h % 8 == 0 && pre.is_contiguous() && dact.is_contiguous(), "activation width must be a multiple of 8 (16-byte vectors) and rows contiguous");
    Tensor dpre = gm::out_empty_like(pre);
    GM_CHECK(!quantize || h % 32 == 0, "activation with an MXFP8 copy: width must be a multiple of 32");
    QuantOut qo = alloc_quant(quantize, rows, in_w, pre);
    launch_activation_bwd(dact.data_ptr(), pre.data_ptr(), dpre.data_ptr(), meta.has_value() ? meta->data_ptr<int>() : nullptr, qo.qp, qo.sp, rows, h, kind, stream());
    if (quantize) return {dpre, qo.q, qo.sf};
    return {dpre};
}

// loss per row; logits overwritten with (softmax - onehot) * grad_scale when write_grad
Tensor ce_fwd_bwd(Tensor& logits, const Tensor& targets, const Tensor& grad_scale, int64_t ignore_index, bool write_grad) {
    c10::cuda::CUDAGuard guard(logits.device());
    GM_CHECK(logits.scalar_type() == torch::kBFloat16 && logits.dim() == 2 && logits.stride(1) == 1 && logits.stride(0) % 8 == 0,
             "logits must be [rows, vocab] bf16 with a row pitch that is a multiple of 8");
    GM_CHECK(targets.scalar_type() == torch::kInt64 && targets.is_contiguous(), "targets must be contiguous int64");
    const int rows = logits.size(0);
    Tensor loss = gm::out_empty({rows}, logits.options().dtype(torch::kFloat32));
    launch_ce_fwd_bwd(logits.data_ptr(), reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()), loss.data_ptr<float>(),
                      grad_scale.data_ptr<float>(), rows, logits.size(1), logits.stride(0), ignore_index, write_grad, stream());
    return loss;
}

void adamw(Tensor& p, const Tensor& g, Tensor& m, Tensor& v, const OptTensor& p_bf16, double lr, double beta1, double beta2,
           double eps, double wd, int64_t step, double grad_scale) {
    c10::cuda::CUDAGuard guard(p.device());
    GM_CHECK(p.scalar_type() == torch::kFloat32 && g.scalar_type() == torch::kFloat32 && p.is_contiguous() && g.is_contiguous(),
             "AdamW expects contiguous fp32 parameters and gradients");
    GM_CHECK(m.scalar_type() == v.scalar_type() && m.is_contiguous() && v.is_contiguous(), "AdamW moments must share a dtype");
    const double bc1 = 1.0 - std::pow(beta1, static_cast<double>(step));
    const double bc2 = std::sqrt(1.0 - std::pow(beta2, static_cast<double>(step)));
    launch_adamw(p.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr(), v.data_ptr(), m.scalar_type() == torch::kBFloat16,
                 p_bf16.has_value() ? p_bf16->data_ptr() : nullptr, p.numel(), lr, beta1, beta2, eps, wd, bc1, bc2, grad_scale, stream());
}

// pointer tables are int64 CUDA tensors holding device addresses (built once per bucket by the caller)
void muon_prepare(const Tensor& grad_ptrs, const Tensor& buf_ptrs, Tensor& packed, Tensor& sumsq, int64_t rows, int64_t cols,
                  int64_t g_stride, int64_t b_stride, double momentum, bool nesterov, bool transpose, double grad_scale) {
    c10::cuda::CUDAGuard guard(packed.device());
    check_bf16(packed, "packed");
    const int n = grad_ptrs.numel();
    GM_CHECK(packed.numel() == n * rows * cols && (rows * cols) % 8 == 0, "packed buffer shape");
    launch_muon_prepare(reinterpret_cast<const float* const*>(grad_ptrs.data_ptr<int64_t>()),
                        reinterpret_cast<float* const*>(buf_ptrs.data_ptr<int64_t>()), packed.data_ptr(), sumsq.data_ptr<float>(), n,
                        rows, cols, g_stride, b_stride, momentum, nesterov, transpose, grad_scale, stream());
}

void muon_apply(const Tensor& weight_ptrs, const OptTensor& bf16_ptrs, const Tensor& update, int64_t rows, int64_t cols,
                int64_t w_stride, double alpha, bool transpose) {
    c10::cuda::CUDAGuard guard(update.device());
    check_bf16(update, "update");
    launch_muon_apply(reinterpret_cast<float* const*>(weight_ptrs.data_ptr<int64_t>()),
                      bf16_ptrs.has_value() ? reinterpret_cast<void* const*>(bf16_ptrs->data_ptr<int64_t>()) : nullptr,
                      update.data_ptr(), weight_ptrs.numel(), rows, cols, w_stride, alpha, transpose, stream());
}

std::vector<long long> to_deltas(const std::vector<int64_t>& deltas) { return std::vector<long long>(deltas.begin(), deltas.end()); }

// Owner-side gradient reduction over peer memory fused with Muon's momentum / Nesterov / bf16 pack / Frobenius normalisation.
// grad_ptrs point into THIS rank's symmetric gradient buffer; peer_deltas[r] = (rank r's buffer base) - (this rank's base).
// bf16 wire: `grad_base` is this rank's flat fp32 gradient buffer and `shadow` its bf16 shadow (same element offsets);
// peer_deltas are then the deltas of the SHADOW buffers and peers' contributions are read from their shadows.
void rs_muon_prepare(const Tensor& grad_ptrs, const Tensor& buf_ptrs, Tensor& packed, Tensor& sumsq, int64_t rows, int64_t cols,
                     int64_t g_stride, int64_t b_stride, double momentum, bool nesterov, bool transpose,
                     const std::vector<int64_t>& peer_deltas, bool normalize, const OptTensor& grad_base, const OptTensor& shadow) {
    c10::cuda::CUDAGuard guard(packed.device());
    check_bf16(packed, "packed");
    const int n = grad_ptrs.numel();
    GM_CHECK(packed.numel() == n * rows * cols && (rows * cols) % 8 == 0, "packed buffer shape");
    auto d = to_deltas(peer_deltas);
    GM_CHECK(grad_base.has_value() == shadow.has_value(), "rs_muon_prepare: grad_base and shadow come together");
    if (shadow.has_value())
        GM_CHECK(grad_base->scalar_type() == torch::kFloat32 && shadow->scalar_type() == torch::kBFloat16 && shadow->numel() >= grad_base->numel(),
                 "rs_muon_prepare: fp32 gradient buffer and a bf16 shadow at least as long");
    GM_CHECK(sumsq.numel() >= n, "rs_muon_prepare: one sum of squares per matrix");
    GM_CHECK(launch_rs_muon_prepare(reinterpret_cast<const float* const*>(grad_ptrs.data_ptr<int64_t>()),
                                    reinterpret_cast<float* const*>(buf_ptrs.data_ptr<int64_t>()), packed.data_ptr(), sumsq.data_ptr<float>(), n,
                                    rows, cols, g_stride, b_stride, momentum, nesterov, transpose, d.data(), d.size(),
                                    grad_base.has_value() ? grad_base->data_ptr<float>() : nullptr,
                                    shadow.has_value() ? shadow->data_ptr() : nullptr, stream()),
             "rs_muon_prepare: at most 16 ranks, column count a multiple of 4");
    // normalize = false leaves `packed` as it is: the caller hands `sumsq` to the first GEMMs of the orthogonalisation instead
    if (normalize) launch_muon_normalize(packed.data_ptr(), sumsq.data_ptr<float>(), n, rows * cols, stream());
}

// W_master += alpha * O on the owner; the refreshed bf16 copy is stored into every rank's weight buffer.
void muon_apply_push(const Tensor& weight_ptrs, const Tensor& bf16_ptrs, const Tensor& update, int64_t rows, int64_t cols,
                     int64_t w_stride, int64_t wb_stride, double alpha, bool transpose, const std::vector<int64_t>& peer_deltas) {
    c10::cuda::CUDAGuard guard(update.device());
    check_bf16(update, "update");
    auto d = to_deltas(peer_deltas);
    GM_CHECK(launch_muon_apply_push(reinterpret_cast<float* const*>(weight_ptrs.data_ptr<int64_t>()),
                                    reinterpret_cast<void* const*>(bf16_ptrs.data_ptr<int64_t>()), update.data_ptr(), weight_ptrs.numel(),
                                    rows, cols, w_stride, wb_stride, alpha, transpose, d.data(), d.size(), stream()),
             "muon_apply_push: at most 16 ranks, column count a multiple of 4");
}

// AdamW on this rank's slice [lo, lo+n) of the flat parameter buffer: gradient summed from all ranks, result stored to all ranks.
void adamw_sharded(Tensor& params, const Tensor& grads, Tensor& m, Tensor& v, const Tensor& decay, int64_t lo, int64_t n, double lr,
                   double beta1, double beta2, double eps, int64_t step, const std::vector<int64_t>& grad_deltas,
                   const std::vector<int64_t>& param_deltas) {
    c10::cuda::CUDAGuard guard(params.device());
    GM_CHECK(params.scalar_type() == torch::kFloat32 && grads.scalar_type() == torch::kFloat32 && decay.scalar_type() == torch::kFloat32,
             "adamw_sharded expects fp32 flat buffers");
    GM_CHECK(m.numel() >= n && v.numel() >= n && m.scalar_type() == v.scalar_type(), "moment buffers must cover the slice");
    const double bc1 = 1.0 - std::pow(beta1, static_cast<double>(step));
    const double bc2 = std::sqrt(1.0 - std::pow(beta2, static_cast<double>(step)));
    auto gd = to_deltas(grad_deltas), pd = to_deltas(param_deltas);
    GM_CHECK(launch_adamw_sharded(params.data_ptr<float>(), grads.data_ptr<float>(), m.data_ptr(), v.data_ptr(),
                                  m.scalar_type() == torch::kBFloat16, decay.data_ptr<float>(), lo, n, lr, beta1, beta2, eps, bc1, bc2,
                                  gd.data(), pd.data(), gd.size(), stream()),
             "adamw_sharded: at most 16 ranks, slice bounds multiples of 4");
}

void cast_bf16(const Tensor& src, Tensor& dst) {
    c10::cuda::CUDAGuard guard(src.device());
    GM_CHECK(src.scalar_type() == torch::kFloat32 && dst.scalar_type() == torch::kBFloat16 && src.is_contiguous() && dst.is_contiguous() &&
             src.numel() == dst.numel(), "cast_bf16 expects contiguous fp32 -> bf16 of equal size");
    launch_cast_bf16(src.data_ptr<float>(), dst.data_ptr(), src.numel(), stream());
}

}  // namespace

// Publish a value into flags[index] of every rank / wait until flags[first .. first + world) of this rank have all reached it.
// The value is `value`, or the content of the int32 device word `value_word` when given (no host state in the launch).
void flag_signal(Tensor& flags, const std::vector<int64_t>& deltas, int64_t index, int64_t value, const OptTensor& value_word) {
    c10::cuda::CUDAGuard guard(flags.device());
    GM_CHECK(flags.scalar_type() == torch::kInt32 && index >= 0 && index < flags.numel(), "flag_signal: int32 flag table, index in range");
    if (value_word.has_value()) GM_CHECK(value_word->is_cuda() && value_word->scalar_type() == torch::kInt32 && value_word->numel() >= 1, "value_word: int32 CUDA tensor");
    auto d = to_deltas(deltas);
    GM_CHECK(launch_flag_signal(flags.data_ptr<int>(), d.data(), d.size(), index, value, value_word.has_value() ? value_word->data_ptr<int>() : nullptr, stream()),
             "flag_signal: at most 16 ranks");
}

void flag_wait(const Tensor& flags, int64_t first, int64_t world, int64_t value, const OptTensor& value_word) {
    c10::cuda::CUDAGuard guard(flags.device());
    GM_CHECK(flags.scalar_type() == torch::kInt32 && first >= 0 && first + world <= flags.numel(), "flag_wait: int32 flag table, range inside it");
    if (value_word.has_value()) GM_CHECK(value_word->is_cuda() && value_word->scalar_type() == torch::kInt32 && value_word->numel() >= 1, "value_word: int32 CUDA tensor");
    GM_CHECK(launch_flag_wait(flags.data_ptr<int>(), first, world, value, value_word.has_value() ? value_word->data_ptr<int>() : nullptr,
                              status_word(flags.device().index()), stream()), "flag_wait: at most 16 ranks");
}

void bump_word(Tensor& word) {
    c10::cuda::CUDAGuard guard(word.device());
    GM_CHECK(word.is_cuda() && word.scalar_type() == torch::kInt32 && word.numel() >= 1, "bump_word: int32 CUDA tensor");
    launch_bump_word(word.data_ptr<int>(), stream());
}

// One-launch barrier over a symmetric int32 flag table of `world` entries per rank (see peer_barrier_kernel).  `budget_cycles`
// = 0 selects the common wait budget; a wait that runs out sets status 601 and returns.
void peer_barrier(Tensor& flags, const std::vector<int64_t>& deltas, int64_t me, Tensor& epoch_word, int64_t budget_cycles) {
    c10::cuda::CUDAGuard guard(flags.device());
    GM_CHECK(flags.is_cuda() && flags.scalar_type() == torch::kInt32 && flags.numel() >= static_cast<int64_t>(deltas.size()),
             "peer_barrier: int32 flag table with one entry per rank");
    GM_CHECK(epoch_word.is_cuda() && epoch_word.scalar_type() == torch::kInt32 && epoch_word.numel() >= 1, "peer_barrier: int32 epoch word");
    auto d = to_deltas(deltas);
    GM_CHECK(launch_peer_barrier(flags.data_ptr<int>(), d.data(), d.size(), me, epoch_word.data_ptr<int>(), status_word(flags.device().index()),
                                 budget_cycles, stream()), "peer_barrier: at most 16 ranks, rank inside the group");
}

// ---- expert-parallel dispatch / combine over peer memory ---------------------------------------------------------------
// `table` is this rank's [world, experts] int32 count table inside a symmetric buffer; deltas[r] = rank r's base - this rank's base.
void ep_push_counts(const Tensor& counts, Tensor& table, const std::vector<int64_t>& deltas, int64_t me) {
    c10::cuda::CUDAGuard guard(counts.device());
    GM_CHECK(counts.scalar_type() == torch::kInt32 && table.scalar_type() == torch::kInt32 && table.is_contiguous(), "ep_push_counts: int32 tensors");
    auto d = to_deltas(deltas);
    GM_CHECK(table.numel() >= static_cast<int64_t>(d.size()) * counts.numel(), "ep_push_counts: count table too small");
    GM_CHECK(launch_ep_push_counts(counts.data_ptr<int>(), table.data_ptr<int>(), d.data(), d.size(), me, counts.numel(), stream()),
             "ep_push_counts: at most 16 ranks and 128 experts");
}

// -> my_base [E], seg_ends [E_local], valid_ends [E_local], tile_expert [cap / 128], meta {tiles, padded rows}
std::vector<Tensor> ep_plan(const Tensor& table, int64_t world, int64_t me, int64_t experts, int64_t cap_rows) {
    c10::cuda::CUDAGuard guard(table.device());
    GM_CHECK(experts % world == 0 && cap_rows % 256 == 0, "ep_plan: experts divisible by the group size, capacity a multiple of 256");
    const int per_rank = experts / world;
    auto opt = table.options().dtype(torch::kInt32);
    Tensor my_base = gm::out_empty({experts}, opt), seg = gm::out_empty({per_rank}, opt), valid = gm::out_empty({per_rank}, opt);
    Tensor tiles = gm::out_zeros({cap_rows / 128}, opt), meta = gm::out_empty({2}, opt);
    GM_CHECK(launch_ep_plan(table.data_ptr<int>(), my_base.data_ptr<int>(), seg.data_ptr<int>(), valid.data_ptr<int>(), tiles.data_ptr<int>(),
                            meta.data_ptr<int>(), world, me, experts, per_rank, cap_rows, status_word(table.device().index()), stream()),
             "ep_plan: at most 16 ranks and 128 experts");
    return {my_base, seg, valid, tiles, meta};
}

void ep_zero_pads(Tensor& buf, const Tensor& seg_ends, const Tensor& valid_ends) {
    c10::cuda::CUDAGuard guard(buf.device());
    check_bf16(buf, "buf");
    GM_CHECK(buf.size(-1) % 8 == 0, "row width must be a multiple of 8");
    launch_ep_zero_pads(buf.data_ptr(), seg_ends.data_ptr<int>(), valid_ends.data_ptr<int>(), seg_ends.numel(), buf.size(-1), stream());
}

// Store row (token of slot i) of `src` into the owner's `recv` buffer; returns (route_row [slots], dgates or empty).
// gates given: rows are scaled by the slot's gate; saved_rows given as well: dgates[i] = <src row, saved_rows[i]>.
std::vector<Tensor> ep_dispatch(const Tensor& src, const Tensor& top_idx, const Tensor& dest, const Tensor& local_seg_ends, const Tensor& my_base,
                                const c10::optional<Tensor>& gates, const c10::optional<Tensor>& saved_rows, Tensor& recv,
                                const std::vector<int64_t>& deltas, int64_t per_rank) {
    c10::cuda::CUDAGuard guard(src.device());
    check_bf16(src, "src");
    check_bf16(recv, "recv");
    GM_CHECK(top_idx.scalar_type() == torch::kInt64 && top_idx.is_contiguous() && top_idx.dim() == 2, "top_idx must be contiguous int64 [tokens, k]");
    const int slots = top_idx.numel(), top_k = top_idx.size(1), d = src.size(-1);
    GM_CHECK(src.size(0) * top_k == slots && recv.size(-1) == d, "ep_dispatch: shapes");
    if (gates.has_value()) GM_CHECK(gates->scalar_type() == torch::kFloat32 && gates->is_contiguous() && gates->numel() == slots, "gates must be contiguous fp32");
    if (saved_rows.has_value()) { check_bf16(*saved_rows, "saved_rows"); GM_CHECK(saved_rows->numel() == static_cast<int64_t>(slots) * d, "saved rows shape"); }
    Tensor route_row = gm::out_empty({slots}, dest.options());
    Tensor dgates = saved_rows.has_value() ? gm::out_empty({slots / top_k, top_k}, src.options().dtype(torch::kFloat32)) : Tensor();
    auto dl = to_deltas(deltas);
    GM_CHECK(launch_ep_dispatch(src.data_ptr(), reinterpret_cast<const long long*>(top_idx.data_ptr<int64_t>()), dest.data_ptr<int>(),
                                local_seg_ends.data_ptr<int>(), my_base.data_ptr<int>(), gates.has_value() ? gates->data_ptr<float>() : nullptr,
                                saved_rows.has_value() ? saved_rows->data_ptr() : nullptr, saved_rows.has_value() ? dgates.data_ptr<float>() : nullptr,
                                recv.data_ptr(), route_row.data_ptr<int>(), dl.data(), dl.size(), slots, d, top_k, per_rank, recv.size(0),
                                status_word(src.device().index()), stream()),
             "ep_dispatch: at most 16 ranks, row width a multiple of 8");
    if (saved_rows.has_value()) return {route_row, dgates};
    return {route_row};
}

// out[t] = sum_k gates[t, k] * (row route_row[t, k] of the owner's `ret` buffer); keep = true also returns the loaded rows [slots, d].
std::vector<Tensor> ep_combine(const Tensor& ret, const Tensor& top_idx, const Tensor& route_row, const c10::optional<Tensor>& gates, bool keep,
                               const std::vector<int64_t>& deltas, int64_t per_rank) {
    c10::cuda::CUDAGuard guard(ret.device());
    check_bf16(ret, "ret");
    const int tokens = top_idx.size(0), top_k = top_idx.size(1), d = ret.size(-1);
    if (gates.has_value()) GM_CHECK(gates->scalar_type() == torch::kFloat32 && gates->is_contiguous(), "gates must be contiguous fp32");
    Tensor out = gm::out_empty({tokens, d}, ret.options());
    Tensor rows = keep ? gm::out_empty({tokens * top_k, d}, ret.options()) : Tensor();
    auto dl = to_deltas(deltas);
    GM_CHECK(launch_ep_combine(ret.data_ptr(), reinterpret_cast<const long long*>(top_idx.data_ptr<int64_t>()), route_row.data_ptr<int>(),
                               gates.has_value() ? gates->data_ptr<float>() : nullptr, out.data_ptr(), keep ? rows.data_ptr() : nullptr, dl.data(),
                               dl.size(), tokens, d, top_k, per_rank, ret.size(0), stream()),
             "ep_combine: at most 16 ranks, row width a multiple of 8");
    if (keep) return {out, rows};
    return {out};
}

// bounds-checked build: the first out-of-range index any kernel met since the last call (0 = none); always 0 in the normal build
int64_t read_bounds_status() {
    for (int v : {read_bounds_moe(), read_bounds_loss(), read_bounds_router()})
        if (v != 0) return v;
    return 0;
}
// bounds-checked build with GM_CANARIES=1: guard bytes around the bindings' allocations that were overwritten since the last call
int64_t verify_guards() { return verify_output_guards(); }
bool guards_enabled() { return output_guards_enabled(); }
bool bounds_checked() {
#ifdef GM_CHECK_BOUNDS
    return true;
#else
    return false;
#endif
}

void register_kernels(pybind11::module_& m) {
    namespace py = pybind11;
    m.def("rmsnorm_fwd", &rmsnorm_fwd, py::arg("x"), py::arg("w"), py::arg("eps"), py::arg("branch") = py::none(),
          py::arg("alpha") = py::none(), py::arg("beta") = py::none(), py::arg("quantize") = false);
    m.def("rmsnorm_bwd", &rmsnorm_bwd, py::arg("dy"), py::arg("x"), py::arg("w"), py::arg("rstd"), py::arg("dres") = py::none());
    m.def("residual_bwd", &residual_bwd);
    m.def("rope_qknorm_fwd", &rope_qknorm_fwd, py::arg("x"), py::arg("out"), py::arg("cos"), py::arg("sin"), py::arg("q_scale"), py::arg("k_scale"),
          py::arg("seq_len"), py::arg("q_heads"), py::arg("k_heads"), py::arg("head_dim"), py::arg("eps"), py::arg("rms"), py::arg("smin"),
          py::arg("smax"), py::arg("copy_cols") = 0);
    m.def("rope_qknorm_bwd", &rope_qknorm_bwd, py::arg("x"), py::arg("dy"), py::arg("dx"), py::arg("cos"), py::arg("sin"), py::arg("q_scale"),
          py::arg("k_scale"), py::arg("seq_len"), py::arg("q_heads"), py::arg("k_heads"), py::arg("head_dim"), py::arg("eps"), py::arg("rms"),
          py::arg("smin"), py::arg("smax"), py::arg("dq32") = py::none(), py::arg("quantize") = false);
    m.def("mla_decode", &mla_decode);
    m.def("mla_decode_ok", &mla_decode_ok);
    m.def("mma_issue_bench", &mma_issue_bench, py::arg("shape"), py::arg("count") = 64);
    m.def("router_fwd", &router_fwd);
    m.def("router_bwd", &router_bwd);
    m.def("route", &route);
    m.def("gather_rows", &gather_rows, py::arg("hidden"), py::arg("src_of_row"), py::arg("meta"), py::arg("top_k"), py::arg("quantize") = false);
    m.def("combine_fwd", &combine_fwd, py::arg("y"), py::arg("dest"), py::arg("gates"), py::arg("top_k_if_no_gates") = 1);
    m.def("read_bounds_status", &read_bounds_status);
    m.def("bounds_checked", &bounds_checked);
    m.def("verify_output_guards", &verify_guards);
    m.def("output_guards_enabled", &guards_enabled);
    m.def("combine_bwd", &combine_bwd, py::arg("dout"), py::arg("y"), py::arg("src_of_row"), py::arg("gates"), py::arg("meta"), py::arg("quantize") = false);
    m.def("activation_fwd", &activation_fwd, py::arg("pre"), py::arg("name"), py::arg("meta") = py::none(), py::arg("quantize") = false);
    m.def("activation_bwd", &activation_bwd, py::arg("dact"), py::arg("pre"), py::arg("name"), py::arg("meta") = py::none(), py::arg("quantize") = false);
    m.def("ce_fwd_bwd", &ce_fwd_bwd);
    m.def("adamw", &adamw);
    m.def("muon_prepare", &muon_prepare);
    m.def("muon_apply", &muon_apply);
    m.def("cast_bf16", &cast_bf16);
    m.def("rs_muon_prepare", &rs_muon_prepare, py::arg("grad_ptrs"), py::arg("buf_ptrs"), py::arg("packed"), py::arg("sumsq"), py::arg("rows"),
          py::arg("cols"), py::arg("g_stride"), py::arg("b_stride"), py::arg("momentum"), py::arg("nesterov"), py::arg("transpose"),
          py::arg("peer_deltas"), py::arg("normalize") = true, py::arg("grad_base") = py::none(), py::arg("shadow") = py::none());
    m.def("muon_apply_push", &muon_apply_push);
    m.def("adamw_sharded", &adamw_sharded);
    m.def("flag_signal", &flag_signal, py::arg("flags"), py::arg("deltas"), py::arg("index"), py::arg("value"), py::arg("value_word") = py::none());
    m.def("flag_wait", &flag_wait, py::arg("flags"), py::arg("first"), py::arg("world"), py::arg("value"), py::arg("value_word") = py::none());
    m.def("bump_word", &bump_word);
    m.def("peer_barrier", &peer_barrier, py::arg("flags"), py::arg("deltas"), py::arg("me"), py::arg("epoch_word"), py::arg("budget_cycles") = 0);
    m.def("ep_push_counts", &ep_push_counts);
    m.def("ep_plan", &ep_plan);
    m.def("ep_zero_pads", &ep_zero_pads);
    m.def("ep_dispatch", &ep_dispatch);
    m.def("ep_combine", &ep_combine);
}

}  // namespace gm

// Python bindings (pybind11 through torch's extension headers).  Kernels live in .cu files that do not
// include torch headers; this file converts tensors to raw pointers, builds TMA descriptors and launches.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <cstring>
#include <list>
#include <unordered_map>

#include "guarded_alloc.h"
#include "gemm/gemm.h"
#include "attention/attn.h"
#include "kernels.h"

namespace {

#define GM_CHECK(cond, msg) TORCH_CHECK(cond, "gpt_moe_b200: ", msg)

cudaStream_t current_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int sm_count() {
    static int sms = 0;
    if (sms == 0) sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    return sms;
}

// One status word per device: kernels write a non-zero code when a bounded wait gives up.
torch::Tensor& status_tensor(int device) {
    static std::unordered_map<int, torch::Tensor> words;
    auto it = words.find(device);
    if (it == words.end()) {
        it = words.emplace(device, torch::zeros({1}, torch::dtype(torch::kInt32).device(torch::kCUDA, device))).first;
    }
    return it->second;
}

int64_t read_status() {
    int device = at::cuda::current_device();
    return status_tensor(device).item<int32_t>();
}
void reset_status() { status_tensor(at::cuda::current_device()).zero_(); }
// the device word itself, for an asynchronous copy to pinned host memory
torch::Tensor status_word_tensor() { return status_tensor(at::cuda::current_device()); }

// ---- tensor map cache -----------------------------------------------------------------------------
struct MapKey {
    const void* ptr; uint64_t cols, rows, batch, rs, bs; uint32_t bc, br; int eb, sw;
    bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        const uint64_t* w = reinterpret_cast<const uint64_t*>(&k);
        size_t h = 1469598103934665603ull;
        for (size_t i = 0; i < sizeof(MapKey) / 8; ++i) h = (h ^ w[i]) * 1099511628211ull;
        return h;
    }
};
// Returned BY VALUE: the cache is emptied when it grows past its limit (runs whose shapes change every step, e.g. the NCCL
// expert-parallel path with its variable row counts, keep adding keys), and a reference handed out earlier in the same call
// would then dangle.
CUtensorMap cached_map(const void* ptr, int elem_bytes, uint64_t cols, uint64_t rows, uint64_t batch,
                       uint64_t row_stride_bytes, uint64_t batch_stride_bytes, uint32_t box_cols, uint32_t box_rows, int swizzle) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    MapKey key;
    std::memset(&key, 0, sizeof(key));
    key.ptr = ptr; key.cols = cols; key.rows = rows; key.batch = batch; key.rs = row_stride_bytes; key.bs = batch_stride_bytes;
    key.bc = box_cols; key.br = box_rows; key.eb = elem_bytes; key.sw = swizzle;
    auto it = cache.find(key);
    if (it != cache.end()) return it->second;
    if (cache.size() > 8192) cache.clear();
    CUtensorMap map;
    GM_CHECK(reinterpret_cast<uintptr_t>(ptr) % 16 == 0, "TMA base address must be 16-byte aligned");
    GM_CHECK(row_stride_bytes % 16 == 0 && (batch == 1 || batch_stride_bytes % 16 == 0), "TMA strides must be multiples of 16 bytes");
    GM_CHECK(gm::make_tensor_map(&map, ptr, elem_bytes, cols, rows, batch, row_stride_bytes, batch_stride_bytes, box_cols, box_rows, swizzle),
             "cuTensorMapEncodeTiled failed");
    return cache.emplace(key, map).first->second;
}

// operand map for the bf16 GEMM: `t` is [rows, cols] or [batch, rows, cols] with cols contiguous
CUtensorMap operand_map(const torch::Tensor& t, bool mn_major, int tile_rows_k_major) {
    GM_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16, "GEMM operands must be CUDA bf16 tensors");
    GM_CHECK(t.dim() == 2 || t.dim() == 3, "GEMM operands must be 2-D or 3-D");
    GM_CHECK(t.stride(-1) == 1, "GEMM operands must have a contiguous last dimension");
    const uint64_t batch = t.dim() == 3 ? t.size(0) : 1;
    const uint64_t rows = t.size(-2), cols = t.size(-1);
    const uint64_t rs = t.stride(-2) * 2, bs = t.dim() == 3 ? t.stride(0) * 2 : 0;
    return cached_map(t.data_ptr(), 2, cols, rows, batch, rs, bs, 64, mn_major ? 64 : tile_rows_k_major, 128);
}

// D[.., M, N] = alpha * op(A) op(B)^T + beta * C, optionally accumulated into an fp32 D.
//   a_mn = false: a is [.., M, K];  a_mn = true: a is [.., K, M]   (same for b with N)
//   mode 1 (grouped M): a [rows, K], b [E, N, K] or [E, K, N], d [rows, N]; tile_expert/num_m_tiles on device
//   mode 2 (grouped K): a [rows, M] (a_mn), b [rows, N] (b_mn), d [E, M, N]; seg_ends on device
void gemm_bf16(const torch::Tensor& a, const torch::Tensor& b, torch::Tensor& d, bool a_mn, bool b_mn, double alpha,
               double beta, const c10::optional<torch::Tensor>& c, bool accumulate, int64_t mode,
               const c10::optional<torch::Tensor>& tile_expert, const c10::optional<torch::Tensor>& num_m_tiles,
               const c10::optional<torch::Tensor>& seg_ends, bool symmetric, const c10::optional<torch::Tensor>& batch_sumsq,
               int64_t scale_mode) {
    c10::cuda::CUDAGuard guard(a.device());
    gm::GemmParams p;
    std::memset(&p, 0, sizeof(p));
    p.mode = static_cast<int>(mode);
    GM_CHECK(d.is_cuda() && d.stride(-1) == 1, "GEMM output must be a CUDA tensor with a contiguous last dimension");
    GM_CHECK(d.scalar_type() == torch::kBFloat16 || d.scalar_type() == torch::kFloat32, "GEMM output must be bf16 or fp32");
    p.M = d.size(-2);
    p.N = d.size(-1);
    p.batch = d.dim() == 3 ? d.size(0) : 1;
    if (mode == gm::GEMM_GROUPED_K) {
        GM_CHECK(a_mn && b_mn, "grouped-K GEMM reads both operands MN-major");
        GM_CHECK(seg_ends.has_value() && seg_ends->scalar_type() == torch::kInt32, "grouped-K GEMM needs int32 seg_ends");
        GM_CHECK(a.size(-1) == p.M && b.size(-1) == p.N && a.size(0) == b.size(0), "grouped-K operand shapes");
        p.K = 0;
        p.seg_ends = seg_ends->data_ptr<int>();
    } else {
        p.K = a_mn ? a.size(-2) : a.size(-1);
        GM_CHECK((b_mn ? b.size(-2) : b.size(-1)) == p.K, "GEMM contraction sizes differ");
        GM_CHECK((b_mn ? b.size(-1) : b.size(-2)) == p.N, "GEMM: B does not match the output width");
        if (mode == gm::GEMM_GROUPED_M) {
            GM_CHECK(tile_expert.has_value() && num_m_tiles.has_value(), "grouped-M GEMM needs tile_expert and num_m_tiles");
            GM_CHECK(!a_mn && a.dim() == 2 && b.dim() == 3 && d.dim() == 2, "grouped-M operand ranks");
            p.tile_expert = tile_expert->data_ptr<int>();
            p.num_m_tiles = num_m_tiles->data_ptr<int>();
        } else {
            GM_CHECK((a_mn ? a.size(-1) : a.size(-2)) == p.M, "GEMM: A does not match the output height");
        }
    }
    p.D = d.data_ptr();
    p.ldd = d.stride(-2);
    p.d_batch_stride = d.dim() == 3 ? d.stride(0) : 0;
    p.out_fp32 = d.scalar_type() == torch::kFloat32;
    p.accumulate = accumulate;
    GM_CHECK(!accumulate || p.out_fp32, "accumulation needs an fp32 output");
    p.alpha = static_cast<float>(alpha);
    p.beta = static_cast<float>(beta);
    if (c.has_value()) {
        GM_CHECK(c->scalar_type() == torch::kBFloat16 && c->stride(-1) == 1, "C must be bf16 with a contiguous last dimension");
        p.C = c->data_ptr();
        p.ldc = c->stride(-2);
        p.c_batch_stride = c->dim() == 3 ? c->stride(0) : 0;
    }
    GM_CHECK(p.ldd % 8 == 0 && (p.C == nullptr || p.ldc % 8 == 0), "output row pitch must be a multiple of 8 elements");
    if (symmetric) {      // the caller vouches that alpha * A B^T + beta * C is symmetric; only the upper triangle of tiles is computed
        GM_CHECK(mode == gm::GEMM_DENSE && p.M == p.N && !p.out_fp32 && !accumulate, "symmetric GEMM: dense, square, bf16 output");
        p.symmetric = 1;
    }
    if (batch_sumsq.has_value()) {
        GM_CHECK(mode == gm::GEMM_DENSE && batch_sumsq->is_cuda() && batch_sumsq->scalar_type() == torch::kFloat32 &&
                 batch_sumsq->is_contiguous() && batch_sumsq->numel() == p.batch && (scale_mode == 1 || scale_mode == 2),
                 "batch_sumsq: one fp32 value per batched problem of a dense GEMM, scale_mode 1 or 2");
        p.batch_sumsq = batch_sumsq->data_ptr<float>();
        p.scale_mode = static_cast<int>(scale_mode);
    }
    p.status = status_tensor(a.device().index()).data_ptr<int>();
    // split-K: a long contraction with too few output tiles to fill the GPU (weight gradients) is shared by several CTAs per tile
    p.split_k = 1;
    if (mode == gm::GEMM_DENSE && p.out_fp32) {
        const int64_t tiles = ((p.M + 255) / 256) * 2 * ((p.N + 255) / 256) * p.batch;      // CTA pairs own 256-row tiles
        const int64_t k_blocks = (p.K + 63) / 64;
        if (tiles * 2 <= sm_count() && k_blocks >= 16)
            p.split_k = static_cast<int>(std::min<int64_t>(sm_count() / tiles, k_blocks / 8));
        if (p.split_k > 1 && !accumulate) d.zero_();
    }
    const CUtensorMap& ta = operand_map(a, a_mn, 128);
    const CUtensorMap& tb = operand_map(b, b_mn, 128);
    const int eb = p.out_fp32 ? 4 : 2;
    const CUtensorMap& td = cached_map(d.data_ptr(), eb, p.N, p.M, d.dim() == 3 ? d.size(0) : 1, p.ldd * eb,
                                       d.dim() == 3 ? d.stride(0) * eb : 0, 128 / eb, 128, 128);
    cudaError_t e = gm::launch_gemm_bf16(ta, tb, td, p, a_mn, b_mn, sm_count(), current_stream());
    GM_CHECK(e == cudaSuccess, cudaGetErrorString(e));
}

// ---- MXFP8 ----------------------------------------------------------------------------------------
int64_t sf_records(int64_t rows, int64_t k) { return ((rows + 127) / 128) * ((k + 127) / 128); }

// x [.., rows, cols] bf16 (last dim contiguous, uniform row pitch) -> (q e4m3 as uint8 [.., rows, cols], scales uint8 [batch, records * 512])
std::vector<torch::Tensor> mxfp8_quantize(const torch::Tensor& x, const c10::optional<torch::Tensor>& rows_limit) {
    c10::cuda::CUDAGuard guard(x.device());
    GM_CHECK(x.is_cuda() && x.scalar_type() == torch::kBFloat16 && (x.dim() == 2 || x.dim() == 3), "mxfp8_quantize wants a 2-D or 3-D bf16 CUDA tensor");
    GM_CHECK(x.stride(-1) == 1 && x.size(-1) % 32 == 0 && x.stride(-2) % 8 == 0, "mxfp8_quantize: last dimension contiguous, multiple of 32");
    const int64_t batch = x.dim() == 3 ? x.size(0) : 1, rows = x.size(-2), cols = x.size(-1);
    GM_CHECK(batch == 1 || rows % 128 == 0 || x.is_contiguous(), "mxfp8_quantize: batched input must be contiguous");
    auto q = gm::out_empty(x.sizes(), x.options().dtype(torch::kUInt8));
    // not cleared: bytes of rows that exist are all written; the rest belongs to rows the GEMM clips
    auto sf = gm::out_empty({batch, sf_records(rows, cols) * 512}, x.options().dtype(torch::kUInt8));
    for (int64_t z = 0; z < batch; ++z) {
        const auto* src = static_cast<const at::BFloat16*>(x.data_ptr()) + (x.dim() == 3 ? z * x.stride(0) : 0);
        gm::launch_quantize_rows(src, q.data_ptr<uint8_t>() + z * rows * cols, sf.data_ptr<uint8_t>() + z * sf.stride(0), rows,
                                 static_cast<int>(cols), x.stride(-2), rows_limit.has_value() ? rows_limit->data_ptr<int>() : nullptr,
                                 current_stream());
    }
    return {q, sf};
}

// w [.., rows, cols] bf16 contiguous -> (q [.., rows, cols], scales along cols, qt [.., cols, rows], scales along the original rows)
std::vector<torch::Tensor> mxfp8_quantize_weight(const torch::Tensor& w) {
    c10::cuda::CUDAGuard guard(w.device());
    GM_CHECK(w.is_cuda() && w.scalar_type() == torch::kBFloat16 && w.is_contiguous() && (w.dim() == 2 || w.dim() == 3), "mxfp8_quantize_weight wants a contiguous bf16 CUDA tensor");
    const int64_t batch = w.dim() == 3 ? w.size(0) : 1, rows = w.size(-2), cols = w.size(-1);
    GM_CHECK(rows % 32 == 0 && cols % 32 == 0, "mxfp8_quantize_weight: both dimensions must be multiples of 32");
    auto opt = w.options().dtype(torch::kUInt8);
    auto q = gm::out_empty(w.sizes(), opt);
    auto qt = w.dim() == 3 ? gm::out_empty({batch, cols, rows}, opt) : gm::out_empty({cols, rows}, opt);
    auto sf = gm::out_empty({batch, sf_records(rows, cols) * 512}, opt);
    auto sft = gm::out_empty({batch, sf_records(cols, rows) * 512}, opt);
    gm::launch_quantize_weight_dual(w.data_ptr(), q.data_ptr(), sf.data_ptr(), qt.data_ptr(), sft.data_ptr(), static_cast<int>(batch),
                                    static_cast<int>(rows), static_cast<int>(cols), sf.stride(0), sft.stride(0), current_stream());
    return {q, sf, qt, sft};
}

// d [.., M, N] bf16 = alpha * a [.., M, K] b [.., N, K]^T from e4m3 bytes and their scale records.
// grouped: a [rows, K] in padded expert-major order, b [E, N, K], tile_expert / num_m_tiles on the device.
void gemm_mxfp8(const torch::Tensor& a, const torch::Tensor& sfa, const torch::Tensor& b, const torch::Tensor& sfb, torch::Tensor& d, double alpha,
                const c10::optional<torch::Tensor>& tile_expert, const c10::optional<torch::Tensor>& num_m_tiles) {
    c10::cuda::CUDAGuard guard(a.device());
    GM_CHECK(a.is_cuda() && a.scalar_type() == torch::kUInt8 && b.scalar_type() == torch::kUInt8 && a.is_contiguous() && b.is_contiguous(), "mxfp8 operands are contiguous uint8 tensors");
    GM_CHECK(d.scalar_type() == torch::kBFloat16 && d.stride(-1) == 1 && d.stride(-2) % 8 == 0, "mxfp8 output is bf16 with a 16-byte aligned row pitch");
    gm::Mxfp8Params p;
    std::memset(&p, 0, sizeof(p));
    p.M = d.size(-2); p.N = d.size(-1); p.K = a.size(-1);
    GM_CHECK(b.size(-1) == p.K && b.size(-2) == p.N && p.K % 128 == 0, "mxfp8 GEMM shapes (K must be a multiple of 128)");
    p.grouped = tile_expert.has_value();
    if (p.grouped) {
        GM_CHECK(a.dim() == 2 && b.dim() == 3 && d.dim() == 2 && num_m_tiles.has_value() && a.size(0) % 256 == 0, "grouped mxfp8 operand ranks (rows padded to 256)");
        p.tile_expert = tile_expert->data_ptr<int>();
        p.num_m_tiles = num_m_tiles->data_ptr<int>();
        p.batch = 1;
    } else {
        GM_CHECK(a.size(-2) == p.M && a.dim() == d.dim() && b.dim() == d.dim(), "mxfp8 GEMM: operand ranks");
        p.batch = d.dim() == 3 ? d.size(0) : 1;
    }
    p.sfa_row_blocks = (a.size(-2) + 127) / 128;
    p.sfb_row_blocks = (p.N + 127) / 128;
    const int64_t kb = p.K / 128;
    GM_CHECK(sfa.numel() == (a.dim() == 3 ? a.size(0) : 1) * p.sfa_row_blocks * kb * 512, "mxfp8 GEMM: A scale tensor size");
    GM_CHECK(sfb.numel() == (b.dim() == 3 ? b.size(0) : 1) * p.sfb_row_blocks * kb * 512, "mxfp8 GEMM: B scale tensor size");
    p.sfa = sfa.data_ptr<uint8_t>();
    p.sfb = sfb.data_ptr<uint8_t>();
    p.alpha = static_cast<float>(alpha);
    p.status = status_tensor(a.device().index()).data_ptr<int>();
    const uint64_t ab = a.dim() == 3 ? a.size(0) : 1, bb = b.dim() == 3 ? b.size(0) : 1;
    const CUtensorMap& ta = cached_map(a.data_ptr(), 1, p.K, a.size(-2), ab, p.K, a.size(-2) * static_cast<uint64_t>(p.K), 128, 128, 128);
    const CUtensorMap& tb = cached_map(b.data_ptr(), 1, p.K, p.N, bb, p.K, static_cast<uint64_t>(p.N) * p.K, 128, 128, 128);
    const CUtensorMap& td = cached_map(d.data_ptr(), 2, p.N, p.M, d.dim() == 3 ? d.size(0) : 1, d.stride(-2) * 2, d.dim() == 3 ? d.stride(0) * 2 : 0, 64, 128, 128);
    // scale arrays as [records, 128 words]: one TMA row per 512-byte record, no swizzle
    GM_CHECK(reinterpret_cast<uintptr_t>(sfa.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(sfb.data_ptr()) % 16 == 0, "scale arrays must be 16-byte aligned");
    const CUtensorMap& tsfa = cached_map(sfa.data_ptr(), 4, 128, sfa.numel() / 512, 1, 512, 0, 128, 1, 0);
    const CUtensorMap& tsfb = cached_map(sfb.data_ptr(), 4, 128, sfb.numel() / 512, 1, 512, 0, 128, 1, 0);
    cudaError_t e = gm::launch_gemm_mxfp8(ta, tb, td, tsfa, tsfb, p, sm_count(), current_stream());
    GM_CHECK(e == cudaSuccess, cudaGetErrorString(e));
}

// map over a [B, T, H, 64] bf16 view whose tokens are rows of a wider matrix (e.g. the packed QKV projection output)
CUtensorMap head_map(const torch::Tensor& t, int box_rows) {
    GM_CHECK(t.is_cuda() && t.scalar_type() == torch::kBFloat16 && t.dim() == 4, "attention operands must be [B, T, H, D] bf16 CUDA tensors");
    GM_CHECK(t.stride(3) == 1 && t.stride(2) == t.size(3) && t.stride(0) == t.size(1) * t.stride(1),
             "attention operands must be token-major with contiguous heads");
    return cached_map(t.data_ptr(), 2, t.size(2) * t.size(3), t.size(0) * t.size(1), 1, t.stride(1) * 2, 0, 64, box_rows, 128);
}

// Returns (out [B,T,H,64] bf16, lse [B,H,T] fp32).
const int* doc_start_ptr(const c10::optional<torch::Tensor>& doc_start, int64_t tokens) {
    if (!doc_start.has_value()) return nullptr;
    GM_CHECK(doc_start->is_cuda() && doc_start->scalar_type() == torch::kInt32 && doc_start->is_contiguous() && doc_start->numel() == tokens,
             "doc_start must be a contiguous int32 CUDA tensor with one entry per token");
    return doc_start->data_ptr<int>();
}

// `window_tensor`: optional 0-dim (or 1-element) int32 CUDA tensor holding the look-back; the kernels read it on the device, so the same
// (captured) launch follows a window schedule without a new host value (the reference's device-resident window,
// experiments/046-fa4-device-window.patch).
const int* window_word(const c10::optional<torch::Tensor>& window_tensor) {
    if (!window_tensor.has_value()) return nullptr;
    GM_CHECK(window_tensor->is_cuda() && window_tensor->scalar_type() == torch::kInt32 && window_tensor->numel() == 1,
             "window_tensor must be a one-element int32 CUDA tensor");
    return window_tensor->data_ptr<int>();
}

// `quantize`: also return the MXFP8 copy of out (payload uint8 [B*T, H*64], scale records), written by the kernel's epilogue.
// `single_tile`: keep the call on the kernel with one query tile per CTA (the other kernel is checked against it).
std::vector<torch::Tensor> attn_fwd(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v, int64_t window, double scale,
                                    double softcap, const c10::optional<torch::Tensor>& doc_start, bool quantize, bool single_tile,
                                    const c10::optional<torch::Tensor>& window_tensor) {
    c10::cuda::CUDAGuard guard(q.device());
    const int B = q.size(0), T = q.size(1), H = q.size(2), D = q.size(3), Hkv = k.size(2);
    GM_CHECK((D == 64 || D == 128) && k.size(3) == D && v.size(3) == 64 && T % 128 == 0 && H % Hkv == 0,
             "attention kernel: query/key heads 64 or 128 wide, value heads 64 wide, sequence length multiple of 128");
    gm::AttnParams p;
    std::memset(&p, 0, sizeof(p));
    p.batch = B; p.heads = H; p.seq_len = T; p.group = H / Hkv; p.qk_dim = D;
    p.window = static_cast<int>(std::min<int64_t>(window, T));
    p.scale = static_cast<float>(scale);
    p.scale_log2e = static_cast<float>(scale * 1.4426950408889634);
    p.softcap = static_cast<float>(softcap);
    p.doc_start = doc_start_ptr(doc_start, static_cast<int64_t>(B) * T);
    auto out = gm::out_empty({B, T, H, 64}, q.options());
    auto lse = gm::out_empty({B, H, T}, q.options().dtype(torch::kFloat32));
    p.out = out.data_ptr(); p.out_stride = H * 64; p.lse = lse.data_ptr<float>();
    torch::Tensor oq, osf;
    if (quantize) {
        const int64_t rows = static_cast<int64_t>(B) * T, cols = static_cast<int64_t>(H) * 64;
        oq = gm::out_empty({rows, cols}, q.options().dtype(torch::kUInt8));
        osf = gm::out_empty({sf_records(rows, cols) * 512}, q.options().dtype(torch::kUInt8));
        p.out_q = oq.data_ptr<uint8_t>();
        p.out_sf = osf.data_ptr<uint8_t>();
    }
    p.status = status_tensor(q.device().index()).data_ptr<int>();
    p.single_tile = single_tile ? 1 : 0;
    p.window_ptr = window_word(window_tensor);
    cudaError_t e = gm::launch_attn_fwd(head_map(q, 128), head_map(k, 128), head_map(v, 128), p, current_stream());
    GM_CHECK(e == cudaSuccess, cudaGetErrorString(e));
    if (quantize) return {out, lse, oq, osf};
    return {out, lse};
}

// Backward.  `unpipelined`: keep the call on the kernel that issues its products in program order (the other is checked against it).
// q, k, v, out, d_out: [B,T,H(kv),64] bf16 views; lse [B,H,T].  dk, dv: [B,T,Hkv,64] bf16 views that are written
// (they may be column slices of a packed gradient buffer).  Returns dq as fp32 [B,T,H,64].
torch::Tensor attn_bwd(const torch::Tensor& q, const torch::Tensor& k, const torch::Tensor& v, const torch::Tensor& out,
                       const torch::Tensor& d_out, const torch::Tensor& lse, torch::Tensor& dk, torch::Tensor& dv, int64_t window,
                       double scale, double softcap, const c10::optional<torch::Tensor>& doc_start, bool unpipelined,
                       const c10::optional<torch::Tensor>& window_tensor) {
    c10::cuda::CUDAGuard guard(q.device());
    const int B = q.size(0), T = q.size(1), H = q.size(2), D = q.size(3), Hkv = k.size(2);
    GM_CHECK((D == 64 || D == 128) && k.size(3) == D && v.size(3) == 64 && T % 128 == 0 && H % Hkv == 0,
             "attention kernel: query/key heads 64 or 128 wide, value heads 64 wide, sequence length multiple of 128");
    GM_CHECK(dk.stride(3) == 1 && dk.stride(2) == D && dv.stride(3) == 1 && dv.stride(2) == 64 && dk.stride(1) % 8 == 0 && dv.stride(1) % 8 == 0,
             "dk/dv must be token-major views with contiguous heads and 16-byte aligned rows");
    GM_CHECK(out.stride(3) == 1 && out.stride(2) == 64 && d_out.stride(3) == 1 && d_out.stride(2) == 64, "out/d_out layout");
    gm::AttnParams p;
    std::memset(&p, 0, sizeof(p));
    p.batch = B; p.heads = H; p.seq_len = T; p.group = H / Hkv; p.qk_dim = D;
    p.window = static_cast<int>(std::min<int64_t>(window, T));
    p.scale = static_cast<float>(scale);
    p.scale_log2e = static_cast<float>(scale * 1.4426950408889634);
    p.softcap = static_cast<float>(softcap);
    p.doc_start = doc_start_ptr(doc_start, static_cast<int64_t>(B) * T);
    p.lse = const_cast<float*>(lse.data_ptr<float>());
    auto delta = gm::out_empty({B, H, T}, lse.options());
    auto dq = gm::out_zeros({B, T, H, D}, lse.options());
    p.delta = delta.data_ptr<float>();
    p.dq_accum = dq.data_ptr<float>();
    p.dk = dk.data_ptr(); p.dv = dv.data_ptr(); p.dkv_stride = dk.stride(1); p.dv_stride = dv.stride(1);
    p.status = status_tensor(q.device().index()).data_ptr<int>();
    p.single_tile = unpipelined ? 1 : 0;
    p.window_ptr = window_word(window_tensor);
    const CUtensorMap& tdq = cached_map(dq.data_ptr(), 4, static_cast<uint64_t>(H) * D, static_cast<uint64_t>(B) * T, 1,
                                        static_cast<uint64_t>(H) * D * 4, 0, 32, 128, 128);
    cudaError_t e = gm::launch_attn_bwd(head_map(q, 128), head_map(k, 128), head_map(v, 128), head_map(d_out, 128), tdq, p,
                                        d_out.data_ptr(), out.data_ptr(), d_out.stride(1), out.stride(1), delta.data_ptr<float>(),
                                        current_stream());
    GM_CHECK(e == cudaSuccess, cudaGetErrorString(e));
    return dq;
}

}  // namespace

namespace gm {
int* status_word(int device) { return status_tensor(device).data_ptr<int>(); }
}  // namespace gm

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("read_status", &read_status, "status word of the current device (0 = no bounded wait gave up)");
    m.def("reset_status", &reset_status);
    m.def("status_word_tensor", &status_word_tensor);
    m.def("gemm_bf16", &gemm_bf16, py::arg("a"), py::arg("b"), py::arg("d"), py::arg("a_mn") = false, py::arg("b_mn") = false,
          py::arg("alpha") = 1.0, py::arg("beta") = 0.0, py::arg("c") = py::none(), py::arg("accumulate") = false,
          py::arg("mode") = 0, py::arg("tile_expert") = py::none(), py::arg("num_m_tiles") = py::none(),
          py::arg("seg_ends") = py::none(), py::arg("symmetric") = false,
          py::arg("batch_sumsq") = py::none(), py::arg("scale_mode") = 0);
    m.def("mxfp8_quantize", &mxfp8_quantize, py::arg("x"), py::arg("rows_limit") = py::none());
    m.def("mxfp8_quantize_weight", &mxfp8_quantize_weight);
    m.def("gemm_mxfp8", &gemm_mxfp8, py::arg("a"), py::arg("sfa"), py::arg("b"), py::arg("sfb"), py::arg("d"), py::arg("alpha") = 1.0,
          py::arg("tile_expert") = py::none(), py::arg("num_m_tiles") = py::none());
    m.def("attn_fwd", &attn_fwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("window"), py::arg("scale"), py::arg("softcap") = 0.0,
          py::arg("doc_start") = py::none(), py::arg("quantize") = false, py::arg("single_tile") = false, py::arg("window_tensor") = py::none());
    m.def("attn_bwd", &attn_bwd, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("out"), py::arg("d_out"), py::arg("lse"), py::arg("dk"),
          py::arg("dv"), py::arg("window"), py::arg("scale"), py::arg("softcap") = 0.0, py::arg("doc_start") = py::none(),
          py::arg("unpipelined") = false, py::arg("window_tensor") = py::none());
    gm::register_kernels(m);
}

// Guarded allocations of the bounds-checked build (see guarded_alloc.h).
#include "guarded_alloc.h"

#ifdef GM_CHECK_BOUNDS
#include <cstdlib>
#include <deque>

namespace gm {
namespace {

constexpr int64_t kGuardBytes = 256;
constexpr int kPattern = 0xA5;
constexpr size_t kMaxRecords = 8192;          // older buffers are dropped unverified: a debugging aid must not hold a training run's memory

struct GuardRecord {
    torch::Tensor raw;                         // uint8 [kGuardBytes + padded payload + kGuardBytes]
    int64_t payload_bytes;
};

std::deque<GuardRecord>& records() {
    static std::deque<GuardRecord> r;
    return r;
}

torch::Tensor guarded(at::IntArrayRef sizes, const at::TensorOptions& options, bool zero) {
    int64_t n = 1;
    for (int64_t s : sizes) n *= s;
    if (!output_guards_enabled() || !options.device().is_cuda() || n == 0) return zero ? torch::zeros(sizes, options) : torch::empty(sizes, options);
    const auto dtype = c10::typeMetaToScalarType(options.dtype());
    const int64_t bytes = n * static_cast<int64_t>(c10::elementSize(dtype));
    const int64_t padded = (bytes + kGuardBytes - 1) / kGuardBytes * kGuardBytes;
    auto raw = torch::empty({kGuardBytes + padded + kGuardBytes}, options.dtype(torch::kUInt8));
    raw.narrow(0, 0, kGuardBytes).fill_(kPattern);
    raw.narrow(0, kGuardBytes + bytes, padded - bytes + kGuardBytes).fill_(kPattern);
    auto payload = raw.narrow(0, kGuardBytes, bytes);
    if (zero) payload.zero_();
    auto& rec = records();
    rec.push_back({raw, bytes});
    if (rec.size() > kMaxRecords) rec.pop_front();
    return payload.view(dtype).view(sizes);
}

}  // namespace

bool output_guards_enabled() {
    static const bool on = [] { const char* e = std::getenv("GM_CANARIES"); return e != nullptr && e[0] == '1'; }();
    return on;
}

torch::Tensor out_empty(at::IntArrayRef sizes, const at::TensorOptions& options) { return guarded(sizes, options, false); }
torch::Tensor out_zeros(at::IntArrayRef sizes, const at::TensorOptions& options) { return guarded(sizes, options, true); }
torch::Tensor out_empty_like(const torch::Tensor& like) {
    return like.is_contiguous() ? guarded(like.sizes(), like.options(), false) : torch::empty_like(like);
}
torch::Tensor out_zeros_like(const torch::Tensor& like) {
    return like.is_contiguous() ? guarded(like.sizes(), like.options(), true) : torch::zeros_like(like);
}

int64_t verify_output_guards() {
    auto& rec = records();
    if (rec.empty()) return 0;
    torch::Tensor bad;                         // device-side count, read once
    for (const GuardRecord& r : rec) {
        const int64_t total = r.raw.numel();
        auto changed = r.raw.narrow(0, 0, kGuardBytes).ne(kPattern).sum() +
                       r.raw.narrow(0, kGuardBytes + r.payload_bytes, total - kGuardBytes - r.payload_bytes).ne(kPattern).sum();
        if (!bad.defined()) bad = changed;
        else if (bad.device() == changed.device()) bad = bad + changed;
        else bad = bad + changed.to(bad.device());
    }
    rec.clear();
    return bad.item<int64_t>();
}

}  // namespace gm
#endif

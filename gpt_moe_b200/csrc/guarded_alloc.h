// Allocation of the tensors the bindings hand to kernels as outputs or scratch.
//
// Normal build: plain torch::empty / torch::zeros.  Bounds-checked build (-DGM_CHECK_BOUNDS=1) with GM_CANARIES=1 in the
// environment: every CUDA tensor is carved out of a larger byte buffer with 256 bytes of a fixed pattern before and after
// its payload (the payload stays 256-byte aligned), and the buffers are remembered.  `verify_output_guards()` counts the
// pattern bytes that have changed since and forgets the buffers: a kernel that wrote before or past an output of its own
// is then reported by the Python layer's status check instead of corrupting a neighbouring allocation unseen.
// The reference has no counterpart (it relies on the kernels being right by construction).
#pragma once
#include <torch/extension.h>

namespace gm {

#ifdef GM_CHECK_BOUNDS
torch::Tensor out_empty(at::IntArrayRef sizes, const at::TensorOptions& options);
torch::Tensor out_zeros(at::IntArrayRef sizes, const at::TensorOptions& options);
torch::Tensor out_empty_like(const torch::Tensor& like);
torch::Tensor out_zeros_like(const torch::Tensor& like);
int64_t verify_output_guards();
bool output_guards_enabled();
#else
inline torch::Tensor out_empty(at::IntArrayRef sizes, const at::TensorOptions& options) { return torch::empty(sizes, options); }
inline torch::Tensor out_zeros(at::IntArrayRef sizes, const at::TensorOptions& options) { return torch::zeros(sizes, options); }
inline torch::Tensor out_empty_like(const torch::Tensor& like) { return torch::empty_like(like); }
inline torch::Tensor out_zeros_like(const torch::Tensor& like) { return torch::zeros_like(like); }
inline int64_t verify_output_guards() { return 0; }
inline bool output_guards_enabled() { return false; }
#endif

}  // namespace gm

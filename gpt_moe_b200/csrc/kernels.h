// Launchers of the non-GEMM kernels (raw pointers; defined in the .cu files) and the pybind registration hook.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace pybind11 { class module_; }

namespace gm {
void register_kernels(pybind11::module_& m);
// device pointer of the per-device status word that kernels set when a bounded wait or a capacity check gives up
int* status_word(int device);
}

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link-time libcuda dependency).
#include "gemm.h"

#include <cudaTypedefs.h>
#include <mutex>

namespace gm {

static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
        }
    });
    return fn;
}

bool make_tensor_map(CUtensorMap* out, const void* base, int elem_bytes, uint64_t cols, uint64_t rows, uint64_t batch,
                     uint64_t row_stride_bytes, uint64_t batch_stride_bytes, uint32_t box_cols, uint32_t box_rows,
                     int swizzle_bytes) {
    auto fn = encode_fn();
    if (fn == nullptr) return false;
    cuuint64_t dims[3] = {cols, rows, batch};
    cuuint64_t strides[2] = {row_stride_bytes, batch_stride_bytes};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t elem_strides[3] = {1, 1, 1};
    CUtensorMapDataType dt = elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                             : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    CUtensorMapSwizzle sw = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                            : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                            : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
    if (batch == 1) strides[1] = row_stride_bytes * rows;   // any multiple of 16 bytes is accepted
    CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

bool make_tensor_map_bf16(CUtensorMap* out, const void* base, uint64_t cols, uint64_t rows, uint64_t batch,
                          uint64_t row_stride_elems, uint64_t batch_stride_elems, uint32_t box_cols, uint32_t box_rows) {
    return make_tensor_map(out, base, 2, cols, rows, batch, row_stride_elems * 2, batch_stride_elems * 2, box_cols, box_rows, 128);
}

}  // namespace gm

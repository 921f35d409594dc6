// Issue and completion time of a chain of tcgen05.mma instructions, measured on the device with clock64.
//
// One CTA, one issuing thread, operands in shared memory (zeros) or TMEM, descriptors formed before the loop.  The figures
// this gives on a B200 decide how the attention kernels are laid out:
//   - an instruction takes max(N / 2, about 56) clocks with M = 128: 65 at N = 128, 130 at N = 256, but still 56-58 at
//     N = 64 or 16, so a product with N = 64 (P V, dV, dK, dQ at head size 64) runs the tensor core at about half rate;
//   - M = 64 takes as long as M = 128 at the same N (half the rate);
//   - the A operand may come from TMEM at the same cost;
//   - forming a descriptor from its fields inside the loop instead of adding to a prepared one costs the issuing thread
//     more than the instruction does.
// Used by `python -m gpt_moe_b200.utils.kernel_cases mma_issue`.
#include "../common/ptx.cuh"
#include "../kernels_decl.h"

namespace gm {

template <int M, int N, bool A_TMEM, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(128, 1) mma_issue_kernel(long long* out, int count, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ uint64_t bar;
    __shared__ uint32_t slot;
    const int warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < 64 * 1024 / 4; i += 128) reinterpret_cast<uint32_t*>(smem)[i] = 0;
    if (threadIdx.x == 0) { mbar_init(&bar, 1); fence_barrier_init(); }
    if (warp == 0) { tmem_alloc(&slot, 512); tmem_relinquish(); }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tb = slot;
    if (threadIdx.x == 0) {
        const uint32_t a_addr = smem_u32(smem), b_addr = smem_u32(smem + 32768);
        constexpr uint32_t idesc = make_idesc_bf16(M, N, A_MN, B_MN);
        uint64_t adesc[4], bdesc[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            adesc[k] = A_MN ? make_smem_desc(a_addr + k * 2048, 128 * 128, 1024) : make_smem_desc(a_addr + k * 32, 16, 1024);
            bdesc[k] = B_MN ? make_smem_desc(b_addr + k * 2048, 128 * 128, 1024) : make_smem_desc(b_addr + k * 32, 16, 1024);
        }
        for (int rep = 0; rep < 3; ++rep) {                      // the last repetition is the one reported
            const long long t0 = clock64();
#pragma unroll 1
            for (int i = 0; i < count; i += 4) {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    if (A_TMEM) umma_f16_ta(tb, tb + 448 + k * 8, bdesc[k], idesc, (i | k) != 0);
                    else umma_f16(tb, adesc[k], bdesc[k], idesc, (i | k) != 0);
                }
            }
            const long long t1 = clock64();
            umma_commit(&bar);
            if (!mbar_wait(&bar, rep & 1)) { atomicExch(status, 701); break; }
            const long long t2 = clock64();
            out[0] = t1 - t0;
            out[1] = t2 - t0;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) { tc_fence_after(); tmem_dealloc(tb, 512); }
}

template <int M, int N, bool A_TMEM, bool A_MN, bool B_MN>
static cudaError_t run_mma_issue(long long* out, int count, int* status, cudaStream_t stream) {
    auto kernel = mma_issue_kernel<M, N, A_TMEM, A_MN, B_MN>;
    constexpr int smem = 66 * 1024;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    kernel<<<1, 128, smem, stream>>>(out, count, status);
    return cudaGetLastError();
}

// shape: 0 M128 N128, 1 M128 N256, 2 M128 N64, 3 M128 N16, 4 M128 N64 with A in TMEM and B MN-major (the P V product),
//        5 M128 N256 with A in TMEM, 6 M64 N256 with A MN-major, 7 M64 N128 with A MN-major.  `count`: a multiple of 4.
cudaError_t launch_mma_issue(int shape, long long* out, int count, int* status, cudaStream_t stream) {
    switch (shape) {
        case 0: return run_mma_issue<128, 128, false, false, false>(out, count, status, stream);
        case 1: return run_mma_issue<128, 256, false, false, false>(out, count, status, stream);
        case 2: return run_mma_issue<128, 64, false, false, false>(out, count, status, stream);
        case 3: return run_mma_issue<128, 16, false, false, false>(out, count, status, stream);
        case 4: return run_mma_issue<128, 64, true, false, true>(out, count, status, stream);
        case 5: return run_mma_issue<128, 256, true, false, false>(out, count, status, stream);
        case 6: return run_mma_issue<64, 256, false, true, false>(out, count, status, stream);
        case 7: return run_mma_issue<64, 128, false, true, false>(out, count, status, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace gm

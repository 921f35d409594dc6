// Allocation-free variant of `residual_bwd` (see residual_bwd_noalloc.h for who needs it and the contract).
// Same arithmetic and the same fixed reduction order as the allocating path in norm_rope.cu: one partial sum per block
// into scratch, then a single block adds the partials.  The scratch is a file-scope device array instead of a tensor.
#include "residual_bwd_noalloc.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int kMaxBlocks = GM_RESIDUAL_BWD_NOALLOC_SCRATCH_FLOATS;
constexpr int kMaxDevices = 64;

// Per-GPU scratch: the partial sum of each block.  Every call overwrites the entries it uses before reading them, so
// nothing has to be cleared between calls.
static __device__ __align__(256) float g_partial_scratch[kMaxBlocks];

// In host code `g_partial_scratch` is only a handle for the symbol, not a device address; the address each device gives
// the array is looked up once (with that device current) and cached here.
float* g_scratch_address[kMaxDevices] = {nullptr};

__global__ void __launch_bounds__(256)
residual_bwd_noalloc_kernel(const float* __restrict__ dxn, const __nv_bfloat16* __restrict__ branch, const float* __restrict__ beta,
                            __nv_bfloat16* __restrict__ dbranch, float* __restrict__ partial, long long n) {
    __shared__ float red[8];
    const float b = *beta;
    float dot = 0.f;
    for (long long i = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) * 4; i < n; i += static_cast<long long>(gridDim.x) * blockDim.x * 4) {
        const float4 g = *reinterpret_cast<const float4*>(dxn + i);
        const uint2 raw = *reinterpret_cast<const uint2*>(branch + i);
        const float2 r0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 r1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        dot += g.x * r0.x + g.y * r0.y + g.z * r1.x + g.w * r1.y;
        const __nv_bfloat162 o0 = __floats2bfloat162_rn(b * g.x, b * g.y), o1 = __floats2bfloat162_rn(b * g.z, b * g.w);
        uint2 out;
        out.x = *reinterpret_cast<const uint32_t*>(&o0);
        out.y = *reinterpret_cast<const uint32_t*>(&o1);
        *reinterpret_cast<uint2*>(dbranch + i) = out;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = dot;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += red[w];
        partial[blockIdx.x] = t;
    }
}

// one block; thread t adds partials t, t+256, ... and the 8 warps are combined in a fixed order
__global__ void __launch_bounds__(256)
residual_bwd_noalloc_finish(const float* __restrict__ partial, float* __restrict__ dbeta, int blocks) {
    __shared__ float red[8][32];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    float s = 0.f;
    if (tx == 0)
        for (int r = ty; r < blocks; r += 8) s += partial[r];
    red[ty][tx] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += red[w][0];
        dbeta[0] = t;
    }
}

}  // namespace

extern "C" int gm_residual_bwd_noalloc(const float* dxn, const void* branch, const float* beta, void* dbranch, float* dbeta,
                                       long long n, void* stream) {
    if (dxn == nullptr || branch == nullptr || beta == nullptr || dbranch == nullptr || dbeta == nullptr) return 1;
    if (n <= 0 || (n % 4) != 0 || n > GM_RESIDUAL_BWD_NOALLOC_MAX_ELEMS) return 1;
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return 2;
    if (g_scratch_address[device] == nullptr) {
        // first call on this device (documented: outside stream capture): resolve the array's device address
        float* address = nullptr;
        if (cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_partial_scratch) != cudaSuccess || address == nullptr) return 2;
        g_scratch_address[device] = address;
    }
    float* scratch = g_scratch_address[device];
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // same block count as the allocating path, so both sum in the same order
    const long long want = n / 4 / 256 + 1;
    const int blocks = static_cast<int>(want < kMaxBlocks ? want : kMaxBlocks);
    // launch errors are returned by the launch that caused them (cudaPeekAtLastError after each would also show an error left
    // by earlier work and cudaGetLastError would clear it: neither is this function's business)
    void* args1[] = {&dxn, &branch, &beta, &dbranch, &scratch, &n};
    if (cudaLaunchKernel(reinterpret_cast<const void*>(residual_bwd_noalloc_kernel), dim3(blocks), dim3(256), args1, 0, s) != cudaSuccess) return 2;
    int blocks_arg = blocks;
    const float* partial = scratch;
    void* args2[] = {&partial, &dbeta, &blocks_arg};
    if (cudaLaunchKernel(reinterpret_cast<const void*>(residual_bwd_noalloc_finish), dim3(1), dim3(256), args2, 0, s) != cudaSuccess) return 2;
    return 0;
}

extern "C" void gm_residual_bwd_noalloc_forget(void) {
    for (int d = 0; d < kMaxDevices; ++d) g_scratch_address[d] = nullptr;
}

// Shared helpers for the hand-written sm_100a kernels.  Every exported launcher has a C ABI
// (raw pointers, sizes, a cudaStream_t) so that it can be called without any binding layer.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define NG_EXPORT extern "C" __attribute__((visibility("default")))

// Status codes returned by launchers (0 = launched).  A launcher never allocates.
enum { NG_OK = 0, NG_BAD_SIZE = 1, NG_LAUNCH_FAILED = 2, NG_BAD_DTYPE = 3 };

// Bits a kernel may set in the engine's device status word instead of trapping.
enum { NG_STATUS_BAD_TOKEN = 1, NG_STATUS_BAD_PAGE = 2, NG_STATUS_BAD_POSITION = 4 };

__device__ __forceinline__ float ng_ld(const float* p) { return *p; }
__device__ __forceinline__ float ng_ld(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void ng_st(float* p, float v) { *p = v; }
__device__ __forceinline__ void ng_st(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// An input that is either one tensor of type TI, or n_part float32 partial sums `stride`
// elements apart (split-K products).  The sum is taken in ascending order and rounded to TO, the
// type the unsplit product would have been stored in, so both routes round at the same place.
template <typename TO, typename TI>
__device__ __forceinline__ float ng_ld_sum(const TI* p, size_t idx, int n_part, size_t stride) {
    if (n_part <= 1) return ng_ld(p + idx);
    float v = 0.f;
    for (int s = 0; s < n_part; ++s) v += ng_ld(p + s * stride + idx);
    TO r;
    ng_st(&r, v);
    return ng_ld(&r);
}

__device__ __forceinline__ float ng_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float ng_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  The order of the
// additions depends only on the block size, so a row's result does not depend on the batch.
__device__ __forceinline__ float ng_block_sum(float v, float* smem32) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
    v = ng_warp_sum(v);
    __syncthreads();
    if (lane == 0) smem32[warp] = v;
    __syncthreads();
    float r = (lane < nwarp) ? smem32[lane] : 0.f;
    r = ng_warp_sum(r);
    return r;
}

// ---- programmatic dependent launch ---------------------------------------------------------
// Every kernel of the package is launched with the "programmatic stream serialization"
// attribute, signals at its top that the next kernel of the stream may be scheduled
// (ng_pdl_trigger), and waits (ng_pdl_wait) before it first reads what earlier kernels wrote or
// writes anything to global memory.  The next kernel's launch latency and prologue then overlap
// this kernel's tail.  Without the attribute both instructions do nothing.
// NEUROGRID_B200_PDL=0 in the environment switches the attribute off.
__device__ __forceinline__ void ng_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void ng_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// For a kernel whose wait is not its first instruction: the pointer through which it reads the previous kernel's
// output, to be taken after the wait.  A load through a const __restrict__ kernel parameter is a read-only load to
// the compiler, one it may start early, above the wait; through the pointer this returns it is an ordinary load
// that follows the wait.
template <typename P>
__device__ __forceinline__ P* ng_after_wait(P* ptr) {
    asm volatile("" : "+l"(ptr) :: "memory");
    return ptr;
}

#include <cstdlib>
#include <cstring>
static inline int ng_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("NEUROGRID_B200_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on;
}

template <typename... KP, typename... A>
static inline void ng_launch(void (*kernel)(KP...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, A... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr;
    memset(&attr, 0, sizeof(attr));
    attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = ng_pdl_enabled() ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, KP(args)...);
}
#define NG_LAUNCH(kernel, grid, block, smem, stream, ...) ng_launch((kernel), dim3(grid), dim3(block), (smem), (stream), __VA_ARGS__)

static inline int ng_launch_status() {
    return cudaGetLastError() == cudaSuccess ? NG_OK : NG_LAUNCH_FAILED;
}

// Embedding gather, residual-add + RMSNorm, SwiGLU gate: the memory-bound row kernels.
//
// Reference counterparts (plain one-thread-per-element kernels): gather
// gpu/cuda/kernels.cu:669-708, RMSNorm gpu/cuda/bf16_utils.cu:57-116, fused add+norm (fp16
// only) gpu/cuda/kernels.cu:196-262, SiLU and multiply gpu/cuda/bf16_utils.cu:122-213.
// Here the residual stream is float32 in both compute dtypes; the residual add, the sum of
// squares and the scaling are done in float32 and only the GEMM operand is rounded.
#include "ng_common.cuh"

// ---------------------------------------------------------------------------------- embed
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                             float* __restrict__ out, int H, int V, int* __restrict__ status) {
    const int row = blockIdx.x;
    int tok = tokens[row];
    const bool bad = tok < 0 || tok >= V;
    if (bad) {
        if (threadIdx.x == 0) atomicOr(status, NG_STATUS_BAD_TOKEN);
        tok = 0;
    }
    const T* src = table + (size_t)tok * H;
    float* dst = out + (size_t)row * H;
    for (int j = threadIdx.x; j < H; j += blockDim.x) dst[j] = bad ? 0.f : ng_ld(src + j);
}

NG_EXPORT int ng_embed(const void* table, int table_bf16, const int* tokens, float* out, int n_rows,
                       int H, int V, int* status, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (H <= 0 || V <= 0) return NG_BAD_SIZE;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_bf16)
        embed_kernel<<<n_rows, threads, 0, stream>>>((const __nv_bfloat16*)table, tokens, out, H, V, status);
    else
        embed_kernel<<<n_rows, threads, 0, stream>>>((const float*)table, tokens, out, H, V, status);
    return ng_launch_status();
}

// ---------------------------------------------------------------------------------- add + rmsnorm
// One block per output row i.  src row = rows ? rows[i] : i.
//   if delta: h[src] += delta[src] (float32 sum, written back)      -- the residual sum
//   out[i] = h[src] * rsqrt(mean(h[src]^2) + eps) * w                -- rounded to TO once
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const TD* __restrict__ delta,
                                   const float* __restrict__ w, TO* __restrict__ out,
                                   const int* __restrict__ rows, int H, float eps) {
    __shared__ float red[32];
    const int i = blockIdx.x;
    const int src = rows ? rows[i] : i;
    float* hr = h + (size_t)src * H;
    float ss = 0.f;
    if (delta) {
        const TD* dr = delta + (size_t)src * H;
        for (int j = threadIdx.x; j < H; j += blockDim.x) {
            const float v = hr[j] + ng_ld(dr + j);
            hr[j] = v;
            ss += v * v;
        }
    } else {
        for (int j = threadIdx.x; j < H; j += blockDim.x) {
            const float v = hr[j];
            ss += v * v;
        }
    }
    ss = ng_block_sum(ss, red);
    const float r = rsqrtf(ss / (float)H + eps);
    TO* orow = out + (size_t)i * H;
    // each thread re-reads exactly the elements it wrote itself
    for (int j = threadIdx.x; j < H; j += blockDim.x) ng_st(orow + j, hr[j] * r * w[j]);
}

NG_EXPORT int ng_add_rmsnorm(float* h, const void* delta, const float* w, void* out, const int* rows,
                             int n_out, int H, float eps, int act_bf16, cudaStream_t stream) {
    if (n_out <= 0) return NG_OK;
    if (H <= 0) return NG_BAD_SIZE;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (act_bf16)
        add_rmsnorm_kernel<<<n_out, threads, 0, stream>>>(h, (const __nv_bfloat16*)delta, w,
                                                         (__nv_bfloat16*)out, rows, H, eps);
    else
        add_rmsnorm_kernel<<<n_out, threads, 0, stream>>>(h, (const float*)delta, w, (float*)out, rows, H, eps);
    return ng_launch_status();
}

// h[row] += delta[row] only (the last residual sum of a model whose output is not normed here)
template <typename TD>
__global__ void add_kernel(float* __restrict__ h, const TD* __restrict__ delta, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) h[i] += ng_ld(delta + i);
}

NG_EXPORT int ng_residual_add(float* h, const void* delta, long long n, int act_bf16, cudaStream_t stream) {
    if (n <= 0) return NG_OK;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (act_bf16) add_kernel<<<blocks, 256, 0, stream>>>(h, (const __nv_bfloat16*)delta, (size_t)n);
    else add_kernel<<<blocks, 256, 0, stream>>>(h, (const float*)delta, (size_t)n);
    return ng_launch_status();
}

// ---------------------------------------------------------------------------------- swiglu
// gu is [n_rows, 2*I]: gate = gu[:, :I], up = gu[:, I:];  out = silu(gate) * up, float32 math.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I) {
    const size_t row = blockIdx.x;
    const int j = blockIdx.y * blockDim.x + threadIdx.x;
    if (j >= I) return;
    const float g = ng_ld(gu + row * 2 * (size_t)I + j);
    const float u = ng_ld(gu + row * 2 * (size_t)I + I + j);
    const float s = g / (1.f + expf(-g));
    ng_st(out + row * (size_t)I + j, s * u);
}

NG_EXPORT int ng_swiglu(const void* gu, void* out, int n_rows, int I, int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (I <= 0 || (I + 255) / 256 > 65535) return NG_BAD_SIZE;
    dim3 grid(n_rows, (I + 255) / 256);
    if (act_bf16) swiglu_kernel<<<grid, 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, I);
    else swiglu_kernel<<<grid, 256, 0, stream>>>((const float*)gu, (float*)out, I);
    return ng_launch_status();
}

// Paged attention for any query length, head size and dtype: the plain, order-fixed kernel.
//
// One warp owns one (query row, head) and walks the visible keys lo..pos in ascending order
// with an online softmax, so the result for a token does not depend on how the request was
// cut into steps or on what else is in the batch.  It is the whole float32 path and the
// in-GPU check for the tensor-core kernels of the bfloat16 path.
//
// Reference: gpu/cuda/paged_attention.cu:278-387 (decode, one block per head, all scores in
// shared memory, context <= 4096) and gpu/cuda/attention.cu:369-500 (prefill, materialised
// [heads, S, S] scores, K/V expanded to all query heads).  Both use scale 1/sqrt(hd), mask
// key > query, query head h reads KV head h / (nH / nKV).  `slopes` (one float per query head, or
// null) adds a position term to the scores: -slope[h] * (query position - key position).
#include "ng_common.cuh"

#define AG_WARPS 4
#define AG_MAX_J 8      // head_dim <= 256

template <typename T>
__global__ void __launch_bounds__(AG_WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                         const int* __restrict__ table, int table_stride, const int* __restrict__ positions,
                         const int* __restrict__ row_entry, T* __restrict__ out, int nH, int nKV, int hd,
                         int page_size, int num_pages, int window, float scale, const float* __restrict__ slopes) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31;
    const int head = blockIdx.y * AG_WARPS + (threadIdx.x >> 5);
    if (head >= nH) return;
    T* o = out + ((size_t)row * nH + head) * hd;
    const int entry = row_entry[row];
    if (entry < 0) {
        for (int j = lane; j < hd; j += 32) ng_st(o + j, 0.f);
        return;
    }
    const int pos = positions[row];
    const int kvh = head / (nH / nKV);
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const float slope = slopes ? slopes[head] : 0.f;          // score bias: -slope * (query position - key position)
    const T* qr = q + ((size_t)row * nH + head) * hd;
    float qv[AG_MAX_J], acc[AG_MAX_J];
#pragma unroll
    for (int j = 0; j < AG_MAX_J; ++j) {
        const int d = lane + 32 * j;
        qv[j] = d < hd ? ng_ld(qr + d) * scale : 0.f;
        acc[j] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int* trow = table + (size_t)entry * table_stride;
    for (int kp = lo; kp <= pos; ++kp) {
        const int page = trow[kp / page_size];
        if (page < 0 || page >= num_pages) continue;
        const size_t base = (((size_t)page * nKV + kvh) * page_size + (kp % page_size)) * hd;
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < AG_MAX_J; ++j) {
            const int d = lane + 32 * j;
            if (d < hd) dot = fmaf(qv[j], ng_ld(k_pages + base + d), dot);
        }
        const float s = ng_warp_sum(dot) - slope * (float)(pos - kp);
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);
        const float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int j = 0; j < AG_MAX_J; ++j) {
            const int d = lane + 32 * j;
            if (d < hd) acc[j] = acc[j] * corr + p * ng_ld(v_pages + base + d);
        }
        m = m_new;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int j = 0; j < AG_MAX_J; ++j) {
        const int d = lane + 32 * j;
        if (d < hd) ng_st(o + d, acc[j] * inv);
    }
}

NG_EXPORT int ng_attention_generic(const void* q, const void* k_pages, const void* v_pages, const int* table,
                                   int table_stride, const int* positions, const int* row_entry, void* out,
                                   int n_rows, int nH, int nKV, int hd, int page_size, int num_pages, int window,
                                   float scale, const float* slopes, int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (hd <= 0 || hd > 32 * AG_MAX_J || nH <= 0 || nKV <= 0 || nH % nKV || page_size <= 0) return NG_BAD_SIZE;
    dim3 grid(n_rows, (nH + AG_WARPS - 1) / AG_WARPS);
    if (act_bf16)
        NG_LAUNCH((attention_generic_kernel<__nv_bfloat16>), grid, AG_WARPS * 32, 0, stream, 
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages, table,
            table_stride, positions, row_entry, (__nv_bfloat16*)out, nH, nKV, hd, page_size, num_pages, window, scale, slopes);
    else
        NG_LAUNCH((attention_generic_kernel<float>), grid, AG_WARPS * 32, 0, stream, 
            (const float*)q, (const float*)k_pages, (const float*)v_pages, table, table_stride, positions,
            row_entry, (float*)out, nH, nKV, hd, page_size, num_pages, window, scale, slopes);
    return ng_launch_status();
}

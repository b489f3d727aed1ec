// Per-head RMSNorm of q and k, position encoding, and the write of k and v into cache pages:
// one pass over the fused q|k|v projection of a ragged batch.
//
// Order as in the reference's attention block (gpu/engine/layer.cu:1665-1707): per-head norm
// over head_dim with one weight vector shared by the heads (layer.cu:1323-1366), then the
// rotation (gpu/cuda/bf16_utils.cu:330-378: angle = pos * theta^(-2i/hd), pairs (2i,2i+1) or
// (i, i+hd/2)), then the cache write at block_table[pos / page] slot pos % page
// (gpu/cuda/paged_attention.cu:81-114).  The reference needs three dtype conversions and one
// cache-write launch per token around these; here it is one launch for all rows.
// Sums, rsqrt, angles and sin/cos are float32 (no fast-math); inv_freq comes from the host.
#include "ng_common.cuh"

#define RC_THREADS 128
#define RC_MAX_PAIRS 4   // head_dim <= 256

template <typename TI, typename T>
__global__ void __launch_bounds__(RC_THREADS)
rope_cache_kernel(const TI* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ qw,
                  const float* __restrict__ kw, const float* __restrict__ inv_freq, int half_pairing,
                  float pos_scale, T* __restrict__ k_pages, T* __restrict__ v_pages,
                  const int* __restrict__ table, int table_stride, const int* __restrict__ positions,
                  const int* __restrict__ row_entry, int nH, int nKV, int hd, int page_size,
                  int num_pages, float eps, int* __restrict__ status, int n_part, size_t pstride) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = blockIdx.y * (RC_THREADS / 32) + (threadIdx.x >> 5);
    const int entry = row_entry[row];
    const int ld = (nH + 2 * nKV) * hd;
    const size_t in = (size_t)row * ld;                 // index of the row's first element in qkv
    T* qo = q_out + (size_t)row * nH * hd;
    if (entry < 0) {                                   // padding row: defined output, no cache write
        if (warp < nH)
            for (int j = lane; j < hd; j += 32) ng_st(qo + (size_t)warp * hd + j, 0.f);
        return;
    }
    const int pos = positions[row];
    size_t page_base = 0;
    bool page_ok = true;
    if (nKV > 0) {
        const int page = table[(size_t)entry * table_stride + pos / page_size];
        page_ok = page >= 0 && page < num_pages;
        if (!page_ok && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, NG_STATUS_BAD_PAGE);
        page_base = (size_t)(page_ok ? page : 0) * nKV * page_size * hd + (size_t)(pos % page_size) * hd;
    }
    const float pf = (float)pos / pos_scale;
    const int half = hd / 2;
    // the angles depend on the row and the pair only: once per warp, for every head it handles
    float sn[RC_MAX_PAIRS], cs[RC_MAX_PAIRS];
#pragma unroll
    for (int u = 0; u < RC_MAX_PAIRS; ++u) {
        const int i = lane + 32 * u;
        sn[u] = 0.f;
        cs[u] = 1.f;
        if (inv_freq && i < half) sincosf(pf * inv_freq[i], &sn[u], &cs[u]);
    }

    for (int head = warp; head < nH + 2 * nKV; head += gridDim.y * (RC_THREADS / 32)) {   // one head per warp
        const size_t src = in + (size_t)head * hd;
        if (head >= nH + nKV) {                        // v: plain copy into its page
            if (page_ok) {
                T* dst = v_pages + page_base + (size_t)(head - nH - nKV) * page_size * hd;
                for (int j = lane; j < hd; j += 32) ng_st(dst + j, ng_ld_sum<T>(qkv, src + j, n_part, pstride));
            }
            continue;
        }
        const bool is_q = head < nH;
        const float* w = is_q ? qw : kw;
        float x1[RC_MAX_PAIRS], x2[RC_MAX_PAIRS];
        float ss = 0.f;
#pragma unroll
        for (int u = 0; u < RC_MAX_PAIRS; ++u) {
            const int i = lane + 32 * u;
            x1[u] = x2[u] = 0.f;
            if (i < half) {
                const int a = half_pairing ? i : 2 * i, b = half_pairing ? i + half : 2 * i + 1;
                x1[u] = ng_ld_sum<T>(qkv, src + a, n_part, pstride);
                x2[u] = ng_ld_sum<T>(qkv, src + b, n_part, pstride);
                ss += x1[u] * x1[u] + x2[u] * x2[u];
            }
        }
        float r = 1.f;
        if (w) {
            ss = ng_warp_sum(ss);
            r = rsqrtf(ss / (float)hd + eps);
        }
        T* dst = is_q ? qo + (size_t)head * hd
                      : k_pages + page_base + (size_t)(head - nH) * page_size * hd;
        if (!is_q && !page_ok) continue;
#pragma unroll
        for (int u = 0; u < RC_MAX_PAIRS; ++u) {
            const int i = lane + 32 * u;
            if (i < half) {
                const int a = half_pairing ? i : 2 * i, b = half_pairing ? i + half : 2 * i + 1;
                float y1 = x1[u], y2 = x2[u];
                if (w) { y1 = y1 * r * w[a]; y2 = y2 * r * w[b]; }
                if (inv_freq) {
                    const float z1 = y1 * cs[u] - y2 * sn[u], z2 = y1 * sn[u] + y2 * cs[u];
                    y1 = z1; y2 = z2;
                }
                ng_st(dst + a, y1);
                ng_st(dst + b, y2);
            }
        }
    }
}

NG_EXPORT int ng_rope_cache(const void* qkv, void* q_out, const float* qw, const float* kw,
                            const float* inv_freq, int half_pairing, float pos_scale, void* k_pages,
                            void* v_pages, const int* table, int table_stride, const int* positions,
                            const int* row_entry, int n_rows, int nH, int nKV, int hd, int page_size,
                            int num_pages, float eps, int* status, int act_bf16, int n_partials,
                            long long partial_stride, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (hd % 2 || hd > 64 * RC_MAX_PAIRS || hd <= 0 || nH <= 0 || nKV < 0 || page_size <= 0) return NG_BAD_SIZE;
    // few rows: one head per warp, for parallelism; many rows: a few blocks per row, whose warps
    // walk the heads and reuse the row's sines and cosines
    const int per_head = ((nH + 2 * nKV) * 32 + RC_THREADS - 1) / RC_THREADS;
    dim3 grid(n_rows, n_rows >= 256 ? min(4, per_head) : per_head);
    if (grid.y > 65535) return NG_BAD_SIZE;
    typedef __nv_bfloat16 bf;
    const size_t ps = (size_t)partial_stride;
#define RC_ARGS(TIN, TT) (const TIN*)qkv, (TT*)q_out, qw, kw, inv_freq, half_pairing, pos_scale, (TT*)k_pages, \
        (TT*)v_pages, table, table_stride, positions, row_entry, nH, nKV, hd, page_size, num_pages, eps, status
    if (act_bf16 && n_partials > 1)
        NG_LAUNCH((rope_cache_kernel<float, bf>), grid, RC_THREADS, 0, stream, RC_ARGS(float, bf), n_partials, ps);
    else if (act_bf16)
        NG_LAUNCH((rope_cache_kernel<bf, bf>), grid, RC_THREADS, 0, stream, RC_ARGS(bf, bf), 1, 0);
    else
        NG_LAUNCH((rope_cache_kernel<float, float>), grid, RC_THREADS, 0, stream, RC_ARGS(float, float), n_partials, ps);
#undef RC_ARGS
    return ng_launch_status();
}

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
// Pairs of a head that one lane handles: 1 (head_dim <= 64), 2 (<= 128) or 4 (<= 256).  The library
// is specialised on it (-DNG_ROPE_PAIRS), so a model compiles the one it needs.
#ifndef NG_ROPE_PAIRS
#error "compile with -DNG_ROPE_PAIRS=<1, 2 or 4>"
#endif
static_assert(NG_ROPE_PAIRS == 1 || NG_ROPE_PAIRS == 2 || NG_ROPE_PAIRS == 4, "pairs per lane: 1, 2 or 4");

// one pair (a, b) of a head, summed over the partial stacks (in ascending order, then rounded to
// TO, as ng_ld_sum does); adjacent pairs take one wide load
__device__ __forceinline__ float2 rc_ld2(const __nv_bfloat16* q) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q));
}
__device__ __forceinline__ float2 rc_ld2(const float* q) { return *reinterpret_cast<const float2*>(q); }
template <typename TO, typename TI>
__device__ __forceinline__ void rc_load_pair(const TI* __restrict__ qkv, size_t ia, size_t ib, bool adjacent, int n_part,
                                             size_t pstride, float& x1, float& x2) {
    if (!adjacent) {
        x1 = ng_ld_sum<TO>(qkv, ia, n_part, pstride);
        x2 = ng_ld_sum<TO>(qkv, ib, n_part, pstride);
        return;
    }
    float2 f = rc_ld2(qkv + ia);
    if (n_part > 1) {
        f.x += 0.f; f.y += 0.f;
        for (int s = 1; s < n_part; ++s) {
            const float2 g = rc_ld2(qkv + ia + (size_t)s * pstride);
            f.x += g.x; f.y += g.y;
        }
        TO r1, r2;
        ng_st(&r1, f.x); ng_st(&r2, f.y);
        f.x = ng_ld(&r1); f.y = ng_ld(&r2);
    }
    x1 = f.x; x2 = f.y;
}
__device__ __forceinline__ void rc_store_pair(__nv_bfloat16* dst, int a, int b, bool adjacent, float y1, float y2) {
    if (adjacent) *reinterpret_cast<__nv_bfloat162*>(dst + a) = __floats2bfloat162_rn(y1, y2);
    else { dst[a] = __float2bfloat16(y1); dst[b] = __float2bfloat16(y2); }
}
__device__ __forceinline__ void rc_store_pair(float* dst, int a, int b, bool adjacent, float y1, float y2) {
    if (adjacent) *reinterpret_cast<float2*>(dst + a) = make_float2(y1, y2);
    else { dst[a] = y1; dst[b] = y2; }
}

// HB heads per warp and pass: their loads are all issued before the first is used.  With few
// rows HB = 1 and a warp per head (parallelism); with many, HB = 4 (loads in flight).
// ``wide``: pairs are adjacent and every row and page is aligned for two-element accesses.
template <typename TI, typename T, int HB, int PAIRS>
__global__ void __launch_bounds__(RC_THREADS)
rope_cache_kernel(const TI* __restrict__ qkv, T* __restrict__ q_out, const float* __restrict__ qw,
                  const float* __restrict__ kw, const float* __restrict__ inv_freq, int half_pairing,
                  float pos_scale, T* __restrict__ k_pages, T* __restrict__ v_pages,
                  const int* __restrict__ table, int table_stride, const int* __restrict__ positions,
                  const int* __restrict__ row_entry, int nH, int nKV, int hd, int page_size,
                  int num_pages, float eps, int* __restrict__ status, int n_part, size_t pstride, int wide) {
    ng_pdl_trigger();
    // What does not depend on the product in front of this kernel comes before the wait for it: the row's entry,
    // position and page (the step's batch description, written before its first kernel) and the angles.
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = blockIdx.y * (RC_THREADS / 32) + (threadIdx.x >> 5);
    const int n_warps = gridDim.y * (RC_THREADS / 32);
    const int entry = row_entry[row];
    const int pos = positions[row];
    const int n_all = nH + 2 * nKV;
    const int ld = n_all * hd;
    const size_t in = (size_t)row * ld;                 // index of the row's first element in qkv
    T* qo = q_out + (size_t)row * nH * hd;
    if (entry < 0) {                                   // padding row: defined output, no cache write
        ng_pdl_wait();
        for (int head = warp; head < nH; head += n_warps)
            for (int j = lane; j < hd; j += 32) ng_st(qo + (size_t)head * hd + j, 0.f);
        return;
    }
    size_t page_base = 0;
    bool page_ok = true;
    if (nKV > 0) {
        const int page = table[(size_t)entry * table_stride + pos / page_size];
        page_ok = page >= 0 && page < num_pages;
        page_base = (size_t)(page_ok ? page : 0) * nKV * page_size * hd + (size_t)(pos % page_size) * hd;
    }
    const float pf = (float)pos / pos_scale;
    const int half = hd / 2;
    const bool adjacent = wide != 0;
    // the angles depend on the row and the pair only: once per warp, for every head it handles
    float sn[PAIRS], cs[PAIRS];
#pragma unroll
    for (int u = 0; u < PAIRS; ++u) {
        const int i = lane + 32 * u;
        sn[u] = 0.f;
        cs[u] = 1.f;
        if (inv_freq && i < half) sincosf(pf * inv_freq[i], &sn[u], &cs[u]);
    }
    ng_pdl_wait();
    qkv = ng_after_wait(qkv);
    if (!page_ok && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, NG_STATUS_BAD_PAGE);

    for (int h0 = warp * HB; h0 < n_all; h0 += n_warps * HB) {
        float x1[HB][PAIRS], x2[HB][PAIRS];
#pragma unroll
        for (int hb = 0; hb < HB; ++hb) {
            const size_t src = in + (size_t)min(h0 + hb, n_all - 1) * hd;
#pragma unroll
            for (int u = 0; u < PAIRS; ++u) {
                const int i = lane + 32 * u;
                // unconditional (indices clamped into the row), so that all loads are in flight together
                const int ic = min(i, half - 1);
                const int a = half_pairing ? ic : 2 * ic, b = half_pairing ? ic + half : 2 * ic + 1;
                rc_load_pair<T>(qkv, src + a, src + b, adjacent, n_part, pstride, x1[hb][u], x2[hb][u]);
                if (i >= half) x1[hb][u] = x2[hb][u] = 0.f;
            }
        }
#pragma unroll
        for (int hb = 0; hb < HB; ++hb) {
            const int head = h0 + hb;
            if (head >= n_all) break;
            const bool is_q = head < nH, is_v = head >= nH + nKV;
            if (!is_q && !page_ok) continue;
            const float* w = is_v ? nullptr : (is_q ? qw : kw);
            float r = 1.f;
            if (w) {
                float ss = 0.f;
#pragma unroll
                for (int u = 0; u < PAIRS; ++u) ss += x1[hb][u] * x1[hb][u] + x2[hb][u] * x2[hb][u];
                ss = ng_warp_sum(ss);
                r = rsqrtf(ss / (float)hd + eps);
            }
            T* dst = is_q ? qo + (size_t)head * hd
                   : is_v ? v_pages + page_base + (size_t)(head - nH - nKV) * page_size * hd
                          : k_pages + page_base + (size_t)(head - nH) * page_size * hd;
#pragma unroll
            for (int u = 0; u < PAIRS; ++u) {
                const int i = lane + 32 * u;
                if (i < half) {
                    const int a = half_pairing ? i : 2 * i, b = half_pairing ? i + half : 2 * i + 1;
                    float y1 = x1[hb][u], y2 = x2[hb][u];
                    if (w) { y1 = y1 * r * w[a]; y2 = y2 * r * w[b]; }
                    if (inv_freq && !is_v) {
                        const float z1 = y1 * cs[u] - y2 * sn[u], z2 = y1 * sn[u] + y2 * cs[u];
                        y1 = z1; y2 = z2;
                    }
                    rc_store_pair(dst, a, b, adjacent, y1, y2);
                }
            }
        }
    }
}

// The common bulk case: bfloat16 in and out, no partial sums, head size 64, pairs (i, i + 32).  Half a warp
// owns a head: lane j of it holds pairs 2j and 2j+1, i.e. the elements 2j, 2j+1 (one 4-byte access) and
// 32+2j, 33+2j (another).  A warp walks head pairs with the loads of RCH_UNROLL of them in flight.
#define RCH_UNROLL 3
__global__ void __launch_bounds__(RC_THREADS)
rope_cache_half64_kernel(const __nv_bfloat16* __restrict__ qkv, __nv_bfloat16* __restrict__ q_out,
                         const float* __restrict__ qw, const float* __restrict__ kw, const float* __restrict__ inv_freq,
                         float pos_scale, __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                         const int* __restrict__ table, int table_stride, const int* __restrict__ positions,
                         const int* __restrict__ row_entry, int nH, int nKV, int page_size, int num_pages, float eps,
                         int* __restrict__ status) {
    constexpr int hd = 64, half = 32;
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.x;
    const int lane = threadIdx.x & 31, sub = lane >> 4, j = lane & 15;
    const int warp = blockIdx.y * (RC_THREADS / 32) + (threadIdx.x >> 5), n_warps = gridDim.y * (RC_THREADS / 32);
    const int entry = row_entry[row];
    const int pos = positions[row];
    const int n_all = nH + 2 * nKV;
    const __nv_bfloat16* in = qkv + (size_t)row * n_all * hd;
    __nv_bfloat16* qo = q_out + (size_t)row * nH * hd;
    if (entry < 0) {                                   // padding row: defined output, no cache write
        for (int head = 2 * warp + sub; head < nH; head += 2 * n_warps)
            *reinterpret_cast<uint2*>(qo + (size_t)head * hd + 4 * j) = make_uint2(0u, 0u);   // 16 lanes x 4 elements
        return;
    }
    size_t page_base = 0;
    bool page_ok = true;
    if (nKV > 0) {
        const int page = table[(size_t)entry * table_stride + pos / page_size];
        page_ok = page >= 0 && page < num_pages;
        if (!page_ok && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, NG_STATUS_BAD_PAGE);
        page_base = (size_t)(page_ok ? page : 0) * nKV * page_size * hd + (size_t)(pos % page_size) * hd;
    }
    const float pf = (float)pos / pos_scale;
    float sn0 = 0.f, cs0 = 1.f, sn1 = 0.f, cs1 = 1.f;
    if (inv_freq) {
        sincosf(pf * inv_freq[2 * j], &sn0, &cs0);
        sincosf(pf * inv_freq[2 * j + 1], &sn1, &cs1);
    }
    const float2 qw_a = qw ? make_float2(qw[2 * j], qw[2 * j + 1]) : make_float2(1.f, 1.f);
    const float2 qw_b = qw ? make_float2(qw[half + 2 * j], qw[half + 2 * j + 1]) : make_float2(1.f, 1.f);
    const float2 kw_a = kw ? make_float2(kw[2 * j], kw[2 * j + 1]) : make_float2(1.f, 1.f);
    const float2 kw_b = kw ? make_float2(kw[half + 2 * j], kw[half + 2 * j + 1]) : make_float2(1.f, 1.f);
    // both halves of a warp walk together (the sums below are shuffles of the whole warp): the loop runs over head pairs
    for (int p0 = warp; 2 * p0 < n_all; p0 += n_warps * RCH_UNROLL) {
        const int h0 = 2 * p0 + sub;
        float2 xa[RCH_UNROLL], xb[RCH_UNROLL];
#pragma unroll
        for (int u = 0; u < RCH_UNROLL; ++u) {
            const int head = min(h0 + 2 * n_warps * u, n_all - 1);       // clamped: every load is issued before the first use
            xa[u] = rc_ld2(in + (size_t)head * hd + 2 * j);
            xb[u] = rc_ld2(in + (size_t)head * hd + half + 2 * j);
        }
#pragma unroll
        for (int u = 0; u < RCH_UNROLL; ++u) {
            const int head = h0 + 2 * n_warps * u;
            // every lane of the half-warp takes part in the sum below, also for a head beyond the last
            const bool live = head < n_all;
            const bool is_q = head < nH, is_v = head >= nH + nKV;
            const bool normed = !is_v && (is_q ? qw != nullptr : kw != nullptr);
            float ss = xa[u].x * xa[u].x + xa[u].y * xa[u].y + xb[u].x * xb[u].x + xb[u].y * xb[u].y;
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (!live || (!is_q && !page_ok)) continue;
            float2 a = xa[u], b = xb[u];
            if (normed) {
                const float r = rsqrtf(ss / (float)hd + eps);
                const float2 wa = is_q ? qw_a : kw_a, wb = is_q ? qw_b : kw_b;
                a.x = a.x * r * wa.x; a.y = a.y * r * wa.y;
                b.x = b.x * r * wb.x; b.y = b.y * r * wb.y;
            }
            if (inv_freq && !is_v) {
                const float a0 = a.x * cs0 - b.x * sn0, b0 = a.x * sn0 + b.x * cs0;
                const float a1 = a.y * cs1 - b.y * sn1, b1 = a.y * sn1 + b.y * cs1;
                a = make_float2(a0, a1);
                b = make_float2(b0, b1);
            }
            __nv_bfloat16* dst = is_q ? qo + (size_t)head * hd
                               : is_v ? v_pages + page_base + (size_t)(head - nH - nKV) * page_size * hd
                                      : k_pages + page_base + (size_t)(head - nH) * page_size * hd;
            *reinterpret_cast<__nv_bfloat162*>(dst + 2 * j) = __floats2bfloat162_rn(a.x, a.y);
            *reinterpret_cast<__nv_bfloat162*>(dst + half + 2 * j) = __floats2bfloat162_rn(b.x, b.y);
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
    if (hd % 2 || hd > 64 * NG_ROPE_PAIRS || hd <= 0 || nH <= 0 || nKV < 0 || page_size <= 0) return NG_BAD_SIZE;
    // few rows: one head per warp, for parallelism; many rows: four heads per warp and pass,
    // whose loads are in flight together, the row's sines and cosines shared by them
    const int n_all = nH + 2 * nKV;
    const bool bulk = n_rows >= 256;
    const int warps = bulk ? (n_all + 3) / 4 : n_all;
    dim3 grid(n_rows, (warps * 32 + RC_THREADS - 1) / RC_THREADS);
    if (grid.y > 65535) return NG_BAD_SIZE;
    typedef __nv_bfloat16 bf;
    const size_t ps = (size_t)partial_stride;
    if (act_bf16 && n_partials <= 1 && half_pairing && hd == 64 && n_rows >= 64 && ((uintptr_t)qkv & 3) == 0 &&
        ((uintptr_t)q_out & 3) == 0 && ((uintptr_t)k_pages & 3) == 0 && ((uintptr_t)v_pages & 3) == 0) {
        const int pairs = (n_all + 1) / 2;                       // half a warp per head
        dim3 g(n_rows, (((pairs + RCH_UNROLL - 1) / RCH_UNROLL) * 32 + RC_THREADS - 1) / RC_THREADS);
        NG_LAUNCH((rope_cache_half64_kernel), g, RC_THREADS, 0, stream, (const bf*)qkv, (bf*)q_out, qw, kw, inv_freq,
                  pos_scale, (bf*)k_pages, (bf*)v_pages, table, table_stride, positions, row_entry, nH, nKV, page_size,
                  num_pages, eps, status);
        return ng_launch_status();
    }
    // two-element accesses: adjacent pairs, every buffer aligned for them (head sizes are even)
    const size_t in_align = (act_bf16 && n_partials <= 1) ? 3 : 7, out_align = act_bf16 ? 3 : 7;
    const int wide = !half_pairing && ((uintptr_t)qkv & in_align) == 0 && ((uintptr_t)q_out & out_align) == 0 &&
                     ((uintptr_t)k_pages & out_align) == 0 && ((uintptr_t)v_pages & out_align) == 0 &&
                     (n_partials <= 1 || (partial_stride % 2) == 0);
#define RC_ARGS(TIN, TT) (const TIN*)qkv, (TT*)q_out, qw, kw, inv_freq, half_pairing, pos_scale, (TT*)k_pages, \
        (TT*)v_pages, table, table_stride, positions, row_entry, nH, nKV, hd, page_size, num_pages, eps, status
#define RC_GO2(TIN, TT, NP, PS, PAIRS) \
    do { if (bulk) NG_LAUNCH((rope_cache_kernel<TIN, TT, 4, PAIRS>), grid, RC_THREADS, 0, stream, RC_ARGS(TIN, TT), NP, PS, wide); \
         else NG_LAUNCH((rope_cache_kernel<TIN, TT, 1, PAIRS>), grid, RC_THREADS, 0, stream, RC_ARGS(TIN, TT), NP, PS, wide); } while (0)
#define RC_GO(TIN, TT, NP, PS) RC_GO2(TIN, TT, NP, PS, NG_ROPE_PAIRS)
    if (act_bf16 && n_partials > 1) RC_GO(float, bf, n_partials, ps);
    else if (act_bf16) RC_GO(bf, bf, 1, 0);
    else RC_GO(float, float, n_partials, ps);
#undef RC_GO
#undef RC_GO2
#undef RC_ARGS
    return ng_launch_status();
}

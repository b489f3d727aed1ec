// Gated short convolution over a ragged batch, prefill portions and decode tokens alike.
//
//   p = [B | C | x]  (row-major [n_rows, 3H], the in_proj output)      u[t] = B[t] * x[t]
//   c[t] = bias + sum_{k<L} w[d,k] * u[t-(L-1)+k]     (tap L-1 multiplies the current token)
//   out[t] = C[t] * c[t]
// u before the first row of a portion comes from the request's state slot (the last L-1
// values of u, float32), u before position 0 is zero whatever the slot holds.  After the
// portion the slot holds the last L-1 values of u again.
//
// The reference computes the same with separate kernels and layout transposes
// (gpu/engine/conv_layer.cu:222-250, gpu/cuda/conv.cu:34-105 for a whole sequence from zero
// state, conv.cu:118-174 for one token) and cannot continue a sequence kernel from a state.
//
// The library is specialised on the conv width (-DNG_CONV_L), so a model compiles its own.
// Grid: (channel blocks, token tiles, entries).  A thread owns one channel of one tile and
// walks its tokens in order with the last L-1 inputs in registers.  Only tile 0 of an entry
// reads the slot, and only tile 0 writes it (after all its reads), so no other block of the
// launch touches a slot while it is read.
#include "ng_common.cuh"

#define CONV_MAX_L 8
#ifndef NG_CONV_L
#error "compile with -DNG_CONV_L=<conv width, 2..8>"
#endif
static_assert(NG_CONV_L >= 2 && NG_CONV_L <= CONV_MAX_L, "conv width must be in [2, 8]");
#define CONV_TILE 32
#define CONV_THREADS 128

template <typename TI, typename T, int L>
__global__ void __launch_bounds__(CONV_THREADS)
shortconv_kernel(const TI* __restrict__ p, const float* __restrict__ w, const float* __restrict__ bias,
                 float* __restrict__ state, T* __restrict__ out, const int* __restrict__ cu_q,
                 const int* __restrict__ ctx_before, const int* __restrict__ slots, int H, int n_part, size_t pstride,
                 int tile) {
    ng_pdl_trigger();
    // The batch description, the taps and the slot (written by the step before) do not depend on the product in
    // front of this kernel: they are read before the wait for it.  A block or thread with nothing to do waits too.
    const int e = blockIdx.z;
    const int q0 = cu_q[e];
    const int qlen = cu_q[e + 1] - q0;
    const int t0 = blockIdx.y * tile;
    const int d = blockIdx.x * CONV_THREADS + threadIdx.x;
    if (t0 >= qlen || d >= H) {
        ng_pdl_wait();
        return;
    }
    const int ctx = ctx_before[e];
    float* st = state + (size_t)slots[e] * (L - 1) * H + d;      // st[j*H]: u at position ctx-(L-1)+j
    const size_t ld = 3 * (size_t)H;
    const size_t iB = (size_t)q0 * ld + d, iC = iB + H, iX = iB + 2 * (size_t)H;   // B, C, x of chunk row 0
#define LDP(base, t) ng_ld_sum<T>(p, (base) + (size_t)(t) * ld, n_part, pstride)

    float wk[L], hist[L - 1], old[L - 1];
#pragma unroll
    for (int k = 0; k < L; ++k) wk[k] = w[(size_t)d * L + k];
    const float b = bias ? bias[d] : 0.f;

    const bool first_tile = (t0 == 0);
    if (first_tile) {
#pragma unroll
        for (int j = 0; j < L - 1; ++j) old[j] = (ctx - (L - 1) + j >= 0) ? st[(size_t)j * H] : 0.f;
    } else {
#pragma unroll
        for (int j = 0; j < L - 1; ++j) old[j] = 0.f;
    }
    ng_pdl_wait();
    p = ng_after_wait(p);
    // hist[j] = u at chunk index t0-(L-1)+j
#pragma unroll
    for (int j = 0; j < L - 1; ++j) {
        const int ti = t0 - (L - 1) + j;
        if (ti >= 0) hist[j] = LDP(iB, ti) * LDP(iX, ti);
        else hist[j] = old[j];                                     // only reached when t0 == 0
    }
    const int t1 = min(t0 + tile, qlen);
#pragma unroll 4
    for (int t = t0; t < t1; ++t) {
        const float u = LDP(iB, t) * LDP(iX, t);
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < L - 1; ++k) acc = fmaf(wk[k], hist[k], acc);
        acc = fmaf(wk[L - 1], u, acc) + b;
        ng_st(out + (size_t)(q0 + t) * H + d, LDP(iC, t) * acc);
#pragma unroll
        for (int k = 0; k < L - 2; ++k) hist[k] = hist[k + 1];
        hist[L - 2] = u;
    }
    if (first_tile) {
        // new slot content: u at chunk indices qlen-(L-1)+j
#pragma unroll
        for (int j = 0; j < L - 1; ++j) {
            const int ti = qlen - (L - 1) + j;
            float v = 0.f;
            if (ti >= 0) {
                v = LDP(iB, ti) * LDP(iX, ti);
            } else {
#pragma unroll
                for (int i = 0; i < L - 1; ++i)
                    if (i == ti + (L - 1)) v = old[i];
            }
            st[(size_t)j * H] = v;
        }
    }
}

// The bulk case (bfloat16 in and out, no partial sums, even width): two channels per thread, so
// that every access is 4 bytes wide.  Same arithmetic and the same ownership of the slot.
template <int L>
__global__ void __launch_bounds__(CONV_THREADS)
shortconv_bf16x2_kernel(const __nv_bfloat16* __restrict__ p, const float* __restrict__ w, const float* __restrict__ bias,
                        float* __restrict__ state, __nv_bfloat16* __restrict__ out, const int* __restrict__ cu_q,
                        const int* __restrict__ ctx_before, const int* __restrict__ slots, int H) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int e = blockIdx.z;
    const int q0 = cu_q[e];
    const int qlen = cu_q[e + 1] - q0;
    const int t0 = blockIdx.y * CONV_TILE;
    if (t0 >= qlen) return;
    const int d = 2 * (blockIdx.x * CONV_THREADS + threadIdx.x);
    if (d >= H) return;
    const int ctx = ctx_before[e];
    float* st = state + (size_t)slots[e] * (L - 1) * H + d;
    const size_t ld = 3 * (size_t)H;
    const __nv_bfloat16* pB = p + (size_t)q0 * ld + d;
    const __nv_bfloat16* pC = pB + H;
    const __nv_bfloat16* pX = pB + 2 * (size_t)H;
    auto ld2 = [](const __nv_bfloat16* q) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(q)); };
    auto u_at = [&](int t) {
        const float2 b = ld2(pB + (size_t)t * ld), x = ld2(pX + (size_t)t * ld);
        return make_float2(b.x * x.x, b.y * x.y);
    };
    float2 wk[L], hist[L - 1], old[L - 1];
#pragma unroll
    for (int k = 0; k < L; ++k) wk[k] = make_float2(w[(size_t)d * L + k], w[(size_t)(d + 1) * L + k]);
    const float2 b = bias ? make_float2(bias[d], bias[d + 1]) : make_float2(0.f, 0.f);
    const bool first_tile = (t0 == 0);
#pragma unroll
    for (int j = 0; j < L - 1; ++j) {
        old[j] = make_float2(0.f, 0.f);
        if (first_tile && ctx - (L - 1) + j >= 0) old[j] = *reinterpret_cast<const float2*>(st + (size_t)j * H);
    }
#pragma unroll
    for (int j = 0; j < L - 1; ++j) {
        const int ti = t0 - (L - 1) + j;
        hist[j] = ti >= 0 ? u_at(ti) : old[j];
    }
    const int t1 = min(t0 + CONV_TILE, qlen);
#pragma unroll 4
    for (int t = t0; t < t1; ++t) {
        const float2 u = u_at(t);
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int k = 0; k < L - 1; ++k) { acc.x = fmaf(wk[k].x, hist[k].x, acc.x); acc.y = fmaf(wk[k].y, hist[k].y, acc.y); }
        acc.x = fmaf(wk[L - 1].x, u.x, acc.x) + b.x;
        acc.y = fmaf(wk[L - 1].y, u.y, acc.y) + b.y;
        const float2 c = ld2(pC + (size_t)t * ld);
        *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(q0 + t) * H + d) = __floats2bfloat162_rn(c.x * acc.x, c.y * acc.y);
#pragma unroll
        for (int k = 0; k < L - 2; ++k) hist[k] = hist[k + 1];
        hist[L - 2] = u;
    }
    if (first_tile) {
#pragma unroll
        for (int j = 0; j < L - 1; ++j) {
            const int ti = qlen - (L - 1) + j;
            float2 v = make_float2(0.f, 0.f);
            if (ti >= 0) {
                v = u_at(ti);
            } else {
#pragma unroll
                for (int i = 0; i < L - 1; ++i)
                    if (i == ti + (L - 1)) v = old[i];
            }
            *reinterpret_cast<float2*>(st + (size_t)j * H) = v;
        }
    }
}


// Long portions (bfloat16, no partial sums, width a multiple of 8): eight channels per thread
// with 16-byte accesses and tiles of 8 tokens, so that a launch has many independent loads in
// flight.  Same arithmetic and the same ownership of the slot.
#define CONV_TILE8 8
struct ng_f8 { float v[8]; };
__device__ __forceinline__ ng_f8 ld_bf16x8(const __nv_bfloat16* q) {
    const uint4 r = *reinterpret_cast<const uint4*>(q);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
    ng_f8 o;
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); o.v[2 * i] = f.x; o.v[2 * i + 1] = f.y; }
    return o;
}
template <int L>
__global__ void __launch_bounds__(CONV_THREADS)
shortconv_bf16x8_kernel(const __nv_bfloat16* __restrict__ p, const float* __restrict__ w, const float* __restrict__ bias,
                        float* __restrict__ state, __nv_bfloat16* __restrict__ out, const int* __restrict__ cu_q,
                        const int* __restrict__ ctx_before, const int* __restrict__ slots, int H) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int e = blockIdx.z;
    const int q0 = cu_q[e];
    const int qlen = cu_q[e + 1] - q0;
    const int t0 = blockIdx.y * CONV_TILE8;
    if (t0 >= qlen) return;
    const int d = 8 * (blockIdx.x * CONV_THREADS + threadIdx.x);
    if (d >= H) return;
    const int ctx = ctx_before[e];
    float* st = state + (size_t)slots[e] * (L - 1) * H + d;
    const size_t ld = 3 * (size_t)H;
    const __nv_bfloat16* pB = p + (size_t)q0 * ld + d;
    const __nv_bfloat16* pC = pB + H;
    const __nv_bfloat16* pX = pB + 2 * (size_t)H;
    const bool first_tile = (t0 == 0);
    const int t1 = min(t0 + CONV_TILE8, qlen);

    // u for chunk indices t0-(L-1) .. t1-1.  Every load is unconditional (its row clamped into the
    // portion) so that all of them are in flight together; what lies outside is replaced after.
    uint4 rb[CONV_TILE8 + L - 1], rx[CONV_TILE8 + L - 1], rc[CONV_TILE8];
#pragma unroll
    for (int j = 0; j < CONV_TILE8 + L - 1; ++j) {
        const int ti = min(max(t0 - (L - 1) + j, 0), qlen - 1);
        rb[j] = *reinterpret_cast<const uint4*>(pB + (size_t)ti * ld);
        rx[j] = *reinterpret_cast<const uint4*>(pX + (size_t)ti * ld);
    }
#pragma unroll
    for (int j = 0; j < CONV_TILE8; ++j)
        rc[j] = *reinterpret_cast<const uint4*>(pC + (size_t)min(t0 + j, qlen - 1) * ld);
    float wk[L][8], b8[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        b8[i] = bias ? bias[d + i] : 0.f;
#pragma unroll
        for (int k = 0; k < L; ++k) wk[k][i] = w[(size_t)(d + i) * L + k];
    }
    float u[CONV_TILE8 + L - 1][8];
#pragma unroll
    for (int j = 0; j < CONV_TILE8 + L - 1; ++j) {
        const int ti = t0 - (L - 1) + j;
        const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&rb[j]);
        const __nv_bfloat162* hx = reinterpret_cast<const __nv_bfloat162*>(&rx[j]);
        const bool in_portion = ti >= 0 && ti < t1;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 fb = __bfloat1622float2(hb[i]), fx = __bfloat1622float2(hx[i]);
            u[j][2 * i] = in_portion ? fb.x * fx.x : 0.f;
            u[j][2 * i + 1] = in_portion ? fb.y * fx.y : 0.f;
        }
    }
    if (first_tile) {                                                // rows before the portion: the slot, position ctx + ti
#pragma unroll
        for (int j = 0; j < L - 1; ++j) {
            const int ti = j - (L - 1);
            if (ctx + ti >= 0) {
                const float4 a = *reinterpret_cast<const float4*>(st + (size_t)j * H);
                const float4 c = *reinterpret_cast<const float4*>(st + (size_t)j * H + 4);
                u[j][0] = a.x; u[j][1] = a.y; u[j][2] = a.z; u[j][3] = a.w;
                u[j][4] = c.x; u[j][5] = c.y; u[j][6] = c.z; u[j][7] = c.w;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < CONV_TILE8; ++j) {
        const int t = t0 + j;
        const __nv_bfloat162* hc = reinterpret_cast<const __nv_bfloat162*>(&rc[j]);
        __nv_bfloat162 o[4];
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            float a0 = 0.f, a1 = 0.f;
#pragma unroll
            for (int k = 0; k < L - 1; ++k) { a0 = fmaf(wk[k][i], u[j + k][i], a0); a1 = fmaf(wk[k][i + 1], u[j + k][i + 1], a1); }
            a0 = fmaf(wk[L - 1][i], u[j + L - 1][i], a0) + b8[i];
            a1 = fmaf(wk[L - 1][i + 1], u[j + L - 1][i + 1], a1) + b8[i + 1];
            const float2 c = __bfloat1622float2(hc[i / 2]);
            o[i / 2] = __floats2bfloat162_rn(c.x * a0, c.y * a1);
        }
        if (t < t1) *reinterpret_cast<uint4*>(out + (size_t)(q0 + t) * H + d) = *reinterpret_cast<const uint4*>(o);
    }
    if (first_tile) {
        // new slot content: u at chunk indices qlen-(L-1)+j (read again: few loads, once per entry)
#pragma unroll
        for (int j = 0; j < L - 1; ++j) {
            const int ti = qlen - (L - 1) + j;
            float* dst = st + (size_t)j * H;
            if (ti < 0) {
                // still the old slot's value, from its index ti + L-1 = qlen + j > j: not yet overwritten
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f), c = a;
                if (ctx + ti >= 0) {
                    a = *reinterpret_cast<const float4*>(st + (size_t)(ti + L - 1) * H);
                    c = *reinterpret_cast<const float4*>(st + (size_t)(ti + L - 1) * H + 4);
                }
                *reinterpret_cast<float4*>(dst) = a;
                *reinterpret_cast<float4*>(dst + 4) = c;
            } else {
                const ng_f8 b = ld_bf16x8(pB + (size_t)ti * ld), x = ld_bf16x8(pX + (size_t)ti * ld);
                *reinterpret_cast<float4*>(dst) = make_float4(b.v[0] * x.v[0], b.v[1] * x.v[1], b.v[2] * x.v[2], b.v[3] * x.v[3]);
                *reinterpret_cast<float4*>(dst + 4) = make_float4(b.v[4] * x.v[4], b.v[5] * x.v[5], b.v[6] * x.v[6], b.v[7] * x.v[7]);
            }
        }
    }
}

template <typename TI, typename T, int L>
static void launch_conv(dim3 grid, cudaStream_t stream, const void* p, const float* w, const float* bias,
                        float* state, void* out, const int* cu_q, const int* ctx_before, const int* slots, int H,
                        int n_part, size_t pstride, int tile) {
    NG_LAUNCH((shortconv_kernel<TI, T, L>), grid, CONV_THREADS, 0, stream, (const TI*)p, w, bias, state, (T*)out, cu_q,
                                                                 ctx_before, slots, H, n_part, pstride, tile);
}

template <typename TI, typename T>
static void dispatch_conv(int L, dim3 grid, cudaStream_t stream, const void* p, const float* w, const float* bias,
                          float* state, void* out, const int* cu_q, const int* ctx_before, const int* slots, int H,
                          int n_part, size_t pstride, int tile) {
    launch_conv<TI, T, NG_CONV_L>(grid, stream, p, w, bias, state, out, cu_q, ctx_before, slots, H, n_part, pstride, tile);
}

// p: [n_rows, 3H] of the activation dtype, or (n_partials > 1) float32 partial sums
// [n_partials][n_rows, 3H] lying partial_stride elements apart.
NG_EXPORT int ng_shortconv(const void* p, const float* w, const float* bias, float* state, void* out,
                           const int* cu_q, const int* ctx_before, const int* slots, int n_entries,
                           int max_q, int H, int L, int act_bf16, int n_partials, long long partial_stride,
                           cudaStream_t stream) {
    if (n_entries <= 0 || max_q <= 0) return NG_OK;
    if (L != NG_CONV_L || H <= 0) return NG_BAD_SIZE;            // the library is built for one width
    dim3 grid((H + CONV_THREADS - 1) / CONV_THREADS, (max_q + CONV_TILE - 1) / CONV_TILE, n_entries);
    if (grid.y > 65535 || grid.z > 65535) return NG_BAD_SIZE;
    const size_t ps = (size_t)partial_stride;
    if (act_bf16 && n_partials <= 1 && H % 8 == 0 && max_q >= 64 && ((uintptr_t)p & 15) == 0 && ((uintptr_t)out & 15) == 0 &&
        ((uintptr_t)state & 15) == 0 && (((uintptr_t)w | (uintptr_t)bias) & 3) == 0) {
        dim3 g8((H / 8 + CONV_THREADS - 1) / CONV_THREADS, (max_q + CONV_TILE8 - 1) / CONV_TILE8, grid.z);
        if (g8.y > 65535) return NG_BAD_SIZE;
        NG_LAUNCH((shortconv_bf16x8_kernel<NG_CONV_L>), g8, CONV_THREADS, 0, stream, (const __nv_bfloat16*)p, w, bias, state,
                  (__nv_bfloat16*)out, cu_q, ctx_before, slots, H);
        return ng_launch_status();
    }
    if (act_bf16 && n_partials <= 1 && H % 2 == 0 && ((uintptr_t)p & 3) == 0 && ((uintptr_t)out & 3) == 0 &&
        ((uintptr_t)state & 7) == 0) {
        dim3 g2((H / 2 + CONV_THREADS - 1) / CONV_THREADS, grid.y, grid.z);
        NG_LAUNCH((shortconv_bf16x2_kernel<NG_CONV_L>), g2, CONV_THREADS, 0, stream, (const __nv_bfloat16*)p, w, bias, state,
                  (__nv_bfloat16*)out, cu_q, ctx_before, slots, H);
        return ng_launch_status();
    }
    // A thread walks the tokens of its tile in order, and every token's loads wait for memory: short portions (the
    // steps of few rows, whose input is a stack of partial sums) are cut into tiles of 4 tokens, so that their
    // tokens are spread over blocks instead; a tile re-reads the L-1 inputs before it, which is then cheap.
    // (A tile is at least L-1 tokens: only the first tile of a portion reaches back into the state slot.)
    const int tile = max_q <= 64 ? (NG_CONV_L - 1 > 4 ? NG_CONV_L - 1 : 4) : CONV_TILE;
    grid.y = (max_q + tile - 1) / tile;
    if (act_bf16 && n_partials > 1)
        dispatch_conv<float, __nv_bfloat16>(L, grid, stream, p, w, bias, state, out, cu_q, ctx_before, slots, H, n_partials, ps, tile);
    else if (act_bf16)
        dispatch_conv<__nv_bfloat16, __nv_bfloat16>(L, grid, stream, p, w, bias, state, out, cu_q, ctx_before, slots, H, 1, 0, tile);
    else
        dispatch_conv<float, float>(L, grid, stream, p, w, bias, state, out, cu_q, ctx_before, slots, H, n_partials, ps, tile);
    return ng_launch_status();
}

// Paged flash attention for prompt portions on the Blackwell tensor cores (bfloat16, head size 64).
//
// One block owns 128 consecutive query rows of one (entry, query head).  Six warps:
//   warps 0-3  softmax: thread r owns query row r = TMEM lane r
//   warp 4     producer: TMA loads of Q and of the K and V tiles, gathered page by page (a lane per page)
//   warp 5     MMA issuer: S = Q K^T and O += P V with tcgen05.mma (one elected lane), accumulators in TMEM
// Per 64-key tile: the issuer computes S (double-buffered in TMEM, so that the next tile's
// scores are computed while this tile's softmax runs); the softmax threads read their row
// of S with tcgen05.ld, mask it, update the running maximum and sum (float32, base 2), write
// P as bfloat16 back into TMEM over the first half of their row of S (tcgen05.st: the MMA
// takes its A operand from there, so P never passes through shared memory), and rescale
// their row of O in TMEM when the maximum moved; the issuer then accumulates P V into O.
// V is used as it lies in the cache ([key][dim], i.e. MN-major for the MMA's B operand).
// The tensor pipe runs the issuer's MMAs in order and a commit covers all of them before it,
// so "S of tile j + 2 is complete" also says that P V of tile j has read its P.
// Keys before the portion come from the pages earlier steps wrote; a missing page is loaded
// from an out-of-range coordinate (TMA fills zeros) and masked.
//
// Every mbarrier wait is bounded; a waiter that gives up sets a status bit and the block
// runs to its end (TMEM is always released).
//
// Long contexts in few blocks: when the launch's blocks fill the GPU's block slots unevenly (say 1.3 waves of
// them, each hundreds of tiles long), the keys of every block are cut into `n_splits` runs of whole tiles, each
// run a block of its own that writes a record (reference point, sum, unnormalised output row, float32) instead
// of the output, and a second small kernel merges the records in ascending order of the runs.  A block with
// fewer than SPLIT_MIN_TILES tiles per run is not cut: its first run does all of it, the others write empty
// records.  The caller decides `n_splits` (1: no records, the output is written directly).
//
// Takes: head size 64, page sizes 8..64 (a page is then a whole number of 1024-byte swizzle
// atoms).  Other shapes use the mma.sync kernel of attention_bf16.cu.
// Reference: gpu/cuda/attention.cu:369-500 (materialised scores, unpaged, K/V expanded per head).
#include "sm100_common.cuh"

#define HD 64
#define BQ 128                 // query rows per block
#define BK 64                  // keys per tile
#define KV_STAGES 3
#define NG_STATUS_ATTN_TIMEOUT 16
#define SPLIT_MIN_TILES 16     // a run of keys is at least this many tiles
#define REC (HD + 2)            // floats of a record: reference point (base 2, scaled), sum, output row
static_assert(BQ == BLOCK_W, "a block's query rows are the 128 rows of the MMA");

// max of three (one instruction on this architecture)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
// two float32 values in one 64-bit register, and the packed add / fused multiply-add on them
// (each half rounded as the scalar instruction rounds)
__device__ __forceinline__ unsigned long long pack2(float a, float b) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ unsigned long long ffma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long fadd2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

struct Smem {
    bf16 q[BQ * HD];                 // 16 KB, K-major swizzled
    bf16 k[KV_STAGES][BK * HD];      // 8 KB each
    bf16 v[KV_STAGES][BK * HD];
    uint64_t q_full, kv_full[KV_STAGES], kv_empty[KV_STAGES], s_full[2], p_full[2], o_ready[2];
    uint32_t tmem_base;
    int pages[1];                    // page ids of the block's keys follow (dynamic)
};

struct Params {
    bf16* out;
    const int* table;
    const int* cu_q;
    const int* ctx_before;
    int* status;
    int table_stride, nH, nKV, ps_log2, num_pages, window, skip_single, table_ints;
    float scale_log2;
    const float* slopes;             // per query head or null: score bias -slope * (query position - key position)
    float inv_scale;
    int n_splits;                    // runs the keys of a block are cut into
    float* scratch;                  // [row][head][run][REC] when n_splits > 1
};

__global__ void __launch_bounds__(192, 2)
attn_prefill_sm100_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                          const __grid_constant__ CUtensorMap map_v, const Params p) {
    extern __shared__ unsigned char smem_raw[];
    Smem* sm = reinterpret_cast<Smem*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    ng_pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.z / p.n_splits, split = blockIdx.z - e * p.n_splits, head = blockIdx.x;
    uint32_t elected;                                          // one lane of each warp, the same one every time it is asked
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(elected));
    const bool leader_of_warp = elected != 0;
    const int q0 = p.cu_q[e], qlen = p.cu_q[e + 1] - q0;     // written by the host copy, before any kernel of the step
    // Blocks start in the order of their index: the heads run fastest and the row tiles from the last one down, so
    // that the blocks with the most keys (the late rows, of every head) start first and the short ones fill the end.
    const int r0 = (gridDim.y - 1 - blockIdx.y) * BQ;
    if (r0 >= qlen || (p.skip_single && qlen == 1)) {
        ng_pdl_wait();                                         // a launch none of whose blocks waited would end before the kernel
        return;                                                // before it, and the kernel after it would start on unfinished data
    }
    const int ctx = p.ctx_before[e];
    const int kvh = head / (p.nH / p.nKV);
    const int rows_here = min(BQ, qlen - r0);
    const int pos_first = ctx + r0, pos_last = ctx + r0 + rows_here - 1;
    const int key_lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    int tile0 = key_lo / BK, tile1 = pos_last / BK;            // inclusive
    if (p.n_splits > 1) {                                      // this block's run of the tiles
        const int n_all = tile1 - tile0 + 1;
        if (n_all >= SPLIT_MIN_TILES * p.n_splits) {
            const int per = (n_all + p.n_splits - 1) / p.n_splits;
            tile0 += split * per;
            tile1 = min(tile1, tile0 + per - 1);
        } else if (split > 0) {
            tile1 = tile0 - 1;
        }
    }
    const int n_tiles = tile1 - tile0 + 1;
    const int kv_end = pos_last + 1;
    if (n_tiles <= 0) {                                        // an empty run: records that the merge passes over
        ng_pdl_wait();                                         // the scratch may still be read by an earlier merge
        if (threadIdx.x < rows_here) {
            float* rec = p.scratch + (((size_t)(q0 + r0 + threadIdx.x) * p.nH + head) * p.n_splits + split) * REC;
            rec[0] = -INFINITY;
            rec[1] = 0.f;
        }
        return;
    }

    if (threadIdx.x == 0) {
        mbar_init(&sm->q_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&sm->kv_full[s], 1); mbar_init(&sm->kv_empty[s], 1); }
        mbar_init(&sm->s_full[0], 1);
        mbar_init(&sm->s_full[1], 1);
        mbar_init(&sm->p_full[0], 4);                          // one arrival per softmax warp; one barrier per S/P buffer:
        mbar_init(&sm->p_full[1], 4);                          // a warp that runs a tile ahead must not complete the tile before it
        mbar_init(&sm->o_ready[0], 1);                         // two, used in turn: a softmax warp that skipped
        mbar_init(&sm->o_ready[1], 1);                         // its waits is never two phases behind on either
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" :: "r"(smem_u32(&sm->tmem_base)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    ng_pdl_wait();                                             // the table, q and the pages are this step's data
    // page ids of the keys this block reads (-1: none)
    const int first_page = (tile0 * BK) >> p.ps_log2;
    const int n_pages = ((kv_end - 1) >> p.ps_log2) - first_page + 1;
    const bool tab_smem = n_pages <= p.table_ints;
    const int* trow = p.table + (size_t)e * p.table_stride;
    if (tab_smem)
        for (int i = threadIdx.x; i < n_pages; i += blockDim.x) sm->pages[i] = trow[first_page + i];
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem = sm->tmem_base;
    const uint32_t tm_s0 = tmem, tm_s1 = tmem + BK, tm_o = tmem + 2 * BK;
    bool ok = true;

    if (warp == 4) {
        // ------------------------------------------------------------------ producer
        // The whole warp walks the tiles; lane i asks for the tile's page i (a box each of K and of V): one lane
        // issuing all of a tile's boxes in turn was the kernel's bound at 16-token pages.
        {
            if (lane == 0) {
                mbar_expect_tx(&sm->q_full, BQ * HD * 2);
                tma_load_2d(sm->q, &map_q, &sm->q_full, head * HD, q0 + r0);
            }
            const int ps = 1 << p.ps_log2;
            const int oob_row = p.num_pages * p.nKV * ps;          // an out-of-range row: TMA fills zeros
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j % KV_STAGES;
                ok = __all_sync(0xffffffffu, mbar_wait(&sm->kv_empty[s], ((j / KV_STAGES) & 1) ^ 1));   // one answer for the warp
                if (!ok) break;
                if (lane == 0) mbar_expect_tx(&sm->kv_full[s], 2 * BK * HD * 2);
                __syncwarp();
                const int key0 = (tile0 + j) * BK;
                const int c = lane << p.ps_log2;                    // one box per page (a tile is 64 / ps pages)
                if (c < BK) {
                    const int key = key0 + c;
                    int page = -1;
                    if (key < kv_end) page = tab_smem ? sm->pages[(key >> p.ps_log2) - first_page] : trow[key >> p.ps_log2];
                    const int row = (page >= 0 && page < p.num_pages) ? (page * p.nKV + kvh) * ps : oob_row;
                    tma_load_2d(sm->k[s] + c * HD, &map_k, &sm->kv_full[s], 0, row);
                    tma_load_2d(sm->v[s] + c * HD, &map_v, &sm->kv_full[s], 0, row);
                }
            }
            if (!ok && lane == 0) atomicOr(p.status, NG_STATUS_ATTN_TIMEOUT);
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer
        // All lanes run the loop and its waits, one elected lane issues: the descriptors and addresses are then
        // the same in every lane and the compiler keeps them in uniform registers, which the MMA instruction
        // reads; computed by a lone lane they cost a move per operand and the issue of a tile's eight MMAs took
        // twice as long.
        {
            const bool leader = leader_of_warp;
            constexpr uint32_t idesc_s = make_idesc(BK, 0), idesc_o = make_idesc(HD, 1);
            ok = __all_sync(0xffffffffu, mbar_wait(&sm->q_full, 0));
            const uint64_t dq = make_desc_sw128(sm->q);
            auto issue_s = [&](int j) {                             // S_j = Q K_j^T into buffer j & 1
                const int s = j % KV_STAGES;
                if (!__all_sync(0xffffffffu, mbar_wait(&sm->kv_full[s], (j / KV_STAGES) & 1))) { ok = false; return; }
                tcgen05_fence_after();
                const uint64_t dk = make_desc_sw128(sm->k[s]);
                if (leader) {
#pragma unroll
                    for (int k = 0; k < HD / 16; ++k)
                        tcgen05_mma_f16((j & 1) ? tm_s1 : tm_s0, dq + (uint64_t)(2 * k), dk + (uint64_t)(2 * k), idesc_s, k > 0);
                    tcgen05_commit(&sm->s_full[j & 1]);
                }
                __syncwarp();
            };
            if (ok) issue_s(0);
            if (ok && n_tiles > 1) issue_s(1);
            for (int j = 0; j < n_tiles && ok; ++j) {
                ok = __all_sync(0xffffffffu, mbar_wait(&sm->p_full[j & 1], (j >> 1) & 1));   // P_j in tensor memory, O rescaled
                if (!ok) break;
                tcgen05_fence_after();
                const int s = j % KV_STAGES;
                const uint64_t dv = make_desc_sw128_mn(sm->v[s]);
                const uint32_t tp = (j & 1) ? tm_s1 : tm_s0;        // P_j lies over the first 32 columns of S_j
                if (leader) {
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)                   // 16 keys per MMA: 8 columns of P, 2048 bytes of V
                        tcgen05_mma_f16_ts(tm_o, tp + 8 * k, dv + (uint64_t)(128 * k), idesc_o, (j > 0 || k > 0));
                    tcgen05_commit(&sm->kv_empty[s]);                        // K_j and V_j may be overwritten
                    tcgen05_commit(&sm->o_ready[j & 1]);                     // O holds tiles 0..j
                }
                __syncwarp();
                if (j + 2 < n_tiles) issue_s(j + 2);                // over S_j and P_j: runs after the product above
            }
            if (!ok && leader) atomicOr(p.status, NG_STATUS_ATTN_TIMEOUT);
        }
    } else {
        // ------------------------------------------------------------------ softmax: thread = query row
        const int r = warp * 32 + lane;
        const int pos = ctx + r0 + min(r, rows_here - 1);           // rows past the portion mirror its last row
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        // m is the reference point of the exponentials.  It follows the running maximum lazily:
        // only when a tile's maximum exceeds it by more than 2^8 is O in TMEM rescaled (which
        // has to wait for the previous P V product); otherwise P simply holds values up to 256.
        float m = -INFINITY, l = 0.f;
        // the bias is added to the raw score in units of 1/scale, so that the scaling below gives score * scale - bias
        const float slope_raw = p.slopes ? p.slopes[head] * p.inv_scale : 0.f;
        for (int j = 0; j < n_tiles && ok; ++j) {
            ok = mbar_wait(&sm->s_full[j & 1], (j >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tcgen05_fence_after();
            const uint32_t ts = ((j & 1) ? tm_s1 : tm_s0) + lane_base;
            const int key0 = (tile0 + j) * BK;
            float sc[BK];
            float mx = -INFINITY;
            tmem_ld64(ts, sc);
            // only tiles that cross a row's diagonal or the window's edge need the mask
            const bool whole = key0 + BK - 1 <= pos_first && (p.window <= 0 || key0 > pos_last - p.window);
            if (whole && slope_raw == 0.f) {
                float m0 = sc[0], m1 = sc[1], m2 = sc[2], m3 = sc[3];    // four chains: a single one waits for itself
#pragma unroll
                for (int i = 4; i < BK - 4; i += 8) {
                    m0 = fmax3(m0, sc[i], sc[i + 1]);
                    m1 = fmax3(m1, sc[i + 2], sc[i + 3]);
                    m2 = fmax3(m2, sc[i + 4], sc[i + 5]);
                    m3 = fmax3(m3, sc[i + 6], sc[i + 7]);
                }
                m0 = fmax3(m0, sc[BK - 4], sc[BK - 3]);
                m1 = fmax3(m1, sc[BK - 2], sc[BK - 1]);
                mx = fmaxf(fmax3(m0, m1, m2), m3);
            } else {
#pragma unroll
                for (int i = 0; i < BK; ++i) {
                    const int key = key0 + i;
                    const bool vis = key <= pos && (p.window <= 0 || key > pos - p.window);
                    sc[i] = vis ? fmaf(slope_raw, (float)(key - pos), sc[i]) : -INFINITY;
                    mx = fmaxf(mx, sc[i]);
                }
            }
            mx *= p.scale_log2;                                        // scale > 0: the maximum of the scaled scores
            float corr = 1.f;
            if (mx > m + 8.f || (m == -INFINITY && mx > -INFINITY)) {     // move the reference point
                corr = ex2(m - mx);                                       // 0 the first time
                m = mx;
            }
            const float ref = m == -INFINITY ? 0.f : m;
            uint32_t pk[BK / 2];
            const unsigned long long scale2 = pack2(p.scale_log2, p.scale_log2), nref2 = pack2(-ref, -ref);
            unsigned long long sum2 = pack2(0.f, 0.f);                  // even and odd keys summed apart
#pragma unroll
            for (int i = 0; i < BK; i += 2) {
                float x0, x1;
                unpack2(ffma2(pack2(sc[i], sc[i + 1]), scale2, nref2), x0, x1);
                const float a = ex2(x0), b = ex2(x1);
                sum2 = fadd2(sum2, pack2(a, b));
                __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                pk[i / 2] = *reinterpret_cast<uint32_t*>(&h);
            }
            float sum_a, sum_b;
            unpack2(sum2, sum_a, sum_b);
            l = l * corr + (sum_a + sum_b);
            if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {         // rescale this warp's rows of O
                ok = mbar_wait(&sm->o_ready[(j - 1) & 1], ((j - 1) >> 1) & 1);   // P_{j-1} V_{j-1} has been added
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tcgen05_fence_after();
#pragma unroll
                for (int c = 0; c < HD; c += 16) {
                    float v[16];
                    tmem_ld16(tm_o + lane_base + c, v);
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] *= corr;
                    tmem_st16(tm_o + lane_base + c, v);
                }
                tmem_st_wait();
            }
            // P row -> tensor memory, over this row's S (whose buffer is free of readers: S_j complete means
            // that the product of tile j - 2, the last reader of this buffer's P, is complete)
            tmem_st32(ts, pk);
            tmem_st_wait();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm->p_full[j & 1]);
        }
        // ---- epilogue: O / l -> out
        if (ok) {
            ok = mbar_wait(&sm->o_ready[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok && p.n_splits > 1) {                                 // this run's record
            tcgen05_fence_after();
            float* rec = p.scratch + (((size_t)(q0 + r0 + r) * p.nH + head) * p.n_splits + split) * REC;
            if (r < rows_here) { rec[0] = m; rec[1] = l; }
#pragma unroll
            for (int c = 0; c < HD; c += 16) {
                float v[16];
                tmem_ld16(tm_o + lane_base + c, v);
                if (r < rows_here) {
#pragma unroll
                    for (int i = 0; i < 16; i += 2) *reinterpret_cast<float2*>(rec + 2 + c + i) = make_float2(v[i], v[i + 1]);
                }
            }
        } else if (ok) {
            tcgen05_fence_after();
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* orow = p.out + ((size_t)(q0 + r0 + r) * p.nH + head) * HD;
#pragma unroll
            for (int c = 0; c < HD; c += 16) {
                float v[16];
                tmem_ld16(tm_o + lane_base + c, v);
                if (r < rows_here) {
                    uint32_t w[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i] * inv, v[2 * i + 1] * inv);
                        w[i] = *reinterpret_cast<uint32_t*>(&h);
                    }
                    *reinterpret_cast<uint4*>(orow + c) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(orow + c + 8) = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
        } else if (lane == 0) {
            atomicOr(p.status, NG_STATUS_ATTN_TIMEOUT);
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 5)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" :: "r"(tmem) : "memory");
}

// out[row, head, :] = sum_s o_s 2^(m_s - m) / sum_s l_s 2^(m_s - m) over the runs s in ascending order, m = max m_s.
// One warp per (row, head); rows of entries that the attention kernel left alone (a single token, when those go
// to the other kernel) are left alone here too.
__global__ void __launch_bounds__(256)
attn_prefill_merge_kernel(const float* __restrict__ scratch, const int* __restrict__ cu_q, bf16* __restrict__ out,
                          int nH, int n_splits, int skip_single) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int e = blockIdx.z, head = blockIdx.x;
    const int q0 = cu_q[e], qlen = cu_q[e + 1] - q0;
    const int r0 = blockIdx.y * BQ;
    if (r0 >= qlen || (skip_single && qlen == 1)) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = r0 + warp; r < min(qlen, r0 + BQ); r += 8) {
        const float* rec = scratch + ((size_t)(q0 + r) * nH + head) * n_splits * REC;
        float m = -INFINITY;
        for (int s = 0; s < n_splits; ++s) m = fmaxf(m, rec[(size_t)s * REC]);
        float l = 0.f, a0 = 0.f, a1 = 0.f;
        if (m > -INFINITY) {
            for (int s = 0; s < n_splits; ++s) {
                const float ms = rec[(size_t)s * REC], ls = rec[(size_t)s * REC + 1];
                if (!(ls > 0.f)) continue;                          // an empty run wrote no output row
                const float f = exp2f(ms - m);
                const float2 o = *reinterpret_cast<const float2*>(rec + (size_t)s * REC + 2 + 2 * lane);
                l += ls * f;
                a0 += o.x * f;
                a1 += o.y * f;
            }
        }
        const float inv = l > 0.f ? 1.f / l : 0.f;
        *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)(q0 + r) * nH + head) * HD + 2 * lane) = __floats2bfloat162_rn(a0 * inv, a1 * inv);
    }
}

// ------------------------------------------------------------------------------------- host
// 1 if the kernel takes this shape
NG_EXPORT int ng_attn_prefill_sm100_takes(int hd, int page_size) {
    return hd == HD && page_size >= 8 && page_size <= 64 && (page_size & (page_size - 1)) == 0;
}

NG_EXPORT int ng_attn_prefill_sm100(const void* q, const void* k_pages, const void* v_pages, const int* table,
                                    int table_stride, const int* cu_q, const int* ctx_before, void* out, int n_rows,
                                    int n_entries, int max_q, int nH, int nKV, int hd, int page_size, int num_pages,
                                    int window, float scale, int skip_single, const float* slopes, float* scratch,
                                    int n_splits, int* status, cudaStream_t stream) {
    if (n_entries <= 0 || max_q <= 0 || n_rows <= 0) return NG_OK;
    if (!ng_attn_prefill_sm100_takes(hd, page_size) || !(scale > 0.f) || nH <= 0 || nKV <= 0 || nH % nKV || (max_q + BQ - 1) / BQ > 65535 ||
        n_splits < 1 || (long long)n_entries * n_splits > 65535 || (n_splits > 1 && !scratch) || !status || ((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15))
        return NG_BAD_SIZE;
    int ps_log2 = 0;
    while ((1 << ps_log2) < page_size) ++ps_log2;
    CUtensorMap mq, mk, mv;
    const long long kv_rows = (long long)num_pages * nKV * page_size;
    if (!tensor_map(q, n_rows, nH * HD, BQ, &mq) || !tensor_map(k_pages, kv_rows, HD, page_size, &mk) ||
        !tensor_map(v_pages, kv_rows, HD, page_size, &mv))
        return NG_LAUNCH_FAILED;
    constexpr int TABLE_INTS = 2048;                           // 8 KB: 32k keys of context at 16 per page
    const size_t smem = sizeof(Smem) + TABLE_INTS * sizeof(int) + 1024;
    static bool attr = false;
    if (!attr) {
        if (cudaFuncSetAttribute(attn_prefill_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return NG_LAUNCH_FAILED;
        attr = true;
    }
    Params p{(bf16*)out, table, cu_q, ctx_before, status, table_stride, nH, nKV, ps_log2, num_pages, window, skip_single,
             TABLE_INTS, scale * 1.4426950408889634f, slopes, 1.f / scale, n_splits, scratch};
    dim3 grid(nH, (max_q + BQ - 1) / BQ, n_entries * n_splits);
    NG_LAUNCH((attn_prefill_sm100_kernel), grid, 192, smem, stream, mq, mk, mv, p);
    if (n_splits > 1)
        NG_LAUNCH((attn_prefill_merge_kernel), dim3(nH, (max_q + BQ - 1) / BQ, n_entries), 256, 0, stream,
                  (const float*)scratch, cu_q, (bf16*)out, nH, n_splits, skip_single);
    return ng_launch_status();
}

// float32 values of scratch that n_splits > 1 needs: a record per (row of q, head, run)
NG_EXPORT long long ng_attn_prefill_sm100_scratch_floats(int n_rows, int nH, int n_splits) {
    return n_splits > 1 ? (long long)n_rows * nH * n_splits * REC : 0;
}

// Paged flash attention for prompt portions on the Blackwell tensor cores (bfloat16, head size 64).
//
// One block owns 128 consecutive query rows of one (entry, query head).  Six warps:
//   warps 0-3  softmax: thread r owns query row r = TMEM lane r
//   warp 4     producer: TMA loads of Q and of the K and V tiles, gathered page by page
//   warp 5     MMA issuer: S = Q K^T and O += P V with tcgen05.mma, accumulators in TMEM
// Per 64-key tile: the issuer computes S (double-buffered in TMEM, so that the next tile's
// scores are computed while this tile's softmax runs); the softmax threads read their row
// of S with tcgen05.ld, mask it, update the running maximum and sum (float32, base 2), write
// P as bfloat16 into shared memory in the swizzled K-major layout the MMA reads, and rescale
// their row of O in TMEM when the maximum moved; the issuer then accumulates P V into O.
// V is used as it lies in the cache ([key][dim], i.e. MN-major for the MMA's B operand).
// Keys before the portion come from the pages earlier steps wrote; a missing page is loaded
// from an out-of-range coordinate (TMA fills zeros) and masked.
//
// Every mbarrier wait is bounded; a waiter that gives up sets a status bit and the block
// runs to its end (TMEM is always released).
//
// Takes: head size 64, page sizes 8..64 (a page is then a whole number of 1024-byte swizzle
// atoms).  Other shapes use the mma.sync kernel of attention_bf16.cu.
// Reference: gpu/cuda/attention.cu:369-500 (materialised scores, unpaged, K/V expanded per head).
#include <cuda.h>
#include <mutex>
#include <unordered_map>

#include "ng_common.cuh"

typedef __nv_bfloat16 bf16;

#define HD 64
#define BQ 128                 // query rows per block
#define BK 64                  // keys per tile
#define KV_STAGES 3
#define NG_SPIN_LIMIT (1u << 20)
#define NG_STATUS_ATTN_TIMEOUT 16

// ------------------------------------------------------------------------------------- PTX
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < NG_SPIN_LIMIT; ++i) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// 64 consecutive float32 columns of this thread's TMEM lane, one load and one wait
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&v)[64]) {
    uint32_t r[64];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x64.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];\n\ttcgen05.wait::ld.sync.aligned;"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]), "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]), "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
                 : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const float (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 :: "r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
                    "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
                    "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
                    "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
                    "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
                    "r"(__float_as_uint(v[15])) : "memory");
}
// 2^x for x <= 0 or a little above (the arguments here are score minus reference): the
// hardware approximation, exact to 2 ulp, -inf -> 0
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// K-major operand tile with 128-byte rows written with the 128-byte swizzle (Q, K, P)
__device__ __forceinline__ uint64_t desc_kmajor(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;                  // 8-row groups 1024 bytes apart
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;                            // 128-byte swizzle
    return d;
}
// MN-major operand tile (V: rows = keys = the MMA's K, 64 dims = 128 bytes contiguous per row)
__device__ __forceinline__ uint64_t desc_mnmajor(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);
    d |= (uint64_t)(1024 >> 4) << 16;                  // leading offset: next 64-wide block of dims (there is one)
    d |= (uint64_t)(1024 >> 4) << 32;                  // stride offset: next group of 8 keys
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// D float32, A/B bfloat16, M = 128, N = n; b_mn: B operand is MN-major
__host__ __device__ constexpr uint32_t make_idesc(int n, int b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BQ >> 4) << 24);
}

struct Smem {
    bf16 q[BQ * HD];                 // 16 KB, K-major swizzled
    bf16 p[2][BQ * BK];              // 2 x 16 KB, K-major swizzled (K = keys): tile j uses buffer j & 1
    bf16 k[KV_STAGES][BK * HD];      // 8 KB each
    bf16 v[KV_STAGES][BK * HD];
    uint64_t q_full, kv_full[KV_STAGES], kv_empty[KV_STAGES], s_full[2], p_full[2], p_free[2], o_ready[2];
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
};

__global__ void __launch_bounds__(192)
attn_prefill_sm100_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                          const __grid_constant__ CUtensorMap map_v, const Params p) {
    extern __shared__ unsigned char smem_raw[];
    Smem* sm = reinterpret_cast<Smem*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    ng_pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.z, head = blockIdx.y;
    const int q0 = p.cu_q[e], qlen = p.cu_q[e + 1] - q0;     // written by the host copy, before any kernel of the step
    const int r0 = (gridDim.x - 1 - blockIdx.x) * BQ;         // late rows see the most keys: start them first
    if (r0 >= qlen || (p.skip_single && qlen == 1)) return;
    const int ctx = p.ctx_before[e];
    const int kvh = head / (p.nH / p.nKV);
    const int rows_here = min(BQ, qlen - r0);
    const int pos_first = ctx + r0, pos_last = ctx + r0 + rows_here - 1;
    const int key_lo = p.window > 0 ? max(0, pos_first - p.window + 1) : 0;
    const int tile0 = key_lo / BK, tile1 = pos_last / BK;      // inclusive
    const int n_tiles = tile1 - tile0 + 1;
    const int kv_end = pos_last + 1;

    if (threadIdx.x == 0) {
        mbar_init(&sm->q_full, 1);
        for (int s = 0; s < KV_STAGES; ++s) { mbar_init(&sm->kv_full[s], 1); mbar_init(&sm->kv_empty[s], 1); }
        mbar_init(&sm->s_full[0], 1);
        mbar_init(&sm->s_full[1], 1);
        mbar_init(&sm->p_full[0], 128);                        // one barrier per P buffer: a warp that runs a tile
        mbar_init(&sm->p_full[1], 128);                        // ahead must not complete the tile before it
        mbar_init(&sm->p_free[0], 1);
        mbar_init(&sm->p_free[1], 1);
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
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = sm->tmem_base;
    const uint32_t tm_s0 = tmem, tm_s1 = tmem + BK, tm_o = tmem + 2 * BK;
    bool ok = true;

    if (warp == 4) {
        // ------------------------------------------------------------------ producer
        if (lane == 0) {
            mbar_expect_tx(&sm->q_full, BQ * HD * 2);
            tma_load_2d(sm->q, &map_q, &sm->q_full, head * HD, q0 + r0);
            const int ps = 1 << p.ps_log2;
            const int oob_row = p.num_pages * p.nKV * ps;          // an out-of-range row: TMA fills zeros
            for (int j = 0; j < n_tiles && ok; ++j) {
                const int s = j % KV_STAGES;
                ok = mbar_wait(&sm->kv_empty[s], ((j / KV_STAGES) & 1) ^ 1);
                if (!ok) break;
                mbar_expect_tx(&sm->kv_full[s], 2 * BK * HD * 2);
                const int key0 = (tile0 + j) * BK;
                for (int c = 0; c < BK; c += ps) {                 // one box per page (a tile is 64 / ps pages)
                    const int key = key0 + c;
                    int page = -1;
                    if (key < kv_end) page = tab_smem ? sm->pages[(key >> p.ps_log2) - first_page] : trow[key >> p.ps_log2];
                    const int row = (page >= 0 && page < p.num_pages) ? (page * p.nKV + kvh) * ps : oob_row;
                    tma_load_2d(sm->k[s] + c * HD, &map_k, &sm->kv_full[s], 0, row);
                    tma_load_2d(sm->v[s] + c * HD, &map_v, &sm->kv_full[s], 0, row);
                }
            }
            if (!ok) atomicOr(p.status, NG_STATUS_ATTN_TIMEOUT);
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc(BK, 0), idesc_o = make_idesc(HD, 1);
            ok = mbar_wait(&sm->q_full, 0);
            const uint64_t dq = desc_kmajor(sm->q);
            auto issue_s = [&](int j) {                             // S_j = Q K_j^T into buffer j & 1
                const int s = j % KV_STAGES;
                if (!mbar_wait(&sm->kv_full[s], (j / KV_STAGES) & 1)) { ok = false; return; }
                tc_fence_after();
                const uint64_t dk = desc_kmajor(sm->k[s]);
#pragma unroll
                for (int k = 0; k < HD / 16; ++k)
                    tc_mma((j & 1) ? tm_s1 : tm_s0, dq + (uint64_t)(2 * k), dk + (uint64_t)(2 * k), idesc_s, k > 0);
                tc_commit(&sm->s_full[j & 1]);
            };
            if (ok) issue_s(0);
            if (ok && n_tiles > 1) issue_s(1);
            for (int j = 0; j < n_tiles && ok; ++j) {
                ok = mbar_wait(&sm->p_full[j & 1], (j >> 1) & 1);   // P_j in shared memory, O rescaled
                if (!ok) break;
                tc_fence_after();
                const int s = j % KV_STAGES;
                const uint64_t dv = desc_mnmajor(sm->v[s]), dp = desc_kmajor(sm->p[j & 1]);
#pragma unroll
                for (int k = 0; k < BK / 16; ++k)                   // 16 keys per MMA: 32 bytes of P, 2048 bytes of V
                    tc_mma(tm_o, dp + (uint64_t)(2 * k), dv + (uint64_t)(128 * k), idesc_o, (j > 0 || k > 0));
                tc_commit(&sm->kv_empty[s]);                        // K_j and V_j may be overwritten
                tc_commit(&sm->p_free[j & 1]);                      // P buffer j & 1 may be overwritten
                tc_commit(&sm->o_ready[j & 1]);                     // O holds tiles 0..j
                if (j + 2 < n_tiles) issue_s(j + 2);                // buffer j & 1 was read before P_j was posted
            }
            if (!ok) atomicOr(p.status, NG_STATUS_ATTN_TIMEOUT);
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
        for (int j = 0; j < n_tiles && ok; ++j) {
            ok = mbar_wait(&sm->s_full[j & 1], (j >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t ts = ((j & 1) ? tm_s1 : tm_s0) + lane_base;
            const int key0 = (tile0 + j) * BK;
            float sc[BK];
            float mx = -INFINITY;
            tmem_ld64(ts, sc);
            // only tiles that cross a row's diagonal or the window's edge need the mask
            const bool whole = key0 + BK - 1 <= pos_first && (p.window <= 0 || key0 > pos_last - p.window);
            if (whole) {
#pragma unroll
                for (int i = 0; i < BK; ++i) mx = fmaxf(mx, sc[i]);
            } else {
#pragma unroll
                for (int i = 0; i < BK; ++i) {
                    const int key = key0 + i;
                    const bool vis = key <= pos && (p.window <= 0 || key > pos - p.window);
                    sc[i] = vis ? sc[i] : -INFINITY;
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
            float sum = 0.f;
            uint32_t pk[BK / 2];
#pragma unroll
            for (int i = 0; i < BK; i += 2) {
                const float a = ex2(fmaf(sc[i], p.scale_log2, -ref)), b = ex2(fmaf(sc[i + 1], p.scale_log2, -ref));
                sum += a + b;
                __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                pk[i / 2] = *reinterpret_cast<uint32_t*>(&h);
            }
            l = l * corr + sum;
            if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {         // rescale this warp's rows of O
                ok = mbar_wait(&sm->o_ready[(j - 1) & 1], ((j - 1) >> 1) & 1);   // P_{j-1} V_{j-1} has been added
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
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
            if (j >= 2) {                                                // the product that read this P buffer is done
                ok = mbar_wait(&sm->p_free[j & 1], ((j >> 1) - 1) & 1);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
            }
            // P row -> shared memory: 16-byte chunk q of row r lies at chunk q ^ (r & 7)
            unsigned char* prow = reinterpret_cast<unsigned char*>(sm->p[j & 1]) + r * 128;
#pragma unroll
            for (int q = 0; q < 8; ++q)
                *reinterpret_cast<uint4*>(prow + ((q ^ (r & 7)) << 4)) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the MMA's reads
            tc_fence_before();
            mbar_arrive(&sm->p_full[j & 1]);
        }
        // ---- epilogue: O / l -> out
        if (ok) {
            ok = mbar_wait(&sm->o_ready[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1);
            ok = __all_sync(0xffffffffu, ok);
        }
        if (ok) {
            tc_fence_after();
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
    tc_fence_before();
    __syncthreads();
    if (warp == 5)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" :: "r"(tmem) : "memory");
}

// ------------------------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}
struct MapKey {
    const void* ptr; long long rows; int cols, box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.cols << 20) ^ ((size_t)k.box_rows << 40);
    }
};
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
static std::mutex g_mutex;

// [rows, cols] row-major bf16 with boxes of box_rows x 64 columns, 128-byte swizzle
static bool tensor_map(const void* ptr, long long rows, int cols, int box_rows, CUtensorMap* out) {
    const MapKey key{ptr, rows, cols, box_rows};
    std::lock_guard<std::mutex> lock(g_mutex);
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return true; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    if (fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps.emplace(key, m);
    *out = m;
    return true;
}

// 1 if the kernel takes this shape
NG_EXPORT int ng_attn_prefill_sm100_takes(int hd, int page_size) {
    return hd == HD && page_size >= 8 && page_size <= 64 && (page_size & (page_size - 1)) == 0;
}

NG_EXPORT int ng_attn_prefill_sm100(const void* q, const void* k_pages, const void* v_pages, const int* table,
                                    int table_stride, const int* cu_q, const int* ctx_before, void* out, int n_rows,
                                    int n_entries, int max_q, int nH, int nKV, int hd, int page_size, int num_pages,
                                    int window, float scale, int skip_single, int* status, cudaStream_t stream) {
    if (n_entries <= 0 || max_q <= 0 || n_rows <= 0) return NG_OK;
    if (!ng_attn_prefill_sm100_takes(hd, page_size) || !(scale > 0.f) || nH <= 0 || nKV <= 0 || nH % nKV || nH > 65535 ||
        n_entries > 65535 || !status || ((uintptr_t)q & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15))
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
             TABLE_INTS, scale * 1.4426950408889634f};
    dim3 grid((max_q + BQ - 1) / BQ, nH, n_entries);
    NG_LAUNCH((attn_prefill_sm100_kernel), grid, 192, smem, stream, mq, mk, mv, p);
    return ng_launch_status();
}

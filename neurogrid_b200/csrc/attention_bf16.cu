// Tensor-core paged attention for the bfloat16 path, specialised on the head size
// (compile with -DNG_HEAD_DIM=<multiple of 16, 16..256>).
//
//  * ng_attn_prefill_bf16: flash attention of prompt portions.  A block owns 64 consecutive
//    query rows of one (entry, query head); 64-key tiles of K and V are gathered from the
//    entry's pages into shared memory with cp.async (two stages), scores and the P*V product
//    run on mma.sync m16n8k16 with float32 accumulators, the softmax is online in float32.
//    Keys before the portion come from the pages earlier steps wrote; the portion's own keys
//    were written by the rope/cache kernel of the same step.
//  * ng_attn_decode_bf16: one query row per entry.  A block owns one (entry, KV head, split
//    of the context): the n_heads / n_kv_heads query heads that share the KV head are the rows
//    of one MMA tile, so K and V are read once for the whole group.  K and V fragments are
//    loaded straight from global memory (the contraction index and the output dimension are
//    permuted so that every lane reads contiguous bytes).  With more than one split the block
//    writes (max, sum, unnormalised output) to scratch and ng_attn_combine merges the splits.
//
// The reference's decode kernel keeps all scores of one head in shared memory, one block per
// head, context <= 4096 (gpu/cuda/paged_attention.cu:278-387); its prefill materialises
// [heads, S, S] scores in HBM with K/V expanded to every query head
// (gpu/cuda/attention.cu:332-363,369-500).
#include "ng_common.cuh"

#ifndef NG_HEAD_DIM
#error "compile with -DNG_HEAD_DIM=<head size>"
#endif
#define HD NG_HEAD_DIM
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 in [16, 256]");

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_ptr) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void cp_async_16(void* smem_ptr, const void* gptr, bool valid) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    const int n = valid ? 16 : 0;                      // src-size 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" :: "r"(addr), "l"(gptr), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" :: "n"(N)); }

// ===================================================================================== prefill
#define PF_ROWS 64            // query rows per block (16 per warp)
#define PF_KEYS 64            // keys per tile
#define PF_THREADS 128
#define PF_LD (HD + 8)        // shared-memory row stride in elements: 16-byte aligned, conflict-free ldmatrix

struct PrefillSmem {
    bf16 q[PF_ROWS][PF_LD];
    bf16 k[2][PF_KEYS][PF_LD];
    bf16 v[2][PF_KEYS][PF_LD];
};

// Gather one 64-key tile of K and V (keys key0..key0+63 of the entry) into stage s.
// `ptab[(key >> ps_log2) - first_page]` is the page of a key: the block's slice of the table in
// shared memory when it fits, else the entry's table row itself (first_page 0).
__device__ __forceinline__ void pf_load_tile(PrefillSmem* sm, int s, const bf16* __restrict__ k_pages,
                                             const bf16* __restrict__ v_pages, const int* __restrict__ ptab,
                                             int first_page, int key0, int kv_end, int kvh, int nKV, int ps_log2,
                                             int num_pages) {
    constexpr int CH = HD / 8;                          // 16-byte chunks per row
#pragma unroll
    for (int c0 = 0; c0 < PF_KEYS * CH; c0 += PF_THREADS) {
        const int c = c0 + threadIdx.x;
        if (PF_KEYS * CH % PF_THREADS != 0 && c >= PF_KEYS * CH) break;
        const int r = c / CH, ch = c % CH;
        const int key = key0 + r;
        bool ok = key < kv_end;
        size_t off = 0;
        if (ok) {
            const int page = ptab[(key >> ps_log2) - first_page];
            ok = page >= 0 && page < num_pages;
            off = ((((size_t)(ok ? page : 0) * nKV + kvh) << ps_log2) + (key & ((1 << ps_log2) - 1))) * HD + ch * 8;
        }
        cp_async_16(&sm->k[s][r][ch * 8], k_pages + off, ok);
        cp_async_16(&sm->v[s][r][ch * 8], v_pages + off, ok);
    }
}

__global__ void __launch_bounds__(PF_THREADS)
attn_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                    const int* __restrict__ table, int table_stride, const int* __restrict__ cu_q,
                    const int* __restrict__ ctx_before, bf16* __restrict__ out, int nH, int nKV, int ps_log2,
                    int num_pages, int window, float scale_log2, int skip_single, int table_ints,
                    const float* __restrict__ slopes) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    PrefillSmem* sm = reinterpret_cast<PrefillSmem*>(smem_raw);
    ng_pdl_trigger();
    ng_pdl_wait();
    // blocks start in index order: heads fastest, row tiles from the last down, so that the blocks with the most
    // keys (late rows, of every head) start first and the short ones fill the end
    const int e = blockIdx.z, head = blockIdx.x;
    const int q0 = cu_q[e], qlen = cu_q[e + 1] - q0;
    const int r0 = (gridDim.y - 1 - blockIdx.y) * PF_ROWS;
    if (r0 >= qlen || (skip_single && qlen == 1)) return;
    const int ctx = ctx_before[e];
    const int kvh = head / (nH / nKV);
    const int* trow = table + (size_t)e * table_stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int rows_here = min(PF_ROWS, qlen - r0);

    // Q tile -> shared memory (rows beyond the portion are zero)
    constexpr int CH = HD / 8;
    for (int c = threadIdx.x; c < PF_ROWS * CH; c += PF_THREADS) {
        const int r = c / CH, ch = c % CH;
        const bool ok = r < rows_here;
        cp_async_16(&sm->q[r][ch * 8], q + ((size_t)(q0 + r0 + (ok ? r : 0)) * nH + head) * HD + ch * 8, ok);
    }
    const int pos_first = ctx + r0, pos_last = ctx + r0 + rows_here - 1;     // positions of this block's rows
    const int key_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
    const int tile0 = key_lo / PF_KEYS, tile1 = pos_last / PF_KEYS;          // inclusive
    const int kv_end = pos_last + 1;
    // page ids of the keys this block reads, once, into shared memory (if they fit)
    const int* ptab = trow;
    int first_page = 0;
    {
        const int fp = (tile0 * PF_KEYS) >> ps_log2;
        const int n_pages = ((kv_end - 1) >> ps_log2) - fp + 1;
        if (n_pages <= table_ints) {
            int* tab = reinterpret_cast<int*>(smem_raw + sizeof(PrefillSmem));
            for (int i = threadIdx.x; i < n_pages; i += PF_THREADS) tab[i] = trow[fp + i];
            ptab = tab;
            first_page = fp;
            __syncthreads();
        }
    }
    pf_load_tile(sm, 0, k_pages, v_pages, ptab, first_page, tile0 * PF_KEYS, kv_end, kvh, nKV, ps_log2, num_pages);
    cp_async_commit();

    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;       // rows g and g+8 of the warp
    const int row_lo = warp * 16 + g, row_hi = row_lo + 8;
    const int pos_lo = ctx + r0 + row_lo, pos_hi = ctx + r0 + row_hi;
    const float slope2 = slopes ? slopes[head] * 1.4426950408889634f : 0.f;   // score bias, base 2

    for (int tile = tile0; tile <= tile1; ++tile) {
        const int s = (tile - tile0) & 1;
        if (tile < tile1) {
            pf_load_tile(sm, s ^ 1, k_pages, v_pages, ptab, first_page, (tile + 1) * PF_KEYS, kv_end, kvh, nKV, ps_log2,
                         num_pages);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        // ---- S = Q K^T for this warp's 16 rows x 64 keys
        float sc[PF_KEYS / 8][4];
#pragma unroll
        for (int i = 0; i < PF_KEYS / 8; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
#pragma unroll
        for (int kb = 0; kb < HD / 16; ++kb) {
            uint32_t a[4];
            ldmatrix_x4(a, &sm->q[warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][kb * 16 + 8 * (lane >> 4)]);
#pragma unroll
            for (int np = 0; np < PF_KEYS / 16; ++np) {        // pairs of 8-key tiles
                uint32_t b[4];
                ldmatrix_x4(b, &sm->k[s][np * 16 + (lane & 7) + 8 * (lane >> 4)][kb * 16 + 8 * ((lane >> 3) & 1)]);
                mma_bf16(sc[2 * np], a, b[0], b[1]);
                mma_bf16(sc[2 * np + 1], a, b[2], b[3]);
            }
        }
        // ---- mask, online softmax (float32, base 2)
        const int key_base = tile * PF_KEYS;
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < PF_KEYS / 8; ++nt) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int key = key_base + nt * 8 + 2 * t + j;
                const bool ok_lo = key <= pos_lo && (window <= 0 || key > pos_lo - window);
                const bool ok_hi = key <= pos_hi && (window <= 0 || key > pos_hi - window);
                sc[nt][j] = ok_lo ? fmaf(sc[nt][j], scale_log2, -slope2 * (float)(pos_lo - key)) : -INFINITY;
                sc[nt][2 + j] = ok_hi ? fmaf(sc[nt][2 + j], scale_log2, -slope2 * (float)(pos_hi - key)) : -INFINITY;
                mx_lo = fmaxf(mx_lo, sc[nt][j]);
                mx_hi = fmaxf(mx_hi, sc[nt][2 + j]);
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
        // a row with no visible key so far keeps m = -inf: use 0 as the reference point there
        const float ref_lo = mn_lo == -INFINITY ? 0.f : mn_lo, ref_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
        const float c_lo = exp2f(m_lo - ref_lo), c_hi = exp2f(m_hi - ref_hi);
        float sum_lo = 0.f, sum_hi = 0.f;
        uint32_t p[PF_KEYS / 16][4];
#pragma unroll
        for (int nt = 0; nt < PF_KEYS / 8; ++nt) {
            const float p0 = exp2f(sc[nt][0] - ref_lo), p1 = exp2f(sc[nt][1] - ref_lo);
            const float p2 = exp2f(sc[nt][2] - ref_hi), p3 = exp2f(sc[nt][3] - ref_hi);
            sum_lo += p0 + p1;
            sum_hi += p2 + p3;
            p[nt >> 1][(nt & 1) * 2 + 0] = pack_bf16(p0, p1);       // a0 / a2: row g
            p[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);       // a1 / a3: row g+8
        }
        l_lo = l_lo * c_lo + sum_lo;
        l_hi = l_hi * c_hi + sum_hi;
        m_lo = mn_lo;
        m_hi = mn_hi;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            o[i][0] *= c_lo; o[i][1] *= c_lo; o[i][2] *= c_hi; o[i][3] *= c_hi;
        }
        // ---- O += P V
#pragma unroll
        for (int kk = 0; kk < PF_KEYS / 16; ++kk) {
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {               // pairs of 8-dim tiles
                uint32_t b[4];
                ldmatrix_x4_trans(b, &sm->v[s][kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][dp * 16 + 8 * (lane >> 4)]);
                mma_bf16(o[2 * dp], p[kk], b[0], b[1]);
                mma_bf16(o[2 * dp + 1], p[kk], b[2], b[3]);
            }
        }
        __syncthreads();                                        // stage s is free for the load after next
    }
    // the sums of a row are spread over the 4 lanes of its quad
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    const float inv_lo = l_lo > 0.f ? 1.f / l_lo : 0.f, inv_hi = l_hi > 0.f ? 1.f / l_hi : 0.f;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        const int d = i * 8 + 2 * t;
        if (row_lo < rows_here)
            *reinterpret_cast<uint32_t*>(out + ((size_t)(q0 + r0 + row_lo) * nH + head) * HD + d) =
                pack_bf16(o[i][0] * inv_lo, o[i][1] * inv_lo);
        if (row_hi < rows_here)
            *reinterpret_cast<uint32_t*>(out + ((size_t)(q0 + r0 + row_hi) * nH + head) * HD + d) =
                pack_bf16(o[i][2] * inv_hi, o[i][3] * inv_hi);
    }
}

NG_EXPORT int ng_attn_prefill_bf16(const void* q, const void* k_pages, const void* v_pages, const int* table,
                                   int table_stride, const int* cu_q, const int* ctx_before, void* out,
                                   int n_entries, int max_q, int nH, int nKV, int hd, int page_size, int num_pages,
                                   int window, float scale, int skip_single, const float* slopes,
                                   cudaStream_t stream) {
    if (n_entries <= 0 || max_q <= 0) return NG_OK;
    if (hd != HD || nH <= 0 || nKV <= 0 || nH % nKV || page_size <= 0 || (max_q + PF_ROWS - 1) / PF_ROWS > 65535 ||
        n_entries > 65535)
        return NG_BAD_SIZE;
    if (page_size & (page_size - 1)) return NG_BAD_SIZE;       // pages are a power of two of tokens
    int ps_log2 = 0;
    while ((1 << ps_log2) < page_size) ++ps_log2;
    constexpr int TABLE_INTS = 4096;                           // 16 KB: 64k keys of context at 16 per page
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)(sizeof(PrefillSmem) + TABLE_INTS * sizeof(int))) != cudaSuccess)
            return NG_LAUNCH_FAILED;
        attr_set = true;
    }
    dim3 grid(nH, (max_q + PF_ROWS - 1) / PF_ROWS, n_entries);
    NG_LAUNCH((attn_prefill_kernel), grid, PF_THREADS, sizeof(PrefillSmem) + TABLE_INTS * sizeof(int), stream, 
        (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, table, table_stride, cu_q, ctx_before,
        (bf16*)out, nH, nKV, ps_log2, num_pages, window, scale * 1.4426950408889634f, skip_single, TABLE_INTS, slopes);
    return ng_launch_status();
}

// ===================================================================================== decode
#define DC_WARPS 4
#define DC_THREADS (DC_WARPS * 32)
#define DC_TILE 64                      // keys per tile: 16 per warp
#define DC_STAGES (HD <= 64 ? 4 : (HD <= 128 ? 3 : 2))
#define DC_REC (HD + 2)                 // scratch record per (row, head, split): [max, sum, o[HD]] float32

struct DecodeSmem {
    bf16 k[DC_STAGES][DC_TILE][PF_LD];
    bf16 v[DC_STAGES][DC_TILE][PF_LD];
};
static_assert(sizeof(DecodeSmem) >= DC_WARPS * 16 * DC_REC * sizeof(float), "the merge buffer reuses the tiles");

// Gather keys key0..key0+63 of the entry (those inside [key_lo, key_end)) into stage s.
// `ptab` holds the page ids of the block's key range (page index minus `first_page`), in shared
// memory when it fits, else it is the entry's row of the block table itself.  The page size
// is a power of two: page and slot are a shift and a mask.
__device__ __forceinline__ void dc_load_tile(DecodeSmem* sm, int s, const bf16* __restrict__ k_pages,
                                             const bf16* __restrict__ v_pages, const int* __restrict__ ptab,
                                             int first_page, int key0, int key_lo, int key_end, int kvh, int nKV,
                                             int ps_log2, int num_pages) {
    constexpr int CH = HD / 8;
#pragma unroll
    for (int c0 = 0; c0 < DC_TILE * CH; c0 += DC_THREADS) {
        const int c = c0 + threadIdx.x;
        if (DC_TILE * CH % DC_THREADS != 0 && c >= DC_TILE * CH) break;
        const int r = c / CH, ch = c % CH;
        const int key = key0 + r;
        bool ok = key >= key_lo && key < key_end;
        size_t off = 0;
        if (ok) {
            const int page = ptab[(key >> ps_log2) - first_page];
            ok = page >= 0 && page < num_pages;
            off = ((((size_t)(ok ? page : 0) * nKV + kvh) << ps_log2) + (key & ((1 << ps_log2) - 1))) * HD + ch * 8;
        }
        cp_async_16(&sm->k[s][r][ch * 8], k_pages + off, ok);
        cp_async_16(&sm->v[s][r][ch * 8], v_pages + off, ok);
    }
}

// A load that stays where it is written: the query rows are the previous kernel's output, and a plain load through a
// const __restrict__ pointer is one the compiler may start early, above the wait for that kernel (it did, once the
// wait was no longer the kernel's first instruction: the rows of the step before came back).
__device__ __forceinline__ uint32_t ld_b32(const bf16* p) {
    uint32_t v;
    asm volatile("ld.global.cg.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// One block per (KV head, entry, split of the context).  The block walks its keys in 64-key
// tiles that cp.async gathers from the pages into a DC_STAGES-deep ring, so that several
// tiles are in flight while one is computed; each warp owns 16 keys of a tile and keeps its
// own online-softmax state over all query heads of the group (the 16 MMA rows); the four
// states are merged through shared memory at the end.
__global__ void __launch_bounds__(DC_THREADS)
attn_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                   const int* __restrict__ table, int table_stride, const int* __restrict__ cu_q,
                   const int* __restrict__ ctx_before, bf16* __restrict__ out, float* __restrict__ scratch,
                   int nH, int nKV, int ps_log2, int num_pages, int window, float scale_log2, int n_splits,
                   int keys_per_split, int table_in_smem, int n_rows, const float* __restrict__ slopes) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    DecodeSmem* sm = reinterpret_cast<DecodeSmem*>(smem_raw);
    ng_pdl_trigger();
    // What the previous kernel of the step writes is this step's query rows and, in the cache, the key and value at
    // each entry's own position.  The batch description (written by the step's host copy before its first kernel) and
    // the keys and values of earlier positions are older: a block reads them before it waits for that kernel, so that
    // its first tiles are on their way while the kernel before it still runs.
    const int e = blockIdx.y, kvh = blockIdx.x, split = blockIdx.z;
    const int row = cu_q[e];
    if (cu_q[e + 1] - row != 1 || row >= n_rows) {               // not a single-token entry, or a row the caller's buffers do not hold
        ng_pdl_wait();                                           // a launch none of whose blocks waited would end before the kernel
        return;                                                  // before it, and the kernel after it would start on unfinished data
    }
    const int G = nH / nKV;                                      // query heads per KV head (<= 16)
    const int pos = ctx_before[e];
    const int kv_end = pos + 1;
    const int key_lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* trow = table + (size_t)e * table_stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int k_begin = (key_lo / DC_TILE) * DC_TILE + split * keys_per_split;
    const int k_end = min(kv_end, k_begin + keys_per_split);
    const int n_tiles = k_end > k_begin ? (k_end - k_begin + DC_TILE - 1) / DC_TILE : 0;
    // page ids of this block's key range, once, into shared memory
    const int* ptab = trow;
    int first_page = 0;
    if (table_in_smem && n_tiles > 0) {
        int* tab = reinterpret_cast<int*>(smem_raw + sizeof(DecodeSmem));
        first_page = k_begin >> ps_log2;
        const int n_pages = ((k_end - 1) >> ps_log2) - first_page + 1;
        for (int i = threadIdx.x; i < n_pages; i += DC_THREADS) tab[i] = trow[first_page + i];
        ptab = tab;
        __syncthreads();
    }
    // the tile that holds this step's own key (position `pos`), if it is among the ones asked for up front, is not old
    const bool own_key_early = pos >= k_begin && pos < k_begin + (DC_STAGES - 1) * DC_TILE;
    if (own_key_early) ng_pdl_wait();
#pragma unroll
    for (int s = 0; s < DC_STAGES - 1; ++s) {
        if (s < n_tiles)
            dc_load_tile(sm, s, k_pages, v_pages, ptab, first_page, k_begin + s * DC_TILE, key_lo, k_end, kvh, nKV,
                         ps_log2, num_pages);
        cp_async_commit();
    }
    if (!own_key_early) ng_pdl_wait();
    // Q fragments (A operand): rows = the group's query heads, rows >= G are zero
    uint32_t qa[HD / 16][4];
    {
        const bf16* qr_lo = q + ((size_t)row * nH + kvh * G + g) * HD;
        const bf16* qr_hi = qr_lo + (size_t)8 * HD;
#pragma unroll
        for (int b = 0; b < HD / 16; ++b) {
            const int d = 16 * b + 2 * t;
            qa[b][0] = g < G ? ld_b32(qr_lo + d) : 0u;
            qa[b][1] = g + 8 < G ? ld_b32(qr_hi + d) : 0u;
            qa[b][2] = g < G ? ld_b32(qr_lo + d + 8) : 0u;
            qa[b][3] = g + 8 < G ? ld_b32(qr_hi + d + 8) : 0u;
        }
    }
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
    // score bias of the two query heads this lane's accumulator rows belong to (base 2)
    const float slope_lo = slopes && g < G ? slopes[kvh * G + g] * 1.4426950408889634f : 0.f;
    const float slope_hi = slopes && g + 8 < G ? slopes[kvh * G + g + 8] * 1.4426950408889634f : 0.f;

    for (int tile = 0; tile < n_tiles; ++tile) {
        const int nxt = tile + DC_STAGES - 1;
        if (nxt < n_tiles)
            dc_load_tile(sm, nxt % DC_STAGES, k_pages, v_pages, ptab, first_page, k_begin + nxt * DC_TILE, key_lo, k_end,
                         kvh, nKV, ps_log2, num_pages);
        cp_async_commit();
        cp_async_wait<DC_STAGES - 1>();                         // tile `tile` has landed
        __syncthreads();
        const int s = tile % DC_STAGES;
        const int key0 = k_begin + tile * DC_TILE + warp * 16;   // this warp's 16 keys
        if (key0 < k_end) {
            float sc[2][4];
            sc[0][0] = sc[0][1] = sc[0][2] = sc[0][3] = sc[1][0] = sc[1][1] = sc[1][2] = sc[1][3] = 0.f;
#pragma unroll
            for (int kb = 0; kb < HD / 16; ++kb) {
                uint32_t b[4];
                ldmatrix_x4(b, &sm->k[s][warp * 16 + (lane & 7) + 8 * (lane >> 4)][kb * 16 + 8 * ((lane >> 3) & 1)]);
                mma_bf16(sc[0], qa[kb], b[0], b[1]);
                mma_bf16(sc[1], qa[kb], b[2], b[3]);
            }
            float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    const int key = key0 + 8 * j + 2 * t + c;
                    const bool ok = key >= key_lo && key < k_end;
                    sc[j][c] = ok ? fmaf(sc[j][c], scale_log2, -slope_lo * (float)(pos - key)) : -INFINITY;
                    sc[j][2 + c] = ok ? fmaf(sc[j][2 + c], scale_log2, -slope_hi * (float)(pos - key)) : -INFINITY;
                    mx_lo = fmaxf(mx_lo, sc[j][c]);
                    mx_hi = fmaxf(mx_hi, sc[j][2 + c]);
                }
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
            mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
            mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
            const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
            const float ref_lo = mn_lo == -INFINITY ? 0.f : mn_lo, ref_hi = mn_hi == -INFINITY ? 0.f : mn_hi;
            const float c_lo = exp2f(m_lo - ref_lo), c_hi = exp2f(m_hi - ref_hi);
            uint32_t pa[4];
            float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float p0 = exp2f(sc[j][0] - ref_lo), p1 = exp2f(sc[j][1] - ref_lo);
                const float p2 = exp2f(sc[j][2] - ref_hi), p3 = exp2f(sc[j][3] - ref_hi);
                sum_lo += p0 + p1;
                sum_hi += p2 + p3;
                pa[2 * j] = pack_bf16(p0, p1);
                pa[2 * j + 1] = pack_bf16(p2, p3);
            }
            l_lo = l_lo * c_lo + sum_lo;
            l_hi = l_hi * c_hi + sum_hi;
            m_lo = mn_lo;
            m_hi = mn_hi;
#pragma unroll
            for (int dp = 0; dp < HD / 16; ++dp) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, &sm->v[s][warp * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)][dp * 16 + 8 * (lane >> 4)]);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    o[2 * dp][c] *= (c < 2 ? c_lo : c_hi);
                    o[2 * dp + 1][c] *= (c < 2 ? c_lo : c_hi);
                }
                mma_bf16(o[2 * dp], pa, b[0], b[1]);
                mma_bf16(o[2 * dp + 1], pa, b[2], b[3]);
            }
        }
        __syncthreads();                                        // the stage may be refilled
    }
    cp_async_wait<0>();
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    // ---- the warps' partial results -> shared memory (the tiles are free now)
    float (*red)[16][DC_REC] = reinterpret_cast<float (*)[16][DC_REC]>(smem_raw);
    if (t == 0) {
        red[warp][g][0] = m_lo; red[warp][g][1] = l_lo;
        red[warp][g + 8][0] = m_hi; red[warp][g + 8][1] = l_hi;
    }
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        red[warp][g][2 + i * 8 + 2 * t] = o[i][0];
        red[warp][g][2 + i * 8 + 2 * t + 1] = o[i][1];
        red[warp][g + 8][2 + i * 8 + 2 * t] = o[i][2];
        red[warp][g + 8][2 + i * 8 + 2 * t + 1] = o[i][3];
    }
    __syncthreads();
    // ---- merge the warps (fixed order), one thread per (head of the group, dim)
    for (int idx = threadIdx.x; idx < G * HD; idx += DC_THREADS) {
        const int hh = idx / HD, d = idx % HD;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < DC_WARPS; ++w) m = fmaxf(m, red[w][hh][0]);
        float l = 0.f, acc = 0.f;
        if (m > -INFINITY) {
#pragma unroll
            for (int w = 0; w < DC_WARPS; ++w) {
                const float f = exp2f(red[w][hh][0] - m);
                l += red[w][hh][1] * f;
                acc += red[w][hh][2 + d] * f;
            }
        }
        const int head = kvh * G + hh;
        if (n_splits == 1) {
            out[((size_t)row * nH + head) * HD + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
        } else {
            float* rec = scratch + (((size_t)row * nH + head) * n_splits + split) * DC_REC;
            rec[2 + d] = acc;
            if (d == 0) { rec[0] = m; rec[1] = l; }
        }
    }
}

// out[row, head, :] = sum_s o_s * 2^(m_s - m) / sum_s l_s * 2^(m_s - m), splits in ascending order
__global__ void attn_combine_kernel(const float* __restrict__ scratch, const int* __restrict__ cu_q,
                                    bf16* __restrict__ out, int nH, int n_splits, int n_rows) {
    ng_pdl_trigger();
    const int e = blockIdx.y, head = blockIdx.x;
    const int row = cu_q[e];                                     // the batch description: older than the step's kernels
    const bool mine = cu_q[e + 1] - row == 1 && row < n_rows;
    ng_pdl_wait();
    if (!mine) return;
    scratch = ng_after_wait(scratch);
    const float* rec = scratch + ((size_t)row * nH + head) * n_splits * DC_REC;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, rec[(size_t)s * DC_REC]);
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float l = 0.f, acc = 0.f;
        if (m > -INFINITY) {
            for (int s = 0; s < n_splits; ++s) {
                const float f = exp2f(rec[(size_t)s * DC_REC] - m);
                l += rec[(size_t)s * DC_REC + 1] * f;
                acc += rec[(size_t)s * DC_REC + 2 + d] * f;
            }
        }
        out[((size_t)row * nH + head) * HD + d] = __float2bfloat16_rn(l > 0.f ? acc / l : 0.f);
    }
}

// n_rows: rows that q, out and the scratch hold; an entry whose row (read from cu_q on the device) lies
// beyond them is skipped
static int attn_decode_launch(const void* q, const void* k_pages, const void* v_pages, const int* table,
                              int table_stride, const int* cu_q, const int* ctx_before, void* out,
                              float* scratch, int n_rows, int n_entries, int nH, int nKV, int hd, int page_size,
                              int num_pages, int window, float scale, int n_splits, int max_ctx,
                              const float* slopes, cudaStream_t stream) {
    if (n_entries <= 0) return NG_OK;
    if (hd != HD || nH <= 0 || nKV <= 0 || nH % nKV || nH / nKV > 16 || page_size <= 0 || n_splits < 1 ||
        n_splits > 65535 || n_entries > 65535 || (n_splits > 1 && !scratch))
        return NG_BAD_SIZE;
    // keys a split covers: the visible range (at most max_ctx keys, +63 for the rounding of its
    // start) cut into n_splits runs of whole 64-key tiles
    const int span = (window > 0 ? min(window, max_ctx) : max_ctx) + DC_TILE;
    int per = (span + n_splits - 1) / n_splits;
    per = ((per + DC_TILE - 1) / DC_TILE) * DC_TILE;
    if (page_size & (page_size - 1)) return NG_BAD_SIZE;       // pages are a power of two of tokens
    int ps_log2 = 0;
    while ((1 << ps_log2) < page_size) ++ps_log2;
    const size_t tab_bytes = ((size_t)per / page_size + 2) * sizeof(int);
    const int table_in_smem = tab_bytes <= 16 * 1024;
    const size_t smem = sizeof(DecodeSmem) + (table_in_smem ? tab_bytes : 0);
    static size_t smem_set = 0;
    if (smem > smem_set) {
        if (cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)(sizeof(DecodeSmem) + 16 * 1024)) != cudaSuccess)
            return NG_LAUNCH_FAILED;
        smem_set = sizeof(DecodeSmem) + 16 * 1024;
    }
    dim3 grid(nKV, n_entries, n_splits);
    NG_LAUNCH((attn_decode_kernel), grid, DC_THREADS, smem, stream, 
        (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, table, table_stride, cu_q, ctx_before,
        (bf16*)out, scratch, nH, nKV, ps_log2, num_pages, window, scale * 1.4426950408889634f, n_splits, per,
        table_in_smem, n_rows, slopes);
    if (n_splits > 1)
        NG_LAUNCH((attn_combine_kernel), dim3(nH, n_entries), HD >= 128 ? 128 : 64, 0, stream, scratch, cu_q, (bf16*)out, nH,
                                                                                   n_splits, n_rows);
    return ng_launch_status();
}

// scratch: n_rows * nH * n_splits * (HD + 2) floats, n_rows = rows of q (unused when n_splits == 1)
NG_EXPORT int ng_attn_decode_bf16(const void* q, const void* k_pages, const void* v_pages, const int* table,
                                  int table_stride, const int* cu_q, const int* ctx_before, void* out,
                                  float* scratch, int n_entries, int nH, int nKV, int hd, int page_size,
                                  int num_pages, int window, float scale, int n_splits, int max_ctx,
                                  const float* slopes, cudaStream_t stream) {
    return attn_decode_launch(q, k_pages, v_pages, table, table_stride, cu_q, ctx_before, out, scratch, 0x7fffffff,
                              n_entries, nH, nKV, hd, page_size, num_pages, window, scale, n_splits, max_ctx, slopes,
                              stream);
}

NG_EXPORT int ng_attn_decode_scratch_floats(int n_rows, int nH, int n_splits) {
    return n_splits > 1 ? n_rows * nH * n_splits * DC_REC : 0;
}

// ===================================================================================== no-allocation variant
// See ng_noalloc.h: the same decode attention with its split scratch inside the library.
#include <mutex>

#include "ng_noalloc.h"

static __device__ __align__(256) float ng_noalloc_scratch[NG_NOALLOC_SCRATCH_FLOATS];

#define NG_NOALLOC_MAX_DEVICES 64
static float* g_noalloc_ptr[NG_NOALLOC_MAX_DEVICES];     // device address of the array, per device
static std::mutex g_noalloc_mutex;

// In host code `ng_noalloc_scratch` is only a handle for the runtime, not a device address:
// the address a kernel can use comes from cudaGetSymbolAddress, asked once per device with
// that device current.
static int noalloc_scratch_address(float** ptr) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NG_NOALLOC_MAX_DEVICES) return NG_NOALLOC_SETUP_FAILED;
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (!g_noalloc_ptr[dev]) {
        float* p = nullptr;
        if (cudaGetSymbolAddress((void**)&p, ng_noalloc_scratch) != cudaSuccess || !p) {
            cudaGetLastError();
            return NG_NOALLOC_SETUP_FAILED;
        }
        g_noalloc_ptr[dev] = p;
    }
    *ptr = g_noalloc_ptr[dev];
    return NG_OK;
}

NG_EXPORT int ng_attn_decode_noalloc_max_floats(void) { return NG_NOALLOC_SCRATCH_FLOATS; }

NG_EXPORT int ng_attn_decode_bf16_noalloc(const void* q, const void* k_pages, const void* v_pages, const int* table,
                                          int table_stride, const int* cu_q, const int* ctx_before, void* out,
                                          int n_rows, int n_entries, int nH, int nKV, int hd, int page_size,
                                          int num_pages, int window, float scale, int n_splits, int max_ctx,
                                          cudaStream_t stream) {
    if (n_entries <= 0) return NG_OK;
    if (n_rows <= 0 || nH <= 0 || n_splits < 1) return NG_BAD_SIZE;
    const long long need = n_splits > 1 ? (long long)n_rows * nH * n_splits * DC_REC : 0;
    if (need > NG_NOALLOC_SCRATCH_FLOATS) return NG_NOALLOC_TOO_LARGE;
    float* scratch = nullptr;
    const int rc = noalloc_scratch_address(&scratch);
    if (rc != NG_OK) return rc;
    // the kernels read each entry's row from cu_q on the device: they are told n_rows, the rows that
    // the capacity check above counted, and skip an entry whose row lies beyond them
    return attn_decode_launch(q, k_pages, v_pages, table, table_stride, cu_q, ctx_before, out, scratch, n_rows,
                              n_entries, nH, nKV, hd, page_size, num_pages, window, scale, n_splits, max_ctx, nullptr,
                              stream);
}

// bfloat16 matrix product on the Blackwell tensor cores:  C[M,N] = X[M,K] * W[N,K]^T
//
// tcgen05.mma with the accumulator in tensor memory, operands staged in shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle), an mbarrier pipeline between one producer thread
// and one MMA-issuing thread, and tcgen05.ld for the epilogue.
//
// The weight matrix is the MMA's M operand (128 rows of W per block) and the tokens are its N
// operand (a tile of TN = 16..256 tokens), so the same kernel serves decode, where M is a
// handful of tokens and the job is to stream W once at memory speed, and prefill, where both
// extents are large.  Both operands are K-major, which is how activations [M,K] and weights
// [N,K] already lie in memory: no transposes.  An optional split of K over blockIdx.z writes
// float32 partial sums that the consumer (the residual-add + norm kernel) adds up.
//
// Epilogues: bf16 store (+ bias), float32 store (logits, partial sums), and SwiGLU: the block's
// 128 MMA rows are 64 gate rows and the 64 matching up rows (two TMA boxes), the up half of the
// accumulator crosses to the gate half's warps through shared memory, and silu(gate) * up is
// stored, so the [M, 2I] intermediate never exists.
//
// EPI_RED serves steps of few tokens, where a kernel launch costs as much as the product itself:
// the epilogue adds the (split-K) product into the float32 residual stream with red.global.add,
// so no kernel runs after it to add partial sums; the order of those float32 additions is not
// fixed.
//
// Every wait on an mbarrier is bounded: after NG_SPIN_LIMIT polls the waiter records a code in
// the status word and the block runs to its end (tensor memory is always released).
//
// The reference calls cuBLAS for every contraction (gpu/cuda/matmul.cu:316-355) and has no
// tensor-core code of its own.
#include "sm100_common.cuh"

// ------------------------------------------------------------------------------------- kernel
struct GemmParams {
    void* out;                 // bf16 [M, ldc] | float [splits][M, ldc]
    const bf16* bias;          // [N] or null (EPI_BF16 only)
    int* status;
    int M, N, K;               // N = rows of W that produce outputs (for SwiGLU: the intermediate size I)
    int ldc;
    int kb_per_split;          // K blocks (of BLOCK_K) per blockIdx.z
    int up_row_offset;         // SwiGLU: W row of up(i) = up_row_offset + i
    int rows;                  // output columns (rows of W) per block: <= 128, SwiGLU <= 64; chosen so that the
                               // blocks fill the SMs evenly
    int w_bytes;               // bytes of W a stage receives (rows, or 2 * rows for SwiGLU, times 128)
    int red_v4;                // EPI_RED: four columns per atomic (N, ldc multiples of 4, out 16-byte aligned)
};

template <int TN, int EPI>
struct Cfg {
    static constexpr int W_BYTES = BLOCK_W * BLOCK_K * 2;
    static constexpr int X_BYTES = TN * BLOCK_K * 2;
    static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
    // up to 6 stages; small token tiles then leave room for two blocks per SM, whose pipelines overlap
    static constexpr int STAGES = (200 * 1024 / STAGE_BYTES) > NG_MAX_STAGES ? NG_MAX_STAGES : (200 * 1024 / STAGE_BYTES);
    static constexpr int TMEM_COLS = TN < 32 ? 32 : TN;                     // a power of two >= 32
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;
    static_assert(TN % 16 == 0 && TN >= 16 && TN <= 256, "token tile must be a multiple of 16 in [16, 256]");
    static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "tensor memory columns: a power of two");
    static_assert(STAGES >= 2, "pipeline needs two stages");
};

// Transposes the 4 x 4 block that the four lanes of a quad hold (lane i: a0..a3 = row 0..3 of its
// column) so that lane i holds row i of the quad's four columns.
__device__ __forceinline__ void quad_transpose(float& a0, float& a1, float& a2, float& a3, int lane) {
    const bool odd = lane & 1, hi = lane & 2;
    float t;
    t = __shfl_xor_sync(0xffffffffu, odd ? a0 : a1, 1); if (odd) a0 = t; else a1 = t;
    t = __shfl_xor_sync(0xffffffffu, odd ? a2 : a3, 1); if (odd) a2 = t; else a3 = t;
    t = __shfl_xor_sync(0xffffffffu, hi ? a0 : a2, 2); if (hi) a0 = t; else a2 = t;
    t = __shfl_xor_sync(0xffffffffu, hi ? a1 : a3, 2); if (hi) a1 = t; else a3 = t;
}
__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" :: "l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

template <int TN, int EPI>
__global__ void __launch_bounds__(128)
gemm_sm100_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                  const GemmParams p) {
    using C = Cfg<TN, EPI>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty = full + C::STAGES;
    uint64_t* accum_ready = empty + C::STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_ready + 1);

    ng_pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int w_row0 = blockIdx.x * p.rows;                  // first output column (row of W) of this block
    const int m0 = blockIdx.y * TN;                          // first token
    const int kb0 = blockIdx.z * p.kb_per_split;
    const int total_kb = (p.K + BLOCK_K - 1) / BLOCK_K;
    const int num_kb = min(p.kb_per_split, total_kb - kb0);  // >= 1 by construction of the grid

    // The weights are constants: the first stages' W tiles are requested at once, by the lane that made the barriers,
    // before the block meets, before tensor memory is there and before the wait on the previous kernel: the stream
    // of W starts while that kernel still runs.  The token operand is its output and is read after the wait.
    const int pre = min(num_kb, C::STAGES);
    constexpr uint32_t X_TX = C::X_BYTES;
    uint32_t elected;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(elected));
    const bool leader = elected != 0;
    if (warp == 0 && leader) {
        asm volatile("prefetch.tensormap [%0];" :: "l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" :: "l"(&map_x) : "memory");
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(accum_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        for (int i = 0; i < pre; ++i) {
            unsigned char* st = tiles + i * C::STAGE_BYTES;
            mbar_expect_tx(&full[i], p.w_bytes + X_TX);
            const int k = (kb0 + i) * BLOCK_K;
            tma_load_2d(st, &map_w, &full[i], k, w_row0);      // map_w has boxes of p.rows rows
            if (EPI == EPI_SWIGLU) tma_load_2d(st + C::W_BYTES / 2, &map_w, &full[i], k, p.up_row_offset + w_row0);
        }
    }
    if (warp == 1) {                                          // one warp allocates tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(tmem_slot)), "r"((uint32_t)C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    // Warp 0 asks for the tiles, warp 1 issues the MMAs.  Each runs its loop and its waits in all lanes and lets one
    // elected lane issue: addresses, coordinates and descriptors are then the same in every lane and stay in uniform
    // registers, which the TMA and MMA instructions read; computed by a lone lane they cost a move per operand.
    if (warp == 0) {
        // ------------------------------------------------------------ producer: TMA loads
        ng_pdl_wait();
        if (leader) {
            for (int i = 0; i < pre; ++i)
                tma_load_2d(tiles + i * C::STAGE_BYTES + C::W_BYTES, &map_x, &full[i], (kb0 + i) * BLOCK_K, m0);
        }
        __syncwarp();
        for (int i = pre; i < num_kb && ok; ++i) {
            const int s = i % C::STAGES;
            ok = __all_sync(0xffffffffu, mbar_wait(&empty[s], ((i / C::STAGES) & 1) ^ 1));      // one answer for the warp
            if (!ok) break;
            unsigned char* st = tiles + s * C::STAGE_BYTES;
            const int k = (kb0 + i) * BLOCK_K;
            if (leader) {
                mbar_expect_tx(&full[s], p.w_bytes + X_TX);
                tma_load_2d(st, &map_w, &full[s], k, w_row0);
                if (EPI == EPI_SWIGLU) tma_load_2d(st + C::W_BYTES / 2, &map_w, &full[s], k, p.up_row_offset + w_row0);
                tma_load_2d(st + C::W_BYTES, &map_x, &full[s], k, m0);
            }
            __syncwarp();
        }
        if (!ok && leader) atomicOr(p.status, NG_STATUS_GEMM_TIMEOUT);
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc = make_idesc(TN);
        for (int i = 0; i < num_kb && ok; ++i) {
            const int s = i % C::STAGES;
            ok = __all_sync(0xffffffffu, mbar_wait(&full[s], (i / C::STAGES) & 1));
            if (!ok) break;
            tcgen05_fence_after();
            unsigned char* st = tiles + s * C::STAGE_BYTES;
            const uint64_t da = make_desc_sw128(st), db = make_desc_sw128(st + C::W_BYTES);
            if (leader) {
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                    const uint64_t koff = (uint64_t)((k * UMMA_K * 2) >> 4);  // 32 bytes per K step, in 16-byte units
                    tcgen05_mma_f16(tmem_base, da + koff, db + koff, idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                tcgen05_commit(&empty[s]);                      // frees the stage when these MMAs have read it
            }
            __syncwarp();
        }
        if (leader) {
            if (ok) tcgen05_commit(accum_ready);
            else atomicOr(p.status, NG_STATUS_GEMM_TIMEOUT);
        }
    }
    __syncwarp();
    // ---------------------------------------------------------------- epilogue: all four warps
    ng_pdl_wait();                                              // before this block writes global memory
    bool ready = mbar_wait(accum_ready, 0);
    ready = __all_sync(0xffffffffu, ready);
    tcgen05_fence_after();
    const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
    if (EPI == EPI_SWIGLU) {
        // lanes 0..63 hold gate(n), lanes 64..127 hold up(n) for n = w_row0 + (lane & 63).  The
        // pipeline's shared memory is free now (every MMA has completed): the up half passes
        // through it, 16 tokens at a time.
        // Both halves work: for tokens 0..7 of a 16-token chunk the up half sends its values to
        // the gate half, for tokens 8..15 the gate half sends to the up half; each thread then
        // gates and stores 8 tokens of its column.
        float (*xch)[17] = reinterpret_cast<float (*)[17]>(tiles);        // [128 lanes][16 tokens]
        const int col = (warp & 1) * 32 + lane;                 // column of the block: gate lane col, up lane 64 + col
        const int n = w_row0 + col;
        const bool up_half = warp >= 2;
        const int tl = warp * 32 + lane;                        // this thread's TMEM lane
        const int peer = up_half ? tl - 64 : tl + 64;
        const int j0 = up_half ? 8 : 0;                         // tokens of the chunk this thread finishes
#pragma unroll 1
        for (int c = 0; c < TN; c += 16) {
            float v[16];
            if (ready) tmem_ld16(lane_addr + c, v);
#pragma unroll
            for (int j = 0; j < 8; ++j) xch[tl][(8 - j0) + j] = up_half ? v[j] : v[8 + j];   // what the peer finishes
            __syncthreads();
            if (ready && col < p.rows && n < p.N) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int m = m0 + c + j0 + j;
                    if (m < p.M) {
                        const float mine = up_half ? v[8 + j] : v[j], theirs = xch[peer][j0 + j];
                        // the unfused path rounds both products to bf16 before the gate: keep that rounding
                        const float g = __bfloat162float(__float2bfloat16_rn(up_half ? theirs : mine));
                        const float u = __bfloat162float(__float2bfloat16_rn(up_half ? mine : theirs));
                        reinterpret_cast<bf16*>(p.out)[(size_t)m * p.ldc + n] = __float2bfloat16_rn(silu_fast(g) * u);
                    }
                }
            }
            __syncthreads();
        }
    } else if (ready) {
        const int col = warp * 32 + lane;
        const int n = w_row0 + col;                             // this thread's output column
#pragma unroll 1
        for (int c = 0; c < TN; c += 16) {
            float v[16];
            tmem_ld16(lane_addr + c, v);
            if (EPI == EPI_RED && p.red_v4) {
                // an atomic add costs the same for one float as for four: the lanes of a quad trade
                // values so that each holds four neighbouring columns of one token, and adds them at once
#pragma unroll
                for (int g = 0; g < 4; ++g) quad_transpose(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3], lane);
                const int qcol = warp * 32 + (lane & ~3), n0 = w_row0 + qcol;
                if (qcol < p.rows && n0 < p.N) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const int m = m0 + c + 4 * g + (lane & 3);
                        if (m < p.M)
                            red_add_v4(reinterpret_cast<float*>(p.out) + (size_t)m * p.ldc + n0, v[4 * g], v[4 * g + 1],
                                       v[4 * g + 2], v[4 * g + 3]);
                    }
                }
                continue;
            }
            if (col < p.rows && n < p.N) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int m = m0 + c + j;
                    if (m < p.M) {
                        if (EPI == EPI_F32) {
                            reinterpret_cast<float*>(p.out)[((size_t)blockIdx.z * p.M + m) * p.ldc + n] = v[j];
                        } else if (EPI == EPI_RED) {
                            atomicAdd(reinterpret_cast<float*>(p.out) + (size_t)m * p.ldc + n, v[j]);
                        } else {
                            const float b = p.bias ? __bfloat162float(p.bias[n]) : 0.f;
                            reinterpret_cast<bf16*>(p.out)[(size_t)m * p.ldc + n] = __float2bfloat16_rn(v[j] + b);
                        }
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)C::TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------------- host
template <int TN, int EPI>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, dim3 grid, cudaStream_t stream) {
    using C = Cfg<TN, EPI>;
    static bool attr = false;
    if (!attr) {
        if (cudaFuncSetAttribute(gemm_sm100_kernel<TN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) != cudaSuccess)
            return NG_LAUNCH_FAILED;
        attr = true;
    }
    NG_LAUNCH((gemm_sm100_kernel<TN, EPI>), grid, 128, C::SMEM, stream, mw, mx, p);
    return ng_launch_status();
}

template <int EPI>
static int dispatch_tn(int tn, const CUtensorMap& mw, const CUtensorMap& mx, const GemmParams& p, dim3 grid,
                       cudaStream_t stream) {
    switch (tn) {
        case 16: return launch<16, EPI>(mw, mx, p, grid, stream);
        case 32: return launch<32, EPI>(mw, mx, p, grid, stream);
        case 64: return launch<64, EPI>(mw, mx, p, grid, stream);
        case 128: return launch<128, EPI>(mw, mx, p, grid, stream);
        case 256: return launch<256, EPI>(mw, mx, p, grid, stream);
    }
    return NG_BAD_SIZE;
}

// x [M,K] bf16, w [n_w_rows,K] bf16 (both row-major, 16-byte aligned, K % 8 == 0).
//   epi 0: out bf16 [M, ldc] = x w^T (+ bias)              N = n_w_rows, splits must be 1
//   epi 1: out float [splits][M, ldc] = partial x w^T      N = n_w_rows
//   epi 2: out bf16 [M, ldc] = silu(x wg^T) * (x wu^T)     wg = w rows [0, N), wu = w rows [up_row_offset, +N)
//   epi 3: out float [M, ldc] += x w^T (atomic adds; any splits)
// tn: token tile (16, 32, 64, 128, 256; 0 = chosen from M).
NG_EXPORT int ng_gemm_sm100(const void* x, const void* w, const void* bias, void* out, int M, int N, int K,
                            int n_w_rows, int ldc, int epi, int splits, int up_row_offset, int tn, int* status,
                            cudaStream_t stream) {
    if (M <= 0 || N <= 0) return NG_OK;
    if (K <= 0 || K % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ldc < N || splits < 1 || !status)
        return NG_BAD_SIZE;
    if (epi < 0 || epi > 3 || ((epi == EPI_BF16 || epi == EPI_SWIGLU) && splits != 1) ||
        (epi == EPI_SWIGLU && up_row_offset + N > n_w_rows))
        return NG_BAD_SIZE;
    if (tn == 0) tn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
    if (splits > total_kb) splits = total_kb;
    const int per = (total_kb + splits - 1) / splits;
    splits = (total_kb + per - 1) / per;                      // every blockIdx.z gets at least one K block
    CUtensorMap mw, mx;
    const int rows = ng_plan_rows(M, N, epi, splits);
    const int w_bytes = (epi == EPI_SWIGLU ? 2 : 1) * rows * BLOCK_K * 2;
    if (!tensor_map(w, n_w_rows, K, rows, &mw)) return NG_LAUNCH_FAILED;
    if (!tensor_map(x, M, K, tn, &mx)) return NG_LAUNCH_FAILED;
    const int red_v4 = epi == EPI_RED && N % 4 == 0 && ldc % 4 == 0 && rows % 4 == 0 && ((uintptr_t)out & 15) == 0;
    GemmParams p{out, (const bf16*)bias, status, M, N, K, ldc, per, up_row_offset, rows, w_bytes, red_v4};
    dim3 grid((N + rows - 1) / rows, (M + tn - 1) / tn, splits);
    if (grid.y > 65535 || grid.z > 65535) return NG_BAD_SIZE;
    switch (epi) {
        case EPI_BF16: return dispatch_tn<EPI_BF16>(tn, mw, mx, p, grid, stream);
        case EPI_F32: return dispatch_tn<EPI_F32>(tn, mw, mx, p, grid, stream);
        case EPI_RED: return dispatch_tn<EPI_RED>(tn, mw, mx, p, grid, stream);
        default: return dispatch_tn<EPI_SWIGLU>(tn, mw, mx, p, grid, stream);
    }
}

// splits the launcher will really use for (K, asked) -- the consumer of partial sums needs it
NG_EXPORT int ng_gemm_sm100_splits(int K, int splits) {
    const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
    if (splits > total_kb) splits = total_kb;
    if (splits < 1) splits = 1;
    const int per = (total_kb + splits - 1) / splits;
    return (total_kb + per - 1) / per;
}

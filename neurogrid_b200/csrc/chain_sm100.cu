// A chain of dependent few-token operations in ONE persistent kernel: products on the tensor
// cores (tcgen05 / TMA / TMEM, the pipeline of gemm_sm100.cu), RMSNorm and the one-token short
// convolution, separated by barriers across the grid instead of kernel boundaries.
//
// Why: a decode step of a handful of tokens is a stream of the weights, cut into about a hundred
// dependent operations of a few microseconds each.  As separate kernels every cut costs the
// stream its start-up again (the launch, the first loads' latency, the drained pipeline at the
// end).  Here one block per SM lives through the whole chain:
//   * the producer thread keeps the shared-memory ring full of weight tiles ACROSS operations
//     (weights depend on nothing), so memory keeps streaming while an operation ends, the grid
//     meets at the barrier and the next operation's token operand is read;
//   * only the token operand of an operation waits for the barrier after the operation that
//     made it (a counter in global memory, release/acquire);
//   * the accumulator is double-buffered in tensor memory, so the epilogue of one tile overlaps
//     the products of the next.
//
// Roles in a block of 192 threads: warp 0 / lane 0 issues TMA loads, warp 1 / lane 0 issues the
// MMAs (warp 1 also owns the tensor-memory allocation), warps 2..5 run the epilogues, the norms
// and the convolutions and meet the other blocks at the barrier after every operation.
//
// Operations (ChainOp, filled by the host):
//   GEMM  out = x w^T for M <= TN tokens; epilogues as in gemm_sm100.cu: float32 partial sums per
//         K split, red.global.add into the float32 residual stream, SwiGLU on 64 gate + 64 up rows
//   NORM  x[i] = rmsnorm(h[rows ? rows[i] : i]) * w   (float32 in, bfloat16 out)
//   CONV  the gated short convolution for entries that bring one token, from the float32 partial
//         sums of in_proj; state slots as in shortconv.cu
//
// Every wait is bounded (mbarrier waits, barrier polls): on a timeout the block records a bit in
// the status word, raises a flag that all its roles watch, and runs to its end; the other
// blocks' waits then run out the same way.  Tensor memory is always released.
//
// The reference runs every one of these operations as a kernel of its own or a cuBLAS call
// (gpu/engine/conv_layer.cu:215-345, gpu/engine/layer.cu:1650-1770).
#include "sm100_common.cuh"

enum { OP_GEMM = 0, OP_NORM = 1, OP_CONV = 2 };
#define CHAIN_THREADS 192
#define CHAIN_EPI_THREADS 128
#define CHAIN_MAX_OPS 64
#define CHAIN_POLL_LIMIT (1u << 21)
#define NG_STATUS_CHAIN_TIMEOUT 32

struct ChainOp {                 // 160 bytes; the host packs it field by field
    unsigned long long p[8];     // GEMM: p0 out
                                 // NORM: p0 h, p1 weight, p2 out, p3 rows (int32) or 0
                                 // CONV: p0 in_proj output (float32 partial sums, or bfloat16 when n_part = 0), p1 conv weight, p2 conv bias or 0, p3 state, p4 out,
                                 //       p5 cu_q, p6 ctx_before, p7 slots
    int type, M, N, K;           // M: tokens (GEMM), rows out (NORM), entries (CONV)
    int rows, n_tiles, splits, kb_per_split;
    int epi, ldc, up_row_offset, w_bytes;
    int w_map, x_map, H, L;
    int n_part, flags;
    long long pstride;
    float eps;
    int pad[3];
};
static_assert(sizeof(ChainOp) == 160, "the host packs 160 bytes per operation");

template <int TN>
struct ChainCfg {
    static constexpr int W_BYTES = BLOCK_W * BLOCK_K * 2;
    static constexpr int X_BYTES = TN * BLOCK_K * 2;
    static constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
    static constexpr int STAGES = TN <= 16 ? 10 : TN <= 32 ? 9 : 7;
    static constexpr int ACC_COLS = TN < 32 ? 32 : TN;
    static constexpr int TMEM_COLS = 2 * ACC_COLS;                       // two accumulators
    static constexpr int XCH_BYTES = 128 * 17 * 4;
    static constexpr int OPS_BYTES = CHAIN_MAX_OPS * (int)sizeof(ChainOp);
    static constexpr int SMEM = STAGES * STAGE_BYTES + XCH_BYTES + OPS_BYTES + 1024 /*alignment*/ + 512 /*barriers*/;
    static_assert(TN == 16 || TN == 32 || TN == 64, "token tile of the chain kernel");
    static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS >= 32 && TMEM_COLS <= 512, "tensor memory columns");
    static_assert(SMEM <= 227 * 1024, "shared memory of one block");
};

// -DCHAIN_TRACE: block CHAIN_TRACE_CTA (default 0) stamps its SM clock at the stations of every
// operation into a device array that ng_chain_trace copies out; for finding where the time of an
// operation goes.  Not compiled otherwise.
#ifdef CHAIN_TRACE
#ifndef CHAIN_TRACE_CTA
#define CHAIN_TRACE_CTA 0
#endif
__device__ long long g_chain_trace[CHAIN_MAX_OPS * 16];
#define TRACE(op, station) do { if (blockIdx.x == CHAIN_TRACE_CTA) g_chain_trace[(op) * 16 + (station)] = clock64(); } while (0)
#else
#define TRACE(op, station) do { } while (0)
#endif

// ------------------------------------------------------------------------------------- helpers
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
// test_wait returns at once; try_wait may suspend the thread for a while when the phase is not
// complete, which a loop that has something else to look at must not do
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Bounded mbarrier wait that also gives up when another role of the block has raised the flag.
__device__ __forceinline__ bool mbar_wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    for (uint32_t i = 0; i < NG_SPIN_LIMIT; ++i) {
        if (mbar_try(bar, parity)) return true;
        if ((i & 1023) == 1023 && *abort_flag) return false;
    }
    return false;
}

// The K blocks of the split that task `task` of operation `o` covers.
__device__ __forceinline__ void task_range(const ChainOp& o, int task, int& tile, int& kb0, int& nkb) {
    tile = task % o.n_tiles;
    const int split = task / o.n_tiles;
    const int total_kb = (o.K + BLOCK_K - 1) / BLOCK_K;
    kb0 = split * o.kb_per_split;
    nkb = min(o.kb_per_split, total_kb - kb0);
}

// A position in the sequence of (operation, task, K block) that a block owns, with what the
// producer needs of the task kept in registers: moving on by one K block costs a few
// instructions, only a new task looks at the operation records again.
struct Cursor {
    int op, task, kb, nkb;          // kb counts from 0 within the task
    int k0, r0, up_r0, w_bytes;     // first K element, first W row (and first up row for SwiGLU), bytes of W per stage
    const CUtensorMap* wmap;
    const CUtensorMap* xmap;
    bool more;
};
__device__ __forceinline__ void cursor_seek(Cursor& c, const ChainOp* ops, const CUtensorMap* maps, int n_ops, int cta, int G) {
    // finds the first task at or after (c.op, c.task) that exists; c.kb = 0
    while (c.op < n_ops) {
        const ChainOp& o = ops[c.op];
        if (o.type == OP_GEMM && c.task < o.n_tiles * o.splits) {
            int tile, kb0;
            task_range(o, c.task, tile, kb0, c.nkb);
            c.kb = 0;
            c.k0 = kb0 * BLOCK_K;
            c.r0 = tile * o.rows;
            c.up_r0 = o.epi == EPI_SWIGLU ? o.up_row_offset + c.r0 : -1;
            c.w_bytes = o.w_bytes;
            c.wmap = maps + o.w_map;
            c.xmap = maps + o.x_map;
            c.more = true;
            return;
        }
        ++c.op;
        c.task = cta;
    }
    c.more = false;
}
__device__ __forceinline__ void cursor_next(Cursor& c, const ChainOp* ops, const CUtensorMap* maps, int n_ops, int cta, int G) {
    if (++c.kb < c.nkb) return;
    c.task += G;
    cursor_seek(c, ops, maps, n_ops, cta, G);
}

// ------------------------------------------------------------------------------------- kernel
template <int TN>
__global__ void __launch_bounds__(CHAIN_THREADS, 1)
chain_sm100_kernel(const CUtensorMap* __restrict__ maps, const ChainOp* __restrict__ g_ops, int n_ops,
                   unsigned* __restrict__ counters, int* __restrict__ status) {
    using C = ChainCfg<TN>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float (*xch)[17] = reinterpret_cast<float (*)[17]>(tiles + C::STAGES * C::STAGE_BYTES);
    ChainOp* ops = reinterpret_cast<ChainOp*>(reinterpret_cast<unsigned char*>(xch) + C::XCH_BYTES);
    uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<unsigned char*>(ops) + C::OPS_BYTES);
    uint64_t* empty = full + C::STAGES;
    uint64_t* acc_ready = empty + C::STAGES;
    uint64_t* acc_free = acc_ready + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* epi_abort = abort_flag + 1;                             // the flag as the epilogue threads agreed to see it
    float* red = reinterpret_cast<float*>(tmem_slot + 4);                 // 4 floats: the norm's block sum

    ng_pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int G = gridDim.x, cta = blockIdx.x;

    // the operations are constants of the launch: every role reads them from shared memory
    for (int i = threadIdx.x; i < n_ops * (int)(sizeof(ChainOp) / 16); i += CHAIN_THREADS)
        reinterpret_cast<uint4*>(ops)[i] = reinterpret_cast<const uint4*>(g_ops)[i];
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_ready[b], 1); mbar_init(&acc_free[b], 1); }
        *abort_flag = 0;
        *epi_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     :: "r"(smem_u32(tmem_slot)), "r"((uint32_t)C::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (threadIdx.x == 0) {
        // ------------------------------------------------------------ producer: TMA loads
        // Two cursors over the same sequence of (operation, task, K block): W tiles run ahead as
        // far as the ring allows, the token tile of a slot follows once its operation's input
        // is complete (the barrier after the operation before it, or the previous kernel).
        Cursor wi, xi;
        wi.op = 0; wi.task = cta; xi.op = 0; xi.task = cta;
        cursor_seek(wi, ops, maps, n_ops, cta, G);
        cursor_seek(xi, ops, maps, n_ops, cta, G);
        uint32_t wn = 0, xn = 0, idle = 0;
        uint32_t ws = 0, wphase = 1, xs = 0;                  // stage and parity of the W cursor, stage of the X cursor
        unsigned seen = 0;
        int gate_open = -1;                                    // operations up to this index may read their input
        bool dep_waited = false;
        while (xi.more) {
            bool progress = false;
            if (wi.more && mbar_test(&empty[ws], wphase)) {
                unsigned char* st = tiles + ws * C::STAGE_BYTES;
                mbar_expect_tx(&full[ws], wi.w_bytes + C::X_BYTES);
                const int k = wi.k0 + wi.kb * BLOCK_K;
                tma_load_2d(st, wi.wmap, &full[ws], k, wi.r0);
                if (wi.up_r0 >= 0) tma_load_2d(st + C::W_BYTES / 2, wi.wmap, &full[ws], k, wi.up_r0);
                ++wn;
                if (++ws == C::STAGES) { ws = 0; wphase ^= 1; }
                cursor_next(wi, ops, maps, n_ops, cta, G);
                progress = true;
            }
            if (xn < wn) {
                if (xi.op > gate_open) {
                    // what operation xi.op reads is complete when the previous kernel is (waited for once,
                    // when no weight tile can be requested meanwhile) and every block has passed the
                    // barrier after operation xi.op - 1
                    if (!dep_waited && !progress) { ng_pdl_wait(); dep_waited = true; }
                    if (dep_waited) {
                        const unsigned target = (unsigned)G * (unsigned)xi.op;
                        if (seen < target) seen = ld_acquire(counters);
                        if (seen >= target) {
                            asm volatile("fence.proxy.async;" ::: "memory");   // those writes before this thread's TMA reads
                            gate_open = xi.op;
                            TRACE(xi.op, 0);
                        }
                    }
                }
                if (xi.op <= gate_open) {
                    tma_load_2d(tiles + xs * C::STAGE_BYTES + C::W_BYTES, xi.xmap, &full[xs], xi.k0 + xi.kb * BLOCK_K, 0);
                    if (xi.kb == 0) TRACE(xi.op, 1);
                    ++xn;
                    if (++xs == C::STAGES) xs = 0;
                    cursor_next(xi, ops, maps, n_ops, cta, G);
                    progress = true;
                }
            }
            if (progress) idle = 0;
            else if (++idle > CHAIN_POLL_LIMIT || ((idle & 1023) == 0 && *abort_flag)) {
                atomicOr(status, NG_STATUS_CHAIN_TIMEOUT);
                *abort_flag = 1;
                break;
            }
        }
    } else if (threadIdx.x == 32) {
        // ------------------------------------------------------------ MMA issuer
        constexpr uint32_t idesc = make_idesc(TN);
        uint32_t n = 0, tcount = 0;
        bool ok = true;
        for (int oi = 0; oi < n_ops && ok; ++oi) {
            const ChainOp& o = ops[oi];
            if (o.type != OP_GEMM) continue;
            const int n_tasks = o.n_tiles * o.splits;
            for (int task = cta; task < n_tasks && ok; task += G) {
                int tile, kb0, nkb;
                task_range(o, task, tile, kb0, nkb);
                const uint32_t b = tcount & 1;
                ok = mbar_wait_or_abort(&acc_free[b], ((tcount >> 1) & 1) ^ 1, abort_flag);   // the epilogue has drained it
                if (!ok) break;
                tcgen05_fence_after();
                const uint32_t acc = tmem_base + b * C::ACC_COLS;
                for (int i = 0; i < nkb; ++i) {
                    const int s = n % C::STAGES;
                    ok = mbar_wait_or_abort(&full[s], (n / C::STAGES) & 1, abort_flag);
                    if (!ok) break;
                    if (i == 0) TRACE(oi, 2);
                    tcgen05_fence_after();
                    unsigned char* st = tiles + s * C::STAGE_BYTES;
                    const uint64_t da = make_desc_sw128(st), db = make_desc_sw128(st + C::W_BYTES);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint64_t koff = (uint64_t)((k * UMMA_K * 2) >> 4);
                        tcgen05_mma_f16(acc, da + koff, db + koff, idesc, (i > 0 || k > 0) ? 1u : 0u);
                    }
                    tcgen05_commit(&empty[s]);
                    ++n;
                }
                if (ok) tcgen05_commit(&acc_ready[b]);
                TRACE(oi, 3);
                ++tcount;
            }
        }
        if (!ok) {
            atomicOr(status, NG_STATUS_CHAIN_TIMEOUT);
            *abort_flag = 1;
        }
    } else if (warp >= 2) {
        // ------------------------------------------------------------ epilogues, norms, convolutions
        const int et = threadIdx.x - 64;                       // 0..127
        const int ew = warp & 3;                               // the quarter of tensor memory this warp may read
        const int tl = ew * 32 + lane;                         // this thread's TMEM lane = row of the W tile
        uint32_t tcount = 0;
        bool ok = true;
        ng_pdl_wait();                                          // before anything of the previous kernel is read or overwritten
        for (int oi = 0; oi < n_ops && ok; ++oi) {
            const ChainOp& o = ops[oi];
            if (o.type == OP_GEMM) {
                const int n_tasks = o.n_tiles * o.splits;
                for (int task = cta; task < n_tasks && ok; task += G) {
                    int tile, kb0, nkb;
                    task_range(o, task, tile, kb0, nkb);
                    const int split = task / o.n_tiles;
                    const uint32_t b = tcount & 1;
                    ok = mbar_wait_or_abort(&acc_ready[b], (tcount >> 1) & 1, abort_flag);
                    if (!ok) *abort_flag = 1;
                    ok = __all_sync(0xffffffffu, ok);
                    if (et == 0) TRACE(oi, 4);
                    tcgen05_fence_after();
                    const uint32_t lane_addr = tmem_base + b * C::ACC_COLS + ((uint32_t)(ew * 32) << 16);
                    const int w_row0 = tile * o.rows;
                    if (o.epi == EPI_SWIGLU) {
                        // lanes 0..63 hold gate(n), lanes 64..127 hold up(n), n = w_row0 + (lane & 63); for tokens
                        // 0..7 of a 16-token chunk the up half sends its values to the gate half, for tokens
                        // 8..15 the other way; each thread then gates and stores 8 tokens of its column
                        const int col = (ew & 1) * 32 + lane;
                        const int nn = w_row0 + col;
                        const bool up_half = ew >= 2;
                        const int peer = up_half ? tl - 64 : tl + 64;
                        const int j0 = up_half ? 8 : 0;
#pragma unroll 1
                        for (int c = 0; c < TN; c += 16) {
                            float v[16];
                            if (ok) tmem_ld16(lane_addr + c, v);
                            else {
#pragma unroll
                                for (int j = 0; j < 16; ++j) v[j] = 0.f;
                            }
#pragma unroll
                            for (int j = 0; j < 8; ++j) xch[tl][(8 - j0) + j] = up_half ? v[j] : v[8 + j];
                            epi_sync();
                            if (ok && col < o.rows && nn < o.N) {
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    const int m = c + j0 + j;
                                    if (m < o.M) {
                                        const float mine = up_half ? v[8 + j] : v[j], theirs = xch[peer][j0 + j];
                                        const float g = __bfloat162float(__float2bfloat16_rn(up_half ? theirs : mine));
                                        const float u = __bfloat162float(__float2bfloat16_rn(up_half ? mine : theirs));
                                        reinterpret_cast<bf16*>(o.p[0])[(size_t)m * o.ldc + nn] = __float2bfloat16_rn(silu_fast(g) * u);
                                    }
                                }
                            }
                            epi_sync();
                        }
                    } else if (ok) {
                        const int nn = w_row0 + tl;
#pragma unroll 1
                        for (int c = 0; c < TN; c += 16) {
                            float v[16];
                            tmem_ld16(lane_addr + c, v);
                            if (tl < o.rows && nn < o.N) {
#pragma unroll
                                for (int j = 0; j < 16; ++j) {
                                    const int m = c + j;
                                    if (m < o.M) {
                                        if (o.epi == EPI_F32)
                                            reinterpret_cast<float*>(o.p[0])[((size_t)split * o.M + m) * o.ldc + nn] = v[j];
                                        else if (o.epi == EPI_RED)
                                            atomicAdd(reinterpret_cast<float*>(o.p[0]) + (size_t)m * o.ldc + nn, v[j]);
                                        else
                                            reinterpret_cast<bf16*>(o.p[0])[(size_t)m * o.ldc + nn] = __float2bfloat16_rn(v[j]);
                                    }
                                }
                            }
                        }
                    }
                    if (et == 0) TRACE(oi, 5);
                    tcgen05_fence_before();
                    epi_sync();
                    if (et == 0) {
                        mbar_arrive(&acc_free[b]);
                        *epi_abort = *abort_flag;                // one reading for all: the roles may raise it any time
                    }
                    epi_sync();
                    ok = *epi_abort == 0;
                    ++tcount;
                }
            } else if (o.type == OP_NORM) {
                const float* h = reinterpret_cast<const float*>(o.p[0]);
                const float* w = reinterpret_cast<const float*>(o.p[1]);
                bf16* out = reinterpret_cast<bf16*>(o.p[2]);
                const int* rows = reinterpret_cast<const int*>(o.p[3]);
                const int H = o.H;
                const bool vec = (H % 4 == 0) && H <= 4 * CHAIN_EPI_THREADS * 8 && ((o.p[0] | o.p[1]) & 15) == 0;
                for (int r = cta; r < o.M; r += G) {
                    const float* hr = h + (size_t)(rows ? rows[r] : r) * H;
                    float ss = 0.f;
                    float4 v[8];
                    if (vec) {                                   // the row stays in registers between the two passes
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int c = 4 * (et + CHAIN_EPI_THREADS * i);
                            v[i] = c < H ? __ldcg(reinterpret_cast<const float4*>(hr + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
                            ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
                        }
                    } else {
                        for (int c = et; c < H; c += CHAIN_EPI_THREADS) { const float x = __ldcg(hr + c); ss += x * x; }
                    }
                    ss = ng_warp_sum(ss);
                    if (lane == 0) red[ew] = ss;
                    epi_sync();
                    const float rs = rsqrtf((red[0] + red[1] + red[2] + red[3]) / (float)H + o.eps);
                    if (vec) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const int c = 4 * (et + CHAIN_EPI_THREADS * i);
                            if (c < H) {
                                const float4 w4 = *reinterpret_cast<const float4*>(w + c);
                                __nv_bfloat162 lo = __floats2bfloat162_rn(v[i].x * rs * w4.x, v[i].y * rs * w4.y);
                                __nv_bfloat162 hi = __floats2bfloat162_rn(v[i].z * rs * w4.z, v[i].w * rs * w4.w);
                                *reinterpret_cast<uint2*>(out + (size_t)r * H + c) =
                                    make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
                            }
                        }
                    } else {
                        for (int c = et; c < H; c += CHAIN_EPI_THREADS)
                            out[(size_t)r * H + c] = __float2bfloat16_rn(__ldcg(hr + c) * rs * w[c]);
                    }
                    epi_sync();
                }
            } else {                                            // OP_CONV: entries that bring one token
                const float* part = reinterpret_cast<const float*>(o.p[0]);
                const float* cw = reinterpret_cast<const float*>(o.p[1]);
                const float* cb = reinterpret_cast<const float*>(o.p[2]);
                float* state = reinterpret_cast<float*>(o.p[3]);
                bf16* out = reinterpret_cast<bf16*>(o.p[4]);
                const int* cu_q = reinterpret_cast<const int*>(o.p[5]);
                const int* ctx_before = reinterpret_cast<const int*>(o.p[6]);
                const int* slots = reinterpret_cast<const int*>(o.p[7]);
                const int H = o.H, L = o.L;
                const size_t ld = 3 * (size_t)H, ps = (size_t)o.pstride;
                for (int idx = cta * CHAIN_EPI_THREADS + et; idx < o.M * H; idx += G * CHAIN_EPI_THREADS) {
                    const int e = idx / H, d = idx - e * H;
                    const int q0 = cu_q[e];
                    if (cu_q[e + 1] - q0 != 1) continue;         // a padding entry
                    const int ctx = ctx_before[e];
                    float* st = state + (size_t)slots[e] * (L - 1) * H + d;
                    // B, C, x: the K-split partial sums added in ascending order and rounded to bfloat16,
                    // where the unsplit product would have been stored
                    float bcx[3];
#pragma unroll
                    for (int t = 0; t < 3; ++t) {
                        const size_t at = (size_t)q0 * ld + (size_t)t * H + d;
                        if (o.n_part == 0) {                     // the product itself, stored in bfloat16
                            bcx[t] = __bfloat162float(__ushort_as_bfloat16(__ldcg(reinterpret_cast<const unsigned short*>(part) + at)));
                        } else {
                            float v = 0.f;
                            for (int s = 0; s < o.n_part; ++s) v += __ldcg(part + s * ps + at);
                            bcx[t] = __bfloat162float(__float2bfloat16_rn(v));
                        }
                    }
                    const float u = bcx[0] * bcx[2];
                    float acc = 0.f;
                    for (int j = 0; j < L - 1; ++j) {
                        const float old = (ctx - (L - 1) + j >= 0) ? st[(size_t)j * H] : 0.f;
                        acc = fmaf(cw[(size_t)d * L + j], old, acc);
                        if (j > 0) st[(size_t)(j - 1) * H] = old;          // the window moves on by one token
                    }
                    st[(size_t)(L - 2) * H] = u;
                    acc = fmaf(cw[(size_t)d * L + L - 1], u, acc) + (cb ? cb[d] : 0.f);
                    out[(size_t)q0 * H + d] = __float2bfloat16_rn(bcx[1] * acc);
                }
            }
            if (!ok) break;
            if (oi + 1 < n_ops) {
                // ---- the grid meets: what this block wrote is visible before its arrival counts
                if (et == 0) TRACE(oi, 6);
                __threadfence();
                epi_sync();
                if (et == 0) {
                    TRACE(oi, 7);
                    atomicAdd(counters, 1u);
                    TRACE(oi, 8);
                    const unsigned target = (unsigned)G * (unsigned)(oi + 1);
                    uint32_t polls = 0;
                    while (ld_acquire(counters) < target) {
                        if (++polls > CHAIN_POLL_LIMIT || ((polls & 255) == 0 && *abort_flag)) {
                            atomicOr(status, NG_STATUS_CHAIN_TIMEOUT);
                            *abort_flag = 1;
                            break;
                        }
                    }
                    *epi_abort = *abort_flag;
                    TRACE(oi, 9);
                }
                epi_sync();
                ok = *epi_abort == 0;
            }
        }
        if (!ok && et == 0) {
            atomicOr(status, NG_STATUS_CHAIN_TIMEOUT);
            *abort_flag = 1;                                     // the producer and the MMA thread stop waiting too
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"((uint32_t)C::TMEM_COLS) : "memory");
    }
    // the last block to leave clears the counters for the next launch (no block still reads them:
    // each passed the last barrier before its last operation)
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned prev = atomicAdd(counters + 1, 1u);
        if (prev == (unsigned)G - 1u) {
            counters[0] = 0u;
            counters[1] = 0u;
            __threadfence();
        }
    }
}

// ------------------------------------------------------------------------------------- host
// The bytes of a TMA tensor map of a [rows, cols] row-major bfloat16 matrix with boxes of
// box_rows x 64 columns, for the host to place in the array the kernel reads (128 bytes).
NG_EXPORT int ng_chain_encode_map(const void* ptr, int rows, int cols, int box_rows, void* out128) {
    if (!ptr || !out128 || rows <= 0 || cols <= 0 || cols % 8 || ((uintptr_t)ptr & 15) || box_rows <= 0 || box_rows > 256)
        return NG_BAD_SIZE;
    CUtensorMap m;
    if (!tensor_map(ptr, rows, cols, box_rows, &m)) return NG_LAUNCH_FAILED;
    static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
    memcpy(out128, &m, sizeof(m));
    return NG_OK;
}

// How a product of M tokens with a [N, K] weight is cut: rows of W per tile, tiles, K splits,
// K blocks per split, bytes of W per stage.  `splits` asks; the answer may be smaller.
NG_EXPORT int ng_chain_plan(int M, int N, int K, int epi, int splits, int* rows, int* n_tiles, int* splits_out,
                            int* kb_per_split, int* w_bytes) {
    if (M <= 0 || N <= 0 || K <= 0 || K % 8 || splits < 1) return NG_BAD_SIZE;
    if (epi == EPI_SWIGLU || epi == EPI_BF16) splits = 1;
    const int total_kb = (K + BLOCK_K - 1) / BLOCK_K;
    if (splits > total_kb) splits = total_kb;
    const int per = (total_kb + splits - 1) / splits;
    splits = (total_kb + per - 1) / per;
    const int r = ng_plan_rows(M, N, epi, splits);
    *rows = r;
    *n_tiles = (N + r - 1) / r;
    *splits_out = splits;
    *kb_per_split = per;
    *w_bytes = (epi == EPI_SWIGLU ? 2 : 1) * r * BLOCK_K * 2;
    return NG_OK;
}

#ifdef CHAIN_TRACE
NG_EXPORT int ng_chain_trace(long long* out, int n) {
    return cudaMemcpyFromSymbol(out, g_chain_trace, sizeof(long long) * (size_t)min(n, CHAIN_MAX_OPS * 16)) == cudaSuccess ? NG_OK
                                                                                                                            : NG_LAUNCH_FAILED;
}
#endif

NG_EXPORT int ng_chain_op_bytes() { return (int)sizeof(ChainOp); }
NG_EXPORT int ng_chain_max_ops() { return CHAIN_MAX_OPS; }

template <int TN>
static int launch_chain(const void* maps, const void* ops, int n_ops, unsigned* counters, int* status, cudaStream_t stream) {
    using C = ChainCfg<TN>;
    static bool attr_set = false;
    static int sms = 0;
    if (!attr_set) {
        if (cudaFuncSetAttribute(chain_sm100_kernel<TN>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) != cudaSuccess)
            return NG_LAUNCH_FAILED;
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, chain_sm100_kernel<TN>, CHAIN_THREADS, C::SMEM) != cudaSuccess ||
            per_sm < 1 || sms < 1)
            return NG_LAUNCH_FAILED;
        attr_set = true;
    }
    // one block per SM, all resident at once (a cooperative launch: the blocks wait on one another)
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(sms);
    cfg.blockDim = dim3(CHAIN_THREADS);
    cfg.dynamicSmemBytes = C::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    memset(attrs, 0, sizeof(attrs));
    attrs[0].id = cudaLaunchAttributeCooperative;
    attrs[0].val.cooperative = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    static bool both = true;                                    // whether the two attributes are taken together
    cfg.numAttrs = (ng_pdl_enabled() && both) ? 2 : 1;
    cudaError_t rc = cudaLaunchKernelEx(&cfg, chain_sm100_kernel<TN>, (const CUtensorMap*)maps, (const ChainOp*)ops, n_ops,
                                        counters, status);
    if (rc != cudaSuccess && cfg.numAttrs == 2) {               // the two attributes together are not taken everywhere
        cudaGetLastError();
        both = false;
        cfg.numAttrs = 1;
        rc = cudaLaunchKernelEx(&cfg, chain_sm100_kernel<TN>, (const CUtensorMap*)maps, (const ChainOp*)ops, n_ops,
                                counters, status);
    }
    if (rc != cudaSuccess) {
        cudaGetLastError();
        return NG_LAUNCH_FAILED;
    }
    return NG_OK;
}

// maps: device array of tensor maps (128 bytes each, 64-byte aligned); ops: device array of n_ops
// ChainOp; counters: two zeroed device words (the kernel leaves them zeroed); tn: 16, 32 or 64,
// at least the token count of every product.
NG_EXPORT int ng_chain_launch(const void* maps, const void* ops, int n_ops, int tn, unsigned* counters, int* status,
                              cudaStream_t stream) {
    if (n_ops <= 0) return NG_OK;
    if (n_ops > CHAIN_MAX_OPS || !maps || !ops || !counters || !status || ((uintptr_t)maps & 63) || ((uintptr_t)ops & 15))
        return NG_BAD_SIZE;
    switch (tn) {
        case 16: return launch_chain<16>(maps, ops, n_ops, counters, status, stream);
        case 32: return launch_chain<32>(maps, ops, n_ops, counters, status, stream);
        case 64: return launch_chain<64>(maps, ops, n_ops, counters, status, stream);
    }
    return NG_BAD_SIZE;
}

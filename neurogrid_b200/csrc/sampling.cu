// Sampling on the device over float32 logits: argmax, temperature softmax, nucleus (top-p)
// cut and an inverse-CDF draw in index order.
//
// The reference samples on the host after copying the logits back every token
// (pkg/inference/sampler.go:25-51): temperature <= 0 -> argmax with the first index winning
// ties (sampler.go:58-73); else logits / temperature -> softmax -> for 0 < top_p < 1 keep the
// most probable tokens through the first cumulative sum >= top_p and renormalise
// (sampler.go:114-149) -> walk the cumulative sum in index order until it exceeds one uniform
// number (sampler.go:170-189).  Here the uniform number comes from the host (a counter-based
// hash of seed, request and step), so a request's draw does not depend on its batch.
//
// Nucleus cut without a sort: the kept set is {i : e_i >= t} for the largest t whose kept
// mass reaches top_p of the total; t is found by bisection on the float bit pattern.  Tokens
// that tie exactly at t are all kept (the reference's sort leaves their order unspecified).
// Scratch: one float per vocabulary entry per row (unnormalised exp values).
#include "ng_common.cuh"

#define SM_THREADS 1024

__device__ __forceinline__ void block_argmax(float& v, int& idx, float* sv, int* si) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    __syncthreads();
    if (lane == 0) { sv[warp] = v; si[warp] = idx; }
    __syncthreads();
    const int nwarp = blockDim.x >> 5;
    v = lane < nwarp ? sv[lane] : -INFINITY;
    idx = lane < nwarp ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
}

// rows: W; one block per row.
__global__ void __launch_bounds__(SM_THREADS)
sample_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temperature,
              const float* __restrict__ top_p, const float* __restrict__ uniform, int* __restrict__ out,
              float* __restrict__ scratch) {
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ float chunk_sum[SM_THREADS];
    __shared__ float bcast;
    __shared__ int chosen;
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* lg = logits + (size_t)row * V;

    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = tid; i < V; i += SM_THREADS) {
        const float v = lg[i];
        if (v > best) { best = v; best_i = i; }      // ascending i per thread: first index wins
    }
    block_argmax(best, best_i, sv, si);
    const float temp = temperature ? temperature[row] : 0.f;
    if (!(temp > 0.f)) {
        if (tid == 0) out[row] = best_i;
        return;
    }
    // e_i = exp((l_i - max) / T), kept unnormalised in scratch
    float* e = scratch + (size_t)row * V;
    float part = 0.f;
    for (int i = tid; i < V; i += SM_THREADS) {
        const float v = expf((lg[i] - best) / temp);
        e[i] = v;
        part += v;
    }
    const float total = ng_block_sum(part, sv);
    __syncthreads();                                  // e[] visible to the whole block

    float thresh = 0.f;
    const float p = top_p ? top_p[row] : 1.f;
    if (p > 0.f && p < 1.f) {
        // largest bit pattern t with mass{e >= t} >= p * total; e in (0, 1], so t in [0, 0x3f800000]
        const float want = p * total;
        unsigned lo = 0u, hi = 0x3f800000u;           // invariant: mass(lo) >= want
        while (lo < hi) {
            const unsigned mid = lo + (hi - lo + 1u) / 2u;
            const float t = __uint_as_float(mid);
            float s = 0.f;
            for (int i = tid; i < V; i += SM_THREADS) {
                const float v = e[i];
                if (v >= t) s += v;
            }
            s = ng_block_sum(s, sv);
            if (s >= want) lo = mid; else hi = mid - 1u;
        }
        thresh = __uint_as_float(lo);
    }
    // inverse CDF in index order over the kept entries: thread t owns indices [t*C, (t+1)*C)
    const int C = (V + SM_THREADS - 1) / SM_THREADS;
    const int i0 = min(tid * C, V), i1 = min(i0 + C, V);
    float mine = 0.f;
    for (int i = i0; i < i1; ++i) {
        const float v = e[i];
        if (v >= thresh) mine += v;
    }
    chunk_sum[tid] = mine;
    if (tid == 0) chosen = -1;
    __syncthreads();
    if (tid == 0) {                                   // exclusive scan, serial: fixed order
        float run = 0.f;
        for (int t = 0; t < SM_THREADS; ++t) {
            const float c = chunk_sum[t];
            chunk_sum[t] = run;
            run += c;
        }
        bcast = run;
    }
    __syncthreads();
    const float kept_total = bcast;
    const float target = uniform[row] * kept_total;
    const float before = chunk_sum[tid];
    if (mine > 0.f && target >= before && target < before + mine) {
        float run = before;
        int pick = -1, last_kept = -1;
        for (int i = i0; i < i1; ++i) {
            const float v = e[i];
            if (v >= thresh) {
                run += v;
                last_kept = i;
                if (target < run) { pick = i; break; }
            }
        }
        if (pick < 0) pick = last_kept;
        atomicMax(&chosen, pick);
    }
    __syncthreads();
    if (tid == 0) out[row] = chosen >= 0 ? chosen : best_i;   // rounding left no owner: most probable token
}

NG_EXPORT int ng_sample(const float* logits, int n_rows, int V, const float* temperature, const float* top_p,
                        const float* uniform, int* out, float* scratch, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (V <= 0) return NG_BAD_SIZE;
    NG_LAUNCH((sample_kernel), n_rows, SM_THREADS, 0, stream, logits, V, temperature, top_p, uniform, out, scratch);
    return ng_launch_status();
}

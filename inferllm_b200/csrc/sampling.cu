// Choosing the next token on the device.
//
// illm_argmax: greedy choice, the lowest id among equal maxima.
// illm_sample: the reference's sampler (llama_sample_top_p_top_k, src/utils.cpp:31-115) as one
// launch, one block per sequence, all in float32:
//   1. z = logit / temp; for each distinct id among the sequence's last tokens
//      z = logit < 0 ? z * penalty : z / penalty                                   (:41-59)
//   2. keep the top_k largest z (top_k <= 0 or >= V keeps all)                      (:21-29,63)
//   3. probabilities exp(z - max) / sum over the kept                              (:65-84)
//   4. keep the shortest prefix, in descending order, whose probability reaches
//      top_p; renormalise                                                          (:86-101)
//   5. draw from what is left with the uniform number u of this sequence           (:111-112)
// Instead of sorting, steps 2 and 4 find their cut value by bisection over the 32 bits of an
// order-preserving integer image of z: the largest c with count(z >= c) >= top_k, and the
// largest c with P(z >= c) >= top_p.  Values equal to the cut are all kept (the reference's
// partial sort keeps an arbitrary subset of equals); step 5 walks the kept ids in ascending
// order of id, which draws from the same distribution as the reference's walk in descending
// order of probability.  The uniform numbers are made on the host by a counter-based
// generator keyed by (seed, request, step), so a draw does not depend on the batch.
#include <math.h>

#include "common.cuh"

#define AM_THREADS 256
#define AM_CHUNK 2048            // elements of a row per block of the first pass

__device__ __forceinline__ void am_better(float& best, int& idx, float ov, int oi) {
    if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
}
// Reduces (best, idx) over the block; valid in warp 0.
__device__ __forceinline__ void am_block(float& best, int& idx, float* bv, int* bi) {
    for (int o = 16; o > 0; o >>= 1)
        am_better(best, idx, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        best = lane < nw ? bv[lane] : -INFINITY;
        idx = lane < nw ? bi[lane] : 0x7fffffff;
        for (int o = 16; o > 0; o >>= 1)
            am_better(best, idx, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
    }
}

// First pass: block (c, b) finds the maximum of elements [c * AM_CHUNK, (c + 1) * AM_CHUNK) of row b.
__global__ void __launch_bounds__(AM_THREADS)
argmax_chunk_kernel(const float* __restrict__ logits, int V, int ld, float* __restrict__ pv, int* __restrict__ pi) {
    pdl_grid_sync();
    __shared__ float bv[32];
    __shared__ int bi[32];
    const float* row = logits + (size_t)blockIdx.y * ld;
    const int c0 = blockIdx.x * AM_CHUNK, c1 = min(V, c0 + AM_CHUNK);
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = c0 + threadIdx.x; i < c1; i += AM_THREADS) am_better(best, idx, row[i], i);
    am_block(best, idx, bv, bi);
    if (threadIdx.x == 0) {
        pv[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = best;
        pi[(size_t)blockIdx.y * gridDim.x + blockIdx.x] = idx;
    }
}

// Second pass: one warp per row over the chunks' results; the lowest id among equal maxima wins,
// whatever the order of the comparisons.
__global__ void argmax_final_kernel(const float* __restrict__ pv, const int* __restrict__ pi, int n_chunks,
                                    int* __restrict__ out) {
    pdl_grid_sync();
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < n_chunks; i += 32)
        am_better(best, idx, pv[(size_t)blockIdx.x * n_chunks + i], pi[(size_t)blockIdx.x * n_chunks + i]);
    for (int o = 16; o > 0; o >>= 1)
        am_better(best, idx, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, idx, o));
    if (threadIdx.x == 0) out[blockIdx.x] = (idx == 0x7fffffff) ? 0 : idx;
}

// scratch_v, scratch_i: B * ceil(V / 2048) floats and ints.
extern "C" int illm_argmax(const float* logits, int B, int V, int ld, int* out, float* scratch_v, int* scratch_i,
                           void* stream) {
    if (B <= 0) return 0;
    if (V <= 0 || B > 65535 || scratch_v == nullptr || scratch_i == nullptr) return ILLM_ERR_BAD_ARG;
    const int n_chunks = (V + AM_CHUNK - 1) / AM_CHUNK;
    illm_launch(argmax_chunk_kernel, dim3(n_chunks, B), dim3(AM_THREADS), 0, (cudaStream_t)stream, logits, V, ld,
                scratch_v, scratch_i);
    illm_launch(argmax_final_kernel, dim3(B), dim3(32), 0, (cudaStream_t)stream, (const float*)scratch_v,
                (const int*)scratch_i, n_chunks, out);
    return illm_launch_status();
}

#define SAMPLE_THREADS 1024

__device__ __forceinline__ unsigned ordered_key(float f) {
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float block_sum_f(float v, float* scratch) { return block_sum(v, scratch); }

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int V, int ld, float* __restrict__ z_all,
              const int* __restrict__ last_tokens, int n_last, float temp, float penalty, int top_k,
              float top_p, const float* __restrict__ uniforms, int* __restrict__ out) {
    pdl_grid_sync();
    __shared__ float scratch[32];
    __shared__ float partial[SAMPLE_THREADS];
    __shared__ int chosen;
    const int tid = threadIdx.x;
    const float* row = logits + (size_t)blockIdx.x * ld;
    float* z = z_all + (size_t)blockIdx.x * V;
    const float inv_temp = 1.0f / temp;

    // 1. temperature and repetition penalty
    for (int i = tid; i < V; i += blockDim.x) z[i] = row[i] * inv_temp;
    __syncthreads();
    if (last_tokens && penalty != 1.0f) {
        const int* lt = last_tokens + (size_t)blockIdx.x * n_last;
        for (int j = tid; j < n_last; j += blockDim.x) {
            const int id = lt[j];
            if (id < 0 || id >= V) continue;
            bool first = true;
            for (int e = 0; e < j; e++)
                if (lt[e] == id) { first = false; break; }
            if (first) z[id] = row[id] < 0.f ? row[id] * inv_temp * penalty : row[id] * inv_temp / penalty;
        }
    }
    __syncthreads();

    // 2. top-k cut: the largest key c with count(key >= c) >= top_k
    unsigned cut = 0u;
    if (top_k > 0 && top_k < V) {
        for (int bit = 31; bit >= 0; bit--) {
            const unsigned cand = cut | (1u << bit);
            float cnt = 0.f;
            for (int i = tid; i < V; i += blockDim.x) cnt += ordered_key(z[i]) >= cand ? 1.f : 0.f;
            cnt = block_sum_f(cnt, scratch);
            if (cnt >= (float)top_k) cut = cand;
        }
    }

    // 3. maximum and normaliser over the kept
    float mx = -INFINITY;
    for (int i = tid; i < V; i += blockDim.x)
        if (ordered_key(z[i]) >= cut) mx = fmaxf(mx, z[i]);
    mx = warp_max(mx);
    __syncthreads();
    if ((tid & 31) == 0) scratch[tid >> 5] = mx;
    __syncthreads();
    mx = scratch[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); w++) mx = fmaxf(mx, scratch[w]);
    float sum = 0.f;
    for (int i = tid; i < V; i += blockDim.x)
        if (ordered_key(z[i]) >= cut) sum += expf(z[i] - mx);
    sum = block_sum_f(sum, scratch);

    // 4. top-p cut: the largest key c with sum(exp, key >= c) >= top_p * sum
    float kept = sum;
    if (top_p < 1.0f) {
        const float need = top_p * sum;
        unsigned pc = 0u;
        for (int bit = 31; bit >= 0; bit--) {
            const unsigned cand = pc | (1u << bit);
            float s = 0.f;
            if (cand >= cut) {
                for (int i = tid; i < V; i += blockDim.x)
                    if (ordered_key(z[i]) >= cand) s += expf(z[i] - mx);
                s = block_sum_f(s, scratch);
            } else {
                s = sum;  // below the top-k cut nothing more is added
            }
            if (s >= need) { pc = cand; kept = s; }
        }
        if (pc > cut) cut = pc;
        // the normaliser of what is kept, summed the same way as the draw below
    }

    // 5. inverse CDF over ascending ids: each thread owns a contiguous range
    const int chunk = (V + blockDim.x - 1) / blockDim.x;
    const int b = tid * chunk, e = min(V, b + chunk);
    float mine = 0.f;
    for (int i = b; i < e; i++)
        if (ordered_key(z[i]) >= cut) mine += expf(z[i] - mx);
    partial[tid] = mine;
    if (tid == 0) chosen = -1;
    __syncthreads();
    if (tid == 0) {
        float total = 0.f;
        for (int i = 0; i < (int)blockDim.x; i++) total += partial[i];
        const float target = uniforms[blockIdx.x] * total;
        float run = 0.f;
        int owner = -1;
        for (int i = 0; i < (int)blockDim.x; i++) {
            if (partial[i] > 0.f) {
                owner = i;
                if (run + partial[i] > target) break;
                run += partial[i];
            }
        }
        // walk the owner's range
        int pick = -1;
        if (owner >= 0) {
            const int ob = owner * chunk, oe = min(V, ob + chunk);
            // `run` may already include the owner when the loop ran to the end: recompute
            float r2 = 0.f;
            for (int i = 0; i < owner; i++) r2 += partial[i];
            for (int i = ob; i < oe; i++) {
                if (ordered_key(z[i]) >= cut) {
                    pick = i;
                    r2 += expf(z[i] - mx);
                    if (r2 > target) break;
                }
            }
        }
        chosen = pick < 0 ? 0 : pick;
    }
    __syncthreads();
    if (tid == 0) out[blockIdx.x] = chosen;
    (void)kept;
}

extern "C" int illm_sample(const float* logits, int B, int V, int ld, float* z_scratch,
                           const int* last_tokens, int n_last, float temp, float penalty, int top_k,
                           float top_p, const float* uniforms, int* out, void* stream) {
    if (B <= 0) return 0;
    if (V <= 0 || !(temp > 0.f) || !(penalty > 0.f)) return ILLM_ERR_BAD_ARG;
    illm_launch(sample_kernel, dim3(B), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, 
        logits, V, ld, z_scratch, last_tokens, n_last, temp, penalty, top_k, top_p, uniforms, out);
    return illm_launch_status();
}

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
              float top_p, const float* __restrict__ uniforms, int* __restrict__ out,
              const int* __restrict__ only_if) {
    pdl_grid_sync();
    if (only_if != nullptr && only_if[blockIdx.x] == 0) return;    // rows that the fast path has finished
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

// ---- The fast paths.  A first pass by many blocks over chunks of 2048 logits, a second by one
// block per row over what the chunks left.  Both give what the kernel above gives up to the order
// in which equal probabilities are walked, and are as deterministic: no sum depends on timing.
//
// Temperature only (top_k off, top_p = 1): the chunks' maxima and sums of exp, then the chunk and
// the element in which the cumulative sum passes u * total.
// top_k <= 64 and at most 64 chunks (with or without top_p): every chunk keeps its own top_k (a
// bisection over the keys held in registers).  The row's top_k are among those candidates: the
// second pass finds the row's cut by the same bisection over them, sorts what lies above it (value
// descending, id ascending), keeps the first top_k and their equals, and applies top_p by the
// reference's own rule, the shortest prefix in descending order that reaches it
// (src/utils.cpp:86-101).
// A row whose candidates do not fit (many equal values) is flagged and done by the kernel above.
#define SK_THREADS 256
#define SK_PER 8
#define SK_CHUNK (SK_THREADS * SK_PER)
#define SK_MAX_K 64
#define SK_CAP 96                 // candidates a chunk may hand on
#define SK_LIST 1024              // candidates a row may sort
#define SK_LAST_SMEM 256          // last tokens kept in shared memory for the repetition penalty
#define SK_SLOTS 24               // candidate places per thread of the second pass: up to 64 chunks
#define SK_MAX_CHUNKS (SK_SLOTS * SK_THREADS / SK_CAP)

__device__ __forceinline__ float sk_scaled(const float* __restrict__ row, int i, float inv_temp, float penalty,
                                           const int* __restrict__ lt, int n_last) {
    const float x = row[i];
    float z = x * inv_temp;
    if (lt != nullptr && penalty != 1.0f) {
        bool hit = false;
        for (int j = 0; j < n_last; j++) hit |= (lt[j] == i);
        if (hit) z = x < 0.f ? x * inv_temp * penalty : x * inv_temp / penalty;
    }
    return z;
}

template <bool TOPK>
__global__ void __launch_bounds__(SK_THREADS)
sample_chunk_kernel(const float* __restrict__ logits, int V, int ld, float* __restrict__ z_all,
                    const int* __restrict__ last_tokens, int n_last, float inv_temp, float penalty, int top_k,
                    float* __restrict__ cmax, float* __restrict__ csum, int* __restrict__ ccount, float* __restrict__ cand_z, int* __restrict__ cand_id) {
    pdl_grid_sync();
    __shared__ float fscr[32];
    __shared__ int iscr[2][SK_THREADS / 32];
    const int chunk = blockIdx.x, b = blockIdx.y, n_chunks = gridDim.x, tid = threadIdx.x;
    const int lane = tid & 31, warp = tid >> 5;
    const float* row = logits + (size_t)b * ld;
    const int* lt = (last_tokens != nullptr && n_last > 0 && penalty != 1.0f) ? last_tokens + (size_t)b * n_last : nullptr;
    __shared__ int lts[SK_LAST_SMEM];
    if (lt != nullptr && n_last <= SK_LAST_SMEM) {          // the row's last tokens, read once per block
        for (int j = tid; j < n_last; j += SK_THREADS) lts[j] = lt[j];
        __syncthreads();
        lt = lts;
    }
    const int i0 = chunk * SK_CHUNK + tid * SK_PER;
    float z[SK_PER];
#pragma unroll
    for (int e = 0; e < SK_PER; e++) z[e] = (i0 + e < V) ? sk_scaled(row, i0 + e, inv_temp, penalty, lt, n_last) : -INFINITY;
    const size_t cidx = (size_t)b * n_chunks + chunk;
    if (!TOPK) {
#pragma unroll
        for (int e = 0; e < SK_PER; e++)
            if (i0 + e < V) z_all[(size_t)b * V + i0 + e] = z[e];
        float m = z[0];
#pragma unroll
        for (int e = 1; e < SK_PER; e++) m = fmaxf(m, z[e]);
        m = warp_max(m);
        if (lane == 0) fscr[warp] = m;
        __syncthreads();
        m = fscr[0];
        for (int w = 1; w < SK_THREADS / 32; w++) m = fmaxf(m, fscr[w]);
        float sum = 0.f;
#pragma unroll
        for (int e = 0; e < SK_PER; e++) sum += (i0 + e < V) ? expf(z[e] - m) : 0.f;
        sum = block_sum(sum, fscr);
        if (tid == 0) {
            cmax[cidx] = m;
            csum[cidx] = sum;
        }
    } else {
    unsigned key[SK_PER];
#pragma unroll
    for (int e = 0; e < SK_PER; e++) key[e] = (i0 + e < V) ? ordered_key(z[e]) : 0u;    // 0 is below every real key
    const int n_valid = min(SK_CHUNK, V - chunk * SK_CHUNK);
    unsigned cut = 0u;
    if (n_valid > top_k) {
        // the largest key c with count(key >= c) >= top_k, bit by bit
        for (int bit = 31; bit >= 0; bit--) {
            const unsigned cand = cut | (1u << bit);
            int cnt = 0;
#pragma unroll
            for (int e = 0; e < SK_PER; e++) cnt += key[e] >= cand ? 1 : 0;
            cnt = __reduce_add_sync(0xffffffffu, cnt);
            if (lane == 0) iscr[bit & 1][warp] = cnt;
            __syncthreads();
            int total = 0;
#pragma unroll
            for (int w = 0; w < SK_THREADS / 32; w++) total += iscr[bit & 1][w];
            if (total >= top_k) cut = cand;
        }
    }
    const unsigned keep = cut == 0u ? 1u : cut;
    // the kept elements in order of their id: an exclusive scan of the threads' counts
    int mine = 0;
#pragma unroll
    for (int e = 0; e < SK_PER; e++) mine += key[e] >= keep ? 1 : 0;
    int incl = mine;
    for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    __syncthreads();
    if (lane == 31) iscr[0][warp] = incl;
    __syncthreads();
    int before = incl - mine, total = 0;
#pragma unroll
    for (int w = 0; w < SK_THREADS / 32; w++) {
        if (w < warp) before += iscr[0][w];
        total += iscr[0][w];
    }
#pragma unroll
    for (int e = 0; e < SK_PER; e++)
        if (key[e] >= keep) {
            if (before < SK_CAP) {
                cand_z[cidx * SK_CAP + before] = z[e];
                cand_id[cidx * SK_CAP + before] = i0 + e;
            }
            before++;
        }
    if (tid == 0) ccount[cidx] = total;
    }
}

__global__ void __launch_bounds__(SK_THREADS)
sample_temp_final_kernel(const float* __restrict__ z_all, int V, int n_chunks, const float* __restrict__ cmax,
                         const float* __restrict__ csum, const float* __restrict__ uniforms, int* __restrict__ out) {
    pdl_grid_sync();
    __shared__ float fscr[32];
    __shared__ float part[SK_THREADS];
    __shared__ float sh_target;
    __shared__ int sh_pick, sh_owner;
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* cm = cmax + (size_t)b * n_chunks;
    const float* cs = csum + (size_t)b * n_chunks;
    float m = -INFINITY;
    for (int c = tid; c < n_chunks; c += SK_THREADS) m = fmaxf(m, cm[c]);
    m = warp_max(m);
    if (lane == 0) fscr[warp] = m;
    __syncthreads();
    m = fscr[0];
    for (int w = 1; w < SK_THREADS / 32; w++) m = fmaxf(m, fscr[w]);
    if (tid == 0) {
        // the chunk in which the cumulative sum passes u * total (chunks in ascending order)
        float total = 0.f;
        for (int c = 0; c < n_chunks; c++) total += cs[c] * expf(cm[c] - m);
        const float target = uniforms[b] * total;
        float run = 0.f, before = 0.f;
        int owner = 0;
        for (int c = 0; c < n_chunks; c++) {
            const float w = cs[c] * expf(cm[c] - m);
            if (w > 0.f) {
                owner = c;
                before = run;
                run += w;
                if (run > target) break;
            }
        }
        sh_owner = owner;
        sh_target = target - before;
    }
    __syncthreads();
    const int i0 = sh_owner * SK_CHUNK + tid * SK_PER;
    float e8[SK_PER], mine = 0.f;
#pragma unroll
    for (int e = 0; e < SK_PER; e++) {
        e8[e] = (i0 + e < V) ? expf(z_all[(size_t)b * V + i0 + e] - m) : 0.f;
        mine += e8[e];
    }
    part[tid] = mine;
    __syncthreads();
    if (tid == 0) {
        float run = 0.f, before = 0.f;
        int owner = 0;
        for (int t = 0; t < SK_THREADS; t++)
            if (part[t] > 0.f) {
                owner = t;
                before = run;
                run += part[t];
                if (run > sh_target) break;
            }
        sh_pick = owner;
        sh_target -= before;
    }
    __syncthreads();
    if (tid == sh_pick) {
        float run = 0.f;
        int pick = min(i0, V - 1);
        for (int e = 0; e < SK_PER; e++)
            if (e8[e] > 0.f) {
                pick = i0 + e;
                run += e8[e];
                if (run > sh_target) break;
            }
        out[b] = pick;
    }
}

__global__ void __launch_bounds__(SK_THREADS)
sample_topk_final_kernel(int n_chunks, int top_k, float top_p, const int* __restrict__ ccount, const float* __restrict__ cand_z,
                         const int* __restrict__ cand_id, const float* __restrict__ uniforms,
                         int* __restrict__ out, int* __restrict__ fallback) {
    pdl_grid_sync();
    __shared__ float lz[SK_LIST];
    __shared__ int lid[SK_LIST];
    __shared__ float le[SK_LIST];
    __shared__ int iscr[2][SK_THREADS / 32];
    __shared__ int n_list, over;
    const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t c0 = (size_t)b * n_chunks;
    if (tid == 0) {
        n_list = 0;
        over = 0;
    }
    __syncthreads();
    // every thread holds the keys of its share of the chunks' candidates (0: an empty place)
    unsigned keys[SK_SLOTS];
    int have = 0;
#pragma unroll
    for (int q = 0; q < SK_SLOTS; q++) {
        const int slot = tid + q * SK_THREADS;
        keys[q] = 0u;
        if (slot < n_chunks * SK_CAP) {
            const int c = slot / SK_CAP, pos = slot - c * SK_CAP, cnt = ccount[c0 + c];
            if (cnt > SK_CAP) over = 1;
            if (pos < cnt && pos < SK_CAP) {
                keys[q] = ordered_key(cand_z[(c0 + c) * SK_CAP + pos]);
                have++;
            }
        }
    }
    // the row's cut: the largest key c with count(key >= c) >= top_k among the candidates
    auto block_count = [&](int mine, int which) {
        mine = __reduce_add_sync(0xffffffffu, mine);
        if (lane == 0) iscr[which][warp] = mine;
        __syncthreads();
        int total = 0;
#pragma unroll
        for (int w = 0; w < SK_THREADS / 32; w++) total += iscr[which][w];
        return total;
    };
    const int n_cand = block_count(have, 1);      // (the calls alternate between the two buffers)
    unsigned cut = 0u;
    if (n_cand > top_k) {
        for (int bit = 31; bit >= 0; bit--) {
            const unsigned cand = cut | (1u << bit);
            int cnt = 0;
#pragma unroll
            for (int q = 0; q < SK_SLOTS; q++) cnt += keys[q] >= cand ? 1 : 0;
            if (block_count(cnt, (bit & 1) ^ 1) >= top_k) cut = cand;
        }
    }
    const unsigned keep = cut == 0u ? 1u : cut;
#pragma unroll
    for (int q = 0; q < SK_SLOTS; q++)
        if (keys[q] >= keep) {
            const int at = atomicAdd(&n_list, 1);
            if (at < SK_LIST) {
                const int slot = tid + q * SK_THREADS, c = slot / SK_CAP, pos = slot - c * SK_CAP;
                const unsigned k = keys[q];
                lz[at] = __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);     // the key's value
                lid[at] = cand_id[(c0 + c) * SK_CAP + pos];
            }
        }
    __syncthreads();
    const int n = n_list;
    if (over || n > SK_LIST || n <= 0) {
        if (tid == 0) fallback[b] = 1;
        return;
    }
    // sort by (value descending, id ascending): a total order, so the order of arrival does not matter
    int P = 32;
    while (P < n) P <<= 1;
    for (int i = n + tid; i < P; i += SK_THREADS) {
        lz[i] = -INFINITY;
        lid[i] = 0x7fffffff;
    }
    __syncthreads();
    for (int k = 2; k <= P; k <<= 1)
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = tid; i < P; i += SK_THREADS) {
                const int x = i ^ j;
                if (x > i) {
                    const float za = lz[i], zb = lz[x];
                    const int ia = lid[i], ib = lid[x];
                    const bool a_first = za > zb || (za == zb && ia < ib);
                    const bool up = (i & k) == 0;          // this pair ends with its first element first
                    if (up != a_first) {
                        lz[i] = zb; lz[x] = za;
                        lid[i] = ib; lid[x] = ia;
                    }
                }
            }
            __syncthreads();
        }
    int kept = min(top_k, n);
    while (kept < n && lz[kept] == lz[kept - 1] && kept >= top_k) kept++;     // equals of the last kept one stay
    const float mx = lz[0];
    for (int i = tid; i < kept; i += SK_THREADS) le[i] = expf(lz[i] - mx);
    __syncthreads();
    if (tid == 0) {
        float total = 0.f;
        for (int i = 0; i < kept; i++) total += le[i];
        int n_keep = kept;
        float kept_sum = total;
        if (top_p < 1.0f) {
            const float need = top_p * total;
            float run = 0.f;
            for (int i = 0; i < kept; i++) {
                run += le[i];
                if (run >= need) {
                    n_keep = i + 1;
                    kept_sum = run;
                    break;
                }
            }
        }
        const float target = uniforms[b] * kept_sum;
        float run = 0.f;
        int pick = lid[n_keep - 1];
        for (int i = 0; i < n_keep; i++) {
            run += le[i];
            if (run > target) {
                pick = lid[i];
                break;
            }
        }
        out[b] = pick;
        fallback[b] = 0;
    }
}

// int32 elements of scratch that illm_sample needs for these settings (0: none)
extern "C" long long illm_sample_scratch_elems(int B, int V, int top_k, float top_p) {
    const long long n_chunks = (V + SK_CHUNK - 1) / SK_CHUNK;
    const bool k_on = top_k > 0 && top_k < V;
    if (k_on && top_k <= SK_MAX_K && n_chunks <= SK_MAX_CHUNKS) return (long long)B * (n_chunks * (1 + 2 * SK_CAP) + 1);
    if (!k_on && !(top_p < 1.0f)) return (long long)B * n_chunks * 2;
    return 0;
}

extern "C" int illm_sample(const float* logits, int B, int V, int ld, float* z_scratch,
                           const int* last_tokens, int n_last, float temp, float penalty, int top_k,
                           float top_p, const float* uniforms, int* out, int* scratch, void* stream) {
    if (B <= 0) return 0;
    if (V <= 0 || !(temp > 0.f) || !(penalty > 0.f) || B > 65535) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int n_chunks = (V + SK_CHUNK - 1) / SK_CHUNK;
    const bool k_on = top_k > 0 && top_k < V;
    if (scratch != nullptr && k_on && top_k <= SK_MAX_K && n_chunks <= SK_MAX_CHUNKS) {
        const size_t nc = (size_t)B * n_chunks;
        int* ccount = scratch;
        float* cand_z = reinterpret_cast<float*>(scratch + nc);
        int* cand_id = scratch + nc + nc * SK_CAP;
        int* fallback = scratch + nc + 2 * nc * SK_CAP;
        illm_launch(sample_chunk_kernel<true>, dim3(n_chunks, B), dim3(SK_THREADS), 0, s, logits, V, ld, z_scratch,
                    last_tokens, n_last, 1.0f / temp, penalty, top_k, (float*)nullptr, (float*)nullptr, ccount, cand_z,
                    cand_id);
        illm_launch(sample_topk_final_kernel, dim3(B), dim3(SK_THREADS), 0, s, n_chunks, top_k, top_p,
                    (const int*)ccount, (const float*)cand_z, (const int*)cand_id, uniforms, out, fallback);
        illm_launch(sample_kernel, dim3(B), dim3(SAMPLE_THREADS), 0, s, logits, V, ld, z_scratch, last_tokens, n_last,
                    temp, penalty, top_k, top_p, uniforms, out, (const int*)fallback);
        return illm_launch_status();
    }
    if (scratch != nullptr && !k_on && !(top_p < 1.0f)) {
        const size_t nc = (size_t)B * n_chunks;
        float* cmax = reinterpret_cast<float*>(scratch);
        float* csum = cmax + nc;
        illm_launch(sample_chunk_kernel<false>, dim3(n_chunks, B), dim3(SK_THREADS), 0, s, logits, V, ld, z_scratch,
                    last_tokens, n_last, 1.0f / temp, penalty, top_k, cmax, csum, (int*)nullptr, (float*)nullptr,
                    (int*)nullptr);
        illm_launch(sample_temp_final_kernel, dim3(B), dim3(SK_THREADS), 0, s, (const float*)z_scratch, V, n_chunks,
                    (const float*)cmax, (const float*)csum, uniforms, out);
        return illm_launch_status();
    }
    illm_launch(sample_kernel, dim3(B), dim3(SAMPLE_THREADS), 0, s, logits, V, ld, z_scratch, last_tokens, n_last, temp,
                penalty, top_k, top_p, uniforms, out, (const int*)nullptr);
    return illm_launch_status();
}

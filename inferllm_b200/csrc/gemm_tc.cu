// bfloat16 matrix product on the 5th-generation tensor cores:  C[M, N] = X[M, K] . W[N, K]^T
// with float32 accumulation in tensor memory.
//
// Both operands are K-major (rows contiguous in K), which is how activations [tokens, K] and
// weights [out, in] lie in memory, so neither is ever transposed (the reference calls
// cublasSgemm(OP_T, OP_N, ...) on the same layouts, src/kern/gpu/kernel_gpu.cu:420-435; formula
// src/kern/naive/naive.cpp:363-379).
//
// One block computes a tile D[128, BN] = A[128 rows, K-range] . B[BN rows, K-range]^T:
//   warp 0   one thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of [128 x 64] and
//            [BN x 64] operand tiles into a ring of shared-memory stages, arming a "full" mbarrier
//            per stage with the byte count;
//   warp 1   owns the tensor memory (tcgen05.alloc) and one thread issues tcgen05.mma
//            (M = 128, N = BN, K = 16, four per stage), then tcgen05.commit on the stage's "empty"
//            barrier so that the loader may refill it, and on a last barrier for the epilogue;
//   warps 2-5 read the accumulators with tcgen05.ld (a thread per row of the tile) and store.
// Two orientations share the kernel.  Prompts (many tokens): A = X, B = W, BN up to 256, a thread
// stores a row of C.  Decoding (at most 64 tokens): A = W, B = X ("swap"), so that the weight rows
// fill the 128 lanes of the MMA and the few tokens are its N; a warp then stores 32 consecutive
// outputs of one token.  For decoding the K range is also split over blockIdx.z, so that some 300
// blocks stream the weights with every SM busy; the partial sums go to a workspace and a second
// kernel adds them in ascending order of the split (the result does not depend on timing).
// Rows beyond M or N and columns beyond K are zero-filled by the TMA unit, so any M, any N and
// any K that is a multiple of 8 (the 16-byte stride rule of tensor maps) is taken.
// Every wait on an mbarrier is bounded: after the limit the thread raises the error word and
// goes on, so a fault in the pipeline ends the kernel instead of hanging the GPU.
#include "tc_common.cuh"

// D[ra, rb] = sum_k A[ra, k] B[rb, k];  SWAP = false: C[ra * ldc + rb];  SWAP = true: C[rb * ldc + ra].
#define TC_MAX_STAGES 12

template <int BN, bool SWAP, typename TOut, bool GATED = false>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               TOut* __restrict__ C, long long split_stride, int ldc, int RA, int RB, int k_iters_total,
               int k_iters_per_split, int STAGES, int* __restrict__ err) {
    constexpr unsigned A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2;
    constexpr unsigned TMEM_COLS = BN < 32 ? 32 : BN;
    constexpr unsigned IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(BN >> 3) << 17) | ((unsigned)(TC_BM >> 4) << 24);
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * TC_MAX_STAGES + 1];
    __shared__ unsigned tmem_holder;

    // operand tiles start on a 1024-byte boundary of the shared window (the swizzle's period)
    const unsigned a_base = (tc_smem_u32(smem_raw) + 1023u) & ~1023u, b_base = a_base + STAGES * A_BYTES;
    const unsigned full0 = tc_smem_u32(&bars[0]), empty0 = tc_smem_u32(&bars[TC_MAX_STAGES]);
    const unsigned done_bar = tc_smem_u32(&bars[2 * TC_MAX_STAGES]);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ra0 = blockIdx.x * TC_BM, rb0 = blockIdx.y * BN;
    const int k_begin = blockIdx.z * k_iters_per_split;
    int k_end = k_begin + k_iters_per_split;
    if (k_end > k_iters_total) k_end = k_iters_total;
    const int n_k = k_end - k_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init(done_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(tc_smem_u32(&tmem_holder)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = tmem_holder;
    // Everything above (barriers, tensor memory) was set up while the previous kernel drained, and
    // the kernel after this one may begin its own set-up now.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            // The weights never depend on an earlier kernel: the first ring of weight tiles is
            // requested before waiting for the previous kernel, so that the memory system is
            // already streaming when the activations become valid.
            const int n_pre = n_k < STAGES ? n_k : STAGES;
            for (int i = 0; i < n_pre; i++) {
                mbar_expect_tx(full0 + 8 * i, A_BYTES + B_BYTES);
                const int kx = (k_begin + i) * TC_BK;
                if (SWAP) tma_load_2d(a_base + i * A_BYTES, &map_a, kx, ra0, full0 + 8 * i);
                else tma_load_2d(b_base + i * B_BYTES, &map_b, kx, rb0, full0 + 8 * i);
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int i = 0; i < n_pre; i++) {
                const int kx = (k_begin + i) * TC_BK;
                if (SWAP) tma_load_2d(b_base + i * B_BYTES, &map_b, kx, rb0, full0 + 8 * i);
                else tma_load_2d(a_base + i * A_BYTES, &map_a, kx, ra0, full0 + 8 * i);
            }
            bool alive = true;
            for (int i = n_pre; i < n_k && alive; i++) {
                const int s = i % STAGES;
                alive = mbar_wait(empty0 + 8 * s, ((i / STAGES) - 1) & 1, err);
                if (!alive) break;
                mbar_expect_tx(full0 + 8 * s, A_BYTES + B_BYTES);
                const int kx = (k_begin + i) * TC_BK;
                tma_load_2d(a_base + s * A_BYTES, &map_a, kx, ra0, full0 + 8 * s);
                tma_load_2d(b_base + s * B_BYTES, &map_b, kx, rb0, full0 + 8 * s);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool alive = true;
            for (int i = 0; i < n_k && alive; i++) {
                const int s = i % STAGES;
                alive = mbar_wait(full0 + 8 * s, (i / STAGES) & 1, err);
                if (!alive) break;
                tc_fence_after();
#pragma unroll
                for (int kk = 0; kk < TC_BK / 16; kk++) {
                    const unsigned long long da = umma_desc_sw128(a_base + s * A_BYTES + kk * 32);
                    const unsigned long long db = umma_desc_sw128(b_base + s * B_BYTES + kk * 32);
                    umma_bf16(tmem, da, db, IDESC, (i > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(empty0 + 8 * s);   // arrives when these MMAs have read the stage
            }
            umma_commit(done_bar);             // arrives when every MMA of the tile is done
        }
    } else {
        // epilogue: warp w may touch the 32 lanes of tensor memory of its quadrant w % 4
        const int quad = warp & 3;
        asm volatile("griddepcontrol.wait;" ::: "memory");   // before any store: the output may alias
        // lanes leave the polling loop one by one: together again before the warp-wide tcgen05.ld
        const bool ok = __all_sync(0xffffffffu, mbar_wait(done_bar, 0, err));
        tc_fence_after();
        const int ra = ra0 + quad * 32 + lane;
        TOut* Cz = C + (size_t)blockIdx.z * split_stride;
        if (ok && n_k > 0) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (rb0 + c0 >= RB) break;   // uniform over the warp
                float v[16];
                tmem_ld16(tmem + ((unsigned)(quad * 32) << 16) + (unsigned)c0, v);
                if (SWAP && GATED) {
                    // weight rows 2i, 2i + 1 are gate and up of output i: neighbouring lanes hold them,
                    // the even lane writes silu(gate) * up (ldc = outputs per token)
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const float up = __shfl_xor_sync(0xffffffffu, v[j], 1);
                        const int rb = rb0 + c0 + j;
                        if (!(lane & 1) && rb < RB && ra + 1 < RA)
                            store_out<TOut>(Cz + (size_t)rb * ldc + (ra >> 1), (v[j] / (1.0f + __expf(-v[j]))) * up);
                    }
                } else if (SWAP) {
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int rb = rb0 + c0 + j;
                        if (rb < RB && ra < RA) store_out<TOut>(Cz + (size_t)rb * ldc + ra, v[j]);
                    }
                } else if (ra < RA) {
                    TOut* dst = Cz + (size_t)ra * ldc + rb0 + c0;
                    if (rb0 + c0 + 16 <= RB && ((ldc & 7) == 0)) {
                        store8(dst, v);
                        store8(dst + 8, v + 8);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j++)
                            if (rb0 + c0 + j < RB) store_out<TOut>(dst + j, v[j]);
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// C[i] = sum over splits (ascending) of partial[s][i]
template <typename TOut>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, TOut* __restrict__ C, long long n, int splits) {
    pdl_grid_sync();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float acc = 0.f;
    for (int s = 0; s < splits; s++) acc += partial[(size_t)s * n + i];
    store_out<TOut>(C + i, acc);
}

// ---- host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// Tensor map of a row-major bfloat16 matrix [rows, K]; boxes of [box_rows, 64], 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return ILLM_ERR_BAD_ARG;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : ILLM_ERR_BAD_ARG;
}

static int g_tc_stages_override = 0;   // set through illm_gemm_bf16_tc_tune, for measurements

// Stages of the operand ring: as many bytes in flight per SM as its shared memory allows, shared
// between the blocks that will be resident on it together.
static int pick_stages(int stage_bytes, long long n_blocks, int k_iters_per_block) {
    if (g_tc_stages_override > 0) return g_tc_stages_override;
    const int per_sm = (int)((n_blocks + 147) / 148);
    const int resident = per_sm < 1 ? 1 : (per_sm > 3 ? 3 : per_sm);
    // an SM has 227 KB; a block costs its ring, 1 KB of alignment slack, 1 KB that the system keeps
    // and its few static bytes
    int stages = (227 * 1024 / resident - 2560) / stage_bytes;
    if (stages > TC_MAX_STAGES) stages = TC_MAX_STAGES;
    if (stages > k_iters_per_block) stages = k_iters_per_block;
    return stages < 2 ? 2 : stages;
}

template <int BN, bool SWAP, typename TOut, bool GATED = false>
static int launch_tc(const CUtensorMap& ma, const CUtensorMap& mb, TOut* C, long long split_stride, int ldc,
                     int RA, int RB, int k_iters, int splits, int* err, cudaStream_t s) {
    const int stage_bytes = TC_BM * TC_BK * 2 + BN * TC_BK * 2;
    const int per_split = (k_iters + splits - 1) / splits;
    dim3 grid((RA + TC_BM - 1) / TC_BM, (RB + BN - 1) / BN, splits);
    const int stages = pick_stages(stage_bytes, (long long)grid.x * grid.y * grid.z, per_split);
    const size_t smem = (size_t)stages * stage_bytes + 1024;
    auto kern = gemm_tc_kernel<BN, SWAP, TOut, GATED>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    illm_launch(kern, dim3(grid), dim3(TC_THREADS), smem, s, ma, mb, C, split_stride, ldc, RA, RB, k_iters, per_split, stages, err);
    return illm_launch_status();
}

extern "C" int illm_gemm_bf16_tc_tune(int stages) {
    g_tc_stages_override = stages;
    return 0;
}

template <typename TOut>
static int run_tc(const void* X, const void* W, TOut* out, int M, int N, int K, float* ws, int splits, int* err,
                  cudaStream_t s, int skip_reduce) {
    const int k_iters = (K + TC_BK - 1) / TC_BK;
    CUtensorMap ma, mb;
    int rc;
    if (M <= 64) {
        // decoding: A = W (its rows on the 128 lanes), B = X, out[m * N + n]
        const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
        if ((rc = make_map(&ma, W, N, K, TC_BM)) != 0) return rc;
        if ((rc = make_map(&mb, X, M, K, bn)) != 0) return rc;
        if (splits > 1) {
            // every split must own at least one K slice
            const int per = (k_iters + splits - 1) / splits;
            splits = (k_iters + per - 1) / per;
        }
        if (splits > 1) {
            const long long n = (long long)M * N;
            if (bn == 16) rc = launch_tc<16, true, float>(ma, mb, ws, n, N, N, M, k_iters, splits, err, s);
            else if (bn == 32) rc = launch_tc<32, true, float>(ma, mb, ws, n, N, N, M, k_iters, splits, err, s);
            else rc = launch_tc<64, true, float>(ma, mb, ws, n, N, N, M, k_iters, splits, err, s);
            if (rc != 0 || skip_reduce) return rc;
            illm_launch(splitk_reduce_kernel<TOut>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, ws, out, n, splits);
            return illm_launch_status();
        }
        if (bn == 16) return launch_tc<16, true, TOut>(ma, mb, out, 0, N, N, M, k_iters, 1, err, s);
        if (bn == 32) return launch_tc<32, true, TOut>(ma, mb, out, 0, N, N, M, k_iters, 1, err, s);
        return launch_tc<64, true, TOut>(ma, mb, out, 0, N, N, M, k_iters, 1, err, s);
    }
    // prompts: A = X (tokens on the lanes), B = W
    if ((rc = make_map(&ma, X, M, K, TC_BM)) != 0) return rc;
    if (N >= 256) {
        if ((rc = make_map(&mb, W, N, K, 256)) != 0) return rc;
        return launch_tc<256, false, TOut>(ma, mb, out, 0, N, M, N, k_iters, 1, err, s);
    }
    if ((rc = make_map(&mb, W, N, K, 128)) != 0) return rc;
    return launch_tc<128, false, TOut>(ma, mb, out, 0, N, M, N, k_iters, 1, err, s);
}

// out_dtype: ILLM_BF16 or ILLM_F32.  `ws`: float workspace of splits * M * N elements (splits > 1
// is honoured for M <= 64 only).  X and W must be 16-byte aligned, K a multiple of 8.
// skip_reduce != 0 (with splits > 1): the slices stay in `ws` for a consumer that adds them up itself
// (illm_add_rmsnorm_partials, illm_rope_kv_write_partials) and `out` is not written.
extern "C" int illm_gemm_bf16_tc(const void* X, const void* W, void* out, int out_dtype, int M, int N, int K,
                                 float* ws, int splits, int* err, void* stream, int skip_reduce) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K & 7) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15) || splits < 1) return ILLM_ERR_BAD_ARG;
    if (splits > 1 && ws == nullptr) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (out_dtype == ILLM_BF16) return run_tc<bf16>(X, W, (bf16*)out, M, N, K, ws, splits, err, s, skip_reduce);
    if (out_dtype == ILLM_F32) return run_tc<float>(X, W, (float*)out, M, N, K, ws, splits, err, s, skip_reduce);
    return ILLM_ERR_BAD_ARG;
}

// Decode-sized product (M <= 64) of a gated feed-forward's packed weight, whose rows are gate and up
// of an output in turn: out[M, N / 2] = silu(gate) * up in bfloat16, straight from the accumulator
// (formula src/kern/naive/naive.cpp:80-89), without splitting K.
extern "C" int illm_gemm_bf16_tc_gated(const void* X, const void* W, void* out, int M, int N, int K, int* err,
                                       void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || (N & 1) || K <= 0 || (K & 7) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int k_iters = (K + TC_BK - 1) / TC_BK;
    CUtensorMap ma, mb;
    int rc;
    const int bn = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    if ((rc = make_map(&ma, W, N, K, TC_BM)) != 0) return rc;
    if ((rc = make_map(&mb, X, M, K, bn)) != 0) return rc;
    bf16* o = (bf16*)out;
    if (bn == 16) return launch_tc<16, true, bf16, true>(ma, mb, o, 0, N / 2, N, M, k_iters, 1, err, s);
    if (bn == 32) return launch_tc<32, true, bf16, true>(ma, mb, o, 0, N / 2, N, M, k_iters, 1, err, s);
    return launch_tc<64, true, bf16, true>(ma, mb, o, 0, N / 2, N, M, k_iters, 1, err, s);
}

// out[i] = sum over slices (ascending) of ws[z][i]: the stand-alone form of the reduction.
extern "C" int illm_splitk_reduce(const float* ws, void* out, int out_dtype, long long n, int splits, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (out_dtype == ILLM_BF16) illm_launch(splitk_reduce_kernel<bf16>, dim3(blocks), dim3(256), 0, s, ws, (bf16*)out, n, splits);
    else if (out_dtype == ILLM_F32) illm_launch(splitk_reduce_kernel<float>, dim3(blocks), dim3(256), 0, s, ws, (float*)out, n, splits);
    else return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}

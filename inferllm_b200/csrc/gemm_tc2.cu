// bfloat16 matrix product for prompts on pairs of SMs:  C[M, N] = X[M, K] . W[N, K]^T,
// tcgen05.mma with cta_group::2, float32 accumulation in tensor memory.
//
// Two blocks of a cluster share one 256 x 256 output tile.  Block r of the pair holds token rows
// [128 r, 128 r + 128) of the tile (its A operand and its half of the accumulator) and loads only
// weight rows [128 r, 128 r + 128) of the tile's 256: the pair's MMA (issued by block 0 for both)
// reads each half of the weight tile from the block that holds it.  Per 64-wide slice of K a block
// therefore moves 32 KB through its shared memory instead of the 48 KB of a 128 x 256 tile on one
// SM, which is what bounds the one-SM kernel (gemm_tc.cu) at about 1.2 PF/s.
// The pairs are persistent: pair p walks tiles p, p + pairs, ... (token tiles of one weight panel
// next to each other, so that a panel comes from HBM once and from L2 otherwise), the TMA ring
// runs across tile borders, and each block owns two accumulators of 256 columns in tensor memory,
// so that the epilogue warps drain tile i while the tensor cores work on tile i + 1.
//   warp 0 (both blocks)  one thread issues the block's TMA loads (cp.async.bulk.tensor with
//                         .cta_group::2: the bytes are counted on block 0's "full" barrier);
//   warp 1 (block 0)      one thread waits for "full", issues four MMAs (M 256, N 256, K 16) per
//                         stage, commits to the "empty" barriers of both blocks, and after a tile's
//                         last slice to both blocks' "accumulator full" barriers;
//   warps 2-5 (both)      tcgen05.ld of the block's own 128 rows, conversion, stores; then an
//                         arrival on block 0's "accumulator empty" barrier.
// EPI 0: plain store.  EPI 1: gated activation: the weight's rows are gate and up of an output in
// turn, a thread of the epilogue then holds both for 8 outputs in the 16 columns it reads, and writes
// silu(gate) * up (formula src/kern/naive/naive.cpp:80-89; the reference runs w3, w1, Silu and Mul
// as four operators, src/core/graph.cpp:57-79), so the packed projection never goes to memory.
// Every wait is bounded and raises the error word.
#include "tc_common.cuh"

#define T2_BN 256
#define T2_HALF 128
#define T2_STAGES 6
#define T2_THREADS 192

__device__ __forceinline__ unsigned cluster_ctarank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in block `rank` of the cluster
__device__ __forceinline__ unsigned map_to_cta(unsigned addr, unsigned rank) {
    unsigned out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
    return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into this block's shared memory whose completion is counted on `bar`, a barrier of
// either block of the pair given by its cluster address
__device__ __forceinline__ void tma_load_2d_pair(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(unsigned tmem_d, unsigned long long da, unsigned long long db,
                                               unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives, when the MMAs issued so far are done, on the barrier at this offset in both blocks
__device__ __forceinline__ void umma_commit_pair(unsigned bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"((unsigned short)3) : "memory");
}

template <int EPI, typename TOut>
__global__ void __launch_bounds__(T2_THREADS)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                TOut* __restrict__ C, int ldc, int RA, int RB, int k_iters, int* __restrict__ err) {
    constexpr unsigned A_BYTES = TC_BM * TC_BK * 2, B_BYTES = T2_HALF * TC_BK * 2;
    constexpr unsigned TMEM_COLS = 512;
    // M 256 (the pair), N 256, bfloat16 x bfloat16 -> float32, both operands K-major
    constexpr unsigned IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(T2_BN >> 3) << 17) | ((unsigned)(256 >> 4) << 24);
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const unsigned base = tc_smem_u32(smem_raw);
    const unsigned a_base = base, b_base = a_base + T2_STAGES * A_BYTES;
    const unsigned bars = b_base + T2_STAGES * B_BYTES;
    const unsigned full0 = bars, empty0 = bars + 8 * T2_STAGES;
    const unsigned acc_full0 = bars + 16 * T2_STAGES, acc_empty0 = acc_full0 + 16;
    unsigned* tmem_holder = reinterpret_cast<unsigned*>(smem_raw + (bars - base) + 16 * T2_STAGES + 32);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const unsigned rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int n_m = (RA + 255) / 256, n_n = (RB + T2_BN - 1) / T2_BN;
    const int n_tiles = n_m * n_n;

    if ((base & 1023u) != 0) {          // no static shared memory is declared: cannot happen; never run misaligned
        if (threadIdx.x == 0) atomicExch(err, TC_ERR_TIMEOUT + 2);
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < T2_STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full0 + 8 * b, 1);
            mbar_init(acc_empty0 + 8 * b, 8);      // four epilogue warps in each of the two blocks
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(tc_smem_u32(tmem_holder)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                 // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const unsigned tmem = *tmem_holder;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

    if (warp == 0) {
        if (lane == 0) {
            bool alive = true, waited = false;
            int it = 0;
            const unsigned full_leader = map_to_cta(full0, 0);      // block 0 counts the bytes of both
            for (int t = pair; t < n_tiles && alive; t += n_pairs) {
                const int ra0 = (t % n_m) * 256 + (int)rank * 128, rb0 = (t / n_m) * T2_BN + (int)rank * T2_HALF;
                for (int k = 0; k < k_iters && alive; k++, it++) {
                    const int s = it % T2_STAGES;
                    if (it >= T2_STAGES) alive = mbar_wait(empty0 + 8 * s, ((it / T2_STAGES) - 1) & 1, err);
                    if (!alive) break;
                    // block 0 arms its barrier with the bytes of both blocks
                    if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * (A_BYTES + B_BYTES));
                    tma_load_2d_pair(b_base + s * B_BYTES, &map_b, k * TC_BK, rb0, full_leader + 8 * s);   // weights first
                    if (!waited) {
                        asm volatile("griddepcontrol.wait;" ::: "memory");
                        waited = true;
                    }
                    tma_load_2d_pair(a_base + s * A_BYTES, &map_a, k * TC_BK, ra0, full_leader + 8 * s);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            bool alive = true;
            int it = 0, ti = 0;
            for (int t = pair; t < n_tiles && alive; t += n_pairs, ti++) {
                const int buf = ti & 1;
                if (ti >= 2) alive = mbar_wait(acc_empty0 + 8 * buf, ((ti >> 1) - 1) & 1, err);
                tc_fence_after();
                for (int k = 0; k < k_iters && alive; k++, it++) {
                    const int s = it % T2_STAGES;
                    alive = mbar_wait(full0 + 8 * s, (it / T2_STAGES) & 1, err);
                    if (!alive) break;
                    tc_fence_after();
#pragma unroll
                    for (int kk = 0; kk < TC_BK / 16; kk++) {
                        const unsigned long long da = umma_desc_sw128(a_base + s * A_BYTES + kk * 32);
                        const unsigned long long db = umma_desc_sw128(b_base + s * B_BYTES + kk * 32);
                        umma_bf16_pair(tmem + buf * T2_BN, da, db, IDESC, (k > 0 || kk > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(empty0 + 8 * s);
                }
                umma_commit_pair(acc_full0 + 8 * buf);
            }
        }
    } else {
        const int quad = warp & 3;
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const unsigned acc_empty_leader = map_to_cta(acc_empty0, 0);
        bool alive = true;
        int ti = 0;
        for (int t = pair; t < n_tiles && alive; t += n_pairs, ti++) {
            const int buf = ti & 1;
            const int ra = (t % n_m) * 256 + (int)rank * 128 + quad * 32 + lane, rb0 = (t / n_m) * T2_BN;
            // lanes leave the polling loop one by one: together again before the warp-wide tcgen05.ld
            alive = __all_sync(0xffffffffu, mbar_wait(acc_full0 + 8 * buf, (ti >> 1) & 1, err));
            if (!alive) break;
            tc_fence_after();
            const unsigned tbase = tmem + ((unsigned)(quad * 32) << 16) + (unsigned)(buf * T2_BN);
            if (EPI == 1) {
                // columns 2i, 2i + 1 of the product are gate and up of output i (ldc = outputs per row)
#pragma unroll 1
                for (int c0 = 0; c0 < T2_BN; c0 += 16) {
                    if (rb0 + c0 >= RB) break;
                    float v[16], r[8];
                    tmem_ld16(tbase + c0, v);
#pragma unroll
                    for (int j = 0; j < 8; j++) r[j] = (v[2 * j] / (1.0f + __expf(-v[2 * j]))) * v[2 * j + 1];
                    if (ra < RA) {
                        const int o0 = (rb0 + c0) / 2;
                        TOut* dst = C + (size_t)ra * ldc + o0;
                        if (o0 + 8 <= ldc && ((ldc & 7) == 0)) {
                            store8(dst, r);
                        } else {
#pragma unroll
                            for (int j = 0; j < 8; j++)
                                if (o0 + j < ldc) store_out<TOut>(dst + j, r[j]);
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < T2_BN; c0 += 16) {
                    if (rb0 + c0 >= RB) break;
                    float v[16];
                    tmem_ld16(tbase + c0, v);
                    if (ra < RA) {
                        TOut* dst = C + (size_t)ra * ldc + rb0 + c0;
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
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty_leader + 8 * buf);
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();                 // neither block leaves while the other may still touch it
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side

typedef CUresult (*T2EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int t2_make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, int box_rows) {
    static T2EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (T2EncodeTiledFn)p;
    }
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

template <int EPI, typename TOut>
static int t2_launch(const void* X, const void* W, TOut* out, int ldc, int M, int N, int K, int* err, cudaStream_t s) {
    CUtensorMap ma, mb;
    int rc;
    if ((rc = t2_make_map(&ma, X, M, K, TC_BM)) != 0) return rc;
    if ((rc = t2_make_map(&mb, W, N, K, T2_HALF)) != 0) return rc;
    const int k_iters = (K + TC_BK - 1) / TC_BK;
    const size_t smem = (size_t)T2_STAGES * (TC_BM * TC_BK * 2 + T2_HALF * TC_BK * 2) + 16 * T2_STAGES + 32 + 16;
    auto kern = gemm_tc2_kernel<EPI, TOut>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int n_tiles = ((M + 255) / 256) * ((N + T2_BN - 1) / T2_BN);
    int pairs = sms / 2;
    if (pairs > n_tiles) pairs = n_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(T2_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_illm_pdl ? 2 : 1;
    g_illm_launches++;
    cudaLaunchKernelEx(&cfg, kern, ma, mb, out, ldc, M, N, k_iters, err);
    return illm_launch_status();
}

// C = X . W^T (epi 0, C [M, N]) or the gated activation of it (epi 1, C [M, N / 2], W's rows gate
// and up of an output in turn).  X, W 16-byte aligned; K % 8 == 0.
extern "C" int illm_gemm_bf16_tc2(const void* X, const void* W, void* out, int out_dtype, int epi, int M, int N,
                                  int K, int* err, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K & 7) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return ILLM_ERR_BAD_ARG;
    if (epi == 1 && (N & 1)) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (epi == 0 && out_dtype == ILLM_BF16) return t2_launch<0, bf16>(X, W, (bf16*)out, N, M, N, K, err, s);
    if (epi == 0 && out_dtype == ILLM_F32) return t2_launch<0, float>(X, W, (float*)out, N, M, N, K, err, s);
    if (epi == 1 && out_dtype == ILLM_BF16) return t2_launch<1, bf16>(X, W, (bf16*)out, N / 2, M, N, K, err, s);
    return ILLM_ERR_BAD_ARG;
}

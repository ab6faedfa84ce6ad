// Causal attention of whole prompts over the paged cache, bfloat16, on the tensor cores.
//
// Flash-attention style: the score matrix is never written out.  A block owns 128 consecutive
// query tokens of one (sequence, head) and walks the keys of that sequence in blocks of 64, from
// the cache pages into shared memory (cp.async, double buffered, XOR-swizzled rows so that
// ldmatrix is conflict-free); each of its 4 warps holds 32 query rows, so that every K or V
// fragment it fetches from shared memory feeds two MMAs: S = Q K^T and O += P V are
// m16n8k16 bfloat16 MMAs with float32 accumulators, and the running maximum, the sum and the
// exponentials are float32 (exp2 on scores pre-multiplied by log2 e).  P is rounded to bfloat16
// for the second product.  This replaces the reference's four launches over a materialised
// [head, T, past+T] float32 score tensor (src/kern/gpu/kernel_gpu.cu:576-591, :504-536, :78-125,
// :593-609; formulas src/kern/naive/naive.cpp:606-632, :531-553, :209-240, :664-691) and its
// grouped-head variant that loops over heads (:688-756).
//
// It reads keys through the sequence's page table, so it serves prompts that start at position 0
// as well as chunks that continue a sequence (past > 0); a window (keys older than `window`
// positions hidden) only adds a mask and a later first block.  Any page size, any number of
// heads and groups; head size 64 or 128 (other sizes take the generic kernel).
// The MMA path here is the warp-level one (mma.sync); the prompts' attention is a few percent of
// a prefill step's arithmetic next to the projections.
#include <math.h>

#include "common.cuh"

#define FA_BN 64
#define FA_THREADS 128

__device__ __forceinline__ unsigned smem_u32(const void* p) {
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void cp_async_16(unsigned dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// element offset of 16-byte chunk `c` of row `r` in a [rows][D] bfloat16 tile with swizzled chunks
template <int D> __device__ __forceinline__ int swz(int r, int c) { return r * D + ((c ^ (r & 7)) << 3); }

template <int D, int MT>
__global__ void __launch_bounds__(FA_THREADS)
attention_prefill_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ kc,
                         const bf16* __restrict__ vc, const int* __restrict__ block_table, int max_pages,
                         const int* __restrict__ cu_q, const int* __restrict__ seq_lens,
                         bf16* __restrict__ out, int nh, int nkv, int page_size, int window,
                         float scale_log2e) {
    pdl_grid_sync();
    constexpr int BM = 4 * MT * 16;   // query rows of the block: MT m-tiles of 16 rows per warp
    constexpr int CH = D / 8;         // 16-byte chunks per row
    constexpr int KS = D / 16;        // k-steps of Q K^T
    constexpr int NT_D = D / 8;       // n-tiles of the output
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* Ks = Qs + BM * D;                 // [2][FA_BN][D]
    bf16* Vs = Ks + 2 * FA_BN * D;          // [2][FA_BN][D]

    // the last tiles of a prompt see the most keys: they are started first
    const int b = blockIdx.z, h = blockIdx.y, tile = gridDim.x - 1 - blockIdx.x;
    const int q0 = cu_q[b], qlen = cu_q[b + 1] - q0;
    const int row0 = tile * BM;
    if (row0 >= qlen) return;
    const int total = seq_lens[b], past = total - qlen;
    const int hk = h / (nh / nkv);
    const int rows_here = (qlen - row0 < BM) ? qlen - row0 : BM;
    const int first_pos = past + row0, last_pos = first_pos + rows_here - 1;
    const int lo_key = (window > 0 && first_pos - window + 1 > 0) ? first_pos - window + 1 : 0;
    const int jb0 = lo_key / FA_BN, jb1 = last_pos / FA_BN;
    const int* bt = block_table + (size_t)b * max_pages;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int mtx = lane >> 3;          // which 8x8 matrix of an ldmatrix.x4 this lane addresses
    const int wrow0 = warp * MT * 16;   // first row of this warp inside the tile

    // ---- Q tile -> shared (zero rows beyond the sequence's tokens)
    for (int i = tid; i < BM * CH; i += FA_THREADS) {
        const int r = i / CH, c = i % CH;
        const bool ok = r < rows_here;
        const bf16* src = ok ? q + (size_t)(q0 + row0 + r) * q_stride + (size_t)h * D + c * 8 : q;
        cp_async_16(smem_u32(Qs + swz<D>(r, c)), src, ok ? 16 : 0);
    }
    auto load_kv = [&](int jb, int buf) {
        bf16* kd = Ks + buf * FA_BN * D;
        bf16* vd = Vs + buf * FA_BN * D;
        for (int i = tid; i < FA_BN * CH; i += FA_THREADS) {
            const int r = i / CH, c = i % CH;
            const int key = jb * FA_BN + r;
            // keys below the window of the tile's first row are seen by no row of the tile, and the
            // pages that held them may have gone back to the pool already (table entry -1): such rows
            // are zero-filled instead of read, so masked scores meet zeros in V, never stale data
            bool ok = key <= last_pos && key >= lo_key;
            size_t off = 0;
            if (ok) {
                const int page = bt[key / page_size];
                ok = page >= 0;
                if (ok) off = (((size_t)page * nkv + hk) * page_size + (key % page_size)) * D + c * 8;
            }
            cp_async_16(smem_u32(kd + swz<D>(r, c)), kc + off, ok ? 16 : 0);
            cp_async_16(smem_u32(vd + swz<D>(r, c)), vc + off, ok ? 16 : 0);
        }
    };
    load_kv(jb0, 0);
    cp_async_commit();

    // ---- per-warp state: MT x 16 query rows; this thread owns rows g and g+8 of each m-tile
    float o[MT][NT_D][4];
    float m_run[MT][2], l_run[MT][2];
    int pos_r[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
#pragma unroll
        for (int i = 0; i < NT_D; i++) o[mt][i][0] = o[mt][i][1] = o[mt][i][2] = o[mt][i][3] = 0.f;
#pragma unroll
        for (int e = 0; e < 2; e++) {
            m_run[mt][e] = -INFINITY;
            l_run[mt][e] = 0.f;
            const int r = wrow0 + mt * 16 + g + e * 8;
            pos_r[mt][e] = (r < rows_here) ? first_pos + r : last_pos;
        }
    }
    // a warp whose rows all lie beyond the prompt has nothing to compute (it still helps loading)
    const bool warp_active = wrow0 < rows_here;
    const int warp_last_pos = (wrow0 + MT * 16 - 1 < rows_here) ? first_pos + wrow0 + MT * 16 - 1 : last_pos;

    for (int jb = jb0; jb <= jb1; jb++) {
        const int buf = (jb - jb0) & 1;
        if (jb < jb1) load_kv(jb + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const bf16* kb = Ks + buf * FA_BN * D;
        const bf16* vb = Vs + buf * FA_BN * D;
        const int key0 = jb * FA_BN;
        // keys of this block all lie after the warp's last row: nothing to add for this warp
        if (warp_active && key0 <= warp_last_pos) {
            // S = Q K^T : (MT x 16) x 64 per warp
            float s[MT][FA_BN / 8][4];
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int i = 0; i < FA_BN / 8; i++) s[mt][i][0] = s[mt][i][1] = s[mt][i][2] = s[mt][i][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                unsigned qf[MT][4];
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    const int r = wrow0 + mt * 16 + (mtx & 1) * 8 + (lane & 7);
                    ldmatrix_x4(qf[mt][0], qf[mt][1], qf[mt][2], qf[mt][3],
                                smem_u32(Qs + swz<D>(r, ks * 2 + (mtx >> 1))));
                }
#pragma unroll
                for (int np = 0; np < FA_BN / 16; np++) {
                    const int r = np * 16 + (mtx >> 1) * 8 + (lane & 7);
                    unsigned b0, b1, b2, b3;
                    ldmatrix_x4(b0, b1, b2, b3, smem_u32(kb + swz<D>(r, ks * 2 + (mtx & 1))));
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) {
                        mma_bf16(s[mt][np * 2], qf[mt], b0, b1);
                        mma_bf16(s[mt][np * 2 + 1], qf[mt], b2, b3);
                    }
                }
            }

            // scale, mask, running maximum; P = exp2(S - m) packed as A fragments
            const bool need_mask = (key0 + FA_BN - 1 > first_pos + wrow0) || (window > 0);
            unsigned pf[MT][FA_BN / 16][4];
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                float m_new[2] = {m_run[mt][0], m_run[mt][1]};
#pragma unroll
                for (int nt = 0; nt < FA_BN / 8; nt++) {
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        float v = s[mt][nt][e] * scale_log2e;
                        if (need_mask) {
                            const int key = key0 + nt * 8 + t4 * 2 + (e & 1);
                            const int pr = pos_r[mt][e >> 1];
                            if (key > pr || (window > 0 && key < pr - window + 1)) v = -INFINITY;
                        }
                        s[mt][nt][e] = v;
                        m_new[e >> 1] = fmaxf(m_new[e >> 1], v);
                    }
                }
                float corr[2], m_use[2], psum[2] = {0.f, 0.f};
#pragma unroll
                for (int e = 0; e < 2; e++) {
                    m_new[e] = fmaxf(m_new[e], __shfl_xor_sync(0xffffffffu, m_new[e], 1));
                    m_new[e] = fmaxf(m_new[e], __shfl_xor_sync(0xffffffffu, m_new[e], 2));
                    m_use[e] = (m_new[e] == -INFINITY) ? 0.f : m_new[e];
                    corr[e] = (m_run[mt][e] == -INFINITY) ? 0.f : fast_exp2(m_run[mt][e] - m_use[e]);
                    m_run[mt][e] = m_new[e];
                }
#pragma unroll
                for (int nt = 0; nt < FA_BN / 8; nt++) {
                    const float p0 = fast_exp2(s[mt][nt][0] - m_use[0]), p1 = fast_exp2(s[mt][nt][1] - m_use[0]);
                    const float p2 = fast_exp2(s[mt][nt][2] - m_use[1]), p3 = fast_exp2(s[mt][nt][3] - m_use[1]);
                    psum[0] += p0 + p1;
                    psum[1] += p2 + p3;
                    pf[mt][nt >> 1][(nt & 1) * 2] = pack_bf16(p0, p1);
                    pf[mt][nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
                }
#pragma unroll
                for (int e = 0; e < 2; e++) l_run[mt][e] = l_run[mt][e] * corr[e] + psum[e];
#pragma unroll
                for (int i = 0; i < NT_D; i++) {
                    o[mt][i][0] *= corr[0];
                    o[mt][i][1] *= corr[0];
                    o[mt][i][2] *= corr[1];
                    o[mt][i][3] *= corr[1];
                }
            }
            // O += P V
#pragma unroll
            for (int ks = 0; ks < FA_BN / 16; ks++) {
#pragma unroll
                for (int np = 0; np < NT_D / 2; np++) {
                    const int r = ks * 16 + (mtx & 1) * 8 + (lane & 7);
                    unsigned b0, b1, b2, b3;
                    ldmatrix_x4_trans(b0, b1, b2, b3, smem_u32(vb + swz<D>(r, np * 2 + (mtx >> 1))));
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) {
                        mma_bf16(o[mt][np * 2], pf[mt][ks], b0, b1);
                        mma_bf16(o[mt][np * 2 + 1], pf[mt][ks], b2, b3);
                    }
                }
            }
        }
        __syncthreads();   // everyone is done with this buffer before the next load overwrites it
    }
    cp_async_wait<0>();

    // ---- normalise and store
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
#pragma unroll
        for (int e = 0; e < 2; e++) {
            float lsum = l_run[mt][e];
            lsum += __shfl_xor_sync(0xffffffffu, lsum, 1);
            lsum += __shfl_xor_sync(0xffffffffu, lsum, 2);
            const int r = wrow0 + mt * 16 + g + e * 8;
            if (r >= rows_here) continue;
            const float inv = 1.0f / lsum;
            bf16* dst = out + ((size_t)(q0 + row0 + r) * nh + h) * D;
#pragma unroll
            for (int i = 0; i < NT_D; i++) {
                __nv_bfloat162 v = __floats2bfloat162_rn(o[mt][i][e * 2] * inv, o[mt][i][e * 2 + 1] * inv);
                *reinterpret_cast<__nv_bfloat162*>(dst + i * 8 + t4 * 2) = v;
            }
        }
    }
}

template <int D>
static int launch(const void* q, int q_stride, const void* kc, const void* vc, const int* block_table,
                  int max_pages, const int* cu_q, const int* seq_lens, void* out, int B, int max_q, int nh,
                  int nkv, int page_size, int window, float scale, cudaStream_t s) {
    constexpr int MT = 2;
    constexpr int BM = 4 * MT * 16;
    const size_t smem = (size_t)(BM + 4 * FA_BN) * D * sizeof(bf16);
    auto kern = attention_prefill_kernel<D, MT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid((max_q + BM - 1) / BM, nh, B);
    illm_launch(kern, dim3(grid), dim3(FA_THREADS), smem, s, (const bf16*)q, q_stride, (const bf16*)kc, (const bf16*)vc, block_table,
                                        max_pages, cu_q, seq_lens, (bf16*)out, nh, nkv, page_size, window,
                                        scale * 1.4426950408889634f);
    return illm_launch_status();
}

extern "C" int illm_attention_prefill(const void* q, int q_stride, const void* kc, const void* vc,
                                      const int* block_table, int max_pages, const int* cu_q,
                                      const int* seq_lens, void* out, int B, int max_q, int nh, int nkv,
                                      int d, int page_size, int window, float scale, void* stream) {
    if (B <= 0 || max_q <= 0) return 0;
    if (nkv <= 0 || nh % nkv || nh > 65535 || B > 65535 || (q_stride & 7)) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (d == 128)
        return launch<128>(q, q_stride, kc, vc, block_table, max_pages, cu_q, seq_lens, out, B, max_q, nh, nkv,
                           page_size, window, scale, s);
    if (d == 64)
        return launch<64>(q, q_stride, kc, vc, block_table, max_pages, cu_q, seq_lens, out, B, max_q, nh, nkv,
                          page_size, window, scale, s);
    return ILLM_ERR_BAD_ARG;
}

// Causal attention of whole prompts over the paged cache on the 5th-generation tensor cores.
//
// One block owns two tiles of 128 consecutive query tokens of one (sequence, head); each tile has
// four softmax warps of its own, a thread of which owns one query row, which is also one lane of
// tensor memory.  Keys and values come in blocks of 64 straight from the cache pages by TMA
// (128-byte swizzle, double buffered) and serve both tiles.  Per tile and block of keys:
//   S = Q K^T      tcgen05.mma, M = 128 rows, N = 64 keys, K = head size, accumulator in the
//                  tile's tensor memory columns [0, 64)
//   softmax        each thread reads its row of S with tcgen05.ld, scales, masks (causal, window),
//                  keeps the running maximum and sum in float32, and writes P = exp2(S - max) as
//                  bfloat16 into shared memory in the swizzled layout the tensor core reads
//   O_blk = P V    tcgen05.mma with V as an MN-major operand (the cache keeps [position, channel]),
//                  into columns [64, 64 + head size); the thread adds it to its row of O, which it
//                  keeps in registers, after scaling O by exp2(old max - new max)
// so the score matrix never exists in memory and nothing of the running state crosses threads.
// One more thread issues the MMAs and another the TMA copies; the MMAs of one tile run while the
// softmax warps of the other tile work, and the scores of a tile's next block are issued right
// behind its P V.  Formulas as in the reference (src/kern/naive/naive.cpp:606-632, :531-553,
// :209-240, :664-691), which materialises S in float32 and runs four launches over it
// (src/kern/gpu/kernel_gpu.cu:576-609, :504-536, :78-125).
// Takes head sizes 64 and 128 and page sizes that are multiples of 64; any number of heads and
// groups; prompts that start at 0 or continue a sequence; an optional window.  Every wait is
// bounded and raises the error word instead of hanging.
#include <cuda.h>
#include <math.h>

#include "common.cuh"

#define FT_BM 128            // rows of a query tile = lanes of tensor memory
#define FT_MAX_TILES 2       // query tiles per block: one's softmax overlaps the other's MMAs
#define FT_BN 64             // keys per ring block (one page piece)
#define FT_THREADS(tiles) (32 * (4 * (tiles) + 2))
#define FT_WAIT_LIMIT (1 << 22)
#define FT_ERR_TIMEOUT 5

namespace {

__device__ __forceinline__ unsigned s_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool bar_wait(unsigned bar, unsigned parity, int* err) {
    for (int i = 0; i < FT_WAIT_LIMIT; i++) {
        unsigned ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        if (i > 256) __nanosleep(20);
    }
    atomicExch(err, FT_ERR_TIMEOUT);
    return false;
}
__device__ __forceinline__ void tma_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major tile, rows of 128 bytes, 128-byte swizzle: 8-row groups 1024 bytes apart.
__device__ __forceinline__ unsigned long long desc_kmajor(unsigned addr) {
    return (unsigned long long)((addr & 0x3FFFF) >> 4) | ((unsigned long long)1 << 16) |
           ((unsigned long long)(1024 >> 4) << 32) | ((unsigned long long)1 << 46) | ((unsigned long long)2 << 61);
}
// MN-major tile (rows = positions of K, 128 bytes = 64 channels of MN each), 128-byte swizzle:
// 8-position groups 1024 bytes apart (stride), the next 64 channels `lbo_bytes` further (leading).
__device__ __forceinline__ unsigned long long desc_mnmajor(unsigned addr, unsigned lbo_bytes) {
    return (unsigned long long)((addr & 0x3FFFF) >> 4) | ((unsigned long long)(lbo_bytes >> 4) << 16) |
           ((unsigned long long)(1024 >> 4) << 32) | ((unsigned long long)1 << 46) | ((unsigned long long)2 << 61);
}
__device__ __forceinline__ void mma_bf16_ss(unsigned tmem_d, unsigned long long da, unsigned long long db,
                                            unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float* v) {
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

}  // namespace

template <int D, int FT_TILES>
__global__ void __launch_bounds__(FT_THREADS(FT_TILES), FT_TILES == 1 ? 2 : 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table,
                            int max_pages, const int* __restrict__ cu_q, const int* __restrict__ seq_lens,
                            bf16* __restrict__ out, int nh, int nkv, int page_size, int window,
                            float scale_log2e, int* __restrict__ err) {
    constexpr int FT_MMA_WARP = 4 * FT_TILES, FT_TMA_WARP = 4 * FT_TILES + 1;
    constexpr int NA = D / 64;                            // 64-channel atoms of the head
    constexpr unsigned Q_TILE = FT_BM * D * 2;            // one query tile: [NA][128 rows][128 B]
    constexpr unsigned KV_BYTES = FT_BN * D * 2;          // K: [NA][64 keys][128 B]; V: the same shape
    constexpr unsigned P_TILE = FT_BM * FT_BN * 2;        // [128 rows][128 B] = 64 keys
    constexpr unsigned Q_ATOM = 128 * 128, KV_ATOM = FT_BN * 128;
    constexpr unsigned TMEM_COLS = 256 * FT_TILES, TILE_COLS = 256, O_COL = FT_BN;   // one-tile blocks share an SM
    constexpr unsigned IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(FT_BN >> 3) << 17) | ((unsigned)(FT_BM >> 4) << 24);
    constexpr unsigned IDESC_O = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(D >> 3) << 17) | ((unsigned)(FT_BM >> 4) << 24);

    // No static shared memory: the dynamic window then starts on a 1024-byte boundary (the
    // swizzle's period) and two one-tile blocks fit an SM.  Barriers sit behind the tiles.
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const unsigned base = s_u32(smem_raw);
    const unsigned q_s = base, k_s = q_s + FT_TILES * Q_TILE, v_s = k_s + 2 * KV_BYTES, p_s = v_s + 2 * KV_BYTES;
    const unsigned bars0 = p_s + FT_TILES * P_TILE;
    unsigned* tmem_holder_p = reinterpret_cast<unsigned*>(smem_raw + (bars0 - base) + 11 * 8);
    const unsigned q_full = bars0, kv_full0 = bars0 + 8, kv_empty0 = bars0 + 24;
    const unsigned s_full0 = bars0 + 40, p_full0 = bars0 + 56, o_full0 = bars0 + 72;
    if ((base & 1023u) != 0) {          // cannot happen without static shared memory; never run misaligned
        if (threadIdx.x == 0) atomicExch(err, FT_ERR_TIMEOUT + 1);
        return;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        bar_init(q_full, 1);
        for (int i = 0; i < 2; i++) {
            bar_init(kv_full0 + 8 * i, 1);
            bar_init(kv_empty0 + 8 * i, 1);
            bar_init(s_full0 + 8 * i, 1);
            bar_init(p_full0 + 8 * i, FT_BM);
            bar_init(o_full0 + 8 * i, 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == FT_MMA_WARP) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(s_u32(tmem_holder_p)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_before();
    __syncthreads();
    fence_after();
    const unsigned tmem = *tmem_holder_p;
    pdl_grid_sync();

    // ---- which rows and keys.  The block owns FT_TILES query tiles of 128 rows; the last blocks of
    // a prompt see the most keys and start first.
    const int b = blockIdx.z, h = blockIdx.y, cta_tile = gridDim.x - 1 - blockIdx.x;
    const int q0 = cu_q[b], qlen = cu_q[b + 1] - q0;
    const int cta_row0 = cta_tile * FT_TILES * FT_BM;
    const int total = seq_lens[b], past = total - qlen;
    const int hk = h / (nh / nkv);
    const int cta_rows = (qlen - cta_row0 < FT_TILES * FT_BM) ? qlen - cta_row0 : FT_TILES * FT_BM;   // <= 0: nothing
    const bool cta_has_rows = cta_rows > 0;
    const int cta_first_pos = past + cta_row0, cta_last_pos = cta_first_pos + cta_rows - 1;
    const int lo_key = (window > 0 && cta_first_pos - window + 1 > 0) ? cta_first_pos - window + 1 : 0;
    const int jb0 = lo_key / FT_BN;                               // first key block of the block's ring
    const int n_blocks = cta_has_rows ? cta_last_pos / FT_BN - jb0 + 1 : 0;
    const int* bt = block_table + (size_t)b * max_pages;
    // per tile: rows, and the range [lo_t, hi_t) of ring blocks it needs (ring block i = key block jb0 + i)
    int rows_t[FT_TILES], lo_t[FT_TILES], hi_t[FT_TILES];
#pragma unroll
    for (int t = 0; t < FT_TILES; t++) {
        const int r0 = cta_row0 + t * FT_BM;
        rows_t[t] = (qlen - r0 < FT_BM) ? qlen - r0 : FT_BM;
        if (rows_t[t] < 0) rows_t[t] = 0;
        const int fp = past + r0, lp = fp + rows_t[t] - 1;
        const int lk = (window > 0 && fp - window + 1 > 0) ? fp - window + 1 : 0;
        lo_t[t] = rows_t[t] > 0 ? lk / FT_BN - jb0 : 0;
        hi_t[t] = rows_t[t] > 0 ? lp / FT_BN - jb0 + 1 : 0;
    }

    if (warp == FT_TMA_WARP) {
        // ---- TMA producer
        if (lane == 0 && cta_has_rows) {
            bar_expect_tx(q_full, FT_TILES * Q_TILE);
            for (int t = 0; t < FT_TILES; t++)
                for (int a = 0; a < NA; a++)
                    tma_2d(q_s + t * Q_TILE + a * Q_ATOM, &map_q, h * D + 64 * a, q0 + cta_row0 + t * FT_BM, q_full);
            bool alive = true;
            for (int i = 0; i < n_blocks && alive; i++) {
                const int buf = i & 1;
                if (i >= 2) alive = bar_wait(kv_empty0 + 8 * buf, ((i >> 1) - 1) & 1, err);
                if (!alive) break;
                const int key0 = (jb0 + i) * FT_BN;
                const int page = bt[key0 / page_size];
                const int row = (page * nkv + hk) * page_size + (key0 % page_size);
                bar_expect_tx(kv_full0 + 8 * buf, 2 * KV_BYTES);
                for (int a = 0; a < NA; a++) {
                    tma_2d(k_s + buf * KV_BYTES + a * KV_ATOM, &map_k, 64 * a, row, kv_full0 + 8 * buf);
                    tma_2d(v_s + buf * KV_BYTES + a * KV_ATOM, &map_v, 64 * a, row, kv_full0 + 8 * buf);
                }
            }
        }
    } else if (warp == FT_MMA_WARP) {
        // ---- MMA issuer: for every ring block, P V of each tile as soon as its P is there, and the
        // scores of the next block for that tile right behind it
        if (lane == 0 && cta_has_rows) {
            bool alive = bar_wait(q_full, 0, err);
            int n_s[FT_TILES], n_p[FT_TILES];     // how many S / P V products each tile has been issued
#pragma unroll
            for (int t = 0; t < FT_TILES; t++) n_s[t] = n_p[t] = 0;
            auto issue_s = [&](int t, int i) {
                const int buf = i & 1;
                if (!bar_wait(kv_full0 + 8 * buf, (i >> 1) & 1, err)) return false;
                fence_after();
#pragma unroll
                for (int kk = 0; kk < D / 16; kk++) {
                    const unsigned qo = t * Q_TILE + (kk >> 2) * Q_ATOM + (kk & 3) * 32;
                    const unsigned ko = buf * KV_BYTES + (kk >> 2) * KV_ATOM + (kk & 3) * 32;
                    mma_bf16_ss(tmem + t * TILE_COLS, desc_kmajor(q_s + qo), desc_kmajor(k_s + ko), IDESC_S, kk > 0);
                }
                mma_commit(s_full0 + 8 * t);
                n_s[t]++;
                return true;
            };
#pragma unroll
            for (int t = 0; t < FT_TILES; t++)
                if (alive && lo_t[t] == 0 && hi_t[t] > 0) alive = issue_s(t, 0);
            for (int i = 0; i < n_blocks && alive; i++) {
                const int buf = i & 1;
#pragma unroll
                for (int t = 0; t < FT_TILES; t++) {
                    if (!alive) break;
                    if (i >= lo_t[t] && i < hi_t[t]) {
                        alive = bar_wait(p_full0 + 8 * t, n_p[t] & 1, err);
                        if (!alive) break;
                        fence_after();
#pragma unroll
                        for (int ks = 0; ks < FT_BN / 16; ks++)
                            mma_bf16_ss(tmem + t * TILE_COLS + O_COL, desc_kmajor(p_s + t * P_TILE + ks * 32),
                                        desc_mnmajor(v_s + buf * KV_BYTES + ks * 16 * 128, KV_ATOM), IDESC_O, ks > 0);
                        mma_commit(o_full0 + 8 * t);
                        n_p[t]++;
                    }
                    // after the last tile's products: everything that reads this ring block has been
                    // issued, so its completion frees the block for the loader
                    if (t == FT_TILES - 1) mma_commit(kv_empty0 + 8 * buf);
                    if (i + 1 >= lo_t[t] && i + 1 < hi_t[t]) alive = issue_s(t, i + 1);
                }
            }
        }
    } else if (warp < 4 * FT_TILES) {
        // ---- softmax and accumulation: thread = query row = lane of tensor memory
        const int t = warp >> 2;                          // which tile this warp group works on
        const int r = threadIdx.x & 127;                  // row inside the tile
        const unsigned lane_addr = ((unsigned)((warp & 3) * 32) << 16) + t * TILE_COLS;
        const int first_pos = cta_first_pos + t * FT_BM;
        const int last_pos = first_pos + rows_t[t] - 1;
        const int pos = (r < rows_t[t]) ? first_pos + r : last_pos;
        float m_run = -INFINITY, l_run = 0.f;
        float o_reg[D];
#pragma unroll
        for (int c = 0; c < D; c++) o_reg[c] = 0.f;
        bool alive = true;
        int n = 0;                                        // blocks this tile has processed
        for (int i = lo_t[t]; i < hi_t[t] && alive; i++, n++) {
            const int key0 = (jb0 + i) * FT_BN;
            const int buf = i & 1;
            alive = bar_wait(s_full0 + 8 * t, n & 1, err);
            if (!alive) break;
            fence_after();
            const bool need_mask = (key0 + FT_BN - 1 > first_pos) || (window > 0);
            // pass 1: the row's maximum over this block (the scale is positive: it is applied to
            // the maximum, not to every score)
            float mx = -INFINITY;
#pragma unroll 1
            for (int c0 = 0; c0 < FT_BN; c0 += 32) {
                float v[32];
                tmem_ld32(tmem + lane_addr + c0, v);
                if (need_mask) {
#pragma unroll
                    for (int c = 0; c < 32; c++) {
                        const int key = key0 + c0 + c;
                        const bool hide = key > pos || (window > 0 && key < pos - window + 1);
                        mx = fmaxf(mx, hide ? -INFINITY : v[c]);
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 32; c++) mx = fmaxf(mx, v[c]);
                }
            }
            const float m_new = fmaxf(m_run, mx * scale_log2e);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
            const float corr = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_use);
            m_run = m_new;
            // pass 2: P = exp2(S * scale - max) -> shared memory (row r of the K-major, swizzled P tile)
            float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
            for (int c0 = 0; c0 < FT_BN; c0 += 32) {
                float v[32];
                tmem_ld32(tmem + lane_addr + c0, v);
                if (need_mask) {
#pragma unroll
                    for (int c = 0; c < 32; c++) {
                        const int key = key0 + c0 + c;
                        const bool hide = key > pos || (window > 0 && key < pos - window + 1);
                        v[c] = hide ? 0.f : fast_exp2(fmaf(v[c], scale_log2e, -m_use));
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 32; c++) v[c] = fast_exp2(fmaf(v[c], scale_log2e, -m_use));
                }
#pragma unroll
                for (int c = 0; c < 32; c++) ps[c & 3] += v[c];
                const unsigned row_addr = p_s + t * P_TILE + r * 128;
#pragma unroll
                for (int q4 = 0; q4 < 4; q4++) {     // four 16-byte chunks of 8 keys
                    const int chunk = (c0 >> 3) + q4;
                    uint4 u;
                    __nv_bfloat162* hp = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
                    for (int e = 0; e < 4; e++) hp[e] = __floats2bfloat162_rn(v[q4 * 8 + 2 * e], v[q4 * 8 + 2 * e + 1]);
                    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(row_addr + ((chunk ^ (r & 7)) << 4)),
                                 "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w) : "memory");
                }
            }
            const float psum = (ps[0] + ps[1]) + (ps[2] + ps[3]);
            l_run = l_run * corr + psum;
            // the block's last ring block may hold positions beyond the sequence: whatever the cache
            // has there must not reach the product (0 x NaN), so those rows of V are cleared (by
            // every tile that uses the block: the writes are the same)
            if (key0 + FT_BN - 1 > cta_last_pos) {
                alive = bar_wait(kv_full0 + 8 * buf, (i >> 1) & 1, err);
                const int key = key0 + r;
                if (r < FT_BN && key > cta_last_pos) {
#pragma unroll
                    for (int a = 0; a < NA; a++) {
                        const unsigned row_addr = v_s + buf * KV_BYTES + a * KV_ATOM + r * 128;
#pragma unroll
                        for (int q8 = 0; q8 < 8; q8++)
                            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(row_addr + q8 * 16), "r"(0u) : "memory");
                    }
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            fence_before();
            bar_arrive(p_full0 + 8 * t);
            // O = O * corr + P V
            alive = alive && bar_wait(o_full0 + 8 * t, n & 1, err);
            if (!alive) break;
            fence_after();
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
                float v[32];
                tmem_ld32(tmem + lane_addr + O_COL + c0, v);
#pragma unroll
                for (int c = 0; c < 32; c++) o_reg[c0 + c] = fmaf(o_reg[c0 + c], corr, v[c]);
            }
        }
        if (alive && r < rows_t[t]) {
            const float inv = 1.0f / l_run;
            bf16* dst = out + ((size_t)(q0 + cta_row0 + t * FT_BM + r) * nh + h) * D;
#pragma unroll
            for (int c = 0; c < D; c += 8) {
                float f[8];
#pragma unroll
                for (int e = 0; e < 8; e++) f[e] = o_reg[c + e] * inv;
                store8(dst + c, f);
            }
        }
    }
    fence_before();
    __syncthreads();
    if (warp == FT_MMA_WARP) {
        fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side

typedef CUresult (*FtEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static FtEncodeTiledFn ft_encode_fn() {
    static FtEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (FtEncodeTiledFn)p;
    }
    return fn;
}

// bfloat16 matrix [rows, cols] with a row pitch of `pitch` elements; boxes of [box_rows, 64].
static int ft_make_map(CUtensorMap* map, const void* ptr, long long rows, long long cols, long long pitch, int box_rows) {
    FtEncodeTiledFn fn = ft_encode_fn();
    if (!fn) return ILLM_ERR_BAD_ARG;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : ILLM_ERR_BAD_ARG;
}

template <int D, int TILES>
static int ft_launch(const void* q, int q_stride, int T, const void* kc, const void* vc, long long n_pages,
                     const int* block_table, int max_pages, const int* cu_q, const int* seq_lens, void* out, int B,
                     int max_q, int nh, int nkv, int page_size, int window, float scale, int* err, cudaStream_t s) {
    CUtensorMap mq, mk, mv;
    int rc;
    if ((rc = ft_make_map(&mq, q, T, (long long)nh * D, q_stride, FT_BM)) != 0) return rc;
    const long long kv_rows = n_pages * nkv * page_size;
    if ((rc = ft_make_map(&mk, kc, kv_rows, D, D, FT_BN)) != 0) return rc;
    if ((rc = ft_make_map(&mv, vc, kv_rows, D, D, FT_BN)) != 0) return rc;
    const size_t smem = (size_t)TILES * FT_BM * D * 2 + 4 * (size_t)FT_BN * D * 2 +
                        (size_t)TILES * FT_BM * FT_BN * 2 + 128;   // + barriers and the tensor-memory address
    auto kern = attention_prefill_tc_kernel<D, TILES>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid((max_q + TILES * FT_BM - 1) / (TILES * FT_BM), nh, B);
    illm_launch(kern, grid, dim3(FT_THREADS(TILES)), smem, s, mq, mk, mv, block_table, max_pages, cu_q, seq_lens,
                (bf16*)out, nh, nkv, page_size, window, scale * 1.4426950408889634f, err);
    return illm_launch_status();
}

// Two query tiles per block when that still gives every SM several blocks; one tile otherwise
// (short prompts: more, smaller blocks balance the causal triangle better).
template <int D>
static int ft_pick(const void* q, int q_stride, int T, const void* kc, const void* vc, long long n_pages,
                   const int* block_table, int max_pages, const int* cu_q, const int* seq_lens, void* out, int B,
                   int max_q, int nh, int nkv, int page_size, int window, float scale, int* err, cudaStream_t s) {
    const long long blocks2 = (long long)((max_q + 2 * FT_BM - 1) / (2 * FT_BM)) * nh * B;
    if (blocks2 >= 4 * 148)
        return ft_launch<D, 2>(q, q_stride, T, kc, vc, n_pages, block_table, max_pages, cu_q, seq_lens, out, B, max_q,
                               nh, nkv, page_size, window, scale, err, s);
    return ft_launch<D, 1>(q, q_stride, T, kc, vc, n_pages, block_table, max_pages, cu_q, seq_lens, out, B, max_q,
                           nh, nkv, page_size, window, scale, err, s);
}

// q: the packed projection [T, q_stride] whose first nh*d columns are the query heads;
// kc, vc: one cache entry [n_pages, nkv, page_size, d].
extern "C" int illm_attention_prefill_tc(const void* q, int q_stride, int T, const void* kc, const void* vc,
                                         long long n_pages, const int* block_table, int max_pages,
                                         const int* cu_q, const int* seq_lens, void* out, int B, int max_q, int nh,
                                         int nkv, int d, int page_size, int window, float scale, int* err,
                                         void* stream) {
    if (B <= 0 || max_q <= 0) return 0;
    if (nkv <= 0 || nh % nkv || nh > 65535 || B > 65535 || (q_stride & 7) || page_size % 64 ||
        ((uintptr_t)q & 15) || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15))
        return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (d == 128)
        return ft_pick<128>(q, q_stride, T, kc, vc, n_pages, block_table, max_pages, cu_q, seq_lens, out, B, max_q,
                              nh, nkv, page_size, window, scale, err, s);
    if (d == 64)
        return ft_pick<64>(q, q_stride, T, kc, vc, n_pages, block_table, max_pages, cu_q, seq_lens, out, B, max_q,
                             nh, nkv, page_size, window, scale, err, s);
    return ILLM_ERR_BAD_ARG;
}

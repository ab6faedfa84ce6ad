// Causal attention of whole prompts over the paged cache on the 5th-generation tensor cores.
//
// One block owns a tile of 128 consecutive query tokens of one (sequence, head); the tiles with the
// most keys before them start first, on all heads.  Two blocks share an SM.
// Four softmax warps: a thread owns one query row, which is also one lane of tensor memory.
// Keys and values come in blocks of 64 straight from the cache pages by TMA (128-byte swizzle), K
// through a ring of three stages and V through a ring of two.  Tensor memory of a block, 256
// columns: two score buffers S0, S1 of 64 columns and the output accumulator O of `head size`.
// Per block of keys i:
//   S(i) = Q K^T   tcgen05.mma, M = 128 rows, N = 64 keys, K = head size, into S(i & 1).  It is
//                  issued one block ahead: the tensor core computes S(i+1) while the softmax warps
//                  work on S(i).
//   softmax        a thread reads its row of S(i) with tcgen05.ld (once), masks (causal, window),
//                  and writes P = exp2(S * scale - m) as bfloat16 pairs back over S(i) with
//                  tcgen05.st: P never goes through shared memory.  m is the row's reference
//                  maximum; it follows the true maximum only when that has grown by more than 8
//                  (a factor of 256, harmless in float32), because moving it means rescaling O in
//                  tensor memory (tcgen05.ld, multiply, tcgen05.st), and after the first blocks of
//                  a row that is rare.  The sum of P is kept against the same reference, so the
//                  result is the exact softmax whatever the reference was.
//   O += P V       tcgen05.mma with P read from tensor memory (operand A) and V as an MN-major
//                  shared-memory operand (the cache keeps [position, channel]), accumulating in O.
// The score matrix never exists in memory, nothing of the running state crosses threads, and O is
// read once, at the end.  One more thread issues the MMAs and another the TMA copies.
// Formulas as in the reference (src/kern/naive/naive.cpp:606-632, :531-553, :209-240, :664-691),
// which materialises S in float32 and runs four launches over it
// (src/kern/gpu/kernel_gpu.cu:576-609, :504-536, :78-125).
// Takes head sizes 64 and 128 and page sizes that are multiples of 64; any number of heads and
// groups; prompts that start at 0 or continue a sequence; an optional window.  Every wait is
// bounded and raises the error word instead of hanging.
#include <cuda.h>
#include <math.h>

#include "common.cuh"

#define FT_BM 128            // rows of a query tile = lanes of tensor memory
#define FT_BN 64             // keys per ring block (one page piece)
#define FT_KSTAGES 3
#define FT_VSTAGES 2
#define FT_THREADS 192       // 4 softmax warps, the MMA warp, the TMA warp
#define FT_WAIT_CLOCKS (1LL << 31)
#define FT_ERR_TIMEOUT 5
#define FT_RESCALE_STEP 8.0f // how far (in powers of two) the maximum may run ahead of the reference

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
// Waits for the phase with the given parity: mbarrier.try_wait suspends the thread until the phase
// completes or a hardware time limit passes, so a waiting warp issues next to nothing (a test_wait
// spin took issue slots from the softmax warps of its SM sub-partition, which are bound by them).
// Bounded by about a second of clocks; false (and the error word set) when that runs out.
__device__ __forceinline__ bool bar_try(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool bar_wait(unsigned bar, unsigned parity, int* err) {
    if (bar_try(bar, parity)) return true;
    const long long t0 = clock64();
    do {
        if (bar_try(bar, parity)) return true;
    } while (clock64() - t0 < FT_WAIT_CLOCKS);
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
// D[tmem] (+)= A[smem] . B[smem]
__device__ __forceinline__ void mma_bf16_ss(unsigned tmem_d, unsigned long long da, unsigned long long db,
                                            unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] . B[smem]: A's row r is lane r, its K elements packed in pairs per column
__device__ __forceinline__ void mma_bf16_ts(unsigned tmem_d, unsigned tmem_a, unsigned long long db,
                                            unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 consecutive columns of this thread's lane; the values may be used after tmem_wait_ld()
__device__ __forceinline__ void tmem_ld32_issue(unsigned taddr, unsigned* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
// Waits for the loads issued so far and pins the registers behind the wait: the compiler sees
// each of them redefined here, so no use can move above it.
template <int N> __device__ __forceinline__ void tmem_wait_ld(unsigned* r) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < N; i++) asm volatile("" : "+r"(r[i]));
}
__device__ __forceinline__ void tmem_st32(unsigned taddr, const unsigned* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

}  // namespace

// Two float32 operations in one instruction (pairs in 64-bit registers) and the maximum of three:
// the softmax warps are bound by how many instructions they issue per score, not by a pipe.
__device__ __forceinline__ unsigned long long f2_pack(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long f2_fma(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ unsigned long long f2_add(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

template <int D>
__global__ void __launch_bounds__(FT_THREADS, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_table,
                            int max_pages, const int* __restrict__ cu_q, const int* __restrict__ seq_lens,
                            bf16* __restrict__ out, int nh, int nkv, int page_size, int window,
                            float scale_log2e, int* __restrict__ err) {
    constexpr int FT_MMA_WARP = 4, FT_TMA_WARP = 5;
    constexpr int NA = D / 64;                            // 64-channel atoms of the head
    constexpr unsigned Q_TILE = FT_BM * D * 2;            // the query tile: [NA][128 rows][128 B]
    constexpr unsigned KV_BYTES = FT_BN * D * 2;          // K: [NA][64 keys][128 B]; V: the same shape
    constexpr unsigned Q_ATOM = 128 * 128, KV_ATOM = FT_BN * 128;
    constexpr unsigned TMEM_COLS = 256, S_COLS = FT_BN, O_COL = 2 * FT_BN;
    constexpr unsigned IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(FT_BN >> 3) << 17) | ((unsigned)(FT_BM >> 4) << 24);
    constexpr unsigned IDESC_O = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(D >> 3) << 17) | ((unsigned)(FT_BM >> 4) << 24);

    // No static shared memory: the dynamic window then starts on a 1024-byte boundary (the
    // swizzle's period) and two blocks fit an SM.  Barriers sit behind the tiles.
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const unsigned base = s_u32(smem_raw);
    const unsigned q_s = base, k_s = q_s + Q_TILE, v_s = k_s + FT_KSTAGES * KV_BYTES;
    const unsigned bars0 = v_s + FT_VSTAGES * KV_BYTES;
    const unsigned q_full = bars0, k_full0 = bars0 + 8, k_empty0 = k_full0 + 8 * FT_KSTAGES;
    const unsigned v_full0 = k_empty0 + 8 * FT_KSTAGES, v_empty0 = v_full0 + 8 * FT_VSTAGES;
    const unsigned s_full0 = v_empty0 + 8 * FT_VSTAGES, p_full0 = s_full0 + 16, pv_done = p_full0 + 16;
    unsigned* tmem_holder_p = reinterpret_cast<unsigned*>(smem_raw + (pv_done + 8 - base));
    if ((base & 1023u) != 0) {          // cannot happen without static shared memory; never run misaligned
        if (threadIdx.x == 0) atomicExch(err, FT_ERR_TIMEOUT + 1);
        return;
    }

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    auto init_barriers = [&]() {
        auto one = [&](unsigned bar, unsigned count) { bar_init(bar, count); };
        one(q_full, 1);
        for (int i = 0; i < FT_KSTAGES; i++) {
            one(k_full0 + 8 * i, 1);
            one(k_empty0 + 8 * i, 1);
        }
        for (int i = 0; i < FT_VSTAGES; i++) {
            one(v_full0 + 8 * i, 1);
            one(v_empty0 + 8 * i, 1);
        }
        one(s_full0, 1);
        one(s_full0 + 8, 1);
        one(p_full0, FT_BM);               // one per score buffer: a fast warp may be a block ahead of a slow one
        one(p_full0 + 8, FT_BM);
        one(pv_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    };
    if (threadIdx.x == 0) init_barriers();
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

    // ---- which rows and keys.  One tile of 128 query rows per block.  Heads vary fastest over the
    // grid and the tiles of a prompt are numbered from its end, so the tiles with the most key
    // blocks (the causal mask gives tile t of a prompt t + 1 blocks of 128 keys) start first, on all
    // heads, and the short ones fill the SMs as those finish.  (Two tiles per block, the x-th from the
    // end and the x-th from the start, which gives all blocks equal work, was slower at every prompt
    // length: 52.5 against 50.2 us at 2,048 tokens of 32 heads, 138 against 101 us at 3,072.)
    const int b = blockIdx.z, h = blockIdx.x;
    const int q0 = cu_q[b], qlen = cu_q[b + 1] - q0;
    const int n_tiles = (qlen + FT_BM - 1) / FT_BM;
    const int tile = n_tiles - 1 - (int)blockIdx.y;           // < 0: this sequence is shorter than the longest
    const int row0 = tile * FT_BM;
    const int total = seq_lens[b], past = total - qlen;
    const int hk = h / (nh / nkv);
    const int rows = tile < 0 ? 0 : ((qlen - row0 < FT_BM) ? qlen - row0 : FT_BM);   // 0: nothing to do
    const bool has_rows = rows > 0;
    const int first_pos = past + row0, last_pos = first_pos + rows - 1;
    const int lo_key = (window > 0 && first_pos - window + 1 > 0) ? first_pos - window + 1 : 0;
    const int jb0 = lo_key / FT_BN;                                        // first key block
    const int n_blocks = has_rows ? last_pos / FT_BN - jb0 + 1 : 0;
    const int* bt = block_table + (size_t)b * max_pages;

    if (warp == FT_TMA_WARP) {
        // ---- TMA producer.  K(i) may be refilled once S(i-3) has been computed, V(i) once P V of
        // block i-2 has; the loop asks in the order in which those come true.
        if (lane == 0 && has_rows) {
            bar_expect_tx(q_full, Q_TILE);
            for (int a = 0; a < NA; a++) tma_2d(q_s + a * Q_ATOM, &map_q, h * D + 64 * a, q0 + row0, q_full);
            auto kv_row = [&](int i) {
                const int key0 = (jb0 + i) * FT_BN;
                return (bt[key0 / page_size] * nkv + hk) * page_size + (key0 % page_size);
            };
            bool alive = true;
            auto load_k = [&](int i) {
                const int st = i % FT_KSTAGES;
                if (i >= FT_KSTAGES && !bar_wait(k_empty0 + 8 * st, ((i / FT_KSTAGES) - 1) & 1, err)) return false;
                const int row = kv_row(i);
                bar_expect_tx(k_full0 + 8 * st, KV_BYTES);
                for (int a = 0; a < NA; a++) tma_2d(k_s + st * KV_BYTES + a * KV_ATOM, &map_k, 64 * a, row, k_full0 + 8 * st);
                return true;
            };
            auto load_v = [&](int i) {
                const int st = i % FT_VSTAGES;
                if (i >= FT_VSTAGES && !bar_wait(v_empty0 + 8 * st, ((i / FT_VSTAGES) - 1) & 1, err)) return false;
                const int row = kv_row(i);
                bar_expect_tx(v_full0 + 8 * st, KV_BYTES);
                for (int a = 0; a < NA; a++) tma_2d(v_s + st * KV_BYTES + a * KV_ATOM, &map_v, 64 * a, row, v_full0 + 8 * st);
                return true;
            };
            for (int i = 0; i < FT_KSTAGES && i < n_blocks && alive; i++) alive = load_k(i);
            for (int i = 0; i < FT_VSTAGES && i < n_blocks && alive; i++) alive = load_v(i);
            for (int i = 0; alive && (i + FT_KSTAGES < n_blocks || i + FT_VSTAGES < n_blocks); i++) {
                if (i + FT_KSTAGES < n_blocks) alive = load_k(i + FT_KSTAGES);
                if (alive && i + FT_VSTAGES < n_blocks) alive = load_v(i + FT_VSTAGES);
            }
        }
    } else if (warp == FT_MMA_WARP) {
        // ---- MMA issuer: S one block ahead of the softmax, P V as soon as P is there
        if (lane == 0 && has_rows) {
            bool alive = bar_wait(q_full, 0, err);
            auto issue_s = [&](int i) {
                const int st = i % FT_KSTAGES;
                if (!bar_wait(k_full0 + 8 * st, (i / FT_KSTAGES) & 1, err)) return false;
                fence_after();
#pragma unroll
                for (int kk = 0; kk < D / 16; kk++) {
                    const unsigned qo = (kk >> 2) * Q_ATOM + (kk & 3) * 32;
                    const unsigned ko = st * KV_BYTES + (kk >> 2) * KV_ATOM + (kk & 3) * 32;
                    mma_bf16_ss(tmem + (i & 1) * S_COLS, desc_kmajor(q_s + qo), desc_kmajor(k_s + ko), IDESC_S, kk > 0);
                }
                mma_commit(s_full0 + 8 * (i & 1));     // the scores are there
                mma_commit(k_empty0 + 8 * st);         // and the K stage has been read
                return true;
            };
            if (alive && n_blocks > 0) alive = issue_s(0);
            for (int i = 0; i < n_blocks && alive; i++) {
                // S(i+1) overwrites the buffer that held P(i-1); P V of block i-1 was issued before
                // and the tensor core runs its instructions in order
                if (i + 1 < n_blocks) alive = issue_s(i + 1);
                if (!alive) break;
                alive = bar_wait(p_full0 + 8 * (i & 1), (i >> 1) & 1, err);
                if (!alive) break;
                const int st = i % FT_VSTAGES;
                alive = bar_wait(v_full0 + 8 * st, (i / FT_VSTAGES) & 1, err);
                if (!alive) break;
                fence_after();
#pragma unroll
                for (int ks = 0; ks < FT_BN / 16; ks++)
                    mma_bf16_ts(tmem + O_COL, tmem + (i & 1) * S_COLS + ks * 8,
                                desc_mnmajor(v_s + st * KV_BYTES + ks * 16 * 128, KV_ATOM), IDESC_O, (i > 0 || ks > 0) ? 1u : 0u);
                mma_commit(v_empty0 + 8 * st);
                mma_commit(pv_done);
            }
        }
    } else {
        // ---- softmax: thread = query row = lane of tensor memory
        const int r = threadIdx.x & 127;
        const unsigned lane_addr = tmem + ((unsigned)(warp * 32) << 16);
        const int pos = (r < rows) ? first_pos + r : last_pos;
        float m_ref = -INFINITY, l_run = 0.f;
        bool alive = has_rows;
        for (int i = 0; i < n_blocks && alive; i++) {
            const int key0 = (jb0 + i) * FT_BN;
            // the lanes leave the polling loop one by one: they are brought together again (and agree on
            // the outcome) before the warp-wide tensor-memory instructions
            alive = __all_sync(0xffffffffu, bar_wait(s_full0 + 8 * (i & 1), (i >> 1) & 1, err));
            if (!alive) break;
            fence_after();
            const unsigned s_addr = lane_addr + (i & 1) * S_COLS;
            unsigned sr[FT_BN];
            tmem_ld32_issue(s_addr, sr);
            tmem_ld32_issue(s_addr + 32, sr + 32);
            tmem_wait_ld<FT_BN>(sr);
            const bool need_mask = (key0 + FT_BN - 1 > first_pos) || (window > 0);
            if (need_mask) {
#pragma unroll
                for (int c = 0; c < FT_BN; c++) {
                    const int key = key0 + c;
                    const bool hide = key > pos || (window > 0 && key < pos - window + 1);
                    if (hide) sr[c] = 0xff800000u;      // -inf
                }
            }
            // the row's maximum over this block (the scale is positive: it is applied to the maximum)
            float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
            for (int c = 0; c < FT_BN; c += 8) {
                mx0 = max3(mx0, __uint_as_float(sr[c]), __uint_as_float(sr[c + 1]));
                mx1 = max3(mx1, __uint_as_float(sr[c + 2]), __uint_as_float(sr[c + 3]));
                mx2 = max3(mx2, __uint_as_float(sr[c + 4]), __uint_as_float(sr[c + 5]));
                mx3 = max3(mx3, __uint_as_float(sr[c + 6]), __uint_as_float(sr[c + 7]));
            }
            const float m_new = fmaxf(m_ref, fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2e);
            // move the reference only when the maximum has run away from it (always at the first
            // finite maximum); the decision is the warp's, because the rescaling of O is
            const bool grown = m_new > m_ref + FT_RESCALE_STEP;      // true for m_ref = -inf, m_new finite
            bool pv_seen = false;
            if (__any_sync(0xffffffffu, grown)) {
                if (i > 0) {
                    pv_seen = true;
                    const float corr = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);   // m_new finite or both -inf
                    const float corr_use = (m_new == -INFINITY) ? 1.f : corr;
                    alive = __all_sync(0xffffffffu, bar_wait(pv_done, (i - 1) & 1, err));   // O holds blocks 0 .. i-1
                    if (!alive) break;
                    fence_after();
#pragma unroll 1
                    for (int c0 = 0; c0 < D; c0 += 32) {
                        unsigned orr[32];
                        tmem_ld32_issue(lane_addr + O_COL + c0, orr);
                        tmem_wait_ld<32>(orr);
#pragma unroll
                        for (int c = 0; c < 32; c++) orr[c] = __float_as_uint(__uint_as_float(orr[c]) * corr_use);
                        tmem_st32(lane_addr + O_COL + c0, orr);
                    }
                    tmem_wait_st();
                    l_run *= corr_use;
                }
                m_ref = m_new;
            }
            const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
            // P = exp2(S * scale - reference) as bfloat16 pairs over the first 32 columns of S(i)
            unsigned pr[FT_BN / 2];
            const unsigned long long scale2 = f2_pack(scale_log2e, scale_log2e), neg_m2 = f2_pack(-m_use, -m_use);
            unsigned long long psa = f2_pack(0.f, 0.f), psb = psa;
#pragma unroll
            for (int c = 0; c < FT_BN; c += 4) {
                float x0, x1, x2, x3;
                f2_unpack(f2_fma(f2_pack(__uint_as_float(sr[c]), __uint_as_float(sr[c + 1])), scale2, neg_m2), x0, x1);
                f2_unpack(f2_fma(f2_pack(__uint_as_float(sr[c + 2]), __uint_as_float(sr[c + 3])), scale2, neg_m2), x2, x3);
                const float p0 = fast_exp2(x0), p1 = fast_exp2(x1), p2 = fast_exp2(x2), p3 = fast_exp2(x3);   // exp2(-inf) = 0
                psa = f2_add(psa, f2_pack(p0, p1));
                psb = f2_add(psb, f2_pack(p2, p3));
                pr[c >> 1] = pack_bf16(p0, p1);
                pr[(c >> 1) + 1] = pack_bf16(p2, p3);
            }
            {
                float a0, a1, b0, b1;
                f2_unpack(psa, a0, a1);
                f2_unpack(psb, b0, b1);
                l_run += (a0 + a1) + (b0 + b1);
            }
            tmem_st32(s_addr, pr);
            tmem_wait_st();
            // the prompt's last block may hold positions beyond the sequence: whatever the cache
            // has there must not reach the product (0 x NaN), so those rows of V are cleared
            if (key0 + FT_BN - 1 > last_pos) {
                const int st = i % FT_VSTAGES;
                alive = __all_sync(0xffffffffu, bar_wait(v_full0 + 8 * st, (i / FT_VSTAGES) & 1, err));
                if (r < FT_BN && key0 + r > last_pos) {
#pragma unroll
                    for (int a = 0; a < NA; a++) {
                        const unsigned row_addr = v_s + st * KV_BYTES + a * KV_ATOM + r * 128;
#pragma unroll
                        for (int q8 = 0; q8 < 8; q8++)
                            asm volatile("st.shared.v4.u32 [%0], {%1,%1,%1,%1};" ::"r"(row_addr + q8 * 16), "r"(0u) : "memory");
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            }
            // Every phase of pv_done is observed, in order, before this thread lets the next one
            // begin: a wait on a phase's parity is only meaningful while the barrier is at most one
            // phase away.  P V of the previous block ended long ago by now; this does not stall.
            if (i > 0 && !pv_seen) alive = __all_sync(0xffffffffu, bar_wait(pv_done, (i - 1) & 1, err));
            fence_before();
            bar_arrive(p_full0 + 8 * (i & 1));
        }
        if (alive && n_blocks > 0) alive = __all_sync(0xffffffffu, bar_wait(pv_done, (n_blocks - 1) & 1, err));
        if (alive && n_blocks > 0) {
            fence_after();
            const float inv = 1.0f / l_run;
            bf16* dst = out + ((size_t)(q0 + row0 + r) * nh + h) * D;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                unsigned orr[32];
                tmem_ld32_issue(lane_addr + O_COL + c0, orr);
                tmem_wait_ld<32>(orr);
                if (r < rows) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        float f[8];
#pragma unroll
                        for (int e = 0; e < 8; e++) f[e] = __uint_as_float(orr[c + e]) * inv;
                        store8(dst + c0 + c, f);
                    }
                }
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

template <int D>
static int ft_launch(const void* q, int q_stride, int T, const void* kc, const void* vc, long long n_pages,
                     const int* block_table, int max_pages, const int* cu_q, const int* seq_lens, void* out, int B,
                     int max_q, int nh, int nkv, int page_size, int window, float scale, int* err, cudaStream_t s) {
    CUtensorMap mq, mk, mv;
    int rc;
    if ((rc = ft_make_map(&mq, q, T, (long long)nh * D, q_stride, FT_BM)) != 0) return rc;
    const long long kv_rows = n_pages * nkv * page_size;
    if ((rc = ft_make_map(&mk, kc, kv_rows, D, D, FT_BN)) != 0) return rc;
    if ((rc = ft_make_map(&mv, vc, kv_rows, D, D, FT_BN)) != 0) return rc;
    const size_t smem = (size_t)FT_BM * D * 2 + (size_t)(FT_KSTAGES + FT_VSTAGES) * FT_BN * D * 2 +
                        256;   // + barriers and the tensor-memory address
    auto kern = attention_prefill_tc_kernel<D>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(nh, (max_q + FT_BM - 1) / FT_BM, B);
    illm_launch(kern, grid, dim3(FT_THREADS), smem, s, mq, mk, mv, block_table, max_pages, cu_q, seq_lens,
                (bf16*)out, nh, nkv, page_size, window, scale * 1.4426950408889634f, err);
    return illm_launch_status();
}

// q: the packed projection [T, q_stride] whose first nh*d columns are the query heads;
// kc, vc: one cache entry [n_pages, nkv, page_size, d].
extern "C" int illm_attention_prefill_tc(const void* q, int q_stride, int T, const void* kc, const void* vc,
                                         long long n_pages, const int* block_table, int max_pages,
                                         const int* cu_q, const int* seq_lens, void* out, int B, int max_q, int nh,
                                         int nkv, int d, int page_size, int window, float scale, int* err,
                                         void* stream) {
    if (B <= 0 || max_q <= 0) return 0;
    if (nkv <= 0 || nh % nkv || max_q > 65535 * FT_BM || B > 65535 || (q_stride & 7) || page_size % 64 ||
        ((uintptr_t)q & 15) || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15))
        return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (d == 128)
        return ft_launch<128>(q, q_stride, T, kc, vc, n_pages, block_table, max_pages, cu_q, seq_lens, out, B, max_q,
                              nh, nkv, page_size, window, scale, err, s);
    if (d == 64)
        return ft_launch<64>(q, q_stride, T, kc, vc, n_pages, block_table, max_pages, cu_q, seq_lens, out, B, max_q,
                             nh, nkv, page_size, window, scale, err, s);
    return ILLM_ERR_BAD_ARG;
}

// Attention of single tokens over long paged caches, bfloat16, as a stream: K and V tiles come
// through a ring of shared-memory stages filled by TMA, and the query heads that share a KV head
// are the rows of one warp-level MMA tile.
//
// A block owns one (token, kv head, split).  Its keys are the 64-key tiles  first + split,
// first + split + n_splits, ...  of the token's range, so that the blocks of a token have equal
// work whatever its length is (the grid is sized for the longest sequence the cache allows and
// does not change from step to step).  One thread issues, per tile, cp.async.bulk.tensor loads of
// [64 keys x 64 channels] boxes of K and V straight from the page that holds them (128-byte
// swizzle; a tile never crosses a page because pages are multiples of 64 positions) into a ring of
// 3 (head size 128) or 6 (head size 64) stages, arming a "full" mbarrier per stage with the byte
// count.  Four consumer warps wait for it; warp w takes keys 16w..16w+15 of every tile:
// S = Q K^T with m16n8k16 MMAs (rows = the G query heads, zero rows above), scaling, masking and
// the running softmax in float32, P V again on MMAs, then an arrive on the stage's "empty"
// barrier.  Nothing but the ring is synchronised inside the loop.  At the end the four warps are
// merged through shared memory in ascending order; with one split the block writes the finished
// heads, otherwise a partial (acc, max, sum) per (token, head, split) that a second kernel adds in
// ascending order of the split.  The result never depends on timing.
// Keys outside [p - window + 1, p] get weight exactly 0 and their V rows are cleared in shared
// memory before the product (a page may still hold another sequence's values there).
// In its second form (FUSE, illm_attention_decode_ring_rope) the kernel also does the position
// encoding and the cache write of the step (what rope_kv.cu does, src/kern/naive/naive.cpp:389-414
// and src/core/op.cpp:414-416 in the reference): the consumer warps rotate the query heads on
// their way into shared memory, and in the block that owns the token's last tile a sixth warp makes
// the token's new K row (rotated) and V row, writes them to the cache page and hands them through
// shared memory to the consumer warp that owns their place in that tile.  The TMA thread starts
// at once: it needs neither.
// Formulas: src/kern/naive/naive.cpp:576-604 (scores with key head h / G), :531-553 (mask),
// :209-240 (softmax), :634-662 (values); the reference's GPU code loops over the heads with one
// library call each (src/kern/gpu/kernel_gpu.cu:688-756).
// Every wait on an mbarrier is bounded: after the limit the thread raises the error word and
// goes on, so a fault in the pipeline ends the kernel instead of hanging the GPU.
#include <math.h>

#include "tc_common.cuh"

#define RD_BN 64                        // keys per tile
#define RD_CONSUMERS 4
#define RD_THREADS ((RD_CONSUMERS + 1) * 32)
#define RD_MAX_SPLITS 32

namespace {

__device__ __forceinline__ void rd_ldm(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void rd_ldm_t(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void rd_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned rd_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ void rd_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Byte offset of the 16-byte chunk c (8 channels) of key row r inside a K or V tile: boxes of 64
// channels, 8 KB each, rows of 128 bytes, the chunk index XORed with the row (128-byte swizzle).
__device__ __forceinline__ unsigned rd_tile_off(int r, int c) {
    return (unsigned)((c >> 3) * (RD_BN * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4));
}
template <int D> __device__ __forceinline__ int rd_qswz(int r, int c) { return r * D + ((c ^ (r & 7)) << 3); }

}  // namespace

// The position encoding and the cache write done by this kernel itself (FUSE): the packed projection
// [T, (nh + 2 nkv) d] comes unrotated, in bfloat16 or as the float32 K slices of a split matrix
// product, and the kernel does what rope_kv.cu does for one token: it rotates the query heads on
// their way into shared memory, and the block that owns the token's last tile rotates the new K row,
// writes it and the V row to the cache page and puts them into the tile it has just loaded.  The
// arithmetic and the rounding are those of rope_kv.cu.
struct RdRope {
    const float* partials;     // K slices [splits][T][width], or nullptr: the bfloat16 projection is read
    int splits;
    long long split_stride;
    const float2* cs;          // cos/sin table [positions][rot / 2]
    int rot, table_positions;
    bf16* kc;                  // the cache entry, for the write of the new row
    bf16* vc;
    int write_kv;
    int* err;                  // the step's error word: 2 no page, 3 position outside the table
};

// 8 channels (chunk c) of head slot `slot` of token t, position-encoded if the chunk is rotated
template <int D>
__device__ __forceinline__ void rd_encoded_chunk(const RdRope& rp, const bf16* __restrict__ qkv, size_t row_off, int slot,
                                                 int c, int p, float* out) {
    auto fetch = [&](int cc, float* o8) {
        const size_t off = row_off + (size_t)slot * D + cc * 8;
        if (rp.partials) {
#pragma unroll
            for (int k = 0; k < 8; k++) o8[k] = 0.f;
            const float* pz = rp.partials + off;
            int z = 0;
            for (; z + 4 <= rp.splits; z += 4) {          // four slices in flight, added in order
                float p8[4][8];
#pragma unroll
                for (int u = 0; u < 4; u++) load8(pz + (size_t)(z + u) * rp.split_stride, p8[u]);
#pragma unroll
                for (int u = 0; u < 4; u++)
#pragma unroll
                    for (int k = 0; k < 8; k++) o8[k] += p8[u][k];
            }
            if (z + 2 <= rp.splits) {
                float p8[2][8];
                load8(pz + (size_t)z * rp.split_stride, p8[0]);
                load8(pz + (size_t)(z + 1) * rp.split_stride, p8[1]);
#pragma unroll
                for (int k = 0; k < 8; k++) o8[k] += p8[0][k];
#pragma unroll
                for (int k = 0; k < 8; k++) o8[k] += p8[1][k];
                z += 2;
            }
            if (z < rp.splits) {
                float p8[8];
                load8(pz + (size_t)z * rp.split_stride, p8);
#pragma unroll
                for (int k = 0; k < 8; k++) o8[k] += p8[k];
            }
        } else {
            load8(qkv + off, o8);
        }
    };
    const int hc = rp.rot >> 4;            // chunks per rotated half
    if (c < 2 * hc) {
        const int cp = c < hc ? c : c - hc;
        float a[8], b[8];
        fetch(cp, a);
        fetch(cp + hc, b);
        const float2* cst = rp.cs + (size_t)p * (rp.rot >> 1) + cp * 8;
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const float2 cc = cst[k];
            out[k] = c < hc ? a[k] * cc.x - b[k] * cc.y : a[k] * cc.y + b[k] * cc.x;
        }
    } else {
        fetch(c, out);
    }
}

template <int D, bool FUSE>
__global__ void __launch_bounds__(RD_THREADS + 32)
attention_decode_ring_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                             const bf16* __restrict__ q, int q_stride, const int* __restrict__ block_table,
                             int max_pages, const int* __restrict__ token_pos, const int* __restrict__ token_seq,
                             float* __restrict__ part_acc, float* __restrict__ part_ml, bf16* __restrict__ out,
                             int n_splits, int nh, int nkv, int G, int page_size, int window, float scale_log2e,
                             int* __restrict__ err, const RdRope rp) {
    constexpr int STAGES = 384 / D;
    constexpr int CH = D / 8, KS = D / 16, NT_D = D / 8;
    constexpr unsigned TILE_BYTES = RD_BN * D * 2;            // a K tile, or a V tile
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) unsigned long long bars[2 * STAGES + 1];
    __shared__ __align__(16) bf16 new_row_s[2 * D];         // FUSE: the token's new K row, then its V row

    const unsigned raw = tc_smem_u32(smem_raw);
    const unsigned base = (raw + 1023u) & ~1023u;             // the swizzle's period
    unsigned char* gbase = smem_raw + (base - raw);
    bf16* Qs = reinterpret_cast<bf16*>(gbase + (size_t)STAGES * 2 * TILE_BYTES);   // [16][D]
    const unsigned full0 = tc_smem_u32(&bars[0]), empty0 = tc_smem_u32(&bars[STAGES]);
    const unsigned row_ready = tc_smem_u32(&bars[2 * STAGES]);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, RD_CONSUMERS);
        }
        mbar_init(row_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();          // the barriers exist; from here the warps go their own ways
    // Programmatic dependent launch.  What the step's sequences hold (positions, page tables) and
    // the K and V of earlier positions were written before this step began, so in the fused form
    // the TMA thread does not wait for the previous kernel (the Q/K/V product): its first tiles are
    // on their way while that kernel drains.  Everything that reads the projection or writes global
    // memory waits.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (!FUSE) asm volatile("griddepcontrol.wait;" ::: "memory");

    const int split = blockIdx.x, hk = blockIdx.y, t = blockIdx.z;
    const int p = token_pos[t];
    const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    const int tile_lo = lo / RD_BN, tile_hi = p / RD_BN;
    const int n_tiles = tile_hi - tile_lo + 1;
    const int n_my = split < n_tiles ? (n_tiles - split + n_splits - 1) / n_splits : 0;
    if (n_my == 0) {
        // no keys for this split: the merge kernel skips partials whose maximum is -inf
        if (FUSE) asm volatile("griddepcontrol.wait;" ::: "memory");
        if (tid < G) {
            const size_t o = ((size_t)t * nh + hk * G + tid) * n_splits + split;
            part_ml[o * 2] = -INFINITY;
            part_ml[o * 2 + 1] = 0.f;
        }
        return;
    }

    int p_tab = p;                                    // the position, kept inside the cos/sin table
    if (FUSE && rp.rot > 0 && p >= rp.table_positions) {
        if (tid == 0) atomicExch(rp.err, 3);
        p_tab = rp.table_positions - 1;
    }
    // FUSE: the block that owns the token's last tile also makes the token's new K and V rows
    const bool new_row_here = FUSE && rp.write_kv && split == (tile_hi - tile_lo) % n_splits;

    if (warp == RD_CONSUMERS + 1) {
        // ---- (FUSE) the helper warp: lane < CH makes a chunk of the new K row (rotated), the next CH
        // lanes a chunk of the V row; they go to the cache page and to shared memory, from where the
        // consumer warp that owns the row's place in the last tile takes them
        if (new_row_here) {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            if (lane < 2 * CH) {
                const bool is_k = lane < CH;
                const int c = is_k ? lane : lane - CH;
                float f[8];
                if (is_k) {
                    rd_encoded_chunk<D>(rp, q, (size_t)t * q_stride, nh + hk, c, p_tab, f);
                } else {
                    RdRope plain = rp;
                    plain.rot = 0;
                    rd_encoded_chunk<D>(plain, q, (size_t)t * q_stride, nh + nkv + hk, c, p_tab, f);
                }
                uint4 v;
                __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
                for (int k = 0; k < 4; k++) h2[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
                *reinterpret_cast<uint4*>(new_row_s + (is_k ? 0 : D) + c * 8) = v;
                const int page = block_table[(size_t)token_seq[t] * max_pages + p / page_size];
                if (page < 0) {
                    atomicExch(rp.err, 2);
                } else {
                    bf16* dst = (is_k ? rp.kc : rp.vc) + (((size_t)page * nkv + hk) * page_size + (p % page_size)) * D + c * 8;
                    *reinterpret_cast<uint4*>(dst) = v;
                }
            }
            __syncwarp();
            if (lane == 0) rd_arrive(row_ready);
        }
        return;
    }
    if (warp == RD_CONSUMERS) {
        // ---- producer
        if (lane == 0) {
            const int* bt = block_table + (size_t)token_seq[t] * max_pages;
            bool alive = true;
            for (int i = 0; i < n_my && alive; i++) {
                const int s = i % STAGES;
                if (i >= STAGES) {
                    alive = mbar_wait(empty0 + 8 * s, ((i / STAGES) - 1) & 1, err, TC_ERR_TIMEOUT_DECODE);
                    if (!alive) break;
                }
                const int key0 = (tile_lo + split + i * n_splits) * RD_BN;
                const int page = bt[key0 / page_size];
                const int row = (page * nkv + hk) * page_size + key0 % page_size;
                const unsigned kdst = base + (unsigned)s * 2 * TILE_BYTES, vdst = kdst + TILE_BYTES;
                mbar_expect_tx(full0 + 8 * s, 2 * TILE_BYTES);
#pragma unroll
                for (int hx = 0; hx < D / 64; hx++) {
                    tma_load_2d(kdst + hx * (RD_BN * 128), &map_k, hx * 64, row, full0 + 8 * s);
                    tma_load_2d(vdst + hx * (RD_BN * 128), &map_v, hx * 64, row, full0 + 8 * s);
                }
            }
        }
        return;
    }

    // ---- consumers.  Q: the G heads of this kv head as rows 0..G-1, zero rows above
    if (FUSE) asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int i = tid; i < 16 * CH; i += RD_CONSUMERS * 32) {
        const int r = i / CH, c = i % CH;
        if (FUSE && r < G) {
            float f[8];
            rd_encoded_chunk<D>(rp, q, (size_t)t * q_stride, hk * G + r, c, p_tab, f);
            store8(Qs + rd_qswz<D>(r, c), f);
        } else {
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (r < G) v = *reinterpret_cast<const uint4*>(q + (size_t)t * q_stride + (size_t)(hk * G + r) * D + c * 8);
            *reinterpret_cast<uint4*>(Qs + rd_qswz<D>(r, c)) = v;
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(RD_CONSUMERS * 32) : "memory");
    // warp w owns keys 16w .. 16w+15 of every tile
    const int g = lane >> 2, t4 = lane & 3, mtx = lane >> 3;
    unsigned qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++)
        rd_ldm(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3],
               tc_smem_u32(Qs + rd_qswz<D>((mtx & 1) * 8 + (lane & 7), ks * 2 + (mtx >> 1))));

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[NT_D][4];
#pragma unroll
    for (int i = 0; i < NT_D; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

    bool alive = true;
    for (int i = 0; i < n_my && alive; i++) {
        const int s = i % STAGES;
        // lanes leave the polling loop one by one: together again before the warp-wide instructions
        alive = __all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, (i / STAGES) & 1, err, TC_ERR_TIMEOUT_DECODE));
        if (!alive) break;
        const int key0 = (tile_lo + split + i * n_splits) * RD_BN + warp * 16;
        if (new_row_here && i == n_my - 1 && warp == ((p & (RD_BN - 1)) >> 4)) {
            // the tile came from the cache before the row of position p was there (or while it was
            // being written): this warp, the only reader of that row, puts in what the helper warp made
            alive = __all_sync(0xffffffffu, mbar_wait(row_ready, 0, err, TC_ERR_TIMEOUT_DECODE));
            if (lane < 2 * CH) {
                const int c = lane < CH ? lane : lane - CH;
                unsigned char* tile = gbase + (size_t)s * 2 * TILE_BYTES + (lane < CH ? 0 : TILE_BYTES);
                *reinterpret_cast<uint4*>(tile + rd_tile_off(p & (RD_BN - 1), c)) =
                    *reinterpret_cast<const uint4*>(new_row_s + (lane < CH ? 0 : D) + c * 8);
            }
            __syncwarp();
        }
        if (key0 <= p && key0 + 15 >= lo) {
            const unsigned kbase = base + (unsigned)s * 2 * TILE_BYTES, vbase = kbase + TILE_BYTES;
            // two accumulator sets shorten the chain of dependent MMAs
            float sa[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            float sb[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
            const int krow = warp * 16 + (mtx >> 1) * 8 + (lane & 7);
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                unsigned b0, b1, b2, b3;
                rd_ldm(b0, b1, b2, b3, kbase + rd_tile_off(krow, ks * 2 + (mtx & 1)));
                if (ks & 1) {
                    rd_mma(sb[0], qf[ks], b0, b1);
                    rd_mma(sb[1], qf[ks], b2, b3);
                } else {
                    rd_mma(sa[0], qf[ks], b0, b1);
                    rd_mma(sa[1], qf[ks], b2, b3);
                }
            }
            float sc[2][4];
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 2; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int key = key0 + nt * 8 + t4 * 2 + (e & 1);
                    const float v = (key > p || key < lo) ? -INFINITY : (sa[nt][e] + sb[nt][e]) * scale_log2e;
                    sc[nt][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            float alpha[2], mref[2];
#pragma unroll
            for (int e = 0; e < 2; e++) {
                mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 1));
                mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 2));
                const float m_new = fmaxf(m_run[e], mx[e]);      // finite: the warp has a valid key
                mref[e] = m_new;
                alpha[e] = fast_exp2(m_run[e] - m_new);          // 0 the first time (m_run = -inf)
                m_run[e] = m_new;
                l_run[e] *= alpha[e];
            }
            unsigned pf[4];
#pragma unroll
            for (int nt = 0; nt < 2; nt++) {
                const float p0 = fast_exp2(sc[nt][0] - mref[0]), p1 = fast_exp2(sc[nt][1] - mref[0]);
                const float p2 = fast_exp2(sc[nt][2] - mref[1]), p3 = fast_exp2(sc[nt][3] - mref[1]);
                l_run[0] += p0 + p1;
                l_run[1] += p2 + p3;
                pf[nt * 2] = rd_pack(p0, p1);
                pf[nt * 2 + 1] = rd_pack(p2, p3);
            }
            if (key0 + 15 > p || key0 < lo) {
                // a tile at the edge of the range: V rows of hidden keys may hold anything (another
                // sequence's old values), and 0 x NaN would not be 0, so they are cleared
                unsigned char* vgen = gbase + (size_t)s * 2 * TILE_BYTES + TILE_BYTES;
                for (int j = lane; j < 16 * CH; j += 32) {
                    const int r = j / CH, c = j % CH;
                    if (key0 + r > p || key0 + r < lo)
                        *reinterpret_cast<uint4*>(vgen + rd_tile_off(warp * 16 + r, c)) = make_uint4(0u, 0u, 0u, 0u);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // before TMA refills the stage
                __syncwarp();
            }
            const int vrow = warp * 16 + (mtx & 1) * 8 + (lane & 7);
#pragma unroll
            for (int np = 0; np < NT_D / 2; np++) {
                unsigned b0, b1, b2, b3;
                rd_ldm_t(b0, b1, b2, b3, vbase + rd_tile_off(vrow, np * 2 + (mtx >> 1)));
                o[np * 2][0] *= alpha[0];
                o[np * 2][1] *= alpha[0];
                o[np * 2][2] *= alpha[1];
                o[np * 2][3] *= alpha[1];
                o[np * 2 + 1][0] *= alpha[0];
                o[np * 2 + 1][1] *= alpha[0];
                o[np * 2 + 1][2] *= alpha[1];
                o[np * 2 + 1][3] *= alpha[1];
                rd_mma(o[np * 2], pf, b0, b1);
                rd_mma(o[np * 2 + 1], pf, b2, b3);
            }
        }
        __syncwarp();
        if (lane == 0) rd_arrive(empty0 + 8 * s);
    }
#pragma unroll
    for (int e = 0; e < 2; e++) {
        l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 1);
        l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 2);
    }

    // ---- merge the warps (ascending) through the ring's memory: every load has landed and been read
    asm volatile("bar.sync 1, %0;" ::"n"(RD_CONSUMERS * 32) : "memory");
    float* mrg = reinterpret_cast<float*>(gbase);            // [RD_CONSUMERS][16][D + 2]
    constexpr int ROW = D + 2;
#pragma unroll
    for (int e = 0; e < 2; e++) {
        const int r = g + e * 8;
        float* dst = mrg + ((size_t)warp * 16 + r) * ROW;
#pragma unroll
        for (int i = 0; i < NT_D; i++) {
            dst[i * 8 + t4 * 2] = o[i][e * 2];
            dst[i * 8 + t4 * 2 + 1] = o[i][e * 2 + 1];
        }
        if (t4 == 0) {
            dst[D] = m_run[e];
            dst[D + 1] = l_run[e];
        }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(RD_CONSUMERS * 32) : "memory");
    for (int idx = tid; idx < G * D; idx += RD_CONSUMERS * 32) {
        const int r = idx / D, c = idx - r * D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < RD_CONSUMERS; w++) M = fmaxf(M, mrg[((size_t)w * 16 + r) * ROW + D]);
        float num = 0.f, den = 0.f;
#pragma unroll
        for (int w = 0; w < RD_CONSUMERS; w++) {
            const float mw = mrg[((size_t)w * 16 + r) * ROW + D];
            const float wgt = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
            num += mrg[((size_t)w * 16 + r) * ROW + c] * wgt;
            den += mrg[((size_t)w * 16 + r) * ROW + D + 1] * wgt;
        }
        const size_t head = (size_t)t * nh + hk * G + r;
        if (n_splits == 1) {
            out[head * D + c] = __float2bfloat16_rn(num / den);
        } else {
            const size_t oidx = head * n_splits + split;
            part_acc[oidx * D + c] = num;
            if (c == 0) {
                part_ml[oidx * 2] = M;
                part_ml[oidx * 2 + 1] = den;
            }
        }
    }
}

// out[t, h, :] = sum over splits (ascending) of acc * 2^(m - M) / sum of l * 2^(m - M); splits
// without keys carry m = -inf and are skipped.
template <int D>
__global__ void attention_decode_ring_merge_kernel(const float* __restrict__ part_acc,
                                                   const float* __restrict__ part_ml, bf16* __restrict__ out,
                                                   int n_splits, int nh) {
    pdl_grid_sync();
    const int h = blockIdx.x, t = blockIdx.y, c = threadIdx.x;
    const size_t o = ((size_t)t * nh + h) * n_splits;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; s++) M = fmaxf(M, part_ml[(o + s) * 2]);
    float num = 0.f, den = 0.f;
    for (int s = 0; s < n_splits; s++) {
        const float m = part_ml[(o + s) * 2];
        if (m == -INFINITY) continue;
        const float w = fast_exp2(m - M);
        den += part_ml[(o + s) * 2 + 1] * w;
        num += part_acc[(o + s) * D + c] * w;
    }
    out[((size_t)t * nh + h) * D + c] = __float2bfloat16_rn(num / den);
}

// ---- host side

typedef CUresult (*RdEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static RdEncodeTiledFn rd_encode_fn() {
    static RdEncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (RdEncodeTiledFn)p;
    }
    return fn;
}

// one cache entry seen as a bfloat16 matrix [rows = pages * kv heads * page_size, d]; boxes of [64, 64]
static int rd_make_map(CUtensorMap* map, const void* ptr, long long rows, int d) {
    RdEncodeTiledFn fn = rd_encode_fn();
    if (!fn) return ILLM_ERR_BAD_ARG;
    cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)d * 2};
    cuuint32_t box[2] = {64, RD_BN};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : ILLM_ERR_BAD_ARG;
}

template <int D>
static int rd_launch(const void* q, int q_stride, const void* kc, const void* vc, long long n_pages,
                     const int* block_table, int max_pages, const int* token_pos, const int* token_seq,
                     float* part_acc, float* part_ml, void* out, int T, int nh, int nkv, int page_size, int window,
                     float scale, int n_splits, int* err, cudaStream_t s, const RdRope* rope) {
    CUtensorMap mk, mv;
    int rc;
    const long long rows = n_pages * nkv * page_size;
    if ((rc = rd_make_map(&mk, kc, rows, D)) != 0) return rc;
    if ((rc = rd_make_map(&mv, vc, rows, D)) != 0) return rc;
    constexpr int STAGES = 384 / D;
    const size_t smem = (size_t)STAGES * 2 * RD_BN * D * 2 + (size_t)16 * D * 2 + 1024;
    RdRope rp = {};
    if (rope) rp = *rope;
    auto launch = [&](auto kern) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        illm_launch(kern, dim3(n_splits, nkv, T), dim3(rope ? RD_THREADS + 32 : RD_THREADS), smem, s, mk, mv, (const bf16*)q, q_stride,
                    block_table, max_pages, token_pos, token_seq, part_acc, part_ml, (bf16*)out, n_splits, nh, nkv,
                    nh / nkv, page_size, window, scale * 1.4426950408889634f, err, rp);
        return illm_launch_status();
    };
    rc = rope ? launch(attention_decode_ring_kernel<D, true>) : launch(attention_decode_ring_kernel<D, false>);
    if (rc != 0 || n_splits == 1) return rc;
    illm_launch(attention_decode_ring_merge_kernel<D>, dim3(nh, T), dim3(D), 0, s, (const float*)part_acc,
                (const float*)part_ml, (bf16*)out, n_splits, nh);
    return illm_launch_status();
}

static int rd_run(const void* q, int q_stride, const void* kc, const void* vc, long long n_pages,
                  const int* block_table, int max_pages, const int* token_pos, const int* token_seq, float* part_acc,
                  float* part_ml, void* out, int T, int nh, int nkv, int d, int page_size, int window, float scale,
                  int n_splits, int* err, void* stream, const RdRope* rope) {
    if (T <= 0) return 0;
    if (nkv <= 0 || nh % nkv || nh / nkv > 16 || T > 65535 || nkv > 65535 || (q_stride & 7) || page_size % RD_BN ||
        n_splits < 1 || n_splits > RD_MAX_SPLITS || ((uintptr_t)kc & 15) || ((uintptr_t)vc & 15) ||
        n_pages * nkv * page_size > 0x7fffffffLL || (n_splits > 1 && (part_acc == nullptr || part_ml == nullptr)))
        return ILLM_ERR_BAD_ARG;
    if (!(rope && rope->partials) && (q == nullptr || ((uintptr_t)q & 15))) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (d == 128)
        return rd_launch<128>(q, q_stride, kc, vc, n_pages, block_table, max_pages, token_pos, token_seq, part_acc,
                              part_ml, out, T, nh, nkv, page_size, window, scale, n_splits, err, s, rope);
    if (d == 64)
        return rd_launch<64>(q, q_stride, kc, vc, n_pages, block_table, max_pages, token_pos, token_seq, part_acc,
                             part_ml, out, T, nh, nkv, page_size, window, scale, n_splits, err, s, rope);
    return ILLM_ERR_BAD_ARG;
}

// q: the packed projection [T, q_stride] whose first nh*d columns are the query heads; kc, vc: one
// cache entry [n_pages, nkv, page_size, d] with page_size a multiple of 64.  Scratch (unused with
// one split): part_acc float [T, nh, n_splits, d], part_ml float [T, nh, n_splits, 2].
extern "C" int illm_attention_decode_ring(const void* q, int q_stride, const void* kc, const void* vc,
                                          long long n_pages, const int* block_table, int max_pages,
                                          const int* token_pos, const int* token_seq, float* part_acc,
                                          float* part_ml, void* out, int T, int nh, int nkv, int d, int page_size,
                                          int window, float scale, int n_splits, int* err, void* stream) {
    return rd_run(q, q_stride, kc, vc, n_pages, block_table, max_pages, token_pos, token_seq, part_acc, part_ml, out, T,
                  nh, nkv, d, page_size, window, scale, n_splits, err, stream, nullptr);
}

// The same with the position encoding and the cache write inside: `qkv` is the unrotated packed
// projection [T, (nh + 2 nkv) d] in bfloat16, or nullptr with `partials`, its `splits` float32 K
// slices [splits][T][(nh + 2 nkv) d].  cos_sin: float32 [table_positions][rot / 2][2] (rot = 0: no
// rotation).  write_kv = 0: the cache already holds this token's K and V (a layer that reads another
// layer's entry).  step_err: the step's error word (2: a sequence without a page for its position,
// 3: a position outside the table).  Needs rot % 16 == 0.
extern "C" int illm_attention_decode_ring_rope(const void* qkv, const float* partials, int splits,
                                               long long split_stride, const float* cos_sin, int rot,
                                               int table_positions, int write_kv, void* kc, void* vc,
                                               long long n_pages, const int* block_table, int max_pages,
                                               const int* token_pos, const int* token_seq, float* part_acc,
                                               float* part_ml, void* out, int T, int nh, int nkv, int d,
                                               int page_size, int window, float scale, int n_splits, int* err,
                                               int* step_err, void* stream) {
    if (rot < 0 || rot > d || (rot & 15) || (rot > 0 && cos_sin == nullptr) || step_err == nullptr ||
        (partials != nullptr && splits < 1))
        return ILLM_ERR_BAD_ARG;
    RdRope rp = {partials, splits, split_stride, (const float2*)cos_sin, rot, table_positions, (bf16*)kc, (bf16*)vc,
                 write_kv, step_err};
    return rd_run(qkv, (nh + 2 * nkv) * d, kc, vc, n_pages, block_table, max_pages, token_pos, token_seq, part_acc,
                  part_ml, out, T, nh, nkv, d, page_size, window, scale, n_splits, err, stream, &rp);
}

// Position encoding of Q and K (rotate-half) fused with the write of K and V into the paged
// cache.
//
// The reference rotates Q and the new K rows in place (src/kern/gpu/kernel_gpu.cu:343-401,
// formula src/kern/naive/naive.cpp:389-414: pair (j, j + rot/2), angle p * theta^(-2j/rot)),
// after the K and V projections have written straight into the cache rows
// (src/core/op.cpp:414-416).  Here one launch reads the packed projection
// qkv[t] = [q heads | k heads | v heads], rotates Q in place, and stores rotated K and plain V
// at the token's place in the cache: page block_table[seq, p / page_size], offset p % page_size
// of a cache laid out [page, kv head, offset, d].  cos and sin come from a float32 table
// [position, rot/2] that the host computed in float64; the rotation itself is float32.
// rot = 0 turns the rotation off (the launch is then only the cache write); write_kv = 0
// leaves the cache alone (a layer that reads another layer's keys and values).
#include "common.cuh"

#define RK_WARPS 4
#define RK_SLOTS_PER_WARP 4         // each warp takes its head slots one after the other

template <typename TA>
__global__ void rope_kv_write_kernel(TA* __restrict__ qkv, const float2* __restrict__ cs,
                                     const int* __restrict__ token_pos,
                                     const int* __restrict__ token_seq,
                                     const int* __restrict__ block_table, int max_pages,
                                     TA* __restrict__ kc, TA* __restrict__ vc, int nh, int nkv, int d,
                                     int rot, int page_size, int write_kv, int table_positions,
                                     int* __restrict__ err, const float* __restrict__ partials, int splits,
                                     long long split_stride, int slots_per_warp) {
    pdl_grid_sync();
    const int t = blockIdx.x;
    const int p = token_pos[t];
    const int half = rot >> 1;
    TA* row = qkv + (size_t)t * (nh + 2 * nkv) * d;
    const size_t head_stride = (size_t)page_size * d;  // between kv heads inside a page
    // this block's share of the head slots: [q heads | k heads | v heads]
    const int n_slots = nh + 2 * nkv;
    const int lane = threadIdx.x & 31;
    const int s0 = blockIdx.y * RK_WARPS * slots_per_warp + (threadIdx.x >> 5) * slots_per_warp;
    const int s1 = min(n_slots, s0 + slots_per_warp);
    const int rest = d - rot;
    // Where K and V of this token go, and its row of the cos/sin table.  Called after the first
    // loads of the projection have been issued: those need nothing but the token's index, while this
    // is a chain of two dependent loads (position, then page).
    TA* kdst = nullptr;
    TA* vdst = nullptr;
    const float2* cst = cs + (size_t)p * half;
    auto resolve = [&]() {
        if (write_kv) {
            const int page = block_table[(size_t)token_seq[t] * max_pages + p / page_size];
            if (page < 0) {
                if (threadIdx.x == 0) atomicExch(err, 2);
                write_kv = 0;
            } else {
                size_t base = ((size_t)page * nkv * page_size + (p % page_size)) * d;
                kdst = kc + base;
                vdst = vc + base;
            }
        }
        if (half > 0 && p >= table_positions) {
            if (threadIdx.x == 0) atomicExch(err, 3);
            return false;
        }
        return true;
    };
    // 8 channels per thread with 16-byte accesses where the sizes allow it: the warp's lanes are
    // spread over (head slot, 8-channel chunk) pairs, two pairs per lane in flight
    const bool vec = ((half & 7) == 0) && ((d & 7) == 0) && ((rot & 7) == 0);
    if (vec) {
        const int cpd = d >> 3, hc = half >> 3;      // chunks per head, chunks per rotated half
        // the projection may still be in K slices (float32, from a split matrix product): a chunk
        // is then the sum of its slices in ascending order, and Q is written to `qkv` for the
        // attention kernel while K and V go to the cache only
        const size_t row_off = (size_t)t * (nh + 2 * nkv) * d;
        auto fetch = [&](const TA* src_elem, float* out8) {
            if (partials) {
                const size_t off = row_off + (size_t)(src_elem - row);
#pragma unroll
                for (int k = 0; k < 8; k++) out8[k] = 0.f;
                for (int z = 0; z < splits; z++) {
                    float p8[8];
                    load8(partials + (size_t)z * split_stride + off, p8);
#pragma unroll
                    for (int k = 0; k < 8; k++) out8[k] += p8[k];
                }
            } else {
                load8(src_elem, out8);
            }
        };
        // The warp's work items: a Q or K head gives hc rotated pairs of chunks plus its chunks
        // outside the rotated part (copied for K, and for Q only when it comes from slices); a V
        // head gives cpd copied chunks.  Lanes take consecutive items, so no lane idles.
        const int ipc = cpd - hc;
        const int n_rot_slots = max(0, min(s1, nh + nkv) - s0), n_v_slots = max(0, (s1 - s0) - n_rot_slots);
        const int n_rot_items = n_rot_slots * ipc, n_items = n_rot_items + n_v_slots * cpd;
        for (int base = 0; base < n_items; base += 64) {
            // kind 1: a rotated pair of chunks; kind 2: a chunk that is only copied
            float a[2][8], b[2][8];
            int kind[2], slot_u[2], c_u[2];
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int idx = base + u * 32 + lane;
                kind[u] = 0;
                if (idx < n_items) {
                    int slot, c;
                    if (idx < n_rot_items) {
                        slot = s0 + idx / ipc;
                        c = idx % ipc;
                        if (c >= hc) c += hc;                 // behind the rotated part
                    } else {
                        slot = s0 + n_rot_slots + (idx - n_rot_items) / cpd;
                        c = (idx - n_rot_items) % cpd;
                    }
                    slot_u[u] = slot;
                    c_u[u] = c;
                    const TA* src = row + (size_t)slot * d;
                    if (slot < nh + nkv && c < hc) {
                        kind[u] = 1;
                        fetch(src + c * 8, a[u]);
                        fetch(src + c * 8 + half, b[u]);
                    } else if (slot >= nh || partials) {      // Q outside the rotated part stays where it is
                        kind[u] = 2;
                        fetch(src + c * 8, a[u]);
                    }
                }
            }
            if (base == 0 && !resolve()) return;
#pragma unroll
            for (int u = 0; u < 2; u++) {
                if (kind[u] == 0) continue;
                const int slot = slot_u[u], c = c_u[u];
                const bool is_q = slot < nh, is_k = !is_q && slot < nh + nkv;
                if (!is_q && !write_kv) continue;
                TA* dst = is_q ? row + (size_t)slot * d
                               : (is_k ? kdst + (size_t)(slot - nh) * head_stride
                                       : vdst + (size_t)(slot - nh - nkv) * head_stride);
                if (kind[u] == 1) {
                    const int j = c * 8;
                    float ra[8], rb[8];
#pragma unroll
                    for (int k = 0; k < 8; k += 2) {
                        const float4 cc = *reinterpret_cast<const float4*>(cst + j + k);   // (cos, sin) x 2
                        ra[k] = a[u][k] * cc.x - b[u][k] * cc.y;
                        rb[k] = a[u][k] * cc.y + b[u][k] * cc.x;
                        ra[k + 1] = a[u][k + 1] * cc.z - b[u][k + 1] * cc.w;
                        rb[k + 1] = a[u][k + 1] * cc.w + b[u][k + 1] * cc.z;
                    }
                    store8(dst + j, ra);
                    store8(dst + j + half, rb);
                } else {
                    store8(dst + c * 8, a[u]);
                }
            }
        }
        return;
    }
    if (!resolve()) return;
    // any other sizes: element by element
    for (int slot = s0; slot < s1; slot++) {
        TA* src = row + (size_t)slot * d;
        if (slot < nh + nkv) {
            const bool is_k = slot >= nh;
            if (is_k && !write_kv) continue;
            TA* dst = is_k ? kdst + (size_t)(slot - nh) * head_stride : src;
            for (int j = lane; j < half; j += 32) {
                const float a = to_f32(src[j]), b = to_f32(src[j + half]);
                const float2 c = cst[j];
                dst[j] = from_f32<TA>(a * c.x - b * c.y);
                dst[j + half] = from_f32<TA>(a * c.y + b * c.x);
            }
            if (is_k)   // K channels outside the rotated part
                for (int c = rot + lane; c < rot + rest; c += 32) dst[c] = src[c];
        } else if (write_kv) {
            TA* dst = vdst + (size_t)(slot - nh - nkv) * head_stride;
            for (int c = lane; c < d; c += 32) dst[c] = src[c];
        }
    }
}

static int rope_launch(void* qkv, const float* cos_sin, const int* token_pos, const int* token_seq,
                       const int* block_table, int max_pages, void* kc, void* vc, int act_dtype, int T, int nh,
                       int nkv, int d, int rot, int page_size, int write_kv, int table_positions, int* err,
                       void* stream, const float* partials, int splits, long long split_stride);

extern "C" int illm_rope_kv_write(void* qkv, const float* cos_sin, const int* token_pos,
                                  const int* token_seq, const int* block_table, int max_pages,
                                  void* kc, void* vc, int act_dtype, int T, int nh, int nkv, int d,
                                  int rot, int page_size, int write_kv, int table_positions,
                                  int* err, void* stream) {
    return rope_launch(qkv, cos_sin, token_pos, token_seq, block_table, max_pages, kc, vc, act_dtype, T, nh, nkv, d,
                       rot, page_size, write_kv, table_positions, err, stream, nullptr, 0, 0);
}

// The same with the packed projection given as `splits` float32 slices [splits][T][(nh+2nkv)*d] of a
// split-K matrix product; `qkv` receives the rotated Q heads (its K and V columns stay unwritten).
// Needs the 16-byte path: d, rot and rot/2 multiples of 8.
extern "C" int illm_rope_kv_write_partials(void* qkv, const float* partials, int splits, long long split_stride,
                                           const float* cos_sin, const int* token_pos, const int* token_seq,
                                           const int* block_table, int max_pages, void* kc, void* vc,
                                           int act_dtype, int T, int nh, int nkv, int d, int rot, int page_size,
                                           int write_kv, int table_positions, int* err, void* stream) {
    if (!partials || splits < 1 || (d & 7) || (rot & 15)) return ILLM_ERR_BAD_ARG;
    return rope_launch(qkv, cos_sin, token_pos, token_seq, block_table, max_pages, kc, vc, act_dtype, T, nh, nkv, d,
                       rot, page_size, write_kv, table_positions, err, stream, partials, splits, split_stride);
}

static int rope_launch(void* qkv, const float* cos_sin, const int* token_pos, const int* token_seq,
                       const int* block_table, int max_pages, void* kc, void* vc, int act_dtype, int T, int nh,
                       int nkv, int d, int rot, int page_size, int write_kv, int table_positions, int* err,
                       void* stream, const float* partials, int splits, long long split_stride) {
    if (T <= 0) return 0;
    if (rot < 0 || rot > d || (rot & 1) || (rot > 0 && cos_sin == nullptr)) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    const int n_slots = nh + 2 * nkv;
    const int spw = RK_SLOTS_PER_WARP;
    dim3 grid(T, (n_slots + RK_WARPS * spw - 1) / (RK_WARPS * spw));
    if (T > 2147483647 / 2 || grid.y > 65535) return ILLM_ERR_BAD_ARG;
    int threads = RK_WARPS * 32;
    if (act_dtype == ILLM_BF16)
        illm_launch(rope_kv_write_kernel<bf16>, dim3(grid), dim3(threads), 0, s, 
            (bf16*)qkv, (const float2*)cos_sin, token_pos, token_seq, block_table, max_pages,
            (bf16*)kc, (bf16*)vc, nh, nkv, d, rot, page_size, write_kv, table_positions, err, partials, splits,
            split_stride, spw);
    else if (act_dtype == ILLM_F32)
        illm_launch(rope_kv_write_kernel<float>, dim3(grid), dim3(threads), 0, s, 
            (float*)qkv, (const float2*)cos_sin, token_pos, token_seq, block_table, max_pages,
            (float*)kc, (float*)vc, nh, nkv, d, rot, page_size, write_kv, table_positions, err, partials, splits,
            split_stride, spw);
    else
        return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}

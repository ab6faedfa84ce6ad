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

template <typename TA>
__global__ void rope_kv_write_kernel(TA* __restrict__ qkv, const float2* __restrict__ cs,
                                     const int* __restrict__ token_pos,
                                     const int* __restrict__ token_seq,
                                     const int* __restrict__ block_table, int max_pages,
                                     TA* __restrict__ kc, TA* __restrict__ vc, int nh, int nkv, int d,
                                     int rot, int page_size, int write_kv, int table_positions,
                                     int* __restrict__ err) {
    const int t = blockIdx.x;
    const int p = token_pos[t];
    const int half = rot >> 1;
    TA* row = qkv + (size_t)t * (nh + 2 * nkv) * d;
    TA* kdst = nullptr;
    TA* vdst = nullptr;
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
        return;
    }
    const size_t head_stride = (size_t)page_size * d;  // between kv heads inside a page
    const int n_rot_heads = write_kv ? nh + nkv : nh;
    const float2* cst = cs + (size_t)p * half;
    for (int i = threadIdx.x; i < n_rot_heads * half; i += blockDim.x) {
        const int head = i / half, j = i - head * half;
        TA* src = row + (size_t)head * d;
        const float a = to_f32(src[j]), b = to_f32(src[j + half]);
        const float2 c = cst[j];
        const float ra = a * c.x - b * c.y;
        const float rb = a * c.y + b * c.x;
        if (head < nh) {
            src[j] = from_f32<TA>(ra);
            src[j + half] = from_f32<TA>(rb);
        } else {
            TA* dst = kdst + (size_t)(head - nh) * head_stride;
            dst[j] = from_f32<TA>(ra);
            dst[j + half] = from_f32<TA>(rb);
        }
    }
    if (!write_kv) return;
    // K channels outside the rotated part
    const int rest = d - rot;
    for (int i = threadIdx.x; i < nkv * rest; i += blockDim.x) {
        const int hk = i / rest, c = rot + (i - hk * rest);
        kdst[(size_t)hk * head_stride + c] = row[(size_t)(nh + hk) * d + c];
    }
    // V
    const TA* vsrc = row + (size_t)(nh + nkv) * d;
    for (int i = threadIdx.x; i < nkv * d; i += blockDim.x) {
        const int hk = i / d, c = i - hk * d;
        vdst[(size_t)hk * head_stride + c] = vsrc[i];
    }
}

extern "C" int illm_rope_kv_write(void* qkv, const float* cos_sin, const int* token_pos,
                                  const int* token_seq, const int* block_table, int max_pages,
                                  void* kc, void* vc, int act_dtype, int T, int nh, int nkv, int d,
                                  int rot, int page_size, int write_kv, int table_positions,
                                  int* err, void* stream) {
    if (T <= 0) return 0;
    if (rot < 0 || rot > d || (rot & 1) || (rot > 0 && cos_sin == nullptr)) return ILLM_ERR_BAD_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    int work = (nh + 2 * nkv) * d / 2;
    int threads = work >= 2048 ? 256 : 128;
    if (act_dtype == ILLM_BF16)
        rope_kv_write_kernel<bf16><<<T, threads, 0, s>>>(
            (bf16*)qkv, (const float2*)cos_sin, token_pos, token_seq, block_table, max_pages,
            (bf16*)kc, (bf16*)vc, nh, nkv, d, rot, page_size, write_kv, table_positions, err);
    else if (act_dtype == ILLM_F32)
        rope_kv_write_kernel<float><<<T, threads, 0, s>>>(
            (float*)qkv, (const float2*)cos_sin, token_pos, token_seq, block_table, max_pages,
            (float*)kc, (float*)vc, nh, nkv, d, rot, page_size, write_kv, table_positions, err);
    else
        return ILLM_ERR_BAD_ARG;
    return illm_launch_status();
}

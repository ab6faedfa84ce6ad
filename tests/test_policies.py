"""Host-side choices that need no GPU: how many blocks the decode attention gives a (token, KV head)
pair, and how many K slices a decode-sized product is cut into."""
from inferllm_b200.kernels import ops


def test_decode_attention_splits_stay_in_range_and_follow_the_measurements():
    for pairs in (1, 8, 32, 64, 96, 128, 160, 192, 256, 320, 384, 512, 1280, 2048):
        for ctx in (1, 64, 65, 512, 1024, 4096, 32768):
            n = ops.attention_decode_ring_splits(pairs, 1, ctx)
            tiles = -(-ctx // 64)
            assert 1 <= n <= min(tiles, 32), (pairs, ctx, n)
    # a grid a little larger than the 296 blocks that run at once is cut into several waves
    # (measured: 320 pairs at context 4096, 129 us in one split, 106 us in six)
    assert 4 <= ops.attention_decode_ring_splits(8, 40, 4096) <= 8
    # grids that fill the GPU in one wave, or in many, stay whole (160 pairs: 56 us in one split,
    # 69 us in two; 512 pairs at context 1024: 44 us in one split, 50 us in two)
    assert ops.attention_decode_ring_splits(5, 32, 4096) == 1
    assert ops.attention_decode_ring_splits(8, 32, 4096) == 1
    assert ops.attention_decode_ring_splits(16, 32, 1024) == 1
    assert ops.attention_decode_ring_splits(64, 32, 4096) == 1
    # few pairs are split until about 160 blocks are at work, never into more blocks than tiles
    assert ops.attention_decode_ring_splits(1, 8, 32768) >= 16
    assert ops.attention_decode_ring_splits(1, 32, 64) == 1
    # the head size scales the bytes a block streams and with them what a split is worth
    assert ops.attention_decode_ring_splits(8, 8, 4096, 64) <= ops.attention_decode_ring_splits(8, 8, 4096, 128) + 1


def test_split_k_of_decode_sized_products():
    for M in (1, 8, 16, 64):
        for N, K in ((4096, 4096), (12288, 4096), (22016, 4096), (4096, 11008), (32000, 4096), (100, 64), (128, 8)):
            n = ops.gemm_tc_splits(M, N, K)
            k_iters = -(-K // 64)
            assert 1 <= n <= 8 and n <= k_iters
            per = -(-k_iters // n)
            assert per * (n - 1) < k_iters          # every slice owns at least one 64-wide piece of K
    assert ops.gemm_tc_splits(65, 4096, 4096) == 1   # larger steps are not split
    assert ops.gemm_tc_splits(8, 22016, 4096) == 1   # 172 tiles fill the GPU by themselves
    assert ops.gemm_tc_splits(8, 4096, 4096) == 8

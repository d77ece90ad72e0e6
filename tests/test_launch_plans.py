"""The arithmetic of the launch plans that needs no GPU (the planners assume 148 SMs without one)."""
import pytest

from mini_inference_engine_b200.kernels import device, ops


def test_decode_plan_keeps_the_cluster_merge_for_few_rows_and_short_contexts():
    assert device.num_sms() == device.B200_SMS or device.num_sms() > 0
    for rows, ctx in [(1, 512), (8, 512), (8, 8192), (8, 32768), (16, 960), (64, 512), (256, 512), (64, 960)]:
        splits, merge, part = ops.decode_plan(rows, 4, ctx, True)
        assert merge == "cluster" and part == 0 and splits == ops.decode_splits(rows, 4, ctx), (rows, ctx)


def test_decode_plan_for_heads_of_64_fills_four_places_per_sm_with_parts_of_two_tiles():
    if device.num_sms() != device.B200_SMS:
        pytest.skip("the expected numbers are for 148 SMs")
    # (rows, context bound) -> parts, page copies by TMA, stages: the measured winners (4 kv heads)
    want = {(8, 960): (8, False, 3), (8, 512): (4, False, 3), (16, 960): (8, True, 2), (20, 960): (4, True, 2),
            (32, 512): (4, True, 2), (40, 512): (2, True, 2), (64, 960): (2, True, 2), (72, 512): (2, True, 2),
            (80, 512): (1, True, 4), (96, 960): (1, True, 4), (128, 512): (1, True, 3), (256, 512): (1, True, 3),
            (1, 960): (8, False, 3), (4, 256): (2, False, 3)}
    for (rows, ctx), (parts, tma, stages) in want.items():
        splits = ops.decode_splits(rows, 4, ctx, 64)
        blocks = rows * 4 * splits
        got = (splits, ops.decode_uses_tma(blocks, 64), ops.decode_stages(blocks, ctx, splits, ops.decode_uses_tma(blocks, 64), 64))
        assert got == (parts, tma, stages), (rows, ctx, got)
        assert blocks <= 4 * 148 or splits == 1
    # merged through scratch (long contexts): the stages as before, whatever the parts
    assert ops.decode_stages(512, 8192, 2, True, 64, clustered=False) == 3
    assert ops.decode_stages(256, 8192, 4, True, 64, clustered=False) == 4


def test_decode_plan_leaves_long_contexts_to_the_cluster_where_it_cuts_as_often():
    if device.num_sms() != device.B200_SMS:
        pytest.skip("the expected numbers are for 148 SMs")
    for rows, ctx, parts in [(64, 8192, 2), (64, 2048, 2), (32, 8192, 4), (32, 2048, 4), (16, 8192, 8)]:
        assert ops.decode_plan(rows, 4, ctx, True) == (parts, "cluster", 0), (rows, ctx)


@pytest.mark.parametrize("rows,ctx,parts", [(48, 4096, 3), (40, 8192, 3), (24, 8192, 6), (20, 1 << 20, 7)])
def test_decode_plan_fills_four_blocks_per_sm_for_long_contexts(rows, ctx, parts):
    sms = device.num_sms()
    if sms != device.B200_SMS:
        pytest.skip("the expected numbers are for 148 SMs")
    splits, merge, part = ops.decode_plan(rows, 4, ctx, True)
    assert (splits, merge, part) == (parts, "scratch", ops.LONG_PART_TILES)
    assert rows * 4 * splits <= 4 * sms                                      # all blocks beside one another
    assert -(-ctx // 64) // splits >= ops.LONG_PART_TILES                   # no part shorter than it pays for


def test_decode_plan_never_cuts_into_more_parts_than_there_are_blocks_for():
    for rows in (16, 17, 31, 64, 100, 147, 148, 149, 1000):
        splits, merge, _ = ops.decode_plan(rows, 4, 65536, True)
        assert 1 <= splits <= 16
        if merge == "scratch":
            assert rows * 4 * splits <= 4 * device.num_sms()


def test_scratch_that_is_outgrown_stays_alive_for_the_graphs_that_hold_its_address():
    import torch
    first = ops._workspace("cpu", "test_scratch", 10, torch.float32)
    first[3] = 7.0
    address = first.data_ptr()
    again = ops._workspace("cpu", "test_scratch", 500, torch.float32)
    assert again.data_ptr() == address                         # large enough: the same tensor
    larger = ops._workspace("cpu", "test_scratch", 5000, torch.float32)
    assert larger.numel() >= 5000 and larger.data_ptr() != address and not larger.any()
    assert any(t.data_ptr() == address for t in ops._outgrown) and first[3] == 7.0
    assert ops._workspace("cpu", "test_scratch", 5001, torch.float32).numel() >= 2 * larger.numel()


def test_decode_plan_for_heads_of_128_counts_two_blocks_per_sm():
    if device.num_sms() != device.B200_SMS:
        pytest.skip("the expected numbers are for 148 SMs")
    assert ops.decode_plan(32, 8, 2048, True, 128) == (1, "cluster", 0)       # 256 blocks fill the two places an SM has
    assert ops.decode_plan(8, 8, 4096, True, 128) == (4, "cluster", 0)
    assert ops.decode_plan(16, 8, 8192, True, 128) == (2, "cluster", 0)
    assert ops.decode_uses_tma(10, 128) and not ops.decode_uses_tma(10, 64) and ops.decode_uses_tma(2 * 148 + 1, 64)
    assert ops.decode_stages(2048, 512, 1, True, 128) == 2 and ops.decode_stages(512, 512, 1, True, 128) == 3
    assert ops.decode_stages(512, 512, 1, False, 128) == 2                   # cp.async: unchanged


def test_paired_product_is_chosen_by_the_share_of_its_tiles_that_a_product_fills():
    from mini_inference_engine_b200.kernels import linear
    if device.num_sms() != device.B200_SMS:
        pytest.skip("the expected numbers are for 148 SMs")
    # gate/up of TinyLlama-1.1B (11,264 outputs) and Llama-3-8B (28,672): shares of the offered tiles, and on which side
    # of the threshold the measured winners fall
    assert abs(linear.pair_fill(2048, 11264) - 0.951) < 1e-3 and abs(linear.pair_fill(512, 11264) - 0.595) < 1e-3
    wins = {(768, 11264), (1024, 11264), (2048, 11264), (256, 28672), (512, 28672), (512, 22016)}
    loses = {(512, 11264), (384, 28672), (384, 22016), (256, 22016), (128, 28672)}
    for M, N in wins:
        assert linear.pair_fill(M, N) >= linear.PAIR_MIN_FILL, (M, N)
    for M, N in loses:
        assert linear.pair_fill(M, N) < linear.PAIR_MIN_FILL, (M, N)
    assert linear.pair_fill(1, 256) < 0.001 and 0.99 < linear.pair_fill(74 * 256, 256) <= 1.0

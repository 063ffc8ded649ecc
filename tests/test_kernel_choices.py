"""Decisions that the Python side takes for the kernels, as plain functions of sizes. No GPU."""
from hi_b200.kernels import ops


def test_key_shares_of_the_tensor_core_prefill_attention():
    """Keys are shared among blocks only where the launch would leave most of the GPU waiting:
    few blocks, each with a long run of key tiles."""
    sms, places = 148, 296
    for blocks, tiles in ((40, 1017), (80, 1017), (160, 1020), (320, 1016), (300, 1000), (40, 600)):
        k = ops.prefill_key_splits(blocks, tiles, sms)
        assert 2 <= k <= 8 and tiles // k >= ops.PREFILL_SPLIT_MIN_SHARE, (blocks, tiles, k)
        fill = lambda n: (blocks * n / places) / -(-blocks * n // places)
        assert fill(k) > fill(1) and fill(k) >= max(fill(n) for n in range(1, 9) if tiles // n >= 128) - 0.05
    # launches of more than 1.25 rounds, short runs of keys, or nothing to do: one block each
    for blocks, tiles in ((1280, 992), (640, 500), (371, 2000), (160, 258), (40, 511), (0, 1000), (296, 1000)):
        assert ops.prefill_key_splits(blocks, tiles, sms) == 1, (blocks, tiles)
    # a smaller GPU has fewer places: the same launch is then more than its rounds' worth
    assert ops.prefill_key_splits(160, 1020, 40) == 1

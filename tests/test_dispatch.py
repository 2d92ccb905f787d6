"""Decisions of the kernel face (csrc/ops.py) that need no device."""


def test_attention_block_shapes_by_batch():
    """Which shape of block the single-token attention kernel gets, by (sequence, kv head) pairs on 148 SMs:
    clusters of four and two while they leave a third or half of the chip free, one large block a pair up to
    the number of SMs, two blocks an SM up to twice that, three beyond."""
    from math_utils_b200.csrc.ops import decode_block_shape
    got = {pairs: decode_block_shape(pairs, 148) for pairs in (12, 24, 25, 36, 37, 38, 96, 148, 149, 296, 297, 768)}
    assert got == {12: 24, 24: 24, 25: 12, 36: 12, 37: 12, 38: 6, 96: 6, 148: 6, 149: 3, 296: 3, 297: 2, 768: 2}

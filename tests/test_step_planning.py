"""Host-side planning of a decode step: into how many slices of its context the attention cuts a sequence."""
from ghost_infer_b200.engine.step import StepContext
from ghost_infer_b200.kernels import ops


def ctx(n_seqs, max_kv_len, sms=148):
    c = StepContext()
    c.n_seqs, c.max_kv_len, c.sm_count, c.is_decode = n_seqs, max_kv_len, sms, True
    return c


def test_slices_fill_the_blocks_an_sm_holds():
    # 8 sequences x 8 kv heads = 64 blocks per slice; two blocks per SM at head size 128, three at 64
    assert ops.attn_decode_blocks_per_sm(128, True) == 2 * ops.TUNE["attn_waves"]
    assert ops.attn_decode_blocks_per_sm(64, True) == 3 * ops.TUNE["attn_waves"]
    assert ctx(8, 2048).decode_splits(8, 4, 16, ops.attn_decode_blocks_per_sm(128, True)) == 4
    assert ctx(8, 2048).decode_splits(8, 4, 16, ops.attn_decode_blocks_per_sm(64, True)) == 6


def test_slices_are_never_shorter_than_128_positions_nor_more_than_32():
    assert ctx(1, 100).decode_splits(8, 4, 16, 2) == 1
    assert ctx(1, 300).decode_splits(8, 4, 16, 2) == 2
    assert ctx(1, 1 << 20).decode_splits(1, 4, 16, 2) == 32


def test_a_full_gpu_takes_one_slice_and_a_fixed_count_wins():
    assert ctx(64, 2048).decode_splits(8, 4, 16, 2) == 1
    c = ctx(64, 2048)
    c.fixed_splits = 3                     # a captured graph keeps the count it was captured with
    assert c.decode_splits(8, 4, 16, 2) == 3


def test_wide_groups_take_several_blocks_per_kv_head():
    # 40 heads on one kv head: three blocks of 16 rows per sequence and slice
    assert ctx(4, 4096).decode_splits(1, 40, 16, 2) == (2 * 148) // (4 * 3)

"""Host-side planning of a decode step: into how many slices of its context the attention cuts a sequence."""
import torch

from ghost_infer_b200.kernels import ops

BF, F32 = torch.bfloat16, torch.float32


def plan(n_seqs, max_kv_len, n_heads, n_kv, head_dim, window=None, dtype=BF, sms=148, kv_lens=None):
    return ops.attn_decode_plan(n_seqs, max_kv_len, sms, n_heads, n_kv, head_dim, window, dtype, kv_lens)


def test_slices_fill_the_blocks_an_sm_holds():
    # 8 sequences x 8 kv heads = 64 blocks per slice; two blocks per SM at head size 128, three at 64
    assert ops.attn_decode_blocks_per_sm(128, True) == 2 * ops.TUNE["attn_waves"]
    assert ops.attn_decode_blocks_per_sm(64, True) == 4 * ops.TUNE["attn_waves"]
    assert plan(8, 2048, 32, 8, 128) == (4, 0)
    assert plan(8, 4096, 32, 8, 64) == (9, 0)


def test_slices_are_never_shorter_than_256_positions_nor_more_than_32():
    assert plan(1, 100, 32, 8, 128) == (1, 0)
    assert plan(1, 300, 32, 8, 128) == (1, 0)
    assert plan(1, 600, 32, 8, 128) == (2, 0)
    assert plan(1, 1 << 20, 4, 1, 128) == (32, 0)
    # the length that counts is the longest sequence's now, not the end of its length bucket (which the plan must
    # still cover: it is kept until a sequence outgrows the bucket)
    assert plan(1, 4096, 32, 8, 128) == (16, 0)
    assert plan(1, 4096, 32, 8, 128, kv_lens=[2049]) == (8, 0)
    assert plan(2, 4096, 32, 8, 128, kv_lens=[300, 1100]) == (4, 0)


def test_many_equal_sequences_take_one_slice_each():
    # 64 sequences x 8 kv heads = 512 blocks for 296 places: cutting them would only add rounds
    assert plan(64, 2048, 32, 8, 128) == (1, 0)
    assert plan(64, 2048, 32, 8, 128, kv_lens=[2048] * 64) == (1, 0)
    # head size 64 with rings of two stages: four blocks per SM (the registers' limit), 592 places; equal lengths still
    # take one slice each
    assert ops.attn_decode_blocks_per_sm(64, True) == 4 * ops.TUNE["attn_waves"]
    assert plan(64, 1280, 32, 8, 64, kv_lens=[1200] * 64) == (1, 0)
    assert plan(18, 2048, 32, 8, 128) == (2, 0)                     # 144 blocks: two equal slices still fit one round


def test_many_unequal_sequences_can_be_cut_so_that_all_blocks_find_a_place_at_once(monkeypatch):
    """With TUNE["attn_own_slices"] and the lengths known: slices of a fixed number of tiles of each sequence's own span,
    the shortest (in steps of 256 keys) with which the blocks of all sequences fit the GPU at once.  The long sequences
    are cut, the short ones are not.  (Off by default: measured, the cut costs more than the evenness wins.)"""
    lens = [260 + 32 * i for i in range(64)]                        # 260 .. 2276
    assert plan(64, 4096, 32, 8, 64, kv_lens=lens) == (1, 0)
    monkeypatch.setitem(ops.TUNE, "attn_own_slices", True)
    n, own = plan(64, 4096, 32, 8, 64, kv_lens=lens)
    assert own > 0 and own % 16 == 0
    blocks = lambda o: sum(-(-(l + 64) // (o * 16)) for l in lens) * 8
    assert blocks(own) <= 592 < blocks(own - 16)                    # the shortest slice that fits
    assert n == -(-4096 // (own * 16))                              # the launch covers the longest a sequence may get
    assert max(lens) > own * 16                                     # the longest are cut
    # without the lengths nothing is known about them: one slice each
    assert plan(64, 4096, 32, 8, 64) == (1, 0)
    # more blocks than places even uncut: one slice each
    assert plan(64, 4096, 32, 8, 128, kv_lens=lens) == (1, 0)
    # padding rows of a recorded step count as a block each
    n2, own2 = plan(68, 4096, 32, 8, 64, kv_lens=lens)
    assert own2 >= own


def test_wide_groups_take_several_blocks_per_kv_head():
    # 40 heads on one kv head: three blocks of 16 rows per sequence and slice
    assert plan(4, 8192, 40, 1, 128) == ((2 * 148) // (4 * 3), 0)


def test_both_tensor_core_kernels_hold_the_same_number_of_blocks(monkeypatch):
    # keys on the rows, six warps with rings of two stages: 98 KB and up to 127 registers at head size 128, 50 KB and
    # 80 registers at 64; heads on the rows, four warps: the shared memory decides at 128, the registers at 64
    for on in (True, False):
        monkeypatch.setitem(ops.TUNE, "attn_keys_on_rows", on)
        assert ops.attn_decode_blocks_per_sm(128, True) == 2 * ops.TUNE["attn_waves"]
        assert ops.attn_decode_blocks_per_sm(64, True) == 4 * ops.TUNE["attn_waves"]


def test_head_sizes_the_tensor_core_kernel_declines_count_eight_rows_a_block():
    # head size 48 in bfloat16 runs the plain kernel: 8 heads a block (two blocks for a group of 16), two blocks per SM
    assert plan(4, 1 << 20, 32, 2, 48) == ((2 * 148) // (4 * 2 * 2), 0)
    assert plan(4, 1 << 20, 32, 2, 128) == (32, 0)


def test_32_bit_slices_follow_the_sequence_s_own_length():
    """In the 32-bit path a slice is eight 32-key tiles of the sequence's own span; the launch holds as many slices
    as the longest sequence needs, whatever the batch."""
    assert ops.OWN_LENGTH_TILES == 8
    assert plan(1, 256, 4, 2, 16, dtype=F32) == (1, 8)
    assert plan(1, 257, 4, 2, 16, dtype=F32) == (2, 8)
    assert plan(64, 257, 4, 2, 16, dtype=F32) == (2, 8)             # the batch does not matter
    assert plan(3, 5000, 4, 2, 16, dtype=F32) == ((5000 + 255) // 256, 8)
    # a window bounds the span: at most window + 31 keys from the tile the window starts in, plus that tile's head
    assert plan(3, 5000, 4, 2, 16, window=100, dtype=F32) == (1, 8)
    assert plan(3, 5000, 4, 2, 16, window=300, dtype=F32) == (2, 8)

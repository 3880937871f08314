"""The host's choices before a launch (no GPU): how many blocks of decode attention fit an
SM, how many key splits a step takes, when the ring form is taken, and which matrix
product a shape goes to."""
import pytest
import torch

from kidi_b200.kernels import attention, skinny, tcgen05

DEVICE = torch.device("cuda:0")     # only its index is used: the SM count is given below


@pytest.fixture(autouse=True)
def a_b200(monkeypatch):
    monkeypatch.setitem(attention._sm_count, 0, 148)
    monkeypatch.setattr(attention, "DECODE_RING", True)
    monkeypatch.setattr(attention, "DECODE_RING_ALWAYS", False)
    monkeypatch.delenv("KIDI_B200_DECODE_SPLITS", raising=False)


def test_blocks_per_sm_follow_the_shared_memory_of_a_block():
    assert attention.blocks_per_sm(128) == 3 and attention.blocks_per_sm(128, ring=True) == 4
    assert attention.blocks_per_sm(64) == 4                       # registers bound it, not memory
    assert attention.blocks_per_sm(256) == 1 and attention.blocks_per_sm(256, ring=True) == 2
    for width in range(16, 257, 16):
        for ring in (False, True):
            blocks = attention.blocks_per_sm(width, ring)
            assert 1 <= blocks <= 4
            assert blocks <= attention.blocks_per_sm(max(16, width - 16), ring)   # wider heads never fit more


def test_the_ring_is_taken_only_where_it_saves_a_round_of_blocks():
    ring = lambda rows, kv_heads=8, width=128: attention.decode_ring(rows, kv_heads, DEVICE, width)
    assert not ring(1) and not ring(8) and not ring(32)           # all on one wave already: 8..256 blocks on 444 places
    assert ring(64)                                               # 512 blocks: 592 places with the ring, 444 without
    assert not ring(100)                                          # 800 blocks: two rounds either way
    assert ring(128)                                              # 1024 blocks: two rounds against three
    assert not ring(64, width=48)                                 # a width the page-copying kernel does not take
    assert not ring(64, width=64)                                 # four blocks an SM fit without it


def test_key_splits_stay_within_the_pages_and_use_idle_sms():
    splits = lambda rows, tokens: attention.decode_splits(rows, 8, tokens, DEVICE, 128)
    assert splits(1, 10) == 1 and splits(8, 64) == 1              # one page: nothing to split
    assert splits(64, 1060) == 1                                  # the ring form: a block per row and head
    for rows in (1, 2, 8, 16, 32):
        for tokens in (100, 1060, 4000, 16000):
            chosen = splits(rows, tokens)
            assert 1 <= chosen <= -(-tokens // 64)
    assert splits(1, 16000) > splits(1, 300) >= 1                 # long sequences of a small batch are split further
    assert splits(8, 1060) > 1                                    # 64 blocks alone would leave most SMs idle


def test_forced_splits_are_clamped_to_the_pages(monkeypatch):
    monkeypatch.setenv("KIDI_B200_DECODE_SPLITS", "7")
    assert attention.decode_splits(8, 8, 1060, DEVICE, 128) == 7
    assert attention.decode_splits(8, 8, 100, DEVICE, 128) == 2


def test_which_product_a_shape_goes_to():
    def operands(rows, features, width=4096):
        # Meta tensors: shapes, strides and element types without memory (the address reads as 0).
        return (torch.empty(rows, width, dtype=torch.bfloat16, device="meta"),
                torch.empty(features, width, dtype=torch.bfloat16, device="meta"))
    assert skinny.fits(*operands(8, 4096)) and skinny.fits(*operands(1, 24576))
    assert skinny.fits(*operands(8, 6144))
    assert skinny._row_tiles(6144, 8, DEVICE) == 4                # 1.3 rounds of heavy blocks on 148 SMs: light blocks
    assert skinny._row_tiles(4096, 8, DEVICE) == 1 and skinny._row_tiles(24576, 8, DEVICE) == 1
    assert skinny._row_tiles(6144, 9, DEVICE) == 1
    assert not skinny.fits(*operands(9, 4096))
    assert not skinny.fits(*operands(8, 4096, width=4100))        # rows that 16-byte vectors cannot read
    assert tcgen05.fits(*operands(16, 24576)) and not tcgen05.fits(*operands(17, 24576))
    assert tcgen05.fits(*operands(64, 65536)) and not tcgen05.fits(*operands(65, 65536))   # as tall as an output head
    assert tcgen05.fits_prompt(*operands(2048, 4096)) and tcgen05.fits_prompt(*operands(1024, 6144))
    assert not tcgen05.fits_prompt(*operands(1023, 4096)) and not tcgen05.fits_prompt(*operands(2048, 4096, width=4100))
    assert tcgen05.MIN_GATED_ROWS == skinny.MAX_ROWS + 1          # no batch size falls between the two kernels

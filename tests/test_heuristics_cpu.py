"""Host-side launch heuristics of the kernel library (no GPU needed: the library loads on a CPU host and these
functions only do arithmetic on the problem shape, for a 148-SM part when no device is visible)."""
import pytest
import torch

from cosmos_b200 import ops


@pytest.fixture(scope="module")
def k():
    if not ops.load_extension():
        pytest.skip("kernel library not built")
    return torch.ops.cosmos_b200


@pytest.mark.parametrize("m,n,k_,epi,want", [
    (32, 6144, 4096, ops.EPI_PLAIN, 6),        # QKV projection of a decode step: 24 tiles, one wave of 144 items
    (32, 4096, 12288, ops.EPI_PLAIN, 9),       # down projection: 16 tiles x 9
    (32, 24576, 4096, ops.EPI_SWIGLU, 3),      # 96 tiles: 3 splits = 1.95 rounds of 148 CTAs
    (1, 24576, 4096, ops.EPI_SWIGLU, 3),
    (256, 24576, 4096, ops.EPI_SWIGLU, 1),     # 192 tiles: more than a wave already
    (256, 6144, 4096, ops.EPI_PLAIN, 3),       # two row tiles: 48 tiles x 3
    (512, 6144, 4096, ops.EPI_PLAIN, 1),       # taller problems do not take the multi-round split
    (32, 151936, 4096, ops.EPI_PLAIN, 1),      # LM head: hundreds of tiles
    (32, 4096, 256, ops.EPI_PLAIN, 1),         # too short a K to split
    (32, 768, 4096, ops.EPI_QKV_ROPE, 1),      # epilogues without a split-K form
])
def test_split_k_choice_for_decode_shapes(k, m, n, k_, epi, want):
    assert k.gemm_pick_k_splits(m, n, k_, epi) == want


def test_split_k_items_fill_whole_rounds(k):
    """Whatever the choice, it never leaves more than a third of the last round of persistent CTAs idle when it
    splits a problem of more than half a wave."""
    for n in range(74 * 256, 148 * 256, 256):
        ks = k.gemm_pick_k_splits(32, n, 4096, ops.EPI_PLAIN)
        items = (n // 256) * ks
        rounds = -(-items // 148)
        assert ks == 1 or items / (rounds * 148) > 0.66, (n, ks)


def test_paged_decode_split_choice(k):
    # long contexts, few (sequence, kv head) pairs: split so that every SM has work
    assert k.paged_decode_pick_splits(1, 8, 8448, 0) >= 8
    # a serving batch with short contexts: no split, no merge kernel
    assert k.paged_decode_pick_splits(256, 8, 416, 0) == 1

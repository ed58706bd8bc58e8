"""Host-side planning helpers of the program builder (no GPU): the K-slice choice of few-row GEMMs
and the per-worker key shares of decode attention."""
import collections

import pytest

from maco_b200.ops.megakernel import attention_pieces, pick_split_k


@pytest.mark.parametrize("groups,kv_len,workers", [(256, 4097, 148), (512, 4097, 148), (64, 4097, 148),
                                                   (6, 1037, 148), (16, 1400, 148), (3, 301, 5), (1, 1, 148)])
def test_attention_pieces_cover_every_key_once_and_balance(groups, kv_len, workers):
    pieces = attention_pieces(groups, kv_len, workers)
    covered = collections.defaultdict(list)
    load = collections.Counter()
    for g, s0, keys, w in pieces:
        assert keys > 0 and 0 <= w < workers
        assert s0 % 128 == 0                              # cuts inside a group sit on chunk boundaries
        covered[g].append((s0, keys))
        load[w] += keys
    assert sorted(covered) == list(range(groups))
    for g, spans in covered.items():                      # contiguous, in order, whole range
        pos = 0
        for s0, keys in spans:
            assert s0 == pos
            pos += keys
        assert pos == kv_len
    target = -(-(groups * kv_len) // workers)
    assert max(load.values()) <= -(-target // 128) * 128 + 128
    # a worker's pieces are consecutive in emission order (its queue reads memory front to back)
    seen, last = set(), None
    for _, _, _, w in pieces:
        if w != last:
            assert w not in seen
            seen.add(w)
            last = w


def test_split_k_fills_the_machine_without_extra_waves():
    W = 148
    for n_tiles, k_blocks in [(20, 80), (20, 64), (100, 80), (20, 200), (5, 80), (25, 80)]:
        sp = pick_split_k(n_tiles, k_blocks, W)
        assert 1 <= sp <= max(1, k_blocks // 2)
        waves = -(-n_tiles * sp // W)
        # never worse than the unsplit GEMM under the same cost model
        assert waves * (-(-k_blocks // sp) + 8) <= -(-n_tiles // W) * (k_blocks + 8)
    assert pick_split_k(20, 80, W) * 20 <= W            # one wave when the tiles fit
    assert pick_split_k(400, 16, W) == 1 or pick_split_k(400, 16, W) <= 8


def test_block_weight_round_trip_and_tile_contiguity():
    import torch
    from maco_b200.ops.gemm import block_weight, unblock_weight
    w = torch.arange(512 * 192, dtype=torch.float32).view(512, 192).to(torch.bfloat16)
    wb = block_weight(w)
    assert wb.shape == (2, 3, 256, 64) and wb.is_contiguous()
    assert torch.equal(wb[1, 2], w[256:512, 128:192])           # one tile's k-block is one contiguous 32 KB block
    assert torch.equal(unblock_weight(wb), w)
    with pytest.raises(ValueError):
        block_weight(w[:100])

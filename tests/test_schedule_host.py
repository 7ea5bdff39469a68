"""The split-KV schedule as the library cuts it on the host (fst_cuda_mla_debug_schedule: no device
involved).  Two rules: token by token (decode; reference src/fst_engine.cpp:3573-3589 attends to one
row's whole context in one call, the split is this build's) and by blocks of query tokens (the
engine's 16-row chunks, 2959, and DSpark's verify blocks, 6005-6014).  Checked here: every visible
row of every token is covered exactly once, a token's partial slots are contiguous and ordered by
rows, the work is balanced, and under the block rule the lanes of a group walk the same pages."""
import numpy as np
import pytest

from fastar_b200 import mla

N_SM = 148


def visible(pos0, q_len, i, causal):
    return pos0 + i + 1 if causal else pos0 + q_len


def check_cover(segs, pos0, q_lens, causal):
    """Every token's rows [0, kvlen) exactly once; parts contiguous per token, ascending with rows."""
    t0 = np.concatenate([[0], np.cumsum(q_lens)])
    next_part = 0
    for b, (p, q) in enumerate(zip(pos0, q_lens)):
        for i in range(q):
            t = int(t0[b]) + i
            mine = segs[segs[:, 0] == t]
            mine = mine[np.argsort(mine[:, 3])]
            want = visible(p, q, i, causal)
            row = 0
            for tok, lo, hi, part, cta in mine:
                assert lo == row and hi > lo, (t, mine)
                assert part == next_part
                next_part += 1
                row = hi
            assert row == want, (t, row, want)
    assert next_part == len(segs)


def cta_cost(segs, n_ctas):
    """Half-tile units: 2 per 64-row tile + 6 per segment, as the cutting rule counts."""
    cost = np.zeros(n_ctas, np.int64)
    for tok, lo, hi, part, cta in segs:
        cost[cta] += 2 * ((hi + 63) // 64 - lo // 64) + 6
    return cost


def test_decode_batch_is_cut_token_by_token_and_balanced():
    rng = np.random.default_rng(0)
    pos0 = rng.integers(1024, 8193, size=64)
    q = np.ones(64, np.int64)
    segs, n_ctas, blocks = mla.debug_schedule(N_SM, pos0, q, causal=False)
    assert not blocks and n_ctas == N_SM
    check_cover(segs, pos0, q, False)
    assert len(segs) <= N_SM + 64
    cost = cta_cost(segs, n_ctas)
    assert cost.max() <= 1.06 * cost.mean(), (cost.max(), cost.mean())
    # thread blocks walk their segments in order of token and rows
    for k in range(n_ctas):
        mine = segs[segs[:, 4] == k]
        assert np.all(np.diff(mine[:, 0]) >= 0)


@pytest.mark.parametrize("G,causal", [(16, True), (5, False), (4, True)])
def test_blocks_of_tokens_are_cut_by_groups_of_lanes(G, causal):
    rng = np.random.default_rng(G)
    pos0 = np.concatenate([rng.integers(0, 20000, size=11), [255, 256, 1023, 16384]])
    q = np.full(len(pos0), G)
    segs, n_ctas, blocks = mla.debug_schedule(N_SM, pos0, q, causal=causal)
    assert blocks and n_ctas == N_SM // G * G
    check_cover(segs, pos0, q, causal)
    # lane i of every group serves token i of a sequence, and the lanes of a group walk the same rows
    # (up to each token's own causal edge)
    for g in range(n_ctas // G):
        lanes = [segs[segs[:, 4] == g * G + i] for i in range(G)]
        ref = lanes[G - 1]                      # the last token of a block sees the most rows
        for i, mine in enumerate(lanes):
            assert np.all(mine[:, 0] % G == i)
            for tok, lo, hi, part, cta in mine:
                twin = ref[(ref[:, 0] == tok - i + G - 1) & (ref[:, 1] == lo)]
                assert len(twin) == 1 and (hi == twin[0, 2] or hi == visible(pos0[tok // G], G, i, causal))
    # groups are balanced by the cost of their last lane
    cost = cta_cost(segs, n_ctas)[G - 1::G]
    assert cost.max() <= 1.08 * cost.mean(), (cost.max(), cost.mean())
    # a group boundary adds one part to the G tokens of the sequence it cuts, nothing else does
    assert len(segs) <= len(pos0) * G + n_ctas


def test_block_rule_declines_what_it_does_not_fit():
    # too few pages for the groups, unequal block lengths, decode: the token rule cuts these
    for pos0, q in (([100, 200], [16, 16]), ([5000, 5000], [16, 8]), ([5000] * 8, [1] * 8), ([5000] * 4, [3] * 4)):
        segs, n_ctas, blocks = mla.debug_schedule(N_SM, pos0, q, causal=True)
        assert not blocks
        check_cover(segs, pos0, q, True)
    # switched off, a verify block is cut token by token over all thread blocks
    segs, n_ctas, blocks = mla.debug_schedule(N_SM, [16384] * 32, [16] * 32, causal=True, by_blocks=False)
    assert not blocks and n_ctas == N_SM
    check_cover(segs, [16384] * 32, [16] * 32, True)
    segs_b, n_b, blocks_b = mla.debug_schedule(N_SM, [16384] * 32, [16] * 32, causal=True)
    assert blocks_b and n_b == 144 and len(segs_b) < len(segs)


def test_empty_and_tiny_calls():
    segs, n_ctas, blocks = mla.debug_schedule(N_SM, [], [], causal=False)
    assert len(segs) == 0
    segs, n_ctas, blocks = mla.debug_schedule(N_SM, [0, 3], [1, 1], causal=True)
    check_cover(segs, [0, 3], [1, 1], True)
    assert n_ctas == 2

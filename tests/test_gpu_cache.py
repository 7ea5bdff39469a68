"""Latent-cache indexing and page mapping through the C ABI: bit-exact against the host twin
of the bookkeeping and against the flat cache of the reference (include/fst_engine.h:108-113,
src/fst_engine.cpp:3534-3544 append, 6132-6147 rollback, 2992-3012 reset)."""
import numpy as np
import pytest

from fastar_b200 import mla, synth
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture()
def ctx():
    c = mla.MlaContext(mla.make_config(n_layers=2, n_pages=40, max_seqs=6, max_tokens=8))
    yield c
    c.close()


def test_page_mapping_matches_twin(ctx):
    tw = O.Pager(40, 64, 6)
    rng = np.random.default_rng(0)
    live = {}
    for it in range(200):
        op = rng.integers(0, 4)
        if op == 0 and len(live) < 6:
            a, b = ctx.seq_alloc(), tw.seq_alloc()
            assert a == b
            live[a] = 0
        elif op == 1 and live:
            s = int(rng.choice(list(live)))
            n = live[s] + int(rng.integers(0, 300))
            rc_t = tw.reserve(s, n)
            if rc_t == 0:
                ctx.seq_reserve(s, n)
                live[s] = n
            else:
                with pytest.raises(mla.MlaError) as e:
                    ctx.seq_reserve(s, n)
                assert e.value.code == mla.ERR_PAGES
        elif op == 2 and live:
            s = int(rng.choice(list(live)))
            n = int(rng.integers(0, live[s] + 1))
            ctx.seq_truncate(s, n)
            assert tw.truncate(s, n) == 0
            live[s] = n
        elif op == 3 and live:
            s = int(rng.choice(list(live)))
            ctx.seq_free(s)
            assert tw.seq_free(s) == 0
            del live[s]
        owned = []
        for s, n in live.items():
            assert np.array_equal(ctx.block_table(s), tw.table(s))
            assert ctx.seq_len(s) == n
            table = [int(x) for x in ctx.block_table(s)]
            # invariants that do not come from the twin: a sequence holds exactly the pages its
            # length needs, every page number is in range
            assert len(table) == (n + 63) // 64
            assert all(0 <= pg < 40 for pg in table)
            owned += table
        assert ctx.free_pages() == tw.free_pages()
        # ... no page is owned twice, and owned + free pages are the whole pool
        assert len(owned) == len(set(owned))
        assert len(owned) + ctx.free_pages() == 40


def test_rows_land_where_the_table_says(ctx):
    rng = np.random.default_rng(1)
    # scramble the free list first
    tmp = [ctx.seq_alloc() for _ in range(3)]
    for s in tmp:
        ctx.seq_reserve(s, 64 * 5)
    for s in (tmp[1], tmp[0], tmp[2]):
        ctx.seq_free(s)
    a, b = ctx.seq_alloc(), ctx.seq_alloc()
    rows_a = rng.integers(0, 2 ** 16, size=(150, 576)).astype(np.uint16)
    rows_b = rng.integers(0, 2 ** 16, size=(70, 576)).astype(np.uint16)
    ctx.cache_write(1, a, 0, rows_a[:100])
    ctx.cache_write(1, b, 0, rows_b)
    ctx.cache_write(1, a, 100, rows_a[100:])
    pool = ctx.pool_read(1).reshape(-1)
    for seq, rows in ((a, rows_a), (b, rows_b)):
        table = ctx.block_table(seq)
        for pos in range(rows.shape[0]):
            off = ctx.row_offset(seq, pos)
            assert off == (int(table[pos // 64]) * 64 + pos % 64) * 576
            assert np.array_equal(pool[off:off + 576], rows[pos])
        # the paged view reads back as the reference's flat [max_seq, row] buffer
        assert np.array_equal(ctx.cache_read(1, seq, 0, rows.shape[0]), rows)
    assert not ctx.pool_read(0).any()  # the other layer's pool is untouched


def test_rollback_zeroes_rows_and_returns_pages(ctx):
    s = ctx.seq_alloc()
    rows = np.full((200, 576), 0x3F80, np.uint16)
    for lid in (0, 1):
        ctx.cache_write(lid, s, 0, rows)
    offs = [ctx.row_offset(s, p) for p in range(200)]
    free0 = ctx.free_pages()
    ctx.seq_truncate(s, 130)  # keeps 3 pages (rows 0..129), frees the 4th
    assert ctx.seq_len(s) == 130 and ctx.free_pages() == free0 + 1
    for lid in (0, 1):
        pool = ctx.pool_read(lid).reshape(-1)
        for p in range(200):
            want = 0x3F80 if p < 130 else 0
            assert np.all(pool[offs[p]:offs[p] + 576] == want), (lid, p)
    with pytest.raises(mla.MlaError):
        ctx.cache_read(0, s, 0, 131)
    with pytest.raises(mla.MlaError):
        ctx.seq_truncate(s, 131)


def test_reset_session(ctx):
    s = ctx.seq_alloc()
    ctx.cache_write(0, s, 0, np.full((64, 576), 7, np.uint16))
    ctx.reset()
    assert ctx.free_pages() == 40
    assert not ctx.pool_read(0).any()
    assert ctx.seq_alloc() == 0
    with pytest.raises(mla.MlaError):
        ctx.seq_len(3)


def test_errors_are_rejected_before_any_launch(ctx):
    n0 = ctx.launch_count()
    s = ctx.seq_alloc()
    with pytest.raises(mla.MlaError) as e:
        ctx.plan([(s, 0, 9)])  # max_tokens = 8
    assert e.value.code == mla.ERR_CAPACITY
    with pytest.raises(mla.MlaError) as e:
        ctx.plan([(s, 64 * 40, 1)])  # needs 41 pages
    assert e.value.code == mla.ERR_PAGES
    with pytest.raises(mla.MlaError) as e:
        ctx.plan([(5, 0, 1)])  # not allocated
    assert e.value.code == mla.ERR_ARG
    with pytest.raises(mla.MlaError) as e:
        ctx.plan([(s, 0, 1), (s, 1, 1)])  # the same sequence twice
    assert e.value.code == mla.ERR_ARG
    ctx.plan([(s, 0, 1)])
    with pytest.raises(mla.MlaError) as e:
        ctx.run_device(0, 1, 1)  # no weights
    assert e.value.code == mla.ERR_STATE
    with pytest.raises(mla.MlaError) as e:
        ctx.run_device(7, 1, 1)
    assert e.value.code == mla.ERR_ARG
    assert ctx.launch_count() == n0
    for _ in range(5):
        ctx.seq_alloc()
    with pytest.raises(mla.MlaError) as e:
        ctx.seq_alloc()
    assert e.value.code == mla.ERR_CAPACITY

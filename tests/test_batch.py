"""The description of a batch as the kernels get it: offsets, block tables, work lists (no GPU needed)."""

import numpy as np
import pytest

from jax_vllm_b200.cache import CacheManager
from jax_vllm_b200.engine.batch import BatchBuilder, StepEntry
from jax_vllm_b200.parts import PagedKVNeed


def manager(page=4, pages=32, live=4):
    return CacheManager([PagedKVNeed(2, 16, None)], page, pages, live, prefix_cache=False)


def filled(builder, entries, table_width=None):
    layout = builder.layout_for(entries, table_width)
    host = np.full(layout.total, -7, dtype=np.int32)
    builder.fill(entries, host, layout)
    return layout, host


def test_a_mixed_batch_is_laid_out_as_the_kernels_read_it():
    m = manager()
    a, b, c = m.admit("a"), m.admit("b"), m.admit("c")
    m.grow(a, 9); a.num_tokens = 6            # 6 tokens in the cache, 3 new
    m.grow(b, 11); b.num_tokens = 10          # a decoded token
    m.grow(c, 5)                              # a fresh portion of 5
    builder = BatchBuilder(1, 4, [(2, 2, 4), (4, 4, 1 << 30)], "cpu")
    entries = [StepEntry(a, [11, 12, 13], (2,)), StepEntry(b, [21], (0,)), StepEntry(c, [31, 32, 33, 34, 35], (0, 4))]
    layout, host = filled(builder, entries)
    v = lambda name: layout.view(host, name)
    assert v("token_ids").tolist() == [11, 12, 13, 21, 31, 32, 33, 34, 35]
    assert v("positions").tolist() == [6, 7, 8, 10, 0, 1, 2, 3, 4]
    assert v("token_entry").tolist() == [0, 0, 0, 1, 2, 2, 2, 2, 2]
    assert v("cu_seqlens").tolist() == [0, 3, 4, 9] and v("start_pos").tolist() == [6, 10, 0]
    assert v("logit_rows").tolist() == [2, 3, 4, 8]
    assert v("state_slots").tolist() == [a.slot, b.slot, c.slot]
    w = layout.table_widths[0]
    assert w == 3                              # the widest entry: 11 tokens in pages of 4
    table = v("table0").reshape(3, w)
    assert table[0].tolist() == a.tables[0][:3] and table[1].tolist() == b.tables[0][:3]
    assert table[2].tolist() == c.tables[0][:2] + [-1]
    # work lists: the 3-token entry in tiles of 2 (class 2..3), the 5-token entry in tiles of 4, the single token apart
    assert v("tiles(2, 2, 4)").reshape(-1, 2).tolist() == [[0, 0], [0, 2]]
    assert v(f"tiles{(4, 4, 1 << 30)}").reshape(-1, 2).tolist() == [[2, 0], [2, 4]]
    assert v("decode").reshape(-1, 2).tolist() == [[1, 0]]
    # every array begins on a 16-byte boundary
    assert all(off % 4 == 0 for off, _ in layout.sections.values())


def test_a_fixed_table_width_pads_with_minus_one_and_refuses_what_does_not_fit():
    m = manager()
    a = m.admit("a")
    m.grow(a, 6); a.num_tokens = 5
    builder = BatchBuilder(1, 4, [], "cpu")
    layout, host = filled(builder, [StepEntry(a, [1], (0,))], table_width=5)
    assert layout.view(host, "table0").tolist() == a.tables[0][:2] + [-1, -1, -1]
    with pytest.raises(RuntimeError, match="too narrow"):
        filled(builder, [StepEntry(a, [1], (0,))], table_width=1)
    b = m.admit("b")
    with pytest.raises(RuntimeError, match="pages"):
        filled(builder, [StepEntry(b, [1, 2, 3], ())])          # nobody grew it
    with pytest.raises(IndexError):
        filled(builder, [StepEntry(a, [1], (1,))])

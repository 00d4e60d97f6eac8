"""The CPU oracle's index surfaces (which cache rows a token attends to) against a plain per-token loop: sliding
window rows through the page -> window-slot map, compressed rows of every ratio, and rows picked by the indexer."""
from types import SimpleNamespace

import torch

from minisgl.ops import api as O

PS = 16


def _fb(positions, slots, table):
    return SimpleNamespace(positions=torch.tensor(positions, dtype=torch.int32),
                           slots=torch.tensor(slots, dtype=torch.int32), page_table=table)


def _table():
    """Two requests on scattered pages: slot 0 uses pages 5, 2, 9, 7; slot 1 pages 1, 8, 3."""
    t = torch.zeros(3, 64, dtype=torch.int32)
    for slot, pages in ((0, [5, 2, 9, 7]), (1, [1, 8, 3])):
        for i, p in enumerate(pages):
            t[slot, i * PS:(i + 1) * PS] = torch.arange(p * PS, (p + 1) * PS, dtype=torch.int32)
    return t


def test_window_rows_follow_the_slot_map_and_mask_what_is_gone():
    table = _table()
    swa_map = torch.full((12,), -1, dtype=torch.int32)
    swa_map[[2, 9, 7, 1, 8, 3]] = torch.tensor([4, 0, 6, 2, 5, 1], dtype=torch.int32)   # page 5 lost its window rows
    fb = _fb([40, 3, 20], [0, 0, 1], table)
    window = 32
    rows = O.swa_rows(fb, swa_map, PS, window)
    assert rows.shape == (3, window)
    for r, (pos, slot) in enumerate([(40, 0), (3, 0), (20, 1)]):
        for c in range(window):
            p = pos - (window - 1) + c                        # oldest position first, the token itself last
            want = -1
            if p >= 0:
                loc = int(table[slot, p])
                s = int(swa_map[loc // PS])
                if s >= 0:
                    want = s * PS + loc % PS
            assert int(rows[r, c]) == want, (r, c)
    assert int(rows[0, -1]) == 0 * PS + 40 % PS                # position 40 -> page 9 -> slot 0
    assert (rows[1] == -1).all()                               # positions 0..3 live on page 5, which has no slot


def test_compressed_rows_of_both_ratios():
    table = _table()
    fb = _fb([40, 3, 47, 15], [0, 0, 1, 1], table)
    for ratio, width in ((4, 12), (16, 4)):
        rows = O.comp_rows_all(fb, PS, ratio, width)
        assert rows.shape == (4, width)
        rpp = PS // ratio
        for r, (pos, slot) in enumerate([(40, 0), (3, 0), (47, 1), (15, 1)]):
            n = (pos + 1) // ratio                              # complete groups so far
            for j in range(width):
                want = -1
                if j < n:
                    loc = int(table[slot, j * ratio + ratio - 1])   # the group's last source token names its row
                    want = (loc // PS) * rpp + (loc % PS) // ratio
                assert int(rows[r, j]) == want, (ratio, r, j)
    # ratio 4, position 3 on page 5: exactly one complete group, row 5 * 4 + 0
    assert O.comp_rows_all(fb, PS, 4, 12)[1].tolist() == [20] + [-1] * 11


def test_rows_from_selected_indices_keep_order_and_padding():
    table = _table()
    fb = _fb([40, 47], [0, 1], table)
    idx = torch.tensor([[9, 0, -1, 3], [11, -1, -1, 2]], dtype=torch.int32)
    rows = O.comp_rows_from_idx(fb, idx, PS, 4)
    full = O.comp_rows_all(fb, PS, 4, 12)
    for r in range(2):
        for c in range(4):
            j = int(idx[r, c])
            assert int(rows[r, c]) == (-1 if j < 0 else int(full[r, j]))

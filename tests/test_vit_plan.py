"""CPU: the host-side plan of the vision encoder (window-major order, attention ranges, 2-D positions) computed
by the backend library equals the oracle's, for the benchmark images and ragged / multi-image / video grids."""
import pytest

import cabi
from oracle import qwen_vit

GRIDS = [[(1, 32, 32)], [(1, 52, 92)], [(1, 8, 8)], [(1, 10, 14)], [(2, 12, 6), (1, 4, 18)], [(1, 2, 2)], [(3, 6, 22)],
         [(1, 16, 16), (1, 18, 10), (2, 8, 8)]]


@pytest.mark.parametrize("grids", GRIDS)
def test_backend_plan_equals_oracle_plan(grids):
    cfg = qwen_vit.CONFIGS[2]
    want = qwen_vit.make_plan(cfg, grids)
    got = cabi.vit_plan(cfg, grids)
    assert got is not None
    assert got["order"] == want.order and got["pos_h"] == want.pos_h and got["pos_w"] == want.pos_w
    n = len(want.pos_h)
    lo = [0] * n
    hi = [0] * n
    for a, b in zip(want.cu_window[:-1], want.cu_window[1:]):
        lo[a:b], hi[a:b] = [a] * (b - a), [b] * (b - a)
    assert got["win_lo"] == lo and got["win_hi"] == hi
    for a, b in zip(want.cu_full[:-1], want.cu_full[1:]):
        lo[a:b], hi[a:b] = [a] * (b - a), [b] * (b - a)
    assert got["full_lo"] == lo and got["full_hi"] == hi
    assert sorted(got["order"]) == list(range(n // 4))              # a permutation of the merged tokens


def test_plan_refuses_grids_that_do_not_merge():
    cfg = qwen_vit.CONFIGS[2]
    assert cabi.vit_plan(cfg, [(1, 7, 8)]) is None
    assert cabi.vit_plan(cfg, [(0, 8, 8)]) is None
    assert cabi.vit_plan(cfg, [(1, 8, 8), (1, 8, 9)]) is None

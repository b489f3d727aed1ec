"""How the attention part plans its launches (host arithmetic only): the cut of a long portion's
keys into runs, and the splits of the context for single-token entries."""
import pytest

from neurogrid_b200.parts import attention


@pytest.fixture(autouse=True)
def b200_sms(monkeypatch):
    monkeypatch.setitem(attention._SM_COUNT, "cpu", 148)        # what sm_count() would ask the device for


def test_short_contexts_and_many_blocks_are_not_cut():
    assert attention.prefill_splits(512, 4096, "cpu") == 1       # below the threshold whatever the filling
    assert attention.prefill_splits(0, 1 << 20, "cpu") == 1
    assert attention.prefill_splits(6 * 296, 32768, "cpu") == 1  # whole rounds: nothing to gain
    assert attention.prefill_splits(512, 32768, "cpu") == 1      # 1.73 rounds: no cut improves the filling by a tenth


def test_uneven_rounds_are_cut_where_the_runs_stay_long():
    assert attention.prefill_splits(384, 32768, "cpu") == 3      # 24 heads x 16 row tiles: 1.3 rounds -> 3.9
    assert attention.prefill_splits(128, 32768, "cpu") == 2      # 512 rows of 32 heads: 0.43 of a round -> 0.86
    n = attention.prefill_splits(384, 8192, "cpu")
    assert 1 <= n <= attention.PREFILL_MAX_SPLITS and 8192 // (64 * n) >= 16     # a run keeps 16 tiles


def test_decode_splits_bounds():
    for batch in (1, 2, 8, 16, 64):
        for ctx in (1, 100, 600, 2100, 8000, 32768):
            for window in (None, 512):
                n = attention.decode_splits(batch, 8, ctx, window, "cpu")
                span = min(window, ctx) if window else ctx
                assert n >= 1 and (n == 1 or span // n >= 256), (batch, ctx, window, n)
    assert attention.decode_splits(8, 8, 2100, None, "cpu") > attention.decode_splits(64, 8, 2100, None, "cpu")

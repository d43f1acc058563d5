"""The tensor-core instruction-rate probe runs and reports sane figures (the numbers themselves are
what `python -m warpir_b200.probe` prints; here only bounds that must hold on any B200)."""
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("pair", [False, True])
def test_full_width_instruction_runs_near_the_arithmetic_rate(pair):
    from warpir_b200 import probe
    r = probe.mma_rate(256, ts=False, pair=pair, batches=256)
    assert r["arithmetic_clocks"] == 128
    # never faster than the arithmetic allows, and not absurdly slower
    assert 0.9 * r["arithmetic_clocks"] <= r["clocks_per_mma"] <= 2.0 * r["arithmetic_clocks"], r
    assert r["issue_clocks_per_mma"] <= r["clocks_per_mma"]


def test_narrow_and_tensor_memory_forms_report():
    from warpir_b200 import probe
    for n in (64, 128):
        for ts in (False, True):
            r = probe.mma_rate(n, ts=ts, pair=False, batches=128, bg_tmem=True, bg_tma=True)
            assert r["clocks_per_mma"] >= 0.9 * r["arithmetic_clocks"], r

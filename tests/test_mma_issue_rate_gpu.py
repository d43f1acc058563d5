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


def test_commits_are_free_and_a_second_issuing_warp_runs():
    """A tcgen05.commit after every block of four 32-clock MMAs does not slow the stream by more than a quarter
    (measured: not at all on an idle SM), and two issuing warps complete the same stream each."""
    from warpir_b200 import probe
    base = probe.mma_rate(64, ts=True, pair=False, batches=256)["clocks_per_mma"]
    with_commits = probe.mma_rate(64, ts=True, pair=False, batches=256, commit_every=1)["clocks_per_mma"]
    assert with_commits <= 1.25 * base, (base, with_commits)
    two = probe.mma_rate(64, ts=True, pair=False, batches=256, commit_every=1, issuers=2)
    assert two["issuers"] == 2 and two["clocks_per_mma"] >= 0.9 * 32, two


def test_issue_loop_shapes_and_replayed_orders_run():
    """The dQ kernel's issue loop runs at the tensor core's rate when it looks at no barrier (768 clocks of
    arithmetic per step) and not faster than that in any shape; a replayed issue order reports its clocks."""
    from warpir_b200 import probe
    issued, total = probe.issue_loop(3, steps=128)
    assert 0.95 * 768 <= total <= 1.15 * 768, total
    for shape in (1, 10):
        _, t = probe.issue_loop(shape, steps=128, busy=1)
        assert t >= 0.95 * 768, (shape, t)
    clocks = probe.mma_pattern([(64, 0, 1, 0), (64, 128, 1, 1), (128, 320, 0, 1)], steps=64)
    assert clocks >= 0.9 * (2 * 4 * 32 + 4 * 64), clocks

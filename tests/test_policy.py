"""The recompute-vs-offload plan is a pure host function: tested here without a GPU."""
import pytest

from flame_b200.errors import InvalidInput
from flame_b200.policy import Decision, SavedTensor, plan

MB = 1 << 20


def dit_tensors(blocks=20):
    per_block = [28 * MB, 28 * MB, 85 * MB, 28 * MB, 170 * MB]
    return [SavedTensor(nbytes=b, group=g, recompute_ms=0.02 * b / MB) for g in range(blocks) for b in per_block]


def test_everything_fits_under_a_fast_link():
    dec, est = plan(dit_tensors(), d2h_gbs=1000, h2d_gbs=1000, fwd_ms=60, bwd_ms=120)
    assert set(dec) == {Decision.OFFLOAD_INT8} and est == 0.0


def test_resident_budget_goes_to_the_last_blocks():
    ts = dit_tensors()
    dec, _ = plan(ts, d2h_gbs=1000, h2d_gbs=1000, fwd_ms=60, bwd_ms=120, device_budget_bytes=2 * 339 * MB)
    resident_groups = {t.group for t, d in zip(ts, dec) if d == Decision.RESIDENT}
    assert resident_groups == {18, 19}


def test_slow_link_switches_cheap_tensors_to_recompute_and_reports_the_rest():
    ts = dit_tensors()
    dec, est = plan(ts, d2h_gbs=5, h2d_gbs=5, fwd_ms=60, bwd_ms=120)
    assert Decision.RECOMPUTE in dec
    dec2, est2 = plan([SavedTensor(t.nbytes, t.group, -1.0) for t in ts], d2h_gbs=5, h2d_gbs=5, fwd_ms=60, bwd_ms=120)
    assert Decision.RECOMPUTE not in dec2 and est2 > est > 0


def test_lossless_tensors_stay_bf16_and_plan_is_deterministic():
    ts = [SavedTensor(100 * MB, 0, allow_lossy=False), SavedTensor(100 * MB, 1)]
    a = plan(ts, d2h_gbs=50, h2d_gbs=50, fwd_ms=10, bwd_ms=20, lossy_codec=Decision.OFFLOAD_FP8)
    assert a[0] == [Decision.OFFLOAD_BF16, Decision.OFFLOAD_FP8]
    assert a == plan(ts, d2h_gbs=50, h2d_gbs=50, fwd_ms=10, bwd_ms=20, lossy_codec=Decision.OFFLOAD_FP8)


def test_bad_rates_are_rejected():
    with pytest.raises(InvalidInput):
        plan(dit_tensors(1), d2h_gbs=0, h2d_gbs=10, fwd_ms=1, bwd_ms=1)


def test_block_plan_keeps_trailing_blocks_resident_and_counts_interference():
    from flame_b200.policy import Block, plan_blocks

    blocks = [Block(340 * MB, 1.64, 3.74) for _ in range(20)]
    free = plan_blocks(blocks, d2h_gbs=57, h2d_gbs=55.5, device_budget_bytes=8 * 340 * MB, interference=0.0)
    # without an interference term the cheapest plan in memory wins among the stall-free ones
    assert free.est_stall_ms < 0.5 and "".join("R" if d == Decision.RESIDENT else "O" for d in free.decisions).endswith("RRRR")
    assert free.decisions.count(Decision.RESIDENT) < 8
    costed = plan_blocks(blocks, d2h_gbs=57, h2d_gbs=55.5, device_budget_bytes=8 * 340 * MB, interference=0.1)
    assert costed.decisions.count(Decision.RESIDENT) == 8 and costed.decisions[:12] == [Decision.OFFLOAD_INT8] * 12
    assert 0 < costed.est_interference_ms < 10
    all_res = plan_blocks(blocks, d2h_gbs=57, h2d_gbs=55.5, device_budget_bytes=10 ** 12)
    assert set(all_res.decisions) == {Decision.RESIDENT} and all_res.link_bytes == 0
    none = plan_blocks(blocks, d2h_gbs=57, h2d_gbs=55.5, device_budget_bytes=0, offload=Decision.OFFLOAD_BF16)
    assert Decision.RESIDENT not in none.decisions and (Decision.RECOMPUTE in none.decisions)


def test_capped_plan_offloads_less_over_a_slower_link():
    """overhead_cap_ms: the fewest resident bytes whose estimated extra time stays under the cap."""
    from flame_b200.policy import Block, plan_blocks

    blocks = [Block(340 * MB, 1.64, 3.74) for _ in range(20)]
    step_ms = 20 * (1.64 + 3.74)
    cap = 0.04 * step_ms
    fast = plan_blocks(blocks, d2h_gbs=57, h2d_gbs=55.5, overhead_cap_ms=cap)
    slow = plan_blocks(blocks, d2h_gbs=10, h2d_gbs=21, overhead_cap_ms=cap)
    slower = plan_blocks(blocks, d2h_gbs=3, h2d_gbs=6, overhead_cap_ms=cap)
    for p in (fast, slow, slower):
        assert p.est_stall_ms + p.est_recompute_ms + p.est_interference_ms <= cap + 1e-9
        # residents are the trailing blocks, recomputed ones the leading blocks
        s = "".join({Decision.RESIDENT: "R", Decision.RECOMPUTE: "C"}.get(d, "O") for d in p.decisions)
        assert s == "C" * s.count("C") + "O" * s.count("O") + "R" * s.count("R")
    assert fast.resident_bytes < slow.resident_bytes <= slower.resident_bytes
    assert fast.link_bytes > slow.link_bytes >= slower.link_bytes
    # a cap nothing but the all-resident plan meets still gives a plan
    none = plan_blocks(blocks, d2h_gbs=57, h2d_gbs=55.5, overhead_cap_ms=1e-6, interference=0.1)
    assert set(none.decisions) == {Decision.RESIDENT}
    assert plan_blocks(blocks, d2h_gbs=10, h2d_gbs=21, overhead_cap_ms=cap).decisions == slow.decisions  # deterministic

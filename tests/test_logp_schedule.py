"""Schedule selection of the fused log-prob (host logic only: no GPU needed)."""
import pytest

from kernel_align_b200.ops import fused_logp


def _never(*a):
    raise AssertionError("a short call must not time candidates")


def test_pinned_schedule_is_parsed_and_validated(monkeypatch):
    monkeypatch.setenv("KA_LOGP_SCHEDULE", "1,4")
    assert fused_logp._pinned_schedule() == (1, 4, 0, 0)
    monkeypatch.setenv("KA_LOGP_SCHEDULE", "2,8,2,3")
    assert fused_logp._pinned_schedule() == (2, 8, 2, 3)
    assert fused_logp._choose_schedule(("k",), 1e15, None, _never) == (2, 8, 2, 3)
    for bad in ("3,8", "2,99", "2,8,4", "2,8,0,9", "x"):
        monkeypatch.setenv("KA_LOGP_SCHEDULE", bad)
        with pytest.raises(ValueError):
            fused_logp._pinned_schedule()


def test_short_calls_take_a_default_by_shard_size(monkeypatch):
    monkeypatch.delenv("KA_LOGP_SCHEDULE", raising=False)
    fused_logp._tuned.clear()
    # a vocabulary sharded eight ways at G = 256: 8.6e12 multiply-adds, a 131 MB shard
    macs = 131072.0 * 4096 * 16032
    assert fused_logp._choose_schedule(("a",), macs, None, _never, shard_bytes=16032 * 4096 * 2) == \
        fused_logp._SMALL_SHARD_SCHEDULE
    # the same work on a full LM head (a few rows): the default
    assert fused_logp._choose_schedule(("b",), 1e12, None, _never, shard_bytes=128256 * 4096 * 2) == \
        fused_logp._DEFAULT_SCHEDULE
    # tiny calls never get the W-stationary order either
    assert fused_logp._choose_schedule(("c",), 1e6, None, _never, shard_bytes=1024) == fused_logp._DEFAULT_SCHEDULE
    # every candidate is a valid (cta_group, cg, order, hint)
    for g, cg, order, hint in fused_logp._SCHEDULES + [fused_logp._SMALL_SHARD_SCHEDULE]:
        assert g in (1, 2) and 1 <= cg <= 64 and order in (0, 1, 2, 3) and hint in (0, 1, 2, 3)
    assert not fused_logp._tuned

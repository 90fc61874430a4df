"""Step timing slots on the host clock (the CUDA-event path is the same code with events)."""
import time

import pytest

from dgpp_b200.utils.step_timing import StepTimer


def test_disabled_timer_is_inert_and_enabled_timer_accumulates(monkeypatch):
    off = StepTimer(enabled=False, use_cuda=False)
    with off.phase("decode"):
        pass
    assert off.timings() == {}
    t = StepTimer(enabled=True, use_cuda=False)
    for _ in range(3):
        with t.phase("decode"):
            time.sleep(0.002)
    with t.phase("pick"):
        pass
    got = t.timings()
    assert got["decode"]["n"] == 3 and got["decode"]["ms"] >= 5.0 and set(got) == {"decode", "pick"}
    assert t.timings(reset=True)["decode"]["n"] == 3 and t.timings() == {}
    with pytest.raises(KeyError):
        with t.phase("nope"):
            pass
    monkeypatch.setenv("DGPP_STEP_TIMING", "1")
    assert StepTimer(use_cuda=False).enabled
    monkeypatch.setenv("DGPP_STEP_TIMING", "0")
    assert not StepTimer(use_cuda=False).enabled

import math

import pytest

from nexus_b200.train.schedule import ConstantLr, InverseSqrt, LinearLr, LrSchedule, WarmupCosine, WSD


def test_warmup_is_nanogpt_style():
    s = LrSchedule(ConstantLr(warmup_steps=9))
    assert s.factor(0) == pytest.approx(0.1) and s.factor(8) == pytest.approx(0.9) and s.factor(9) == 1.0


def test_cosine_linear_wsd_invsqrt():
    c = LrSchedule(WarmupCosine(10, 110, 0.1))
    assert c.factor(10) == pytest.approx(1.0) and c.factor(60) == pytest.approx(0.55) and c.factor(500) == 0.1
    l = LrSchedule(LinearLr(0, 100, 0.0))
    assert l.factor(50) == pytest.approx(0.5)
    w = LrSchedule(WSD(2, 5, 4, 0.0))
    assert w.factor(6) == 1.0 and w.factor(7) == pytest.approx(0.75) and w.factor(10) == pytest.approx(0.0)
    ws = LrSchedule(WSD(0, 0, 4, 0.0, sqrt_decay=True))
    assert ws.factor(0) == pytest.approx(1 - math.sqrt(0.25))
    i = LrSchedule(InverseSqrt(3))
    assert i.factor(3) == pytest.approx(1.0) and i.factor(15) == pytest.approx(0.5)
    assert LrSchedule().describe() == "constant"


def test_invalid_arguments():
    with pytest.raises(ValueError):
        WarmupCosine(10, 5)
    with pytest.raises(ValueError):
        LrSchedule().factor(-1)
    with pytest.raises(ValueError):
        InverseSqrt(0)

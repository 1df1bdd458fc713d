"""Statistics of the paired benchmark protocol (rotated arms, A/A control, bootstrap interval); no GPU."""
import math

import pytest

from conftest import pkg


def test_rotation_visits_every_position_equally():
    P = pkg("paired")
    order = []
    arms = {n: (lambda n=n: order.append(n) or 1.0) for n in ("a", "b", "c")}
    res = P.rotated_rounds(arms, 6)
    assert [len(v) for v in res.values()] == [6, 6, 6]
    rounds = [order[i:i + 3] for i in range(0, 18, 3)]
    assert rounds[0] == ["a", "b", "c"] and rounds[1] == ["b", "c", "a"] and rounds[2] == ["c", "a", "b"]
    for pos in range(3):                                   # each arm runs first, second and third twice
        assert sorted(r[pos] for r in rounds) == ["a", "a", "b", "b", "c", "c"]


def test_ratio_stats_cancels_common_drift():
    P = pkg("paired")
    drift = [1.0, 1.1, 0.9, 1.2, 0.8, 1.05]                # a load that hits both arms of a round alike
    a = [1000.0 * d for d in drift]
    b = [800.0 * d for d in drift]
    st = P.ratio_stats(a, b)
    assert st["median"] == pytest.approx(1.25) and st["min"] == pytest.approx(1.25) and st["max"] == pytest.approx(1.25)
    assert st["ci95"][0] == pytest.approx(1.25) and st["ci95"][1] == pytest.approx(1.25)
    aa = P.ratio_stats(a, a)
    assert aa["median"] == 1.0 and aa["geo_mean"] == 1.0


def test_ratio_stats_interval_brackets_the_mean_and_is_deterministic():
    P = pkg("paired")
    a = [100, 104, 98, 101, 99, 103]
    b = [100, 100, 100, 100, 100, 100]
    s1, s2 = P.ratio_stats(a, b, seed=3), P.ratio_stats(a, b, seed=3)
    assert s1 == s2
    assert s1["ci95"][0] <= s1["geo_mean"] <= s1["ci95"][1]
    assert s1["min"] == 0.98 and s1["max"] == 1.04
    assert math.isclose(s1["median"], 1.005)
    with pytest.raises(ValueError):
        P.ratio_stats([1.0], [1.0, 2.0])

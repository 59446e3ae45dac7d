"""Support-layer utilities: branch-free abs, wall-clock checkpoint timer."""
import math
import time

import hipress_b200 as hp


def test_fast_abs_all_types():
    C = hp._C
    for v in (0, 1, -1, 123456, -123456, 2**31 - 1, -(2**31 - 1)):
        assert C.fast_abs_i32(v) == abs(v)
    for v in (0, -1, 2**62, -(2**62), -(2**63 - 1)):
        assert C.fast_abs_i64(v) == abs(v)
    for v in (0.0, -0.0, 1.5, -1.5, -2.0 ** -100, float("inf"), float("-inf")):   # exact in fp32
        assert C.fast_abs_f32(v) == abs(v) and math.copysign(1.0, C.fast_abs_f32(v)) == 1.0
        assert C.fast_abs_f64(v) == abs(v) and math.copysign(1.0, C.fast_abs_f64(v)) == 1.0
    assert math.isnan(C.fast_abs_f64(float("nan")))


def test_time_cost_checkpoints():
    t = hp._C.TimeCost()
    t.start()
    time.sleep(0.01)
    t.record("a")
    time.sleep(0.02)
    t.record("b")
    iv = t.intervals(1e3)
    assert [k for k, _ in iv] == ["a", "b"]
    assert 8 <= iv[0][1] < 200 and 15 <= iv[1][1] < 300
    assert "[a]" in t.print_by_us() and "ms" in t.print_by_ms() and "s" in t.print_by_s()

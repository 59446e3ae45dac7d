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


def test_clock_sampler_windows_samples_with_a_fake_nvidia_smi(tmp_path, monkeypatch):
    """The sampler reads nvidia-smi's CSV; a fake one on PATH prints timestamped rows.  Samples
    inside the marks are reported; when none fall inside, the whole span is, and the summary says so."""
    import os
    import stat
    import time
    from hipress_b200.utils import ClockSampler
    fake = tmp_path / "nvidia-smi"
    fake.write_text("#!/bin/bash\n"
                    "for i in $(seq 1 200); do\n"
                    "  echo \"$(date +'%Y/%m/%d %H:%M:%S.%3N'), 0, 1800, 1965, 650.0, 0x0, Not Active, Not Active, Not Active, Active\"\n"
                    "  sleep 0.02\n"
                    "done\n")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", str(tmp_path) + os.pathsep + os.environ["PATH"])
    with ClockSampler(0) as c:
        time.sleep(0.3)
        c.mark_start()
        time.sleep(0.3)
        c.mark_end()
        time.sleep(0.1)
    s = c.summary()
    assert s["sm_mhz"] == 1800 and s["sm_max_mhz"] == 1965 and s["reasons"] == ["sw_power_cap"]
    assert s["window"] == "timed region" and 3 <= s["samples"] <= 30
    total = len(c.rows())
    assert total > s["samples"]                       # samples outside the marks were left out
    c.t_start, c.t_end = time.time() + 100, time.time() + 101   # a region nothing fell into
    s2 = c.summary()
    assert s2["samples"] == total and "no sample fell inside" in s2["window"]


def test_prefer_sharded_rule():
    """The exchange-form rule: all-gather form wherever it was measured faster (2 and 4 ranks, any size),
    sharded only where it was measured faster: large buckets at 8 ranks."""
    from hipress_b200.parallel import prefer_sharded
    mb = 1 << 20
    for world in (1, 2, 4):
        for size in (256 * 1024, 25 * mb, 512 * mb):
            assert not prefer_sharded(size, world)
    assert not prefer_sharded(25 * mb, 8)
    assert not prefer_sharded(64 * mb, 8)
    assert prefer_sharded(512 * mb, 8)

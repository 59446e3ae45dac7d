"""The host runtime's plain-C++ parts (worker pool, finish queues, task watchdog) under
ThreadSanitizer and AddressSanitizer + UBSan: a stress test with several submitting threads, a
polling thread, failing jobs and a shutdown with work queued.  No GPU involved.  (The reference
shares one static stream between its five threads and bumps its round-robin counter without
synchronisation, ref hp_cuda.cpp:789, 930; it has no test of its runtime at all.)"""
import subprocess

import pytest

from hipress_b200.build import build_sanitized


@pytest.mark.parametrize("kind", ["thread", "address"])
def test_runtime_stress_under_sanitizer(kind):
    try:
        exe = build_sanitized(kind)
    except RuntimeError as exc:   # a toolchain without the sanitizer runtime
        if "sanitize" in str(exc) or "cannot find" in str(exc):
            pytest.skip(f"-fsanitize={kind} is not available here")
        raise
    env = {"TSAN_OPTIONS": "halt_on_error=1 exitcode=66", "ASAN_OPTIONS": "detect_leaks=1 exitcode=66",
           "UBSAN_OPTIONS": "halt_on_error=1 exitcode=66", "PATH": "/usr/bin:/bin"}
    proc = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env=env)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "runtime_stress: ok" in proc.stdout
    assert "Sanitizer" not in proc.stderr, proc.stderr


@pytest.mark.parametrize("kind", ["thread", "address"])
def test_threaded_cpu_codecs_under_sanitizer(kind):
    """TBQ / TernGrad split over several threads, and two callers at once, with the results compared to the
    one-thread run inside the executable."""
    try:
        exe = build_sanitized(kind, target="codec")
    except RuntimeError as exc:
        if "sanitize" in str(exc) or "cannot find" in str(exc):
            pytest.skip(f"-fsanitize={kind} is not available here")
        raise
    env = {"TSAN_OPTIONS": "halt_on_error=1 exitcode=66", "ASAN_OPTIONS": "detect_leaks=1 exitcode=66",
           "UBSAN_OPTIONS": "halt_on_error=1 exitcode=66", "PATH": "/usr/bin:/bin"}
    proc = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300, env=env)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "codec_threads: ok" in proc.stdout
    assert "Sanitizer" not in proc.stderr, proc.stderr

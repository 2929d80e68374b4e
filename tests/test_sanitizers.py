"""The host runtime under ThreadSanitizer and AddressSanitizer + UBSan: rings, the key-value store, the RDMA
engine on the software fabric (credit back-pressure, immediates, rendezvous, shutdown with work in flight) and the
TCP endpoint, hammered from several threads (csrc/host/stress/host_stress.cpp). Any report fails the test."""
import subprocess

import pytest

from dlslime_b200 import _build


@pytest.mark.parametrize("sanitizer", ["thread", "address,undefined"])
@pytest.mark.timeout(900)
def test_host_stress_under_sanitizer(sanitizer):
    exe = _build.build_stress(sanitizer)
    env = {"TSAN_OPTIONS": "halt_on_error=0 exitcode=66", "ASAN_OPTIONS": "detect_leaks=0", "UBSAN_OPTIONS": "print_stacktrace=1 halt_on_error=1",
           "PATH": "/usr/bin:/bin"}
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=800, env=env)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-6000:]
    assert "ALL OK" in r.stdout
    assert "WARNING: ThreadSanitizer" not in r.stderr and "ERROR: AddressSanitizer" not in r.stderr and "runtime error" not in r.stderr

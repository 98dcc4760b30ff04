"""The C++ host runtime (cache manager, scheduler) under AddressSanitizer and
UndefinedBehaviorSanitizer: the CPU tests of both run again, in a child process, against a build
made with ``AIEN_B200_HOST_SANITIZE=1``; a memory error or undefined behaviour aborts that process."""
import os
import subprocess
import sys

import pytest

from aien_sovereign_core_mv_b200.csrc import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cache_manager_and_scheduler_under_sanitizers():
    preload = build.sanitizer_preload()
    if preload is None:
        pytest.skip("no C++ compiler here ships libasan.so")
    env = dict(os.environ, AIEN_B200_HOST_SANITIZE="1", LD_PRELOAD=preload,
               ASAN_OPTIONS="detect_leaks=0:abort_on_error=1", UBSAN_OPTIONS="halt_on_error=1:print_stacktrace=1")
    proc = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider",
                           os.path.join(ROOT, "tests", "test_cache_manager.py"), os.path.join(ROOT, "tests", "test_scheduler.py")],
                          cwd=ROOT, env=env, capture_output=True, text=True, timeout=900)
    tail = (proc.stdout + proc.stderr)[-3000:]
    assert proc.returncode == 0, tail
    assert "passed" in proc.stdout and "AddressSanitizer" not in tail and "runtime error" not in tail, tail

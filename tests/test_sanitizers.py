"""Builds the C++ test binary under ThreadSanitizer and AddressSanitizer and runs the CPU suites.

Takes several minutes, so it only runs when TPB_RUN_SANITIZERS=1 (the reference runs the same two
configurations as CI jobs, .circleci/config.yml:281-294 and cmake/Sanitize.cmake).
"""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.skipif(os.environ.get("TPB_RUN_SANITIZERS") != "1",
                                reason="set TPB_RUN_SANITIZERS=1 to build and run the sanitizer configurations")


@pytest.mark.parametrize("kind,env,needle", [
    # die_after_fork=0: some tests fork peer processes after earlier tests have started the timer thread.
    ("thread", {"TSAN_OPTIONS": "halt_on_error=0:die_after_fork=0"}, "WARNING: ThreadSanitizer"),
    ("address", {"ASAN_OPTIONS": "protect_shadow_gap=0"}, "ERROR: AddressSanitizer"),
])
def test_cpu_suites_are_clean_under_sanitizer(kind, env, needle):
    build = f"build-{'tsan' if kind == 'thread' else 'asan'}"
    subprocess.run(["make", "-j", f"SANITIZE={kind}", f"BUILD={build}", f"{build}/bin/tpb_test"],
                   cwd=ROOT, check=True, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, timeout=1800)
    run = subprocess.run([os.path.join(ROOT, build, "bin", "tpb_test")], cwd=ROOT, env={**os.environ, **env},
                         stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=1800)
    assert run.returncode == 0, run.stdout[-4000:]
    assert needle not in run.stdout, run.stdout[-4000:]
    assert "LeakSanitizer" not in run.stdout, run.stdout[-4000:]

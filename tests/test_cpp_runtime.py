"""Runs the native C++ runtime test program (csrc/test/runtime_test.cpp): device, queues,
notifiers, allocators, guard and tensor construction exercised without Python bindings.
The counterpart of the reference's gtest suite (torch_mlu/csrc/test/aten/*.cpp)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BINARY = os.path.join(ROOT, "catch_b200", "lib", "b200_runtime_test")


def _run(env_extra):
    if not os.path.exists(BINARY):
        sys.path.insert(0, ROOT)
        from catch_b200 import _build
        _build.build()
    env = dict(os.environ, **env_extra)
    return subprocess.run([BINARY], env=env, capture_output=True, text=True, timeout=300)


def test_cpp_runtime_suite_on_host_simulation():
    r = _run({"CATCH_B200_BACKEND": "hostsim", "CATCH_B200_HOSTSIM_DEVICES": "2"})
    assert r.returncode == 0 and "ALL PASSED" in r.stdout, r.stdout + r.stderr


@pytest.mark.gpu
def test_cpp_runtime_suite_on_the_gpu():
    r = _run({"CATCH_B200_BACKEND": "cuda"})
    assert r.returncode == 0 and "ALL PASSED" in r.stdout, r.stdout + r.stderr

"""The reference's OWN test programs, compiled unmodified against this repository's
drop-in headers (include/w4/) and, for the GPU suite, linked with libw4b200
(`make -C oracle dropin dropin_gpu`, where the reference tree is present; the
binaries travel under oracle/_ref/). Skipped where they were not built."""
import os
import re
import subprocess

import pytest

REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


def run(name):
    path = os.path.join(REF, name)
    if not os.path.exists(path):
        pytest.skip(f"{name} not built")
    r = subprocess.run([path], capture_output=True, text=True, timeout=600)
    tail = r.stdout.strip().splitlines()[-1]
    assert r.returncode == 0, r.stdout[-2000:]
    return tail


def test_reference_host_suite_against_dropin_headers():
    # tests/test_oracle.cpp of the reference: 212922 checks
    tail = run("dropin_test_oracle")
    assert re.search(r"212922 checks, 0 failures", tail), tail


@pytest.mark.gpu
def test_reference_gpu_suite_against_dropin_library():
    # tests/test_gpu.cu of the reference: 568 checks (bitwise dequant, oracle 1e-3,
    # cuBLAS cross-check 2e-3, dispatcher memcmp, paged == contiguous, ~150 contract throws)
    tail = run("dropin_test_gpu")
    assert re.search(r"568 checks, 0 failures", tail), tail

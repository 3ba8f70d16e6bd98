"""vkML's own C++ hazard suite on the B200: tests/cpp/test_aliasing.cpp ("on every registered
device": read-after-write and write-after-read between the dispatches of one submission, an
assignment into live storage, a node's storage handed out again mid-span) compiled unmodified by
oracle/Makefile with the B200 adapter in the device slot."""
import os
import re
import subprocess

import pytest

pytestmark = pytest.mark.gpu

BINARY = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                      "test_aliasing_b200")
CPU_ONLY_ASSERTIONS = 34  # what the same binary checks when no device is present


def test_the_reference_hazard_suite_passes_on_the_device():
    if not os.path.exists(BINARY):
        pytest.skip("oracle/_ref/test_aliasing_b200 not built")
    run = subprocess.run([BINARY], capture_output=True, text=True, timeout=300)
    out = run.stdout + run.stderr
    assert run.returncode == 0 and "Status: SUCCESS!" in out, out[-3000:]
    assertions = int(re.search(r"assertions:\s+(\d+)\s+\|\s+(\d+) passed", out).group(2))
    assert assertions > CPU_ONLY_ASSERTIONS, f"the device was not exercised ({assertions} assertions)"

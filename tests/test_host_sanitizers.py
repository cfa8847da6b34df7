"""Race / memory checks of the C++ host runtime: the multi-thread soak program is compiled with
ThreadSanitizer and with AddressSanitizer + UBSan and must run clean (the device-side sanitizer is
not available on the GPU pool, so the host runtime is where sanitizers run)."""
import os
import shutil
import subprocess
import tempfile

import pytest

HOST = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc", "host")


@pytest.mark.parametrize("san", ["thread", "address,undefined"])
def test_host_runtime_soak_under_sanitizer(san):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    with tempfile.TemporaryDirectory() as d:
        exe = os.path.join(d, "soak")
        cmd = ["g++", "-std=c++17", "-O1", "-g", f"-fsanitize={san}", "-pthread",
               os.path.join(HOST, "tests", "soak_host_runtime.cpp"), os.path.join(HOST, "block_manager.cpp"),
               os.path.join(HOST, "worker.cpp"), "-o", exe]
        b = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
        if b.returncode != 0 and "sanitizer" in (b.stderr or "").lower() and "cannot find" in b.stderr:
            pytest.skip("sanitizer runtime not installed")
        assert b.returncode == 0, b.stderr[-2000:]
        r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
        out = r.stdout + r.stderr
        assert r.returncode == 0 and "OK" in r.stdout, out[-3000:]
        assert "WARNING: ThreadSanitizer" not in out and "ERROR: AddressSanitizer" not in out and "runtime error" not in out, out[-3000:]

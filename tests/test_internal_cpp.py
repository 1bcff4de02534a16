"""Builds and runs the torch-free C++ unit tests (tests/internal)."""
import os
import subprocess


def test_native_cpp_units(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = str(tmp_path / "test_native")
    srcs = ["tests/internal/test_native.cpp", "csrc/engine/progress.cpp", "csrc/net/tcp_mesh.cpp", "csrc/pg/cpu_algos.cpp"]
    subprocess.check_call(["g++", "-std=c++17", "-O1", "-pthread", "-o", exe] + [os.path.join(root, s) for s in srcs])
    out = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "0 failed" in out.stdout

"""Host code under ThreadSanitizer and AddressSanitizer / UBSan.

compute-sanitizer cannot be used on the GPU pool these kernels are developed on, so the race and
memory checks that can run anywhere run here: the torch-free host sources (progress engine, TCP mesh,
host collectives, distributed memory, coherence protocol, scheduler, cluster manager) are compiled with
``-fsanitize=thread`` and again with ``-fsanitize=address,undefined`` and driven from several threads by
the two test programs under ``tests/internal``.  A sanitizer report fails the test.
"""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")

PROGRAMS = {
    "native": (["tests/internal/test_native.cpp", "csrc/engine/progress.cpp", "csrc/net/tcp_mesh.cpp", "csrc/pg/cpu_algos.cpp"], False),
    # dmem_manager.cpp calls the CUDA runtime for device regions; the tests only register host memory, but the
    # program still has to link against libcudart
    "runtime": (["tests/internal/test_runtime_native.cpp", "csrc/cluster/cluster_manager.cpp", "csrc/cluster/scheduler.cpp",
                 "csrc/cluster/agent.cpp", "csrc/coherence/coherence.cpp", "csrc/dmem/dmem_manager.cpp"], True),
}
SANITIZERS = {
    "thread": ["-fsanitize=thread"],
    "address": ["-fsanitize=address,undefined", "-fno-omit-frame-pointer"],
}


def _sanitizer_works(flags, tmp_path) -> bool:
    src = tmp_path / "probe.cpp"
    src.write_text("int main() { return 0; }\n")
    exe = tmp_path / "probe"
    try:
        subprocess.check_call(["g++"] + flags + [str(src), "-o", str(exe)], stderr=subprocess.DEVNULL)
        return subprocess.run([str(exe)], capture_output=True, timeout=30).returncode == 0
    except Exception:  # noqa: BLE001
        return False


@pytest.mark.parametrize("program", sorted(PROGRAMS))
@pytest.mark.parametrize("sanitizer", sorted(SANITIZERS))
def test_host_code_under_sanitizer(program, sanitizer, tmp_path):
    if shutil.which("g++") is None:
        pytest.skip("no g++")
    flags = SANITIZERS[sanitizer]
    if not _sanitizer_works(flags, tmp_path):
        pytest.skip(f"-fsanitize={sanitizer} is not usable with this toolchain")
    srcs, needs_cuda = PROGRAMS[program]
    if needs_cuda and not os.path.exists(os.path.join(CUDA, "include", "cuda_runtime_api.h")):
        pytest.skip("no CUDA headers")
    exe = str(tmp_path / f"{program}_{sanitizer}")
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-pthread"] + flags + ["-o", exe] + [os.path.join(ROOT, s) for s in srcs]
    env = dict(os.environ)
    if needs_cuda:
        cmd += ["-I", os.path.join(CUDA, "include"), "-L", os.path.join(CUDA, "lib64"), "-lcudart"]
        env["LD_LIBRARY_PATH"] = os.path.join(CUDA, "lib64") + os.pathsep + env.get("LD_LIBRARY_PATH", "")
    subprocess.check_call(cmd)
    env["TSAN_OPTIONS"] = "halt_on_error=0 exitcode=66"
    env["ASAN_OPTIONS"] = "detect_leaks=0 protect_shadow_gap=0 exitcode=66"
    env["UBSAN_OPTIONS"] = "print_stacktrace=1 halt_on_error=0"
    out = subprocess.run([exe], capture_output=True, text=True, timeout=600, env=env)
    report = out.stdout[-4000:] + out.stderr[-6000:]
    assert "WARNING: ThreadSanitizer" not in out.stderr, report
    assert "ERROR: AddressSanitizer" not in out.stderr, report
    assert "runtime error:" not in out.stderr, report
    assert out.returncode == 0, report
    assert "0 failed" in out.stdout, report

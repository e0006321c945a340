"""The C11 host layer under AddressSanitizer and UndefinedBehaviorSanitizer, on a machine
without a GPU (the reference's sanitizer lanes also build with CUDA disabled, Makefile:752-849;
compute-sanitizer is not available on the GPU pool). clori_b200/csrc/host/*.c is compiled
with -fsanitize=address,undefined -fno-sanitize-recover together with a device-less stand-in
for the shim and a driver that walks the block pool, the geometry helpers and the refusal
ladders; any report aborts the run."""
import glob
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_host_layer_is_clean_under_asan_and_ubsan(tmp_path):
    if not shutil.which("gcc"):
        pytest.skip("gcc is required")
    exe = str(tmp_path / "host_driver")
    sources = sorted(glob.glob(os.path.join(ROOT, "clori_b200", "csrc", "host", "*.c")))
    extra = [os.path.join(ROOT, "tests", "sanitize", name) for name in ("shim_absent.c", "host_driver.c")]
    cmd = ["gcc", "-std=c11", "-O1", "-g", "-D_GNU_SOURCE", "-fsanitize=address,undefined", "-fno-sanitize-recover=all",
           "-fno-omit-frame-pointer", "-Wall", "-Wextra", "-Wno-unused-parameter", "-Werror", "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(ROOT, "clori_b200", "csrc", "host")] + sources + extra + ["-lm", "-o", exe]
    built = subprocess.run(cmd, capture_output=True, text=True)
    assert built.returncode == 0, built.stderr[-3000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=1", UBSAN_OPTIONS="halt_on_error=1")
    ran = subprocess.run([exe], capture_output=True, text=True, env=env, timeout=300)
    assert ran.returncode == 0, (ran.stdout[-2000:], ran.stderr[-4000:])
    assert "host layer clean under the sanitizers" in ran.stdout

"""The C ABI from a C program: no Python, no torch in the calling process."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "sageattention-autotune_b200", "sageattention")


@pytest.mark.gpu
def test_c_program_runs_the_whole_path(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    assert os.path.exists(nvcc), "nvcc is needed to build the C caller"
    assert os.path.exists(os.path.join(LIBDIR, "libsage_b200.so")), "build the library first"
    exe = str(tmp_path / "demo")
    subprocess.run([nvcc, "-x", "c", os.path.join(ROOT, "tests", "c_abi", "demo.c"), "-I", os.path.join(ROOT, "include"),
                    "-L", LIBDIR, "-lsage_b200", "-lcudart", "-lm", "-o", exe], check=True, capture_output=True, text=True)
    env = dict(os.environ, LD_LIBRARY_PATH=LIBDIR + os.pathsep + os.environ.get("LD_LIBRARY_PATH", ""))
    r = subprocess.run([exe], env=env, capture_output=True, text=True, timeout=300)
    print(r.stdout, r.stderr)
    assert r.returncode == 0 and "PASS" in r.stdout, (r.returncode, r.stdout, r.stderr)

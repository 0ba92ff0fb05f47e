"""The C++ protocol adapters (include/slime_pseudopod.hpp) over the C ABI, exercised by a small C++ program."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build_adapter_test():
    from slime_b200 import build
    lib = build.build()
    exe = os.path.join(ROOT, "tests", "cpp", "test_adapters")
    src = os.path.join(ROOT, "tests", "cpp", "test_adapters.cpp")
    hdr = os.path.join(ROOT, "include", "slime_pseudopod.hpp")
    if (not os.path.exists(exe) or os.path.getmtime(exe) < max(os.path.getmtime(src), os.path.getmtime(hdr), os.path.getmtime(lib))):
        env = dict(os.environ)
        env.pop("CC", None); env.pop("CXX", None)
        subprocess.run([os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc"), "-std=c++17", "-Wno-deprecated-gpu-targets",
                        "-I" + os.path.join(ROOT, "include"), "-o", exe, src, "-L" + os.path.dirname(lib), "-lslime_ca",
                        "-Xlinker", "-rpath", "-Xlinker", os.path.dirname(lib)], check=True, env=env)
    return exe


def test_protocol_adapters():
    exe = build_adapter_test()
    out = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert out.stdout.strip().endswith("ok")

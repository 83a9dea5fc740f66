"""The drop-in boundary, compiled: (1) the adapter of integration/xnor_b200_adapter.cpp against the reference's own
headers (Darknet::Layer, NetworkState, get_cuda_stream, CHECK_CUDA ... as a -DDARKNET_GPU build sees them), wherever the
reference tree is mounted; (2) a plain-C translation unit that includes include/xnor_b200.h, links libxnor_b200.so and calls
the host-only entry points.  No GPU is needed for either."""
import os
import shutil
import subprocess

import pytest

from darknet_b200 import capi
from oracle.binding import reference_dir

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def cuda_include():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return os.path.join(os.path.dirname(os.path.dirname(os.path.realpath(nvcc))), "include")


def test_adapter_compiles_against_the_reference_headers():
    ref = reference_dir()
    if not os.path.isdir(os.path.join(ref, "src-lib")):
        pytest.skip("reference tree not mounted")
    gen = os.path.join(ROOT, "oracle", "_ref", "gen")
    if not os.path.exists(os.path.join(gen, "darknet_version.h")):
        pytest.skip("oracle/_ref not built (make -C oracle ref)")
    cmd = ["g++", "-std=c++17", "-fsyntax-only", "-Wall", "-Werror=return-type", "-DDARKNET_GPU", "-DDARKNET_GPU_CUDA",
           "-I", os.path.join(ROOT, "oracle", "ref_stub"), "-I", gen, "-I", os.path.join(ref, "src-lib"), "-I", os.path.join(ref, "src-other"),
           "-I", os.path.join(ROOT, "include"), "-I", cuda_include(), os.path.join(ROOT, "integration", "xnor_b200_adapter.cpp")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    errors = [ln for ln in r.stderr.splitlines() if "error" in ln]
    assert r.returncode == 0, "\n".join(errors[:20])


def test_header_is_plain_c_and_links(tmp_path):
    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    assert os.path.exists(capi.LIB_PATH)
    exe = str(tmp_path / "c_abi_smoke")
    lib_dir = os.path.dirname(capi.LIB_PATH)
    subprocess.check_call(["gcc", "-std=c99", "-pedantic", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "integration", "c_abi_smoke.c"), "-o", exe, "-L", lib_dir, "-lxnor_b200",
                           "-Wl,-rpath," + lib_dir])
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, f"exit {r.returncode}: {r.stdout} {r.stderr}"
    assert r.stdout.strip() == "ok|scratch buffer too small"

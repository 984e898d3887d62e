"""CPU test of the header-only C++ shim (include/psb_views.hpp): a caller written against the REFERENCE's headers compiles
and links unchanged with the shim in place of the reference's implementation, and - there being no GPU here - its calls come
back as exceptions carrying the library's "no device" status (never a silent fallback).  Needs the reference checkout for its
headers; skipped where that is absent."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("PSB_REFERENCE_DIR", "/root/reference")


@pytest.mark.skipif(not os.path.exists(os.path.join(REF, "src", "search", "ivfrespq", "ivfrespq_search.cuh")),
                    reason="the reference's headers are not on this machine")
def test_reference_caller_builds_against_the_shim(tmp_path):
    from paraselect_b200 import api, build
    build.ensure_built()
    exe = str(tmp_path / "shim_caller")
    cmd = ["g++", "-std=c++20", "-DUSE_NVTX=0", "-I", os.path.join(REF, "src"), "-I", REF, "-I", "/usr/local/cuda/include",
           "-I", os.path.join(ROOT, "include"), os.path.join(ROOT, "tests", "cpp", "shim_caller.cpp"), "-o", exe,
           "-L", os.path.dirname(api.LIB_PATH), "-lpsb", "-Wl,-rpath," + os.path.dirname(api.LIB_PATH),
           "-L", "/usr/local/cuda/lib64", "-lcudart"]   # the sign-codec index keeps device memory of its own, as the reference's does
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    run = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    out = run.stdout
    if api.device_count() == 0:
        assert "RUNTIME_ERROR" in out and "no CUDA device" in out   # PSB_NO_DEVICE -> std::runtime_error, no fallback
        assert "FLAT_RUNTIME_ERROR" in out
        assert "SIGN_RUNTIME_ERROR" in out and "SIGN_BAD_REQUEST_REFUSED" in out
    else:
        assert "SEARCH_OK 1" in out and "BAD_REQUEST_REFUSED" in out and "FLAT_OK" in out
        assert "SIGN_OK" in out and "SIGN_BAD_REQUEST_REFUSED" in out

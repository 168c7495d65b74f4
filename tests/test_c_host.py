"""The C ABI from a C host: tests/c_abi/predict_from_c.c is compiled with gcc against include/zant_b200.h,
linked with the in-tree library and run.  Without a GPU it checks the library's refusal to compute; on a
GPU it checks a convolution from the reference's unit tests, a three-node plan and its graph replay."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "c_abi", "predict_from_c.c")
LIB_DIR = os.path.join(ROOT, "z-ant_b200")


def _build(tmp_path, zb):
    zb.lib()                                                    # make sure the library is built
    exe = os.path.join(tmp_path, "predict_from_c")
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    subprocess.check_call([cc, "-std=c11", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"), SRC, "-o", exe,
                           "-L", LIB_DIR, "-lzant_b200", "-Wl,-rpath," + LIB_DIR])
    return exe


def _run(exe):
    return subprocess.run([exe], capture_output=True, text=True, timeout=120)


def test_c_host_without_gpu_gets_the_refusal(tmp_path, zb):
    import torch
    if torch.cuda.is_available():
        pytest.skip("this machine has a GPU: covered by the gpu test")
    r = _run(_build(str(tmp_path), zb))
    assert r.returncode == 0, r.stderr
    assert "CudaUnavailable" in r.stdout


@pytest.mark.gpu
def test_c_host_runs_operator_plan_and_graph(tmp_path, zb):
    r = _run(_build(str(tmp_path), zb))
    assert r.returncode == 0, r.stderr
    assert "agree with the reference's numbers" in r.stdout

"""Builds and runs the C++ host mirror of the reference's Kernel trait against the device."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB_DIR = os.path.join(ROOT, "rust-model-inference_b200", "lib")


def _build(tmp_path):
    exe = str(tmp_path / "test_kernel_trait")
    subprocess.check_call(["g++", "-std=c++17", "-O1", os.path.join(ROOT, "tests", "cpp", "test_kernel_trait.cpp"), "-o", exe,
                           "-L" + LIB_DIR, "-lrmi_cuda", "-Wl,-rpath," + LIB_DIR])
    return exe


def test_cpp_host_mirror_compiles_and_links(rmi, tmp_path):
    rmi.lib()
    assert os.path.exists(_build(tmp_path))


@pytest.mark.gpu
def test_cpp_host_mirror_runs_the_reference_unit_tests(rmi, tmp_path):
    rmi.lib()
    # a two-layer model file for the per-step session interface
    from tests.synth_model import tiny_cfg
    cfg = tiny_cfg()
    path = str(tmp_path / "tiny.gguf")
    rmi.synth.write_qwen3_gguf(path, cfg, rmi.synth.qwen3_tensors(cfg, 3))
    out = subprocess.run([_build(tmp_path), path], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "all kernel-trait checks passed" in out.stdout

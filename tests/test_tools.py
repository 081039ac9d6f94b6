"""Command-line tools driven through mock environment variables, as the reference tests its
scripts (gpu-mojo/scripts/test_gpu_specs.py, test_macos_env.py): subprocess + MOCK_* variables."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def run(mod, *args, **env):
    e = dict(os.environ, PYTHONPATH=str(ROOT), CUDA_VISIBLE_DEVICES="")
    e.update(env)
    return subprocess.run([sys.executable, "-m", mod, *args], capture_output=True, text=True, env=e, cwd=ROOT)


def test_gpu_specs_platform_and_compute_cap_mocks():
    m = "zero_to_hero_b200.utils.gpu_specs"
    r = run(m, "--platform", MOCK_GPU_PLATFORM="nvidia", MOCK_COMPUTE_CAP="10.0")
    assert r.returncode == 0 and r.stdout.strip() == "nvidia"
    r = run(m, "--compute-cap", MOCK_GPU_PLATFORM="nvidia", MOCK_COMPUTE_CAP="10.0")
    assert r.stdout.strip() == "10.0"
    r = run(m, "--compute-cap", MOCK_GPU_PLATFORM="apple")
    assert r.returncode == 0 and r.stdout.strip() == ""
    assert run(m, "--platform", MOCK_GPU_PLATFORM="apple").stdout.strip() == "apple"
    assert run(m, "--check-platform", "nvidia", MOCK_GPU_PLATFORM="nvidia").returncode == 0
    assert run(m, "--check-platform", "amd", MOCK_GPU_PLATFORM="nvidia").returncode == 1
    assert run(m, "--check-platform", "apple_silicon", MOCK_GPU_PLATFORM="apple").returncode == 0


def test_gpu_specs_reports_blackwell():
    m = "zero_to_hero_b200.utils.gpu_specs"
    r = run(m, MOCK_GPU_PLATFORM="nvidia", MOCK_COMPUTE_CAP="10.0", MOCK_GPU_NAME="NVIDIA B200")
    assert "Blackwell" in r.stdout and "Tensor Memory Kb Per Sm: 256" in r.stdout and "228" in r.stdout
    r = run(m, "--summary", MOCK_GPU_PLATFORM="nvidia", MOCK_COMPUTE_CAP="9.0")
    assert "Hopper" in r.stdout and "sm_90" in r.stdout
    r = run(m, "--occupancy", "--threads", "192", "--regs", "168", "--smem", "115712",
            MOCK_GPU_PLATFORM="nvidia", MOCK_COMPUTE_CAP="10.0")
    assert "2 blocks/SM" in r.stdout  # the flash-attention forward launch configuration


def test_occupancy_arithmetic():
    from zero_to_hero_b200.utils.gpu_specs import occupancy
    o = occupancy("10.0", 192, 121, 197888)  # the GEMM kernel: shared memory allows one CTA
    assert o["blocks_per_sm"] == 1 and o["limiter"] == "shared_memory"
    o = occupancy("10.0", 256, 32, 0)
    assert o["blocks_per_sm"] == 8 and o["limiter"] == "threads" and o["occupancy"] == 1.0


def test_check_env_with_mocks():
    m = "zero_to_hero_b200.utils.check_env"
    good = dict(MOCK_NVCC_VERSION="12.9", MOCK_COMPUTE_CAP="10.0", MOCK_DRIVER_VERSION="580.159",
                MOCK_TORCH_CUDA="12.8", MOCK_LIBS_BUILT="1")
    r = run(m, "--json", **good)
    assert r.returncode == 0 and all(c["ok"] for c in json.loads(r.stdout))
    r = run(m, **{**good, "MOCK_NVCC_VERSION": "12.4"})
    assert r.returncode == 1 and "[FAIL] nvcc" in r.stdout
    r = run(m, **{**good, "MOCK_COMPUTE_CAP": "9.0", "MOCK_LIBS_BUILT": "0"})
    assert r.returncode == 0 and r.stdout.count("[warn]") == 2  # not required: building needs no GPU


def test_traced_variant_of_a_kernel_builds_and_exports_its_reader():
    """`utils/kernel_trace.py` compiles a kernel's sources with -DZ2H_KERNEL_TRACE; the marks compile to
    nothing in the product build, so only this keeps them compiling. CPU: nvcc cross-compiles."""
    import ctypes
    import shutil
    if shutil.which("nvcc") is None and not __import__("pathlib").Path("/usr/local/cuda/bin/nvcc").exists():
        pytest.skip("no nvcc")
    from zero_to_hero_b200.utils import kernel_trace
    lib = kernel_trace.build_trace_lib("flash_bwd")
    assert isinstance(lib, ctypes.CDLL)
    assert hasattr(lib, "z2h_flash_bwd_trace_read") and hasattr(lib, "z2h_flash_bwd")
    assert set(kernel_trace.EPI) >= {"bias", "gelu_save_grad", "mul_aux"}

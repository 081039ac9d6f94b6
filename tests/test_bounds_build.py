"""The self-checking debug build (-DZ2H_BOUNDS, csrc/common/checked.cuh): it compiles for sm_100a
without a GPU, and on a GPU the tail-shape kernel tests pass against it with a clean status word
(a violation would show as status 8 | site << 8)."""
import ctypes
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def test_bounds_variant_builds_and_exports_the_c_abi():
    from zero_to_hero_b200.build import build_all
    from zero_to_hero_b200.ops import _lib

    lib = build_all(bounds=True)["cuda"]
    assert lib.name == "libz2h_bounds.so" and lib.exists()
    product = build_all()["cuda"]
    assert product.name == "libz2h.so" and product.exists()   # the product library is untouched
    handle = ctypes.CDLL(str(lib))
    for sym in ("z2h_gemm_bf16", "z2h_flash_fwd", "z2h_embed_fwd", "z2h_reduce_bucket"):
        assert hasattr(handle, sym)
    assert "site 3" in _lib.describe_status(8 | (3 << 8)) and "GEMM" in _lib.describe_status(8 | (3 << 8))


@pytest.mark.gpu
def test_tail_shapes_pass_under_the_checked_build():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from zero_to_hero_b200.build import build_all
    build_all(bounds=True)
    env = dict(os.environ, Z2H_NATIVE_LIB="bounds")
    r = subprocess.run([sys.executable, "-m", "pytest", str(ROOT / "tests" / "test_kernels_gpu.py"), "-q", "-x",
                        "-k", "gemm or flash_attention_fwd_bwd or embedding"],
                       env=env, capture_output=True, text=True, timeout=900, cwd=str(ROOT))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert " passed" in r.stdout

"""Environment check for building and running this framework on a Linux + NVIDIA box.

    python -m zero_to_hero_b200.utils.check_env [--json]

The reference ships a macOS / Xcode / Metal validator for its Mojo toolchain
(gpu-mojo/scripts/check_macos_env.py) that can be driven by MOCK_* environment variables; this is
the counterpart for this framework's toolchain: nvcc and its version, compute capability
(sm_100 expected), driver, PyTorch + CUDA, the built native libraries. Mock variables for tests:
MOCK_NVCC_VERSION, MOCK_COMPUTE_CAP, MOCK_DRIVER_VERSION, MOCK_TORCH_CUDA, MOCK_LIBS_BUILT.
Exit code 0 when every required check passes, 1 otherwise. Read-only.
"""
from __future__ import annotations

import argparse
import json
import os
import re
import shutil
import subprocess
import sys
from pathlib import Path


def _run(cmd: list[str]) -> str:
    try:
        return subprocess.run(cmd, capture_output=True, text=True, timeout=20).stdout
    except Exception:
        return ""


def nvcc_version() -> str | None:
    if "MOCK_NVCC_VERSION" in os.environ:
        return os.environ["MOCK_NVCC_VERSION"] or None
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    m = re.search(r"release (\d+\.\d+)", _run([exe, "--version"]))
    return m.group(1) if m else None


def compute_cap() -> str | None:
    if "MOCK_COMPUTE_CAP" in os.environ:
        return os.environ["MOCK_COMPUTE_CAP"] or None
    out = _run(["nvidia-smi", "--query-gpu=compute_cap", "--format=csv,noheader"]).strip()
    return out.splitlines()[0].strip() if out else None


def driver_version() -> str | None:
    if "MOCK_DRIVER_VERSION" in os.environ:
        return os.environ["MOCK_DRIVER_VERSION"] or None
    out = _run(["nvidia-smi", "--query-gpu=driver_version", "--format=csv,noheader"]).strip()
    return out.splitlines()[0].strip() if out else None


def torch_cuda() -> str | None:
    if "MOCK_TORCH_CUDA" in os.environ:
        return os.environ["MOCK_TORCH_CUDA"] or None
    try:
        import torch
        return torch.version.cuda
    except Exception:
        return None


def libs_built() -> bool:
    if "MOCK_LIBS_BUILT" in os.environ:
        return os.environ["MOCK_LIBS_BUILT"] == "1"
    return (Path(__file__).resolve().parent.parent / "lib" / "libz2h.so").exists()


def _ver(s: str) -> tuple[int, ...]:
    return tuple(int(x) for x in re.findall(r"\d+", s)[:2])


def collect() -> list[dict]:
    checks = []

    def add(name, value, ok, required, hint=""):
        checks.append({"check": name, "value": value, "ok": bool(ok), "required": required, "hint": hint})

    v = nvcc_version()
    add("nvcc", v, v is not None and _ver(v) >= (12, 8), True, "CUDA 12.8+ is needed to compile for sm_100a")
    c = compute_cap()
    add("compute capability", c, c is not None and c.startswith("10."), False,
        "the kernels are written for sm_100a (B200); building works without a GPU, running does not")
    d = driver_version()
    add("driver", d, d is not None and _ver(d) >= (570, 0), False, "a 570+ driver is needed for sm_100")
    t = torch_cuda()
    add("torch CUDA", t, t is not None, True, "install a CUDA build of PyTorch")
    add("native libraries", "built" if libs_built() else "missing", libs_built(), False,
        "run `python -m zero_to_hero_b200.build`")
    return checks


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args(argv)
    checks = collect()
    if a.json:
        print(json.dumps(checks, indent=2))
    else:
        for c in checks:
            mark = "ok " if c["ok"] else ("FAIL" if c["required"] else "warn")
            print(f"[{mark}] {c['check']}: {c['value']}" + ("" if c["ok"] else f"  -> {c['hint']}"))
    return 0 if all(c["ok"] or not c["required"] for c in checks) else 1


if __name__ == "__main__":
    sys.exit(main())

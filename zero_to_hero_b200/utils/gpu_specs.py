"""GPU specification report with a Blackwell row, occupancy arithmetic and mockable detection.

    python -m zero_to_hero_b200.utils.gpu_specs                 # full report
    python -m zero_to_hero_b200.utils.gpu_specs --platform      # nvidia | amd | apple | unknown
    python -m zero_to_hero_b200.utils.gpu_specs --compute-cap   # e.g. 10.0 (empty if not NVIDIA)
    python -m zero_to_hero_b200.utils.gpu_specs --check-platform nvidia   # exit code 0 / 1
    python -m zero_to_hero_b200.utils.gpu_specs --summary
    python -m zero_to_hero_b200.utils.gpu_specs --occupancy --threads 192 --regs 168 --smem 115712

Same command-line contract as the reference's gpu-mojo/scripts/gpu_specs.py (whose architecture
table stops at Hopper, :235-250): detection tries NVML, then torch, then `nvidia-smi`, and the
environment variables MOCK_GPU_PLATFORM / MOCK_COMPUTE_CAP replace detection so the tool can be
tested on machines without that hardware. Everything here only *reads* GPU state.
"""
from __future__ import annotations

import argparse
import os
import platform
import shutil
import subprocess
import sys
from dataclasses import dataclass, field

ARCH_BY_CAP = {
    "5.0": "Maxwell", "5.2": "Maxwell", "5.3": "Maxwell", "6.0": "Pascal", "6.1": "Pascal", "6.2": "Pascal",
    "7.0": "Volta", "7.2": "Volta", "7.5": "Turing", "8.0": "Ampere", "8.6": "Ampere", "8.7": "Ampere",
    "8.9": "Ada", "9.0": "Hopper", "10.0": "Blackwell", "10.1": "Blackwell", "10.3": "Blackwell",
    "12.0": "Blackwell",
}
# per-SM limits by compute-capability major/minor: (shared KB, max threads, max blocks, registers)
SM_LIMITS = {
    "5": (64, 2048, 32, 65536), "6": (96, 2048, 32, 65536), "7.0": (96, 2048, 32, 65536),
    "7.5": (64, 1024, 16, 65536), "8.0": (164, 2048, 32, 65536), "8.6": (100, 1536, 16, 65536),
    "8.7": (164, 1536, 16, 65536), "8.9": (100, 1536, 24, 65536), "9.0": (228, 2048, 32, 65536),
    "10.0": (228, 2048, 32, 65536), "10.3": (228, 2048, 32, 65536), "12.0": (100, 1536, 24, 65536),
}
# what a datacenter Blackwell SM adds on top of the generic limits
BLACKWELL_EXTRAS = {"tensor_memory_kb_per_sm": 256, "tensor_memory_columns": 512,
                    "max_shared_kb_per_block": 227, "max_cluster_size_portable": 8,
                    "tensor_core_generation": 5}


@dataclass
class GPUSpecs:
    vendor: str
    device_name: str
    architecture: str
    compute_capability: str = ""
    compute_units: int | None = None
    registers_per_unit: int | None = None
    shared_memory_per_unit_kb: int | None = None
    max_threads_per_unit: int | None = None
    max_blocks_per_unit: int | None = None
    total_memory_gb: float | None = None
    additional_info: dict = field(default_factory=dict)


def sm_limits(cap: str) -> tuple[int, int, int, int]:
    return SM_LIMITS.get(cap) or SM_LIMITS.get(cap.split(".")[0]) or SM_LIMITS["9.0"]


def detect_platform() -> str:
    mock = os.environ.get("MOCK_GPU_PLATFORM")
    if mock:
        return {"apple": "apple_silicon", "applesilicon": "apple_silicon"}.get(mock.lower(), mock.lower())
    if platform.system() == "Darwin" and platform.machine() == "arm64":
        return "apple_silicon"
    try:
        import torch
        if torch.cuda.is_available():
            return "amd" if getattr(torch.version, "hip", None) else "nvidia"
    except Exception:
        pass
    if shutil.which("nvidia-smi"):
        try:
            if subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=10).stdout.strip():
                return "nvidia"
        except Exception:
            pass
    if shutil.which("rocm-smi"):
        return "amd"
    return "unknown"


def _specs_from_cap(name: str, cap: str, sms=None, mem_gb=None, regs=None, threads=None) -> GPUSpecs:
    smem, max_threads, max_blocks, max_regs = sm_limits(cap)
    info = {"unit_type": "Streaming Multiprocessor (SM)"}
    if cap.startswith("10."):
        info.update(BLACKWELL_EXTRAS)
    return GPUSpecs("NVIDIA", name, ARCH_BY_CAP.get(cap, f"Compute {cap}"), cap, sms, regs or max_regs, smem,
                    threads or max_threads, max_blocks, mem_gb, info)


def get_nvidia_specs(device_index: int = 0) -> GPUSpecs:
    mock_cap = os.environ.get("MOCK_COMPUTE_CAP")
    if os.environ.get("MOCK_GPU_PLATFORM"):
        return _specs_from_cap(os.environ.get("MOCK_GPU_NAME", "Mock NVIDIA GPU"), mock_cap or "10.0")
    try:  # NVML first: works without a CUDA context
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        name = pynvml.nvmlDeviceGetName(h)
        name = name.decode() if isinstance(name, bytes) else name
        major, minor = pynvml.nvmlDeviceGetCudaComputeCapability(h)
        mem = pynvml.nvmlDeviceGetMemoryInfo(h).total / 1e9
        sms = None
        try:
            import torch
            if torch.cuda.is_available():
                sms = torch.cuda.get_device_properties(device_index).multi_processor_count
        except Exception:
            pass
        return _specs_from_cap(name, f"{major}.{minor}", sms, mem)
    except Exception:
        pass
    try:
        import torch
        if torch.cuda.is_available():
            d = torch.cuda.get_device_properties(device_index)
            return _specs_from_cap(d.name, f"{d.major}.{d.minor}", d.multi_processor_count, d.total_memory / 1e9,
                                   getattr(d, "regs_per_multiprocessor", None),
                                   getattr(d, "max_threads_per_multi_processor", None))
    except Exception:
        pass
    out = subprocess.run(["nvidia-smi", "--query-gpu=name,compute_cap,memory.total", "--format=csv,noheader,nounits",
                          "-i", str(device_index)], capture_output=True, text=True, timeout=10).stdout.strip()
    if not out:
        raise RuntimeError("no NVIDIA GPU found by NVML, torch or nvidia-smi")
    name, cap, mem = [s.strip() for s in out.splitlines()[0].split(",")]
    return _specs_from_cap(name, cap, None, float(mem) / 1024)


def get_other_specs(kind: str) -> GPUSpecs:
    if kind == "amd":
        return GPUSpecs("AMD", os.environ.get("MOCK_GPU_NAME", "AMD GPU"), "ROCm", additional_info={
            "unit_type": "Compute Unit (CU)", "note": "this framework has no AMD code path"})
    return GPUSpecs("Apple", os.environ.get("MOCK_GPU_NAME", "Apple Silicon GPU"), "Metal", additional_info={
        "unit_type": "GPU core", "note": "this framework has no Metal code path"})


def occupancy(cap: str, threads_per_block: int, regs_per_thread: int, smem_per_block: int) -> dict:
    """Resident blocks per SM and which resource limits them (register allocation is per warp in
    units of 256 registers; every block also reserves 1 KiB of shared memory)."""
    smem_kb, max_threads, max_blocks, regs = sm_limits(cap)
    warps = (threads_per_block + 31) // 32
    regs_per_warp = ((regs_per_thread * 32 + 255) // 256) * 256
    limits = {
        "threads": max_threads // (warps * 32),
        "registers": regs // (regs_per_warp * warps) if regs_per_thread else max_blocks,
        "shared_memory": (smem_kb * 1024) // (smem_per_block + 1024),
        "blocks": max_blocks,
    }
    blocks = max(0, min(limits.values()))
    limiter = min(limits, key=limits.get)
    return {"blocks_per_sm": blocks, "warps_per_sm": blocks * warps, "limiter": limiter, "limits": limits,
            "occupancy": blocks * warps * 32 / max_threads}


def print_specs(s: GPUSpecs, summary: bool = False) -> None:
    if summary:
        mem = f", {s.total_memory_gb:.0f}GB" if s.total_memory_gb else ""
        cap = f" (sm_{s.compute_capability.replace('.', '')})" if s.compute_capability else ""
        print(f"GPU: {s.device_name}{cap}{mem}")
        print(f"Architecture: {s.architecture}")
        return
    print(f"Vendor: {s.vendor}")
    print(f"Device: {s.device_name}")
    print(f"Architecture: {s.architecture}")
    if s.compute_capability:
        print(f"Compute Capability: {s.compute_capability}")
    unit = s.additional_info.get("unit_type", "unit")
    if s.compute_units:
        print(f"{unit} count: {s.compute_units}")
    for label, v in [("Registers per Unit", s.registers_per_unit), ("Shared Memory per Unit (KB)", s.shared_memory_per_unit_kb),
                     ("Max Threads per Unit", s.max_threads_per_unit), ("Max Blocks per Unit", s.max_blocks_per_unit)]:
        if v:
            print(f"{label}: {v:,}")
    if s.total_memory_gb:
        print(f"Total Memory: {s.total_memory_gb:.1f}GB")
    for k, v in s.additional_info.items():
        if k != "unit_type":
            print(f"{k.replace('_', ' ').title()}: {v}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="GPU specification detection")
    ap.add_argument("--platform", action="store_true")
    ap.add_argument("--compute-cap", action="store_true")
    ap.add_argument("--check-platform", metavar="NAME")
    ap.add_argument("--summary", action="store_true")
    ap.add_argument("--occupancy", action="store_true")
    ap.add_argument("--threads", type=int, default=256)
    ap.add_argument("--regs", type=int, default=64)
    ap.add_argument("--smem", type=int, default=0)
    a = ap.parse_args(argv)
    try:
        kind = detect_platform()
        name = "apple" if kind == "apple_silicon" else kind
        if a.platform:
            print(name)
            return 0
        if a.compute_cap:
            cap = ""
            if kind == "nvidia":
                try:
                    cap = get_nvidia_specs().compute_capability
                except Exception as e:
                    print(f"Warning: failed to get NVIDIA compute capability: {e}", file=sys.stderr)
            print(cap)
            return 0
        if a.check_platform:
            want = a.check_platform.lower().replace("_", "")
            want = "apple" if want == "applesilicon" else want
            return 0 if want == name else 1
        if kind == "unknown":
            print("GPU: No compatible GPU detected" if a.summary else
                  "No compatible GPU detected or unsupported platform.")
            print(f"Platform: {kind}")
            return 0
        specs = get_nvidia_specs() if kind == "nvidia" else get_other_specs(kind)
        if a.occupancy:
            cap = specs.compute_capability or "10.0"
            o = occupancy(cap, a.threads, a.regs, a.smem)
            print(f"sm_{cap.replace('.', '')}: {o['blocks_per_sm']} blocks/SM ({o['warps_per_sm']} warps, "
                  f"{o['occupancy']:.0%}), limited by {o['limiter']}; limits {o['limits']}")
            return 0
        if not a.summary:
            print(f"Detected Platform: {kind.replace('_', ' ').title()}\n")
        print_specs(specs, a.summary)
        return 0
    except Exception as e:
        print(f"Error detecting GPU specifications: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())

"""In-tree build of the native libraries.

`build_all()` compiles every `.cu` / `.cpp` under `csrc/` for sm_100a with nvcc and links
`zero_to_hero_b200/lib/libz2h.so` (CUDA kernels + C ABI) and `libz2h_host.so` (host-only C++:
micrograd engine, CPU oracles). nvcc cross-compiles without a GPU, so this also is the
"does it build" check. Objects are cached under `build/`, named by the content of their source and of all headers.

Run as `python -m zero_to_hero_b200.build [--force] [--verbose] [--bounds]`. `--bounds` builds the
self-checking debug variant `libz2h_bounds.so` (-DZ2H_BOUNDS, see csrc/common/checked.cuh), which
`Z2H_NATIVE_LIB=bounds` selects at run time.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIBDIR = Path(__file__).resolve().parent / "lib"
OBJDIR = ROOT / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=default",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def _headers_stamp() -> str:
    """Names the state of all headers by their content (not by path or time, so a copy of the tree on
    another machine finds the objects that came with it up to date)."""
    h = hashlib.sha1()
    for p in sorted(list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h")) + list(CSRC.rglob("*.hpp"))):
        h.update(str(p.relative_to(CSRC)).encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:12]


def _compile(src: Path, obj: Path, cmd: list[str], verbose: bool) -> tuple[Path, str]:
    obj.parent.mkdir(parents=True, exist_ok=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    if verbose:
        print(r.stderr, file=sys.stderr)
    return obj, r.stderr


def build_all(force: bool = False, verbose: bool = False, bounds: bool = False) -> dict[str, Path]:
    """Compile all native sources; returns {'cuda': path, 'host': path}. `bounds`: the CUDA library
    is built with -DZ2H_BOUNDS into libz2h_bounds.so (the product library is left alone)."""
    nvcc = _nvcc()
    hdr = _headers_stamp()
    flavour = "b" if bounds else ""
    extra = ["-DZ2H_BOUNDS"] if bounds else []

    def obj_for(src: Path) -> Path:
        # the object's name carries the content of its source and of every header: an object that
        # exists is up to date, whatever the file times say (they do not survive a copy of the tree)
        tag = hashlib.sha1(hdr.encode() + src.read_bytes()).hexdigest()[:12] + flavour
        return OBJDIR / src.relative_to(CSRC).with_suffix(f".{tag}.o")

    LIBDIR.mkdir(parents=True, exist_ok=True)
    cu_srcs = sorted(p for p in CSRC.rglob("*.cu"))
    host_srcs = sorted(p for p in (CSRC / "cpu").rglob("*.cpp"))
    jobs = []
    cu_objs, host_objs = [], []
    for src in cu_srcs:
        obj = obj_for(src)
        cu_objs.append(obj)
        if force or not obj.exists():
            cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append((src, obj, cmd))
    for src in host_srcs:
        obj = obj_for(src)
        host_objs.append(obj)
        if force or not obj.exists():
            cmd = ["g++", *CXX_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            jobs.append((src, obj, cmd))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            futs = [ex.submit(_compile, s, o, c, verbose) for s, o, c in jobs]
            for f in futs:
                f.result()
    out = {}
    cuda_lib = LIBDIR / ("libz2h_bounds.so" if bounds else "libz2h.so")
    if cu_objs and (jobs or force or not cuda_lib.exists()):
        cmd = [nvcc, "-shared", "-o", str(cuda_lib), *map(str, cu_objs),
               "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed: {r.stderr}")
    out["cuda"] = cuda_lib
    host_lib = LIBDIR / "libz2h_host.so"
    if host_objs and (jobs or force or not host_lib.exists()):
        cmd = ["g++", "-shared", "-o", str(host_lib), *map(str, host_objs), "-pthread"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed: {r.stderr}")
    out["host"] = host_lib
    # objects of earlier header states are never used again: drop them, keeping both flavours of the
    # current state (the cache otherwise grows by a full set per header edit)
    keep = set()
    for src in cu_srcs + host_srcs:
        tag = hashlib.sha1(hdr.encode() + src.read_bytes()).hexdigest()[:12]
        keep.update({tag, tag + "b"})
    if OBJDIR.exists():
        for old in OBJDIR.rglob("*.o"):
            parts = old.name.split(".")
            if len(parts) >= 3 and parts[-2] not in keep:
                old.unlink(missing_ok=True)
    return out


def main() -> None:
    libs = build_all(force="--force" in sys.argv, verbose="--verbose" in sys.argv, bounds="--bounds" in sys.argv)
    for k, v in libs.items():
        print(f"{k}: {v} ({v.stat().st_size if v.exists() else 0} bytes)")


if __name__ == "__main__":
    main()
